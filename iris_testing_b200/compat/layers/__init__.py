"""Layer ops under the reference's module names."""
