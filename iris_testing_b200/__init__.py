"""iris_testing_b200 — Blackwell-native MoE expert-parallel library."""
__version__ = "0.1.0"
