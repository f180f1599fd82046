"""``Expert`` / ``expert`` (layers/expert.py:6-65)."""
from ...ops.expert import Expert, expert  # noqa: F401
