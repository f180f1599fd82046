"""``custom_a2a`` / ``AllToAllOp`` (layers/all_to_all.py:10-125)."""
from ...ops.dispatch import AllToAllOp, custom_a2a  # noqa: F401
