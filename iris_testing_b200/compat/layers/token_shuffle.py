"""``TokenShuffle`` / ``shuffle`` (layers/token_shuffle.py:7-61), plus the inverse."""
from ...ops.shuffle import TokenShuffle, shuffle, unshuffle  # noqa: F401
