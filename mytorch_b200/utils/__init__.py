"""Host-side utilities of the training step (input pipeline)."""
from .data import DataLoader, Dataset, TokenLoader  # noqa: F401
