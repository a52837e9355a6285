"""Host-side utilities of the training step (input pipeline, activation checkpointing)."""
from .checkpoint import checkpoint  # noqa: F401
from .data import DataLoader, Dataset, TokenLoader  # noqa: F401
