"""`cupyx` stand-in (see the sibling `cupy` package)."""
