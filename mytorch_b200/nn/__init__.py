"""`mytorch.nn` for the GPT training step (mytorch/nn/modules/__init__.py:9-16)."""
from . import functional
from .modules import (Module, ModuleList, Sequential, Linear, Embedding, LayerNorm, RMSNorm, GELU,
                      ReLUSquared, Softmax, Dropout, CrossEntropyLoss, Parameter, init)

__all__ = ["functional", "Module", "ModuleList", "Sequential", "Linear", "Embedding", "LayerNorm", "RMSNorm",
           "GELU", "ReLUSquared", "Softmax", "Dropout", "CrossEntropyLoss", "Parameter", "init"]
