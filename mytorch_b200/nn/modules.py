"""Module system and the layers of the GPT training step: `Module` with the
parameter/buffer registry and tied-weight de-duplication of
mytorch/nn/modules/base_module.py:5-315, and Linear, Embedding, LayerNorm,
RMSNorm, GELU, ReLUSquared, Dropout (p = 0), CrossEntropyLoss, ModuleList,
Sequential (mytorch/nn/modules/**). Parameters are drawn on the host with the
NumPy global generator, as in mytorch/nn/initializations.py:44-56, so that a
seed gives the same weights as the reference."""
import math

import numpy as np

from ..array import DeviceArray
from ..tensor import Tensor
from . import functional as F


def Parameter(array):
    t = Tensor(array, requires_grad=True)
    t.is_param = True
    return t


class Module:
    def __init__(self):
        object.__setattr__(self, "_modules", {})
        object.__setattr__(self, "_params", {})
        object.__setattr__(self, "_buffers", {})
        object.__setattr__(self, "training", True)

    def __setattr__(self, name, value):
        if isinstance(value, Module):
            self._modules[name] = value
        elif isinstance(value, Tensor) and value.requires_grad:
            value.is_param = True
            self._params[name] = value
        elif name in self._params and value is None:
            del self._params[name]
        object.__setattr__(self, name, value)

    def register_buffer(self, name, tensor, persistent=True):
        self._buffers[name] = (tensor, persistent)
        object.__setattr__(self, name, tensor)

    def __call__(self, *a, **k):
        return self.forward(*a, **k)

    # -- traversal; parameters() de-duplicates tied tensors by device pointer
    # (base_module.py:35-57), the *_no_dedup forms do not (:59-65) --
    def _named_parameters_no_dedup(self, prefix=""):
        for n, p in self._params.items():
            yield prefix + n, p
        for mn, m in self._modules.items():
            yield from m._named_parameters_no_dedup(prefix + mn + ".")

    def _parameters_no_dedup(self):
        return [p for _, p in self._named_parameters_no_dedup()]

    def named_parameters(self):
        seen = set()
        for n, p in self._named_parameters_no_dedup():
            if p.data.ptr in seen:
                continue
            seen.add(p.data.ptr)
            yield n, p

    def parameters(self):
        return [p for _, p in self.named_parameters()]

    def modules(self):
        yield self
        for m in self._modules.values():
            yield from m.modules()

    def apply(self, fn):
        for m in self._modules.values():
            m.apply(fn)
        fn(self)
        return self

    def train(self):
        for m in self.modules():
            object.__setattr__(m, "training", True)
        return self

    def eval(self):
        for m in self.modules():
            object.__setattr__(m, "training", False)
        return self

    def to(self, device=None):
        return self

    def state_dict(self):
        """name -> NumPy array, tied weights listed under every name
        (base_module.py:220-241)."""
        sd = {n: p.numpy() for n, p in self._named_parameters_no_dedup()}
        for n, (b, persistent) in self._buffers.items():
            if persistent and b is not None:
                sd[n] = b.numpy()
        return sd

    def load_state_dict(self, state_dict, strict=True, device=None):
        missing = []
        for n, p in self._named_parameters_no_dedup():
            if n in state_dict:
                a = np.asarray(state_dict[n])
                if a.shape != p.shape:
                    raise ValueError(f"shape mismatch for {n}: {a.shape} vs {p.shape}")
                p.data.set_from_numpy(a)
            else:
                missing.append(n)
        if strict and missing:
            raise KeyError(f"missing keys: {missing}")
        return missing

    def zero_grad(self):
        for p in self.parameters():
            p.grad = None

    def num_parameters(self):
        return sum(p.data.size for p in self.parameters())


class ModuleList(Module):
    def __init__(self, modules=()):
        super().__init__()
        self._list = []
        for m in modules:
            self.append(m)

    def append(self, m):
        self._modules[str(len(self._list))] = m
        self._list.append(m)

    def __iter__(self):
        return iter(self._list)

    def __len__(self):
        return len(self._list)

    def __getitem__(self, i):
        return self._list[i]


class Sequential(ModuleList):
    def __init__(self, *modules):
        super().__init__(modules)

    def forward(self, x):
        for m in self._list:
            x = m(x)
        return x


def _uniform(shape, lo, hi):
    return np.random.uniform(lo, hi, size=shape).astype(np.float32)


class Linear(Module):
    """weight [out, in], U(-1/sqrt(in), 1/sqrt(in)) (modules/layers/linear.py:7-48)."""

    def __init__(self, in_features, out_features, bias=True, auto=False, fused=True, act_func=None):
        super().__init__()
        self.in_features, self.out_features, self.act_func = in_features, out_features, act_func
        k = math.sqrt(1 / in_features)
        self.weight = Parameter(DeviceArray.from_numpy(_uniform((out_features, in_features), -k, k)))
        self.use_bias = bool(bias)
        self.bias = Parameter(DeviceArray.from_numpy(_uniform((out_features,), 0.0, 1.0))) if bias else None

    def forward(self, x):
        return F.linear(x, self.weight, self.bias, act_func=self.act_func)


class Embedding(Module):
    """weight [num_embeddings, dim] ~ N(0,1) (modules/layers/embedding.py:7-28)."""

    def __init__(self, num_embeddings, embedding_dim, fused=True):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = Parameter(DeviceArray.from_numpy(np.random.randn(num_embeddings, embedding_dim).astype(np.float32)))

    def forward(self, indices):
        return F.embedding(indices, self.weight)


class LayerNorm(Module):
    """modules/norm/layernorm.py:6-58: weight ones, bias zeros, eps 1e-5."""

    def __init__(self, embed_dim, weight=True, bias=True, eps=1e-5, auto=False, fused=True):
        super().__init__()
        self.eps = eps
        self.weight = Parameter(DeviceArray.from_numpy(np.ones(embed_dim, np.float32))) if weight else None
        self.bias = Parameter(DeviceArray.from_numpy(np.zeros(embed_dim, np.float32))) if bias else None

    def forward(self, x):
        return F.layernorm(x, self.weight, self.bias, self.eps, self.training)


class RMSNorm(Module):
    """modules/norm/rmsnorm.py:6-55."""

    def __init__(self, embed_dim, weight=True, eps=1e-5, auto=False, fused=True):
        super().__init__()
        self.eps = eps
        self.weight = Parameter(DeviceArray.from_numpy(np.ones(embed_dim, np.float32))) if weight else None

    def forward(self, x):
        return F.rmsnorm(x, self.weight, self.eps, self.training)


class GELU(Module):
    def forward(self, x):
        return F.gelu(x)


class ReLUSquared(Module):
    def forward(self, x):
        return F.relu_squared(x)


class Softmax(Module):
    def __init__(self, auto=False, fused=True):
        super().__init__()

    def forward(self, x, dim=-1):
        return F.softmax(x, dim)


class Dropout(Module):
    def __init__(self, dropout_p=0.0):
        super().__init__()
        self.p = dropout_p

    def forward(self, x):
        return F.dropout(x, self.p, self.training)


class CrossEntropyLoss(Module):
    """modules/losses/cross_entropy.py:4-12."""

    def __init__(self, ignore_index=-100, softcap=None, auto=False, fused=True, fused_backward=False):
        super().__init__()
        self.ignore_index, self.softcap = ignore_index, softcap
        self.fused_backward = fused_backward     # see F.cross_entropy: the logits are overwritten in forward

    def forward(self, logits, targets):
        return F.cross_entropy(logits, targets, self.ignore_index, self.softcap, fused_backward=self.fused_backward)


# initialisers (mytorch/nn/initializations.py:44-56), host RNG then upload
class init:
    @staticmethod
    def normal_(t, mean=0.0, std=1.0):
        t.data.set_from_numpy(np.random.normal(mean, std, size=t.shape).astype(np.float32))
        return t

    @staticmethod
    def uniform_(t, low=0.0, high=1.0):
        t.data.set_from_numpy(_uniform(t.shape, low, high))
        return t

    @staticmethod
    def zeros_(t):
        t.data.zero_()
        return t

    @staticmethod
    def ones_(t):
        t.data.fill_(1.0)
        return t
