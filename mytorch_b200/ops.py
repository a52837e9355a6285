"""Functional forms of the Tensor glue ops plus concatenate and stack
(mytorch/ops.py:1-160 of the reference, the part the GPT model files use). Every op is a
strided copy on the device (mt_copy_strided) with a backward that copies the matching block of
the incoming gradient."""
import numpy as np

from .array import DeviceArray
from .tensor import Tensor, _contig_strides, _graph, _norm_dim, _strided_copy, _wants_graph


def transpose(input, dim1, dim2):
    return input.transpose(dim1, dim2)


def permute(input, *dims):
    return input.permute(*dims)


def reshape(input, *shape):
    return input.reshape(*shape)


def sum(input, dim=None, keepdims=False):
    return input.sum(dim, keepdims)


def mean(input, dim=None, keepdims=False):
    return input.mean(dim, keepdims)


def chunk(input, chunks, dim=0):
    return input.chunk(chunks=chunks, dim=dim)


def _join(tensors, dim, new_axis, name):
    if len(tensors) == 0:
        raise ValueError(f"{'stack' if new_axis else 'concatenate'}() expects a non-empty list of Tensors")
    first = tensors[0]
    if any(t.dtype != first.dtype for t in tensors):
        raise TypeError("all tensors must share one dtype")
    if new_axis:
        d = _norm_dim(dim, first.ndim + 1)
        if any(t.shape != first.shape for t in tensors):
            raise ValueError("stack() needs tensors of one shape")
        part_shapes = [t.shape[:d] + (1,) + t.shape[d:] for t in tensors]
    else:
        d = _norm_dim(dim, first.ndim)
        if any(t.shape[:d] + t.shape[d + 1:] != first.shape[:d] + first.shape[d + 1:] for t in tensors):
            raise ValueError("concatenate() needs tensors that agree outside the joined dimension")
        part_shapes = [t.shape for t in tensors]
    sizes = [s[d] for s in part_shapes]
    out_shape = part_shapes[0][:d] + (int(np.sum(sizes)),) + part_shapes[0][d + 1:]
    out_data = DeviceArray.empty(out_shape, first.dtype)
    ost = _contig_strides(out_shape)
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int64)
    for t, shp, off in zip(tensors, part_shapes, offs):
        _strided_copy(t.data, out_data, shp, _contig_strides(shp), ost, dst_offset=int(off) * ost[d])
    out = Tensor(out_data)
    if _wants_graph(*tensors):
        def _bw(g):
            for t, shp, off in zip(tensors, part_shapes, offs):
                if t.requires_grad:
                    piece = DeviceArray.empty(t.shape, g.dtype)
                    _strided_copy(g, piece, shp, ost, _contig_strides(shp), src_offset=int(off) * ost[d])
                    t._accumulate(piece)
        _graph(out, tuple(tensors), _bw, name)
    return out


def concatenate(tensors, dim=0):
    """Joins tensors along an existing dimension (mytorch/ops.py:62-111)."""
    return _join(list(tensors), dim, False, "<ConcatBackward>")


def stack(tensors, dim=0):
    """Joins tensors of one shape along a new dimension (mytorch/ops.py:113-160)."""
    return _join(list(tensors), dim, True, "<StackBackward>")
