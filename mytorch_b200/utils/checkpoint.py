"""Activation checkpointing (mytorch/utils/checkpoint.py:39-121): the wrapped function runs
without recording a graph, keeps only its inputs, and is run again - this time recorded - when its
output's gradient arrives, so the activations inside it live only during that backward."""
from ..tensor import Tensor, no_grad


def checkpoint(fn, *args, iter_gc=10):
    """out = fn(*args) with the intermediates of `fn` recomputed in the backward pass.

    `fn` is a function or a Module; Tensor arguments receive gradients, anything else is passed
    through. `iter_gc` is accepted for compatibility with the reference (which forces a garbage
    collection every `iter_gc` backward calls to break reference cycles); this implementation
    drops its closures as they run and needs none."""
    name = getattr(fn, "__name__", fn.__class__.__name__)
    call = getattr(fn, "__call__", fn)
    with no_grad():
        out = call(*[a.detach() if isinstance(a, Tensor) else a for a in args])
    if not isinstance(out, Tensor):
        raise TypeError("checkpoint: the wrapped function must return one Tensor")
    tensor_args = [a for a in args if isinstance(a, Tensor)]
    params = list(fn.parameters()) if hasattr(fn, "parameters") else []
    if not (Tensor.build_graph_enabled() and (any(a.requires_grad for a in tensor_args) or params)):
        return out

    def backward_fn(grad_output):
        leaves = []
        for a in args:
            if isinstance(a, Tensor):
                leaf = a.detach()
                leaf.requires_grad = a.requires_grad
                leaves.append(leaf)
            else:
                leaves.append(a)
        # Gradients of parameters used inside `fn` are written by this nested backward. The outer
        # backward already counts this node as a writer of each of them (they are its parents
        # below), so the nested one must not report them as final on its own.
        hook, Tensor.param_ready_hook = Tensor.param_ready_hook, None
        try:
            again = call(*leaves)
            again.backward(grad_output)
        finally:
            Tensor.param_ready_hook = hook
        for a, leaf in zip(args, leaves):
            if isinstance(a, Tensor) and a.requires_grad and leaf.grad is not None:
                a._accumulate(leaf.grad)
                leaf.grad = None

    res = Tensor(out.data)
    res.requires_grad = True
    res.grad_fn, res.grad_fn_name = backward_fn, f"<Checkpoint{name}Backward>"
    res._add_parents(*tensor_args, *params)
    return res
