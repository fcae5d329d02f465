"""Calling an autograd Function when nothing can need a gradient."""
import torch


class _NoGradCtx:
    """Stand-in for the autograd context in a forward whose result will never be differentiated."""
    needs_input_grad = (False,) * 16

    def save_for_backward(self, *tensors):
        pass

    def mark_dirty(self, *tensors):
        pass

    def mark_non_differentiable(self, *tensors):
        pass

    def set_materialize_grads(self, value):
        pass


def call(fn, *args):
    """fn.apply(*args); when gradients are switched off, or no tensor argument requires one, fn.forward
    runs directly with a throw-away context (Function.apply costs 10-20 us of host time per call even
    then, which is a large share of an inference step made of 20-100 us kernels)."""
    if torch.is_grad_enabled():
        for a in args:
            if isinstance(a, torch.Tensor) and a.requires_grad:
                return fn.apply(*args)
        return _direct(fn, args)
    return _direct(fn, args)


def _direct(fn, args):
    with torch.no_grad():
        return fn.forward(_NoGradCtx(), *args)
