"""Shared arithmetic of the bfloat-emulated normalisation layers (LayerNorm, GroupNorm, BatchNorm); the
sequences of vector operations, each followed by a rounding to the vector format, are those of the reference's
mx/norm_utils.py (forward :25-114, input gradient :117-183, LayerNorm's input gradient :186-258).

    forward:   m = mean(x); d = x - m; v = mean(d * d); s = 1 / sqrt(v + eps); n = d * s; y = w * n + b
    backward:  with h = g * w:  dx = h * s  -  d * (mean(h * d) * s^2 * s)  +  mean(-(h * s))
    LayerNorm: the same gradient rebuilt from n and (v + eps), the mean term taken last, as DeepSpeed does
"""
import collections

from .vector_ops import (vec_add, vec_div, vec_mul, vec_quantize, vec_recip, vec_reduce_mean, vec_sqrt, vec_sub)

Normed = collections.namedtuple("Normed", "output x_shift x_norm x_std_inv x_mean x_vare")


def _as_list(axes):
    if type(axes) is not list:
        assert type(axes) is int
        return [axes]
    return axes


def _per_channel(t, like, weight_axis):
    """A per-channel vector shaped to broadcast against `like` along weight_axis (None: as it is)."""
    if weight_axis is None:
        return t
    shape = [1] * like.ndim
    shape[weight_axis] = like.shape[weight_axis]
    return t.view(shape)


def _grouped(shape, axis, groups):
    """(N, C, ...) -> (N, groups, C / groups, ...): the shape a GroupNorm reduces over."""
    C = shape[axis]
    assert C % groups == 0
    out = list(shape)
    out[axis] = groups
    out.insert(axis + 1, C // groups)
    return out


def norm_forward(x, axes, weight, bias, eps, mx_specs, groups=None, weight_axis=None, use_running_stats=False,
                 running_mean=None, running_var=None):
    """x, weight and bias already rounded.  `axes`: the dimensions averaged over; with `groups`, axes[0] is
    split into (groups, C / groups) first.  With use_running_stats the stored mean and variance replace
    the batch statistics."""
    sp = mx_specs
    axes = _as_list(axes)
    w, b = _per_channel(weight, x, weight_axis), _per_channel(bias, x, weight_axis)
    full_shape = list(x.shape)
    if groups:
        x = x.view(_grouped(full_shape, axes[0], groups))
        axes = [a + 1 for a in axes]
    stat_shape = [1 if (i == 0 or i in axes) else n for i, n in enumerate(x.shape)]
    if use_running_stats:
        assert running_mean is not None and running_var is not None
        mean = vec_quantize(running_mean, mx_specs=sp).view(stat_shape)
        shift = vec_sub(x, mean, mx_specs=sp)
        var = vec_quantize(running_var, mx_specs=sp).view(stat_shape)
    else:
        mean = vec_reduce_mean(x, axes, keepdim=True, mx_specs=sp)
        shift = vec_sub(x, mean, mx_specs=sp)
        var = vec_reduce_mean(vec_mul(shift, shift, mx_specs=sp), axes, keepdim=True, mx_specs=sp)
    vare = vec_add(var, eps, mx_specs=sp)
    std_inv = vec_recip(vec_sqrt(vare, mx_specs=sp), mx_specs=sp)
    normed = vec_mul(shift, std_inv, mx_specs=sp)
    if groups:
        normed = normed.view(full_shape)
    out = vec_add(vec_mul(w, normed, mx_specs=sp), b, mx_specs=sp)
    return Normed(out, shift, normed, std_inv, mean, vare)


def norm_backward(grad_output, axes, weight, x_shift, x_std_inv, mx_specs, groups=None, weight_axis=None):
    """Gradient with respect to the input from the shifted input and 1 / std kept by the forward pass."""
    sp = mx_specs
    axes = _as_list(axes)
    full_shape = list(grad_output.shape)
    h = vec_mul(grad_output, _per_channel(weight, grad_output, weight_axis), mx_specs=sp)
    if groups:
        h = h.view(_grouped(full_shape, axes[0], groups))
        axes = [a + 1 for a in axes]
    direct = vec_mul(h, x_std_inv, mx_specs=sp)
    mean_term = vec_reduce_mean(-direct, axes, keepdim=True, mx_specs=sp)
    t = vec_reduce_mean(vec_mul(h, x_shift, mx_specs=sp), axes, keepdim=True, mx_specs=sp)
    t = vec_mul(vec_mul(t, vec_mul(x_std_inv, x_std_inv, mx_specs=sp), mx_specs=sp), x_std_inv, mx_specs=sp)
    dx = vec_add(vec_add(direct, vec_mul(-t, x_shift, mx_specs=sp), mx_specs=sp), mean_term, mx_specs=sp)
    return dx.view(full_shape) if groups else dx


def norm_backward_ln(grad_output, axes, weight, x_norm, x_vare, mx_specs, groups=None, weight_axis=None):
    """LayerNorm's input gradient from the normalised input and (variance + eps)."""
    sp = mx_specs
    axes = _as_list(axes)
    full_shape = list(grad_output.shape)
    h = vec_mul(grad_output, _per_channel(weight, grad_output, weight_axis), mx_specs=sp)
    if groups:
        h = h.view(_grouped(full_shape, axes[0], groups))
        axes = [a + 1 for a in axes]
    std = vec_sqrt(x_vare, mx_specs=sp)
    std_inv = vec_div(1.0, std, mx_specs=sp)
    direct = vec_mul(h, std_inv, mx_specs=sp)
    t = vec_mul(vec_mul(h, x_norm, mx_specs=sp), std, mx_specs=sp)          # h * (x - mean)
    t = vec_reduce_mean(t, axes, keepdim=True, mx_specs=sp)
    t = vec_mul(t, vec_div(1.0, x_vare, mx_specs=sp), mx_specs=sp)
    dx = vec_add(direct, vec_mul(-t, x_norm, mx_specs=sp), mx_specs=sp)
    dx = vec_add(dx, -vec_reduce_mean(dx, axes, keepdim=True, mx_specs=sp), mx_specs=sp)
    return dx.view(full_shape) if groups else dx
