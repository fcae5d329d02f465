"""bfloat-emulated BatchNorm over (N, C, ...) inputs, statistics per channel over the batch and spatial
dimensions; drop-in for the reference's mx/batchnorm.py (autograd function :16-129, function :132-145,
modules :148-237).  In training the batch statistics are used and the running averages, when tracked, are
updated in place as (1 - momentum) * running + momentum * batch, every product and the sum rounded; in
evaluation the running statistics are used."""
import torch
import torch.nn.functional as F

from .norm_utils import norm_backward, norm_forward
from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test
from .vector_ops import vec_add, vec_mul, vec_quantize, vec_reduce_sum

f_batch_norm = F.batch_norm


class BatchNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, running_mean, running_var, weight, bias, is_training=False, momentum=0.1, eps=1e-5,
                mx_specs=None):
        sp = mx_specs
        if not is_training:
            assert running_mean is not None and running_var is not None
        x = vec_quantize(x, mx_specs=sp)
        bf_w = vec_quantize(weight, mx_specs=sp)
        C = x.shape[1]
        not_channel = [0] + list(range(2, x.ndim))
        r = norm_forward(x, not_channel, bf_w, vec_quantize(bias, mx_specs=sp), eps, sp, weight_axis=1,
                         use_running_stats=not is_training, running_mean=running_mean, running_var=running_var)
        if is_training:
            # the variance folded into the running average is the one with eps already added
            for running, batch in ((running_mean, r.x_mean), (running_var, r.x_vare)):
                if running is not None:
                    running.copy_(vec_add(vec_mul(1 - momentum, running, mx_specs=sp),
                                          vec_mul(momentum, batch.view(C), mx_specs=sp), mx_specs=sp))
        ctx.save_for_backward(r.x_shift, r.x_norm, r.x_std_inv, bf_w if sp["quantize_backprop"] else weight)
        ctx.mx_specs = get_backwards_mx_specs(sp)
        return r.output

    @staticmethod
    def backward(ctx, grad_output):
        sp = ctx.mx_specs
        x_shift, x_norm, x_std_inv, weight = ctx.saved_tensors
        not_channel = [0] + list(range(2, grad_output.ndim))
        g = vec_quantize(grad_output, mx_specs=sp)
        grad_bias = vec_reduce_sum(g, not_channel, mx_specs=sp)
        grad_weight = vec_reduce_sum(vec_mul(g, x_norm, mx_specs=sp), not_channel, mx_specs=sp)
        grad_input = norm_backward(g, not_channel, weight, x_shift, x_std_inv, sp, weight_axis=1)
        return (grad_input, None, None, grad_weight, grad_bias, None, None, None, None)


def batch_norm(x, running_mean, running_var, weight, bias, is_training=False, momentum=0.1, eps=1e-5,
               mx_specs=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return f_batch_norm(x, running_mean, running_var, weight, bias, is_training, momentum, eps)
    return BatchNormFunction.apply(x, running_mean, running_var, weight, bias, is_training, momentum, eps,
                                   apply_mx_specs(mx_specs))


class _BatchNorm(torch.nn.modules.batchnorm._BatchNorm):
    def __init__(self, num_features, mx_specs=None, name=None, **kwargs):
        super().__init__(num_features, **kwargs)
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.mx_specs = apply_mx_specs(mx_specs)
        self.name = name

    def forward(self, input):
        if self.mx_none:
            return super().forward(input)
        self._check_input_dim(input)
        factor = 0.0 if self.momentum is None else self.momentum
        if self.training and self.track_running_stats and self.num_batches_tracked is not None:
            self.num_batches_tracked += 1
            if self.momentum is None:
                factor = 1.0 / float(self.num_batches_tracked)          # cumulative moving average
        # evaluation falls back to the batch statistics only when no running statistics exist
        use_batch = self.training or (self.running_mean is None and self.running_var is None)
        stats = not self.training or self.track_running_stats
        return batch_norm(input, self.running_mean if stats else None, self.running_var if stats else None,
                          self.weight, self.bias, is_training=use_batch, momentum=factor, eps=self.eps,
                          mx_specs=self.mx_specs)


def _dims(*allowed):
    def check(self, input):
        if input.dim() not in allowed:
            raise ValueError("expected %s input (got %dD input)" % (" or ".join("%dD" % d for d in allowed), input.dim()))
    return check


class BatchNorm1d(_BatchNorm):
    _check_input_dim = _dims(2, 3)


class BatchNorm2d(_BatchNorm):
    _check_input_dim = _dims(4)


class BatchNorm3d(_BatchNorm):
    _check_input_dim = _dims(5)
