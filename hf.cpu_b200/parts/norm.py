"""Norms.  RMSNorm: ``y_i = (x_i * rsqrt(mean(x^2) + eps)) * w_i`` (src/mathx.c:65-75, used at src/model.c:580,
:611, :632).  Dynamic Tanh: ``y_i = tanh(alpha * x_i) * w_i + b_i`` with a learned scalar ``alpha``: element-wise,
no mean or variance of the row is taken (the reference has no such norm).  Layer norm with a weight and no bias:
``y_i = (x_i - mean) / sqrt(var + eps) * w_i``, the variance being the mean of the squared deviations (nor this one)."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Norm, register_part


class RmsNorm(Norm):
    """``offset`` is added to the stored weight: a weight stored around zero (``x / rms * (1 + w)``) has offset 1.  The
    sum is made once, in float32, when the weights are bound; every kernel that applies this norm then reads a float32
    weight (1 + w has more digits than bfloat16 keeps)."""
    graph_safe = True

    def __init__(self, size: int, eps: float, tensor: str, offset: float = 0.0, **_):
        self.size, self.eps, self.tensor, self.offset = int(size), float(eps), tensor, float(offset)
        self.weight = None
        self._w32 = None

    def tensor_specs(self):
        # random weights are drawn around the value that makes the norm's factor about one
        return [TensorSpec(self.tensor, (self.size,), init="normal" if self.offset else "norm")]

    def bind(self, tensors, run_dtype, device):
        self.weight = tensors[self.tensor].contiguous()
        if self.offset:
            self.weight = (self.weight.to(torch.float32) + self.offset).contiguous()

    def fused_args(self):
        return self.weight, self.eps

    def shift_args(self):
        """(float32 weight, eps, whether the mean is taken off) for the kernel that applies a norm with a token shift
        behind it."""
        if self._w32 is None:
            self._w32 = self.weight.to(torch.float32).contiguous()
        return self._w32, self.eps, False

    def forward(self, x, out, rows=None):
        with kernels.phase("glue"):
            kernels.rmsnorm(x, self.weight, self.eps, out, rows)
        return out


class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * w`` with a weight and no bias.  The weight is kept in float32 (the norm is computed
    there in both run types)."""
    graph_safe = True

    def __init__(self, size: int, eps: float, tensor: str, optional: bool = False, **_):
        self.size, self.eps, self.tensor, self.optional = int(size), float(eps), tensor, bool(optional)
        self.weight = None

    def tensor_specs(self):
        # ``optional``: a norm that nothing reads (the second norm of a layer without a feed-forward) may be stored or not
        return [TensorSpec(self.tensor, (self.size,), init="norm", optional=self.optional)]

    def bind(self, tensors, run_dtype, device):
        if self.optional and self.tensor not in tensors:
            return
        self.weight = tensors[self.tensor].to(torch.float32).contiguous()

    def fused_args(self):
        return self.weight, self.eps, {"center": True}

    def shift_args(self):
        return self.weight, self.eps, True

    def forward(self, x, out, rows=None):
        with kernels.phase("glue"):
            kernels.layernorm(x, self.weight, self.eps, out, rows)
        return out


class ShiftedNorm(Norm):
    """A norm with the token shift of the block behind it, as one object that a sublayer's last product can be handed: in
    a step in which every request brings one token, that product's tail norms the new stream, shifts it by the
    request's previous row and leaves the new row in its place.  Made per step by the block in front; not registered."""

    def __init__(self, norm, mu, state, ctx):
        self.norm, self.mu, self.state, self.ctx = norm, mu, state, ctx

    def fused_args(self):
        w, eps, center = self.norm.shift_args()
        return w, eps, {"center": center, "shift": (self.mu, self.state, self.ctx.seq_slots)}

    def forward(self, x, out, rows=None):
        w, eps, center = self.norm.shift_args()
        with kernels.phase("glue"):
            kernels.norm_shift(x, w, eps, center, self.mu, self.state, self.ctx, out)
        return out


class DynamicTanh(Norm):
    """``tanh(alpha * x) * w + b``; the tensors are ``tensor`` (w), ``tensor + bias_suffix`` and ``tensor + alpha_suffix``
    (a scalar).  Being element-wise it also serves as the norm of a sublayer's *output* (:meth:`add_into`)."""
    graph_safe = True

    def __init__(self, size: int, tensor: str, bias_suffix: str = ".b", alpha_suffix: str = ".alpha", optional: bool = False, **_):
        self.size, self.tensor = int(size), tensor
        self.names = (tensor + alpha_suffix, tensor, tensor + bias_suffix)
        self.optional = bool(optional)
        self.params = None          # (alpha, w, b)

    def tensor_specs(self):
        a, w, b = self.names
        return [TensorSpec(w, (self.size,), init="norm", optional=self.optional),
                TensorSpec(b, (self.size,), optional=self.optional),
                TensorSpec(a, (), init="norm", optional=self.optional)]

    def bind(self, tensors, run_dtype, device):
        if self.optional and any(n not in tensors for n in self.names):
            return
        alpha, w, b = (tensors[n].contiguous() for n in self.names)
        self.params = (alpha.reshape(1), w, b)

    def forward(self, x, out, rows=None):
        with kernels.phase("glue"):
            kernels.dyt(x, self.params, out, rows)
        return out

    def add_into(self, y, residual, next_norm=None, out=None, mix=None):
        """residual += norm(y); when ``next_norm`` is another Dynamic Tanh, ``out = next_norm(residual)`` comes out of
        the same pass.  Returns whether ``out`` was written.  ``mix`` = (rows, weights) adds a weighted sum of rows per
        token to y (a routed feed-forward's chosen experts), summed by the same pass; y may then be None."""
        fused = out is not None and isinstance(next_norm, DynamicTanh)
        with kernels.phase("glue"):
            kernels.dyt_residual(y, self.params, residual, next_norm.params if fused else None, out if fused else None, mix=mix)
        return fused

    def add_product_into(self, a, w, bias, y_buf, residual, next_norm=None, out=None, mix=None):
        """The same for a sublayer whose output is a product, ``a @ w.T + bias (+ mix)``: where the product is split over
        its inner dimension, the partial sums are summed by this norm's own pass."""
        fused = out is not None and isinstance(next_norm, DynamicTanh)
        kernels.linear_dyt_residual(a, w, bias, y_buf, self.params, residual, next_norm.params if fused else None,
                                    out if fused else None, mix=mix)
        return fused


register_part("norm", "rmsnorm", RmsNorm)
register_part("norm", "layernorm", LayerNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
