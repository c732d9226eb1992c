"""Norms, fused with the residual addition that precedes them: RMSNorm, and the layer norm with weight and bias.

`out = x * rsqrt(mean(x^2) + eps) * gamma` (eps inside the root), all in 32-bit (src/transformer/norm.zig:6-33; device
version src/cuda/layer_kernels.cu:17-43).  The reference adds residuals with separate kernels
(`addKernel`, layer_kernels.cu:46-59); here the pending term is added into the 32-bit residual
stream by the same kernel that normalises it.
"""
from __future__ import annotations

from .base import LazyNorm, Norm, NormedTerm, ParamDecl, Residual, register_part


class RmsNorm(Norm):
    """`offset`: what is added to the stored weight before it multiplies (1 for a weight stored around zero:
    `x / rms(x) * (1 + w)`); the sum is made once at load, in 32-bit."""
    graph_safe = True      # forward launches kernels only; nothing is read back to the host

    def __init__(self, size: int, eps: float, weight: str, offset: float = 0.0):
        self.size, self.eps, self.weight_name, self.offset = int(size), float(eps), weight, float(offset)
        self.weight = None

    def params(self):
        return {self.weight_name: ParamDecl((self.size,), "vector", init="norm_weight" if self.offset == 0.0 else "conv")}

    def bind(self, tensors, dtype):
        self.weight = tensors[self.weight_name]
        if self.offset != 0.0:
            self.weight = (self.weight.float() + self.offset).contiguous()
        self.dtype = dtype

    def forward(self, h, delta, step, lazy=False, rows=None):
        res = h if isinstance(h, Residual) else Residual(h)
        if isinstance(delta, NormedTerm):
            # the pending term is normed on its way into the stream, in the same kernel
            ops = step.ops
            if rows is not None:
                picked = ops.gather_add(res.data, delta.data, rows, delta.gamma, delta.eps)
                return ops.add_rmsnorm(picked, None, self.weight, self.eps, self.dtype)
            return ops.add_rmsnorm(res.data, delta.data, self.weight, self.eps, self.dtype, delta.gamma, delta.eps)
        x = LazyNorm(res, delta, self.weight, self.eps, self.dtype, rows)
        if lazy and getattr(step.ops, "fuses_norm", False):
            return x
        return x.materialize(step.ops)


class LayerNorm(Norm):
    """`(x - mean) / sqrt(var + eps) * weight + bias` over the row, the variance being the mean of the squared
    deviations; all in 32-bit.  The pending term is added into the 32-bit residual stream by the same kernel."""
    graph_safe = True
    kernel_libs = ("layernorm",)

    def __init__(self, size: int, eps: float, weight: str, bias: str = None):
        self.size, self.eps, self.weight_name = int(size), float(eps), weight
        self.bias_name = bias if bias is not None else weight + ".bias"
        self.weight = self.bias = None

    def params(self):
        return {self.weight_name: ParamDecl((self.size,), "vector", init="norm_weight"),
                self.bias_name: ParamDecl((self.size,), "vector", init="conv")}

    def bind(self, tensors, dtype):
        self.weight, self.bias = tensors[self.weight_name], tensors[self.bias_name]
        self.dtype = dtype

    def forward(self, h, delta, step, lazy=False, rows=None):
        res = h if isinstance(h, Residual) else Residual(h)
        ops = step.ops
        if isinstance(delta, NormedTerm):
            raise TypeError("a layer norm takes a plain pending term")
        x = LazyNorm(res, delta, self.weight, self.eps, self.dtype, rows, beta=self.bias)
        if lazy and getattr(ops, "fuses_layernorm", False):
            return x                         # a product kernel applies it (steps of few rows)
        return x.materialize(ops)


register_part("norm", "rmsnorm", RmsNorm)
register_part("norm", "layernorm", LayerNorm)
