"""Matrix-memory mixer with exponential gates kept in logarithms (the mLSTM cell of the xLSTM family).

    q = h . W_q^T * dim^-1/2,  k = h . W_k^T   [heads x dim]      v = h . W_v^T   [heads x vdim]          (no biases)
    i = cap tanh((h . W_i^T + b_i) / cap),   f = logsigmoid(cap tanh((h . W_f^T + b_f) / cap))          log gates, per head
    per head, with S = 0, n = 0, m = 0 for a new request:
        m' = max(f + m, i);   S <- exp(f + m - m') S + exp(i - m') k v^T;   n <- the same with k alone;   m <- m'
        o = S^T q / (max(|n . q|, exp(-m)) + 1e-6)
    out = ( o / rms(o) per head * norm weight * sigmoid(h . W_g^T) ) . W_o^T

Kept per request, 32-bit: [heads, dim + 1, vdim + 1], S with the normaliser n as one more column (the column of a value
that is always 1) and m, copied for every column, as one more row; zero for a new request, which is where m starts.  The
gates, the decays, the state, the read-out and its norm are 32-bit in every mode; the six projections run as one product.
`names` gives the tensors' names.
"""
from __future__ import annotations

import torch

from .base import Mixer, ParamDecl, StateNeed, register_part, stack_rows

DEFAULT_NAMES = {"q": "mlstm_q.weight", "k": "mlstm_k.weight", "v": "mlstm_v.weight", "g": "mlstm_gate.weight",
                 "i": "mlstm_igate.weight", "i_bias": "mlstm_igate.bias", "f": "mlstm_fgate.weight", "f_bias": "mlstm_fgate.bias",
                 "norm": "mlstm_norm.weight", "o": "mlstm_out.weight"}


class MLstm(Mixer):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True             # forward launches kernels only; nothing is read back to the host
    kernel_libs = ("mlstm",)

    def __init__(self, hidden: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float, names=None):
        self.hidden, self.heads, self.dim, self.vdim = int(hidden), int(heads), int(dim), int(vdim)
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        if not 1 <= self.dim <= 256:
            raise ValueError(f"the matrix-memory kernel takes head sizes up to 256, not {self.dim}")
        if self.gate_cap <= 0:
            raise ValueError("the gates' cap is positive")
        self.names = {**DEFAULT_NAMES, **(names or {})}

    def params(self):
        nm, H, D, V, W = self.names, self.heads, self.dim, self.vdim, self.hidden
        return {nm["q"]: ParamDecl((H * D, W)), nm["k"]: ParamDecl((H * D, W)), nm["v"]: ParamDecl((H * V, W)),
                nm["g"]: ParamDecl((H * V, W)), nm["i"]: ParamDecl((H, W)), nm["f"]: ParamDecl((H, W)),
                nm["i_bias"]: ParamDecl((H,), "vector", init="conv"), nm["f_bias"]: ParamDecl((H,), "vector", init="conv"),
                nm["norm"]: ParamDecl((H * V,), "vector", init="norm_weight"), nm["o"]: ParamDecl((W, H * V))}

    def cache_need(self):
        return StateNeed((self.heads, self.dim + 1, self.vdim + 1))

    def bind(self, tensors, dtype):
        nm = self.names
        # one product for everything that reads h, every output on a 16-byte boundary: q | k | v | gate | i | f
        self.w_all, self.at = stack_rows([tensors[nm[k]] for k in ("q", "k", "v", "g", "i", "f")])
        self.b_i, self.b_f = tensors[nm["i_bias"]].float().contiguous(), tensors[nm["f_bias"]].float().contiguous()
        self.norm_w, self.w_o = tensors[nm["norm"]], tensors[nm["o"]]
        self.dtype = dtype

    def forward(self, x, step, cache, write_cache=True):
        ops = step.ops
        y = ops.linear(x, self.w_all)
        o = ops.mlstm(y, self.at, self.b_i, self.b_f, self.gate_cap, self.norm_w, self.eps, cache.state, step, self.heads, self.dim,
                      self.vdim, write_cache)
        return ops.linear(o, self.w_o)


register_part("mixer", "mlstm", MLstm)
