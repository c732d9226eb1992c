"""Gated delta rule mixer.

    q, k = h . W_q^T, h . W_k^T   [kv_heads x dim]      v = h . W_v^T   [heads x vdim]       (no biases)
    each passes a short causal depthwise convolution over time (no bias) and SiLU
    q, k <- unit vectors per head: x / sqrt(sum(x^2) + 1e-6);  q also times dim^-1/2
    beta = sigmoid(h . W_b^T),   g = exp(-exp(A_log) * softplus(h . W_a^T + dt_bias))        one per head
    per head (head i reads q/k head i // (heads / kv_heads)):
        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
    out = ( o / rms(o) * norm weight * silu(h . W_g^T) ) . W_o^T                              rms over vdim

Kept per request: S [heads, dim, vdim] and the convolutions' last taps - 1 inputs, both 32-bit.  Unit
norms, beta, g, the state and the output norm are 32-bit in every mode.  The six input projections run as
one product and the three convolutions as one.  `names` gives the tensors' names.

Options, for designs that vary the rule:
    decay="channel"    one decay per head and key channel, g [heads, dim], scaling the rows of S one by one:
                       S <- diag(g) S.  The projection W_a and dt_bias are then heads * dim wide; A_log stays per head.
    decay_rank=r       the decay's projection through r dimensions: a = (h . W_a1^T) . W_a2^T   (names a1, a2)
    gate_rank=r        the output gate's likewise: (h . W_g1^T) . W_g2^T                         (names g1, g2)
    gate_act           "silu" or "sigmoid": what the output gate passes before it multiplies the normed read-out
"""
from __future__ import annotations

import torch

from .base import Mixer, ParamDecl, StateNeed, register_part, stack_rows

DEFAULT_NAMES = {"q": "delta_q.weight", "k": "delta_k.weight", "v": "delta_v.weight", "q_conv": "delta_q_conv.weight",
                 "k_conv": "delta_k_conv.weight", "v_conv": "delta_v_conv.weight", "b": "delta_beta.weight",
                 "a": "delta_a.weight", "a_log": "delta_a_log", "dt_bias": "delta_dt_bias", "g": "delta_gate.weight",
                 "norm": "delta_norm.weight", "o": "delta_out.weight", "a1": "delta_a_down.weight", "a2": "delta_a_up.weight",
                 "g1": "delta_gate_down.weight", "g2": "delta_gate_up.weight"}
UNIT_EPS = 1e-6


class GatedDelta(Mixer):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True             # forward launches kernels only; nothing is read back to the host
    kernel_libs = ("causal_conv", "gated_delta")

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float, names=None,
                 decay: str = "head", decay_rank=None, gate_rank=None, gate_act: str = "silu"):
        self.hidden, self.heads, self.kv_heads = int(hidden), int(heads), int(kv_heads)
        self.dim, self.vdim, self.taps, self.eps = int(dim), int(vdim), int(taps), float(eps)
        if decay not in ("head", "channel") or gate_act not in ("silu", "sigmoid"):
            raise ValueError("decay is 'head' or 'channel', gate_act 'silu' or 'sigmoid'")
        self.decay, self.gate_act = decay, gate_act
        self.decay_rank = None if decay_rank is None else int(decay_rank)
        self.gate_rank = None if gate_rank is None else int(gate_rank)
        if (self.decay_rank is not None and self.decay_rank < 1) or (self.gate_rank is not None and self.gate_rank < 1):
            raise ValueError("a projection's inner size is at least 1")
        self.a_cols = self.heads * (self.dim if decay == "channel" else 1)
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads cannot share {self.kv_heads} query/key heads evenly")
        if self.taps < 1 or self.taps > 16:
            raise ValueError(f"the convolution kernels take 1 to 16 taps, not {self.taps}")
        if not 1 <= self.dim <= 256:
            raise ValueError(f"the delta-rule kernel takes head sizes up to 256, not {self.dim}")
        self.names = {**DEFAULT_NAMES, **(names or {})}
        self.qk_cols, self.v_cols = 2 * self.kv_heads * self.dim, self.heads * self.vdim

    def params(self):
        nm, H, G, D, V, L, W = self.names, self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.hidden
        conv = lambda c: ParamDecl((c, L), "vector", alt_shapes=((c, 1, L),), init="conv")
        p = {nm["q"]: ParamDecl((G * D, W)), nm["k"]: ParamDecl((G * D, W)), nm["v"]: ParamDecl((H * V, W)),
             nm["q_conv"]: conv(G * D), nm["k_conv"]: conv(G * D), nm["v_conv"]: conv(H * V),
             nm["b"]: ParamDecl((H, W)),
             nm["a_log"]: ParamDecl((H,), "vector", init="conv"), nm["dt_bias"]: ParamDecl((self.a_cols,), "vector", init="conv"),
             nm["norm"]: ParamDecl((V,), "vector", init="norm_weight"), nm["o"]: ParamDecl((W, H * V))}
        if self.decay_rank is None:
            p[nm["a"]] = ParamDecl((self.a_cols, W))
        else:
            p[nm["a1"]], p[nm["a2"]] = ParamDecl((self.decay_rank, W)), ParamDecl((self.a_cols, self.decay_rank))
        if self.gate_rank is None:
            p[nm["g"]] = ParamDecl((H * V, W))
        else:
            p[nm["g1"]], p[nm["g2"]] = ParamDecl((self.gate_rank, W)), ParamDecl((H * V, self.gate_rank))
        return p

    def cache_need(self):
        return (StateNeed((self.heads, self.dim, self.vdim)), StateNeed((max(self.taps - 1, 1), self.qk_cols + self.v_cols)))

    def bind(self, tensors, dtype):
        nm = self.names
        # one product for everything that reads h: q | k | v | gate (or its inner part) | b | a (or its inner part)
        g_in, a_in = ("g" if self.gate_rank is None else "g1"), ("a" if self.decay_rank is None else "a1")
        qkv = torch.cat([tensors[nm[k]] for k in ("q", "k", "v")], dim=0)
        self.w_all, (_, self.gate_at, self.b_at, self.a_at) = stack_rows([qkv] + [tensors[nm[k]] for k in (g_in, "b", a_in)])
        self.w_g2 = None if self.gate_rank is None else tensors[nm["g2"]]
        self.w_a2 = None if self.decay_rank is None else tensors[nm["a2"]]
        self.conv_w = torch.cat([tensors[nm[k]].reshape(-1, self.taps) for k in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w, self.w_o = tensors[nm["a_log"]], tensors[nm["dt_bias"]], tensors[nm["norm"]], tensors[nm["o"]]
        self.dtype = dtype

    def forward(self, x, step, cache, write_cache=True):
        ops, H = step.ops, self.heads
        matrix_state, conv_state = cache
        y = ops.linear(x, self.w_all)
        c0, g0, b0, a0 = self.qk_cols + self.v_cols, self.gate_at, self.b_at, self.a_at
        qkv = ops.causal_conv(y[:, :c0], self.conv_w, None, conv_state.state, step, True, write_cache)
        gate = y[:, g0:g0 + self.v_cols] if self.w_g2 is None else ops.linear(y[:, g0:g0 + self.gate_rank], self.w_g2)
        a = y[:, a0:a0 + self.a_cols] if self.w_a2 is None else ops.linear(y[:, a0:a0 + self.decay_rank], self.w_a2)
        o = ops.gated_delta(qkv, y[:, b0:b0 + H], a, gate, self.a_log, self.dt_bias, self.norm_w, self.eps, matrix_state.state,
                            step, H, self.kv_heads, self.dim, self.vdim, write_cache, UNIT_EPS,
                            channel_decay=self.decay == "channel", gate_act=self.gate_act)
        return ops.linear(o, self.w_o)


register_part("mixer", "gated_delta", GatedDelta)
