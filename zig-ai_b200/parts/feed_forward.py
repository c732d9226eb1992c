"""SwiGLU feed-forward: `down( silu(gate(x)) * up(x) )`, no biases
(src/transformer/ffn.zig:7-34; device activation src/cuda/layer_kernels.cu:62-70; tensor names
src/transformer/hybrid_layer.zig:313-321).  The gate and up matrices are stacked into one
[2F, hidden] matrix at load so that one product feeds the activation.
"""
from __future__ import annotations

import torch

from .base import FeedForward, ParamDecl, make_part, register_part


class SwiGlu(FeedForward):
    """`names` gives the three tensors' names (gate, up, down).  `activation`: what the gate passes, silu by default, or
    one of gelu (erf), gelu_tanh, relu: `down( act(gate(x)) * up(x) )`."""
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True      # forward launches kernels only; nothing is read back to the host
    kernel_libs = ("gemm_tc_pair",)       # gate/up products of many rows with the activation as their epilogue (bfloat16)

    def __init__(self, hidden: int, ff_dim: int, names=None, activation: str = "silu"):
        self.hidden, self.ff_dim, self.activation = int(hidden), int(ff_dim), str(activation)
        if self.activation not in ("silu", "gelu", "gelu_erf", "gelu_tanh", "relu"):
            raise ValueError(f"unknown activation '{self.activation}'")
        self.names = {"gate": "ffn_gate.weight", "up": "ffn_up.weight", "down": "ffn_down.weight", **(names or {})}

    def params(self):
        nm = self.names
        return {
            nm["gate"]: ParamDecl((self.ff_dim, self.hidden)),
            nm["up"]: ParamDecl((self.ff_dim, self.hidden)),
            nm["down"]: ParamDecl((self.hidden, self.ff_dim)),
        }

    def bind(self, tensors, dtype):
        nm = self.names
        self.w_gate_up = torch.cat([tensors[nm["gate"]], tensors[nm["up"]]], dim=0).contiguous()
        self.w_down = tensors[nm["down"]]
        self.dtype = dtype

    def forward(self, x, step):
        ops = step.ops
        if self.activation == "silu":
            a = ops.linear_swiglu(x, self.w_gate_up, self.ff_dim)
        else:
            a = ops.linear_glu(x, self.w_gate_up, self.ff_dim, self.activation)
        return ops.linear(a, self.w_down)


class DenseMlp(FeedForward):
    """`down( act(up(x)) )`, no gate and no biases; `activation` is one of gelu (the exact one, with erf),
    gelu_tanh, silu, relu.  `names` gives the two tensors' names."""
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True

    def __init__(self, hidden: int, ff_dim: int, activation: str = "gelu", names=None):
        self.hidden, self.ff_dim, self.activation = int(hidden), int(ff_dim), str(activation)
        if self.activation not in ("gelu", "gelu_erf", "gelu_tanh", "silu", "relu"):
            raise ValueError(f"unknown activation '{self.activation}'")
        self.names = {"up": "ffn_up.weight", "down": "ffn_down.weight", **(names or {})}

    def params(self):
        return {self.names["up"]: ParamDecl((self.ff_dim, self.hidden)),
                self.names["down"]: ParamDecl((self.hidden, self.ff_dim))}

    def bind(self, tensors, dtype):
        self.w_up, self.w_down = tensors[self.names["up"]], tensors[self.names["down"]]
        self.dtype = dtype

    def forward(self, x, step):
        ops = step.ops
        return ops.linear(ops.linear_activation(x, self.w_up, self.activation), self.w_down)


class ClampedGlu(FeedForward):
    """A gated feed-forward with bounded branches, no biases:

        g = min(gate(x), limit);  u = clamp(up(x), -limit, limit);  out = down( g * sigmoid(alpha * g) * (u + 1) )

    The gate and up matrices are stacked into one [2F, hidden] matrix at load.  `names` gives the tensors' names."""
    accepts_lazy_input = True
    graph_safe = True

    def __init__(self, hidden: int, ff_dim: int, limit: float, alpha: float = 1.702, names=None):
        self.hidden, self.ff_dim, self.limit, self.alpha = int(hidden), int(ff_dim), float(limit), float(alpha)
        self.names = {"gate": "ffn_gate.weight", "up": "ffn_up.weight", "down": "ffn_down.weight", **(names or {})}

    def params(self):
        nm = self.names
        return {nm["gate"]: ParamDecl((self.ff_dim, self.hidden)), nm["up"]: ParamDecl((self.ff_dim, self.hidden)),
                nm["down"]: ParamDecl((self.hidden, self.ff_dim))}

    def bind(self, tensors, dtype):
        nm = self.names
        self.w_gate_up = torch.cat([tensors[nm["gate"]], tensors[nm["up"]]], dim=0).contiguous()
        self.w_down = tensors[nm["down"]]
        self.dtype = dtype

    def forward(self, x, step):
        ops = step.ops
        return ops.linear(ops.linear_clamped_glu(x, self.w_gate_up, self.ff_dim, self.limit, self.alpha), self.w_down)


class RoutedExperts(FeedForward):
    """A mixture of `experts` small SwiGLU feed-forwards, of which every token uses `top`:

        s = sigmoid(x . Wr^T)                 router, 32-bit
        chosen = the `top` experts with the largest s;   w_e = s_e   (divided by their sum with `renormalize`)
        out = sum over chosen e of  down_e( silu(gate_e(w_e x)) * up_e(w_e x) )          weight_on="input"
                                or  w_e down_e( silu(gate_e(x)) * up_e(x) )              weight_on="output"

    Experts have no biases.  The router's matrix is kept in 32-bit.  `names`: "router", and "gate", "up", "down" with
    `{e}` standing for the expert's number.

    Options: `score="softmax"` (s = softmax of the router's logits over all experts; with `renormalize` the chosen scores
    are divided by their sum + 1e-20); `expert_act="clamped"` with `limit` and `alpha` (experts of the bounded form
    min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u, -limit, limit) + 1)); `shared`, the `PartSpec` of a feed-forward
    that every token passes beside its experts (its tensors under its own names) and whose output is added."""
    accepts_lazy_input = False    # the router and the experts read the normed rows themselves
    graph_safe = True             # routing stays on the device: forward launches kernels only
    kernel_libs = ("moe", "gemm_tc")      # (gemm_tc: the grouped products of steps with many rows an expert, bfloat16)

    def __init__(self, hidden: int, ff_dim: int, experts: int, top: int, renormalize: bool = False, weight_on: str = "input",
                 names=None, score: str = "sigmoid", expert_act: str = "silu", limit: float = 0.0, alpha: float = 1.702, shared=None):
        self.hidden, self.ff_dim, self.experts, self.top = int(hidden), int(ff_dim), int(experts), int(top)
        self.renormalize, self.weight_on = bool(renormalize), weight_on
        if not 1 <= self.top <= self.experts or self.top > 32:
            raise ValueError(f"a token uses between 1 and min(experts, 32) experts, not {self.top} of {self.experts}")
        if weight_on not in ("input", "output"):
            raise ValueError("weight_on is 'input' or 'output'")
        if score not in ("sigmoid", "softmax") or expert_act not in ("silu", "clamped"):
            raise ValueError("score is 'sigmoid' or 'softmax', expert_act 'silu' or 'clamped'")
        self.score, self.expert_act, self.limit, self.alpha = score, expert_act, float(limit), float(alpha)
        self.shared = None if shared is None else make_part("feed_forward", shared)
        if self.shared is not None:
            self.kernel_libs = type(self).kernel_libs + tuple(getattr(self.shared, "kernel_libs", ()))
        self.names = {"router": "ffn_router.weight", "gate": "ffn_gate.{e}.weight", "up": "ffn_up.{e}.weight",
                      "down": "ffn_down.{e}.weight", **(names or {})}

    def params(self):
        nm, p = self.names, {self.names["router"]: ParamDecl((self.experts, self.hidden), "vector", init="conv")}
        for e in range(self.experts):
            p[nm["gate"].format(e=e)] = ParamDecl((self.ff_dim, self.hidden))
            p[nm["up"].format(e=e)] = ParamDecl((self.ff_dim, self.hidden))
            p[nm["down"].format(e=e)] = ParamDecl((self.hidden, self.ff_dim))
        if self.shared is not None:
            p.update(self.shared.params())
        return p

    def bind(self, tensors, dtype):
        nm, E = self.names, range(self.experts)
        if self.shared is not None:
            self.shared.bind({k: tensors[k] for k in self.shared.params()}, dtype)
        self.w_router = tensors[nm["router"]].float().contiguous()
        self.w_gate_up = torch.stack([torch.cat([tensors[nm["gate"].format(e=e)], tensors[nm["up"].format(e=e)]], dim=0)
                                      for e in E]).contiguous()                                  # [E, 2F, hidden]
        self.w_down = torch.stack([tensors[nm["down"].format(e=e)] for e in E]).contiguous()   # [E, hidden, F]
        self.dtype = dtype

    def forward(self, x, step):
        ops = step.ops
        if self.score == "sigmoid" and self.expert_act == "silu":
            y = ops.routed_experts(x, self.w_router, self.w_gate_up, self.w_down, self.top, self.renormalize, self.weight_on)
        else:
            y = ops.routed_experts(x, self.w_router, self.w_gate_up, self.w_down, self.top, self.renormalize, self.weight_on,
                                   score=self.score, act=self.expert_act, limit=self.limit, alpha=self.alpha)
        if self.shared is None:
            return y
        return ops.weighted_sum(y, self.shared.forward(x, step), 1.0, 1.0)


register_part("feed_forward", "swiglu", SwiGlu)
register_part("feed_forward", "routed_experts", RoutedExperts)
register_part("feed_forward", "clamped_glu", ClampedGlu)
register_part("feed_forward", "dense", DenseMlp)
