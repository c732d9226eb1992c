"""The Lolivik design as a list of layers made from parts.

Every layer is a post-norm residual block: its sublayers read the residual stream itself, and each sublayer's output passes
an RMS norm and a factor before it joins the stream.  Three mixers: grouped-query attention without rotation whose queries
and keys are normed over the whole projection, whose queries grow with the logarithm of the position, and whose scores are
capped, get a learned bias by distance and share the softmax with a sink; a matrix memory with log gates; and grouped-query
attention with per-head norms, a partial rotation of pairs (2i, 2i+1) with frequencies stretched by wavelength, and a
sliding window that keeps the request's first positions.  Attention layers may mix their values with those of the first
layer that does.  The feed-forward is a dense gated unit (tanh GELU) or a mixture of bounded gated units chosen by softmax
scores, with a shared unit beside them.  Final norm, untied head.

Tensor names: `embed`, `head`, `final.norm`, and per layer i `l<i>.norm1`, `norm2`, `l<i>.mix.<tensor>` (a norm's weight:
the tensor's name + `.norm`, a bias + `.b`), `l<i>.mlp.gate`, `up`, `down`, or `l<i>.mlp.router`, `l<i>.mlp.e<n>.gate`, `up`,
`down` and `l<i>.mlp.shared.gate`, `up`, `down`.
"""
from __future__ import annotations

from ..config.base import ConfigError, register_architecture
from ..config.lolivik import ARCHITECTURE, LolivikConfig
from ..parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec

ATTENTION_NAMES = {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_norm": "mix.q.norm", "k_norm": "mix.k.norm",
                   "rel": "mix.rel", "sink": "mix.sink", "vmix": "mix.vmix"}
MLSTM_NAMES = {"q": "mix.q", "k": "mix.k", "v": "mix.v", "g": "mix.g", "i": "mix.i", "i_bias": "mix.i.b", "f": "mix.f",
               "f_bias": "mix.f.b", "norm": "mix.norm", "o": "mix.o"}
MLP_NAMES = {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}
EXPERT_NAMES = {"router": "mlp.router", "gate": "mlp.e{e}.gate", "up": "mlp.e{e}.up", "down": "mlp.e{e}.down"}
SHARED_NAMES = {"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"}
UNIT_ALPHA = 1.702          # the bounded gated unit's sigmoid slope: a constant of the design


def mixer_spec(cfg: LolivikConfig, i: int, kind: str, m: dict, v_mix) -> PartSpec:
    W, eps = cfg.width, cfg.norm_eps
    if kind == "mlstm":
        return PartSpec("mlstm", dict(hidden=W, heads=m["heads"], dim=m["dim"], vdim=m["vdim"], gate_cap=m["gate_cap"], eps=eps,
                                      names=MLSTM_NAMES))
    common = dict(hidden=W, heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"], qk_norm=True, eps=eps,
                  scale=m["scale"], v_mix=v_mix, names=ATTENTION_NAMES)
    if kind == "attention":
        if "bias_rows" not in m:
            raise ConfigError(f"layers[{i}].mixer: the rows of the distance-bias table come from the stored tensor l{i}.mix.rel "
                              f"(or from the key bias_rows)")
        return PartSpec("attention", dict(
            common, position=PartSpec("none", {}), norm_scope="whole", q_temp=(m["q_temp"]["coef"], m["q_temp"]["every"]),
            softcap=m["softcap"], rel_bias={"rows": m["bias_rows"], "max": m["bias_max"]}, sink=True))
    rot = m["rot"]
    scaling = None if rot["scaling"] is None else dict(rot["scaling"], kind="wavelength")
    position = PartSpec("rotary_interleaved", dict(head_dim=m["dim"], theta=rot["base"], rotary_dim=rot["dims"], scaling=scaling)) \
        if rot["dims"] else PartSpec("none", {})
    return PartSpec("attention", dict(common, position=position, norm_scope="head", window=m["mask"]["size"],
                                      keep_first=m["mask"]["keep_first"]))


def feed_forward_spec(cfg: LolivikConfig, mlp: dict) -> PartSpec:
    W = cfg.width
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", dict(hidden=W, ff_dim=mlp["ff"], activation="gelu_tanh", names=MLP_NAMES))
    shared = None
    if mlp.get("shared"):
        shared = PartSpec("clamped_glu", dict(hidden=W, ff_dim=mlp["shared"]["ff"], limit=mlp["shared"]["limit"], alpha=UNIT_ALPHA,
                                              names=SHARED_NAMES))
    return PartSpec("routed_experts", dict(
        hidden=W, ff_dim=mlp["expert"]["ff"], experts=mlp["router"]["experts"], top=mlp["router"]["top"], renormalize=True,
        weight_on="output", score="softmax", expert_act="clamped", limit=mlp["expert"]["limit"], alpha=UNIT_ALPHA, shared=shared,
        names=EXPERT_NAMES))


def build_spec(cfg: LolivikConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm", dict(size=W, eps=eps, weight=name))
    layers, order, mixing_seen = [], [], False
    for i, layer in enumerate(cfg.layers):
        v_mix = None
        if layer["mixer"].get("v_mix"):
            v_mix, mixing_seen = ("mix" if mixing_seen else "first"), True
        block = dict(mixer=mixer_spec(cfg, i, layer["type"], layer["mixer"], v_mix), mixer_norm=norm("norm1"), mult=cfg.residual_mult)
        if layer["mlp"] is not None:
            block.update(feed_forward=feed_forward_spec(cfg, layer["mlp"]), ff_norm=norm("norm2"))
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("postnorm_residual", block)))
        order.append(LayerCall(i))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("embedding", dict(weight="embed")),
        layers=layers, order=order, final_norm=norm("final.norm"), head=PartSpec("linear_head", dict(weight="head", tied=False)))


register_architecture(ARCHITECTURE, LolivikConfig, build_spec, replace=True)
