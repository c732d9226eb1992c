"""Configuration of the Lolivik design, read from its own config.json keys.

    architecture      "Lolivik"
    vocab, width      vocabulary and model width
    norm.eps          eps of every RMS norm (inside the root)
    residual_mult     factor on every normed sublayer output before it joins the residual stream
    layers            one entry per layer: `type` (which mixer), `mixer` (its sizes and constants) and `mlp`
                      (null, {kind: "dense", ff}, or {kind: "moe", expert: {ff, limit}, router: {experts, top},
                      shared: {ff, limit} or null})

Mixers by `type`:
    attention     heads, kv_heads, dim, vdim, scale, softcap, bias_max, q_temp {coef, every}, v_mix; the number of rows of
                  its distance-bias table is the first dimension of the stored `l<i>.mix.rel`
    mlstm         heads, dim, vdim, gate_cap
    attention_2   heads, kv_heads, dim, vdim, scale, mask {size, keep_first}, rot {base, dims, scaling {factor, low, high,
                  original} or null}, v_mix
Every size and constant comes from the file (or a tensor's shape); nothing is assumed equal to anything else.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .base import ConfigError, ModelConfig, read_key

ARCHITECTURE = "Lolivik"
MAX_POSITIONS = 1 << 20      # the design names no limit; block tables and graphs are sized by the cache, not by this
MIXERS = ("attention", "mlstm", "attention_2")


def _object(d, key, where, required=True):
    v = d.get(key) if isinstance(d, dict) else None
    if v is None and not required:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: required key '{key}' should be an object")
    return v


def _sizes(m, names, where):
    out = {k: read_key(m, k, int, where=where) for k in names}
    for k, v in out.items():
        if v < 1:
            raise ConfigError(f"{where}: '{k}' should be at least 1, got {v}")
    return out


def _heads(m, where):
    out = _sizes(m, ("heads", "kv_heads", "dim", "vdim"), where)
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"{where}: heads should be a multiple of kv_heads")
    out["scale"] = read_key(m, "scale", float, where=where)
    out["v_mix"] = read_key(m, "v_mix", bool, default=False, where=where)
    return out


def _attention(m, where):
    out = _heads(m, where)
    out["softcap"] = read_key(m, "softcap", float, where=where)
    out["bias_max"] = read_key(m, "bias_max", float, where=where)
    temp = _object(m, "q_temp", where)
    out["q_temp"] = {"coef": read_key(temp, "coef", float, where=where + ".q_temp"),
                     "every": read_key(temp, "every", int, where=where + ".q_temp")}
    if out["softcap"] <= 0 or out["q_temp"]["every"] < 1:
        raise ConfigError(f"{where}: softcap should be positive and q_temp.every at least 1")
    if m.get("bias_rows") is not None:
        out["bias_rows"] = read_key(m, "bias_rows", int, where=where)
    return out


def _attention_2(m, where):
    out = _heads(m, where)
    mask, rot = _object(m, "mask", where), _object(m, "rot", where)
    out["mask"] = {"size": read_key(mask, "size", int, where=where + ".mask"),
                   "keep_first": read_key(mask, "keep_first", int, default=0, where=where + ".mask")}
    if out["mask"]["size"] < 1 or out["mask"]["keep_first"] < 0:
        raise ConfigError(f"{where}.mask: size should be at least 1 and keep_first not negative")
    out["rot"] = {"base": read_key(rot, "base", float, where=where + ".rot"), "dims": read_key(rot, "dims", int, where=where + ".rot")}
    if out["rot"]["base"] <= 0 or out["rot"]["dims"] % 2 or not 0 <= out["rot"]["dims"] <= out["dim"]:
        raise ConfigError(f"{where}.rot: base should be positive, dims even and at most dim")
    sc = _object(rot, "scaling", where + ".rot", required=False)
    out["rot"]["scaling"] = None
    if sc is not None:
        out["rot"]["scaling"] = {k: read_key(sc, k, float, where=where + ".rot.scaling") for k in ("factor", "low", "high", "original")}
        if out["rot"]["scaling"]["high"] == out["rot"]["scaling"]["low"]:
            raise ConfigError(f"{where}.rot.scaling: low and high should differ")
    return out


def _mlstm(m, where):
    out = _sizes(m, ("heads", "dim", "vdim"), where)
    out["gate_cap"] = read_key(m, "gate_cap", float, where=where)
    if out["gate_cap"] <= 0:
        raise ConfigError(f"{where}: gate_cap should be positive")
    return out


def _unit(d, where):
    out = {"ff": read_key(d, "ff", int, where=where), "limit": read_key(d, "limit", float, where=where)}
    if out["ff"] < 1 or out["limit"] <= 0:
        raise ConfigError(f"{where}: ff and limit should be positive")
    return out


def _mlp(mlp, where):
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"{where} should be an object or null")
    kind = read_key(mlp, "kind", str, where=where)
    if kind == "dense":
        out = {"kind": kind, "ff": read_key(mlp, "ff", int, where=where)}
        if out["ff"] < 1:
            raise ConfigError(f"{where}: ff should be positive")
        return out
    if kind == "moe":
        router = _object(mlp, "router", where)
        out = {"kind": kind, "expert": _unit(_object(mlp, "expert", where), where + ".expert"),
               "router": {"experts": read_key(router, "experts", int, where=where + ".router"),
                          "top": read_key(router, "top", int, where=where + ".router")}}
        if not 1 <= out["router"]["top"] <= out["router"]["experts"]:
            raise ConfigError(f"{where}: 1 <= router.top <= router.experts")
        shared = _object(mlp, "shared", where, required=False)
        out["shared"] = None if shared is None else _unit(shared, where + ".shared")
        return out
    raise ConfigError(f"{where}: unknown kind '{kind}'; known: dense, moe")


@dataclass
class LolivikConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    residual_mult: float = 1.0
    layers: List[Dict[str, Any]] = field(default_factory=list)
    max_positions: int = MAX_POSITIONS

    # the names the engine and the command line use for every architecture
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LolivikConfig":
        vocab, width = read_key(d, "vocab", int), read_key(d, "width", int)
        if vocab < 1 or width < 1:
            raise ConfigError("vocab and width should be positive")
        norm = _object(d, "norm", "config.json")
        layers_in = read_key(d, "layers", list)
        if not layers_in:
            raise ConfigError("'layers' should list at least one layer")
        layers, mixed_width = [], None
        readers = {"attention": _attention, "mlstm": _mlstm, "attention_2": _attention_2}
        for i, entry in enumerate(layers_in):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where} should be an object")
            kind = read_key(entry, "type", str, where=where)
            if kind not in readers:
                raise ConfigError(f"{where}: unknown mixer type '{kind}'; known: {', '.join(MIXERS)}")
            m = readers[kind](_object(entry, "mixer", where), where + ".mixer")
            if m.get("v_mix"):
                # mixed values are sums of two layers' value rows: all mixing layers have rows of one width
                mine = m["kv_heads"] * m["vdim"]
                if mixed_width is not None and mine != mixed_width:
                    raise ConfigError(f"{where}.mixer: layers with v_mix should have equal kv_heads * vdim ({mine} != {mixed_width})")
                mixed_width = mine
            layers.append({"type": kind, "mixer": m, "mlp": _mlp(entry.get("mlp"), where + ".mlp")})
        return cls(ARCHITECTURE, vocab=vocab, width=width, norm_eps=read_key(norm, "eps", float, where="norm"),
                   residual_mult=read_key(d, "residual_mult", float, default=1.0), layers=layers,
                   max_positions=read_key(d, "max_positions", int, default=MAX_POSITIONS))

    def complete(self, shapes) -> None:
        """The rows of an attention layer's distance-bias table, where config.json does not give them: the first
        dimension of the stored `l<i>.mix.rel`."""
        for i, layer in enumerate(self.layers):
            name = f"l{i}.mix.rel"
            if layer["type"] == "attention" and "bias_rows" not in layer["mixer"] and name in shapes and len(shapes[name]) == 2:
                layer["mixer"]["bias_rows"] = int(shapes[name][0])

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "residual_mult": self.residual_mult, "layers": copy.deepcopy(self.layers)}
        if self.max_positions != MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out
