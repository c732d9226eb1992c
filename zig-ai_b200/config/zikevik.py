"""Configuration of the Zikevik design, read from its own config.json keys.

    architecture      "Zikevik"
    vocab, width      vocabulary and model width
    embedding.scale   factor on the embedding rows
    norm.eps          eps of every RMS norm (layer norms, the latents' norms, the delta rule's output norm), inside the root
    layers            one entry per layer: `type` (which mixer), `mixer` (its sizes and constants), `mlp` (null,
                      {kind: "dense", ff}, or {kind: "moe", expert: {ff}, router: {experts, top}}), and optionally
                      `weights_of`: the earlier layer whose tensors this layer uses (with a cache and state of its own)

Mixers by `type`:
    channel_delta     heads, kv_heads, dim, vdim, conv: the gated delta rule with a decay per head and key channel; the inner
                      sizes of its two low-rank projections are read from the stored tensors' shapes
    latent_attention  heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {base, dims}
Every size and constant comes from the file; nothing is assumed equal to anything else.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .base import ConfigError, ModelConfig, read_key

ARCHITECTURE = "Zikevik"
MAX_POSITIONS = 1 << 20      # the design names no limit; block tables and graphs are sized by the cache, not by this
MIXERS = ("channel_delta", "latent_attention")


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


def _channel_delta(m, where):
    out = _sizes(m, ("heads", "kv_heads", "dim", "vdim", "conv"), where)
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"{where}: heads should be a multiple of kv_heads")
    # inner sizes of the decay's and the gate's projections: optional here, else taken from the tensors' shapes at load
    for k in ("decay_rank", "gate_rank"):
        if m.get(k) is not None:
            out[k] = read_key(m, k, int, where=where)
            if out[k] < 1:
                raise ConfigError(f"{where}: '{k}' should be at least 1")
    return out


def _latent(m, where):
    out = _sizes(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"), where)
    out["scale"] = read_key(m, "scale", float, where=where)
    rot = _object(m, "rot", where)
    out["rot"] = {"base": read_key(rot, "base", float, where=where + ".rot"), "dims": read_key(rot, "dims", int, where=where + ".rot")}
    if out["rot"]["base"] <= 0:
        raise ConfigError(f"{where}.rot: base should be positive")
    if out["rot_dim"] % 2 or out["rot"]["dims"] != out["rot_dim"]:
        raise ConfigError(f"{where}: rot_dim should be even and rot.dims equal to it (the whole shared key part is rotated)")
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
        expert, router = _object(mlp, "expert", where), _object(mlp, "router", where)
        out = {"kind": kind, "expert": {"ff": read_key(expert, "ff", int, where=where + ".expert")},
               "router": {"experts": read_key(router, "experts", int, where=where + ".router"),
                          "top": read_key(router, "top", int, where=where + ".router")}}
        if out["expert"]["ff"] < 1 or not 1 <= out["router"]["top"] <= out["router"]["experts"]:
            raise ConfigError(f"{where}: expert.ff should be positive and 1 <= router.top <= router.experts")
        return out
    raise ConfigError(f"{where}: unknown kind '{kind}'; known: dense, moe")


@dataclass
class ZikevikConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    embedding_scale: float = 1.0
    norm_eps: float = 1e-6
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
    def from_dict(cls, d: Dict[str, Any]) -> "ZikevikConfig":
        vocab, width = read_key(d, "vocab", int), read_key(d, "width", int)
        if vocab < 1 or width < 1:
            raise ConfigError("vocab and width should be positive")
        norm = _object(d, "norm", "config.json")
        embedding = _object(d, "embedding", "config.json")
        layers_in = read_key(d, "layers", list)
        if not layers_in:
            raise ConfigError("'layers' should list at least one layer")
        layers = []
        for i, entry in enumerate(layers_in):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where} should be an object")
            kind = read_key(entry, "type", str, where=where)
            m = _object(entry, "mixer", where)
            if kind == "channel_delta":
                m = _channel_delta(m, where + ".mixer")
            elif kind == "latent_attention":
                m = _latent(m, where + ".mixer")
            else:
                raise ConfigError(f"{where}: unknown mixer type '{kind}'; known: {', '.join(MIXERS)}")
            layer = {"type": kind, "mixer": m, "mlp": _mlp(entry.get("mlp"), where + ".mlp")}
            if entry.get("weights_of") is not None:
                src = read_key(entry, "weights_of", int, where=where)
                if not 0 <= src < i or "weights_of" in layers[src]:
                    raise ConfigError(f"{where}: weights_of should name an earlier layer that has tensors of its own")
                theirs = {k: v for k, v in layers[src].items() if k != "weights_of"}
                if theirs != layer:
                    raise ConfigError(f"{where}: a layer that uses layer {src}'s tensors should equal it in type, mixer and mlp")
                layer["weights_of"] = src
            layers.append(layer)
        return cls(ARCHITECTURE, vocab=vocab, width=width, embedding_scale=read_key(embedding, "scale", float, where="embedding"),
                   norm_eps=read_key(norm, "eps", float, where="norm"), layers=layers,
                   max_positions=read_key(d, "max_positions", int, default=MAX_POSITIONS))

    def complete(self, shapes) -> None:
        """The inner sizes of a delta layer's decay and gate projections, where config.json does not give them: the
        first dimension of the stored `l<i>.mix.a1` and `l<i>.mix.g1`."""
        for i, layer in enumerate(self.layers):
            if layer["type"] != "channel_delta":
                continue
            src = layer.get("weights_of", i)
            for key, tensor in (("decay_rank", f"l{src}.mix.a1"), ("gate_rank", f"l{src}.mix.g1")):
                if key not in layer["mixer"] and tensor in shapes and len(shapes[tensor]) == 2:
                    layer["mixer"][key] = int(shapes[tensor][0])

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "embedding": {"scale": self.embedding_scale},
               "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}
        if self.max_positions != MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out
