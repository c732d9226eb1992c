"""A plain, slow implementation of the Zikevik design: whole sequences, no cache, one function per
mechanism, float64 on the CPU.  It shares no code with the engine: the configuration is read as a
dict and the tensors as a dict of float64 tensors by stored name.

The design in short (T tokens, width W):

    x_0    = table[token] * embedding.scale
    layer:   x += mixer(rms(x) * (1 + norm1));   x += ff(rms(x) * (1 + norm2))      (ff optional)
    logits = head . (rms(x) * (1 + final.norm))

with two kinds of mixer: a gated delta rule whose state decays per key channel (`channel_delta`: short
convolutions, unit-length q and k, a low-rank decay projection, a low-rank sigmoid output gate) and causal
attention over a shared low-rank latent (`latent_attention`: queries through a normed latent of their own,
pairwise-interleaved rotation, a sink in the softmax's denominator, one sigmoid gate per head); and two
kinds of feed-forward: a dense gated one and a mixture of small gated ones with a sigmoid router whose
weights scale the experts' inputs.  A layer may use another layer's tensors (`weights_of`).
"""
from __future__ import annotations

import json
import math
import os

import torch

F64 = torch.float64
UNIT_EPS = 1e-6            # inside the root of the unit norms of q and k


def read_config(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_weights(model_dir):
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(F64)
    return out


# ----------------------------------------------------------------------------- small pieces
def rms(x, eps, weight=None):
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def offset_norm(x, w, eps):
    """RMS norm whose stored weight lies around zero."""
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def short_conv(x, taps):
    """x [T, C], taps [C, L]: y[t, c] = sum_i taps[c, L-1-i] x[t-i, c], zeros before the start."""
    T, C = x.shape
    L = taps.shape[1]
    y = torch.zeros_like(x)
    for i in range(L):
        if i < T:
            y[i:] += taps[:, L - 1 - i] * x[:T - i]
    return y


def rotate_pairs(x, positions, base, dims):
    """x [T, heads, D]: the pair (x[2i], x[2i+1]), i < dims/2, turns by position * base^(-2i/dims)."""
    i = torch.arange(dims // 2, dtype=F64)
    ang = (positions.to(F64)[:, None] * base ** (-2.0 * i / dims))[:, None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- the delta rule with a decay per key channel
def channel_delta(h, m, w, p, eps):
    """h [T, W]; m the mixer's sizes; w the tensors; p the prefix '<layer>.mix.'."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, D)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, D)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + UNIT_EPS) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + UNIT_EPS)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                        # [T, H]
    a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]                   # [T, H * D]
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * softplus(a).view(T, H, D))
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=F64)
    for head in range(H):
        kv = head // (H // G)
        S = torch.zeros(D, V, dtype=F64)
        for t in range(T):
            S = g[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, head] = S.T @ q[t, kv]
    out = rms(out, eps, w[p + "norm"]) * gate
    return out.reshape(T, H * V) @ w[p + "o"].T


# ----------------------------------------------------------------------------- attention over a latent, with a sink
def latent_attention(h, m, w, p, eps):
    T = h.shape[0]
    H, D, Dr, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms(h @ w[p + "dq"].T, eps, w[p + "dq.norm"])
    q = (cq @ w[p + "uq"].T).view(T, H, D + Dr)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], pos, m["rot"]["base"], m["rot"]["dims"])
    d = h @ w[p + "dkv"].T
    c = rms(d[:, :R], eps, w[p + "dkv.norm"])
    k_rot = rotate_pairs(d[:, None, R:], pos, m["rot"]["base"], m["rot"]["dims"])[:, 0]       # [T, Dr], one for all heads
    k_plain = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, Dv)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    s = s.masked_fill(pos[None, :] > pos[:, None], -math.inf)
    # the sink: one more term in the denominator, with no value
    sink = w[p + "sink"][:, None, None].expand(H, T, 1)
    prob = torch.softmax(torch.cat([s, sink], dim=-1), dim=-1)[..., :T]
    o = torch.einsum("hij,jhd->ihd", prob, v)
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * Dv) @ w[p + "o"].T


# ----------------------------------------------------------------------------- feed-forwards
def gated_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_ff(h, mlp, w, p, margins_out=None):
    """Every token goes to its `top` experts by sigmoid score; an expert sees score * h.  `margins_out`: a list that
    receives, per token, how far the last chosen expert's router logit lies above the first one not chosen."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[p + "router"].T                                      # [T, E]
    s = torch.sigmoid(z)
    chosen = torch.topk(s, top, dim=-1).indices
    if margins_out is not None:
        zs = z.sort(dim=-1, descending=True).values
        margins_out.append(zs[:, top - 1] - zs[:, top] if top < E else torch.full((h.shape[0],), math.inf, dtype=F64))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += gated_ff((s[t, e] * h[t])[None], w, f"{p}e{e}.")[0]
    return out


def feed_forward(h, mlp, w, p, margins_out=None):
    if mlp["kind"] == "dense":
        return gated_ff(h, w, p)
    if mlp["kind"] == "moe":
        return routed_ff(h, mlp, w, p, margins_out)
    raise ValueError(mlp["kind"])


# ----------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, layers_out=None, margins_out=None):
    """Logits [T, vocab] of one sequence.  `layers_out`: a list that receives the stream after every layer;
    `margins_out`: one that receives every routed layer's margins (see routed_ff)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        p = f"l{src}."
        n = offset_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "channel_delta":
            x = x + channel_delta(n, layer["mixer"], w, p + "mix.", eps)
        elif layer["type"] == "latent_attention":
            x = x + latent_attention(n, layer["mixer"], w, p + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + feed_forward(offset_norm(x, w[p + "norm2"], eps), layer["mlp"], w, p + "mlp.", margins_out)
        if layers_out is not None:
            layers_out.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T
