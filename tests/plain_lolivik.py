"""The Lolivik design, plainly: whole sequences, one function per mechanism, 64-bit unless told otherwise, no cache and no
code shared with the package.  `forward(cfg, tensors, tokens)` returns the logits of every position (and, on request,
the residual stream after every layer); `tensors` maps the stored names to torch tensors, `cfg` is config.json as a dict.

Notation: W x for a stored matrix W [out, in]; t, j positions of one sequence counted from 0; h the input of a sublayer.

    layer          x <- x + m * rms(mixer(x)) * w1 ;  x <- x + m * rms(ff(x)) * w2        (the sublayers read x itself)
    attention      q, k normed over the whole projection, q_t times 1 + c ln(floor((t + 1) / every) + 1),
                   s_tj = cap tanh(q_t . k_j scale / cap) + rel[bucket(t - j), head],  j <= t,
                   weights exp(s_tj) / (sum_j exp(s_tj) + exp(sink_head)), values mixed with the first mixing layer's
    mlstm          a matrix memory per head with a scalar input gate and forget gate kept in logarithms and a running maximum
    attention_2    q, k normed per head, pairs (2i, 2i + 1) of the first dims turned by t f_i with stretched f_i,
                   j visible if j <= t and (t - j < size or j < keep_first), ordinary softmax, mixed values
    feed-forward   down(gelu_tanh(gate h) * up h), or `top` of `experts` bounded gated units by softmax score
                   (weights renormalised over the chosen) plus a shared unit
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def bucket(n: int, rows: int, far: float) -> int:
    """The row of the distance-bias table for a distance n >= 0: one row per distance below rows/2, then rows that
    widen geometrically up to the distance `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def value_mix(v, v_first, lam):
    return v if v_first is None else (1.0 - lam) * v + lam * v_first


def attention_bias(m, T, tensors, pre, dt):
    """The additive term of the scores [H, T, T] (distance bias) and the mask of visible pairs [T, T]."""
    rel = tensors[pre + "rel"].to(dt)
    B, H = rel.shape
    idx = torch.tensor([[bucket(t - j, B, m["bias_max"]) if j <= t else 0 for j in range(T)] for t in range(T)])
    return rel[idx].permute(2, 0, 1), torch.tril(torch.ones(T, T, dtype=torch.bool))


def attention(m, tensors, pre, h, eps, v_first, dt):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    W = lambda n: tensors[pre + n].to(dt)
    q, k, v = h @ W("q").T, h @ W("k").T, h @ W("v").T
    q, k = rms(q, eps) * W("q.norm"), rms(k, eps) * W("k.norm")
    pos = torch.arange(T, dtype=dt)
    temp = 1.0 + m["q_temp"]["coef"] * torch.log(torch.floor((pos + 1) / m["q_temp"]["every"]) + 1.0)
    q = q * temp[:, None]
    lam = W("vmix") if m.get("v_mix") else None
    v_mixed = value_mix(v, v_first if m.get("v_mix") else None, lam)
    qh = q.reshape(T, H, D).permute(1, 0, 2)
    kh = k.reshape(T, G, D).permute(1, 0, 2).repeat_interleave(H // G, dim=0)
    vh = v_mixed.reshape(T, G, Dv).permute(1, 0, 2).repeat_interleave(H // G, dim=0)
    s = qh @ kh.transpose(1, 2) * m["scale"]
    s = m["softcap"] * torch.tanh(s / m["softcap"])
    bias, visible = attention_bias(m, T, tensors, pre, dt)
    s = (s + bias).masked_fill(~visible[None], float("-inf"))
    sink = W("sink")
    top = torch.maximum(s.max(dim=-1).values, sink[:, None])
    e = torch.exp(s - top[..., None])
    p = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None] - top)[..., None])
    o = (p @ vh).permute(1, 0, 2).reshape(T, H * Dv)
    return o @ W("o").T, v_mixed


def stretched_frequencies(rot, dt):
    n = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / n) for i in range(n // 2)], dtype=torch.float64)
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f.tolist():
            wave = 2.0 * math.pi / fi
            if wave < sc["original"] / sc["high"]:
                out.append(fi)
            elif wave > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = torch.tensor(out, dtype=torch.float64)
    return f.to(dt)


def rotate_pairs(x, f):
    """x [T, heads, D]: the pairs (2i, 2i + 1), i < len(f), turn by t f_i; the rest passes."""
    T, n = x.shape[0], 2 * f.shape[0]
    a = torch.arange(T, dtype=f.dtype)[:, None] * f[None, :]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, w = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = u * cos - w * sin
    out[..., 1:n:2] = w * cos + u * sin
    return out


def attention_2(m, tensors, pre, h, eps, v_first, dt):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    W = lambda n: tensors[pre + n].to(dt)
    q, k, v = (h @ W("q").T).reshape(T, H, D), (h @ W("k").T).reshape(T, G, D), h @ W("v").T
    q, k = rms(q, eps) * W("q.norm"), rms(k, eps) * W("k.norm")
    f = stretched_frequencies(m["rot"], dt)
    q, k = rotate_pairs(q, f), rotate_pairs(k, f)
    lam = W("vmix") if m.get("v_mix") else None
    v_mixed = value_mix(v, v_first if m.get("v_mix") else None, lam)
    qh = q.permute(1, 0, 2)
    kh = k.permute(1, 0, 2).repeat_interleave(H // G, dim=0)
    vh = v_mixed.reshape(T, G, Dv).permute(1, 0, 2).repeat_interleave(H // G, dim=0)
    s = qh @ kh.transpose(1, 2) * m["scale"]
    t, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    visible = (j <= t) & ((t - j < m["mask"]["size"]) | (j < m["mask"]["keep_first"]))
    p = torch.softmax(s.masked_fill(~visible[None], float("-inf")), dim=-1)
    o = (p @ vh).permute(1, 0, 2).reshape(T, H * Dv)
    return o @ W("o").T, v_mixed


def mlstm(m, tensors, pre, h, eps, dt):
    T = h.shape[0]
    H, D, Dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    W = lambda n: tensors[pre + n].to(dt)
    q = (h @ W("q").T).reshape(T, H, D) * D ** -0.5
    k = (h @ W("k").T).reshape(T, H, D)
    v = (h @ W("v").T).reshape(T, H, Dv)
    gi = cap * torch.tanh((h @ W("i").T + W("i.b")) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ W("f").T + W("f.b")) / cap))
    out = torch.zeros(T, H, Dv, dtype=dt)
    for a in range(H):
        S, n, top = torch.zeros(D, Dv, dtype=dt), torch.zeros(D, dtype=dt), torch.zeros((), dtype=dt)
        for t in range(T):
            new = torch.maximum(gf[t, a] + top, gi[t, a])
            keep, take = torch.exp(gf[t, a] + top - new), torch.exp(gi[t, a] - new)
            S = keep * S + take * torch.outer(k[t, a], v[t, a])
            n = keep * n + take * k[t, a]
            top = new
            out[t, a] = (S.T @ q[t, a]) / (torch.maximum(torch.abs(n @ q[t, a]), torch.exp(-top)) + 1e-6)
    o = rms(out, eps).reshape(T, H * Dv) * W("norm") * torch.sigmoid(h @ W("g").T)
    return o @ W("o").T


def bounded_unit(tensors, pre, h, limit, dt):
    W = lambda n: tensors[pre + n].to(dt)
    g = torch.clamp(h @ W("gate").T, max=limit)
    u = torch.clamp(h @ W("up").T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W("down").T


def feed_forward(mlp, tensors, pre, h, dt, margins_out=None):
    """`margins_out`: a list that receives, for a mixture of experts, per token how far the last chosen score lies above the
    first one left out, as a share of the former (where that is tiny, a lower precision may choose otherwise)."""
    W = lambda n: tensors[pre + n].to(dt)
    if mlp["kind"] == "dense":
        return (gelu_tanh(h @ W("gate").T) * (h @ W("up").T)) @ W("down").T
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.softmax(h @ W("router").T, dim=-1)
    if margins_out is not None and top < E:
        ranked = s.sort(dim=-1, descending=True).values
        margins_out.append((ranked[:, top - 1] - ranked[:, top]) / ranked[:, top - 1])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top]
        total = sum(s[t, e] for e in chosen) + 1e-20
        for e in chosen:
            out[t] += s[t, e] / total * bounded_unit(tensors, f"{pre}e{e}.", h[t:t + 1], mlp["expert"]["limit"], dt)[0]
    if mlp.get("shared"):
        out = out + bounded_unit(tensors, pre + "shared.", h, mlp["shared"]["limit"], dt)
    return out


def forward(cfg, tensors, tokens, dt=torch.float64, layers_out=None, margins_out=None):
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = tensors["embed"].to(dt)[torch.tensor(tokens, dtype=torch.long)]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "mlstm":
            y = mlstm(m, tensors, pre + "mix.", x, eps, dt)
        else:
            fn = attention if layer["type"] == "attention" else attention_2
            y, v = fn(m, tensors, pre + "mix.", x, eps, v_first, dt)
            if m.get("v_mix") and v_first is None:
                v_first = v
        x = x + mult * rms(y, eps) * tensors[pre + "norm1"].to(dt)
        if layer["mlp"] is not None:
            y = feed_forward(layer["mlp"], tensors, pre + "mlp.", x, dt, margins_out)
            x = x + mult * rms(y, eps) * tensors[pre + "norm2"].to(dt)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms(x, eps) * tensors["final.norm"].to(dt)
    return x @ tensors["head"].to(dt).T
