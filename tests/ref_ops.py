"""Plain PyTorch versions of the engine's kernels, one function per kernel with the kernel's own
signature.  Two uses: each CUDA kernel is compared with its function here (`-m gpu`), and the
engine's host logic (step function, cache, scheduler) is run on the CPU with this module standing
in for the kernels (`-m "not gpu"`).  Never used by the engine itself.

Formulas: see tests/plain_lfm2.py for the citations of the reference; these functions add only
what the cache brings (pages, block tables, state slots).
"""
from __future__ import annotations

import torch

device_type = "cpu"


def require():
    return None


fuses_norm = False      # norms run on their own here


def _f(x):
    return x.to(torch.float32)


# ---- the status word, as the kernels keep it (csrc/common.cuh: ZaiStatusBit): an id outside its bound is
# replaced by id 0 and a bit is raised; the step's results are then void.
STATUS_BITS = {1: "a bounded wait inside a kernel ran out", 2: "a token id outside the vocabulary",
               4: "a block-table entry outside the page pool", 8: "a state slot outside the slots",
               16: "a position outside its request's block-table row"}
_status = torch.zeros(1, dtype=torch.int32)


def status_tensor(device=None):
    return _status


def read_status(device=None) -> int:
    v = int(_status.item())
    _status.zero_()
    return v


def describe_status(code: int) -> str:
    return "; ".join(text for bit, text in STATUS_BITS.items() if code & bit) or f"status {code}"


def _raise(bit: int) -> None:
    _status[0] |= bit


def _checked(ids, bound: int, bit: int):
    """`ids` with every entry outside [0, bound) replaced by 0 (and the bit raised if there is one)."""
    bad = (ids < 0) | (ids >= bound)
    if bool(bad.any()):
        _raise(bit)
        ids = torch.where(bad, torch.zeros_like(ids), ids)
    return ids


def embed(ids, table, scale=1.0):
    return _f(table[_checked(ids.long(), table.shape[0], 2)]) * scale


def _normed(delta, gamma, eps):
    d = _f(delta)
    return d * torch.rsqrt((d * d).mean(dim=-1, keepdim=True) + eps) * _f(gamma)


def add_rmsnorm(h, delta, w, eps, out_dtype, delta_gamma=None, delta_eps=0.0):
    if delta is not None:
        h += _f(delta) if delta_gamma is None else _normed(delta, delta_gamma, delta_eps)
    ms = (h * h).mean(dim=-1, keepdim=True)
    return (h * torch.rsqrt(ms + eps) * _f(w)).to(out_dtype)


def linear(x, w, out_dtype=None, bias=None):
    out_dtype = out_dtype or x.dtype
    if bias is not None:
        return (_f(x) @ _f(w).T + _f(bias)).to(out_dtype)
    if x.dtype == w.dtype and x.dtype != torch.float32 and x.device.type == "cuda":
        return (x @ w.T).to(out_dtype)
    return (_f(x) @ _f(w).T).to(out_dtype)


def linear_swiglu(x, w_gate_up, ff_dim):
    return silu_mul(linear(x, w_gate_up), ff_dim)


def silu_mul(gu, ff_dim):
    g, u = _f(gu[:, :ff_dim]), _f(gu[:, ff_dim:])
    return (g * torch.sigmoid(g) * u).to(gu.dtype)


def short_conv(bcx, conv_w, conv_b, state, step, taps, write_state=True):
    N, C3 = bcx.shape
    C = C3 // 3
    L = taps
    out = torch.empty((N, C), dtype=bcx.dtype, device=bcx.device)
    cu = step.cu_q.tolist()
    slots = _checked(step.slot_ids.long(), state.shape[0], 8).tolist()
    for s in range(step.n_seqs):
        a, b = cu[s], cu[s + 1]
        x = _f(bcx[a:b])
        u = x[:, :C] * x[:, 2 * C:]
        hist = state[slots[s]][:L - 1] if L > 1 else state[slots[s]][:0]
        full = torch.cat([hist, u], dim=0)                        # [(L-1)+n, C]
        y = torch.zeros_like(u)
        for j in range(L):
            y += full[j:j + (b - a)] * conv_w[:, j][None, :]
        if conv_b is not None:
            y += conv_b[None, :]
        out[a:b] = (x[:, C:2 * C] * y).to(bcx.dtype)
        if write_state and L > 1:
            state[slots[s]][:L - 1] = full[full.shape[0] - (L - 1):]
    return out


def linear_short_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state=True):
    return short_conv(linear(x, w_in), conv_w, conv_b, state, step, taps, write_state)


def _rms(x, w, eps):
    ms = (x * x).mean(dim=-1, keepdim=True)
    y = x * torch.rsqrt(ms + eps)
    return y * w if w is not None else y


def _rotate(x, positions, rotary_dim, theta, table=None):
    if rotary_dim == 0:
        return x
    half = rotary_dim // 2
    if table is not None:
        cos, sin = table[:, None, :, 0], table[:, None, :, 1]
    else:
        i = torch.arange(half, dtype=torch.float32, device=x.device)
        freq = torch.exp(-(2.0 * i / rotary_dim) * torch.log(torch.tensor(float(theta))))
        ang = positions.to(torch.float32)[:, None] * freq[None, :]
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:rotary_dim]
    out = x.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:rotary_dim] = a * sin + b * cos
    return out


def _page_rows(step, cache):
    """For every row of the step: (page id, offset inside the page)."""
    ps = cache.page_size
    pos = step.positions.long()
    bt = cache.block_table.long()
    idx = pos // ps
    outside = (idx < 0) | (idx >= bt.shape[1])
    if bool(outside.any()):
        _raise(16)
    page = bt[step.seq_idx.long(), torch.where(outside, torch.zeros_like(idx), idx)]
    page = torch.where(outside, torch.zeros_like(page), _checked(page, cache.pages.shape[0], 4))
    return page, pos % ps


def qk_norm_rope(qkv, q_w, k_w, eps, rotary_dim, theta, step, cache, heads, kv_heads, head_dim,
                 has_kv=True, write=True, return_k=False):
    N = qkv.shape[0]
    D = head_dim
    q = _f(qkv[:, :heads * D]).reshape(N, heads, D)
    if q_w is not None:
        q = _rms(q, q_w, eps)
    q = _rotate(q, step.positions, rotary_dim, theta).to(qkv.dtype).reshape(N, heads * D)
    k_out = None
    if has_kv:
        k = _f(qkv[:, heads * D:(heads + kv_heads) * D]).reshape(N, kv_heads, D)
        if k_w is not None:
            k = _rms(k, k_w, eps)
        k = _rotate(k, step.positions, rotary_dim, theta).to(qkv.dtype)
        v = qkv[:, (heads + kv_heads) * D:].reshape(N, kv_heads, D)
        if write:
            page, off = _page_rows(step, cache)
            cache.pages[page, 0, :, off, :] = k.to(cache.pages.dtype)
            cache.pages[page, 1, :, off, :] = v.to(cache.pages.dtype)
        if return_k:
            k_out = k.reshape(N, kv_heads * D)
    return q, k_out


def kv_write(k, v, step, cache, kv_heads, head_dim):
    N = k.shape[0]
    page, off = _page_rows(step, cache)
    cache.pages[page, 0, :, off, :] = k.reshape(N, kv_heads, head_dim).to(cache.pages.dtype)
    cache.pages[page, 1, :, off, :] = v.reshape(N, kv_heads, head_dim).to(cache.pages.dtype)


def paged_attention(q, step, cache, heads, kv_heads, head_dim, scale, window=None, chunk=None, softcap=None, bias=None, sink=None,
                    keep_first=0, impl=None):
    N = q.shape[0]
    D, ps = head_dim, cache.page_size
    out = torch.empty((N, heads * D), dtype=q.dtype, device=q.device)
    cu, ctx = step.cu_q.tolist(), step.ctx_lens.tolist()
    group = heads // kv_heads
    for s in range(step.n_seqs):
        a, b = cu[s], cu[s + 1]
        total = ctx[s] + (b - a)
        n_pages = -(-total // ps)
        if n_pages > cache.block_table.shape[1]:
            _raise(16)
        ids = _checked(cache.block_table[s, :n_pages].long(), cache.pages.shape[0], 4)
        ids = torch.cat([ids, ids.new_zeros(n_pages - ids.shape[0])])
        kv = _f(cache.pages[ids])                                  # [pages, 2, Hkv, ps, D]
        k = kv[:, 0].permute(1, 0, 2, 3).reshape(kv_heads, n_pages * ps, D)[:, :total]
        v = kv[:, 1].permute(1, 0, 2, 3).reshape(kv_heads, n_pages * ps, D)[:, :total]
        qs = _f(q[a:b]).reshape(b - a, heads, D).permute(1, 0, 2)   # [Hq, n, D]
        k = k.repeat_interleave(group, dim=0)
        v = v.repeat_interleave(group, dim=0)
        sc = torch.einsum("hnd,hkd->hnk", qs, k) * scale
        qpos = torch.arange(ctx[s], total, device=q.device)[:, None]
        kpos = torch.arange(total, device=q.device)[None, :]
        mask = kpos > qpos
        if softcap:
            sc = softcap * torch.tanh(sc / softcap)
        if bias is not None:                 # by distance, the table's last row for everything beyond it
            dist = torch.clamp(qpos - kpos, min=0, max=bias.shape[0] - 1)
            sc = sc + _f(bias)[dist].permute(2, 0, 1)
        if window is not None:
            mask = mask | ((kpos <= qpos - window) & (kpos >= int(keep_first or 0)))
        if chunk is not None:
            mask = mask | (kpos < qpos - qpos % chunk)
        sc = sc.masked_fill(mask[None], float("-inf"))
        if sink is not None:                 # one more term of the denominator, with no value
            sc = torch.cat([sc, _f(sink)[:, None, None].expand(heads, b - a, 1)], dim=-1)
            p = torch.softmax(sc, dim=-1)[..., :-1]
        else:
            p = torch.softmax(sc, dim=-1)
        o = torch.einsum("hnk,hkd->hnd", p, v).permute(1, 0, 2).reshape(b - a, heads * D)
        out[a:b] = o.to(q.dtype)
    return out


def add_cast(h, delta, out_dtype, delta_gamma=None, delta_eps=0.0):
    if delta is not None:
        h += _f(delta) if delta_gamma is None else _normed(delta, delta_gamma, delta_eps)
    return h.to(out_dtype) if out_dtype != h.dtype else h.clone()


def gather_add(h, pending, rows, pending_gamma=None, pending_eps=0.0):
    r = rows.long()
    out = h[r].clone()
    if pending is not None:
        out += _f(pending[r]) if pending_gamma is None else _normed(pending[r], pending_gamma, pending_eps)
    return out


def argmax(logits):
    """First index of the maximum of each row."""
    m = logits.max(dim=-1, keepdim=True).values
    V = logits.shape[-1]
    idx = torch.arange(V, device=logits.device)[None, :].expand_as(logits)
    return torch.where(logits == m, idx, V).min(dim=-1).values.to(torch.int32)


def sample(logits, temperature, top_k, top_p, u):
    """Row-wise sampling with given uniforms: temperature <= 0 is greedy; otherwise logits/T,
    top-k (values >= the k-th largest), top-p (shortest descending prefix reaching p), then the
    inverse CDF in index order over the kept set."""
    R, V = logits.shape
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    for r in range(R):
        T = float(temperature[r])
        if T <= 0:
            out[r] = argmax(logits[r:r + 1])[0]
            continue
        w = logits[r].to(torch.float64) / T
        k = int(top_k[r])
        if 0 < k < V:
            kth = torch.sort(w, descending=True).values[k - 1]
            w = torch.where(w >= kth, w, torch.tensor(float("-inf"), dtype=torch.float64, device=w.device))
        p = torch.softmax(w, dim=-1)
        tp = float(top_p[r])
        if tp < 1.0:
            sp, si = torch.sort(p, descending=True, stable=True)
            cum = torch.cumsum(sp, 0)
            cutoff = int((cum >= tp).nonzero()[0]) + 1 if bool((cum >= tp).any()) else V
            thresh = sp[cutoff - 1]
            p = torch.where(p >= thresh, p, torch.zeros_like(p))
        c = torch.cumsum(p, 0)
        target = float(u[r]) * float(c[-1])
        hit = (c >= target).nonzero()
        out[r] = int(hit[0]) if hit.numel() else V - 1
    return out


def repetition_penalty(logits, tokens, counts, offsets, penalty):
    off = offsets.tolist()
    for r in range(logits.shape[0]):
        p = float(penalty[r])
        for i in range(off[r], off[r + 1]):
            t = int(tokens[i])
            for _ in range(int(counts[i])):
                v = logits[r, t]
                logits[r, t] = v / p if v > 0 else (v * p if v < 0 else v)
    return logits


# ---- recurrent mixers and what goes with them (the kernels of csrc/causal_conv.cu, selective_scan.cu, min_gru.cu,
# gated_delta.cu, and the additions to activation.cu and rope_kv.cu)
def _silu(x):
    return x * torch.sigmoid(x)


def _softplus(x):
    return torch.where(x > 20, x, torch.log1p(torch.exp(torch.clamp(x, max=20))))


def activation(x, kind):
    v = _f(x)
    if kind in ("gelu", "gelu_erf"):
        y = 0.5 * v * (1.0 + torch.erf(v * 0.7071067811865476))
    elif kind == "gelu_tanh":
        y = 0.5 * v * (1.0 + torch.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))
    elif kind == "silu":
        y = _silu(v)
    elif kind == "relu":
        y = torch.relu(v)
    else:
        raise KeyError(kind)
    return y.to(x.dtype)


def linear_activation(x, w, kind):
    return activation(linear(x, w), kind)


def weighted_sum(a, b, wa, wb):
    return (wa * _f(a) + wb * _f(b)).to(a.dtype)


def _spans(step, state):
    cu = step.cu_q.tolist()
    slots = _checked(step.slot_ids.long(), state.shape[0], 8).tolist()
    return [(cu[s], cu[s + 1], slots[s]) for s in range(step.n_seqs) if cu[s + 1] > cu[s]]


def causal_conv(x, taps, bias, state, step, act=True, write_state=True):
    N, C = x.shape
    L = taps.shape[1]
    out = torch.empty((N, C), dtype=x.dtype, device=x.device)
    for a, b, slot in _spans(step, state):
        hist = state[slot][:L - 1] if L > 1 else state[slot][:0]
        full = torch.cat([hist, _f(x[a:b])], dim=0)
        y = torch.zeros((b - a, C), dtype=torch.float32, device=x.device)
        for j in range(L):
            y += full[j:j + (b - a)] * taps[:, j][None, :]
        if bias is not None:
            y += bias[None, :]
        out[a:b] = (_silu(y) if act else y).to(x.dtype)
        if write_state and L > 1:
            state[slot][:L - 1] = full[full.shape[0] - (L - 1):]
    return out


def selective_scan(x, proj, z, w_dt, b_dt, a_log, d_skip, state, step, dt_rank, write_state=True):
    N, I = x.shape
    S, R = a_log.shape[1], int(dt_rank)
    p = _f(proj)
    dt = _softplus(p[:, :R] @ _f(w_dt).T + b_dt)
    A = -torch.exp(a_log)
    xs = _f(x)
    y = torch.empty((N, I), dtype=torch.float32, device=x.device)
    for a, b, slot in _spans(step, state):
        h = state[slot].clone()
        for t in range(a, b):
            h = torch.exp(dt[t][:, None] * A) * h + (dt[t] * xs[t])[:, None] * p[t, R:R + S][None, :]
            y[t] = h @ p[t, R + S:R + 2 * S] + d_skip * xs[t]
        if write_state:
            state[slot] = h
    return (y * _silu(_f(z))).to(x.dtype)


def min_gru(zxg, b_z, b_x, state, step, write_state=True):
    N, W = zxg.shape[0], zxg.shape[1] // 3
    v = _f(zxg)
    z = torch.sigmoid(v[:, :W] + (b_z if b_z is not None else 0.0))
    u = v[:, W:2 * W] + (b_x if b_x is not None else 0.0)
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    out = torch.empty((N, W), dtype=torch.float32, device=zxg.device)
    for a, b, slot in _spans(step, state):
        s = state[slot].clone()
        for t in range(a, b):
            s = (1.0 - z[t]) * s + z[t] * cand[t]
            out[t] = s
        if write_state:
            state[slot] = s
    return (out * _silu(v[:, 2 * W:])).to(zxg.dtype)


def gated_delta(qkv, b, a, gate, a_log, dt_bias, norm_w, eps, state, step, heads, kv_heads, dim, vdim, write_state=True,
                unit_eps=1e-6, channel_decay=False, gate_act="silu"):
    N = qkv.shape[0]
    H, G, D, V = heads, kv_heads, dim, vdim
    x = _f(qkv)
    q = x[:, :G * D].reshape(N, G, D)
    k = x[:, G * D:2 * G * D].reshape(N, G, D)
    v = x[:, 2 * G * D:].reshape(N, H, V)
    q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + unit_eps) * D ** -0.5
    k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + unit_eps)
    beta = torch.sigmoid(_f(b))
    if channel_decay:                                            # one decay per head and key channel: [N, H, D]
        g = torch.exp(-torch.exp(a_log)[None, :, None] * _softplus(_f(a) + dt_bias).reshape(N, H, D))
    else:
        g = torch.exp(-torch.exp(a_log) * _softplus(_f(a) + dt_bias))[:, :, None].expand(N, H, D)
    rep = H // G
    o = torch.zeros((N, H, V), dtype=torch.float32, device=qkv.device)
    for lo, hi, slot in _spans(step, state):
        S = state[slot].clone()                                  # [H, D, V]
        for t in range(lo, hi):
            kt = k[t].repeat_interleave(rep, dim=0)              # [H, D]
            qt = q[t].repeat_interleave(rep, dim=0)
            S = g[t][:, :, None] * S
            u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, kt))
            S = S + kt[:, :, None] * u[:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, qt)
        if write_state:
            state[slot] = S
    o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * norm_w
    act = torch.sigmoid(_f(gate)) if gate_act == "sigmoid" else _silu(_f(gate))
    return (o * act.reshape(N, H, V)).reshape(N, H * V).to(qkv.dtype)


def value_norm_pad(qkv, heads, kv_heads, dim, vdim, eps, normed=True):
    N = qkv.shape[0]
    H, G, D, Dv = heads, kv_heads, dim, vdim
    Dp = max(D, Dv)
    x = _f(qkv)
    q = x[:, :H * D].reshape(N, H, D)
    k = x[:, H * D:(H + G) * D].reshape(N, G, D)
    v = x[:, (H + G) * D:].reshape(N, G, Dv)
    if normed:
        v = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)
    pad = lambda t: torch.nn.functional.pad(t, (0, Dp - t.shape[-1]))
    return torch.cat([pad(q).reshape(N, -1), pad(k).reshape(N, -1), pad(v).reshape(N, -1)], dim=1).to(qkv.dtype)


# ---- what the layer-norm, chunked-attention and latent-attention designs add (the kernels of csrc/layernorm.cu,
# qkv_prepare.cu, latent_attention.cu, and the additions to activation.cu, rope_kv.cu and attention*.cu)
def add_layernorm(h, delta, w, b, eps, out_dtype):
    if delta is not None:
        h += _f(delta)
    mu = h.mean(dim=-1, keepdim=True)
    d = h - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return (d * torch.rsqrt(var + eps) * _f(w) + _f(b)).to(out_dtype)


def stretched_frequencies(rotary_dim, theta, scaling):
    """(frequencies in 64-bit, factor on cos and sin) of a rotation, stretched if `scaling` = (factor, original, fast, slow)."""
    import math
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / rotary_dim)
    if scaling is None:
        return f, 1.0
    if scaling[0] == "wavelength":          # stretched by wavelength: (tag, factor, low, high, original)
        _, factor, low, high, original = scaling
        out = []
        for fi in f.tolist():
            wave = 2.0 * math.pi / fi
            if wave < original / high:
                out.append(fi)
            elif wave > original / low:
                out.append(fi / factor)
            else:
                smooth = (original / wave - low) / (high - low)
                out.append((1.0 - smooth) * fi / factor + smooth * fi)
        return torch.tensor(out, dtype=torch.float64), 1.0
    factor, original, fast, slow = scaling
    where = lambda turns: rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
    lo, hi = max(math.floor(where(fast)), 0), min(math.ceil(where(slow)), rotary_dim - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rope_table(step, rotary_dim, theta, device, scaling=None):
    key = ("rope", rotary_dim, float(theta), scaling)
    t = step.scratch.get(key)
    if t is None:
        f, mag = stretched_frequencies(rotary_dim, theta, scaling)
        ang = step.positions.to(torch.float64)[:, None] * f[None, :]
        t = torch.stack([torch.cos(ang) * mag, torch.sin(ang) * mag], dim=-1).to(torch.float32)
        step.scratch[key] = t
    return t


def qkv_prepare(y, q_w, k_w, eps, scope, table, rot, step, cache, heads, kv_heads, dim, vdim, cache_dim, write=True, temp=None,
                v_first=None, v_lambda=None):
    """From projection rows y = [q (H D) | k (G D) | v (G Dv) | ...]: RMS norm of q and k (scope 0 none, 1 per head,
    2 over the whole projection), rotation of pairs (i, i + rot/2) from the table, k and v into the pages (heads
    `cache_dim` wide, zeros behind their own values); returns q [N, H * cache_dim]."""
    N = y.shape[0]
    H, G, D, Dv, Dp = heads, kv_heads, dim, vdim, cache_dim
    q, k, v = _f(y[:, :H * D]), _f(y[:, H * D:(H + G) * D]), y[:, (H + G) * D:(H + G) * D + G * Dv]
    if scope == 2:
        q, k = _rms(q, q_w, eps), _rms(k, k_w, eps)
    q, k = q.reshape(N, H, D), k.reshape(N, G, D)
    if scope == 1:
        q, k = _rms(q, q_w, eps), _rms(k, k_w, eps)
    q, k = _rotate(q, step.positions, rot, 1.0, table), _rotate(k, step.positions, rot, 1.0, table)
    if temp:                                 # the queries' temperature, a step function of the position
        coef, every = temp
        q = q * (1.0 + coef * torch.log((torch.div(step.positions + 1, every, rounding_mode="floor") + 1).float()))[:, None, None]
    if v_first is not None:                  # values mixed with an earlier layer's values of the same rows
        v = ((1.0 - _f(v_lambda)) * _f(v) + _f(v_lambda) * _f(v_first)).to(y.dtype)
    pad = lambda t, n: torch.cat([t, t.new_zeros(t.shape[:-1] + (n - t.shape[-1],))], dim=-1)
    if write:
        page, off = _page_rows(step, cache)
        cache.pages[page, 0, :, off, :] = pad(k, Dp).to(cache.pages.dtype)
        cache.pages[page, 1, :, off, :] = pad(_f(v).reshape(N, G, Dv), Dp).to(cache.pages.dtype)
    return pad(q, Dp).to(y.dtype).reshape(N, H * Dp)


def sigmoid_gate(o, gate, heads, head_dim, per_head):
    """o [N, heads * head_dim] times sigmoid(gate): gate [N, heads] (one number per head) or [N, heads * head_dim]."""
    N = o.shape[0]
    g = torch.sigmoid(_f(gate))
    if per_head:
        return (_f(o).reshape(N, heads, head_dim) * g[:, :, None]).reshape(N, heads * head_dim).to(o.dtype)
    return (_f(o) * g).to(o.dtype)


def head_linear(x, w):
    """x [N, H, K] (a strided view is fine) times w [H, O, K] per head -> [N, H, O]."""
    return torch.einsum("nhk,hok->nho", _f(x), _f(w)).to(x.dtype).contiguous()


def latent_prepare(q, dkv, norm_w, eps, table, step, cache, heads, dim, rot_dim, rank):
    """The rotated parts of the queries q [N, H, dim + rot_dim] -> [N, H, rot_dim]; if `dkv` [N, rank + rot_dim] is
    given, the normed latent and the rotated shared key part of every row go into the request's pages."""
    q_rot = _rotate(_f(q[:, :, dim:]), step.positions, rot_dim, 1.0, table).to(q.dtype).contiguous()
    if dkv is not None:
        c = _rms(_f(dkv[:, :rank]), norm_w, eps)
        r = _rotate(_f(dkv[:, None, rank:]), step.positions, rot_dim, 1.0, table)[:, 0]
        page, off = _page_rows(step, cache)
        cache.pages[page, off, :] = torch.cat([c, r], dim=-1).to(cache.pages.dtype)
    return q_rot


def latent_attention(q_lat, q_rot, step, cache, heads, rank, rot_dim, scale, impl=None, sink=None):
    """Causal attention of every head against the cached rows [latent | rotated key part]: scores
    (q_lat . latent + q_rot . key part) * scale, output sum_j p_j latent_j, [N, H, rank].  `sink` [H]: one more
    term exp(sink_h) in the denominator."""
    N = q_lat.shape[0]
    ps = cache.page_size
    out = torch.empty((N, heads, rank), dtype=q_lat.dtype, device=q_lat.device)
    cu, ctx = step.cu_q.tolist(), step.ctx_lens.tolist()
    for s in range(step.n_seqs):
        a, b = cu[s], cu[s + 1]
        total = ctx[s] + (b - a)
        n_pages = -(-total // ps)
        if n_pages > cache.block_table.shape[1]:
            _raise(16)
        ids = _checked(cache.block_table[s, :n_pages].long(), cache.pages.shape[0], 4)
        ids = torch.cat([ids, ids.new_zeros(n_pages - ids.shape[0])])
        rows = _f(cache.pages[ids]).reshape(n_pages * ps, rank + rot_dim)[:total]
        sc = (torch.einsum("nhr,kr->hnk", _f(q_lat[a:b]), rows[:, :rank])
              + torch.einsum("nhr,kr->hnk", _f(q_rot[a:b]), rows[:, rank:])) * scale
        qpos = torch.arange(ctx[s], total, device=q_lat.device)[:, None]
        kpos = torch.arange(total, device=q_lat.device)[None, :]
        sc = sc.masked_fill((kpos > qpos)[None], float("-inf"))
        if sink is not None:
            extra = _f(sink)[:, None, None].expand(heads, b - a, 1)
            prob = torch.softmax(torch.cat([sc, extra], dim=-1), dim=-1)[..., :total]
        else:
            prob = torch.softmax(sc, dim=-1)
        out[a:b] = torch.einsum("hnk,kr->nhr", prob, rows[:, :rank]).to(q_lat.dtype)
    return out


def clamped_glu(gu, ff_dim, limit, alpha):
    g = torch.clamp(_f(gu[:, :ff_dim]), max=limit)
    u = torch.clamp(_f(gu[:, ff_dim:]), min=-limit, max=limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(gu.dtype)


def linear_clamped_glu(x, w_gate_up, ff_dim, limit, alpha):
    return clamped_glu(linear(x, w_gate_up), ff_dim, limit, alpha)


def scale_softcap(logits, scale, cap):
    y = _f(logits) * scale
    return y if cap is None else cap * torch.tanh(y / cap)


def rmsnorm_rows(x, w, eps):
    """RMS norm of activation rows with a 32-bit weight (or None), computed in 32-bit, in x's dtype."""
    v = _f(x)
    y = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)
    return (y if w is None else y * w).to(x.dtype)


def routed_experts(x, w_router, w_gate_up, w_down, top, renorm=False, weight_on="input", score="sigmoid", act="silu", limit=0.0,
                   alpha=1.702):
    """Every row to the `top` experts with the largest sigmoid(x . w_router^T); the scores weigh the experts' inputs
    or outputs; w_gate_up [E, 2F, W] (gate rows, then up rows), w_down [E, W, F]."""
    N, W = x.shape
    E, F = w_gate_up.shape[0], w_gate_up.shape[1] // 2
    z = _f(x) @ _f(w_router).t()
    s = torch.softmax(z, dim=-1) if score == "softmax" else torch.sigmoid(z)
    val, idx = torch.topk(s, int(top), dim=-1)
    if renorm:
        val = val / (val.sum(-1, keepdim=True) + 1e-20)
    out = torch.zeros((N, W), dtype=torch.float32, device=x.device)
    for n in range(N):
        for k in range(int(top)):
            e, w = int(idx[n, k]), val[n, k]
            xin = (_f(x[n]) * w).to(x.dtype) if weight_on == "input" else x[n]
            gu = _f(xin) @ _f(w_gate_up[e]).t()
            if act == "clamped":
                g, u = torch.clamp(gu[:F], max=limit), torch.clamp(gu[F:], min=-limit, max=limit)
                hid = (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(x.dtype)
            else:
                hid = (_silu(gu[:F]) * gu[F:]).to(x.dtype)
            y = _f(hid) @ _f(w_down[e]).t()
            out[n] += y if weight_on == "input" else y * w
    return out.to(x.dtype)


def act_mul(gu, ff_dim, kind):
    return (_f(activation(_f(gu[:, :ff_dim]), kind)) * _f(gu[:, ff_dim:2 * ff_dim])).to(gu.dtype)


def linear_glu(x, w_gate_up, ff_dim, kind):
    return act_mul(linear(x, w_gate_up), ff_dim, kind)


def mlstm(y, at, bias_i, bias_f, cap, norm_w, eps, state, step, heads, dim, vdim, write_state=True, precision=torch.float32):
    """The matrix memory with log gates over the stacked projections y (columns `at`: q, k, v, output gate, the two log
    gates' inputs); state [slots, H, D + 1, Dv + 1]: S with the normaliser as its last column, the running maximum of
    every column in the last row.  `precision`: the type the recurrence is computed in (64-bit: the exact answer for a
    32-bit kernel's test)."""
    _f = lambda t: t.to(precision)
    N, H, D, Dv = y.shape[0], heads, dim, vdim
    q_at, k_at, v_at, g_at, i_at, f_at = at
    q = _f(y[:, q_at:q_at + H * D]).reshape(N, H, D) * D ** -0.5
    k = _f(y[:, k_at:k_at + H * D]).reshape(N, H, D)
    v = torch.cat([_f(y[:, v_at:v_at + H * Dv]).reshape(N, H, Dv), torch.ones(N, H, 1, device=y.device, dtype=precision)], dim=-1)
    gi = cap * torch.tanh((_f(y[:, i_at:i_at + H]) + _f(bias_i)) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((_f(y[:, f_at:f_at + H]) + _f(bias_f)) / cap))
    out = torch.zeros((N, H, Dv), dtype=precision, device=y.device)
    for a, b, slot in _spans(step, state):
        S, m = _f(state[slot][:, :D, :]).clone(), _f(state[slot][:, D, 0]).clone()
        for t in range(a, b):
            new = torch.maximum(gf[t] + m, gi[t])
            keep, take = torch.exp(gf[t] + m - new), torch.exp(gi[t] - new)
            S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
            m = new
            r = torch.einsum("hdc,hd->hc", S, q[t])
            out[t] = r[:, :Dv] / (torch.maximum(r[:, Dv].abs(), torch.exp(-m)) + 1e-6)[:, None]
        if write_state:
            state[slot][:, :D, :] = S.to(state.dtype)
            state[slot][:, D, :] = m[:, None].to(state.dtype)
    o = out * torch.rsqrt((out * out).mean(-1, keepdim=True) + eps)
    g = torch.sigmoid(_f(y[:, g_at:g_at + H * Dv]))
    return (o.reshape(N, H * Dv) * _f(norm_w) * g).to(y.dtype)
