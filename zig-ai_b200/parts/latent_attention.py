"""Attention over a shared low-rank latent.

Per position the layer keeps one vector: a latent c of `rank` values and one rotated key part r of `rot_dim`
values that all heads share.

    q      = x . Wq^T                      per head [dim unrotated | rot_dim rotated]
    d      = x . Wdkv^T                    [rank + rot_dim]
    c      = rms(d[:rank]) * norm weight;  r = rotate(d[rank:])             -> the request's pages, [c | r] per position
    per head h:  k_j = Wuk_h c_j,  v_j = Wuv_h c_j
                 s_j = (q_h[:dim] . k_j + rotate(q_h[dim:]) . r_j) * scale   for cached j <= the query's position
                 o_h = sum_j softmax(s)_j v_j
    out    = ( concat_h(o_h) * sigmoid(x . Wg^T) ) . Wo^T                    (`gate="element"`; None: no gate)

The rotation pairs (i, i + rot_dim/2) over the whole rotated part, with the position part's frequencies.  A position
part that pairs (2i, 2i + 1) is served by reordering, once at load, the rows of the projections that make the rotated
parts of q and of the shared key (a dot product does not change when both vectors are reordered alike).

Options, for designs that vary the layer:
    q_rank=r        queries through a latent of their own: c_q = rms(x . Wdq^T) * norm weight,  q = c_q . Wuq^T
                    (names dq, dq_norm, uq instead of q)
    sink=True       one learned number per head (name sink) whose exponential is one more term of the softmax's
                    denominator: it has no key and no value and is not scaled
    gate="head"     one sigmoid gate per head, sigmoid(x . Wg^T)_h with Wg [heads, hidden], on the head's output

Keys and values are never expanded: q_h[:dim] . (Wuk_h c_j) = (Wuk_h^T q_h[:dim]) . c_j and
sum_j p_j (Wuv_h c_j) = Wuv_h (sum_j p_j c_j), so the attention kernel runs every head against the cached
vectors themselves (query [rank | rot_dim], value = the latent) and two small per-head products sit before and
after it.  Scores, softmax and the weighted sum are 32-bit.

`kv_proj=False`: the layer has no Wdkv and reads the pages another layer wrote (that layer's `rank`, `rot_dim`
and rotation must equal this one's); everything else is its own.
"""
from __future__ import annotations

import torch

from .base import Mixer, PagedRowsNeed, ParamDecl, PartSpec, make_part, register_part, stack_rows

DEFAULT_NAMES = {"q": "attn_q.weight", "dkv": "attn_kv_down.weight", "dkv_norm": "attn_kv_norm.weight",
                 "uk": "attn_k_up.weight", "uv": "attn_v_up.weight", "g": "attn_gate.weight", "o": "attn_output.weight",
                 "dq": "attn_q_down.weight", "dq_norm": "attn_q_norm.weight", "uq": "attn_q_up.weight", "sink": "attn_sink"}


class LatentAttention(Mixer):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True             # forward launches kernels only; nothing is read back to the host
    kernel_libs = ("latent_attention", "qkv_prepare")

    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, rank: int, scale: float, eps: float,
                 position: PartSpec, kv_proj: bool = True, gate="element", names=None, q_rank=None, sink: bool = False):
        self.hidden, self.heads, self.dim, self.rot_dim = int(hidden), int(heads), int(dim), int(rot_dim)
        self.vdim, self.rank, self.scale, self.eps = int(vdim), int(rank), float(scale), float(eps)
        self.kv_proj, self.gate = bool(kv_proj), gate
        if gate not in (None, "element", "head"):
            raise ValueError("gate is None, 'element' or 'head'")
        if self.rot_dim % 2:
            raise ValueError("the rotated part has an even number of dimensions")
        self.q_rank, self.sink = (None if q_rank is None else int(q_rank)), bool(sink)
        if self.q_rank is not None and self.q_rank < 1:
            raise ValueError("the queries' latent has at least one dimension")
        self.position = make_part("position", position)
        self.rot_order = self.position.to_half_split(self.rot_dim)     # None: the rotated parts are paired as stored
        self.gate_cols = 0 if not gate else (self.heads if gate == "head" else self.heads * self.vdim)
        self.names = {**DEFAULT_NAMES, **(names or {})}

    def params(self):
        nm, H, D, Dr, Dv, R, W = self.names, self.heads, self.dim, self.rot_dim, self.vdim, self.rank, self.hidden
        p = {nm["uk"]: ParamDecl((H * D, R)), nm["uv"]: ParamDecl((H * Dv, R)), nm["o"]: ParamDecl((W, H * Dv))}
        if self.q_rank is None:
            p[nm["q"]] = ParamDecl((H * (D + Dr), W))
        else:
            p[nm["dq"]] = ParamDecl((self.q_rank, W))
            p[nm["dq_norm"]] = ParamDecl((self.q_rank,), "vector", init="norm_weight")
            p[nm["uq"]] = ParamDecl((H * (D + Dr), self.q_rank))
        if self.kv_proj:
            p[nm["dkv"]] = ParamDecl((R + Dr, W))
            p[nm["dkv_norm"]] = ParamDecl((R,), "vector", init="norm_weight")
        if self.gate:
            p[nm["g"]] = ParamDecl((self.gate_cols, W))
        if self.sink:
            p[nm["sink"]] = ParamDecl((H,), "vector", init="conv")
        return p

    def cache_need(self):
        return PagedRowsNeed(self.rank + self.rot_dim)

    def bind(self, tensors, dtype):
        nm, H, D, Dr, Dv, R = self.names, self.heads, self.dim, self.rot_dim, self.vdim, self.rank
        w_q = tensors[nm["q"] if self.q_rank is None else nm["uq"]]
        w_dkv = tensors[nm["dkv"]] if self.kv_proj else None
        if self.rot_order is not None:
            # the rows that make rotated dimensions, in the order in which the kernels pair (i, i + rot_dim/2)
            order = torch.tensor(self.rot_order, device=w_q.device)
            w_q = w_q.reshape(H, D + Dr, -1).clone()
            w_q[:, D:] = w_q[:, D:][:, order]
            w_q = w_q.reshape(H * (D + Dr), -1).contiguous()
            if w_dkv is not None:
                w_dkv = torch.cat([w_dkv[:R], w_dkv[R:][order]], dim=0)
        first = w_q if self.q_rank is None else tensors[nm["dq"]]
        mats = [first] + ([tensors[nm["g"]]] if self.gate else []) + ([w_dkv] if self.kv_proj else [])
        self.w_in, at = stack_rows(mats)                             # q (or its latent) | gate | latent: everything that reads x
        self.w_uq = None if self.q_rank is None else w_q
        self.q_norm = tensors.get(nm["dq_norm"]) if self.q_rank is not None else None
        self.q_cols = first.shape[0]
        self.gate_at = at[1] if self.gate else 0
        self.dkv_at = at[-1] if self.kv_proj else 0
        self.c_norm = tensors.get(nm["dkv_norm"])
        self.w_sink = tensors[nm["sink"]] if self.sink else None
        self.w_uk_t = tensors[nm["uk"]].reshape(H, D, R).transpose(1, 2).contiguous()     # [H, R, D]: q_h[:dim] -> the latent's space
        self.w_uv = tensors[nm["uv"]].reshape(H, Dv, R).contiguous()                      # [H, Dv, R]: the latent's space -> v
        self.w_o = tensors[nm["o"]]
        self.dtype = dtype

    def forward(self, x, step, cache, write_cache=True):
        ops, H, D, Dr, Dv, R = step.ops, self.heads, self.dim, self.rot_dim, self.vdim, self.rank
        y = ops.linear(x, self.w_in)
        N = y.shape[0]
        if self.w_uq is None:
            q = y[:, :self.q_cols].view(N, H, D + Dr)
        else:
            q = ops.linear(ops.rmsnorm_rows(y[:, :self.q_cols], self.q_norm, self.eps), self.w_uq).view(N, H, D + Dr)
        _, table = self.position.table(step, y.device)
        own = self.kv_proj and write_cache
        q_rot = ops.latent_prepare(q, y[:, self.dkv_at:self.dkv_at + R + Dr] if own else None, self.c_norm, self.eps, table,
                                   step, cache, H, D, Dr, R)
        q_lat = ops.head_linear(q[:, :, :D], self.w_uk_t)            # [N, H, R]
        o_lat = ops.latent_attention(q_lat, q_rot, step, cache, H, R, Dr, self.scale, sink=self.w_sink)
        o = ops.head_linear(o_lat, self.w_uv).view(N, H * Dv)
        if self.gate:
            o = ops.sigmoid_gate(o, y[:, self.gate_at:self.gate_at + self.gate_cols], H, Dv, self.gate == "head")
        return ops.linear(o, self.w_o)


register_part("mixer", "latent_attention", LatentAttention)
