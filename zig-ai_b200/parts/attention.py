"""Grouped-query attention over the paged cache.

    q = x.Wq^T [N,Hq,D]   k = x.Wk^T, v = x.Wv^T [N,Hkv,D]       (no biases)
    q, k = rms(q, q_norm), rms(k, k_norm)  per head over D           (if qk_norm)
    q, k = position(q, k)                                           (v is neither normed nor rotated)
    k, v of the new positions are written into the request's pages
    s = q.k^T * scale over the request's cached positions <= the query's (and inside the window)
    out = softmax(s).v  -> [N, Hq*D] . Wo^T

Options beside that: `scale` (default 1/sqrt(D)); `value_dim`, a value head size Dv other than D; `value_norm`,
values divided by their root mean square over Dv (no weight) before they are cached; `names`, the
tensors' names.  With Dv != D every head is kept at max(D, Dv) with zeros behind its own values (zeros
change neither a score nor a sum), so the same pages and kernels serve; the q/k norm still averages
over D.

Further options, for designs that have them: `bias` (q, k and v projections with biases, added in the product);
`norm_scope="whole"` (one RMS norm over all rows of the q projection, and one over all of k, weights of that size,
before the split into heads); `chunk` (a query sees back to the start of its chunk of that many positions,
counted from position 0 of the request: j <= i and j // chunk == i // chunk); `gate="head"` (a fourth
projection of one number per query head; a head's output is multiplied by its sigmoid before the output
projection); a position part that pairs dimensions (2i, 2i+1) or stretches its frequencies.  With any of them
the projections run as one product q|k|v|gate and one kernel norms, rotates and writes the pages
(`ops.qkv_prepare`); an interleaved pairing is turned into the half-split one by reordering the rows of the q
and k projections (with their biases and norm weights) at load.

Options that shape the scores or the values (they also take the one-product path, and the general attention kernel):
    q_temp=(coef, every)   the queries at position p times 1 + coef ln(floor((p + 1) / every) + 1)
    softcap=c              s <- c tanh(s / c), after the scale and before anything is added
    rel_bias={rows, max}   a learned table `rel` [rows, heads] added to the score by distance n = i - j: row n for n < rows/2,
                           beyond that rows that widen geometrically, min(rows - 1, rows/2 + floor(ln(n / (rows/2)) /
                           ln(max / (rows/2)) * (rows - rows/2))); not scaled, not capped.  The table is laid out by distance
                           once at load (`distance_table`)
    sink=True              a learned number per head `sink` whose exponential joins the softmax's denominator (no key, no value)
    keep_first=n           with a window: the first n positions of the request stay visible to every later query, at their
                           true positions; their pages are never given back
    v_mix="first"|"mix"    values shared across layers: a "first" layer leaves its values with the step, a "mix" layer
                           caches (1 - lambda) v + lambda v_first with its learned scalar `vmix` (the first layer's is stored
                           and unused)

Reference: projections src/transformer/hybrid_attn.zig:285-354, per-head norm :371-382 (device
:719,723), scale 1/sqrt(D) :571, causal mask :587, softmax :578-600, query head hq reads kv head
hq // (Hq/Hkv) :553-569 and src/cuda/paged_attention.cu:142, output projection :622-640; tensor
names :250-267.  Softmax and the norms are 32-bit.
"""
from __future__ import annotations

import math

import torch

from .base import Mixer, PagedKVNeed, ParamDecl, make_part, register_part, PartSpec


class Attention(Mixer):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True      # forward launches kernels only; nothing is read back to the host
    kernel_libs = ("attention", "attention_mma", "attention_tma", "attention_tc")   # (all but the first: bfloat16 only)

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, qk_norm: bool, eps: float,
                 position: PartSpec, window=None, scale=None, kv_proj: bool = True, value_dim=None,
                 value_norm: bool = False, names=None, bias: bool = False, norm_scope: str = "head", chunk=None, gate=None,
                 q_temp=None, softcap=None, rel_bias=None, sink: bool = False, keep_first: int = 0, v_mix=None):
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads cannot share {self.kv_heads} key/value heads evenly")
        self.qk_norm, self.eps = bool(qk_norm), float(eps)
        self.window = None if window is None else int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.kv_proj = bool(kv_proj)
        self.position = make_part("position", position)
        self.value_dim = self.head_dim if value_dim is None else int(value_dim)
        self.value_norm = bool(value_norm)
        if (self.value_norm or self.value_dim != self.head_dim) and not self.kv_proj:
            raise ValueError("a value norm or a value head size of its own needs the layer's own k/v projections")
        self.cache_dim = max(self.head_dim, self.value_dim)      # the head size of the pages and the kernels
        self.names = {"q": "attn_q.weight", "k": "attn_k.weight", "v": "attn_v.weight", "o": "attn_output.weight",
                      "q_norm": "attn_q_norm.weight", "k_norm": "attn_k_norm.weight", "q_bias": "attn_q.bias",
                      "k_bias": "attn_k.bias", "v_bias": "attn_v.bias", "g": "attn_gate.weight", "rel": "attn_rel_bias",
                      "sink": "attn_sink", "vmix": "attn_vmix", **(names or {})}
        self.bias, self.norm_scope, self.gate = bool(bias), str(norm_scope), gate
        self.chunk = None if chunk is None else int(chunk)
        if self.norm_scope not in ("head", "whole") or self.gate not in (None, "head"):
            raise ValueError("norm_scope is 'head' or 'whole'; gate is None or 'head'")
        if self.chunk is not None and (self.chunk < 1 or self.window is not None):
            raise ValueError("a chunk holds at least one position, and chunks and a window exclude each other")
        self.q_temp = None if q_temp is None else (float(q_temp[0]), int(q_temp[1]))
        self.softcap = None if softcap is None else float(softcap)
        self.rel_bias = None if rel_bias is None else {"rows": int(rel_bias["rows"]), "max": float(rel_bias["max"])}
        self.sink, self.keep_first, self.v_mix = bool(sink), int(keep_first or 0), v_mix
        if self.v_mix not in (None, "first", "mix"):
            raise ValueError("v_mix is None, 'first' or 'mix'")
        if self.keep_first and self.window is None:
            raise ValueError("kept first positions go with a window")
        if self.q_temp is not None and self.q_temp[1] < 1:
            raise ValueError("q_temp counts positions in groups of at least one")
        if self.rel_bias is not None and (self.rel_bias["rows"] < 2 or self.rel_bias["max"] <= self.rel_bias["rows"] // 2):
            raise ValueError("a distance-bias table has at least two rows and reaches beyond its one-distance rows")
        self.shaped = bool(self.softcap or self.rel_bias or self.sink or self.keep_first)
        # the options that the one-product, one-preparation path serves
        self.prepared = bool(self.bias or self.norm_scope == "whole" or self.gate or self.chunk is not None
                             or self.shaped or self.q_temp or self.v_mix
                             or getattr(self.position, "pairing", "half_split") != "half_split"
                             or getattr(self.position, "scaling", None) is not None)
        if self.prepared and (self.value_norm or not self.kv_proj):
            raise ValueError("value_norm and a borrowed cache are not combined with bias, whole norm, chunk or gate")
        if self.prepared:
            self.kernel_libs = type(self).kernel_libs + ("qkv_prepare",)

    def params(self):
        q_dim, kv_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        nm = self.names
        p = {nm["q"]: ParamDecl((q_dim, self.hidden)),
             nm["o"]: ParamDecl((self.hidden, self.heads * self.value_dim))}
        if self.kv_proj:
            p[nm["k"]] = ParamDecl((kv_dim, self.hidden))
            p[nm["v"]] = ParamDecl((self.kv_heads * self.value_dim, self.hidden))
        whole = self.norm_scope == "whole"
        if self.qk_norm:
            p[nm["q_norm"]] = ParamDecl((q_dim if whole else self.head_dim,), "vector", init="norm_weight")
            if self.kv_proj:
                p[nm["k_norm"]] = ParamDecl((kv_dim if whole else self.head_dim,), "vector", init="norm_weight")
        if self.bias:
            p[nm["q_bias"]] = ParamDecl((q_dim,), "vector", init="conv")
            p[nm["k_bias"]] = ParamDecl((kv_dim,), "vector", init="conv")
            p[nm["v_bias"]] = ParamDecl((self.kv_heads * self.value_dim,), "vector", init="conv")
        if self.gate:
            p[nm["g"]] = ParamDecl((self.heads, self.hidden))
        if self.rel_bias:
            p[nm["rel"]] = ParamDecl((self.rel_bias["rows"], self.heads), "vector", init="conv")
        if self.sink:
            p[nm["sink"]] = ParamDecl((self.heads,), "vector", init="conv")
        if self.v_mix:
            p[nm["vmix"]] = ParamDecl((), "vector", init="mix")
        return p

    def cache_need(self):
        return PagedKVNeed(self.kv_heads, self.cache_dim, self.window, self.chunk, self.keep_first)

    def distance_table(self, rel):
        """The bias by distance, [distances, heads]: row n holds `rel[bucket(n)]`; the last row stands for every distance
        from there on (the first distance of the table's last bucket).  Made once at load, in 64-bit on the host."""
        rows, far = self.rel_bias["rows"], self.rel_bias["max"]
        half = rows // 2
        buckets, n = [], 0
        while True:
            b = n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))
            buckets.append(b)
            if b == rows - 1:
                break
            n += 1
        idx = torch.tensor(buckets, dtype=torch.long, device=rel.device)
        return rel.float().index_select(0, idx).contiguous()

    def _bind_prepared(self, tensors, dtype):
        """One matrix q|k|v|gate (and one bias vector), the rows of q and k in the order in which the rotation pairs
        (i, i + dims/2)."""
        nm, H, G, D, Dv, Dp = self.names, self.heads, self.kv_heads, self.head_dim, self.value_dim, self.cache_dim
        perm = self.position.to_half_split(D)
        idx = None if perm is None else torch.tensor(perm, dtype=torch.long, device=tensors[nm["q"]].device)

        def heads_reordered(t, n_heads):          # t: [n_heads * D, ...] (rows of a projection, a bias, a whole norm's weight)
            if idx is None or t is None:
                return t
            return t.reshape((n_heads, D) + tuple(t.shape[1:])).index_select(1, idx).reshape(t.shape).contiguous()

        q, k, v = heads_reordered(tensors[nm["q"]], H), heads_reordered(tensors[nm["k"]], G), tensors[nm["v"]]
        mats = [q, k, v] + ([tensors[nm["g"]]] if self.gate else [])
        self.w_qkv = torch.cat(mats, dim=0).contiguous()
        self.b_qkv = None
        if self.bias:
            b = [heads_reordered(tensors[nm["q_bias"]], H), heads_reordered(tensors[nm["k_bias"]], G), tensors[nm["v_bias"]]]
            if self.gate:
                b.append(b[0].new_zeros(H))
            self.b_qkv = torch.cat(b).to(self.w_qkv.dtype).contiguous()
        self.q_norm, self.k_norm = tensors.get(nm["q_norm"]), tensors.get(nm["k_norm"])
        if self.norm_scope == "whole":
            self.q_norm, self.k_norm = heads_reordered(self.q_norm, H), heads_reordered(self.k_norm, G)
        elif idx is not None and self.q_norm is not None:
            self.q_norm, self.k_norm = self.q_norm[idx].contiguous(), self.k_norm[idx].contiguous()
        self.norm_eps = self.eps
        self.w_o = tensors[nm["o"]]
        if Dp != Dv:
            w = self.w_o.reshape(self.hidden, H, Dv)
            self.w_o = torch.cat([w, w.new_zeros(self.hidden, H, Dp - Dv)], dim=2).reshape(self.hidden, -1).contiguous()
        self.gate_at = H * D + G * D + G * Dv
        self.v_at = H * D + G * D
        self.bias_table = self.distance_table(tensors[nm["rel"]]) if self.rel_bias else None
        self.sink_w = tensors[nm["sink"]].float().contiguous() if self.sink else None
        self.v_lambda = tensors[nm["vmix"]].float().reshape(1).contiguous() if self.v_mix == "mix" else None
        self.dtype = dtype

    def _forward_prepared(self, x, step, cache, write_cache):
        ops, H, G, D, Dv, Dp = step.ops, self.heads, self.kv_heads, self.head_dim, self.value_dim, self.cache_dim
        y = ops.linear(x, self.w_qkv, bias=self.b_qkv)
        dims, table = self.position.table(step, y.device)
        scope = 0 if not self.qk_norm else (2 if self.norm_scope == "whole" else 1)
        more = {}
        if self.q_temp:
            more["temp"] = self.q_temp
        if self.v_mix == "first":
            step.scratch["attention.v_first"] = y[:, self.v_at:self.v_at + G * Dv]     # (kept alive with the step)
        elif self.v_mix == "mix":
            if "attention.v_first" not in step.scratch:
                raise RuntimeError("a layer mixes its values with an earlier layer's, and no earlier layer has left any")
            more.update(v_first=step.scratch["attention.v_first"], v_lambda=self.v_lambda)
        q = ops.qkv_prepare(y, self.q_norm, self.k_norm, self.norm_eps, scope, table, dims, step, cache, H, G, D, Dv, Dp,
                            write_cache, **more)
        if self.shaped:
            o = ops.paged_attention(q, step, cache, H, G, Dp, self.scale, self.window, softcap=self.softcap, bias=self.bias_table,
                                    sink=self.sink_w, keep_first=self.keep_first)
        else:
            o = ops.paged_attention(q, step, cache, H, G, Dp, self.scale, self.window, chunk=self.chunk)
        if self.gate:
            o = ops.sigmoid_gate(o, y[:, self.gate_at:self.gate_at + H], H, Dp, True)
        return ops.linear(o, self.w_o)

    def bind(self, tensors, dtype):
        if self.prepared:
            return self._bind_prepared(tensors, dtype)
        nm = self.names
        mats = [tensors[nm["q"]]]
        if self.kv_proj:
            mats += [tensors[nm["k"]], tensors[nm["v"]]]
        self.w_qkv = torch.cat(mats, dim=0).contiguous()
        self.w_o = tensors[nm["o"]]
        self.q_norm = tensors.get(nm["q_norm"])
        self.k_norm = tensors.get(nm["k_norm"])
        self.norm_eps = self.eps
        D, Dv, Dp = self.head_dim, self.value_dim, self.cache_dim
        if Dp != D and self.qk_norm:
            # the kernels average a head's squares over the Dp values they see, of which Dp - D are zero:
            # mean_D = mean_Dp * Dp / D, so  rsqrt(mean_D + eps) = rsqrt(mean_Dp + eps D / Dp) * sqrt(D / Dp)
            grow = lambda g: None if g is None else torch.cat([g * (D / Dp) ** 0.5, g.new_zeros(Dp - D)]).contiguous()
            self.q_norm, self.k_norm, self.norm_eps = grow(self.q_norm), grow(self.k_norm), self.eps * D / Dp
        if Dp != Dv:
            # the heads come out of attention Dp wide with zeros behind their Dv values: the output
            # projection gets zero columns there
            w = self.w_o.reshape(self.hidden, self.heads, Dv)
            self.w_o = torch.cat([w, w.new_zeros(self.hidden, self.heads, Dp - Dv)], dim=2).reshape(self.hidden, -1).contiguous()
        self.dtype = dtype

    def forward(self, x, step, cache, write_cache=True):
        if self.prepared:
            return self._forward_prepared(x, step, cache, write_cache)
        ops = step.ops
        write = write_cache and self.kv_proj
        qkv = ops.linear(x, self.w_qkv)
        if self.value_norm or self.value_dim != self.head_dim:
            qkv = ops.value_norm_pad(qkv, self.heads, self.kv_heads, self.head_dim, self.value_dim, self.eps, self.value_norm)
        rot = self.position.rotary()
        fused = getattr(ops, "fused_decode_attention_available", None)
        if (rot is not None and step.decode_only and self.kv_proj and fused is not None
                and fused(qkv.dtype, self.heads, self.kv_heads, self.cache_dim)):
            # every row is one token: norm, rotation, page write, attention and the combination of
            # the key chunks run as one kernel
            o = ops.decode_attention_fused(qkv, self.q_norm, self.k_norm, self.norm_eps, rot[0], rot[1], step, cache,
                                           self.heads, self.kv_heads, self.cache_dim, self.scale, self.window, write)
            return ops.linear(o, self.w_o)
        if rot is not None:
            q, _ = ops.qk_norm_rope(qkv, self.q_norm, self.k_norm, self.norm_eps, rot[0], rot[1], step, cache,
                                    self.heads, self.kv_heads, self.cache_dim, self.kv_proj, write, False)
        else:
            q, k = ops.qk_norm_rope(qkv, self.q_norm, self.k_norm, self.norm_eps, 0, 1.0, step, cache,
                                    self.heads, self.kv_heads, self.cache_dim, self.kv_proj, False, self.kv_proj)
            q, k = self.position.apply(q, k, step.positions, step)
            if write:
                v = qkv[:, (self.heads + self.kv_heads) * self.cache_dim:]
                ops.kv_write(k, v, step, cache, self.kv_heads, self.cache_dim)
        o = ops.paged_attention(q, step, cache, self.heads, self.kv_heads, self.cache_dim, self.scale, self.window)
        return ops.linear(o, self.w_o)


register_part("mixer", "attention", Attention)
