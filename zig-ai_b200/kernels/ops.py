"""The kernels as functions on torch CUDA tensors.

One function per kernel (or per small group launched together); every function launches on the
current CUDA stream and allocates its outputs with torch.  There is no CPU path: calling any of
these without the compiled libraries or without a CUDA device raises.  Plain matrix products go to
cuBLAS through `torch.matmul`, as the reference sends every projection to `cublasSgemm_v2`
(src/matmul/cublas.zig:515-548); the 32-bit mode runs them as true 32-bit products (TF32 off).
"""
from __future__ import annotations

import ctypes
import math
import os
import sys
import weakref
from ctypes import c_float, c_int, c_void_p

import torch

from ..parts.base import LazyNorm
from . import build

device_type = "cuda"

_F32, _BF16 = 0, 1
_P, _I, _F = c_void_p, c_int, c_float

_SIGNATURES = {
    "embed": {
        "zai_embed": [_P, _P, _I, _P, _I, _I, _I, _F, _P, _P],
        "zai_gather_add": [_P, _P, _P, _I, _P, _I, _I, _P],
        "zai_gather_add_normed": [_P, _P, _P, _I, _P, _F, _P, _I, _I, _P],
    },
    "norm": {"zai_add_rmsnorm": [_P, _P, _P, _P, _I, _F, _I, _I, _P],
             "zai_add_normed_rmsnorm": [_P, _P, _P, _F, _P, _P, _I, _F, _I, _I, _P],
             "zai_add_normed_cast": [_P, _P, _P, _F, _P, _I, _I, _I, _P],
             "zai_rmsnorm_rows": [_P, _P, _I, _I, _P, _F, _I, _I, _P]},
    "moe": {"zai_moe_route": [_P, _P, _P, _P, _P, _I, _I, _P, _I, _I, _I, _I, _I, _I, _P],
            "zai_moe_max_tiles": [_I, _I, _I, _I],
            "zai_moe_gather": [_P, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
            "zai_moe_gemm": [_P, _I, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _F, _P],
            "zai_moe_combine": [_P, _I, _P, _P, _P, _I, _I, _I, _I, _P]},
    "layernorm": {"zai_add_layernorm": [_P, _P, _P, _P, _P, _I, _F, _I, _I, _P]},
    "qkv_prepare": {
        "zai_qkv_prepare": [_P, _I, _I, _P, _P, _F, _I, _P, _I, _P, _P, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P,
                            _F, _I, _P, _I, _P, _P],
        "zai_latent_prepare": [_P, _I, _P, _I, _I, _P, _F, _P, _P, _P, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P],
        "zai_sigmoid_gate": [_P, _P, ctypes.c_longlong, ctypes.c_longlong, _P, _I, _I, _I, _I, _I, _I, _P],
    },
    "latent_attention": {
        "zai_latent_attention": [_P, _P, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P, _P],
        "zai_latent_attention_mma_supports": [_I, _I],
        "zai_latent_attention_mma": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P, _P],
    },
    "activation": {"zai_silu_mul": [_P, _P, _I, _I, _I, _P],
                   "zai_clamped_glu": [_P, _P, _I, _I, _I, _F, _F, _P],
                   "zai_act_mul": [_P, _P, _I, _I, _I, _I, _P],
                   "zai_scale_softcap": [_P, ctypes.c_longlong, _F, _F, _P],
                   "zai_activation": [_P, _P, _I, _I, ctypes.c_longlong, _P],
                   "zai_weighted_sum": [_P, _P, _P, _I, _F, _F, ctypes.c_longlong, _P]},
    "causal_conv": {"zai_causal_conv": [_P, _I, _P, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P]},
    "selective_scan": {"zai_selective_scan": [_P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                                              _I, _P, _P, _P, _I, _I, _I, _P]},
    "min_gru": {"zai_min_gru": [_P, _P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _I, _I, _P]},
    "gated_delta": {
        "zai_delta_prepare": [_P, _P, _P, _P, _I, _P, _I, _P, _I, _I, _P, _P, _I, _I, _I, _I, _F, _P],
        "zai_gated_delta": [_P, _P, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
        "zai_gated_rmsnorm": [_P, _P, _P, _P, _I, _I, _F, _I, _I, _I, _I, _P],
        "zai_gated_delta_single_supports": [_I, _I],
        "zai_gated_delta_single": [_P, _P, _I, _P, _I, _P, _I, _P, _I, _I, _P, _P, _P, _F, _F, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                                   _P, _I, _I, _P],
    },
    "shortconv": {"zai_short_conv": [_P, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P]},
    "rope_kv": {
        "zai_rope_table": [_P, _P, _P, _I, _I, _P],
        "zai_rope_table_scaled": [_P, _P, _P, _I, _I, ctypes.c_double, _P],
        "zai_qk_norm_rope": [_P, _I, _I, _P, _P, _F, _P, _I, _P, _P, _P, _I, _P, _I, _P, _P,
                             _I, _I, _I, _I, _I, _I, _I, _P, _P],
        "zai_kv_write": [_P, _I, _P, _I, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _P, _P],
        "zai_value_norm_pad": [_P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    },
    "attention": {
        "zai_paged_attention_general": [_P, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
        "zai_paged_attention_scored": [_P, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P, _F, _P, _I, _P, _I, _P],
    },
    "mlstm": {"zai_mlstm": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _F, _P, _F, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I,
                            _P]},
    "attention_mma": {
        "zai_attention_mma_supports": [_I, _I, _I],
        "zai_prefill_attention_mma": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
        "zai_decode_attention_mma": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
        "zai_prefill_attention_mma_scored": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _F, _P, _I, _P, _I, _P],
        "zai_decode_attention_mma_scored": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _F, _P, _I, _P, _I,
                                            _P],
        "zai_decode_attention_fused": [_P, _P, _P, _P, _P, _I, _P, _P, _F, _P, _I, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I,
                                       _F, _I, _I, _I, _I, _P, _P],
        "zai_decode_chunk_keys": [],
        "zai_prefill_block_rows": [],
    },
    "decode_gemm": {
        "zai_skinny_gemm_supports": [_I, _I, _I, _I, _I],
        "zai_skinny_gemm": [_P, _P, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _I, _P],
        "zai_skinny_gemm_clamped_glu": [_P, _P, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _F, _F, _P],
        "zai_skinny_gemm_layernorm": [_P, _P, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _I, _F, _F, _P],
        "zai_skinny_conv": [_P, _P, _P, _P, _P, _P, _P, _F, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
        "zai_skinny_hint_next": [_P, ctypes.c_longlong],
    },
    "stream_gemm": {
        "zai_stream_gemm_supports": [_I, _I, _I, _I],
        "zai_stream_force_cluster": [_I],
        "zai_stream_force_rows": [_I],
        "zai_stream_debug": [_P],
        "zai_stream_gemm": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
        "zai_stream_conv": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    },
    "gemm_tc": {
        "zai_gemm_tc_supports": [_I, _I, _I, _I],
        "zai_gemm_tc": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
        "zai_gemm_tc_grouped": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    },
    "gemm_tc_pair": {
        "zai_gemm_pair_supports": [_I, _I, _I, _I],
        "zai_gemm_pair": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    },
    "attention_tma": {
        "zai_decode_attention_tma_supports": [_I, _I, _I, _I],
        "zai_decode_attention_tma": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _F, _P, _I, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I,
                                     _I, _F, _I, _I, _I, _P],
    },
    "attention_tc": {
        "zai_prefill_attention_tc_supports": [_I, _I, _I, _I],
        "zai_prefill_attention_tc": [_P, _P, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P, _P, _P],
        "zai_prefill_attention_tc_splits": [_I, _I, _I, _I],
    },
    "sampling": {
        "zai_argmax": [_P, _P, _I, _I, _P, _P],
        "zai_repetition_penalty": [_P, _P, _P, _P, _P, _I, _I, _P],
        "zai_repetition_penalty_counts": [_P, _P, _P, _P, _P, _I, _I, _P],
        "zai_count_tokens": [_P, _P, _P, _I, _I, _P],
        "zai_sample": [_P, _P, _P, _P, _P, _P, _I, _I, _P, _P],
    },
}

_fns = {}


class KernelError(RuntimeError):
    pass


def _fn(lib_name: str, fn_name: str):
    f = _fns.get(fn_name)
    if f is None:
        lib = build.load(lib_name)
        f = getattr(lib, fn_name)
        f.argtypes = _SIGNATURES[lib_name][fn_name]
        f.restype = c_int
        _fns[fn_name] = f
    return f


launches = 0        # kernels of this package launched so far (a count of launcher calls that ran)


def _check(code: int, what: str, n: int = 1) -> None:
    global launches
    if code == 0:
        launches += n
        return
    if code == -1:
        raise KernelError(f"{what}: element type not supported by the kernel")
    if code == -2:
        raise KernelError(f"{what}: a size is outside what the kernel supports")
    raise KernelError(f"{what}: CUDA error {code} at launch")


CORE_LIBS = ("embed", "norm", "activation", "rope_kv")
BF16_LIBS = ("decode_gemm",)
# libraries that a part may name and only a bfloat16 model uses
BF16_ONLY = ("gemm_tc", "gemm_tc_pair", "stream_gemm", "attention_mma", "attention_tma", "attention_tc")
ATTENTION_LIBS = ("attention", "attention_mma", "attention_tma", "attention_tc")


def require(dtype=None, extra=()) -> None:
    """Fail loudly unless a CUDA device is present and the libraries load that a model of `dtype`
    uses (all of them if no dtype is given).  What is missing or out of date is compiled now, several
    sources at a time; a library outside this set is compiled when it is first called.  `extra`:
    further libraries that the model's parts name (`kernel_libs`)."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this engine has no CPU path")
    bf16 = dtype is None or dtype == torch.bfloat16
    libs = list(CORE_LIBS) + [x for x in extra if x not in CORE_LIBS and (bf16 or x not in BF16_ONLY)]
    if dtype is None:
        libs += ["shortconv", "sampling", *ATTENTION_LIBS]
    if bf16:
        libs += list(BF16_LIBS)
        if dtype is None or USE_TC_GEMM:
            libs.append("gemm_tc")
        if dtype is None:
            libs.append("gemm_tc_pair")
        if dtype is None or USE_STREAM_GEMM:
            libs.append("stream_gemm")
    libs = list(dict.fromkeys(libs))
    build.build_some(libs, verbose=True)
    for lib in libs:
        build.load(lib)


_SKINNY_VARIANTS = {1: "bf16", 2: "norm, bf16", 3: "f32", 4: "norm, f32", 5: "swiglu", 6: "norm, swiglu", 7: "conv",
                    8: "norm, conv"}


def _kernel_at(lib: str, line: int, cache={}) -> str:
    """The name of the __global__ function whose body holds `line` of csrc/<lib>.cu."""
    import re
    if lib not in cache:
        with open(os.path.join(build.CSRC, lib + ".cu")) as f:
            cache[lib] = f.read().split("\n")
    name = "?"
    for text in cache[lib][:line]:
        m = re.search(r"__global__[^(]*?(\w+)\s*\(", re.sub(r"__(launch_bounds|maxnreg)__\([^)]*\)", "", text))
        if m:
            name = m.group(1)
    return name


def timeline():
    """With libraries built under ZAI_TIMELINE=1: the kernels run since the last call, as a list of
    (kernel, ns when the kernel's first block reached its dependency wait, ns when the wait was
    over) in the order of the second time; marks set inside kernels come as ("<library> mark <n>",
    ns, ns).  Reads the device."""
    import ctypes
    if not build.TIMELINE:
        raise KernelError("the libraries were built without ZAI_TIMELINE=1")
    torch.cuda.synchronize()
    out = []
    buf = (ctypes.c_ulonglong * (3 * 16384))()
    for name in build.sources():
        lib = build.load(name)
        fn = lib.zai_timeline_read
        fn.argtypes = [ctypes.c_void_p, c_int]
        fn.restype = c_int
        n = fn(ctypes.cast(buf, ctypes.c_void_p), 16384)
        if n < 0:
            raise KernelError(f"zai_timeline_read failed in {name}")
        for i in range(n):
            ident, a, b = int(buf[3 * i]), int(buf[3 * i + 1]), int(buf[3 * i + 2])
            if ident >> 32 == 2:
                out.append((f"{name} block {ident & 0xffffffff}", a, b))
            elif ident >> 32:
                out.append((f"{name} mark {ident & 255}", b, b))
            else:
                kernel, variant = _kernel_at(name, ident >> 8), ident & 255
                if name == "decode_gemm" and variant:
                    kernel += f" ({_SKINNY_VARIANTS.get(variant, variant)})"
                out.append((kernel, a, b))
    out.sort(key=lambda r: r[2])
    return out


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"element type {t.dtype} is not supported")


def _ptr(t):
    return None if t is None else t.data_ptr()


_stream_handle = None


def begin_forward() -> None:
    """Called once at the start of a forward pass: the current stream is looked up here and reused by
    every launch of the pass (the lookup costs about as much as a launch)."""
    global _stream_handle
    _stream_handle = torch.cuda.current_stream().cuda_stream


def end_forward() -> None:
    global _stream_handle
    _stream_handle = None


def _stream():
    return _stream_handle if _stream_handle is not None else torch.cuda.current_stream().cuda_stream



def _cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernels take contiguous CUDA tensors")


# ----------------------------------------------------------------------------- timing by kernel class
# The reference prints, per stage of a step, the time its kernels took (PERF_STAGE, src/main.zig:817-931,
# 1369-1412).  Here `profile_begin()` makes every kernel function below record a CUDA event before and
# after its launches under the name of its class; `profile_end()` waits and returns milliseconds per
# class.  No special build is needed; steps must be launched kernel by kernel for it (a replayed graph
# has no place for events), so their sum is larger than a graphed step's time: it is the shares that count.
_profile = None
_profile_depth = 0


def profile_begin() -> None:
    global _profile
    _profile = []


def profile_end() -> dict:
    """Milliseconds per kernel class since `profile_begin()` (waits for the device)."""
    global _profile
    records, _profile = _profile or [], None
    torch.cuda.synchronize()
    out = {}
    for name, a, b in records:
        out[name] = out.get(name, 0.0) + a.elapsed_time(b)
    return out


def _timed(name):
    """Record the decorated kernel function under class `name` while a profile is open (`name` may be a
    function of the call's arguments and result).  A call that launched nothing (returned None) is not
    recorded."""
    def wrap(f):
        import functools

        @functools.wraps(f)
        def g(*args, **kwargs):
            global _profile_depth
            if _profile is None or _profile_depth:             # (a kernel function called by another counts with it)
                return f(*args, **kwargs)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            _profile_depth += 1
            try:
                r = f(*args, **kwargs)
            finally:
                _profile_depth -= 1
            if r is None and f.__name__.startswith("_"):
                return r
            b.record()
            _profile.append((name(*args, **kwargs) if callable(name) else name, a, b))
            return r
        return g
    return wrap


def _product_class(x, w, epilogue, *rest, **kw):
    return {_EPI_F32: "head", _EPI_SWIGLU: "products (gate/up + SwiGLU)", 3: "products (in_proj + conv)"}.get(epilogue, "products")


# ----------------------------------------------------------------------------- kernels
fuses_norm = True       # `linear` and `linear_swiglu` take a LazyNorm and apply it inside the product kernel
fuses_layernorm = True  # ... also one that is a layer norm (`LazyNorm.beta`)

_EPI_BF16, _EPI_F32, _EPI_SWIGLU = 0, 1, 2
_EPI_F32_PAIR = 3          # (grouped tcgen05 products) 32-bit results, two weight tiles a stage


@_timed("embedding")
def embed(ids, table, scale=1.0):
    """Rows of the table as 32-bit residual rows, times `scale`."""
    _cuda(ids, table)
    N, (V, H) = ids.numel(), table.shape
    out = torch.empty((N, H), dtype=torch.float32, device=table.device)
    _check(_fn("embed", "zai_embed")(_ptr(out), _ptr(table), _dt(table), _ptr(ids), N, H, V, float(scale),
                                     _status_ptr(table.device), _stream()), "embed")
    return out


@_timed("norm")
def gather_add(h, pending, rows, pending_gamma=None, pending_eps=0.0):
    """h[rows] + pending[rows]; with `pending_gamma` the pending rows pass an RMS norm with that weight first."""
    _cuda(h, pending, rows, pending_gamma)
    R, H = rows.numel(), h.shape[1]
    out = torch.empty((R, H), dtype=torch.float32, device=h.device)
    if pending_gamma is not None:
        _check(_fn("embed", "zai_gather_add_normed")(_ptr(out), _ptr(h), _ptr(pending), _dt(pending), _ptr(pending_gamma),
                                                     float(pending_eps), _ptr(rows), R, H, _stream()), "gather_add_normed")
        return out
    pd = _dt(pending) if pending is not None else _F32
    _check(_fn("embed", "zai_gather_add")(_ptr(out), _ptr(h), _ptr(pending), pd, _ptr(rows), R, H, _stream()),
           "gather_add")
    return out


@_timed("norm")
def add_rmsnorm(h, delta, w, eps, out_dtype, delta_gamma=None, delta_eps=0.0):
    """h += delta (in place, 32-bit), then the RMS norm of h with weight w.  With `delta_gamma` the pending
    term passes an RMS norm of its own (that weight, `delta_eps`) before it is added."""
    _cuda(h, delta, w, delta_gamma)
    if h.dtype != torch.float32 or w.dtype != torch.float32:
        raise KernelError("the residual stream and norm weights are 32-bit")
    N, H = h.shape
    out = torch.empty((N, H), dtype=out_dtype, device=h.device)
    if delta is not None and delta.dtype != out_dtype:
        raise KernelError("the pending term should have the model's dtype")
    if delta_gamma is not None:
        _check(_fn("norm", "zai_add_normed_rmsnorm")(_ptr(h), _ptr(delta), _ptr(delta_gamma), float(delta_eps), _ptr(w), _ptr(out),
                                                     _dt(out), float(eps), N, H, _stream()), "add_normed_rmsnorm")
        return out
    _check(_fn("norm", "zai_add_rmsnorm")(_ptr(h), _ptr(delta), _ptr(w), _ptr(out), _dt(out), float(eps), N, H,
                                          _stream()), "add_rmsnorm")
    return out


@_timed("norm")
def add_cast(h, delta, out_dtype, delta_gamma=None, delta_eps=0.0):
    """h += delta (in place, 32-bit; with `delta_gamma` the pending term passes an RMS norm with that weight first; nothing
    with no delta), then h rounded to `out_dtype`: the input of a sublayer that reads the residual stream itself."""
    _cuda(h, delta, delta_gamma)
    if h.dtype != torch.float32 or (delta_gamma is not None and delta_gamma.dtype != torch.float32):
        raise KernelError("the residual stream and norm weights are 32-bit")
    if delta is not None and delta.dtype != out_dtype:
        raise KernelError("the pending term should have the model's dtype")
    N, H = h.shape
    out = torch.empty((N, H), dtype=out_dtype, device=h.device)
    _check(_fn("norm", "zai_add_normed_cast")(_ptr(h), _ptr(delta), _ptr(delta_gamma), float(delta_eps), _ptr(out), _dt(out), N, H,
                                              _stream()), "add_cast")
    return out


# ---- which weights follow which.  The few-rows product kernels ask the weights of the product after
# them into L2 while they run.  Nobody has to tell them the order: a call notes that its weights came
# after the last call's, and the next time the last call's weights are used, that is the hint.  (Weak
# references: a hint never outlives the tensor it points to.  A wrong hint, after a change of model
# or of step shape, costs a useless prefetch once and is then replaced.)
_follower = {}          # data_ptr of a weight -> weak reference to the weight used after it last time
_last_weight = [0]


def _hint_next_weights(w) -> None:
    p = w.data_ptr()
    last = _last_weight[0]
    if len(_follower) > 8192:                     # many models have come and gone: start over
        _follower.clear()
    if last and last != p:
        known = _follower.get(last)
        if known is None or known() is not w:
            _follower[last] = weakref.ref(w)
    _last_weight[0] = p
    nxt = _follower.get(p)
    nxt = nxt() if nxt is not None else None
    if nxt is not None and nxt.is_cuda and nxt.device == w.device:
        _fn("decode_gemm", "zai_skinny_hint_next")(nxt.data_ptr(), nxt.numel() * nxt.element_size())


_through = {}           # (weights, bias) by address -> (weak reference to the weights, W . beta in 32-bit)


def _bias_through(w, beta):
    """W . beta [O] in 32-bit: what a layer norm's bias contributes to every row of the product behind it.  Made the first
    time a pair is met (steps run kernel by kernel before any graph is captured) and kept while the weights live."""
    key = (w.data_ptr(), beta.data_ptr())
    hit = _through.get(key)
    if hit is not None and hit[0]() is w:
        return hit[1]
    if len(_through) > 4096:
        _through.clear()
    if torch.backends.cuda.matmul.allow_tf32:
        torch.backends.cuda.matmul.allow_tf32 = False
    v = torch.mv(w.float(), beta.float()).contiguous()
    _through[key] = (weakref.ref(w), v)
    return v


@_timed(_product_class)
def _skinny(x, w, epilogue, out_cols, out_dtype, glu=None):
    """The few-rows product kernel, if it takes these operands; else None.  `glu` = (limit, slope): the gated epilogue
    with bounded branches instead of SiLU(gate) * up."""
    lazy = isinstance(x, LazyNorm)
    M = (x.rows.numel() if x.rows is not None else x.residual.data.shape[0]) if lazy else x.shape[0]
    O, K = w.shape
    if w.dtype != torch.bfloat16 or (not lazy and x.dtype != torch.bfloat16) or (lazy and x.dtype != torch.bfloat16):
        return None
    if not lazy and not x.is_contiguous():
        return None
    if not _fn("decode_gemm", "zai_skinny_gemm_supports")(M, O, K, epilogue, int(lazy)):
        return None
    y = torch.empty((M, out_cols), dtype=out_dtype, device=w.device)
    _hint_next_weights(w)
    if glu is not None:
        fn, tail = _fn("decode_gemm", "zai_skinny_gemm_clamped_glu"), (float(glu[0]), float(glu[1]), _stream())
    else:
        fn, tail = _fn("decode_gemm", "zai_skinny_gemm"), (epilogue, _stream())
    if lazy:
        res = x.residual
        _cuda(res.data, x.delta, x.gamma, x.rows)
        h_out = torch.empty_like(res.data) if (x.rows is None and x.delta is not None) else None
        if getattr(x, "beta", None) is not None:
            # a layer norm: the kernel takes the mean off; the norm's bias goes through the product once per matrix
            limit, slope = (float(glu[0]), float(glu[1])) if glu is not None else (0.0, 1.0)
            _check(_fn("decode_gemm", "zai_skinny_gemm_layernorm")(
                _ptr(y), _ptr(w), _ptr(res.data), _ptr(x.delta), _ptr(x.gamma), _ptr(_bias_through(w, x.beta)), _ptr(x.rows),
                _ptr(h_out), float(x.eps), M, O, K, epilogue, limit, slope, _stream()), "skinny_gemm")
        else:
            _check(fn(_ptr(y), _ptr(w), None, _ptr(res.data), _ptr(x.delta), _ptr(x.gamma), _ptr(x.rows), _ptr(h_out),
                      float(x.eps), M, O, K, *tail), "skinny_gemm")
        if h_out is not None:
            res.data = h_out
    else:
        _cuda(x)
        _check(fn(_ptr(y), _ptr(w), _ptr(x), None, None, None, None, None, 0.0, M, O, K, *tail), "skinny_gemm")
    return y


TC_MIN_ROWS = 128        # from this many rows on a product may go to the tcgen05 kernel
# Measured on B200 (graph-timed, weights from HBM) the library's two-block 256x256 tiles are 1.15x to
# 2x faster than this one-block 128x{128,256} kernel at the shapes of the LFM2 models, so products go
# to the library unless ZAI_TC_GEMM=1 asks for the tcgen05 kernel (its tests call it directly).
USE_TC_GEMM = os.environ.get("ZAI_TC_GEMM", "0") == "1"

# ---- the status word: one int32 per device that kernels OR bits into (csrc/common.cuh: ZaiStatusBit).
# A kernel that meets an id outside its bound uses id 0 instead, and a kernel whose bounded wait runs
# out stops waiting; both raise a bit here, and whoever reads the step's results reads this word
# with them and throws the step away if it is not zero.
STATUS_BITS = {1: "a bounded wait inside a kernel ran out", 2: "a token id outside the vocabulary",
               4: "a block-table entry outside the page pool", 8: "a state slot outside the slots",
               16: "a position outside its request's block-table row"}
_status = {}


def status_tensor(device=None) -> torch.Tensor:
    """The device's status word (int32 [1]), made at first use."""
    dev = torch.device("cuda") if device is None else torch.device(device)
    index = torch.cuda.current_device() if dev.index is None else dev.index
    entry = _status.get(index)
    if entry is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
        entry = _status[index] = (t, t.data_ptr())
    return entry[0]


def _status_ptr(device) -> int:
    entry = _status.get(device.index)
    if entry is None:
        status_tensor(device)
        entry = _status[torch.cuda.current_device() if device.index is None else device.index]
    return entry[1]


def describe_status(code: int) -> str:
    return "; ".join(text for bit, text in STATUS_BITS.items() if code & bit) or f"status {code}"


def read_status(device=None) -> int:
    """The status word, cleared (reads the device: waits for the work queued so far)."""
    t = status_tensor(device)
    v = int(t.item())
    if v:
        t.zero_()
    return v


def tc_status() -> int:
    """1 if a bounded wait of a kernel ran out since the status word was last read, else 0 (reads the device)."""
    return 1 if read_status() & 1 else 0


@_timed(_product_class)
def _tensor_core(x, w, epilogue, out_cols, out_dtype):
    """The tcgen05 product kernel, if it takes these operands and is the faster choice; else None."""
    N, (O, K) = x.shape[0], w.shape
    if not USE_TC_GEMM or N < TC_MIN_ROWS or w.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
        return None
    if not x.is_contiguous() or not _fn("gemm_tc", "zai_gemm_tc_supports")(N, O, K, epilogue):
        return None
    y = torch.empty((N, out_cols), dtype=out_dtype, device=w.device)
    _check(_fn("gemm_tc", "zai_gemm_tc")(_ptr(y), _ptr(w), _ptr(x), _status_ptr(w.device), N, O, K, epilogue, _stream()),
           "gemm_tc")
    return y


# Steps of 17 to 128 rows: the weight-streaming tcgen05 kernel (csrc/stream_gemm.cu), with SwiGLU or the
# short convolution as its epilogue.  Measured on B200 it is behind the library's product plus the
# separate activation / convolution kernel at the shapes of the LFM2 models (a block's K loop costs about
# 0.4 us per 64-k slice whatever the slice holds: see profiles/stream_gemm_tcgen05_17_128_rows.md), so it
# is an option: ZAI_STREAM_GEMM=1 turns it on.
USE_STREAM_GEMM = os.environ.get("ZAI_STREAM_GEMM", "0") == "1"
STREAM_MIN_ROWS, STREAM_MAX_ROWS = 17, 128


@_timed(_product_class)
def _stream_product(x, w, epilogue, out_cols, out_dtype):
    """The weight-streaming product kernel, if it takes these operands; else None."""
    N, (O, K) = x.shape[0], w.shape
    if (not USE_STREAM_GEMM or not STREAM_MIN_ROWS <= N <= STREAM_MAX_ROWS or w.dtype != torch.bfloat16
            or x.dtype != torch.bfloat16 or not x.is_contiguous() or not w.is_contiguous()):
        return None
    if not _fn("stream_gemm", "zai_stream_gemm_supports")(N, O, K, epilogue):
        return None
    y = torch.empty((N, out_cols), dtype=out_dtype, device=w.device)
    _check(_fn("stream_gemm", "zai_stream_gemm")(_ptr(y), _ptr(w), _ptr(x), _status_ptr(w.device), N, O, K, epilogue,
                                                 _stream()), "stream_gemm")
    return y


def linear(x, w, out_dtype=None, bias=None):
    """x [N, K] times w [O, K] transposed.  x may be a LazyNorm.  Few rows in bfloat16 go to the
    fused few-rows kernel, many rows to the tcgen05 kernel where it is the faster one; a matrix kept
    in 32-bit is multiplied in 32-bit; the rest is the library's.  With `bias` [O] (in w's dtype) the
    library's product adds it before the result is rounded."""
    in_dtype = x.dtype
    out_dtype = out_dtype or in_dtype
    if bias is not None:
        if isinstance(x, LazyNorm):
            x = x.materialize(sys.modules[__name__])
        return _library_product(x, w, out_dtype, bias)
    if in_dtype == torch.bfloat16 and out_dtype in (torch.bfloat16, torch.float32):
        y = _skinny(x, w, _EPI_F32 if out_dtype == torch.float32 else _EPI_BF16, w.shape[0], out_dtype)
        if y is not None:
            return y
    if isinstance(x, LazyNorm):
        x = x.materialize(sys.modules[__name__])
    if x.dtype == torch.bfloat16 and out_dtype in (torch.bfloat16, torch.float32):
        epi = _EPI_F32 if out_dtype == torch.float32 else _EPI_BF16
        y = _stream_product(x, w, epi, w.shape[0], out_dtype)
        if y is None:
            y = _tensor_core(x, w, epi, w.shape[0], out_dtype)
        if y is not None:
            return y
    return _library_product(x, w, out_dtype)


@_timed(lambda x, w, out_dtype, bias=None: "head" if out_dtype == torch.float32 and x.dtype != torch.float32 else "products")
def _library_product(x, w, out_dtype, bias=None):
    """The library's matrix product: true 32-bit where an operand or the result is 32-bit."""
    if bias is not None:
        if x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
            torch.backends.cuda.matmul.allow_tf32 = False
        if not (x.dtype == w.dtype == bias.dtype == out_dtype):
            raise KernelError("a product with a bias takes operands, bias and result of one dtype")
        return torch.addmm(bias, x, w.t())
    if x.dtype == torch.float32 or w.dtype == torch.float32 or out_dtype == torch.float32:
        if torch.backends.cuda.matmul.allow_tf32:
            torch.backends.cuda.matmul.allow_tf32 = False
        if x.dtype == w.dtype == torch.bfloat16:
            # 32-bit logits from 16-bit operands: the product itself accumulates in 32-bit
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.matmul(x.float(), w.float().t()).to(out_dtype)
    return torch.matmul(x, w.t())


# The two-block tcgen05 kernel (csrc/gemm_tc_pair.cu) runs the gate/up product with SwiGLU in its
# epilogue in the time the library's product and the activation kernel take together where the model is
# 1024 wide (a prefill of 2048 tokens at the 350M shape: 1.98-2.01 ms either way, measured in one run)
# and is 1 % and 2 % behind them at the widths of the 700M and 1.2B shapes.  So gate/up products of
# PAIR_SWIGLU_MIN_ROWS rows or more go to it where K is at most PAIR_SWIGLU_MAX_K; ZAI_PAIR_GEMM=1 sends
# them there at every width, ZAI_PAIR_GEMM=0 never.
PAIR_SWIGLU_MIN_ROWS = int(os.environ.get("ZAI_PAIR_SWIGLU_MIN_ROWS", "1024"))
PAIR_SWIGLU_MAX_K = 1024
_pair_env = os.environ.get("ZAI_PAIR_GEMM", "auto")
USE_PAIR_GEMM = _pair_env != "0"             # False: never; True: by the rule above (or always, with PAIR_GEMM_ALWAYS)
PAIR_GEMM_ALWAYS = _pair_env == "1"


@_timed(_product_class)
def gemm_pair(x, w, epilogue, out_cols, out_dtype, wide=-1):
    """The two-block tcgen05 product kernel: x [N, K] times w [O, K] transposed with the epilogue
    (0 bfloat16, 1 32-bit, 2 SwiGLU over stacked gate|up rows); None if it does not take the operands."""
    _cuda(x, w)
    N, (O, K) = x.shape[0], w.shape
    if w.dtype != torch.bfloat16 or x.dtype != torch.bfloat16 or not x.is_contiguous() or not w.is_contiguous():
        return None
    if not _fn("gemm_tc_pair", "zai_gemm_pair_supports")(N, O, K, epilogue):
        return None
    y = torch.empty((N, out_cols), dtype=out_dtype, device=w.device)
    _check(_fn("gemm_tc_pair", "zai_gemm_pair")(_ptr(y), _ptr(w), _ptr(x), _status_ptr(w.device), N, O, K, epilogue, wide,
                                                _stream()), "gemm_pair")
    return y


def linear_swiglu(x, w_gate_up, ff_dim):
    """silu(x . Wgate^T) * (x . Wup^T) with the two matrices stacked as [2F, K]."""
    if x.dtype == torch.bfloat16:
        y = _skinny(x, w_gate_up, _EPI_SWIGLU, ff_dim, torch.bfloat16)
        if y is not None:
            return y
        if isinstance(x, LazyNorm):
            x = x.materialize(sys.modules[__name__])
        y = _stream_product(x, w_gate_up, _EPI_SWIGLU, ff_dim, torch.bfloat16)
        if y is None:
            y = _tensor_core(x, w_gate_up, _EPI_SWIGLU, ff_dim, torch.bfloat16)
        if y is not None:
            return y
        if USE_PAIR_GEMM and x.shape[0] >= PAIR_SWIGLU_MIN_ROWS and (PAIR_GEMM_ALWAYS or x.shape[1] <= PAIR_SWIGLU_MAX_K):
            y = gemm_pair(x, w_gate_up, _EPI_SWIGLU, ff_dim, torch.bfloat16)
            if y is not None:
                return y
    return silu_mul(linear(x, w_gate_up), ff_dim)


@_timed("activation")
def silu_mul(gu, ff_dim):
    _cuda(gu)
    N = gu.shape[0]
    out = torch.empty((N, ff_dim), dtype=gu.dtype, device=gu.device)
    _check(_fn("activation", "zai_silu_mul")(_ptr(out), _ptr(gu), _dt(gu), N, ff_dim, _stream()), "silu_mul")
    return out


_EPI_CONV = 3
FUSED_CONV_MAX_TAPS = 4


def linear_short_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state=True):
    """z = C * conv(state ++ B * x~) with (B, C, x~) = x . w_in^T: the short convolution's input
    projection, gates, taps and state update.  A step of single tokens (at most 16) runs as one
    kernel, the convolution being the product's epilogue; other steps as the product and the
    convolution kernel."""
    lazy = isinstance(x, LazyNorm)
    M = (x.rows.numel() if x.rows is not None else x.residual.data.shape[0]) if lazy else x.shape[0]
    O, K = w_in.shape
    C = O // 3
    fused = (step.decode_only and taps <= FUSED_CONV_MAX_TAPS and w_in.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
             and (not lazy or x.rows is None) and state.dtype == torch.float32 and state.shape[-1] == C
             and M == step.n_seqs and _fn("decode_gemm", "zai_skinny_gemm_supports")(M, O, K, _EPI_CONV, int(lazy)))
    if not fused:
        if (USE_STREAM_GEMM and step.decode_only and STREAM_MIN_ROWS <= M <= STREAM_MAX_ROWS and M == step.n_seqs
                and taps <= FUSED_CONV_MAX_TAPS and w_in.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
                and (not lazy or x.rows is None) and state.dtype == torch.float32 and state.shape[-1] == C and w_in.is_contiguous()
                and _fn("stream_gemm", "zai_stream_gemm_supports")(M, O, K, _EPI_CONV)):
            if lazy:
                x = x.materialize(sys.modules[__name__])
            return _stream_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state, M, C, K)
        return short_conv(linear(x, w_in), conv_w, conv_b, state, step, taps, write_state)
    return _skinny_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state, lazy, M, C, K)


@_timed("products (in_proj + conv)")
def _stream_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state, M, C, K):
    _cuda(x, w_in, conv_w, conv_b, state)
    z = torch.empty((M, C), dtype=torch.bfloat16, device=w_in.device)
    _check(_fn("stream_gemm", "zai_stream_conv")(
        _ptr(z), _ptr(w_in), _ptr(x), _status_ptr(w_in.device), _ptr(conv_w), _ptr(conv_b), _ptr(state), _ptr(step.slot_ids),
        M, C, K, int(taps), state.shape[1], int(bool(write_state)), state.shape[0], _stream()), "stream_conv")
    return z


@_timed("products (in_proj + conv)")
def _skinny_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state, lazy, M, C, K):
    _cuda(w_in, conv_w, conv_b, state)
    z = torch.empty((M, C), dtype=torch.bfloat16, device=w_in.device)
    fn = _fn("decode_gemm", "zai_skinny_conv")
    _hint_next_weights(w_in)
    tail = (_ptr(conv_w), _ptr(conv_b), _ptr(state), _ptr(step.slot_ids), M, C, K, int(taps), state.shape[1],
            int(bool(write_state)), state.shape[0], _status_ptr(state.device), _stream())
    if lazy:
        res = x.residual
        _cuda(res.data, x.delta, x.gamma)
        h_out = torch.empty_like(res.data) if x.delta is not None else None
        _check(fn(_ptr(z), _ptr(w_in), None, _ptr(res.data), _ptr(x.delta), _ptr(x.gamma), _ptr(h_out), float(x.eps), *tail),
               "skinny_conv")
        if h_out is not None:
            res.data = h_out
    else:
        _cuda(x)
        _check(fn(_ptr(z), _ptr(w_in), _ptr(x), None, None, None, None, 0.0, *tail), "skinny_conv")
    return z


@_timed("conv")
def short_conv(bcx, conv_w, conv_b, state, step, taps, write_state=True):
    _cuda(bcx, conv_w, conv_b, state)
    N, C = bcx.shape[0], bcx.shape[1] // 3
    z = torch.empty((N, C), dtype=bcx.dtype, device=bcx.device)
    if state.dtype != torch.float32 or state.shape[-1] != C:
        raise KernelError("the conv state is 32-bit [slots, rows, channels]")
    _check(_fn("shortconv", "zai_short_conv")(
        _ptr(z), _ptr(bcx), _dt(bcx), _ptr(conv_w), _ptr(conv_b), _ptr(state), _ptr(step.seq_idx), _ptr(step.cu_q),
        _ptr(step.slot_ids), N, step.n_seqs, C, int(taps), state.shape[1], int(step.decode_only),
        int(write_state), state.shape[0], _status_ptr(state.device), _stream()), "short_conv", 1 if (step.decode_only or taps == 1 or not write_state) else 2)
    return z


_inv_freq_cache = {}


def inverse_frequencies(rotary_dim: int, theta: float, device, scaling=None) -> torch.Tensor:
    """theta^(-2i/n) for i < n/2, computed in 64-bit.  With `scaling` = (factor, original, fast, slow) the
    frequencies are stretched for contexts longer than `original` positions: pair i keeps f_i where it turns more
    than `fast` times within `original` positions, turns at f_i / factor where it turns fewer than `slow` times, and
    in between the two are mixed by a ramp that is linear in i (see `rotation_magnitude` for what goes with it)."""
    key = (rotary_dim, float(theta), str(device), scaling)
    t = _inv_freq_cache.get(key)
    if t is None:
        i = torch.arange(rotary_dim // 2, dtype=torch.float64)
        t = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / rotary_dim)
        if scaling is not None and scaling[0] == "wavelength":
            # by wavelength l = 2 pi / f: kept below original / high, divided by factor above original / low, between the
            # two mixed linearly in original / l
            _, factor, low, high, original = scaling
            wave = 2.0 * math.pi / t
            smooth = (original / wave - low) / (high - low)
            mixed = (1.0 - smooth) * t / factor + smooth * t
            t = torch.where(wave < original / high, t, torch.where(wave > original / low, t / factor, mixed))
        elif scaling is not None:
            factor, original, fast, slow = (float(v) for v in scaling)
            where = lambda turns: rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))
            lo = max(math.floor(where(fast)), 0)
            hi = min(math.ceil(where(slow)), rotary_dim - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            t = t / factor * ramp + t * (1.0 - ramp)
        t = t.to(device)
        _inv_freq_cache[key] = t
    return t


def rotation_magnitude(scaling) -> float:
    """The factor on cosines and sines of a stretched rotation: 0.1 ln(factor) + 1."""
    return 1.0 if scaling is None or scaling[0] == "wavelength" else 0.1 * math.log(float(scaling[0])) + 1.0


@_timed("q/k norm, rotation, page write")
def rope_table(step, rotary_dim: int, theta: float, device, scaling=None) -> torch.Tensor:
    """(cos, sin) of position * frequency for every row of the step, [N, rotary_dim/2, 2] 32-bit,
    computed once per step and rotation and kept with the step.  `scaling`: see `inverse_frequencies`."""
    key = ("rope", rotary_dim, float(theta), scaling)
    t = step.scratch.get(key)
    if t is None:
        half = rotary_dim // 2
        t = torch.empty((step.n_tokens, half, 2), dtype=torch.float32, device=device)
        freq = inverse_frequencies(rotary_dim, theta, device, scaling)
        if scaling is None:
            _check(_fn("rope_kv", "zai_rope_table")(_ptr(t), _ptr(step.positions), _ptr(freq), step.n_tokens, half, _stream()),
                   "rope_table")
        else:
            _check(_fn("rope_kv", "zai_rope_table_scaled")(_ptr(t), _ptr(step.positions), _ptr(freq), step.n_tokens, half,
                                                           rotation_magnitude(scaling), _stream()), "rope_table")
        step.scratch[key] = t
    return t


@_timed("q/k norm, rotation, page write")
def qk_norm_rope(qkv, q_w, k_w, eps, rotary_dim, theta, step, cache, heads, kv_heads, head_dim,
                 has_kv=True, write=True, return_k=False):
    _cuda(qkv, q_w, k_w)
    N, cols = qkv.shape
    q = torch.empty((N, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    k_out = torch.empty((N, kv_heads * head_dim), dtype=qkv.dtype, device=qkv.device) if (return_k and has_kv) else None
    table = rope_table(step, rotary_dim, theta, qkv.device) if rotary_dim else None
    do_write = bool(write and has_kv)
    pages, bt = cache.pages, cache.block_table
    if do_write and pages.dtype != qkv.dtype:
        raise KernelError("the pages and the activations should have one dtype")
    _check(_fn("rope_kv", "zai_qk_norm_rope")(
        _ptr(qkv), cols, _dt(qkv), _ptr(q_w), _ptr(k_w), float(eps), _ptr(table), int(rotary_dim),
        _ptr(step.positions), _ptr(step.seq_idx), _ptr(bt) if do_write else None,
        bt.shape[1] if do_write else 0, _ptr(pages) if do_write else None, cache.page_size, _ptr(q), _ptr(k_out),
        N, heads, kv_heads, head_dim, int(has_kv), int(do_write), pages.shape[0] if do_write else 0,
        _status_ptr(qkv.device), _stream()), "qk_norm_rope")
    return q, k_out


@_timed("q/k norm, rotation, page write")
def kv_write(k, v, step, cache, kv_heads, head_dim):
    if k.stride(-1) != 1 or v.stride(-1) != 1:
        raise KernelError("k and v rows should be contiguous")
    N = k.shape[0]
    _check(_fn("rope_kv", "zai_kv_write")(
        _ptr(k), k.stride(0), _ptr(v), v.stride(0), _dt(k), _ptr(step.positions), _ptr(step.seq_idx),
        _ptr(cache.block_table), cache.block_table.shape[1], _ptr(cache.pages), cache.page_size, N, kv_heads,
        head_dim, cache.pages.shape[0], _status_ptr(k.device), _stream()), "kv_write")


USE_TC_ATTENTION = os.environ.get("ZAI_TC_ATTENTION", "1") == "1"     # tcgen05 prefill attention where the sizes allow



_span_tickets = {}


def _attention_tickets(device, n):
    """Zeroed counters for the span attention's shared tiles (the kernel leaves them zero)."""
    t = _span_tickets.get(device)
    if t is None or t.numel() < n:
        t = torch.zeros((max(n, 1024),), dtype=torch.int32, device=device)
        _span_tickets[device] = t
    return t

@_timed("attention")
def paged_attention(q, step, cache, heads, kv_heads, head_dim, scale, window=None, impl=None, chunk=None, softcap=None, bias=None,
                    sink=None, keep_first=0):
    """Causal attention of the step's rows over their requests' pages.  bfloat16 runs on the
    tensor cores (a split-key kernel when every span is one token, else the flash-style kernel)
    for the head sizes those kernels have; everything else, and `impl="general"`, runs the
    general kernel.  `impl="mma"` / `impl="tcgen05"` pick between the two span kernels.
    `window`: a query sees the last `window` positions; `chunk`: it sees back to the start of its chunk of that
    many positions (the kernels take the chunk as a negative window).
    Shaped scores (the general kernel): `softcap` (s <- cap tanh(s / cap)), `bias` [distances, heads] 32-bit (added after the
    cap by min(distance, last row)), `sink` [heads] 32-bit (a term of the denominator alone), `keep_first` (with a window:
    the request's first positions stay visible)."""
    _cuda(q, bias, sink)
    if softcap or bias is not None or sink is not None or keep_first:
        if chunk is not None or (keep_first and not window):
            raise KernelError("shaped scores go with a window or none; kept first positions need a window")
        N = q.shape[0]
        out = torch.empty((N, heads * head_dim), dtype=q.dtype, device=q.device)
        bt = cache.block_table
        if (cache.pages.dtype != q.dtype or N != step.n_tokens or (bias is not None and (bias.dtype != torch.float32 or bias.shape[1] != heads))
                or (sink is not None and (sink.dtype != torch.float32 or sink.numel() != heads))):
            raise KernelError("paged_attention: operands do not fit together")
        shaped = (float(softcap or 0.0), _ptr(bias), 0 if bias is None else bias.shape[0], _ptr(sink), int(keep_first or 0))
        if (impl != "general" and q.dtype == torch.bfloat16 and q.is_contiguous()
                and _fn("attention_mma", "zai_attention_mma_supports")(head_dim, heads, kv_heads)):
            # the tensor-core kernels with the scores shaped inside them
            def single_tokens(n):
                # rows 0..n-1 are one token each, row i of span i: keys split over blocks, then combined (with the sink)
                keys = _fn("attention_mma", "zai_decode_chunk_keys")()
                n_chunks = max(-(-int(step.max_kv_len) // keys), 1)
                part_o = torch.empty((n, heads, n_chunks, head_dim), dtype=torch.float32, device=q.device)
                part_ml = torch.empty((n, heads, n_chunks, 2), dtype=torch.float32, device=q.device)
                _check(_fn("attention_mma", "zai_decode_attention_mma_scored")(
                    _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(q), _ptr(cache.pages), _ptr(bt), bt.shape[1], _ptr(step.positions), n,
                    n_chunks, cache.page_size, heads, kv_heads, head_dim, float(scale), int(window or 0), cache.pages.shape[0],
                    _status_ptr(q.device), *shaped, _stream()), "decode attention (scored)", 2)

            if step.decode_only:
                single_tokens(N)
                return out
            # the one-token spans at the front of a mixed step go to the kernel for single tokens, as without shaping
            ns = int(getattr(step, "single_first", 0)) if SPLIT_MIXED_ATTENTION else 0
            if ns:
                single_tokens(ns)
            block_rows = _fn("attention_mma", "zai_prefill_block_rows")()
            n_tiles = (step.attn_tiles - ns) if getattr(step, "attn_tiles", None) else sum(-(-n // block_rows) for n in step.q_lens[ns:])
            _check(_fn("attention_mma", "zai_prefill_attention_mma_scored")(
                _ptr(out), _ptr(q), _ptr(cache.pages), _ptr(bt[ns:]), bt.shape[1], _ptr(step.cu_q[ns:]), _ptr(step.ctx_lens[ns:]),
                step.n_seqs - ns, n_tiles, cache.page_size, heads, kv_heads, head_dim, float(scale), int(window or 0),
                cache.pages.shape[0], _status_ptr(q.device), *shaped, _stream()), "prefill attention (scored)")
            return out
        _check(_fn("attention", "zai_paged_attention_scored")(
            _ptr(out), _ptr(q), _ptr(cache.pages), _dt(q), _ptr(bt), bt.shape[1], _ptr(step.positions), _ptr(step.seq_idx),
            cache.page_size, N, heads, kv_heads, head_dim, float(scale), int(window or 0), cache.pages.shape[0],
            _status_ptr(q.device), float(softcap or 0.0), _ptr(bias), 0 if bias is None else bias.shape[0], _ptr(sink),
            int(keep_first or 0), _stream()), "paged_attention (scored)")
        return out
    if chunk is not None:
        if window is not None:
            raise KernelError("a window and chunks exclude each other")
        window = -int(chunk)
    N = q.shape[0]
    if N != step.n_tokens:
        raise KernelError(f"{N} query rows for a step of {step.n_tokens} rows")
    out = torch.empty((N, heads * head_dim), dtype=q.dtype, device=q.device)
    if cache.pages.dtype != q.dtype:
        raise KernelError("the pages and the queries should have one dtype")
    bt = cache.block_table
    if (impl != "general" and q.dtype == torch.bfloat16
            and _fn("attention_mma", "zai_attention_mma_supports")(head_dim, heads, kv_heads)):
        def single_tokens(n):
            # rows 0..n-1 are one token each, row i of span i: keys split over blocks, then combined
            chunk = _fn("attention_mma", "zai_decode_chunk_keys")()
            n_chunks = max(-(-int(step.max_kv_len) // chunk), 1)
            part_o = torch.empty((n, heads, n_chunks, head_dim), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((n, heads, n_chunks, 2), dtype=torch.float32, device=q.device)
            _check(_fn("attention_mma", "zai_decode_attention_mma")(
                _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(q), _ptr(cache.pages), _ptr(bt), bt.shape[1],
                _ptr(step.positions), n, n_chunks, cache.page_size, heads, kv_heads, head_dim, float(scale),
                int(window or 0), cache.pages.shape[0], _status_ptr(q.device), _stream()), "decode attention", 2)

        if step.decode_only:
            single_tokens(N)
        else:
            # the one-token spans at the front of a mixed step (decoding requests beside prompt portions)
            # would each fill a whole block of query rows of the span kernel: they go to the other one
            ns = int(getattr(step, "single_first", 0)) if (SPLIT_MIXED_ATTENTION and q.is_contiguous()) else 0
            if ns:
                single_tokens(ns)
            S = step.n_seqs - ns
            cu_q, ctx_lens, bt = step.cu_q[ns:], step.ctx_lens[ns:], bt[ns:]
            block_rows = _fn("attention_mma", "zai_prefill_block_rows")()
            n_tiles = (step.attn_tiles - ns) if getattr(step, "attn_tiles", None) else sum(-(-n // block_rows) for n in step.q_lens[ns:])
            if (impl != "mma" and (USE_TC_ATTENTION or impl == "tcgen05") and q.is_contiguous()
                    and _fn("attention_tc", "zai_prefill_attention_tc_supports")(head_dim, heads, kv_heads, cache.page_size)):
                # few tiles of query rows over long contexts: several blocks share a tile's keys and leave their
                # parts in scratch, the last to finish combines them (tickets: zero before and after)
                splits = _fn("attention_tc", "zai_prefill_attention_tc_splits")(n_tiles, heads, bt.shape[1], cache.page_size)
                part_o = part_ml = None
                tickets = _attention_tickets(q.device, n_tiles * heads if splits > 1 else 0)   # (made at the first call, which no graph captures)
                if splits > 1:
                    part_o = torch.empty((n_tiles * heads * splits, 64 * 128), dtype=torch.float32, device=q.device)
                    part_ml = torch.empty((n_tiles * heads * splits, 2 * 128), dtype=torch.float32, device=q.device)
                _check(_fn("attention_tc", "zai_prefill_attention_tc")(
                    _ptr(out), _ptr(q), _ptr(cache.pages), cache.pages.shape[0], _status_ptr(q.device), _ptr(bt), bt.shape[1],
                    _ptr(cu_q), _ptr(ctx_lens), N, S, n_tiles, cache.page_size, heads, kv_heads,
                    head_dim, float(scale), int(window or 0), splits, _ptr(part_o), _ptr(part_ml), _ptr(tickets),
                    _stream()), "prefill attention (tcgen05)")
                return out
            _check(_fn("attention_mma", "zai_prefill_attention_mma")(
                _ptr(out), _ptr(q), _ptr(cache.pages), _ptr(bt), bt.shape[1], _ptr(cu_q), _ptr(ctx_lens),
                S, n_tiles, cache.page_size, heads, kv_heads, head_dim, float(scale), int(window or 0),
                cache.pages.shape[0], _status_ptr(q.device), _stream()), "prefill attention")
        return out
    _check(_fn("attention", "zai_paged_attention_general")(
        _ptr(out), _ptr(q), _ptr(cache.pages), _dt(q), _ptr(bt), bt.shape[1],
        _ptr(step.positions), _ptr(step.seq_idx), cache.page_size, N, heads, kv_heads, head_dim, float(scale),
        int(window or 0), cache.pages.shape[0], _status_ptr(q.device), _stream()), "paged_attention")
    return out


_tickets = {}
SPLIT_MIXED_ATTENTION = os.environ.get("ZAI_SPLIT_MIXED_ATTENTION", "1") == "1"
USE_TMA_ATTENTION = os.environ.get("ZAI_TMA_ATTENTION", "1") == "1"   # keys and values by TMA where the sizes allow
DECODE_BLOCKS_WANTED = 500


def fused_decode_attention_available(dtype, heads, kv_heads, head_dim) -> bool:
    return dtype == torch.bfloat16 and bool(_fn("attention_mma", "zai_attention_mma_supports")(head_dim, heads, kv_heads))


@_timed("attention (with q/k norm, rotation, page write)")
def decode_attention_fused(qkv, q_w, k_w, eps, rotary_dim, theta, step, cache, heads, kv_heads, head_dim, scale,
                           window=None, write=True):
    """A decode step's attention in one kernel, from the qkv projection's rows [B, (Hq + 2 Hkv) D]:
    q/k RMSNorm, rotation, the new key and value into their page, attention over the pages in chunks
    of keys, and the combination of the chunks.  Every row of the step is one token."""
    _cuda(qkv, q_w, k_w)
    B, cols = qkv.shape
    if B != step.n_tokens:
        raise KernelError(f"{B} rows for a step of {step.n_tokens} rows")
    dev = qkv.device
    out = torch.empty((B, heads * head_dim), dtype=qkv.dtype, device=dev)
    # keys per block: about DECODE_BLOCKS_WANTED blocks (a little more than the SMs hold at once), so
    # that a block's start-up and its partial sums are spread over many keys without leaving SMs
    # idle (a power of two between 256 and 1024)
    want = int(step.max_kv_len) * B * kv_heads // DECODE_BLOCKS_WANTED
    chunk = 256
    while chunk < 1024 and chunk * 3 < want * 2:
        chunk *= 2
    chunk = int(os.environ.get("ZAI_DECODE_CHUNK", chunk))
    n_chunks = max(-(-int(step.max_kv_len) // chunk), 1)
    part_o = torch.empty((B, heads, n_chunks, head_dim), dtype=torch.float32, device=dev)
    part_ml = torch.empty((B, heads, n_chunks, 2), dtype=torch.float32, device=dev)
    tickets = _tickets.get(str(dev))
    if tickets is None or tickets.numel() < B * kv_heads:
        tickets = torch.zeros(max(B * kv_heads, 65536), dtype=torch.int32, device=dev)
        _tickets[str(dev)] = tickets
    table = rope_table(step, rotary_dim, theta, dev) if rotary_dim else None
    bt = cache.block_table
    if USE_TMA_ATTENTION and _fn("attention_tma", "zai_decode_attention_tma_supports")(head_dim, heads, kv_heads, cache.page_size):
        _check(_fn("attention_tma", "zai_decode_attention_tma")(
            _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(tickets), _status_ptr(dev), _ptr(qkv), cols, _ptr(q_w), _ptr(k_w),
            float(eps), _ptr(table), int(rotary_dim), _ptr(cache.pages), cache.pages.shape[0], _ptr(bt), bt.shape[1],
            _ptr(step.positions), B, n_chunks, cache.page_size, heads, kv_heads, head_dim, float(scale), int(window or 0),
            int(bool(write)), chunk, _stream()), "decode_attention_tma")
        return out
    _check(_fn("attention_mma", "zai_decode_attention_fused")(
        _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(tickets), _ptr(qkv), cols, _ptr(q_w), _ptr(k_w), float(eps),
        _ptr(table), int(rotary_dim), _ptr(cache.pages), _ptr(bt), bt.shape[1], _ptr(step.positions), B, n_chunks,
        cache.page_size, heads, kv_heads, head_dim, float(scale), int(window or 0), int(bool(write)), chunk,
        cache.pages.shape[0], _status_ptr(dev), _stream()), "decode_attention_fused")
    return out


@_timed("sampling")
def argmax(logits, with_status=False):
    """First index of each row's maximum, int32 [R]; `with_status`: [R + 1], the device's status word behind
    the ids (one copy to the host then brings both)."""
    _cuda(logits)
    R, V = logits.shape
    out = torch.empty((R + (1 if with_status else 0),), dtype=torch.int32, device=logits.device)
    _check(_fn("sampling", "zai_argmax")(_ptr(out), _ptr(logits), R, V,
                                         _status_ptr(logits.device) if with_status else None, _stream()), "argmax")
    return out


@_timed("sampling")
def repetition_penalty(logits, tokens, counts, offsets, penalty):
    """In place: logits[r, tokens[i]] is penalised counts[i] times for offsets[r] <= i < offsets[r+1]."""
    _cuda(logits, tokens, counts, offsets, penalty)
    R, V = logits.shape
    _check(_fn("sampling", "zai_repetition_penalty")(_ptr(logits), _ptr(tokens), _ptr(counts), _ptr(offsets),
                                                     _ptr(penalty), R, V, _stream()), "repetition_penalty")
    return logits


@_timed("sampling")
def repetition_penalty_counts(logits, counts, slots, penalty):
    """A copy of logits [R, V] with the repetition penalty applied from a table of counts [slots, V] on the
    device (slots [R] int32, negative: the row has none)."""
    _cuda(logits, counts, slots, penalty)
    R, V = logits.shape
    if counts.dtype != torch.int32 or counts.shape[1] != V or logits.dtype != torch.float32:
        raise KernelError("the penalty takes 32-bit logits and int32 counts [slots, vocabulary]")
    out = torch.empty_like(logits)
    _check(_fn("sampling", "zai_repetition_penalty_counts")(_ptr(out), _ptr(logits), _ptr(counts), _ptr(slots), _ptr(penalty),
                                                           R, V, _stream()), "repetition_penalty_counts")
    return out


@_timed("sampling")
def count_tokens(counts, ids, slots, rows):
    """counts[slots[r], ids[r]] += 1 for the first `rows` rows that have a slot."""
    _cuda(counts, ids, slots)
    _check(_fn("sampling", "zai_count_tokens")(_ptr(counts), _ptr(ids), _ptr(slots), int(rows), counts.shape[1], _stream()),
           "count_tokens")


@_timed("sampling")
def sample(logits, temperature, top_k, top_p, u, with_status=False):
    _cuda(logits, temperature, top_k, top_p, u)
    R, V = logits.shape
    out = torch.empty((R + (1 if with_status else 0),), dtype=torch.int32, device=logits.device)
    _check(_fn("sampling", "zai_sample")(_ptr(out), _ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                         _ptr(u), R, V, _status_ptr(logits.device) if with_status else None, _stream()), "sample")
    return out


# ----------------------------------------------------------------------------- recurrent mixers and what goes with them
ACTIVATIONS = {"gelu": 0, "gelu_erf": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}


@_timed("activation")
def activation(x, kind):
    """An activation by name (gelu / gelu_erf, gelu_tanh, silu, relu), computed in 32-bit."""
    _cuda(x)
    out = torch.empty_like(x)
    _check(_fn("activation", "zai_activation")(_ptr(out), _ptr(x), _dt(x), ACTIVATIONS[kind], x.numel(), _stream()), "activation")
    return out


def linear_activation(x, w, kind):
    """act(x . w^T): the product (x may be a LazyNorm), then the activation."""
    return activation(linear(x, w), kind)


@_timed("activation")
def weighted_sum(a, b, wa, wb):
    """wa * a + wb * b, in 32-bit, rounded once."""
    _cuda(a, b)
    if a.shape != b.shape or a.dtype != b.dtype:
        raise KernelError("the two terms should have one shape and dtype")
    out = torch.empty_like(a)
    _check(_fn("activation", "zai_weighted_sum")(_ptr(out), _ptr(a), _ptr(b), _dt(a), float(wa), float(wb), a.numel(), _stream()),
           "weighted_sum")
    return out


DELTA_SINGLE_MAX_ROWS = 16      # single-token steps of at most this many requests run the delta rule as one kernel
CHUNKED_SCAN_MIN_ROWS = 256     # steps with prompt portions of this many rows or more run the linear recurrences in chunks


def _scan_chunks(step, n_rows, channel_blocks=16):
    """(rows per chunk, upper bound of the chunks) for a recurrence that is linear in its state, or (0, 0) where
    the rows of each request are walked in one pass: steps of single tokens and small steps.  Chunks are as long
    as still gives about a thousand blocks (chunks x blocks of channels), between 16 and 256 rows.  Both numbers
    depend only on the step's row and request counts, which a captured step shape keeps."""
    if step.decode_only or n_rows < CHUNKED_SCAN_MIN_ROWS:
        return 0, 0
    chunk = 256
    while chunk > 16 and (n_rows // chunk) * channel_blocks < 1024:
        chunk //= 2
    return chunk, n_rows // chunk + step.n_seqs


def _rows_view(x):
    """(pointer, row stride) of a 2-D tensor whose rows are contiguous (a column slice of a wider matrix)."""
    if x.dim() != 2 or x.stride(1) != 1 or not x.is_cuda:
        raise KernelError("kernels take CUDA matrices with contiguous rows")
    return x.data_ptr(), x.stride(0)


@_timed("conv")
def causal_conv(x, taps, bias, state, step, act=True, write_state=True):
    """Causal depthwise convolution over time of x [N, C] (a column slice is fine) with taps [C, L], the
    request's last L-1 inputs in `state` [slots, L-1, C] (32-bit), an optional bias and SiLU."""
    _cuda(taps, bias, state)
    xp, xs = _rows_view(x)
    N, C = x.shape
    L = taps.shape[1]
    if state.dtype != torch.float32 or state.shape[-1] != C or (L > 1 and state.shape[1] != L - 1):
        raise KernelError("the conv state is 32-bit [slots, taps - 1, channels]")
    out = torch.empty((N, C), dtype=x.dtype, device=x.device)
    single = bool(step.decode_only and N == step.n_seqs)
    _check(_fn("causal_conv", "zai_causal_conv")(
        _ptr(out), C, xp, xs, _dt(x), _ptr(taps), _ptr(bias), _ptr(state), _ptr(step.seq_idx), _ptr(step.cu_q),
        _ptr(step.slot_ids), N, step.n_seqs, C, L, int(bool(act)), int(single), int(bool(write_state)), state.shape[0],
        _status_ptr(x.device), _stream()), "causal_conv", 1 if (single or not write_state or L == 1) else 2)
    return out


@_timed("recurrence")
def selective_scan(x, proj, z, w_dt, b_dt, a_log, d_skip, state, step, dt_rank, write_state=True):
    """The selective-scan recurrence: x [N, I] (after its convolution), proj [N, R + 2S] = (dt_in | B | C), z [N, I]
    (a column slice is fine), w_dt [I, R], b_dt [I], a_log [I, S], d_skip [I], state [slots, I, S] 32-bit.
    Returns (scan + d_skip * x) * silu(z) in x's dtype."""
    _cuda(x, w_dt, b_dt, a_log, d_skip, state)
    N, I = x.shape
    S, R = a_log.shape[1], int(dt_rank)
    pp, ps = _rows_view(proj)
    zp, zs = _rows_view(z)
    if proj.shape[1] < R + 2 * S or w_dt.dtype != x.dtype or proj.dtype != x.dtype or z.dtype != x.dtype:
        raise KernelError("selective_scan: operands do not fit together")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (I, S):
        raise KernelError("the scan state is 32-bit [slots, inner, state]")
    y = torch.empty((N, I), dtype=x.dtype, device=x.device)
    chunk, max_chunks = _scan_chunks(step, N, -(-I // (128 if S <= 16 else 64)))
    ends = torch.empty((max_chunks, I, S), dtype=torch.float32, device=x.device) if chunk else None
    sums = torch.empty((max_chunks, I), dtype=torch.float32, device=x.device) if chunk else None
    # the step sizes' products dt_in . w_dt^T for all rows as one matrix product with a 32-bit result; a step of
    # single tokens sums them inside its kernel (a launch less a layer, and the weights are read once either way)
    single = bool(step.decode_only and N == step.n_seqs)
    dt_raw = None if single else linear(proj[:, :R], w_dt, out_dtype=torch.float32)
    _check(_fn("selective_scan", "zai_selective_scan")(
        _ptr(y), _ptr(x), pp, ps, zp, zs, _dt(x), _ptr(dt_raw), _ptr(w_dt), _ptr(b_dt), _ptr(a_log), _ptr(d_skip), _ptr(state),
        _ptr(step.cu_q), _ptr(step.slot_ids), N, step.n_seqs, I, S, R, int(bool(write_state)), state.shape[0],
        _status_ptr(x.device), _ptr(ends), _ptr(sums), chunk, max_chunks, int(bool(step.decode_only)), _stream()),
        "selective_scan", 3 if chunk else 1)
    return y


@_timed("recurrence")
def min_gru(zxg, b_z, b_x, state, step, write_state=True):
    """The minimal gated recurrence over zxg [N, 3W] = (gate | candidate | output gate) with the state [slots, W]
    in 32-bit; returns state * silu(output gate) per row, [N, W]."""
    _cuda(b_z, b_x, state)
    p, stride = _rows_view(zxg)
    N, W = zxg.shape[0], zxg.shape[1] // 3
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (W,):
        raise KernelError("the recurrence's state is 32-bit [slots, width]")
    out = torch.empty((N, W), dtype=zxg.dtype, device=zxg.device)
    chunk, max_chunks = _scan_chunks(step, N, -(-W // 128))
    ends = torch.empty((2, max_chunks, W), dtype=torch.float32, device=zxg.device) if chunk else None
    _check(_fn("min_gru", "zai_min_gru")(_ptr(out), p, stride, _dt(zxg), _ptr(b_z), _ptr(b_x), _ptr(state), _ptr(step.cu_q),
                                         _ptr(step.slot_ids), N, step.n_seqs, W, int(bool(write_state)), state.shape[0],
                                         _status_ptr(zxg.device), _ptr(ends), _ptr(ends[1]) if chunk else None, chunk, max_chunks,
                                         _stream()), "min_gru", 3 if chunk else 1)
    return out


@_timed("recurrence")
def gated_delta(qkv, b, a, gate, a_log, dt_bias, norm_w, eps, state, step, heads, kv_heads, dim, vdim, write_state=True,
                unit_eps=1e-6, channel_decay=False, gate_act="silu"):
    """The gated delta rule over the rows of a step.  qkv [N, 2 G D + H V] (q heads, k heads, v heads, after their
    convolutions), b [N, H], a [N, H] (with `channel_decay` [N, H D]: a decay per head and key channel, `dt_bias` as wide),
    gate [N, H V] (column slices are fine), state [slots, H, D, V] 32-bit.
    Returns rms(o) * norm_w * act(gate) per head (`gate_act`: silu or sigmoid), [N, H V] in qkv's dtype."""
    _cuda(a_log, dt_bias, norm_w, state)
    N = qkv.shape[0]
    H, G, D, V = int(heads), int(kv_heads), int(dim), int(vdim)
    qp, qs = _rows_view(qkv)
    bp, bs = _rows_view(b)
    ap, as_ = _rows_view(a)
    gp, gs = _rows_view(gate)
    ch, act = int(bool(channel_decay)), {"silu": 0, "sigmoid": 1}[gate_act]
    if (state.dtype != torch.float32 or tuple(state.shape[1:]) != (H, D, V) or a.shape[1] != (H * D if ch else H)
            or dt_bias.numel() != a.shape[1] or b.shape[1] != H):
        raise KernelError("gated_delta: operands do not fit together")
    dev = qkv.device
    lib = "gated_delta"
    if step.decode_only and N == step.n_seqs and N <= DELTA_SINGLE_MAX_ROWS and _fn(lib, "zai_gated_delta_single_supports")(D, V):
        # every request brings one token: norms, gates, the state's update and read-out and the output norm in one kernel
        # (few requests: the step is a chain of launches and two fewer count; with many the states' bytes count and the
        # three kernels stream them as fast, measured within the spread between runs at 64 requests)
        out = torch.empty((N, H * V), dtype=qkv.dtype, device=dev)
        _check(_fn(lib, "zai_gated_delta_single")(
            _ptr(out), qp, qs, bp, bs, ap, as_, gp, gs, _dt(qkv), _ptr(a_log), _ptr(dt_bias), _ptr(norm_w), float(eps),
            float(unit_eps), _ptr(state), _ptr(step.slot_ids), N, H, G, D, V, int(bool(write_state)), state.shape[0],
            _status_ptr(dev), ch, act, _stream()), "gated_delta_single")
        return out
    qk = torch.empty((N, 2, G, D), dtype=torch.float32, device=dev)
    bg = torch.empty((N, 2, H), dtype=torch.float32, device=dev)
    gch = torch.empty((N, H, D), dtype=torch.float32, device=dev) if ch else None
    o = torch.empty((N, H * V), dtype=torch.float32, device=dev)
    out = torch.empty((N, H * V), dtype=qkv.dtype, device=dev)
    _check(_fn(lib, "zai_delta_prepare")(_ptr(qk), _ptr(bg), _ptr(gch), qp, qs, bp, bs, ap, as_, _dt(qkv), _ptr(a_log), _ptr(dt_bias),
                                         N, H, G, D, float(unit_eps), _stream()), "delta_prepare")
    vp = qp + 2 * G * D * qkv.element_size()
    _check(_fn(lib, "zai_gated_delta")(_ptr(o), _ptr(qk), _ptr(bg), _ptr(gch), vp, qs, _dt(qkv), _ptr(state), _ptr(step.cu_q),
                                       _ptr(step.slot_ids), N, step.n_seqs, H, G, D, V, int(bool(write_state)), state.shape[0],
                                       _status_ptr(dev), _stream()), "gated_delta")
    _check(_fn(lib, "zai_gated_rmsnorm")(_ptr(out), _ptr(o), _ptr(norm_w), gp, gs, _dt(qkv), float(eps), N, H, V, act, _stream()),
           "gated_rmsnorm")
    return out


@_timed("q/k norm, rotation, page write")
def value_norm_pad(qkv, heads, kv_heads, dim, vdim, eps, normed=True):
    """Prepares projection rows [N, H D + G D + G Dv] for the attention kernels: value heads divided by their root
    mean square over Dv (no weight) if `normed`, and, where D != Dv, every head filled with zeros up to max(D, Dv).
    Works in place where no head changes its size."""
    _cuda(qkv)
    N = qkv.shape[0]
    H, G, D, Dv = int(heads), int(kv_heads), int(dim), int(vdim)
    if qkv.shape[1] != H * D + G * D + G * Dv:
        raise KernelError("value_norm_pad: the rows do not hold q, k and v heads of these sizes")
    if D == Dv:
        if not normed:
            return qkv
        out = qkv
    else:
        out = torch.empty((N, (H + 2 * G) * max(D, Dv)), dtype=qkv.dtype, device=qkv.device)
    _check(_fn("rope_kv", "zai_value_norm_pad")(_ptr(out), _ptr(qkv), qkv.shape[1], _dt(qkv), N, H, G, D, Dv, float(eps),
                                                int(bool(normed)), _stream()), "value_norm_pad")
    return out


# ----------------------------------------------------------------------------- layer norm, prepared projections, latent attention
@_timed("norm")
def add_layernorm(h, delta, w, b, eps, out_dtype):
    """h += delta (in place, 32-bit), then the layer norm of h with weight w and bias b."""
    _cuda(h, delta, w, b)
    if h.dtype != torch.float32 or w.dtype != torch.float32 or b.dtype != torch.float32:
        raise KernelError("the residual stream and norm weights are 32-bit")
    N, H = h.shape
    out = torch.empty((N, H), dtype=out_dtype, device=h.device)
    if delta is not None and delta.dtype != out_dtype:
        raise KernelError("the pending term should have the model's dtype")
    _check(_fn("layernorm", "zai_add_layernorm")(_ptr(h), _ptr(delta), _ptr(w), _ptr(b), _ptr(out), _dt(out), float(eps), N, H,
                                                 _stream()), "add_layernorm")
    return out


@_timed("q/k norm, rotation, page write")
def qkv_prepare(y, q_w, k_w, eps, scope, table, rot, step, cache, heads, kv_heads, dim, vdim, cache_dim, write=True, temp=None,
                v_first=None, v_lambda=None):
    """From projection rows y = [q (H D) | k (G D) | v (G Dv) | ...]: the RMS norm of q and k (`scope` 0 none, 1 per head,
    2 over the whole projection), the rotation of pairs (i, i + rot/2) from `table`, k and v into the pages (heads
    `cache_dim` wide, zeros behind their own values); returns q [N, H * cache_dim].  `temp` = (coef, every): the queries times
    1 + coef ln(floor((position + 1) / every) + 1).  `v_first` [N, G * Dv] (a column slice is fine) with `v_lambda` (one 32-bit
    number on the device): the values cached are (1 - lambda) v + lambda v_first."""
    _cuda(q_w, k_w, table, v_lambda)
    fp, fs = (None, 0) if v_first is None else _rows_view(v_first)
    if v_first is not None and (v_first.dtype != y.dtype or v_first.shape != (y.shape[0], int(kv_heads) * int(vdim))
                                or v_lambda is None or v_lambda.dtype != torch.float32):
        raise KernelError("qkv_prepare: the first values do not fit this layer's")
    yp, ys = _rows_view(y)
    N = y.shape[0]
    H, G, D, Dv, Dp = int(heads), int(kv_heads), int(dim), int(vdim), int(cache_dim)
    if y.shape[1] < (H + G) * D + G * Dv:
        raise KernelError("qkv_prepare: the rows do not hold q, k and v heads of these sizes")
    pages, bt = cache.pages, cache.block_table
    if pages.dtype != y.dtype or tuple(pages.shape[1:]) != (2, G, cache.page_size, Dp):
        raise KernelError("the pages should have the activations' dtype and heads of the cache's size")
    q = torch.empty((N, H * Dp), dtype=y.dtype, device=y.device)
    _check(_fn("qkv_prepare", "zai_qkv_prepare")(
        yp, ys, _dt(y), _ptr(q_w), _ptr(k_w), float(eps), int(scope), _ptr(table), int(rot), _ptr(step.positions), _ptr(step.seq_idx),
        _ptr(bt), bt.shape[1], _ptr(pages), cache.page_size, _ptr(q), N, H, G, D, Dv, Dp, int(bool(write)), pages.shape[0],
        _status_ptr(y.device), float(temp[0]) if temp else 0.0, int(temp[1]) if temp else 0, fp, fs, _ptr(v_lambda) if fp else None,
        _stream()), "qkv_prepare")
    return q


@_timed("activation")
def sigmoid_gate(o, gate, heads, head_dim, per_head):
    """o [N, heads * head_dim] times sigmoid(gate): gate [N, heads] (one number per head) or [N, heads * head_dim]; a
    column slice is fine for the gate."""
    _cuda(o)
    gp, gs = _rows_view(gate)
    N = o.shape[0]
    if gate.dtype != o.dtype or o.shape[1] != heads * head_dim or gate.shape[1] != (heads if per_head else heads * head_dim):
        raise KernelError("sigmoid_gate: operands do not fit together")
    out = torch.empty_like(o)
    _check(_fn("qkv_prepare", "zai_sigmoid_gate")(_ptr(out), _ptr(o), heads * head_dim, head_dim, gp, gs, _dt(o), int(bool(per_head)),
                                                  N, int(heads), int(head_dim), _stream()), "sigmoid_gate")
    return out


@_timed("products")
def head_linear(x, w):
    """x [N, H, K] (a strided view is fine) times w [H, O, K] per head -> [N, H, O]: the library's batched product,
    true 32-bit where the operands are."""
    if x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        torch.backends.cuda.matmul.allow_tf32 = False
    N, H, _ = x.shape
    out = torch.empty((N, H, w.shape[1]), dtype=x.dtype, device=x.device)
    torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))
    return out


@_timed("q/k norm, rotation, page write")
def latent_prepare(q, dkv, norm_w, eps, table, step, cache, heads, dim, rot_dim, rank):
    """The rotated parts of the queries q [N, H, dim + rot_dim] -> [N, H, rot_dim]; if `dkv` [N, rank + rot_dim] (a column
    slice is fine) is given, the normed latent and the rotated shared key part of every row go into the request's pages."""
    _cuda(norm_w, table)
    N = q.shape[0]
    H, D, Dr, R = int(heads), int(dim), int(rot_dim), int(rank)
    if q.dim() != 3 or q.stride(2) != 1 or q.stride(1) != D + Dr or tuple(q.shape[1:]) != (H, D + Dr):
        raise KernelError("latent_prepare: q is [N, heads, dim + rot_dim] with contiguous rows")
    q_rot = torch.empty((N, H, Dr), dtype=q.dtype, device=q.device)
    dp, ds = (None, 0) if dkv is None else _rows_view(dkv)
    pages, bt = cache.pages, cache.block_table
    if dkv is not None and (pages.dtype != q.dtype or tuple(pages.shape[1:]) != (cache.page_size, R + Dr)):
        raise KernelError("the pages should have the activations' dtype and rows of rank + rot_dim values")
    _check(_fn("qkv_prepare", "zai_latent_prepare")(
        q.data_ptr(), q.stride(0), dp, ds, _dt(q), _ptr(norm_w), float(eps), _ptr(table), _ptr(step.positions), _ptr(step.seq_idx),
        _ptr(bt), bt.shape[1], _ptr(pages), cache.page_size, _ptr(q_rot), N, H, D, Dr, R, pages.shape[0], _status_ptr(q.device),
        _stream()), "latent_prepare")
    return q_rot


LATENT_SPLIT_KEYS = 256          # keys per range where a step's rows are too few to fill the device
LATENT_WARPS_WANTED = 1024       # from this many warps (rows x groups of 16 heads x blocks of output columns) on, no ranges
USE_LATENT_MMA = os.environ.get("ZAI_LATENT_MMA", "1") == "1"


@_timed("attention")
def latent_attention(q_lat, q_rot, step, cache, heads, rank, rot_dim, scale, impl=None, sink=None):
    """Causal attention of every head against the cached rows [latent | rotated key part]: scores
    (q_lat . latent + q_rot . key part) * scale, output sum_j p_j latent_j, [N, H, rank].  bfloat16 with a rank
    that is a multiple of 32 and rank + rot_dim a multiple of 16 runs on the tensor cores (steps of many rows: the four
    warps of a block share the tiles of cached rows; steps of few rows: a warp a row and range of keys, the ranges added
    up by a second kernel); everything else, and `impl="general"`, runs the general kernel.  `sink` [H] 32-bit: one more
    term exp(sink_h) in every row's denominator (no key, no value, not scaled)."""
    _cuda(q_lat, q_rot, sink)
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != int(heads)):
        raise KernelError("latent_attention: the sink is one 32-bit number per head")
    N = q_lat.shape[0]
    H, R, Dr = int(heads), int(rank), int(rot_dim)
    pages, bt = cache.pages, cache.block_table
    if N != step.n_tokens or pages.dtype != q_lat.dtype or tuple(pages.shape[1:]) != (cache.page_size, R + Dr):
        raise KernelError("latent_attention: operands do not fit together")
    out = torch.empty((N, H, R), dtype=q_lat.dtype, device=q_lat.device)
    if (impl != "general" and (USE_LATENT_MMA or impl in ("mma", "mma_rows", "mma_ranges")) and q_lat.dtype == torch.bfloat16
            and _fn("latent_attention", "zai_latent_attention_mma_supports")(R, Dr)):
        warps = N * (-(-H // 16)) * (-(-R // (128 if R <= 128 else 256)))
        n_splits = 1 if warps >= LATENT_WARPS_WANTED else max(-(-int(step.max_kv_len) // LATENT_SPLIT_KEYS), 1)
        if impl in ("mma_rows", "mma_ranges"):               # (tests pick the kernel whatever the step's size)
            n_splits = 1 if impl == "mma_rows" else max(-(-int(step.max_kv_len) // LATENT_SPLIT_KEYS), 1)
        split_keys = LATENT_SPLIT_KEYS if n_splits > 1 else 1 << 30           # one range: all keys
        part_o = part_ml = None
        if n_splits > 1:
            part_o = torch.empty((N, H, n_splits, R), dtype=torch.float32, device=q_lat.device)
            part_ml = torch.empty((N, H, n_splits, 2), dtype=torch.float32, device=q_lat.device)
        _check(_fn("latent_attention", "zai_latent_attention_mma")(
            _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(q_lat), _ptr(q_rot), _ptr(pages), _ptr(bt), bt.shape[1],
            _ptr(step.positions), _ptr(step.seq_idx), cache.page_size, N, H, R, Dr, float(scale), split_keys, n_splits,
            pages.shape[0], _status_ptr(q_lat.device), _ptr(sink), _stream()), "latent_attention_mma", 2 if n_splits > 1 else 1)
        return out
    _check(_fn("latent_attention", "zai_latent_attention")(
        _ptr(out), _ptr(q_lat), _ptr(q_rot), _ptr(pages), _dt(q_lat), _ptr(bt), bt.shape[1], _ptr(step.positions), _ptr(step.seq_idx),
        cache.page_size, N, H, R, Dr, float(scale), pages.shape[0], _status_ptr(q_lat.device), _ptr(sink), _stream()),
        "latent_attention")
    return out


@_timed("activation")
def clamped_glu(gu, ff_dim, limit, alpha):
    """min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + 1) on the stacked gate|up rows."""
    _cuda(gu)
    N = gu.shape[0]
    out = torch.empty((N, ff_dim), dtype=gu.dtype, device=gu.device)
    _check(_fn("activation", "zai_clamped_glu")(_ptr(out), _ptr(gu), _dt(gu), N, int(ff_dim), float(limit), float(alpha), _stream()),
           "clamped_glu")
    return out


def linear_clamped_glu(x, w_gate_up, ff_dim, limit, alpha):
    """The stacked gate|up product (x may be a LazyNorm) and the bounded gated activation: for few rows in bfloat16 the
    activation is the product kernel's epilogue, else a kernel of its own behind the product."""
    if x.dtype == torch.bfloat16:
        y = _skinny(x, w_gate_up, _EPI_SWIGLU, ff_dim, torch.bfloat16, glu=(limit, alpha))
        if y is not None:
            return y
    return clamped_glu(linear(x, w_gate_up), ff_dim, limit, alpha)


@_timed("head")
def scale_softcap(logits, scale, cap):
    """In place on 32-bit logits: times `scale`, then cap * tanh(logits / cap) if a cap is given."""
    _cuda(logits)
    if logits.dtype != torch.float32:
        raise KernelError("logits are 32-bit")
    _check(_fn("activation", "zai_scale_softcap")(_ptr(logits), logits.numel(), float(scale), float(cap or 0.0), _stream()),
           "scale_softcap")
    return logits


# ----------------------------------------------------------------------------- norm of activation rows, routed experts
@_timed("norm")
def rmsnorm_rows(x, w, eps):
    """RMS norm of activation rows x [N, C] (a column slice is fine) with the 32-bit weight w (or None), computed in
    32-bit, in x's dtype."""
    _cuda(w)
    xp, xs = _rows_view(x)
    N, C = x.shape
    if w is not None and (w.dtype != torch.float32 or w.numel() != C):
        raise KernelError("rmsnorm_rows: the weight is 32-bit, one value a column")
    out = torch.empty((N, C), dtype=x.dtype, device=x.device)
    _check(_fn("norm", "zai_rmsnorm_rows")(_ptr(out), xp, xs, _dt(x), _ptr(w), float(eps), N, C, _stream()), "rmsnorm_rows")
    return out


USE_MOE_GROUPED_TC = os.environ.get("ZAI_MOE_GROUPED_TC", "1") == "1"
USE_MOE_DOWN_PAIR = os.environ.get("ZAI_MOE_DOWN_PAIR", "1") == "1"      # the down product: two weight tiles a stage
MOE_GROUPED_TILE_ROWS = 64   # from this many rows per expert on average, tiles of 128 rows on the tcgen05 kernel (bfloat16)
MOE_TALL_TILE_ROWS = 32      # from this many rows per expert on average, tiles of 64 rows instead of 16 (bfloat16)


@_timed("experts")
def routed_experts(x, w_router, w_gate_up, w_down, top, renorm=False, weight_on="input", score="sigmoid", act="silu", limit=0.0,
                   alpha=1.702):
    """A mixture of gated feed-forwards.  x [N, W]; w_router [E, W] 32-bit; w_gate_up [E, 2 F, W] (an expert's gate rows,
    then its up rows); w_down [E, W, F].  Every row goes to the `top` experts with the largest sigmoid(x . w_router^T)
    (32-bit); the scores are the weights (divided by their sum with `renorm`), applied to the expert's input or to its
    output; the row's results are summed in 32-bit.  Nothing is read back to the host.  `score="softmax"`: the scores are the
    softmax of the router's logits over all experts (`renorm` divides by the chosen scores' sum + 1e-20).  `act="clamped"`:
    the experts are bounded gated units min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u, -limit, limit) + 1)."""
    if score not in ("sigmoid", "softmax") or act not in ("silu", "clamped"):
        raise KernelError("routed_experts: score is sigmoid or softmax, act silu or clamped")
    gated = 2 if act == "clamped" else 1
    _cuda(w_router, w_gate_up, w_down)
    xp, xs = _rows_view(x)
    N, W = x.shape
    E, F = w_gate_up.shape[0], w_gate_up.shape[1] // 2
    top = int(top)
    if (w_router.dtype != torch.float32 or tuple(w_router.shape) != (E, W) or tuple(w_gate_up.shape) != (E, 2 * F, W)
            or tuple(w_down.shape) != (E, W, F) or w_gate_up.dtype != x.dtype or w_down.dtype != x.dtype
            or weight_on not in ("input", "output")):
        raise KernelError("routed_experts: operands do not fit together")
    dev, dt, lib = x.device, _dt(x), "moe"
    out = torch.empty((N, W), dtype=x.dtype, device=dev)
    if N == 0:
        return out
    tall = dt == _BF16 and W % 8 == 0 and F % 8 == 0 and N * top >= MOE_TALL_TILE_ROWS * E
    # many rows an expert: tiles of 128 rows and both products on the 5th-generation tensor cores (grouped tcgen05)
    grouped = (tall and USE_MOE_GROUPED_TC and N * top >= MOE_GROUPED_TILE_ROWS * E
               and _fn("gemm_tc", "zai_gemm_tc_supports")(128, 2 * F, W, _EPI_SWIGLU if act == "silu" else _EPI_BF16)
               and _fn("gemm_tc", "zai_gemm_tc_supports")(128, W, F, _EPI_F32))
    TM = 128 if grouped else 64 if tall else 16
    max_tiles = _fn(lib, "zai_moe_max_tiles")(N, top, E, TM)
    if max_tiles < 0:
        raise KernelError("routed_experts: too many rows")
    meta = torch.empty((4 * N * top + E + max_tiles,), dtype=torch.int32, device=dev)
    ids, rank, dest = meta[:N * top], meta[N * top:2 * N * top], meta[2 * N * top:3 * N * top]
    wts = meta[3 * N * top:4 * N * top].view(torch.float32)
    counts, tile_expert = meta[4 * N * top:4 * N * top + E], meta[4 * N * top + E:]
    on_input = int(weight_on == "input")
    _check(_fn(lib, "zai_moe_route")(_ptr(ids), _ptr(wts), _ptr(rank), _ptr(counts), xp, xs, dt, _ptr(w_router), N, W, E, top,
                                     int(bool(renorm)), int(score == "softmax"), _stream()), "moe_route")
    rows = max_tiles * TM
    x_sorted = torch.empty((rows, W), dtype=x.dtype, device=dev)
    _check(_fn(lib, "zai_moe_gather")(_ptr(x_sorted), _ptr(dest), _ptr(tile_expert), xp, xs, dt, _ptr(ids), _ptr(wts), _ptr(rank),
                                      _ptr(counts), N, W, E, top, TM, max_tiles, on_input, _stream()), "moe_gather")
    hidden = torch.empty((rows, F), dtype=x.dtype, device=dev)
    y = torch.empty((rows, W), dtype=torch.float32, device=dev)
    if grouped:
        tc = _fn("gemm_tc", "zai_gemm_tc_grouped")
        if gated == 2:        # the plain grouped product, then the bounded activation on its gate|up rows
            gu = torch.empty((rows, 2 * F), dtype=x.dtype, device=dev)
            _check(tc(_ptr(gu), _ptr(w_gate_up), _ptr(x_sorted), _ptr(tile_expert), _status_ptr(dev), max_tiles, E, 2 * F, W,
                      _EPI_BF16, _stream()), "gemm_tc_grouped (gate/up)")
            hidden = clamped_glu(gu, F, limit, alpha)
        else:
            _check(tc(_ptr(hidden), _ptr(w_gate_up), _ptr(x_sorted), _ptr(tile_expert), _status_ptr(dev), max_tiles, E, 2 * F, W,
                      _EPI_SWIGLU, _stream()), "gemm_tc_grouped (gate/up)")
        _check(tc(_ptr(y), _ptr(w_down), _ptr(hidden), _ptr(tile_expert), _status_ptr(dev), max_tiles, E, W, F,
                  _EPI_F32_PAIR if USE_MOE_DOWN_PAIR else _EPI_F32, _stream()),
               "gemm_tc_grouped (down)")
        _check(_fn(lib, "zai_moe_combine")(_ptr(out), dt, _ptr(y), _ptr(dest), _ptr(wts), N, W, top, 1 - on_input, _stream()),
               "moe_combine")
        return out
    _check(_fn(lib, "zai_moe_gemm")(_ptr(hidden), int(dt == _F32), _ptr(x_sorted), _ptr(w_gate_up), dt, _ptr(tile_expert), max_tiles,
                                    TM, W, F, gated, float(limit), float(alpha), _stream()), "moe_gemm (gate/up)")
    _check(_fn(lib, "zai_moe_gemm")(_ptr(y), 1, _ptr(hidden), _ptr(w_down), dt, _ptr(tile_expert), max_tiles, TM, F, W, 0, 0.0, 0.0,
                                    _stream()), "moe_gemm (down)")
    _check(_fn(lib, "zai_moe_combine")(_ptr(out), dt, _ptr(y), _ptr(dest), _ptr(wts), N, W, top, 1 - on_input, _stream()),
           "moe_combine")
    return out


# ----------------------------------------------------------------------------- gated feed-forward with any activation, mLSTM
_ACT_KINDS = {"gelu": 0, "gelu_erf": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}


@_timed("activation")
def act_mul(gu, ff_dim, kind):
    """act(gate) * up on the stacked gate|up rows; `kind` as in `activation`."""
    _cuda(gu)
    if kind not in _ACT_KINDS:
        raise KernelError(f"unknown activation '{kind}'")
    N = gu.shape[0]
    out = torch.empty((N, ff_dim), dtype=gu.dtype, device=gu.device)
    _check(_fn("activation", "zai_act_mul")(_ptr(out), _ptr(gu), _dt(gu), N, int(ff_dim), _ACT_KINDS[kind], _stream()), "act_mul")
    return out


def linear_glu(x, w_gate_up, ff_dim, kind):
    """The stacked gate|up product (x may be a LazyNorm) and act(gate) * up; SiLU takes the fused ways of `linear_swiglu`."""
    if kind == "silu":
        return linear_swiglu(x, w_gate_up, ff_dim)
    if kind == "gelu_tanh" and x.dtype == torch.bfloat16:
        y = _skinny(x, w_gate_up, _EPI_SWIGLU, ff_dim, torch.bfloat16, glu=(-1.0, 0.0))     # few rows: the product's epilogue
        if y is not None:
            return y
    return act_mul(linear(x, w_gate_up), ff_dim, kind)


@_timed("recurrence")
def mlstm(y, at, bias_i, bias_f, cap, norm_w, eps, state, step, heads, dim, vdim, write_state=True):
    """The matrix memory with log gates.  y [N, cols]: the stacked projections, `at` the first columns of q (H D), k (H D), v (H
    Dv), the output gate (H Dv) and the inputs of the log input and forget gates (H each); bias_i, bias_f [H], norm_w [H Dv]
    32-bit; state [slots, H, D + 1, Dv + 1] 32-bit (the normaliser as the last column, every column's running maximum as
    the last row).  Returns rms_per_head(o) * norm_w * sigmoid(gate), [N, H Dv]."""
    _cuda(bias_i, bias_f, norm_w, state)
    yp, ys = _rows_view(y)
    N, H, D, Dv = y.shape[0], int(heads), int(dim), int(vdim)
    if (state.dtype != torch.float32 or tuple(state.shape[1:]) != (H, D + 1, Dv + 1) or bias_i.dtype != torch.float32
            or bias_f.dtype != torch.float32 or norm_w.dtype != torch.float32 or norm_w.numel() != H * Dv or N != step.n_tokens):
        raise KernelError("mlstm: operands do not fit together")
    out = torch.empty((N, H * Dv), dtype=y.dtype, device=y.device)
    part = torch.empty((N, H, Dv + 2), dtype=torch.float32, device=y.device)
    q_at, k_at, v_at, g_at, i_at, f_at = (int(a) for a in at)
    _check(_fn("mlstm", "zai_mlstm")(_ptr(out), _ptr(part), yp, ys, _dt(y), q_at, k_at, v_at, g_at, i_at, f_at, _ptr(bias_i),
                                     _ptr(bias_f), float(cap), _ptr(norm_w), float(eps), _ptr(state), _ptr(step.cu_q),
                                     _ptr(step.slot_ids), state.shape[0], _status_ptr(y.device), N, step.n_seqs, H, D, Dv,
                                     int(bool(write_state)), _stream()), "mlstm", 2)
    return out
