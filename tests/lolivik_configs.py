"""Small configurations of the Lolivik design for the tests.  Between them they differ in every size and option: layer order
and count, each mixer in front of each feed-forward and of none, one key/value head for many query heads and as many as
there are, key sizes larger and smaller than value sizes, bias tables of few and many rows, windows smaller and larger
than a page with none, few and many kept first positions, rotations of a part of a head and of all of it with and
without stretched frequencies, one expert a token, several and all, experts with and without a shared unit, a residual
factor of 1 and others, the first mixing layer of either attention kind, widths that are no multiple of four."""


def attention(heads, kv_heads, dim, vdim, scale, softcap, bias_rows, bias_max, coef, every, v_mix=True, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap, "bias_rows": bias_rows,
         "bias_max": bias_max, "q_temp": {"coef": coef, "every": every}, "v_mix": v_mix}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def windowed(heads, kv_heads, dim, vdim, scale, size, keep_first, base, dims, scaling=None, v_mix=True, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size, "keep_first": keep_first},
         "rot": {"base": base, "dims": dims, "scaling": scaling}, "v_mix": v_mix}
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def memory(heads, dim, vdim, cap, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top, shared=None):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top},
            "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


def stretch(factor, low, high, original):
    return {"factor": factor, "low": low, "high": high, "original": original}


def config(vocab, width, eps, mult, layers):
    return {"architecture": "Lolivik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}


L_A = config(131, 48, 1e-5, 0.5, [
    windowed(4, 2, 12, 6, 0.3, 11, 3, 10000.0, 8, stretch(4.0, 1.0, 3.0, 40), mlp=moe(20, 1.5, 5, 2, shared=(28, 2.5))),
    memory(3, 8, 12, 10.0, mlp=dense(72)),
    attention(4, 2, 10, 6, 0.25, 12.0, 10, 60, 0.4, 16, mlp=moe(24, 3.0, 4, 4)),
    memory(2, 12, 6, 6.0),
    attention(6, 1, 8, 12, 0.3, 30.0, 7, 25, 0.2, 5, mlp=dense(40)),
])

L_B = config(257, 66, 1e-6, 1.0, [
    memory(2, 16, 8, 20.0, mlp=moe(32, 2.0, 3, 1, shared=(16, 1.0))),
    attention(3, 3, 16, 20, 0.2, 8.0, 16, 100, 0.3, 32, mlp=dense(100)),
    windowed(6, 3, 16, 20, 0.25, 40, 0, 500.0, 16, None, mlp=moe(40, 2.0, 7, 3)),
    windowed(6, 3, 8, 20, 0.35, 5, 9, 300.0, 4, stretch(8.0, 2.0, 5.0, 64)),
    attention(3, 1, 24, 60, 0.15, 50.0, 4, 9, 0.0, 1, v_mix=False, mlp=moe(16, 4.0, 2, 2, shared=(40, 2.0))),
])

# one layer of each kind, alone: a fault shows in the mechanism that has it
ONLY = {
    "attention": config(97, 40, 1e-5, 0.7, [attention(4, 2, 10, 6, 0.3, 15.0, 12, 50, 0.3, 8)]),
    "attention_dense": config(97, 40, 1e-5, 1.0, [attention(2, 2, 12, 12, 0.25, 20.0, 8, 30, 0.5, 4, v_mix=False, mlp=dense(64))]),
    "windowed": config(97, 40, 1e-5, 0.7, [windowed(4, 1, 12, 8, 0.3, 9, 2, 10000.0, 6, stretch(4.0, 1.0, 2.0, 32))]),
    "windowed_plain": config(97, 40, 1e-5, 0.3, [windowed(3, 3, 8, 16, 0.35, 20, 0, 100.0, 8, None, v_mix=False)]),
    "memory": config(97, 40, 1e-5, 0.7, [memory(3, 10, 14, 14.0)]),
    "memory_experts": config(97, 40, 1e-5, 1.0, [memory(2, 6, 10, 8.0, mlp=moe(24, 2.0, 6, 2, shared=(12, 2.0)))]),
    "experts_one_of_many": config(97, 40, 1e-5, 1.0, [memory(2, 8, 8, 12.0, mlp=moe(12, 1.0, 9, 1))]),
    "mixed_values": config(97, 40, 1e-5, 0.6, [windowed(2, 2, 8, 10, 0.3, 12, 1, 1000.0, 8, None),
                                              attention(4, 2, 6, 10, 0.3, 25.0, 6, 20, 0.1, 3),
                                              windowed(5, 1, 10, 20, 0.2, 7, 4, 1000.0, 2, None)]),
    # attention made sharp by its scale: nearly all weight on one key, so a key lost or seen too early shows
    "sharp_windowed": config(97, 40, 1e-5, 1.0, [windowed(3, 1, 10, 14, 2.0, 13, 3, 300.0, 4, None, v_mix=False)]),
    "sharp_attention": config(97, 40, 1e-5, 1.0, [attention(3, 1, 10, 14, 2.0, 40.0, 12, 70, 0.2, 16, v_mix=False)]),
}

# sizes that the tensor-core kernels and the few-rows product kernels take, for the whole-model GPU tests in bfloat16
L_C = config(1000, 320, 1e-6, 0.4, [
    attention(8, 2, 64, 64, 0.125, 25.0, 32, 1000, 0.25, 64, mlp=dense(512)),
    memory(4, 64, 64, 13.0, mlp=moe(128, 2.5, 8, 2, shared=(192, 2.0))),
    windowed(4, 4, 64, 32, 0.125, 100, 4, 10000.0, 32, stretch(6.0, 1.0, 3.0, 256), mlp=moe(64, 3.0, 4, 1)),
    memory(2, 32, 128, 12.0, mlp=dense(448)),
    attention(4, 2, 32, 64, 0.18, 30.0, 16, 300, 0.3, 128, mlp=moe(96, 2.0, 6, 3, shared=(64, 1.5))),
])

ALL = {"A": (L_A, 31), "B": (L_B, 37), "C": (L_C, 41)}
PAGE_SIZE = {"A": 8, "B": 16, "C": 64}
