"""Small configurations of the Zikevik design for the tests.  Between them they differ in every size and option: layer
order and count, either mixer in front of either feed-forward and of none, fewer query/key heads than value heads and
as many, convolutions of two to five taps, inner sizes of the decay and gate projections that differ and that agree,
unrotated parts larger and smaller than the rotated part, a query latent smaller than, equal to and larger than the
key/value latent, one expert a token, several, and all of them, layers that run on an earlier layer's tensors, widths
that are no multiple of four."""


def delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank, mlp=None, weights_of=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank,
         "gate_rank": gate_rank}
    return _layer("channel_delta", m, mlp, weights_of)


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, mlp=None, weights_of=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    return _layer("latent_attention", m, mlp, weights_of)


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(kind, m, mlp, weights_of):
    out = {"type": kind, "mixer": m, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def again(layers, i):
    """A layer that runs on layer i's tensors."""
    return dict(layers[i], weights_of=i)


def config(vocab, width, eps, scale, layers):
    return {"architecture": "Zikevik", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "layers": layers}


def _with_repeats(layers, repeats):
    out = list(layers)
    for i in repeats:
        out.append(again(out, i))
    return out


Z_A = config(131, 48, 1e-5, 0.7, _with_repeats([
    delta(4, 2, 8, 12, 3, 5, 7, mlp=dense(80)),
    latent(3, 12, 8, 20, 24, 16, 0.2, 10000.0, mlp=moe(24, 5, 2)),
    latent(2, 8, 4, 16, 24, 24, 0.35, 500.0),
], [0, 1]))

Z_B = config(257, 66, 1e-6, 1.5, [
    latent(4, 16, 16, 8, 40, 20, 0.25, 500.0, mlp=dense(100)),
    delta(3, 3, 16, 8, 2, 4, 4, mlp=moe(40, 3, 3)),
    delta(2, 1, 12, 20, 5, 9, 3),
    dict(delta(3, 3, 16, 8, 2, 4, 4, mlp=moe(40, 3, 3)), weights_of=1),
    latent(5, 4, 6, 12, 17, 48, 0.3, 300.0, mlp=moe(16, 7, 1)),
])

# one layer of each kind, alone: a fault shows in the mechanism that has it
ONLY = {
    "delta": config(97, 40, 1e-5, 1.0, [delta(4, 2, 8, 12, 3, 6, 5)]),
    "delta_ff": config(97, 40, 1e-5, 0.5, [delta(2, 2, 12, 6, 4, 3, 8, mlp=dense(64))]),
    "delta_one_tap": config(97, 40, 1e-5, 1.0, [delta(3, 1, 10, 10, 1, 4, 4)]),
    "latent": config(97, 40, 1e-5, 1.0, [latent(3, 10, 6, 14, 20, 12, 0.3, 300.0)]),
    "latent_experts": config(97, 40, 1e-5, 2.0, [latent(2, 6, 6, 10, 20, 30, 0.4, 300.0, mlp=moe(24, 6, 2))]),
    "experts_one_of_many": config(97, 40, 1e-5, 1.0, [delta(2, 2, 8, 8, 2, 3, 3, mlp=moe(12, 9, 1))]),
    "twice": config(97, 40, 1e-5, 1.0, _with_repeats([latent(3, 10, 6, 14, 20, 12, 0.3, 300.0, mlp=moe(16, 4, 2)),
                                                      delta(2, 1, 8, 12, 3, 4, 6, mlp=dense(56))], [0, 1, 0])),
    # attention made sharp by its scale: nearly all weight on one key, so a key lost or seen too early shows
    "sharp_latent": config(97, 40, 1e-5, 1.0, [latent(3, 10, 6, 14, 20, 12, 1.5, 300.0)]),
}

# sizes that the tensor-core kernels and the few-rows product kernels take, for the whole-model GPU tests in bfloat16
Z_C = config(1000, 320, 1e-6, 0.8, _with_repeats([
    delta(4, 2, 64, 64, 4, 16, 24, mlp=dense(512)),
    latent(4, 48, 32, 64, 160, 96, 0.1, 10000.0, mlp=moe(128, 8, 2)),
    latent(8, 16, 32, 48, 128, 64, 0.15, 20000.0, mlp=dense(448)),
    delta(2, 2, 32, 128, 3, 8, 8, mlp=moe(64, 4, 1)),
], [1, 0]))

ALL = {"A": (Z_A, 31), "B": (Z_B, 37), "C": (Z_C, 41)}
PAGE_SIZE = {"A": 8, "B": 16, "C": 64}


# ----------------------------------------------------------------------------- configurations drawn at random
import copy  # noqa: E402


def odd_configuration(g):
    """Sizes that are no multiple of eight anywhere: widths, heads, head sizes, ranks, inner sizes, experts."""
    layers = []
    for i in range(g.randint(2, 5)):
        own = [j for j, l in enumerate(layers) if "weights_of" not in l]
        if own and g.random() < 0.2:
            j = g.choice(own); layers.append(dict(copy.deepcopy(layers[j]), weights_of=j)); continue
        r = g.random()
        if r < 0.1: mlp = None
        elif r < 0.45: mlp = dense(g.choice([100, 130, 257, 300]))
        else:
            E = g.choice([1, 3, 5, 7, 12]); mlp = moe(g.choice([20, 52, 100, 132]), E, g.choice([1, min(2, E), E]))
        if g.random() < 0.45:
            heads = g.choice([1, 2, 3, 5, 6]); kv = g.choice([k for k in (1, 2, 3, 5, 6) if heads % k == 0])
            layers.append(delta(heads, kv, g.choice([12, 20, 24, 40, 72]), g.choice([12, 20, 36, 40, 100]), g.choice([1, 2, 3, 5, 7]),
                                g.choice([3, 5, 12, 20]), g.choice([3, 7, 12, 36]), mlp=mlp))
        else:
            layers.append(latent(g.choice([1, 3, 5, 7, 9, 17]), g.choice([4, 12, 20, 24, 40]), g.choice([2, 6, 12, 20, 24]), g.choice([12, 20, 36, 100]),
                                 g.choice([20, 40, 72, 100, 132]), g.choice([20, 36, 72, 100]), g.choice([0.1, 0.2]),
                                 g.choice([10000.0, 1e6]), mlp=mlp))
    return config(g.choice([101, 449, 1001]), g.choice([50, 100, 132, 250, 98]), g.choice([1e-5, 1e-6]), g.choice([0.5, 1.0]), layers)


def medium_configuration(g):
    """Sizes between the tiny test models and a real model's layers, which the tensor-core kernels take in bfloat16."""
    layers = []
    for i in range(g.randint(3, 7)):
        own = [j for j, l in enumerate(layers) if "weights_of" not in l]
        if own and g.random() < 0.2:
            j = g.choice(own); layers.append(dict(copy.deepcopy(layers[j]), weights_of=j)); continue
        r = g.random()
        if r < 0.1: mlp = None
        elif r < 0.45: mlp = dense(g.choice([96, 200, 320, 512, 768]))
        else:
            E = g.choice([2, 4, 6, 8, 16]); mlp = moe(g.choice([48, 64, 96, 136, 256]), E, g.choice([1, 2, min(4, E)]))
        if g.random() < 0.45:
            heads = g.choice([1, 2, 3, 4, 6, 8]); kv = g.choice([k for k in (1, 2, 3, 4, 6, 8) if heads % k == 0])
            layers.append(delta(heads, kv, g.choice([16, 32, 48, 64, 128]), g.choice([16, 32, 64, 96, 128]), g.choice([2, 3, 4, 5]),
                                g.choice([8, 16, 24, 40]), g.choice([8, 16, 32, 48]), mlp=mlp))
        else:
            layers.append(latent(g.choice([2, 3, 4, 6, 8, 16]), g.choice([16, 32, 48, 64]), g.choice([8, 16, 32, 64]), g.choice([16, 32, 48, 64, 128]),
                                 g.choice([32, 48, 64, 96, 128, 256]), g.choice([48, 64, 96, 128, 192]), g.choice([0.08, 0.125, 0.2]),
                                 g.choice([10000.0, 20000.0, 5e5]), mlp=mlp))
    return config(g.choice([257, 500, 1000, 2048]), g.choice([96, 128, 160, 200, 256, 320, 384]), g.choice([1e-5, 1e-6]), g.choice([0.5, 1.0, 2.0]), layers)
