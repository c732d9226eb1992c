"""The Zikevik design through the engine's host logic on the CPU: the step function, the cache (pages of latent rows,
slots of recurrent state, a layer that runs on another layer's tensors with a cache and state of its own) and the batch
description run with the plain PyTorch kernels of tests/ref_ops.py in place of the CUDA kernels and are compared with
the plain whole-sequence implementation (tests/plain_zikevik.py): each mechanism alone, whole prompts, token-by-token
decoding, portions down to two tokens, batches of unequal requests in a pool so small that pages and slots are used
again, far rows and page borders with attention made sharp, a sink made large, a state that keeps a far token, decays
that differ from channel to channel, the router's weight on the experts' input, the first tokens of a request, long
decoding, and greedy generation through the entry point."""
import copy
import json
import os
import random

import pytest
import torch

import plain_zikevik as P
import ref_ops
from zikevik_configs import ALL, ONLY, PAGE_SIZE, config, delta, dense, latent, moe
from zig_ai_b200.config import ConfigError, config_from_dict
from zig_ai_b200.engine import Engine
from zig_ai_b200.engine.runner import load_runner
from zig_ai_b200.weights import write_random_model
from zig_ai_b200.weights.safetensors_io import SafetensorsFile, write_safetensors

ATOL = 3e-4          # float32 on the CPU against float64, logits of size one to ten


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("zikevik")
    out = {}
    for name, (cfg, seed) in list(ALL.items())[:2] + [(k, (c, 5)) for k, c in ONLY.items()]:
        d = str(root / name)
        write_random_model(config_from_dict(cfg), seed, d, matrix_std="fan_in")
        out[name] = d
    return out


def plain(model_dir, tokens, cfg=None, weights=None):
    return P.forward(cfg or P.read_config(model_dir), weights or P.read_weights(model_dir), tokens)


def runner(model_dir, page_size=8, max_tokens=512, max_requests=4):
    return load_runner(model_dir, "float32", max_tokens=max_tokens, max_requests=max_requests, page_size=page_size,
                       device="cpu", ops=ref_ops)


def tokens(vocab, n, seed):
    g = random.Random(seed)
    return [g.randrange(vocab) for _ in range(n)]


def close(got, want, what="", atol=ATOL):
    err = (got.double() - want).abs().max()
    assert err < atol, f"{what}: off by {float(err):.3e}"


def run_cut(r, rid, toks, cuts):
    r.add_request(rid)
    got, at = [], 0
    for n in cuts:
        got.append(r.step([(rid, toks[at:at + n], list(range(n)))]))
        at += n
    assert at == len(toks)
    r.end_request(rid)
    return torch.cat(got)


def with_tensors(model_dir, out_dir, change):
    """A copy of a model folder whose stored tensors `change` has altered (it gets them by name, bfloat16 as stored, and
    alters the dict in place)."""
    os.makedirs(out_dir, exist_ok=True)
    f = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
    tensors = {n: f.read(n).clone() for n in f.names()}
    change(tensors)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors)
    with open(os.path.join(model_dir, "config.json")) as src, open(os.path.join(out_dir, "config.json"), "w") as dst:
        dst.write(src.read())
    return out_dir


@pytest.mark.parametrize("name", ["delta", "delta_ff", "delta_one_tap", "latent", "latent_experts", "experts_one_of_many", "twice"])
def test_each_mechanism_alone(models, name):
    r = runner(models[name])
    toks = tokens(r.model.vocab_size, 45, 1)
    want = plain(models[name], toks)
    close(run_cut(r, "w", toks, [45]), want, "whole")
    close(run_cut(r, "d", toks, [1] * 45), want, "token by token")
    close(run_cut(r, "p", toks, [2, 7, 1, 3, 16, 2, 9, 5]), want, "portions")


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_decode_and_portions(models, name):
    r = runner(models[name], PAGE_SIZE[name])
    toks = tokens(r.model.vocab_size, 75, 2)
    want = plain(models[name], toks)
    close(run_cut(r, "w", toks, [75]), want, "whole")
    close(run_cut(r, "d", toks, [43] + [1] * 32), want, "decoded tail")
    for seed, sizes in ((3, (2, 3, 5)), (4, (2, 11, 17)), (5, (7, 8, 9, 16))):
        g, cuts, left = random.Random(seed), [], 75
        while left:
            n = min(g.choice(sizes), left)
            cuts.append(n)
            left -= n
        close(run_cut(r, f"p{seed}", toks, cuts), want, f"portions {sizes}")
    assert r.cache.stats()["slots_used"] == 0


@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_and_tiny_requests(models, name):
    """Requests of one to three tokens (shorter than the convolutions' reach) and small portions from the start: the
    zeros before a sequence's start, the empty state and the attention of a first token on itself and the sink."""
    r = runner(models[name], PAGE_SIZE[name])
    for n in (1, 2, 3):
        toks = tokens(r.model.vocab_size, n, 10 + n)
        close(run_cut(r, f"t{n}", toks, [n]), plain(models[name], toks), f"{n} tokens")
    toks = tokens(r.model.vocab_size, 9, 20)
    close(run_cut(r, "s", toks, [1, 2, 1, 2, 3]), plain(models[name], toks), "small portions from the start")


@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_requests_together_in_a_small_pool(models, name):
    """Four slots and a pool of a few pages: requests wait for room, and the pages and slots of finished requests go
    to the next ones (whose state starts from zero all the same); a request is sometimes left out of a step; every row
    equals the request alone."""
    ps = PAGE_SIZE[name]
    lengths = [23, 40, 9, 31, 1, 17, 28, 2, 36]
    r = runner(models[name], ps, max_tokens=6 * 16, max_requests=4)
    V = r.model.vocab_size
    reqs = {f"r{i}": tokens(V, n, 100 + i) for i, n in enumerate(lengths)}
    want = {k: plain(models[name], t) for k, t in reqs.items()}
    g = random.Random(9)
    waiting, live, at, got = list(reqs), [], {}, {k: [] for k in reqs}
    room = r.cache.num_pages * ps
    slots_seen = set()
    while waiting or live:
        while waiting and len(live) < 4 and sum(-(-len(reqs[x]) // ps) * ps for x in live + [waiting[0]]) <= room:
            k = waiting.pop(0)
            live.append(k)
            at[k] = 0
            r.add_request(k)
            slots_seen.add(r.cache.requests[k].slot)
        entries = []
        for k in live:
            if len(live) > 1 and g.random() < 0.25:
                continue
            left = len(reqs[k]) - at[k]
            n = 1 if left <= len(reqs[k]) // 3 else min(g.choice([2, 3, 5, 8]), left)
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
        if not entries:
            continue
        out = r.step(entries)
        row = 0
        for k, toks, _ in entries:
            got[k].append(out[row:row + len(toks)])
            row += len(toks)
            at[k] += len(toks)
            if at[k] == len(reqs[k]):
                live.remove(k)
                r.end_request(k)
    for k in reqs:
        close(torch.cat(got[k]), want[k], f"request {k}")
    st = r.cache.stats()
    assert st["slots_used"] == 0 and len(slots_seen) <= 4 and st["pages_reused"] > 0
    r.cache.check()


def test_sharp_latent_attention_over_far_keys_and_page_borders(models):
    """Sharp scores put nearly all weight on one cached row, wherever it lies: the first rows, rows at page borders and
    rows hundreds of positions back; the plain implementation with another first token differs, so a lost row shows."""
    name, ps = "sharp_latent", 8
    V = P.read_config(models[name])["vocab"]
    toks = tokens(V, 12 * ps + 5, 61)
    want = plain(models[name], toks)
    other = [(toks[0] + 1) % V] + toks[1:]
    assert (plain(models[name], other)[len(toks) // 2:] - want[len(toks) // 2:]).abs().max() > 0.05     # the far key counts
    sharp = 2e-3
    r = runner(models[name], ps, max_tokens=128)
    close(run_cut(r, "w", toks, [len(toks)]), want, "whole", sharp)
    head = [ps - 1, 1, 1, ps - 2, 2 * ps + 1, ps, 3]
    rest = len(toks) - sum(head) - 2 * ps - 3
    close(run_cut(r, "b", toks, head + [rest] + [1] * (2 * ps + 3)), want, "page borders", sharp)


def test_a_large_sink_takes_its_share(models, tmp_path):
    """Sinks between 1 and 4 (the scores are of size one): the sink holds a large part of every softmax's denominator,
    most of all at the first tokens.  The plain implementation without it, with it scaled like a score, or counted
    once per key differs by far more than the limit; the engine agrees with the right one, in prompts and decoding."""
    name = "latent"
    heads = P.read_config(models[name])["layers"][0]["mixer"]["heads"]

    def change(t):
        t["l0.mix.sink"] = torch.linspace(1.0, 4.0, heads).to(torch.bfloat16)
    d = with_tensors(models[name], str(tmp_path / "sink"), change)
    cfg, W = P.read_config(d), P.read_weights(d)
    toks = tokens(cfg["vocab"], 40, 70)
    want = P.forward(cfg, W, toks)
    scale = cfg["layers"][0]["mixer"]["scale"]
    for wrong_sink in (W["l0.mix.sink"] - 50.0, W["l0.mix.sink"] * scale):
        wrong = dict(W, **{"l0.mix.sink": wrong_sink})
        assert (P.forward(cfg, wrong, toks) - want).abs().max() > 0.05
    r = runner(d)
    close(run_cut(r, "w", toks, [40]), want, "whole")
    close(run_cut(r, "d", toks, [1] * 40), want, "token by token")
    close(run_cut(r, "p", toks, [3, 2, 9, 1, 17, 8]), want, "portions")


def test_the_state_keeps_a_far_token(models, tmp_path):
    """With decays close to one the delta rule's state still holds what the first token wrote a hundred tokens on:
    another first token moves the last rows, so a state that was lost, zeroed or swapped on the way shows.  Decoded
    one by one, in portions and whole."""
    name = "delta"

    def change(t):
        t["l0.mix.A_log"] = torch.full_like(t["l0.mix.A_log"], -7.0)
    d = with_tensors(models[name], str(tmp_path / "slow"), change)
    cfg, W = P.read_config(d), P.read_weights(d)
    V, n = cfg["vocab"], 120
    toks = tokens(V, n, 71)
    want = P.forward(cfg, W, toks)
    other = [(toks[0] + 1) % V] + toks[1:]
    assert (P.forward(cfg, W, other)[-20:] - want[-20:]).abs().max() > 0.02
    r = runner(d)
    close(run_cut(r, "w", toks, [n]), want, "whole")
    close(run_cut(r, "d", toks, [10] + [1] * 110), want, "110 decoded tokens")
    close(run_cut(r, "p", toks, [2, 31, 2, 50, 3, 30, 2]), want, "portions")


def test_decays_differ_from_channel_to_channel(models):
    """The plain implementation with every head's decays replaced by their mean over the key channels gives other
    logits, so a kernel that took one decay per head would show; the engine agrees with the right one."""
    name = "delta"
    cfg, W = P.read_config(models[name]), P.read_weights(models[name])
    m = cfg["layers"][0]["mixer"]
    toks = tokens(cfg["vocab"], 60, 72)
    want = P.forward(cfg, W, toks)
    H, D = m["heads"], m["dim"]
    mean_rows = lambda t: t.reshape(H, D, -1).mean(1, keepdim=True).expand(H, D, -1).reshape(t.shape)
    wrong = dict(W, **{"l0.mix.a2": mean_rows(W["l0.mix.a2"]), "l0.mix.dt_bias": mean_rows(W["l0.mix.dt_bias"])})
    assert (P.forward(cfg, wrong, toks) - want).abs().max() > 0.02
    r = runner(models[name])
    close(run_cut(r, "w", toks, [60]), want, "whole")
    close(run_cut(r, "d", toks, [20] + [1] * 40), want, "decoded")


def test_the_routers_weight_scales_the_experts_input(models):
    """Scores on the experts' outputs instead of their inputs, or divided by their sum, give other logits (the
    experts are not linear); the engine agrees with the weight on the input, not renormalized."""
    name = "latent_experts"
    cfg, W = P.read_config(models[name]), P.read_weights(models[name])
    toks = tokens(cfg["vocab"], 50, 73)
    want = P.forward(cfg, W, toks)

    def on_output(h, mlp, w, p, margins_out=None):
        s = torch.sigmoid(h @ w[p + "router"].T)
        out = torch.zeros_like(h)
        for t in range(h.shape[0]):
            for e in torch.topk(s[t], mlp["router"]["top"]).indices.tolist():
                out[t] += s[t, e] * P.gated_ff(h[t][None], w, f"{p}e{e}.")[0]
        return out
    right = P.routed_ff
    try:
        P.routed_ff = on_output
        assert (P.forward(cfg, W, toks) - want).abs().max() > 0.02
    finally:
        P.routed_ff = right
    r = runner(models[name])
    close(run_cut(r, "w", toks, [50]), want, "whole")
    close(run_cut(r, "d", toks, [25] + [1] * 25), want, "decoded")


def test_a_layer_on_another_layers_tensors_has_its_own_cache_and_state(models):
    """The second run of a layer sees other inputs than the first: were its rows written to the first run's pages, or
    its state kept in the first run's slot, decoding would differ from the whole prompt."""
    name = "twice"
    r = runner(models[name])
    paged = [g for g in r.cache.groups if g.paged]
    state = [g for g in r.cache.groups if not g.paged]
    assert sum(len(g.members) for g in paged) == 3 and sum(len(g.members) for g in state) == 2 * 2
    toks = tokens(r.model.vocab_size, 70, 74)
    want = plain(models[name], toks)
    close(run_cut(r, "d", toks, [9] + [1] * 61), want, "decoded")
    assert len([n for n in r.model.param_decls() if n.startswith("l2.") or n.startswith("l3.") or n.startswith("l4.")]) == 0


def test_long_decoding(models):
    """175 tokens decoded one by one across many pages; the latent layers keep every page."""
    name = "A"
    ps = PAGE_SIZE[name]
    r = runner(models[name], ps, max_tokens=256)
    toks = tokens(r.model.vocab_size, 180, 40)
    want = plain(models[name], toks)
    r.add_request("l")
    got = [r.step([("l", toks[:5], list(range(5)))])]
    for i in range(5, 180):
        got.append(r.step([("l", toks[i:i + 1], [0])]))
    close(torch.cat(got), want, "175 decoded tokens")
    for g in r.cache.paged_groups():
        assert r.cache.groups[g].pool.n_used == -(-180 // ps)
    r.end_request("l")
    r.cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(models, name):
    g = random.Random(3)
    cfg = P.read_config(models[name])
    prompts = [[g.randrange(cfg["vocab"]) for _ in range(n)] for n in (7, 13, 1, 22)]
    eng = Engine(models[name], "float32", max_num_seqs=3, max_batched_tokens=6, max_model_len=64,
                 page_size=PAGE_SIZE[name], device="cpu", ops=ref_ops)
    got = eng.generate(prompts, max_new_tokens=8, temperature=0.0)
    W = P.read_weights(models[name])
    for p, out in zip(prompts, got):
        assert len(out) == 8
        logits = P.forward(cfg, W, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert float(row.max() - row[tok]) < ATOL, f"token {i} is not the plain implementation's choice"
    assert eng.stats()["slots_used"] == 0


def test_configuration_is_read_and_checked():
    cfg = config_from_dict(ALL["B"][0])
    assert cfg.architecture == "Zikevik" and cfg.vocab_size == 257 and cfg.hidden_size == 66 and len(cfg.layers) == 5
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    for change, text in ((lambda c: c["layers"][0].update(type="rwkv"), "unknown mixer type"),
                         (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
                         (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "q_rank"),
                         (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
                         (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14), "rot_dim"),
                         (lambda c: c["layers"][1]["mixer"].update(heads=4, kv_heads=3), "multiple"),
                         (lambda c: c["layers"][1]["mixer"].update(conv=0), "at least 1"),
                         (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown kind"),
                         (lambda c: c["layers"][1]["mlp"]["router"].update(top=4), "top"),
                         (lambda c: c["layers"][1]["mlp"].pop("expert"), "expert"),
                         (lambda c: c["layers"][3].update(weights_of=3), "weights_of"),
                         (lambda c: c["layers"][4].update(weights_of=3), "weights_of"),
                         (lambda c: c["layers"][3]["mixer"].update(vdim=9), "equal"),
                         (lambda c: c.pop("norm"), "norm"),
                         (lambda c: c.pop("embedding"), "embedding"),
                         (lambda c: c.update(layers=[]), "at least one")):
        bad = copy.deepcopy(ALL["B"][0])
        change(bad)
        with pytest.raises(ConfigError, match=text):
            config_from_dict(bad)


def test_tensors_are_named_and_shaped_by_the_configuration(models):
    from zig_ai_b200.models import build_model
    decls = build_model(config_from_dict(ALL["B"][0])).param_decls()
    assert decls["embed"].shape == (257, 66) and decls["head"].shape == (257, 66) and decls["final.norm"].shape == (66,)
    assert decls["l0.mix.dq"].shape == (20, 66) and decls["l0.mix.dq.norm"].shape == (20,) and decls["l0.mix.uq"].shape == (4 * 32, 20)
    assert decls["l0.mix.dkv"].shape == (56, 66) and decls["l0.mix.dkv.norm"].shape == (40,)
    assert decls["l0.mix.uk"].shape == (64, 40) and decls["l0.mix.uv"].shape == (32, 40)
    assert decls["l0.mix.sink"].shape == (4,) and decls["l0.mix.g"].shape == (4, 66) and decls["l0.mix.o"].shape == (66, 32)
    assert decls["l1.mix.q"].shape == (48, 66) and decls["l1.mix.v"].shape == (24, 66) and decls["l1.mix.v.conv"].shape == (24, 2)
    assert decls["l1.mix.b"].shape == (3, 66) and decls["l1.mix.A_log"].shape == (3,) and decls["l1.mix.dt_bias"].shape == (48,)
    assert decls["l1.mix.a1"].shape == (4, 66) and decls["l1.mix.a2"].shape == (48, 4)
    assert decls["l1.mix.g1"].shape == (4, 66) and decls["l1.mix.g2"].shape == (24, 4) and decls["l1.mix.norm"].shape == (8,)
    assert decls["l1.mlp.router"].shape == (3, 66) and decls["l1.mlp.e2.gate"].shape == (40, 66) and decls["l1.mlp.e2.down"].shape == (66, 40)
    assert decls["l2.mix.q"].shape == (12, 66) and decls["l2.mix.v"].shape == (40, 66) and "l2.norm2" not in decls
    assert not [n for n in decls if n.startswith("l3.")] and decls["l4.mlp.e6.up"].shape == (16, 66)
    stored = set(SafetensorsFile(f"{models['B']}/model.safetensors").names())
    assert stored == set(decls)


def test_inner_sizes_come_from_the_stored_tensors(models, tmp_path):
    """A config.json that does not give the inner sizes of the decay's and the gate's projections: they are read from
    the stored tensors' shapes, also for a layer that runs on another layer's tensors."""
    name = "B"
    d = with_tensors(models[name], str(tmp_path / "m"), lambda t: None)
    cfg = P.read_config(d)
    for layer in cfg["layers"]:
        if layer["type"] == "channel_delta":
            assert layer["mixer"].pop("decay_rank") and layer["mixer"].pop("gate_rank")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    r = runner(d, PAGE_SIZE[name])
    toks = tokens(cfg["vocab"], 30, 80)
    close(run_cut(r, "p", toks, [11, 2, 1, 16]), plain(models[name], toks), "portions")


def random_configuration(g):
    """A small Zikevik configuration drawn at random: layer kinds and order, head counts, head sizes that differ between
    q/k and v, fewer query/key heads than value heads, taps, inner sizes, ranks and rotated parts, one expert a token up
    to all of them, layers without feed-forward, layers that run on an earlier layer's tensors."""
    layers = []
    for i in range(g.randint(2, 6)):
        own = [j for j, l in enumerate(layers) if "weights_of" not in l]
        if own and g.random() < 0.2:
            j = g.choice(own)
            layers.append(dict(copy.deepcopy(layers[j]), weights_of=j))
            continue
        r = g.random()
        if r < 0.25:
            mlp = None
        elif r < 0.55:
            mlp = dense(g.choice([24, 56, 100]))
        else:
            experts = g.choice([1, 2, 3, 5, 8, 11])
            mlp = moe(g.choice([8, 20, 36]), experts, g.choice([1, min(2, experts), min(4, experts), experts]))
        if g.random() < 0.45:
            heads = g.choice([1, 2, 3, 4, 6])
            kv = g.choice([k for k in (1, 2, 3, 4, 6) if heads % k == 0])
            layers.append(delta(heads, kv, g.choice([4, 8, 12, 16]), g.choice([4, 8, 10, 24]), g.choice([1, 2, 3, 4, 6]),
                                g.choice([1, 3, 8]), g.choice([2, 5, 8]), mlp=mlp))
        else:
            layers.append(latent(g.choice([1, 2, 3, 5]), g.choice([4, 6, 16]), g.choice([2, 4, 8, 12]), g.choice([4, 10, 16]),
                                 g.choice([8, 17, 24, 32]), g.choice([6, 16, 40]), g.choice([0.15, 0.3, 0.5]),
                                 g.choice([300.0, 10000.0, 1e6]), mlp=mlp))
    return config(g.choice([61, 97, 130]), g.choice([24, 40, 50, 64]), g.choice([1e-5, 1e-6]), g.choice([0.5, 1.0, 1.7]), layers)


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(tmp_path, seed):
    g = random.Random(3000 + seed)
    cfg = random_configuration(g)
    d = str(tmp_path / "m")
    write_random_model(config_from_dict(cfg), seed, d, matrix_std="fan_in")
    toks = tokens(cfg["vocab"], 70, seed)
    want = plain(d, toks)
    r = runner(d, g.choice([4, 8, 16]), max_tokens=128)
    close(run_cut(r, "w", toks, [70]), want, "whole")
    close(run_cut(r, "p", toks, [9, 2, 17, 1, 1, 3, 30, 2, 5]), want, "portions")
    close(run_cut(r, "d", toks, [50] + [1] * 20), want, "decoded tail")
    r.cache.check()
