"""The Lolivik design through the engine's host logic on the CPU: the step function, the cache (pages of keys and values,
a window that keeps the request's first pages, slots of recurrent state, values handed from the first mixing layer to the
later ones within a step) and the batch description run with the plain PyTorch kernels of tests/ref_ops.py in place of
the CUDA kernels and are compared with the plain whole-sequence implementation (tests/plain_lolivik.py): each mechanism
alone, whole prompts, token-by-token decoding, portions down to two tokens, batches of unequal requests in a pool so small
that pages and slots are used again, keys far away, at page borders and just inside and outside the window and the kept
first positions with attention made sharp, the distance bias's buckets, the sink, the queries' temperature steps, the
state's running maximum, the first tokens of a request, long decoding, and greedy generation through the entry point."""
import json
import math
import os
import random

import pytest
import torch

import plain_lolivik as P
import ref_ops
from lolivik_configs import ALL, ONLY, PAGE_SIZE, attention, config, dense, memory, moe, windowed
from zig_ai_b200.config import ConfigError, config_from_dict
from zig_ai_b200.engine import Engine
from zig_ai_b200.engine.runner import load_runner
from zig_ai_b200.weights import write_random_model
from zig_ai_b200.weights.safetensors_io import SafetensorsFile, write_safetensors

ATOL = 3e-4          # float32 on the CPU against float64, logits of size one to ten


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("lolivik")
    out = {}
    for name, (cfg, seed) in list(ALL.items())[:2] + [(k, (c, 5)) for k, c in ONLY.items()]:
        d = str(root / name)
        write_random_model(config_from_dict(cfg), seed, d, matrix_std="fan_in")
        out[name] = d
    return out


def read_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    f = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
    return cfg, {n: f.read(n) for n in f.names()}


def plain(model_dir, tokens):
    cfg, tensors = read_model(model_dir)
    return P.forward(cfg, tensors, tokens)


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


@pytest.mark.parametrize("name", sorted(ONLY))
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
    """Requests of one to three tokens and small portions from the start: the empty state whose running maximum starts at
    zero, the attention of a first token on itself and the sink, positions below the first temperature step."""
    r = runner(models[name], PAGE_SIZE[name])
    for n in (1, 2, 3):
        toks = tokens(r.model.vocab_size, n, 10 + n)
        close(run_cut(r, f"t{n}", toks, [n]), plain(models[name], toks), f"{n} tokens")
    toks = tokens(r.model.vocab_size, 9, 20)
    close(run_cut(r, "s", toks, [1, 2, 1, 2, 3]), plain(models[name], toks), "small portions from the start")


@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_requests_together_in_a_small_pool(models, name):
    """Four slots and a pool of a few pages: requests wait for room, and the pages and slots of finished requests go to the
    next ones (whose state starts from zero all the same); a request is sometimes left out of a step; every row equals
    the request alone."""
    ps = PAGE_SIZE[name]
    lengths = [23, 40, 9, 31, 1, 17, 28, 2, 36]
    r = runner(models[name], ps, max_tokens=6 * 16, max_requests=4)
    V = r.model.vocab_size
    reqs = {f"r{i}": tokens(V, n, 100 + i) for i, n in enumerate(lengths)}
    want = {k: plain(models[name], t) for k, t in reqs.items()}
    g = random.Random(9)
    waiting, live, at, got = list(reqs), [], {}, {k: [] for k in reqs}
    room = r.cache.num_pages * ps
    slots_seen = []
    while waiting or live:
        while waiting and len(live) < 4 and sum(-(-len(reqs[x]) // ps) * ps for x in live + [waiting[0]]) <= room:
            k = waiting.pop(0)
            live.append(k)
            at[k] = 0
            r.add_request(k)
            slots_seen.append(r.cache.requests[k].slot)
        entries = []
        for k in live:
            if len(live) > 1 and g.random() < 0.25:
                continue
            left = len(reqs[k]) - at[k]
            n = 1 if left <= len(reqs[k]) // 3 else min(g.choice([2, 3, 5, 8]), left)
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
        if not entries:
            continue
        logits = r.step(entries)
        row = 0
        for k, toks, w in entries:
            got[k].append(logits[row:row + len(w)].clone())
            row += len(w)
        for k in [k for k in live if at[k] == len(reqs[k])]:
            live.remove(k)
            r.end_request(k)
        r.cache.check()
    for k in reqs:
        close(torch.cat(got[k]), want[k], f"request {k} among others")
    assert len(slots_seen) > len(set(slots_seen)) and r.cache.pages_reused > 0     # slots and pages were used again


def sharp_key(tensors, pre, key_dim, value_width):
    """Make layer `pre`'s attention depend on single keys: the k projection is scaled up so that scores differ by many
    units and nearly all weight lies on one key."""
    tensors[pre + "k"] = (tensors[pre + "k"].float() * 6.0).to(torch.bfloat16)


@pytest.mark.parametrize("name,window,keep", [("sharp_windowed", 13, 3)])
def test_window_edges_and_kept_first_positions(models, tmp_path, name, window, keep):
    """With attention made sharp a key just inside the window, just outside it, a kept first position and the first one
    that is not kept all show in the logits: every cut of the request agrees with the whole sequence, for queries in
    prompt portions and decoded one by one, with pages of 4 (window and kept positions end inside pages)."""
    d = with_tensors(models[name], str(tmp_path / "sharp"), lambda t: sharp_key(t, "l0.mix.", 10, 14))
    cfg, tensors = read_model(d)
    r = runner(d, page_size=4)
    toks = tokens(cfg["vocab"], 60, 7)
    want = P.forward(cfg, tensors, toks)
    # the mask matters: the same model with a window one position longer or one kept position more gives other logits
    for dw, dk in ((1, 0), (-1, 0), (0, 1), (0, -1)):
        other = json.loads(json.dumps(cfg))
        other["layers"][0]["mixer"]["mask"] = {"size": window + dw, "keep_first": keep + dk}
        assert (P.forward(other, tensors, toks) - want).abs().max() > 1e-2
    close(run_cut(r, "w", toks, [60]), want, "whole")
    close(run_cut(r, "d", toks, [5] + [1] * 55), want, "decoded across the window's edge")
    close(run_cut(r, "p", toks, [3, 10, 2, 13, 1, 14, 2, 2, 13]), want, "portions that end at the window's edges")
    # pages behind the window went back to the pool while the request ran, the kept first page stayed
    r.add_request("k")
    r.step([("k", toks[:40], [])])
    r.step([("k", toks[40:41], [])])
    table = r.cache.requests["k"].tables[0]
    assert table[0] > 0 and -1 in table[1:]
    r.end_request("k")


def test_far_keys_buckets_sink_and_temperature(models, tmp_path):
    """The distance bias, the sink and the queries' temperature each change the logits of a long request, far keys (beyond the
    table's last bucket) count, and all cuts agree with the whole sequence across page borders (pages of 8)."""
    name = "sharp_attention"

    def change(t):
        sharp_key(t, "l0.mix.", 10, 14)
        t["l0.mix.rel"] = (t["l0.mix.rel"].float() * 30.0).to(torch.bfloat16)      # buckets that differ by units
        t["l0.mix.sink"] = (t["l0.mix.sink"].float() * 10.0 + 2.0).to(torch.bfloat16)
    d = with_tensors(models[name], str(tmp_path / "far"), change)
    cfg, tensors = read_model(d)
    toks = tokens(cfg["vocab"], 150, 11)
    want = P.forward(cfg, tensors, toks)
    for key, value in (("bias_max", 200), ("softcap", 10.0), ("q_temp", {"coef": 0.2, "every": 17})):
        other = json.loads(json.dumps(cfg))
        other["layers"][0]["mixer"][key] = value
        assert (P.forward(other, tensors, toks) - want).abs().max() > 1e-2, key
    no_sink = dict(tensors)
    no_sink["l0.mix.sink"] = tensors["l0.mix.sink"] - 30.0
    assert (P.forward(cfg, no_sink, toks) - want).abs().max() > 1e-2
    r = runner(d, page_size=8)
    close(run_cut(r, "w", toks, [150]), want, "whole")
    close(run_cut(r, "d", toks, [100] + [1] * 50), want, "decoded")
    close(run_cut(r, "p", toks, [8, 8, 7, 2, 15, 64, 1, 31, 14]), want, "portions across page borders and temperature steps")


def test_distance_table_matches_the_bucket_rule():
    from zig_ai_b200.parts.attention import Attention
    from zig_ai_b200.parts.base import PartSpec
    for rows, far in ((16, 240), (7, 25), (4, 9), (32, 1000), (12, 70), (2, 3)):
        a = Attention(hidden=8, heads=2, kv_heads=1, head_dim=4, qk_norm=False, eps=1e-5, position=PartSpec("none", {}),
                      rel_bias={"rows": rows, "max": far})
        rel = torch.arange(rows * 2, dtype=torch.float32).reshape(rows, 2)
        table = a.distance_table(rel)
        for n in list(range(table.shape[0] + 5)) + [10 * far]:
            assert torch.equal(table[min(n, table.shape[0] - 1)], rel[P.bucket(n, rows, far)]), (rows, far, n)


def test_state_keeps_a_far_token_and_its_running_maximum(models, tmp_path):
    """An input gate that is large for one token and a forget gate near one: the state holds that token for the rest of
    the request, the running maximum jumps there, and portions, single tokens and the whole sequence agree."""
    def change(t):
        t["l0.mix.i.b"] = torch.full_like(t["l0.mix.i.b"], -6.0)
        t["l0.mix.f.b"] = torch.full_like(t["l0.mix.f.b"], 8.0)
        t["l0.mix.i"] = (t["l0.mix.i"].float() * 8.0).to(torch.bfloat16)
    d = with_tensors(models["memory"], str(tmp_path / "mem"), change)
    cfg, tensors = read_model(d)
    toks = tokens(cfg["vocab"], 90, 13)
    want = P.forward(cfg, tensors, toks)
    r = runner(d, page_size=8)
    close(run_cut(r, "w", toks, [90]), want, "whole")
    close(run_cut(r, "d", toks, [20] + [1] * 70), want, "long decoding")
    close(run_cut(r, "p", toks, [2, 2, 31, 16, 17, 2, 20]), want, "portions")


def test_long_decoding(models):
    r = runner(models["A"], PAGE_SIZE["A"], max_tokens=256)
    toks = tokens(r.model.vocab_size, 160, 17)
    close(run_cut(r, "d", toks, [4] + [1] * 156), plain(models["A"], toks), "156 decoded tokens")


def test_config_errors():
    good = ONLY["mixed_values"]
    for path, value in ((("layers", 0, "type"), "conv"), (("layers", 1, "mixer", "softcap"), 0.0),
                        (("layers", 0, "mixer", "mask", "size"), 0), (("layers", 2, "mixer", "vdim"), 12), (("norm",), None)):
        bad = json.loads(json.dumps(good))
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            config_from_dict(bad)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(models, name):
    """`Engine.generate` (scheduler, sampler, step function, prompts in portions of six tokens beside decoding requests)
    against the plain implementation's choice at every produced token."""
    cfg, tensors = read_model(models[name])
    g = random.Random(3)
    prompts = [[g.randrange(cfg["vocab"]) for _ in range(n)] for n in (7, 13, 1, 22)]
    eng = Engine(models[name], "float32", max_num_seqs=3, max_batched_tokens=6, max_model_len=64,
                 page_size=PAGE_SIZE[name], device="cpu", ops=ref_ops)
    got = eng.generate(prompts, max_new_tokens=8, temperature=0.0)
    for p, out in zip(prompts, got):
        assert len(out) == 8
        logits = P.forward(cfg, tensors, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert float(row.max() - row[tok]) < ATOL, f"token {i} is not the plain implementation's choice"
    assert eng.stats()["slots_used"] == 0


def test_configuration_round_trip():
    cfg = config_from_dict(ALL["B"][0])
    assert cfg.architecture == "Lolivik" and cfg.vocab_size == 257 and cfg.hidden_size == 66 and len(cfg.layers) == 5
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
