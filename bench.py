#!/usr/bin/env python3
"""Benchmark: decode tokens per second of the LFM2-350M shape on one B200, with prefill, roofline
and end-to-end figures on the same JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 requests whose contexts lie between 2048 and 4096
tokens; weights are random (seeded), token ids are random: there is no dataset.  `value` times the
step function and the sampling kernel on the device with CUDA events; `e2e` times the same steps
through `Engine.step()`, the call a user makes, with host token lists in and out.  The decode step
reads about 0.7 GB of weights, more than the 126 MB L2, so consecutive steps cannot be served from L2.
"""
import argparse
import json
import os
import random
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LFM2_350M = {
    "architectures": ["Lfm2ForCausalLM"], "hidden_size": 1024, "num_hidden_layers": 16,
    "full_attn_idxs": [2, 5, 8, 10, 12, 14], "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 64,
    "block_ff_dim": 6656, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256, "vocab_size": 65536,
    "rope_theta": 1000000.0, "conv_L_cache": 3, "conv_bias": False, "use_qk_norm": True, "norm_eps": 1e-5,
    "tie_embedding": True, "max_position_embeddings": 128000,
}
SHAPES = {
    "350m": dict(hidden_size=1024, num_attention_heads=16, block_ff_dim=6656),
    "700m": dict(hidden_size=1536, num_attention_heads=24, block_ff_dim=10752),
    "1.2b": dict(hidden_size=2048, num_attention_heads=32, block_ff_dim=12288),
}
CONTEXT = 4096
PREFILL_TOKENS = 2048


def shape_config(name):
    d = dict(LFM2_350M)
    d.update(SHAPES[name])
    return d


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, flops, src = 6650.0, 1590.0, "fallback"
    try:
        with open(path) as f:
            d = json.load(f)
        hbm = float(d.get("hbm_gbs", hbm))
        flops = float(d.get("bf16_tflops", flops))
        src = "measured"
    except (OSError, ValueError):
        pass
    return hbm, flops, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [x.strip() for x in line.split(",")]))

    def mark(self):
        """The timed region starts here: earlier samples do not count."""
        self.t0 = time.perf_counter()

    def stop(self):
        if self.proc:
            time.sleep(0.05)
            self.proc.terminate()
        t0 = getattr(self, "t0", 0.0)
        self.rows = [r for t, r in self.rows if t >= t0] or [r for t, r in self.rows[-3:]]
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def model_numbers(cfg):
    """Matrix parameters read once per decode step, their flops per token, KV bytes per token."""
    H, F, V = cfg.hidden_size, cfg.ff_dim, cfg.vocab_size
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    n_attn = len(cfg.attention_layers)
    n_conv = cfg.num_hidden_layers - n_attn
    per_layer_ff = 3 * H * F
    conv = 3 * H * H + H * H
    attn = (Hq + 2 * Hkv) * D * H + Hq * D * H
    layer_params = cfg.num_hidden_layers * per_layer_ff + n_conv * conv + n_attn * attn
    head = V * H
    kv_bytes_per_token = n_attn * 2 * Hkv * D * 2
    state_bytes = n_conv * (cfg.conv_L_cache - 1) * H * 4
    return dict(layer_params=layer_params, head_params=head, kv_bytes_per_token=kv_bytes_per_token,
                state_bytes=state_bytes, n_attn=n_attn, attn_dims=(Hq, D))


PROFILE_RANGE = False      # --profile-range: the timed decode steps lie between cudaProfilerStart and cudaProfilerStop


def decode_requests(eng, B, steps_needed, seed):
    """Add B requests with contexts spread over CONTEXT / 2..CONTEXT and run until all of them decode."""
    from zig_ai_b200.sampling import SamplingParams
    g = random.Random(seed)
    lo = CONTEXT // 2
    hi = CONTEXT - steps_needed - 160          # room for the tokens decoded while later requests still prefill
    lens = [lo + (hi - lo) * i // max(B - 1, 1) for i in range(B)] if B > 1 else [(lo + hi) // 2]
    V = eng.config.vocab_size
    ids = [eng.add_request([g.randrange(V) for _ in range(n)],
                           SamplingParams(temperature=0.0, max_new_tokens=CONTEXT - n)) for n in lens]
    while any(eng.requests[i].computed < len(eng.requests[i].prompt) or not eng.requests[i].output for i in ids):
        eng.step()
    return ids


def time_decode(eng, B, steps, warmup, clocks=None):
    """Device-timed decode steps of batch B (step function + sampling kernel, no host read-back),
    then the same number of steps through Engine.step().  Returns (ms/step device, ms/step e2e,
    context tokens read per step, launches per step, h2d bytes, d2h bytes)."""
    import torch
    from zig_ai_b200.kernels import ops
    if clocks:
        clocks.start()                       # nvidia-smi takes a while to give its first sample
    ids = decode_requests(eng, B, 2 * (steps + warmup) + 4, seed=B)
    eng.flush()                              # no step on its way while the runner is driven directly
    reqs = [eng.requests[i] for i in ids]
    runner = eng.runner
    ctx_tokens = sum(r.computed for r in reqs)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    # the host work of every step (page reservation, packing) is done before the clock starts; the
    # timed region holds, per step, the pinned-to-device copy of the batch description, the step's
    # kernels and the sampling kernel, with no read-back in between
    prepared = [runner.prepare_decode([(r.request_id, [(7 * k + j) % 1000], [0]) for j, r in enumerate(reqs)])
                for k in range(warmup + steps)]
    for k in range(warmup):
        ops.argmax(runner.run_prepared(prepared[k]))
    torch.cuda.synchronize()
    launches0 = ops.launches
    if clocks:
        clocks.mark()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps - 1)]
    if PROFILE_RANGE:
        torch.cuda.profiler.start()          # a profiler started with --profile-from-start off sees only these steps
    start.record()
    for k in range(steps):
        ops.argmax(runner.run_prepared(prepared[warmup + k]))
        if k < steps - 1:
            marks[k].record()
    stop.record()
    torch.cuda.synchronize()
    if PROFILE_RANGE:
        torch.cuda.profiler.stop()
    dev_ms = start.elapsed_time(stop) / steps
    edges = [start] + marks + [stop]
    per_step = [edges[k].elapsed_time(edges[k + 1]) for k in range(steps)]
    launches = (ops.launches - launches0) / steps
    # the scheduler's view has to follow what was run behind its back
    for r in reqs:
        r.computed = runner.processed[r.request_id]
        r.output += [0] * (r.computed + 1 - len(r.prompt) - len(r.output))
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e2e_steps = []
    for _ in range(steps):
        t1 = time.perf_counter()
        eng.step()
        e2e_steps.append((time.perf_counter() - t1) * 1e3)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    if os.environ.get("ZAI_BENCH_STEPS"):
        worst = max(range(steps), key=lambda k: per_step[k])
        worst_e = max(range(steps), key=lambda k: e2e_steps[k])
        print(f"[bench] batch {B}: device median {sorted(per_step)[steps // 2]:.3f} ms, worst {per_step[worst]:.3f} ms at step "
              f"{worst}; e2e median {sorted(e2e_steps)[steps // 2]:.3f} ms, worst {e2e_steps[worst_e]:.3f} ms at step {worst_e}; "
              f"kernel status {ops.tc_status()}",
              file=sys.stderr, flush=True)
    clock_info = clocks.stop() if clocks else None
    eng.flush()
    for r in list(reqs):
        if r.request_id in eng.requests:
            eng.scheduler.running.remove(r)
            runner.end_request(r.request_id)
            eng.requests.pop(r.request_id)
    width = next(iter(runner.graphs.widths.values())) if runner.graphs else 0
    bucket = runner.graphs.bucket(B) if runner.graphs else B
    h2d = 4 * (3 * bucket + (bucket + 1) + 3 * bucket + bucket * width)
    d2h = 4 * (B + 1)                        # the token ids and the kernels' status word behind them
    return dev_ms, e2e_ms, ctx_tokens, launches, h2d, d2h, clock_info


def time_prefill(eng, reps=5):
    import torch
    g = random.Random(99)
    V = eng.config.vocab_size
    runner = eng.runner
    times = []
    for i in range(reps + 2):
        toks = [g.randrange(V) for _ in range(PREFILL_TOKENS)]
        rid = f"prefill{i}"
        runner.add_request(rid)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([(rid, toks, [PREFILL_TOKENS - 1])])
        stop.record()
        torch.cuda.synchronize()
        runner.end_request(rid)
        if i >= 2:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def run_ours(args):
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    from zig_ai_b200.kernels import build
    build.build_all(verbose=False)
    hbm_peak, flops_peak, peak_src = peaks()
    cfg = config_from_dict(shape_config(args.model))
    nums = model_numbers(cfg)
    if args.workload == "mixed":
        return run_mixed(args, cfg)
    if args.only == "vunolorn":
        return run_vunolorn(args)
    if args.only == "pikasun":
        return run_pikasun(args)
    if args.only == "zikevik":
        return run_zikevik(args)
    if args.only == "lolivik":
        return run_lolivik(args)
    if args.only == "long":
        return run_long(args)
    if args.only == "sample":
        return run_sample(args)
    if args.only == "table":
        return run_table(args)
    if args.only == "stream":
        return run_stream_table(cfg, args.batch)
    with tempfile.TemporaryDirectory(prefix="lfm2_350m_") as d:
        z.write_random_model(cfg, 0, d)
        eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048 + 64, max_model_len=CONTEXT,
                       max_tokens=64 * CONTEXT, page_size=args.page_size)
        if args.only == "gemm":
            return run_gemm_table(cfg)
        if args.only == "prefill":
            print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "ms": round(time_prefill(eng, reps=args.steps), 3)}))
            return 0
        if args.only == "timeline":
            return run_timeline(eng, args.batch)
        if args.only == "decode":
            ms, e2e, ctx, launches, _, _, _ = time_decode(eng, args.batch, args.steps, args.warmup)
            print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": round(ms, 4),
                              "e2e_ms_per_step": round(e2e, 4), "launches_per_step": launches}))
            return 0
        prefill_ms = time_prefill(eng, reps=15)
        clocks = ClockSampler()
        dev_ms, e2e_ms, ctx_tokens, launches, h2d, d2h, clock_info = time_decode(eng, 8, args.steps, args.warmup, clocks)
        points = {}
        for B in (1, 64):
            ms, _, _, _, _, _, _ = time_decode(eng, B, max(args.steps // 2, 20), args.warmup)
            points[f"decode_b{B}"] = round(B / ms * 1e3, 1)
    weight_bytes = 2 * (nums["layer_params"] + nums["head_params"])
    step_bytes = weight_bytes + ctx_tokens * nums["kv_bytes_per_token"] + 8 * nums["state_bytes"]
    achieved = step_bytes / (dev_ms * 1e-3) / 1e9
    Hq, D = nums["attn_dims"]
    T = PREFILL_TOKENS
    prefill_flops = 2 * T * nums["layer_params"] + 2 * 1 * nums["head_params"] + nums["n_attn"] * 2 * T * T * Hq * D
    out = {
        "metric": f"decode tok/s @ batch 8 (LFM2-{args.model.upper()} shape, context 2048-4096)",
        "value": round(8 / dev_ms * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)",
        "impl": "ours",
        "config": {"model": f"LFM2-{args.model.upper()} shape", "layers": cfg.num_hidden_layers, "layers_of_config": 16,
                   "attn_layers": nums["n_attn"], "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "ff_dim": cfg.ff_dim,
                   "vocab": cfg.vocab_size, "conv_taps": cfg.conv_L_cache, "global_batch": 8, "seq_len": CONTEXT,
                   "mean_context": round(ctx_tokens / 8), "page_size": args.page_size, "parallelism": "single GPU",
                   "l2": f"step reads {weight_bytes / 1e9:.2f} GB of weights (> 126 MB L2)", "peaks": peak_src},
        "e2e": {"value": round(8 / e2e_ms * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(round(launches * args.steps)),
        "prefill": {"value": round(T / prefill_ms * 1e3, 1), "tokens": T, "ms": round(prefill_ms, 3),
                    "frac": round(prefill_flops / (prefill_ms * 1e-3) / (flops_peak * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4)},
        "points": points,
        "clocks": clock_info,
    }
    print(json.dumps(out))
    return 0


def measure_shape(model, steps, warmup, page_size=64):
    """Every figure of one model shape: decode at batch 1, 8 and 64 (device-timed and through Engine.step),
    the prefill of 2048 tokens, each with the bytes or flops it has to move and the fraction of the peak."""
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    hbm_peak, flops_peak, peak_src = peaks()
    cfg = config_from_dict(shape_config(model))
    nums = model_numbers(cfg)
    rows = []
    with tempfile.TemporaryDirectory(prefix=f"lfm2_{model.replace('.', '_')}_") as d:
        z.write_random_model(cfg, 0, d)
        eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048 + 64, max_model_len=CONTEXT,
                       max_tokens=64 * CONTEXT, page_size=page_size)
        prefill_ms = time_prefill(eng, reps=max(min(steps, 20), 5))
        Hq, D = nums["attn_dims"]
        T = PREFILL_TOKENS
        flops = 2 * T * nums["layer_params"] + 2 * nums["head_params"] + nums["n_attn"] * 2 * T * T * Hq * D
        rows.append({"model": model, "point": "prefill 2048", "ms": round(prefill_ms, 3), "tokens_per_s": round(T / prefill_ms * 1e3),
                     "work": f"{flops / 1e12:.3f} TFLOP", "achieved": f"{flops / prefill_ms / 1e9:.0f} TFLOP/s",
                     "frac_of_peak": round(flops / (prefill_ms * 1e-3) / (flops_peak * 1e12), 3)})
        weight_bytes = 2 * (nums["layer_params"] + nums["head_params"])
        for B in (1, 8, 64):
            dev_ms, e2e_ms, ctx_tokens, launches, _, _, _ = time_decode(eng, B, max(steps, 20), warmup)
            step_bytes = weight_bytes + ctx_tokens * nums["kv_bytes_per_token"] + B * nums["state_bytes"]
            rows.append({"model": model, "point": f"decode batch {B}", "ms": round(dev_ms, 4), "e2e_ms": round(e2e_ms, 4),
                         "tokens_per_s": round(B / dev_ms * 1e3), "e2e_tokens_per_s": round(B / e2e_ms * 1e3),
                         "mean_context": round(ctx_tokens / B), "work": f"{step_bytes / 1e9:.3f} GB",
                         "achieved": f"{step_bytes / dev_ms / 1e6:.0f} GB/s",
                         "frac_of_peak": round(step_bytes / (dev_ms * 1e-3) / 1e9 / hbm_peak, 3),
                         "launches_per_step": round(launches)})
    return rows, peak_src


# ----------------------------------------------------------------------------- the Vunolorn hybrid beside LFM2
def vunolorn_config(width, layers=16, vocab=65536):
    """A Vunolorn model of a real model's proportions: groups of four layers (attention beside the minimal gated
    recurrence with a dense feed-forward four times the width, two selective scans twice the width with 16 states,
    a gated delta rule with value heads of 128), head size 64 throughout."""
    heads = width // 64
    group = [
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 4 * width},
         "mixer": {"left": {"heads": heads, "kv_heads": heads // 2, "dim": 64, "vdim": 64, "scale": 0.125,
                            "rot": {"base": 1000000.0, "dims": 64}},
                   "right": {"width": width}, "left_scale": 1.0, "right_scale": 1.0}},
        {"type": "mamba1", "mlp": None, "mixer": {"inner": 2 * width, "state": 16, "dt_rank": width // 16, "conv": 4}},
        {"type": "mamba1", "mlp": None, "mixer": {"inner": 2 * width, "state": 16, "dt_rank": width // 16, "conv": 4}},
        {"type": "delta", "mlp": None, "mixer": {"heads": heads, "kv_heads": heads // 2, "dim": 64, "vdim": 128, "conv": 4}},
    ]
    return {"architecture": "Vunolorn", "vocab": vocab, "width": width, "embedding": {"scale": float(width) ** 0.5},
            "norm": {"eps": 1e-6}, "layers": [dict(group[i % 4]) for i in range(layers)]}


def engine_numbers(eng):
    """From the engine itself, for any architecture: matrix parameters a step reads, bytes of keys and values per
    cached position, bytes of per-request state."""
    decls = eng.runner.model.param_decls()
    numel = lambda shape: int(__import__("math").prod(shape))
    matrix = sum(numel(d.shape) for d in decls.values() if d.role == "matrix")
    if getattr(eng.runner.model.head, "tied", False):
        matrix += sum(numel(d.shape) for d in decls.values() if d.role == "table")
    cache = eng.runner.cache
    state = sum(len(g.members) * numel(g.need.shape) * 4 for g in cache.groups if not g.paged)
    routed = []        # (experts, experts a token uses, parameters of one expert) of every mixture of experts
    for blk in eng.runner.model.blocks:
        ff = getattr(blk, "feed_forward", None)
        if ff is not None and hasattr(ff, "experts") and hasattr(ff, "top"):
            routed.append((ff.experts, ff.top, 3 * ff.hidden * ff.ff_dim))
    return dict(matrix_params=matrix, kv_bytes_per_token=cache.bytes_per_token(), state_bytes=state, routed=routed)


def params_read(nums, tokens):
    """Matrix parameters that a step of `tokens` rows reads: everything but the experts that none of its rows chose
    (expected, for rows that choose independently and evenly)."""
    unread = sum(E * (1.0 - top / E) ** tokens * per for E, top, per in nums["routed"])
    return nums["matrix_params"] - unread


def kernel_classes(eng, entries):
    """Milliseconds per kernel class of one step launched kernel by kernel (CUDA events around every kernel
    function; the shares are what it is for)."""
    from zig_ai_b200.kernels import ops
    runner = eng.runner
    graphs, runner.use_graphs = runner.use_graphs, False
    try:
        for rid, _, _ in entries:
            if not runner.has_request(rid):
                runner.add_request(rid)
        runner.step([(rid, toks, want) for rid, toks, want in entries])          # warm-up: same shapes
        for rid, _, _ in entries:
            runner.end_request(rid)
            runner.add_request(rid)
        ops.profile_begin()
        runner.step([(rid, toks, want) for rid, toks, want in entries])
        out = ops.profile_end()
        for rid, _, _ in entries:
            runner.end_request(rid)
    finally:
        runner.use_graphs = graphs
    return {k: round(v, 4) for k, v in sorted(out.items(), key=lambda kv: -kv[1])}


def recurrent_kernel_rooflines(width, hbm_peak):
    """Each kernel of the recurrent mixers alone at the sizes of `vunolorn_config(width)`, beside LFM2's short
    convolution at the same width (the like kernel of the closest model): a prompt portion of 2048 tokens of one
    request and a step of 64 single tokens, timed with CUDA events over inputs that are rotated through more
    memory than the L2 holds; bytes are what the kernel has to read and write once."""
    import torch
    from zig_ai_b200.engine.batch import pack_step
    from zig_ai_b200.kernels import ops
    dev, bf = torch.device("cuda"), torch.bfloat16
    heads, G, D, V, I, S, R, W, L = width // 64, width // 128, 64, 128, 2 * width, 16, width // 16, width, 4
    rows = []

    def timed(f, n_sets):
        for i in range(3):
            f(i % n_sets)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        reps = 20
        a.record()
        for i in range(reps):
            f(i % n_sets)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    for point, q_lens in (("prompt portion of 2048", [2048]), ("64 single tokens", [1] * 64)):
        N, B = sum(q_lens), len(q_lens)
        step = pack_step(ops, bf, dev, [(s, 100, [0] * n, [], s + 1) for s, n in enumerate(q_lens)],
                         {0: [[1, 2] + [0] * 40 for _ in q_lens]})
        n_sets = max(2, int(160e6 // max(N * 6 * I, 1)) + 1) if N > 64 else 24       # inputs and states rotate: more than L2
        rnd = lambda *shape: [torch.randn(*shape, device=dev).to(bf) for _ in range(n_sets)]
        st = lambda *shape: [torch.zeros(B + 1, *shape, device=dev) for _ in range(n_sets)]
        # selective scan
        x, proj, xz = rnd(N, I), rnd(N, R + 2 * S), rnd(N, 2 * I)
        w_dt, b_dt, a_log, dsk = torch.randn(I, R, device=dev).to(bf) * 0.1, torch.zeros(I, device=dev), torch.zeros(I, S, device=dev), torch.ones(I, device=dev)
        state = st(I, S)
        ms = timed(lambda i: ops.selective_scan(x[i], proj[i], xz[i][:, I:], w_dt, b_dt, a_log, dsk, state[i], step, R), n_sets)
        rows.append(("selective scan", point, ms, N * (3 * I + R + 2 * S) * 2 + B * I * S * 8))
        # causal convolution (the scan's, 2W channels)
        conv_w, conv_b, cstate = torch.randn(I, L, device=dev) * 0.1, torch.zeros(I, device=dev), st(L - 1, I)
        ms = timed(lambda i: ops.causal_conv(xz[i][:, :I], conv_w, conv_b, cstate[i], step, True), n_sets)
        rows.append(("causal convolution + SiLU", point, ms, N * 2 * I * 2 + B * (L - 1) * I * 8))
        # minimal gated recurrence
        zxg, gstate = rnd(N, 3 * W), st(W)
        bz = torch.zeros(W, device=dev)
        ms = timed(lambda i: ops.min_gru(zxg[i], bz, bz, gstate[i], step), n_sets)
        rows.append(("minimal gated recurrence", point, ms, N * 4 * W * 2 + B * W * 8))
        # gated delta rule (prepare + recurrence + output norm)
        cols = 2 * G * D + heads * V
        qkv, rest, dstate = rnd(N, cols), rnd(N, heads * V + 2 * heads), st(heads, D, V)
        al, nw = torch.zeros(heads, device=dev), torch.ones(V, device=dev)
        ms = timed(lambda i: ops.gated_delta(qkv[i], rest[i][:, heads * V:heads * V + heads], rest[i][:, heads * V + heads:],
                                             rest[i][:, :heads * V], al, al, nw, 1e-6, dstate[i], step, heads, G, D, V), n_sets)
        rows.append(("gated delta rule (3 kernels)", point, ms,
                     N * (cols + 2 * heads * V + 2 * heads) * 2 + N * (2 * G * D + heads * V + 2 * heads) * 8 + B * heads * D * V * 8))
        # LFM2's short convolution at the same width (3 taps, gates B and C): the like kernel of the closest model
        bcx, sstate = rnd(N, 3 * W), st(2, W)
        sw = torch.randn(W, 3, device=dev) * 0.1
        ms = timed(lambda i: ops.short_conv(bcx[i], sw, None, sstate[i], step, 3), n_sets)
        rows.append(("LFM2 short convolution", point, ms, N * 4 * W * 2 + B * 2 * W * 8))
    return [{"kernel": k, "point": p, "width": width, "us": round(ms * 1e3, 2), "MB": round(b / 1e6, 3),
             "GB_per_s": round(b / ms / 1e6, 1), "frac_of_copy_peak": round(b / ms / 1e6 / hbm_peak, 4)} for k, p, ms, b in rows]


def run_vunolorn(args):
    """Prefill and decode throughput of the Vunolorn hybrid at two widths beside the LFM2 shape of the same width,
    layer count and vocabulary; the time of a prefill and of a decode step by kernel class; and the recurrent
    kernels alone against the copy bandwidth.  JSON lines, then markdown tables."""
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    hbm_peak, flops_peak, peak_src = peaks()
    rows, classes, kernels = [], [], []
    for width, lfm2 in ((1024, "350m"), (2048, "1.2b")):
        for label, cfg_dict in ((f"Vunolorn-{width}", vunolorn_config(width)), (f"LFM2-{lfm2.upper()}", shape_config(lfm2))):
            cfg = config_from_dict(cfg_dict)
            with tempfile.TemporaryDirectory(prefix="bench_hybrid_") as d:
                z.write_random_model(cfg, 0, d)
                eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048 + 64, max_model_len=CONTEXT,
                               max_tokens=64 * CONTEXT, page_size=args.page_size)
                nums = engine_numbers(eng)
                prefill_ms = time_prefill(eng, reps=5)
                T = PREFILL_TOKENS
                rows.append({"model": label, "width": width, "matrix_params_M": round(nums["matrix_params"] / 1e6, 1),
                             "point": "prefill 2048", "ms": round(prefill_ms, 3), "tokens_per_s": round(T / prefill_ms * 1e3),
                             "matrix_TFLOP_per_s": round(2 * T * nums["matrix_params"] / prefill_ms / 1e9, 1)})
                print(json.dumps(rows[-1]), flush=True)
                for B in (1, 8, 64):
                    dev_ms, e2e_ms, ctx_tokens, launches, _, _, _ = time_decode(eng, B, max(min(args.steps, 100), 20), args.warmup)
                    step_bytes = 2 * nums["matrix_params"] + ctx_tokens * nums["kv_bytes_per_token"] + 2 * B * nums["state_bytes"]
                    rows.append({"model": label, "width": width, "point": f"decode batch {B}", "ms": round(dev_ms, 4),
                                 "e2e_ms": round(e2e_ms, 4), "tokens_per_s": round(B / dev_ms * 1e3),
                                 "e2e_tokens_per_s": round(B / e2e_ms * 1e3), "GB_a_step": round(step_bytes / 1e9, 3),
                                 "frac_of_copy_peak": round(step_bytes / (dev_ms * 1e-3) / 1e9 / hbm_peak, 3),
                                 "launches_per_step": round(launches)})
                    print(json.dumps(rows[-1]), flush=True)
                g = random.Random(5)
                V = eng.config.vocab_size
                eng.flush()
                pre = kernel_classes(eng, [("kc", [g.randrange(V) for _ in range(T)], [T - 1])])
                dec = kernel_classes(eng, [(f"kc{i}", [g.randrange(V)], [0]) for i in range(64)])
                classes.append({"model": label, "prefill_2048_ms_by_class": pre, "decode_64_first_token_ms_by_class": dec})
                print(json.dumps(classes[-1]), flush=True)
                del eng
                torch.cuda.empty_cache()
        kernels += recurrent_kernel_rooflines(width, hbm_peak)
    for r in kernels:
        print(json.dumps(r), flush=True)
    print(f"\npeaks ({peak_src}): {hbm_peak:.0f} GB/s copy bandwidth, {flops_peak:.0f} TFLOP/s bf16 product (burst)\n")
    print("| model | point | ms a step (device) | tokens/s (device) | tokens/s (end to end) | of the copy peak |")
    print("|---|---|---|---|---|---|")
    for r in rows:
        print(f"| {r['model']} | {r['point']} | {r['ms']} | {r['tokens_per_s']} | {r.get('e2e_tokens_per_s', '')} | {r.get('frac_of_copy_peak', '')} |")
    print("\n| kernel | point | width | us | MB | GB/s | of the copy peak |")
    print("|---|---|---|---|---|---|---|")
    for r in kernels:
        print(f"| {r['kernel']} | {r['point']} | {r['width']} | {r['us']} | {r['MB']} | {r['GB_per_s']} | {r['frac_of_copy_peak']} |")
    return 0


# ----------------------------------------------------------------------------- the Pikasun design beside LFM2
def pikasun_config(width, layers=16, vocab=65536, ff=None):
    """A Pikasun model of a real model's proportions: groups of four layers (attention inside chunks of 1024
    positions with a quarter as many key/value heads as query heads; a latent layer of rank 256 with a rotated part
    of 32; a latent layer that reads the one before; another latent layer of its own), head size 64 throughout, a
    gated feed-forward behind every layer."""
    heads = width // 64
    ff = ff or 3 * width
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    stretched = {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    latent = lambda src: {"type": "latent_attention", "mlp": dict(mlp),
                          "mixer": dict({"heads": heads, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 256, "scale": 96 ** -0.5,
                                         "rot": dict(stretched)}, **({} if src is None else {"kv_from": src}))}
    out = []
    for i in range(layers):
        if i % 4 == 0:
            out.append({"type": "attention", "mlp": dict(mlp),
                        "mixer": {"heads": heads, "kv_heads": max(heads // 4, 1), "dim": 64, "vdim": 64, "scale": 0.125,
                                  "rot": {"base": 1000000.0, "dims": 64}, "mask": {"size": 1024}}})
        else:
            out.append(latent(i - 1 if i % 4 == 2 else None))
    return {"architecture": "Pikasun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "logit_softcap": 30.0, "layers": out}


def pikasun_kernel_rooflines(width, hbm_peak, flops_peak):
    """The attention kernels of the design alone at the sizes of `pikasun_config(width)`, beside the like kernel of
    LFM2 at the same width (grouped-query attention, head size 64): a portion of 2048 tokens and 64 single tokens over
    contexts of 2048.  Latent attention against the tensor peak (its keys are read once per row and group of heads from
    the L2 cache; the products decide) and, for single tokens, against the copy bandwidth (the cached rows decide)."""
    import torch
    from zig_ai_b200.cache.manager import CacheView
    from zig_ai_b200.engine.batch import pack_step
    from zig_ai_b200.kernels import ops
    ops.require(torch.bfloat16, ("latent_attention", "qkv_prepare", "layernorm"))
    dev, dt = torch.device("cuda"), torch.bfloat16
    H, G, R, Dr, ps = width // 64, max(width // 256, 1), 256, 32, 64
    g = torch.Generator().manual_seed(1)
    rows = []

    def step_of(ctx, q_lens):
        spans, tables, at = [], [], 1
        width_pages = max(-(-(c + n) // ps) for c, n in zip(ctx, q_lens))
        for s_, (c, n) in enumerate(zip(ctx, q_lens)):
            need = -(-(c + n) // ps)
            tables.append(list(range(at, at + need)) + [0] * (width_pages - need))
            at += need
            spans.append((s_, c, [0] * n, [], s_ + 1))
        return pack_step(ops, dt, dev, spans, {0: tables}), at

    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        total = 0.0
        for _ in range(reps):
            flush.zero_()                                    # larger than L2: the timed call starts cold
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / reps

    for point, ctx, q_lens in (("2048-token portion", [0], [2048]), ("64 single tokens, context 2048", [2047] * 64, [1] * 64)):
        step, n_pages = step_of(ctx, q_lens)
        N = sum(q_lens)
        keys = sum((c + n) * n - n * (n - 1) // 2 for c, n in zip(ctx, q_lens))           # (query, key) pairs
        cached = sum(c + n for c, n in zip(ctx, q_lens))
        lat_pages = (torch.randn(n_pages, ps, R + Dr, generator=g) * 0.3).to(dt).to(dev)
        view = CacheView(0, lat_pages, step.block_tables[0], ps)
        q_lat = torch.randn(N, H, R, generator=g).to(dt).to(dev)
        q_rot = torch.randn(N, H, Dr, generator=g).to(dt).to(dev)
        for label, impl in (("latent attention (tensor cores)", None), ("latent attention (general kernel)", "general")):
            if impl == "general" and N > 64:
                continue
            ms = timed(lambda: ops.latent_attention(q_lat, q_rot, step, view, H, R, Dr, 0.1, impl=impl), 10)
            rows.append((label, point, ms, 2.0 * keys * H * (2 * R + Dr), cached * (R + Dr) * 2 + N * H * (2 * R + Dr) * 2))
        kv_pages = (torch.randn(n_pages, 2, G, ps, 64, generator=g) * 0.3).to(dt).to(dev)
        kview = CacheView(0, kv_pages, step.block_tables[0], ps)
        q = torch.randn(N, H * 64, generator=g).to(dt).to(dev)
        for label, chunk in (("grouped-query attention (LFM2's kernel)", None), ("the same inside chunks of 1024", 1024)):
            ms = timed(lambda: ops.paged_attention(q, step, kview, H, G, 64, 0.125, None, chunk=chunk), 10)
            pairs = keys if chunk is None else sum(min(p % chunk + 1, p + 1) for c, n in zip(ctx, q_lens) for p in range(c, c + n))
            rows.append((label, point, ms, 4.0 * pairs * H * 64, cached * 2 * G * 64 * 2 + 2 * N * H * 64 * 2))
        h = torch.randn(N, width, generator=g).to(dev)
        delta = torch.randn(N, width, generator=g).to(dt).to(dev)
        w, b = torch.ones(width, device=dev), torch.zeros(width, device=dev)
        rows.append(("layer norm + residual", point, timed(lambda: ops.add_layernorm(h, delta, w, b, 1e-6, dt)), 0.0, N * width * 12))
        rows.append(("RMS norm + residual (LFM2's kernel)", point, timed(lambda: ops.add_rmsnorm(h, delta, w, 1e-6, dt)), 0.0, N * width * 12))
    return [{"kernel": k, "point": p, "width": width, "us": round(ms * 1e3, 2), "GFLOP": round(fl / 1e9, 2), "MB": round(by / 1e6, 2),
             "TFLOP_per_s": round(fl / ms / 1e9, 1), "of_tensor_peak": round(fl / ms / 1e9 / flops_peak, 4),
             "GB_per_s": round(by / ms / 1e6, 1), "of_copy_peak": round(by / ms / 1e6 / hbm_peak, 4)} for k, p, ms, fl, by in rows]


def run_pikasun(args):
    """Prefill and decode throughput of the Pikasun design at two widths beside the LFM2 shape of the same width,
    layer count and vocabulary; the time of a prefill and of a decode step by kernel class; and its attention and norm
    kernels alone beside LFM2's.  JSON lines, then markdown tables."""
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    hbm_peak, flops_peak, peak_src = peaks()
    rows, classes, kernels = [], [], []
    for width, lfm2 in ((1024, "350m"), (2048, "1.2b")):
        for label, cfg_dict in ((f"Pikasun-{width}", pikasun_config(width)), (f"LFM2-{lfm2.upper()}", shape_config(lfm2))):
            cfg = config_from_dict(cfg_dict)
            with tempfile.TemporaryDirectory(prefix="bench_pikasun_") as d:
                z.write_random_model(cfg, 0, d)
                eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048 + 64, max_model_len=CONTEXT,
                               max_tokens=64 * CONTEXT, page_size=args.page_size)
                nums = engine_numbers(eng)
                prefill_ms = time_prefill(eng, reps=5)
                T = PREFILL_TOKENS
                rows.append({"model": label, "width": width, "matrix_params_M": round(nums["matrix_params"] / 1e6, 1),
                             "point": "prefill 2048", "ms": round(prefill_ms, 3), "tokens_per_s": round(T / prefill_ms * 1e3),
                             "matrix_TFLOP_per_s": round(2 * T * nums["matrix_params"] / prefill_ms / 1e9, 1)})
                print(json.dumps(rows[-1]), flush=True)
                for B in (1, 8, 64):
                    dev_ms, e2e_ms, ctx_tokens, launches, _, _, _ = time_decode(eng, B, max(min(args.steps, 100), 20), args.warmup)
                    step_bytes = 2 * nums["matrix_params"] + ctx_tokens * nums["kv_bytes_per_token"] + 2 * B * nums["state_bytes"]
                    rows.append({"model": label, "width": width, "point": f"decode batch {B}", "ms": round(dev_ms, 4),
                                 "e2e_ms": round(e2e_ms, 4), "tokens_per_s": round(B / dev_ms * 1e3),
                                 "e2e_tokens_per_s": round(B / e2e_ms * 1e3), "GB_a_step": round(step_bytes / 1e9, 3),
                                 "frac_of_copy_peak": round(step_bytes / (dev_ms * 1e-3) / 1e9 / hbm_peak, 3),
                                 "launches_per_step": round(launches)})
                    print(json.dumps(rows[-1]), flush=True)
                g = random.Random(5)
                V = eng.config.vocab_size
                eng.flush()
                pre = kernel_classes(eng, [("kc", [g.randrange(V) for _ in range(T)], [T - 1])])
                dec = kernel_classes(eng, [(f"kc{i}", [g.randrange(V)], [0]) for i in range(64)])
                classes.append({"model": label, "prefill_2048_ms_by_class": pre, "decode_64_first_token_ms_by_class": dec})
                print(json.dumps(classes[-1]), flush=True)
                del eng
                torch.cuda.empty_cache()
        kernels += pikasun_kernel_rooflines(width, hbm_peak, flops_peak)
    for r in kernels:
        print(json.dumps(r), flush=True)
    print(f"\npeaks ({peak_src}): {hbm_peak:.0f} GB/s copy bandwidth, {flops_peak:.0f} TFLOP/s bf16 product (burst)\n")
    print("| model | point | ms a step (device) | tokens/s (device) | tokens/s (end to end) | of the copy peak | launches a step |")
    print("|---|---|---|---|---|---|---|")
    for r in rows:
        print(f"| {r['model']} | {r['point']} | {r['ms']} | {r['tokens_per_s']} | {r.get('e2e_tokens_per_s', '')} | "
              f"{r.get('frac_of_copy_peak', '')} | {r.get('launches_per_step', '')} |")
    print("\n| kernel | point | width | us | GFLOP | TFLOP/s | of the tensor peak | MB | GB/s | of the copy peak |")
    print("|---|---|---|---|---|---|---|---|---|---|")
    for r in kernels:
        print(f"| {r['kernel']} | {r['point']} | {r['width']} | {r['us']} | {r['GFLOP']} | {r['TFLOP_per_s']} | {r['of_tensor_peak']} | "
              f"{r['MB']} | {r['GB_per_s']} | {r['of_copy_peak']} |")
    return 0


# ----------------------------------------------------------------------------- the Zikevik design beside Pikasun
def zikevik_config(width, layers=16, vocab=65536):
    """A Zikevik model of a real model's proportions: groups of four layers (a delta rule with a decay per key channel in
    front of a dense feed-forward; latent attention in front of eight experts of which a token uses two; latent attention
    in front of a dense feed-forward; the delta rule in front of the experts).  Head size 64, value heads of 128 in the
    delta rule, latents of rank 256 for keys/values and 384 for queries, a rotated part of 32.  A token's two experts hold
    as many parameters as the dense feed-forward of three times the width."""
    heads = width // 64
    dense = {"kind": "dense", "ff": 3 * width}
    moe = {"kind": "moe", "expert": {"ff": 3 * width // 2}, "router": {"experts": 8, "top": 2}}
    delta = {"heads": heads, "kv_heads": heads // 2, "dim": 64, "vdim": 128, "conv": 4, "decay_rank": width // 16, "gate_rank": width // 8}
    latent = {"heads": heads, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 256, "q_rank": 384, "scale": 96 ** -0.5,
              "rot": {"base": 10000.0, "dims": 32}}
    group = [("channel_delta", delta, dense), ("latent_attention", latent, moe), ("latent_attention", latent, dense),
             ("channel_delta", delta, moe)]
    return {"architecture": "Zikevik", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": [{"type": t, "mixer": dict(m), "mlp": dict(f)} for t, m, f in (group[i % 4] for i in range(layers))]}


def zikevik_kernel_rooflines(width, hbm_peak, flops_peak):
    """Every kernel that the design adds, alone at the sizes of `zikevik_config(width)`, beside the like kernel of the
    closest existing design at the same sizes: the delta rule with a decay per key channel beside the one with a decay
    per head (Vunolorn's); latent attention with a sink beside the one without (Pikasun's); the routed experts beside a
    dense gated feed-forward with a token's share of their parameters; the norm of activation rows beside the residual
    norm.  A portion of 2048 tokens and 64 single tokens (over contexts of 2048 where there is one), timed with CUDA
    events, the L2 flushed before every call."""
    import torch
    from zig_ai_b200.cache.manager import CacheView
    from zig_ai_b200.engine.batch import pack_step
    from zig_ai_b200.kernels import ops
    ops.require(torch.bfloat16, ("latent_attention", "qkv_prepare", "causal_conv", "gated_delta", "moe"))
    dev, dt = torch.device("cuda"), torch.bfloat16
    H, G, D, V, R, Dr, Rq, ps = width // 64, width // 128, 64, 128, 256, 32, 384, 64
    E, top, F = 8, 2, 3 * width // 2
    g = torch.Generator().manual_seed(1)
    rnd = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).to(dt).to(dev)
    rows = []

    def step_of(ctx, q_lens):
        spans, tables, at = [], [], 1
        width_pages = max(-(-(c + n) // ps) for c, n in zip(ctx, q_lens))
        for s_, (c, n) in enumerate(zip(ctx, q_lens)):
            need = -(-(c + n) // ps)
            tables.append(list(range(at, at + need)) + [0] * (width_pages - need))
            at += need
            spans.append((s_, c, [0] * n, [], s_ + 1))
        return pack_step(ops, dt, dev, spans, {0: tables}), at

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        total = 0.0
        for _ in range(reps):
            flush.zero_()                                    # larger than L2: the timed call starts cold
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / reps

    for point, ctx, q_lens in (("2048-token portion", [0], [2048]), ("64 single tokens, context 2048", [2047] * 64, [1] * 64)):
        step, n_pages = step_of(ctx, q_lens)
        N, B = sum(q_lens), len(q_lens)
        # the delta rule: norms and gates, the recurrence, the output norm
        cols = 2 * G * D + H * V
        qkv, gate, b = rnd(N, cols), rnd(N, H * V), rnd(N, H)
        a_ch, a_hd = rnd(N, H * D), rnd(N, H)
        state = torch.zeros(B + 1, H, D, V, device=dev)
        al, nw = torch.zeros(H, device=dev), torch.ones(V, device=dev)
        by = N * (cols + 2 * H * V + H) * 2 + B * H * D * V * 8
        ms = timed(lambda: ops.gated_delta(qkv, b, a_ch, gate, al, torch.zeros(H * D, device=dev), nw, 1e-6, state, step, H, G, D, V,
                                           channel_decay=True, gate_act="sigmoid"))
        rows.append(("delta rule, a decay per key channel", point, ms, 0.0, by + N * H * D * 2))
        ms = timed(lambda: ops.gated_delta(qkv, b, a_hd, gate, al, torch.zeros(H, device=dev), nw, 1e-6, state, step, H, G, D, V))
        rows.append(("delta rule, a decay per head (Vunolorn's)", point, ms, 0.0, by + N * H * 2))
        # latent attention
        keys = sum((c + n) * n - n * (n - 1) // 2 for c, n in zip(ctx, q_lens))           # (query, key) pairs
        cached = sum(c + n for c, n in zip(ctx, q_lens))
        view = CacheView(0, rnd(n_pages, ps, R + Dr, s=0.3), step.block_tables[0], ps)
        q_lat, q_rot, sink = rnd(N, H, R), rnd(N, H, Dr), torch.zeros(H, device=dev)
        fl, by = 2.0 * keys * H * (2 * R + Dr), cached * (R + Dr) * 2 + N * H * (2 * R + Dr) * 2
        for label, sk in (("latent attention with a sink", sink), ("latent attention (Pikasun's)", None)):
            rows.append((label, point, timed(lambda: ops.latent_attention(q_lat, q_rot, step, view, H, R, Dr, 0.1, sink=sk)), fl, by))
        # the feed-forwards
        x = rnd(N, width)
        w_router = (torch.randn(E, width, generator=g) * 0.05).to(dev)
        w_gu, w_dn = rnd(E, 2 * F, width, s=0.02), rnd(E, width, F, s=0.02)
        used = min(E, N * top)
        rows.append((f"routed experts ({top} of {E})", point, timed(lambda: ops.routed_experts(x, w_router, w_gu, w_dn, top)),
                     2.0 * N * top * 3 * width * F, used * 3 * width * F * 2 + N * width * 4))
        d_gu, d_dn = rnd(2 * top * F, width, s=0.02), rnd(width, top * F, s=0.02)
        rows.append(("dense gated feed-forward of a token's share", point,
                     timed(lambda: ops.linear(ops.linear_swiglu(x, d_gu, top * F), d_dn)), 2.0 * N * 3 * width * top * F,
                     3 * width * top * F * 2 + N * width * 4))
        # norms
        y = rnd(N, Rq + H + R + Dr + 8)
        wq = torch.ones(Rq, device=dev)
        rows.append(("norm of activation rows (the query latent)", point, timed(lambda: ops.rmsnorm_rows(y[:, :Rq], wq, 1e-6)), 0.0, N * Rq * 4))
        h, delta_ = torch.randn(N, width, generator=g).to(dev), rnd(N, width)
        w1 = torch.ones(width, device=dev)
        rows.append(("RMS norm + residual (shared with LFM2)", point, timed(lambda: ops.add_rmsnorm(h, delta_, w1, 1e-6, dt)), 0.0, N * width * 12))
    return [{"kernel": k, "point": p, "width": width, "us": round(ms * 1e3, 2), "GFLOP": round(fl / 1e9, 2), "MB": round(by / 1e6, 2),
             "TFLOP_per_s": round(fl / ms / 1e9, 1), "of_tensor_peak": round(fl / ms / 1e9 / flops_peak, 4),
             "GB_per_s": round(by / ms / 1e6, 1), "of_copy_peak": round(by / ms / 1e6 / hbm_peak, 4)} for k, p, ms, fl, by in rows]


def run_zikevik(args):
    """Prefill and decode throughput of the Zikevik design at two widths beside the Pikasun design (the closest one:
    latent attention in front of gated feed-forwards) of the same width, layer count and vocabulary; the time of a prefill
    and of a decode step by kernel class; and its kernels alone beside the like kernels.  JSON lines, then markdown."""
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    hbm_peak, flops_peak, peak_src = peaks()
    rows, classes, kernels = [], [], []
    for width in (1024, 2048):
        for label, cfg_dict in ((f"Zikevik-{width}", zikevik_config(width)), (f"Pikasun-{width}", pikasun_config(width))):
            cfg = config_from_dict(cfg_dict)
            with tempfile.TemporaryDirectory(prefix="bench_zikevik_") as d:
                z.write_random_model(cfg, 0, d)
                eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048 + 64, max_model_len=CONTEXT,
                               max_tokens=64 * CONTEXT, page_size=args.page_size)
                nums = engine_numbers(eng)
                active = params_read(nums, 1)
                prefill_ms = time_prefill(eng, reps=5)
                T = PREFILL_TOKENS
                rows.append({"model": label, "width": width, "matrix_params_M": round(nums["matrix_params"] / 1e6, 1),
                             "active_params_M": round(active / 1e6, 1), "point": "prefill 2048", "ms": round(prefill_ms, 3),
                             "tokens_per_s": round(T / prefill_ms * 1e3),
                             "matrix_TFLOP_per_s": round(2 * T * active / prefill_ms / 1e9, 1)})
                print(json.dumps(rows[-1]), flush=True)
                for B in (1, 8, 64):
                    dev_ms, e2e_ms, ctx_tokens, launches, _, _, _ = time_decode(eng, B, max(min(args.steps, 100), 20), args.warmup)
                    read = params_read(nums, B)       # of the experts, a step reads those that its tokens chose
                    step_bytes = 2 * read + ctx_tokens * nums["kv_bytes_per_token"] + 2 * B * nums["state_bytes"]
                    rows.append({"model": label, "width": width, "point": f"decode batch {B}", "ms": round(dev_ms, 4),
                                 "e2e_ms": round(e2e_ms, 4), "tokens_per_s": round(B / dev_ms * 1e3),
                                 "e2e_tokens_per_s": round(B / e2e_ms * 1e3), "GB_a_step": round(step_bytes / 1e9, 3),
                                 "frac_of_copy_peak": round(step_bytes / (dev_ms * 1e-3) / 1e9 / hbm_peak, 3),
                                 "launches_per_step": round(launches)})
                    print(json.dumps(rows[-1]), flush=True)
                g = random.Random(5)
                V = eng.config.vocab_size
                eng.flush()
                pre = kernel_classes(eng, [("kc", [g.randrange(V) for _ in range(T)], [T - 1])])
                dec = kernel_classes(eng, [(f"kc{i}", [g.randrange(V)], [0]) for i in range(64)])
                classes.append({"model": label, "prefill_2048_ms_by_class": pre, "decode_64_first_token_ms_by_class": dec})
                print(json.dumps(classes[-1]), flush=True)
                del eng
                torch.cuda.empty_cache()
        kernels += zikevik_kernel_rooflines(width, hbm_peak, flops_peak)
    for r in kernels:
        print(json.dumps(r), flush=True)
    print(f"\npeaks ({peak_src}): {hbm_peak:.0f} GB/s copy bandwidth, {flops_peak:.0f} TFLOP/s bf16 product (burst)\n")
    print("| model | point | ms a step (device) | tokens/s (device) | tokens/s (end to end) | of the copy peak | launches a step |")
    print("|---|---|---|---|---|---|---|")
    for r in rows:
        print(f"| {r['model']} | {r['point']} | {r['ms']} | {r['tokens_per_s']} | {r.get('e2e_tokens_per_s', '')} | "
              f"{r.get('frac_of_copy_peak', '')} | {r.get('launches_per_step', '')} |")
    print("\n| kernel | point | width | us | GFLOP | TFLOP/s | of the tensor peak | MB | GB/s | of the copy peak |")
    print("|---|---|---|---|---|---|---|---|---|---|")
    for r in kernels:
        print(f"| {r['kernel']} | {r['point']} | {r['width']} | {r['us']} | {r['GFLOP']} | {r['TFLOP_per_s']} | {r['of_tensor_peak']} | "
              f"{r['MB']} | {r['GB_per_s']} | {r['of_copy_peak']} |")
    return 0


def lolivik_config(width, layers=16, vocab=65536):
    """A Lolivik model of a real model's proportions: groups of four layers (attention with shaped scores in front of a dense
    gated feed-forward; a matrix memory in front of eight bounded experts of which a token uses two, with a shared unit;
    windowed attention that keeps its first positions in front of the experts; a matrix memory in front of the dense
    feed-forward).  Head size 64 (values too), four query heads a key/value head, a window of 1024, bias tables of 32 rows."""
    heads = width // 64
    dense = {"kind": "dense", "ff": 3 * width}
    moe = {"kind": "moe", "expert": {"ff": width, "limit": 7.0}, "router": {"experts": 8, "top": 2}, "shared": {"ff": width, "limit": 7.0}}
    att = {"heads": heads, "kv_heads": heads // 4, "dim": 64, "vdim": 64, "scale": 0.125, "softcap": 30.0, "bias_rows": 32,
           "bias_max": 4096, "q_temp": {"coef": 0.1, "every": 1024}, "v_mix": True}
    win = {"heads": heads, "kv_heads": heads // 4, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": 1024, "keep_first": 4},
           "rot": {"base": 5e5, "dims": 32, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 8192}}, "v_mix": True}
    mem = {"heads": heads // 2, "dim": 64, "vdim": 128, "gate_cap": 12.0}
    group = [("attention", att, dense), ("mlstm", mem, moe), ("attention_2", win, moe), ("mlstm", mem, dense)]
    return {"architecture": "Lolivik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "layers": [{"type": t, "mixer": dict(m), "mlp": dict(f)} for t, m, f in (group[i % 4] for i in range(layers))]}


def lolivik_kernel_rooflines(width, hbm_peak, flops_peak):
    """Every kernel that the design adds, alone at the sizes of `lolivik_config(width)`, beside the like kernel of an
    existing design at the same sizes: attention with capped scores, a bias by distance and a sink, and windowed attention
    with kept first positions, each beside plain grouped-query attention (LFM2's); the matrix memory beside the delta rule
    with a decay per head (Vunolorn's, Zikevik's); the experts with softmax scores and bounded units beside those with
    sigmoid scores and SiLU units (Zikevik's); the tanh-GELU gate beside the SiLU gate; the residual addition that rounds
    the stream beside the one that norms it.  A portion of 2048 tokens and 64 single tokens over contexts of 2048, timed with
    CUDA events, the L2 flushed before every call."""
    import torch
    from zig_ai_b200.cache.manager import CacheView
    from zig_ai_b200.engine.batch import pack_step
    from zig_ai_b200.kernels import ops
    ops.require(torch.bfloat16, ("attention", "attention_mma", "attention_tma", "attention_tc", "qkv_prepare", "mlstm", "causal_conv",
                                 "gated_delta", "moe", "gemm_tc"))
    dev, dt = torch.device("cuda"), torch.bfloat16
    H, G, D, ps = width // 64, width // 256, 64, 64
    Hm, Dm, Vm = width // 128, 64, 128
    E, top, F = 8, 2, width
    g = torch.Generator().manual_seed(1)
    rnd = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).to(dt).to(dev)
    rows = []

    def step_of(ctx, q_lens):
        spans, tables, at = [], [], 1
        width_pages = max(-(-(c + n) // ps) for c, n in zip(ctx, q_lens))
        for s_, (c, n) in enumerate(zip(ctx, q_lens)):
            need = -(-(c + n) // ps)
            tables.append(list(range(at, at + need)) + [0] * (width_pages - need))
            at += need
            spans.append((s_, c, [0] * n, [], s_ + 1))
        return pack_step(ops, dt, dev, spans, {0: tables}), at

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        total = 0.0
        for _ in range(reps):
            flush.zero_()                                    # larger than L2: the timed call starts cold
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / reps

    for point, ctx, q_lens in (("2048-token portion", [0], [2048]), ("64 single tokens, context 2048", [2047] * 64, [1] * 64)):
        step, n_pages = step_of(ctx, q_lens)
        N, B = sum(q_lens), len(q_lens)
        # attention: (query, key) pairs seen with and without the window
        pairs = lambda w: sum(sum(min(c + i + 1, w) for i in range(n)) for c, n in zip(ctx, q_lens))
        cached = sum(c + n for c, n in zip(ctx, q_lens))
        view = CacheView(0, rnd(n_pages, 2, G, ps, D, s=0.5), step.block_tables[0], ps)
        q = rnd(N, H * D)
        bias, sink = (torch.randn(700, H, generator=g) * 0.5).to(dev), torch.zeros(H, device=dev)
        by = cached * 2 * G * D * 2 + 2 * N * H * D * 2
        full, win = 4.0 * pairs(1 << 30) * H * D, 4.0 * pairs(1024) * H * D
        rows.append(("attention: capped scores, bias by distance, sink", point,
                     timed(lambda: ops.paged_attention(q, step, view, H, G, D, 0.125, softcap=30.0, bias=bias, sink=sink)), full, by))
        rows.append(("grouped-query attention (LFM2's)", point, timed(lambda: ops.paged_attention(q, step, view, H, G, D, 0.125)), full, by))
        if N > B:       # (spans: the same work on the span kernel of the generation before, which is the one that shapes scores)
            rows.append(("grouped-query attention, the mma.sync span kernel", point,
                         timed(lambda: ops.paged_attention(q, step, view, H, G, D, 0.125, impl="mma")), full, by))
        rows.append(("windowed attention, first positions kept", point,
                     timed(lambda: ops.paged_attention(q, step, view, H, G, D, 0.125, 1024, keep_first=4)), win, by))
        rows.append(("windowed attention (LFM2's kernels)", point, timed(lambda: ops.paged_attention(q, step, view, H, G, D, 0.125, 1024)), win, by))
        # the matrix memory beside the delta rule at the same heads and sizes
        at, cols = [], 0
        for n in (Hm * Dm, Hm * Dm, Hm * Vm, Hm * Vm, Hm, Hm):
            at.append(cols)
            cols += -(-n // 8) * 8
        y = rnd(N, cols)
        zeros_h, nw = torch.zeros(Hm, device=dev), torch.ones(Hm * Vm, device=dev)
        state = torch.zeros(B + 1, Hm, Dm + 1, Vm + 1, device=dev)
        by = N * (cols + Hm * Vm) * 2 + B * Hm * Dm * Vm * 8
        rows.append(("matrix memory with log gates", point,
                     timed(lambda: ops.mlstm(y, at, zeros_h, zeros_h, 15.0, nw, 1e-6, state, step, Hm, Dm, Vm)), 0.0, by))
        qkv, gate, b_, a_hd = rnd(N, 2 * Hm * Dm + Hm * Vm), rnd(N, Hm * Vm), rnd(N, Hm), rnd(N, Hm)
        dstate = torch.zeros(B + 1, Hm, Dm, Vm, device=dev)
        rows.append(("delta rule, a decay per head (Vunolorn's)", point,
                     timed(lambda: ops.gated_delta(qkv, b_, a_hd, gate, zeros_h, zeros_h, torch.ones(Vm, device=dev), 1e-6, dstate, step,
                                                   Hm, Hm, Dm, Vm)), 0.0, by))
        # the feed-forwards
        x = rnd(N, width)
        w_router = (torch.randn(E, width, generator=g) * 0.05).to(dev)
        w_gu, w_dn = rnd(E, 2 * F, width, s=0.02), rnd(E, width, F, s=0.02)
        used = min(E, N * top)
        fl, by = 2.0 * N * top * 3 * width * F, used * 3 * width * F * 2 + N * width * 4
        rows.append((f"routed experts, softmax scores, bounded units ({top} of {E})", point,
                     timed(lambda: ops.routed_experts(x, w_router, w_gu, w_dn, top, True, "output", score="softmax", act="clamped",
                                                      limit=7.0, alpha=1.702)), fl, by))
        rows.append((f"routed experts, sigmoid scores, SiLU units (Zikevik's)", point,
                     timed(lambda: ops.routed_experts(x, w_router, w_gu, w_dn, top)), fl, by))
        d_gu, d_dn = rnd(2 * 3 * width, width, s=0.02), rnd(width, 3 * width, s=0.02)
        fl, by = 2.0 * N * 3 * width * 3 * width, 3 * width * 3 * width * 2 + N * width * 4
        rows.append(("dense gated feed-forward, tanh GELU", point,
                     timed(lambda: ops.linear(ops.linear_glu(x, d_gu, 3 * width, "gelu_tanh"), d_dn)), fl, by))
        rows.append(("dense gated feed-forward, SiLU (LFM2's)", point,
                     timed(lambda: ops.linear(ops.linear_swiglu(x, d_gu, 3 * width), d_dn)), fl, by))
        # the residual addition
        h, delta_ = torch.randn(N, width, generator=g).to(dev), rnd(N, width)
        w1 = torch.ones(width, device=dev)
        rows.append(("residual + normed term, stream rounded", point, timed(lambda: ops.add_cast(h, delta_, dt, w1, 1e-6)), 0.0, N * width * 12))
        rows.append(("RMS norm + residual (shared with LFM2)", point, timed(lambda: ops.add_rmsnorm(h, delta_, w1, 1e-6, dt)), 0.0, N * width * 12))
    return [{"kernel": k, "point": p, "width": width, "us": round(ms * 1e3, 2), "GFLOP": round(fl / 1e9, 2), "MB": round(by / 1e6, 2),
             "TFLOP_per_s": round(fl / ms / 1e9, 1), "of_tensor_peak": round(fl / ms / 1e9 / flops_peak, 4),
             "GB_per_s": round(by / ms / 1e6, 1), "of_copy_peak": round(by / ms / 1e6 / hbm_peak, 4)} for k, p, ms, fl, by in rows]


def run_lolivik(args):
    """Prefill and decode throughput of the Lolivik design at two widths beside the Zikevik design (the closest one: a
    recurrent mixer and attention with a sink in front of dense feed-forwards and routed experts) of the same width, layer
    count and vocabulary; the time of a prefill and of a decode step by kernel class; and its kernels alone beside the like
    kernels.  JSON lines, then markdown."""
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    hbm_peak, flops_peak, peak_src = peaks()
    rows, classes, kernels = [], [], []
    for width in (1024, 2048):
        for label, cfg_dict in ((f"Lolivik-{width}", lolivik_config(width)), (f"Zikevik-{width}", zikevik_config(width))):
            cfg = config_from_dict(cfg_dict)
            with tempfile.TemporaryDirectory(prefix="bench_lolivik_") as d:
                z.write_random_model(cfg, 0, d)
                eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048 + 64, max_model_len=CONTEXT,
                               max_tokens=64 * CONTEXT, page_size=args.page_size)
                nums = engine_numbers(eng)
                active = params_read(nums, 1)
                prefill_ms = time_prefill(eng, reps=5)
                T = PREFILL_TOKENS
                rows.append({"model": label, "width": width, "matrix_params_M": round(nums["matrix_params"] / 1e6, 1),
                             "active_params_M": round(active / 1e6, 1), "point": "prefill 2048", "ms": round(prefill_ms, 3),
                             "tokens_per_s": round(T / prefill_ms * 1e3),
                             "matrix_TFLOP_per_s": round(2 * T * active / prefill_ms / 1e9, 1)})
                print(json.dumps(rows[-1]), flush=True)
                for B in (1, 8, 64):
                    dev_ms, e2e_ms, ctx_tokens, launches, _, _, _ = time_decode(eng, B, max(min(args.steps, 100), 20), args.warmup)
                    read = params_read(nums, B)       # of the experts, a step reads those that its tokens chose
                    step_bytes = 2 * read + ctx_tokens * nums["kv_bytes_per_token"] + 2 * B * nums["state_bytes"]
                    rows.append({"model": label, "width": width, "point": f"decode batch {B}", "ms": round(dev_ms, 4),
                                 "e2e_ms": round(e2e_ms, 4), "tokens_per_s": round(B / dev_ms * 1e3),
                                 "e2e_tokens_per_s": round(B / e2e_ms * 1e3), "GB_a_step": round(step_bytes / 1e9, 3),
                                 "frac_of_copy_peak": round(step_bytes / (dev_ms * 1e-3) / 1e9 / hbm_peak, 3),
                                 "launches_per_step": round(launches)})
                    print(json.dumps(rows[-1]), flush=True)
                g = random.Random(5)
                V = eng.config.vocab_size
                eng.flush()
                pre = kernel_classes(eng, [("kc", [g.randrange(V) for _ in range(T)], [T - 1])])
                dec = kernel_classes(eng, [(f"kc{i}", [g.randrange(V)], [0]) for i in range(64)])
                classes.append({"model": label, "prefill_2048_ms_by_class": pre, "decode_64_first_token_ms_by_class": dec})
                print(json.dumps(classes[-1]), flush=True)
                del eng
                torch.cuda.empty_cache()
        kernels += lolivik_kernel_rooflines(width, hbm_peak, flops_peak)
    for r in kernels:
        print(json.dumps(r), flush=True)
    print(f"\npeaks ({peak_src}): {hbm_peak:.0f} GB/s copy bandwidth, {flops_peak:.0f} TFLOP/s bf16 product (burst)\n")
    print("| model | point | ms a step (device) | tokens/s (device) | tokens/s (end to end) | of the copy peak | launches a step |")
    print("|---|---|---|---|---|---|---|")
    for r in rows:
        print(f"| {r['model']} | {r['point']} | {r['ms']} | {r['tokens_per_s']} | {r.get('e2e_tokens_per_s', '')} | "
              f"{r.get('frac_of_copy_peak', '')} | {r.get('launches_per_step', '')} |")
    print("\n| kernel | point | width | us | GFLOP | TFLOP/s | of the tensor peak | MB | GB/s | of the copy peak |")
    print("|---|---|---|---|---|---|---|---|---|---|")
    for r in kernels:
        print(f"| {r['kernel']} | {r['point']} | {r['width']} | {r['us']} | {r['GFLOP']} | {r['TFLOP_per_s']} | {r['of_tensor_peak']} | "
              f"{r['MB']} | {r['GB_per_s']} | {r['of_copy_peak']} |")
    return 0


def run_table(args):
    """The tracked table: the 350M, 700M and 1.2B shapes, decode at batch 1/8/64 device-timed and end to end,
    the prefill of 2048 tokens, and the mixed workload of the 700M shape, as JSON lines and as markdown."""
    hbm_peak, flops_peak, peak_src = peaks()
    all_rows = []
    for model in ("350m", "700m", "1.2b"):
        rows, _ = measure_shape(model, args.steps, args.warmup, args.page_size)
        for r in rows:
            print(json.dumps(r), flush=True)
        all_rows += rows
    print(f"\npeaks ({peak_src}): {hbm_peak:.0f} GB/s copy bandwidth, {flops_peak:.0f} TFLOP/s bf16 product (burst)\n")
    print("| shape | point | ms a step (device) | tokens/s (device) | ms a step (end to end) | tokens/s (end to end) | bytes or flops a step | achieved | of the measured peak |")
    print("|---|---|---|---|---|---|---|---|---|")
    for r in all_rows:
        print(f"| LFM2-{r['model'].upper()} | {r['point']} | {r['ms']} | {r['tokens_per_s']} | {r.get('e2e_ms', '')} | "
              f"{r.get('e2e_tokens_per_s', '')} | {r['work']} | {r['achieved']} | {r['frac_of_peak']} |")
    return 0


def run_long(args):
    """Further context lengths (one shape, --model): a prompt of --context tokens prefilled in portions of 2048
    (each portion timed: its products are the same, its attention grows with the cached context), and decode
    steps at batch 8 with contexts spread over the upper half of --context."""
    global CONTEXT
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    hbm_peak, flops_peak, peak_src = peaks()
    cfg = config_from_dict(shape_config(args.model))
    nums = model_numbers(cfg)
    CONTEXT = args.context
    B = 8
    with tempfile.TemporaryDirectory(prefix="lfm2_long_") as d:
        z.write_random_model(cfg, 0, d)
        eng = z.Engine(d, "bfloat16", max_num_seqs=B, max_batched_tokens=2048 + 64, max_model_len=CONTEXT,
                       max_tokens=(B + 1) * CONTEXT, page_size=args.page_size)
        runner = eng.runner
        g = random.Random(5)
        Hq, D = nums["attn_dims"]
        T = PREFILL_TOKENS
        for rep in range(2):                                   # the first pass warms up (graphs of the portions' shapes are captured)
            rid = f"long{rep}"
            runner.add_request(rid)
            portions = []
            for c in range(CONTEXT // T):
                toks = [g.randrange(cfg.vocab_size) for _ in range(T)]
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                start.record()
                runner.step([(rid, toks, [T - 1])])
                stop.record()
                torch.cuda.synchronize()
                portions.append(start.elapsed_time(stop))
            runner.end_request(rid)
        total_ms = sum(portions)
        # flops: every portion's products, and attention of its 2048 rows over the cached context and itself
        products = 2 * T * nums["layer_params"] + 2 * nums["head_params"]
        attn = [nums["n_attn"] * 2 * 2 * Hq * D * (T * c * T + T * T // 2) for c in range(CONTEXT // T)]
        flops = len(portions) * products + sum(attn)
        print(json.dumps({"only": "long", "model": args.model, "point": f"prefill {CONTEXT} in portions of {T}",
                          "ms": round(total_ms, 2), "tokens_per_s": round(CONTEXT / total_ms * 1e3),
                          "first_portion_ms": round(portions[0], 3), "last_portion_ms": round(portions[-1], 3),
                          "tflop": round(flops / 1e12, 2), "achieved_tflops": round(flops / total_ms / 1e9),
                          "frac_of_peak": round(flops / (total_ms * 1e-3) / (flops_peak * 1e12), 3),
                          "last_portion_attention_share_of_flops": round(attn[-1] / (products + attn[-1]), 3),
                          "last_portion_frac_of_peak": round((products + attn[-1]) / (portions[-1] * 1e-3) / (flops_peak * 1e12), 3),
                          "peaks": peak_src}), flush=True)
        weight_bytes = 2 * (nums["layer_params"] + nums["head_params"])
        dev_ms, e2e_ms, ctx_tokens, launches, _, _, _ = time_decode(eng, B, max(args.steps, 20), args.warmup)
        step_bytes = weight_bytes + ctx_tokens * nums["kv_bytes_per_token"] + B * nums["state_bytes"]
        print(json.dumps({"only": "long", "model": args.model, "point": f"decode batch {B}", "mean_context": round(ctx_tokens / B),
                          "ms": round(dev_ms, 4), "e2e_ms": round(e2e_ms, 4), "tokens_per_s": round(B / dev_ms * 1e3),
                          "e2e_tokens_per_s": round(B / e2e_ms * 1e3), "gb": round(step_bytes / 1e9, 3),
                          "achieved_gbs": round(step_bytes / dev_ms / 1e6),
                          "frac_of_peak": round(step_bytes / (dev_ms * 1e-3) / 1e9 / hbm_peak, 3), "peaks": peak_src}), flush=True)
    return 0


def run_sample(args):
    """Sampling: the kernel alone at the shape's vocabulary (1, 8 and 64 rows; twenty eager calls, so about 13 us
    of each figure are the launch), and decode steps through Engine.step() with sampled requests."""
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    from zig_ai_b200.kernels import ops
    from zig_ai_b200.sampling import SamplingParams
    cfg = config_from_dict(shape_config(args.model))
    V = cfg.vocab_size
    ops.require(torch.bfloat16)
    kinds = (("temperature 0.8", 0, 1.0), ("top-k 40", 40, 1.0), ("top-p 0.9", 0, 0.9), ("top-k 40, top-p 0.9", 40, 0.9))
    for R in (1, 8, 64):
        logits = torch.randn(R, V, device="cuda") * 3
        row = {"only": "sample", "rows": R, "vocab": V}
        for name, tk, tp in kinds:
            t = torch.full((R,), 0.8, device="cuda")
            k = torch.full((R,), tk, dtype=torch.int32, device="cuda")
            p = torch.full((R,), tp, device="cuda")
            u = torch.rand(R, device="cuda")
            for _ in range(3):
                ops.sample(logits, t, k, p, u)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(20):
                ops.sample(logits, t, k, p, u)
            b.record()
            torch.cuda.synchronize()
            row[name + " us"] = round(a.elapsed_time(b) * 50, 1)
        print(json.dumps(row), flush=True)
    g = random.Random(3)
    with tempfile.TemporaryDirectory(prefix="lfm2_sample_") as d:
        z.write_random_model(cfg, 0, d)
        for name, sp in (("greedy", dict(temperature=0.0)), ("temperature 0.8", dict(temperature=0.8)),
                         ("temperature 0.8, top-k 40, top-p 0.9", dict(temperature=0.8, top_k=40, top_p=0.9)),
                         ("and repetition penalty 1.1", dict(temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.1))):
            eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048 + 64, max_model_len=CONTEXT, max_tokens=64 * CONTEXT)
            row = {"only": "sample", "requests": name}
            for B in (8, 64):
                ids = [eng.add_request([g.randrange(V) for _ in range(2048 + 20 * i)], SamplingParams(max_new_tokens=300, seed=i, **sp))
                       for i in range(B)]
                while any(eng.requests[i].computed < len(eng.requests[i].prompt) or not eng.requests[i].output for i in ids):
                    eng.step()
                for _ in range(20):
                    eng.step()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(100):
                    eng.step()
                torch.cuda.synchronize()
                row[f"ms a step at batch {B}"] = round((time.perf_counter() - t0) * 10, 4)
                while eng.has_work():
                    eng.step()
            print(json.dumps(row), flush=True)
            del eng
    return 0


def run_timeline(eng, B):
    """One decode step's kernels on the device's own clock (libraries built with ZAI_TIMELINE=1): when
    each kernel's first block was resident and waiting, when its wait for the kernel before it ended,
    and how long until the next kernel's wait ended (its share of the step)."""
    import collections
    from zig_ai_b200.kernels import ops
    ids = decode_requests(eng, B, 40, seed=B)
    eng.flush()
    reqs = [eng.requests[i] for i in ids]
    runner = eng.runner
    prepared = [runner.prepare_decode([(r.request_id, [(7 * k + j) % 1000], [0]) for j, r in enumerate(reqs)])
                for k in range(12)]
    for k in range(10):
        ops.argmax(runner.run_prepared(prepared[k]))
    ops.timeline()
    for k in range(10, 12):
        ops.argmax(runner.run_prepared(prepared[k]))
    tl = [r for r in ops.timeline() if " mark " not in r[0] and " block " not in r[0]]
    starts = [i for i, r in enumerate(tl) if r[0] == "embed_kernel"]
    step = tl[starts[-1]:]
    t0 = step[0][2]
    print(f"batch {B}: {len(step)} kernels, {(step[-1][2] - t0) / 1e3:.1f} us from the first kernel's start to the last one's")
    print("  # kernel                                   resident at   wait over   waited   until next (us)")
    agg = collections.OrderedDict()
    for i, (name, a, b) in enumerate(step):
        nxt = step[i + 1][2] if i + 1 < len(step) else b
        print(f"{i:3d} {name:40s} {(a - t0) / 1e3:10.2f} {(b - t0) / 1e3:11.2f} {(b - a) / 1e3:8.2f} {(nxt - b) / 1e3:8.2f}")
        e = agg.setdefault(name, [0, 0.0])
        e[0] += 1
        e[1] += (nxt - b) / 1e3
    print("by kernel (launches, us in the step, us each):")
    for name, (n, us) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        print(f"  {name:40s} {n:3d} {us:8.1f} {us / n:7.2f}")
    return 0


def run_gemm_table(cfg):
    """The products of the model's layers at 2048, 512 and 128 rows: the tcgen05 kernel of this package
    against the library's product (plus the activation kernel where the tcgen05 kernel fuses it), each
    timed as a CUDA graph of 20 calls that rotate over copies of the weights (so they come from HBM)."""
    import ctypes
    import torch
    from zig_ai_b200.kernels import ops
    ops.require()
    fn = ops._fn("gemm_tc", "zai_gemm_tc")
    fn2 = ops._fn("gemm_tc_pair", "zai_gemm_pair")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    H, F = cfg.hidden_size, cfg.ff_dim
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    shapes = [("out_proj", H, H, 0), ("qkv", qkv, H, 0), ("in_proj", 3 * H, H, 0), ("gate_up+swiglu", 2 * F, H, 2), ("down", H, F, 0)]

    def graph_time(f, reps=20):
        for _ in range(2):
            f()
        torch.cuda.synchronize()
        g, s = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(s):
            with torch.cuda.graph(g):
                ops.begin_forward()
                for _ in range(reps):
                    f()
                ops.end_forward()
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (5 * reps) * 1e3

    rows = []
    for N in (2048, 512, 128):
        for name, O, K, epi in shapes:
            ws = [torch.randn(O, K).to(torch.bfloat16).cuda() for _ in range(max(2, min(8, int(200e6 // (O * K * 2)))))]
            x = torch.randn(N, K).to(torch.bfloat16).cuda()
            y = torch.empty((N, O // 2 if epi == 2 else O), dtype=torch.bfloat16, device="cuda")
            it = [0]

            def tc():
                w = ws[it[0] % len(ws)]
                it[0] += 1
                fn(y.data_ptr(), w.data_ptr(), x.data_ptr(), status.data_ptr(), N, O, K, epi, ops._stream())

            def lib():
                w = ws[it[0] % len(ws)]
                it[0] += 1
                if epi == 2:
                    ops.silu_mul(torch.matmul(x, w.t()), O // 2)
                else:
                    torch.matmul(x, w.t())
            def pair(wide):
                def f():
                    w = ws[it[0] % len(ws)]
                    it[0] += 1
                    fn2(y.data_ptr(), w.data_ptr(), x.data_ptr(), status.data_ptr(), N, O, K, epi, wide, ops._stream())
                return f
            t, t2 = graph_time(tc), graph_time(lib)
            tw, tn = graph_time(pair(1)), graph_time(pair(0))
            tp = min(tw, tn)
            rows.append({"rows": N, "product": name, "O": O, "K": K, "pair_us": round(tp, 1), "pair_wide_us": round(tw, 1),
                         "pair_narrow_us": round(tn, 1), "pair_tflops": round(2 * N * O * K / tp / 1e6),
                         "tcgen05_us": round(t, 1),
                         "tcgen05_tflops": round(2 * N * O * K / t / 1e6), "library_us": round(t2, 1),
                         "library_tflops": round(2 * N * O * K / t2 / 1e6)})
            print(json.dumps(rows[-1]))
    print(json.dumps({"only": "gemm", "status": int(status.item())}))
    return 0


def run_stream_table(cfg, only_rows=0):
    """The products of a layer at 24, 64 and 128 rows: the weight-streaming tcgen05 kernel of this package
    (csrc/stream_gemm.cu, with SwiGLU fused where the layer has it) against the library's product (plus the
    activation kernel), each timed as a CUDA graph of 20 calls that rotate over copies of the weights."""
    import torch
    from zig_ai_b200.kernels import ops
    ops.require()
    ops.USE_STREAM_GEMM = True
    H, F = cfg.hidden_size, cfg.ff_dim
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    shapes = [("out_proj", H, H, 0), ("qkv", qkv, H, 0), ("in_proj", 3 * H, H, 0), ("gate_up+swiglu", 2 * F, H, 2), ("down", H, F, 0),
              ("head", cfg.vocab_size, H, 1)]

    def graph_time(f, reps=20):
        for _ in range(2):
            f()
        torch.cuda.synchronize()
        g, s = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(s):
            with torch.cuda.graph(g):
                ops.begin_forward()
                for _ in range(reps):
                    f()
                ops.end_forward()
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (5 * reps) * 1e3

    for N in ((only_rows,) if only_rows in (24, 64, 128) else (24, 64, 128)):
        for name, O, K, epi in shapes:
            ws = [torch.randn(O, K).to(torch.bfloat16).cuda() for _ in range(max(2, min(8, int(300e6 // (O * K * 2)))))]
            x = torch.randn(N, K).to(torch.bfloat16).cuda()
            it = [0]

            def mine():
                w = ws[it[0] % len(ws)]
                it[0] += 1
                if epi == 2:
                    ops.linear_swiglu(x, w, O // 2)
                else:
                    ops.linear(x, w, torch.float32 if epi == 1 else None)

            def lib():
                w = ws[it[0] % len(ws)]
                it[0] += 1
                if epi == 2:
                    ops.silu_mul(torch.matmul(x, w.t()), O // 2)
                elif epi == 1:
                    torch.mm(x, w.t(), out_dtype=torch.float32)
                else:
                    torch.matmul(x, w.t())
            t1, t2 = graph_time(mine), graph_time(lib)
            print(json.dumps({"rows": N, "product": name, "O": O, "K": K, "stream_us": round(t1, 2), "library_us": round(t2, 2),
                              "stream_GBs": round(O * K * 2 / t1 / 1e3)}), flush=True)
    print(json.dumps({"only": "stream", "status": ops.read_status()}))
    return 0


def run_mixed(args, cfg):
    """64 requests with prompts of 256..2048 random tokens and 256 new tokens each, chunked prefill
    interleaved with decoding, through Engine.step(): tokens per second end to end."""
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.sampling import SamplingParams
    g = random.Random(7)
    with tempfile.TemporaryDirectory(prefix="lfm2_mixed_") as d:
        z.write_random_model(cfg, 0, d)
        eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048, max_model_len=CONTEXT,
                       max_tokens=64 * 2560)
        V = cfg.vocab_size
        for rep in range(2):                       # the first pass warms up graphs and allocator
            prompts = [[g.randrange(V) for _ in range(g.randint(256, 2048))] for _ in range(64)]
            ids = [eng.add_request(p, SamplingParams(temperature=0.0, max_new_tokens=256)) for p in prompts]
            torch.cuda.synchronize()
            t0, steps0, done = time.perf_counter(), eng.n_steps, 0
            while done < len(ids):
                done += len(eng.step())
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        n_prompt = sum(len(p) for p in prompts)
        st = eng.stats()
    out = {"metric": f"mixed workload tok/s (LFM2-{args.model.upper()} shape, 64 requests, prompts 256-2048, 256 new tokens each)",
           "value": round(64 * 256 / dt, 1), "unit": "generated tokens/s", "n_gpus": 1, "seconds": round(dt, 3),
           "prompt_tokens": n_prompt, "prompt_tokens_per_s": round(n_prompt / dt, 1), "steps": eng.n_steps - steps0,
           "mean_step_ms": round(dt * 1e3 / max(eng.n_steps - steps0, 1), 3),
           "pages_high_water": max(v for k, v in st.items() if k.endswith("pages_high_water")),
           "preemptions": st["preemptions"], "step_graph_replays": eng.runner.shape_graphs.replays,
           "step_graphs_kept": len(eng.runner.shape_graphs.graphs), "dtype": "bf16", "data": "synthetic", "impl": "ours"}
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "gemm", "timeline", "table", "stream", "long", "sample", "vunolorn", "pikasun", "zikevik", "lolivik"],
                    help="profiling aid: run only the batch-8 decode steps or only the prefill (prints a short line); "
                         "table: every figure of the 350M, 700M and 1.2B shapes (profiles/measurements.md); pikasun: the Pikasun design beside LFM2 at equal width; zikevik: the Zikevik design beside Pikasun at equal width, and its kernels beside the like ones; lolivik: the Lolivik design beside Zikevik at equal width, and its kernels beside the like ones; vunolorn: the "
                         "Vunolorn hybrid at two widths beside LFM2 at equal width, and its recurrent kernels alone")
    ap.add_argument("--batch", type=int, default=8, help="with --only decode: the batch size; with --only stream: 24, 64 or "
                                                         "128 runs that row count only")
    ap.add_argument("--profile-range", action="store_true",
                    help="mark the device-timed decode steps for a profiler (ncu --profile-from-start off)")
    ap.add_argument("--page-size", type=int, default=64, help="positions per cache page")
    ap.add_argument("--context", type=int, default=32768, help="with --only long: the context length (a multiple of 2048)")
    ap.add_argument("--model", default="350m", choices=sorted(SHAPES), help="which LFM2 shape (default: the 350M shape)")
    ap.add_argument("--workload", default="steps", choices=["steps", "mixed"],
                    help="mixed: 64 requests, chunked prefill interleaved with decoding, end to end")
    args = ap.parse_args()
    global PROFILE_RANGE
    PROFILE_RANGE = args.profile_range
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Zig 0.16 program (build.zig); no Zig compiler exists in this image and it "
                          "has no Python package to install, and it publishes no LFM2 figures"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    args.warmup = max(args.warmup, 3)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
