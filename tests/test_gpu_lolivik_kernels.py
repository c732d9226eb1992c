"""The kernels and kernel options that the Lolivik design adds, each alone against its plain PyTorch version
(tests/ref_ops.py), in 32-bit and in bfloat16: the residual addition of a normed term with the stream's rounding; the
queries' temperature and the mixed values in the q/k/v preparation; attention with capped scores, a bias by distance, a
sink and kept first positions under a window (spans beside single tokens; planted keys just inside and outside the
window and the kept positions; a sink that takes nearly everything); the matrix memory with log gates (spans beside
single tokens, a second step that continues from the first one's state, an input gate that jumps); the routed experts
with softmax scores and bounded units; the gated activation with other activations than SiLU."""
import pytest
import torch

import ref_ops
from test_gpu_kernels import fill_pages, make_step, plant_key
from test_gpu_recurrent_kernels import MANY_SINGLES, STEPS
from zig_ai_b200.cache.manager import CacheView

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from zig_ai_b200.kernels import ops as o
    o.require(extra=("attention", "qkv_prepare", "mlstm", "moe", "gemm_tc"))
    return o


def tol(dtype):
    return dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,H", [(5, 96), (3, 1000), (70, 1024), (1, 66), (513, 2050)])
def test_add_cast(dtype, N, H):
    o = ops()
    g = torch.Generator().manual_seed(2)
    h = (torch.randn(N, H, generator=g) * 3).cuda()
    delta = torch.randn(N, H, generator=g).to(dtype).cuda()
    gamma = (0.3 * (1 + 0.1 * torch.randn(H, generator=g))).cuda()
    for d, gm in ((None, None), (delta, None), (delta, gamma)):
        ha, hb = h.clone(), h.clone()
        a = o.add_cast(ha, d, dtype, gm, 1e-5)
        b = ref_ops.add_cast(hb, d, dtype, gm, 1e-5)
        assert a.dtype == dtype and torch.allclose(ha, hb, atol=2e-6, rtol=2e-6)
        assert torch.allclose(a.float(), b.float(), **tol(dtype))
        assert torch.equal(a, ha.to(dtype))                       # the output is the updated stream, rounded once


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,Dv,scope,rot,ps", [(4, 2, 16, 8, 2, 0, 8), (3, 1, 24, 40, 1, 8, 16), (8, 1, 64, 32, 2, 0, 64), (6, 3, 12, 12, 1, 12, 4)])
def test_qkv_prepare_temperature_and_mixed_values(dtype, H, G, D, Dv, scope, rot, ps):
    o = ops()
    g = torch.Generator().manual_seed(3)
    Dp = max(D, Dv)
    ctx, q_lens = [0, 5, 126, 300], [9, 1, 4, 1]
    num_pages = 128
    step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 4)
    N = sum(q_lens)
    y = torch.randn(N, (H + G) * D + G * Dv + 8, generator=g).to(dtype).cuda()
    first_wide = torch.randn(N, G * Dv + 16, generator=g).to(dtype).cuda()
    first = first_wide[:, 8:8 + G * Dv]                            # a column slice, as a layer leaves it
    lam = torch.tensor([0.35]).cuda()
    nq = H * D if scope == 2 else D
    nk = G * D if scope == 2 else D
    qw, kw = (1 + 0.1 * torch.randn(nq, generator=g)).cuda(), (1 + 0.1 * torch.randn(nk, generator=g)).cuda()
    table = None
    if rot:
        ang = torch.randn(N, rot // 2, generator=g)
        table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).cuda()
    for temp, vf in (((0.3, 4), None), (None, first), ((0.25, 128), first), ((0.5, 1), None)):
        pa = torch.zeros(num_pages, 2, G, ps, Dp, dtype=dtype).cuda()
        pb = pa.clone()
        kw_more = dict(temp=temp, v_first=vf, v_lambda=lam if vf is not None else None)
        a = o.qkv_prepare(y, qw, kw, 1e-5, scope, table, rot, step, CacheView(0, pa, step.block_tables[0], ps), H, G, D, Dv, Dp, True, **kw_more)
        b = ref_ops.qkv_prepare(y, qw, kw, 1e-5, scope, table, rot, step, CacheView(0, pb, step.block_tables[0], ps), H, G, D, Dv, Dp, True, **kw_more)
        assert torch.allclose(a.float(), b.float(), **tol(dtype)), (temp, vf is not None)
        assert torch.allclose(pa.float(), pb.float(), **tol(dtype)), (temp, vf is not None)
        plain = ref_ops.qkv_prepare(y, qw, kw, 1e-5, scope, table, rot, step, CacheView(0, pb.clone(), step.block_tables[0], ps), H, G, D, Dv, Dp, True)
        if temp and temp[1] < 100:
            assert (a.float() - plain.float()).abs().max() > 0.05    # the temperature counts at these positions
    assert o.read_status() == 0


def distance_bias(rows, H, g):
    return (torch.randn(rows, H, generator=g) * 1.5).cuda()


SCORED = [(4, 2, 16, 16), (3, 1, 32, 8), (8, 1, 64, 64), (6, 3, 48, 4), (2, 2, 96, 16), (5, 5, 80, 32)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,ps", SCORED)
def test_attention_with_shaped_scores(dtype, Hq, Hkv, D, ps):
    """Spans that start at 0, inside a page and far into a request beside single tokens; every option alone and all together."""
    o = ops()
    g = torch.Generator().manual_seed(8)
    bias, sink = distance_bias(37, Hq, g), (torch.randn(Hq, generator=g) * 2).cuda()
    # (the third step: nine decoding requests in front of two portions, of which eight go to the kernel for single tokens)
    for ctx, q_lens in (([0, ps - 1, 2 * ps, 301, 5, 63], [150, 2, 1, 1, 37, 66]), ([0, 1, 254, 255, 256, 700, 63, 1029], [1] * 8),
                        ([3, 70, 0, 129, 64, 300, 31, 32, 5, 0, 200], [1] * 9 + [70, 131])):
        num_pages = sum(-(-(c + n) // ps) for c, n in zip(ctx, q_lens)) + 8
        step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 9)
        pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, num_pages, g)
        q = torch.randn(sum(q_lens), Hq * D, generator=g).to(dtype).cuda()
        view = CacheView(0, pages, step.block_tables[0], ps)
        base = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5)
        for opts in (dict(softcap=1.5), dict(bias=bias), dict(sink=sink), dict(window=40, keep_first=3), dict(window=7, keep_first=70),
                     dict(window=100, keep_first=0, sink=sink), dict(softcap=2.0, bias=bias, sink=sink),
                     dict(softcap=2.0, bias=bias, sink=sink, window=33, keep_first=5)):
            b = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, **opts)
            for impl in (None, "general"):                           # (bfloat16: the tensor-core kernels, then the general one)
                a = o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, impl=impl, **opts)
                assert torch.allclose(a.float(), b.float(), **tol(dtype)), (q_lens[:3], sorted(opts), impl)
            assert (b.float() - base.float()).abs().max() > 0.02, sorted(opts)     # the option counts
    assert o.read_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edges_and_kept_positions_with_planted_keys(dtype):
    """One key that the query matches sits just inside the window, just outside it, at the last kept position and at the
    first one that is not kept: the row's output is that key's value exactly when the key is visible, for a row of a
    span and for a single token, with pages of 8 (all four places inside pages and at page borders)."""
    o = ops()
    g = torch.Generator().manual_seed(12)
    Hq, Hkv, D, ps, window, keep = 2, 1, 32, 8, 24, 5
    key = torch.randn(D, generator=g)
    key = key / key.norm() * 8.0
    value = torch.full((D,), 3.0)
    for ctx, q_lens in (([200], [1]), ([150], [51])):
        pos = ctx[0] + q_lens[0] - 1                                # the last row's position
        for at, seen in ((pos - window + 1, True), (pos - window, False), (keep - 1, True), (keep, False), (0, True), (pos, True)):
            num_pages = 64
            step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 13)
            pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, num_pages, g)
            pages[:, 0] *= 0.05                                     # all other keys nearly orthogonal to everything
            plant_key(pages, step, ps, 0, at, 0, key, value)
            q = (torch.randn(sum(q_lens), Hq * D, generator=g) * 0.1).to(dtype).cuda()
            q[-1] = key.repeat(Hq).to(dtype).cuda()
            view = CacheView(0, pages, step.block_tables[0], ps)
            b = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, 1.0, window, keep_first=keep)
            for impl in (None, "general"):
                a = o.paged_attention(q, step, view, Hq, Hkv, D, 1.0, window, keep_first=keep, impl=impl)
                assert torch.allclose(a.float(), b.float(), **tol(dtype)), (q_lens, at, impl)
                assert bool((a[-1].float() - 3.0).abs().max() < 0.05) == seen, (q_lens, at, seen, impl)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_large_sink_takes_the_weight_and_a_small_one_none(dtype):
    o = ops()
    g = torch.Generator().manual_seed(14)
    Hq, Hkv, D, ps = 3, 1, 16, 8
    ctx, q_lens = [0, 90], [20, 1]
    step = make_step(o, dtype, ctx, q_lens, ps, 64, 15)
    pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, 64, g)
    q = torch.randn(sum(q_lens), Hq * D, generator=g).to(dtype).cuda()
    view = CacheView(0, pages, step.block_tables[0], ps)
    plain = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, 0.25)
    for impl in (None, "general"):
        big = o.paged_attention(q, step, view, Hq, Hkv, D, 0.25, sink=torch.tensor([40.0, -40.0, 40.0]).cuda(), impl=impl)
        big = big.float().reshape(-1, Hq, D)
        assert big[:, 0].abs().max() < 1e-3 and big[:, 2].abs().max() < 1e-3
        assert torch.allclose(big[:, 1], plain.float().reshape(-1, Hq, D)[:, 1], **tol(dtype))


def mlstm_columns(H, D, V):
    """Column offsets of a stacked projection q | k | v | gate | i | f, every part on a multiple of eight columns."""
    at, out = 0, []
    for n in (H * D, H * D, H * V, H * V, H, H):
        out.append(at)
        at += -(-n // 8) * 8
    return out, at


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,V", [(2, 32, 64), (3, 10, 14), (4, 64, 64), (1, 128, 40), (2, 16, 130), (5, 12, 12), (1, 200, 31), (2, 33, 31)])
def test_mlstm(dtype, H, D, V):
    o = ops()
    g = torch.Generator().manual_seed(8)
    at, cols = mlstm_columns(H, D, V)
    bias_i, bias_f = (torch.randn(H, generator=g) - 1.0).cuda(), (torch.randn(H, generator=g) + 3.0).cuda()
    norm_w = (1 + 0.1 * torch.randn(H * V, generator=g)).cuda()
    state_a = torch.zeros(22, H, D + 1, V + 1).cuda()
    state_b = state_a.clone()
    for q_lens in STEPS + (MANY_SINGLES,):
        step = make_step(o, dtype, [3] * len(q_lens), q_lens, 8, 256, 5)
        N = sum(q_lens)
        y = torch.randn(N, cols, generator=g)
        y[:, at[4]:at[4] + H] *= 4.0                                   # input gates that jump by several units
        y = y.to(dtype).cuda()
        ya = o.mlstm(y, at, bias_i, bias_f, 11.0, norm_w, 1e-5, state_a, step, H, D, V, True)
        # the exact answer: the recurrence in 64-bit (per-head norms of read-outs with cancelling terms carry the 32-bit
        # sums' rounding of long rows, so the 32-bit kernel is held to 2e-4 of it)
        yb = ref_ops.mlstm(y, at, bias_i, bias_f, 11.0, norm_w, 1e-5, state_b, step, H, D, V, True, precision=torch.float64)
        limit = dict(atol=2e-4, rtol=2e-4) if dtype == torch.float32 else tol(dtype)
        assert torch.allclose(ya.float(), yb.float(), **limit), (q_lens, float((ya.float() - yb.float()).abs().max()))
        assert torch.allclose(state_a, state_b, atol=1e-4, rtol=1e-4), q_lens
    keep = state_a.clone()
    o.mlstm(y, at, bias_i, bias_f, 11.0, norm_w, 1e-5, state_a, step, H, D, V, False)      # write_state off: the state stays
    assert torch.equal(state_a, keep)
    assert o.read_status() == 0


def expert_tensors(g, E, F, W, dtype):
    w_router = (torch.randn(E, W, generator=g) * 0.3).cuda()
    w_gate_up = (torch.randn(E, 2 * F, W, generator=g) * W ** -0.5 * 2).to(dtype).cuda()
    w_down = (torch.randn(E, W, F, generator=g) * F ** -0.5).to(dtype).cuda()
    return w_router, w_gate_up, w_down


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,W,F,E,top", [(1, 64, 32, 4, 2), (7, 48, 24, 5, 5), (40, 128, 96, 8, 4), (300, 128, 64, 8, 2), (700, 256, 128, 8, 4),
                                         (16, 66, 20, 3, 1), (2000, 128, 128, 4, 2)])
def test_routed_experts_softmax_scores_bounded_units(dtype, N, W, F, E, top):
    o = ops()
    g = torch.Generator().manual_seed(17)
    w_router, w_gate_up, w_down = expert_tensors(g, E, F, W, dtype)
    x = torch.randn(N, W, generator=g).to(dtype).cuda()
    kw = dict(score="softmax", act="clamped", limit=1.2, alpha=1.702)
    a = o.routed_experts(x, w_router, w_gate_up, w_down, top, True, "output", **kw)
    b = ref_ops.routed_experts(x, w_router, w_gate_up, w_down, top, True, "output", **kw)
    # a row whose scores around the cut lie closer together than the router's rounding may go to another expert in the two versions
    z = (x.float() @ w_router.t()).sort(dim=-1, descending=True).values
    sure = torch.ones(N, dtype=torch.bool, device="cuda") if top == E else (z[:, top - 1] - z[:, top]) > 1e-3
    assert int(sure.sum()) >= N - max(2, N // 100)
    assert torch.allclose(a.float()[sure], b.float()[sure], **tol(dtype))
    unbounded = ref_ops.routed_experts(x, w_router, w_gate_up, w_down, top, True, "output", score="softmax", act="clamped", limit=50.0)
    assert (unbounded.float() - b.float()).abs().max() > 0.05            # the bound counts
    assert o.read_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["gelu_tanh", "gelu", "relu", "silu"])
def test_gated_activation(dtype, kind):
    o = ops()
    g = torch.Generator().manual_seed(21)
    gu = (torch.randn(37, 2 * 72, generator=g) * 2).to(dtype).cuda()
    assert torch.allclose(o.act_mul(gu, 72, kind).float(), ref_ops.act_mul(gu, 72, kind).float(), **tol(dtype))
    for rows, K, F in ((37, 40, 72), (5, 256, 128), (16, 1024, 384), (1, 128, 64)):      # (few rows in bfloat16: the product's epilogue)
        x = torch.randn(rows, K, generator=g).to(dtype).cuda()
        w = (torch.randn(2 * F, K, generator=g) * K ** -0.5).to(dtype).cuda()
        assert torch.allclose(o.linear_glu(x, w, F, kind).float(), ref_ops.linear_glu(x, w, F, kind).float(), **tol(dtype)), (rows, K, F)
