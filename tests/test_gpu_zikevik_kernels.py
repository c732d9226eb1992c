"""The kernels and kernel options that the Zikevik design adds, each alone against its plain PyTorch version
(tests/ref_ops.py), in 32-bit and in bfloat16: the delta rule with one decay per head and key channel and a sigmoid
output gate (spans beside single tokens, a second step that continues from the first one's state, fewer query/key
heads than heads and as many); latent attention with a sink in the softmax's denominator (every kernel variant; a sink
that takes nearly everything, one that takes nothing, the first token alone with it); the norm of activation rows in a
column slice; the routed experts (one expert a row, several, all; the score on the input or on the output, divided by
the scores' sum or not; few rows and many; a row's result whatever else the step holds)."""
import pytest
import torch

import ref_ops
from test_gpu_kernels import make_step
from test_gpu_pikasun_kernels import latent_pages
from test_gpu_recurrent_kernels import MANY_SINGLES, STEPS
from zig_ai_b200.cache.manager import CacheView

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from zig_ai_b200.kernels import ops as o
    o.require(extra=("causal_conv", "gated_delta", "latent_attention", "qkv_prepare", "moe", "gemm_tc"))
    return o


def tol(dtype):
    return dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("gate_act", ["sigmoid", "silu"])
@pytest.mark.parametrize("H,G,D,V", [(6, 2, 32, 40), (2, 2, 16, 24), (3, 1, 40, 33), (4, 2, 64, 128), (2, 1, 128, 48),
                                     (1, 1, 200, 20), (2, 1, 8, 70), (5, 5, 12, 12)])
def test_gated_delta_with_a_decay_per_key_channel(dtype, gate_act, H, G, D, V):
    o = ops()
    g = torch.Generator().manual_seed(8)
    a_log = torch.randn(H, generator=g).cuda() * 0.5
    dt_bias = torch.randn(H * D, generator=g).cuda() * 0.5
    norm_w = (1 + 0.1 * torch.randn(V, generator=g)).cuda()
    state_a = (torch.randn(22, H, D, V, generator=g) * 0.3).cuda()
    state_b = state_a.clone()
    cols = 2 * G * D + H * V
    for q_lens in STEPS + (MANY_SINGLES,):
        step = make_step(o, dtype, [3] * len(q_lens), q_lens, 8, 256, 5)
        N = sum(q_lens)
        qkv = torch.randn(N, cols, generator=g).to(dtype).cuda()
        rest = torch.randn(N, H * V + H + 3, generator=g).to(dtype).cuda()
        gate, b = rest[:, :H * V], rest[:, H * V:H * V + H]
        a = (torch.randn(N, H * D, generator=g) * 2).to(dtype).cuda()          # decays from nearly 0 to nearly 1 within a head
        ya = o.gated_delta(qkv, b, a, gate, a_log, dt_bias, norm_w, 1e-5, state_a, step, H, G, D, V, True,
                           channel_decay=True, gate_act=gate_act)
        yb = ref_ops.gated_delta(qkv, b, a, gate, a_log, dt_bias, norm_w, 1e-5, state_b, step, H, G, D, V, True,
                                 channel_decay=True, gate_act=gate_act)
        assert torch.allclose(ya.float(), yb.float(), **tol(dtype)), q_lens
        assert torch.allclose(state_a, state_b, atol=1e-4, rtol=1e-4), q_lens
    keep = state_a.clone()
    o.gated_delta(qkv, b, a, gate, a_log, dt_bias, norm_w, 1e-5, state_a, step, H, G, D, V, False, channel_decay=True,
                  gate_act=gate_act)                                            # write_state off: the state stays
    assert torch.equal(state_a, keep) and torch.equal(state_a[0], state_b[0])


def test_one_channels_decay_touches_that_row_of_the_state_alone():
    """One key channel of one head forgets everything (a large decay input), the others keep everything: after a step
    with no write (beta 0) the state has that row at zero and every other row as it was."""
    o = ops()
    dtype, H, G, D, V = torch.float32, 3, 1, 16, 8
    g = torch.Generator().manual_seed(9)
    state = torch.randn(4, H, D, V, generator=g).cuda()
    before = state.clone()
    step = make_step(o, dtype, [5], [1], 8, 16, 5)
    qkv = torch.randn(1, 2 * G * D + H * V, generator=g).cuda()
    b = torch.full((1, H), -80.0).cuda()                                        # beta = 0: nothing is written
    a = torch.full((1, H * D), -80.0).cuda()                                    # softplus = 0: decay 1
    a[0, 1 * D + 5] = 80.0                                                      # head 1, key channel 5: decay exp(-80 e^A)
    o.gated_delta(qkv, b, a, torch.zeros(1, H * V).cuda(), torch.zeros(H).cuda(), torch.zeros(H * D).cuda(), torch.ones(V).cuda(),
                  1e-5, state, step, H, G, D, V, True, channel_decay=True, gate_act="sigmoid")
    want = before.clone()
    want[1, 1, 5] = 0.0
    assert torch.allclose(state, want, atol=1e-6, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,R,Dr,ps", [(4, 160, 32, 64), (7, 128, 16, 32), (3, 24, 8, 8), (5, 40, 16, 16), (2, 17, 6, 8), (16, 256, 64, 32),
                                       (9, 300, 2, 16), (1, 512, 64, 16)])
def test_latent_attention_with_a_sink(dtype, H, R, Dr, ps):
    o = ops()
    g = torch.Generator().manual_seed(11)
    sink = (torch.randn(H, generator=g) * 2).cuda()
    for ctx, q_lens in (([0, ps - 1, 2 * ps, 301, 5, 63], [150, 2, 1, 1, 37, 66]), ([0, 1, 254, 255, 256, 700, 63, 1029], [1] * 8)):
        num_pages = sum(-(-(c + n) // ps) for c, n in zip(ctx, q_lens)) + 8
        step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 12)
        pages = latent_pages(step, ctx, q_lens, ps, R + Dr, dtype, num_pages, g)
        N = sum(q_lens)
        q_lat = torch.randn(N, H, R, generator=g).to(dtype).cuda()
        q_rot = torch.randn(N, H, Dr, generator=g).to(dtype).cuda()
        view = CacheView(0, pages, step.block_tables[0], ps)
        scale = (R + Dr) ** -0.5
        b = ref_ops.latent_attention(q_lat, q_rot, step, view, H, R, Dr, scale, sink=sink)
        none = ref_ops.latent_attention(q_lat, q_rot, step, view, H, R, Dr, scale)
        assert (b.float() - none.float()).abs().max() > 0.1                     # the sink counts
        for impl in (None, "general") + (("mma_rows", "mma_ranges") if dtype == torch.bfloat16 and R % 32 == 0 and Dr % 16 == 0 else ()):
            a = o.latent_attention(q_lat, q_rot, step, view, H, R, Dr, scale, impl=impl, sink=sink)
            assert torch.allclose(a.float(), b.float(), **tol(dtype)), (q_lens, impl)
        step.max_kv_len = 5000                      # more ranges of keys than any request needs (a captured graph's bound)
        a2 = o.latent_attention(q_lat, q_rot, step, view, H, R, Dr, scale, sink=sink)
        assert torch.allclose(a2.float(), b.float(), **tol(dtype)), q_lens
    assert o.read_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_sinks_that_take_everything_and_nothing(dtype):
    """A sink far above every score leaves nearly nothing of the values; one far below changes nothing; a first token
    alone shares its softmax with the sink: its weight is 1 / (1 + exp(sink - score))."""
    o = ops()
    g = torch.Generator().manual_seed(13)
    H, R, Dr, ps = 4, 64, 16, 16
    for ctx, q_lens in (([0, 40, 300], [70, 1, 1]), ([0], [1])):
        step = make_step(o, dtype, ctx, q_lens, ps, 64, 14)
        pages = latent_pages(step, ctx, q_lens, ps, R + Dr, dtype, 64, g)
        N = sum(q_lens)
        q_lat = (torch.randn(N, H, R, generator=g) * 0.2).to(dtype).cuda()
        q_rot = (torch.randn(N, H, Dr, generator=g) * 0.2).to(dtype).cuda()
        view = CacheView(0, pages, step.block_tables[0], ps)
        plain = o.latent_attention(q_lat, q_rot, step, view, H, R, Dr, 0.1)
        high = o.latent_attention(q_lat, q_rot, step, view, H, R, Dr, 0.1, sink=torch.full((H,), 40.0).cuda())
        low = o.latent_attention(q_lat, q_rot, step, view, H, R, Dr, 0.1, sink=torch.full((H,), -60.0).cuda())
        assert float(high.float().abs().max()) < 1e-6 and torch.allclose(low.float(), plain.float(), atol=1e-6, rtol=0)
    sink = torch.tensor([0.0, 1.0, -1.0, 3.0]).cuda()
    got = o.latent_attention(q_lat, q_rot, step, view, H, R, Dr, 0.1, sink=sink).float()
    row = pages[int(step.block_tables[0][0, 0]), 0].float()
    score = (q_lat[0].float() @ row[:R] + q_rot[0].float() @ row[R:]) * 0.1
    want = (1.0 / (1.0 + torch.exp(sink - score)))[:, None] * row[None, :R]
    assert torch.allclose(got[0], want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,C,eps", [(5, 96, 1e-6), (3, 1000, 1e-5), (1, 20, 1e-5), (70, 17, 1e-3), (300, 1536, 1e-6), (9, 4, 1e-5)])
def test_norm_of_activation_rows(dtype, N, C, eps):
    o = ops()
    g = torch.Generator().manual_seed(15)
    wide = (torch.randn(N, C + 24, generator=g) * 3).to(dtype).cuda()
    x = wide[:, 8:8 + C]                                                         # a column slice of a wider product
    w = (1 + 0.2 * torch.randn(C, generator=g)).cuda()
    for weight in (w, None):
        a, b = o.rmsnorm_rows(x, weight, eps), ref_ops.rmsnorm_rows(x, weight, eps)
        assert a.shape == (N, C) and a.dtype == dtype and torch.allclose(a.float(), b.float(), **tol(dtype))


def expert_tensors(g, E, F, W, dtype):
    w_router = (torch.randn(E, W, generator=g) * W ** -0.5 * 2).cuda()
    w_gate_up = (torch.randn(E, 2 * F, W, generator=g) * W ** -0.5).to(dtype).cuda()
    w_down = (torch.randn(E, W, F, generator=g) * F ** -0.5).to(dtype).cuda()
    return w_router, w_gate_up, w_down


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("weight_on,renorm", [("input", False), ("output", False), ("input", True), ("output", True)])
@pytest.mark.parametrize("N,W,F,E,top", [(1, 64, 24, 5, 2), (7, 40, 20, 9, 1), (33, 66, 16, 7, 7), (70, 128, 64, 8, 2), (300, 192, 96, 8, 1),
                                         (600, 256, 136, 4, 2), (5, 50, 12, 3, 3), (40, 320, 128, 1, 1), (130, 96, 40, 40, 6), (1500, 128, 72, 3, 2),
                                         (2100, 64, 24, 16, 1), (900, 200, 328, 2, 2)])
def test_routed_experts(dtype, weight_on, renorm, N, W, F, E, top):
    o = ops()
    g = torch.Generator().manual_seed(17)
    w_router, w_gate_up, w_down = expert_tensors(g, E, F, W, dtype)
    wide = torch.randn(N, W + 16, generator=g).to(dtype).cuda()
    x = wide[:, 8:8 + W]
    a = o.routed_experts(x, w_router, w_gate_up, w_down, top, renorm, weight_on)
    b = ref_ops.routed_experts(x, w_router, w_gate_up, w_down, top, renorm, weight_on)
    assert a.shape == (N, W) and a.dtype == dtype
    # a row whose top scores lie closer together than the router's rounding may go to another expert in the two versions
    s = torch.sigmoid(x.float() @ w_router.t()).sort(dim=-1, descending=True).values
    sure = torch.ones(N, dtype=torch.bool, device="cuda") if top == E else (s[:, top - 1] - s[:, top]) > 1e-4
    assert int(sure.sum()) >= N - max(2, N // 100)
    assert torch.allclose(a.float()[sure], b.float()[sure], **tol(dtype))
    assert o.read_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_rows_experts_do_not_depend_on_the_other_rows(dtype, monkeypatch):
    """The same rows alone, among few others and among many (other tile heights, other places in the sorted layout):
    bit for bit the same results from the kernels that share an order of summation (tiles of 16 and of 64 rows), and
    from the grouped tensor-core products whatever else the step holds; between the two, equal within rounding."""
    o = ops()
    g = torch.Generator().manual_seed(19)
    W, F, E, top = 128, 64, 8, 2
    w_router, w_gate_up, w_down = expert_tensors(g, E, F, W, dtype)
    x = torch.randn(700, W, generator=g).to(dtype).cuda()
    many = o.routed_experts(x, w_router, w_gate_up, w_down, top)                 # bfloat16: the grouped products
    perm = torch.randperm(700, generator=g).cuda()
    assert torch.equal(o.routed_experts(x[perm].contiguous(), w_router, w_gate_up, w_down, top), many[perm])
    half = o.routed_experts(x[:400].contiguous(), w_router, w_gate_up, w_down, top)
    assert torch.equal(half, many[:400])
    monkeypatch.setattr(o, "USE_MOE_GROUPED_TC", False)
    all_rows = o.routed_experts(x, w_router, w_gate_up, w_down, top)
    assert torch.allclose(all_rows.float(), many.float(), **tol(dtype))
    for rows in ([0], [3, 4, 5], list(range(100, 140)), list(range(690, 700)) + list(range(10))):
        part = o.routed_experts(x[rows].contiguous(), w_router, w_gate_up, w_down, top)
        assert torch.equal(part, all_rows[rows]), rows[:3]
    assert o.read_status() == 0


def test_the_router_picks_the_largest_scores_and_the_lower_index_of_equals():
    """Router rows made so that the scores are known: expert e's score grows with e, two experts tie at the top.  One
    expert's down projection is the only one that is not zero, so the output tells whether that expert was chosen."""
    o = ops()
    dtype, W, F, E = torch.float32, 32, 8, 6
    x = torch.zeros(4, W).cuda()
    x[:, 0] = 1.0
    x[:, 1] = torch.tensor([0.5, -0.5, 1.0, 2.0]).cuda()
    w_router = torch.zeros(E, W).cuda()
    w_router[:, 0] = torch.tensor([0.1, 0.2, 0.9, 0.3, 0.9, 0.4]).cuda()        # experts 2 and 4 tie
    w_gate_up = torch.zeros(E, 2 * F, W).cuda()
    w_gate_up[:, :, 1] = 1.0                                                    # gate = up = the expert's input's column 1
    for chosen_by_top in ((2, 1), (4, 2), (5, 3), (0, 6)):
        expert, top = chosen_by_top
        w_down = torch.zeros(E, W, F).cuda()
        w_down[expert, 0, :] = 1.0
        got = o.routed_experts(x, w_router, w_gate_up, w_down, top)
        hit = got[:, 0].abs() > 0
        assert bool(hit.all()), chosen_by_top
        if top > 1:
            less = o.routed_experts(x, w_router, w_gate_up, w_down, top - 1)
            assert not bool((less[:, 0].abs() > 0).any()), chosen_by_top
        s = torch.sigmoid(w_router[expert, 0])
        z = s * x[:, 1]
        assert torch.allclose(got[:, 0], F * z * torch.sigmoid(z) * z, atol=1e-5, rtol=1e-5)     # the score scales the input
