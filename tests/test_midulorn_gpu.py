"""Midulorn on the GPU: every new kernel against its plain reference at sizes of its own (with
inputs made so that a far key, a sink or a stretch's edge shows), then bin/trace_run replaying
requests whole, decoded token by token, in portions and mixed with pages and slots used again, in
32-bit and bfloat16, against the plain model; the edges of a stretch through the engine; greedy
generation through ``Engine.generate`` (graphs, steps launched ahead) and the command line;
configurations drawn at random."""
import numpy as np
import pytest
import torch

from tests import helpers
from tests.helpers import TraceRunner
from tests.midulorn_cases import CASES, SHARPEN, model_dir, plain_logits, random_tokens, weights

pytestmark = pytest.mark.gpu

STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def up64(n):
    return (n + 63) // 64 * 64


class _Batch:
    pass


class _Ctx:
    def __init__(self, device="cuda:0"):
        from garuda_b200.engine.batch import Workspace
        self.ws = Workspace(torch.device(device))
        self.batch = _Batch()


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def both(request):
    from garuda_b200.kernels.ops import CudaOps
    from tests.plain.cpu_ops import CpuOps
    dt = STORE[request.param]
    return CudaOps("cuda:0", tensor_cores=dt == torch.bfloat16), CpuOps(), dt


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(hash((shape, seed)) % (1 << 31))
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(got, want, dt, what, tol=None):
    got, want = got.float().cpu(), want.float()
    tol = tol or (2e-2 if dt == torch.bfloat16 else 2e-5)
    err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-6)
    assert torch.isfinite(got).all() and err <= tol, f"{what}: {err:.2e}"


def step_batch(lens, starts, slots, page_size, seed=1):
    """A batch of requests that bring ``lens`` tokens from positions ``starts``, their pages drawn at
    random from the pool; returns (batch, block table, pages in the pool)."""
    b = _Batch()
    R = len(lens)
    b.cu_q = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    b.kv_lens = torch.tensor([s + n for s, n in zip(starts, lens)], dtype=torch.int32)
    b.positions = torch.tensor(np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lens)]), dtype=torch.int32)
    b.slots = torch.tensor(slots, dtype=torch.int32)
    b.token_req = torch.repeat_interleave(torch.arange(R, dtype=torch.int32), torch.tensor(lens))
    b.num_requests, b.max_q_len, b.min_q_len = R, max(lens), min(lens)
    b.num_tokens, b.max_kv_len = sum(lens), int(b.kv_lens.max())
    width = (b.max_kv_len + page_size - 1) // page_size + 1
    table = -torch.ones(R, width, dtype=torch.int32)
    perm = np.random.default_rng(seed).permutation(R * width)
    at = 0
    for r in range(R):
        n = (int(b.kv_lens[r]) + page_size - 1) // page_size
        table[r, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    return b, table, R * width


def batches(b):
    ctx_g, ctx_r = _Ctx(), _Ctx("cpu")
    ctx_r.batch = b
    bg = _Batch()
    for k, v in vars(b).items():
        setattr(bg, k, v.cuda() if torch.is_tensor(v) else v)
    ctx_g.batch = bg
    return ctx_g, ctx_r


# ---------------------------------------------------------------------------- kernels
@pytest.mark.parametrize("T,d", [(1, 40), (37, 200), (5, 1030), (3, 4096)])
def test_norm_after_the_sum_in_one_pass(both, T, d):
    ops, ref, dt = both
    x, y, row, w = rnd(T, d, seed=1), rnd(T, d, seed=2), rnd(d, seed=3), rnd(d, seed=4)
    for yy, rr, alpha in ((y, row, 1.7), (None, None, 1.0), (y, None, 0.5), (None, row, 1.0)):
        want = x.clone()
        ref.post_norm(want, yy, alpha, w, 1e-5, row=rr)
        got = x.clone().cuda()
        rounded = torch.empty(T, d, dtype=torch.bfloat16, device="cuda")
        ops.post_norm(got, None if yy is None else yy.cuda(), alpha, w.cuda(), 1e-5, row=None if rr is None else rr.cuda(), rounded=rounded)
        close(got, want, torch.float32, f"post_norm {T}x{d}")
        close(rounded, want.bfloat16(), torch.bfloat16, "its rounded copy", 1e-2)


def test_a_factor_on_the_sum_is_a_smaller_eps():
    """rms_eps(alpha v) = rms_(eps / alpha^2)(v): what the block's pass over the residual relies on."""
    from tests.plain.cpu_ops import CpuOps
    ref = CpuOps()
    x, y, w = rnd(9, 70, seed=1), rnd(9, 70, seed=2) * 1e-3, rnd(70, seed=3)
    a, eps = 2.5, 1e-3
    one = x.clone() * 1e-3
    ref.post_norm(one, y, a, w, eps)
    two = x.clone() * 1e-3 + y / a
    ref.post_norm(two, None, 1.0, w, eps / (a * a))
    assert (one - two).abs().max() <= 1e-6 * one.abs().max()


@pytest.mark.parametrize("T,H,group", [(1, 3, 14), (33, 6, 20), (70, 8, 128)])
def test_a_gate_per_head(both, T, H, group):
    ops, ref, dt = both
    x = rnd(T, H * group, dtype=dt, seed=1)
    wide = rnd(T, H + 5, scale=2.0, seed=2)
    gate = wide[:, 2:2 + H]                                        # a column range of a wider row
    want = x.clone()
    ref.group_gate_mul(want, gate, group)
    got = x.clone().cuda()
    ops.group_gate_mul(got, wide.cuda()[:, 2:2 + H], group)
    close(got, want, dt, "group_gate_mul")


@pytest.mark.parametrize("M,N,K", [(21, 77, 40), (3, 320, 160), (300, 1024, 256), (2048, 512, 128)])
def test_xielu_behind_a_product(both, M, N, K):
    ops, ref, dt = both
    a, w = rnd(M, K, dtype=dt, seed=1), rnd(N, K, dtype=dt, scale=0.3, seed=2)
    ctx_g, ctx_r = _Ctx(), _Ctx("cpu")
    want = torch.empty(M, N, dtype=dt)
    ref.linear_xielu(ctx_r, a, w, want, 0.8, 1.3)
    got = torch.empty(M, N, dtype=dt, device="cuda")
    ops.linear_xielu(ctx_g, a.cuda(), w.cuda(), got, 0.8, 1.3)
    close(got, want, dt, "linear_xielu")
    z = rnd(M, N, scale=3.0, seed=3)
    want = torch.empty(M, N)
    ref.xielu(z, want, 0.8, 1.3)
    got = torch.empty(M, N, device="cuda")
    ops.xielu(z.cuda(), got, 0.8, 1.3)
    close(got, want, torch.float32, "xielu")


@pytest.mark.parametrize("lens,starts,slots", [([5, 1, 200, 64, 65], [0, 7, 3, 0, 10], [2, 0, -1, 3, 1]), ([1, 1, 1], [4, 0, 9], [1, -1, 0]),
                                               ([700], [0], [3]), ([2, 129], [0, 5], [0, 1])])
def test_gated_recurrence_steps(both, lens, starts, slots):
    """Mixed steps (single tokens beside long portions, which are cut into stretches that run side
    by side); a row whose slot is negative is padding and touches no state."""
    ops, ref, dt = both
    W = 200
    b, _, _ = step_batch(lens, starts, slots, 8)
    ctx_g, ctx_r = batches(b)
    T = b.num_tokens
    proj, bz, bu = rnd(T, 3 * W + 5, seed=1), rnd(W, seed=2), rnd(W, seed=3)
    state = rnd(4, W + 3, seed=4)
    cols = (2, W + 3, 2 * W + 5)
    want, s_want = torch.zeros(T, W, dtype=dt), state.clone()
    ref.mingru(ctx_r, proj, cols, bz, bu, s_want, want)
    got, s_got = torch.zeros(T, W, dtype=dt, device="cuda"), state.clone().cuda()
    ops.mingru(ctx_g, proj.cuda(), cols, bz.cuda(), bu.cuda(), s_got, got)
    close(got, want, dt, f"mingru {lens}", 2e-2 if dt == torch.bfloat16 else 5e-5)
    close(s_got, s_want, torch.float32, "its state", 5e-5)


def test_gated_recurrence_carries_its_state_over_steps():
    """700 tokens at once against the same tokens in steps of 1, 2, 64, 65 and 300."""
    from garuda_b200.kernels.ops import CudaOps
    ops = CudaOps("cuda:0")
    W, T = 96, 700
    proj = rnd(T, 3 * W, seed=7).cuda()
    out_a, out_b = torch.zeros(T, W, device="cuda"), torch.zeros(T, W, device="cuda")
    state_a, state_b = torch.zeros(2, W, device="cuda"), torch.zeros(2, W, device="cuda")
    b, _, _ = step_batch([T], [0], [1], 8)
    ctx, _ = batches(b)
    ops.mingru(ctx, proj, (0, W, 2 * W), None, None, state_a, out_a)
    at = 0
    for n in (1, 2, 64, 65, 300, 1, 267):
        b, _, _ = step_batch([n], [at], [0], 8)
        ctx, _ = batches(b)
        ops.mingru(ctx, proj[at:at + n], (0, W, 2 * W), None, None, state_b, out_b[at:at + n])
        at += n
    assert at == T
    close(out_b, out_a.cpu(), torch.float32, "cut against whole", 1e-5)
    close(state_b[0], state_a[1].cpu(), torch.float32, "the states", 1e-5)


@pytest.mark.parametrize("taps,H,G,dim,vdim", [(1, 4, 2, 24, 40), (3, 4, 1, 64, 64), (4, 3, 3, 12, 20), (16, 2, 1, 8, 8)])
def test_convolved_projections_into_pages(both, taps, H, G, dim, vdim):
    ops, ref, dt = both
    ps = 8
    b, table, pages = step_batch([5, 1, 30, 2], [0, 7, 3, 0], [2, 0, 3, 1], ps)
    ctx_g, ctx_r = batches(b)
    T, C = b.num_tokens, H * dim + G * (dim + vdim)
    proj, bias, cw = rnd(T, C, seed=1), rnd(C, seed=2), rnd(C, taps, seed=3)
    state = rnd(4, max(taps - 1, 1) * C, seed=4)
    qw, kw, vf = rnd(dim, seed=5), rnd(dim, seed=6), rnd(T, G * vdim, seed=7)
    for mode in ("source", "mix", None):
        kp, vp = torch.zeros(pages, G, ps, dim, dtype=dt), torch.zeros(pages, G, ps, vdim, dtype=dt)
        q, s, vo = torch.zeros(T, H, dim, dtype=dt), state.clone(), torch.zeros(T, G * vdim)
        ref.conv_qkv_append(ctx_r, proj, bias, cw, taps, s, q, kp, vp, table, H, G, dim, vdim, qw, kw, 1e-5, ps,
                            v_first_in=vf if mode == "mix" else None, v_first_out=vo if mode == "source" else None, mix=0.3)
        kg, vg = torch.zeros_like(kp).cuda(), torch.zeros_like(vp).cuda()
        qg, sg, vog = torch.zeros_like(q).cuda(), state.clone().cuda(), torch.zeros_like(vo).cuda()
        ops.conv_qkv_append(ctx_g, proj.cuda(), bias.cuda(), cw.cuda(), taps, sg, qg, kg, vg, table.cuda(), H, G, dim, vdim,
                            qw.cuda(), kw.cuda(), 1e-5, ps, v_first_in=vf.cuda() if mode == "mix" else None,
                            v_first_out=vog if mode == "source" else None, mix=0.3)
        for a, w_, what in ((qg, q, "queries"), (kg, kp, "keys"), (vg, vp, "values")):
            close(a, w_, dt, f"{what}, {taps} taps, {mode}")
        close(sg, s, torch.float32, "the kept rows")
        close(vog, vo, torch.float32, "the values handed on")


@pytest.mark.parametrize("H,G,dim,vdim,ps", [(6, 2, 24, 40, 8), (4, 2, 64, 64, 32), (8, 2, 32, 64, 16), (2, 2, 128, 128, 64)])
@pytest.mark.parametrize("chunk", [0, 7, 16, 33, 80])
def test_attention_with_sinks_distance_and_stretches(both, H, G, dim, vdim, ps, chunk):
    """Mixed steps over pages drawn at random; stretches that end inside a page, at its border and
    beyond the step's first token. One key far back is made to stand out (its row and the queries
    scaled), one head's sink is made to dominate, so that a lost key or sink shows in the output."""
    ops, ref, dt = both
    lens, starts = [5, 1, 60, 2, 1], [0, 37, 13, 190, 300]
    b, table, pages = step_batch(lens, starts, [0, 1, 2, 3, 0], ps)
    bg = batches(b)[0].batch
    T = b.num_tokens
    q, kp, vp = rnd(T, H, dim, dtype=dt, seed=1), rnd(pages, G, ps, dim, dtype=dt, seed=2), rnd(pages, G, ps, vdim, dtype=dt, seed=3)
    far = int(table[4, 2])                                         # request 4 reads position 2 * ps + 1 from 300
    kp[far, :, 1, :] = (q[T - 1, 0, :].float() * 2.0).to(dt)
    sinks, r1, r2 = rnd(H, seed=4), torch.rand(H), torch.rand(H) * 2
    sinks[1] = 6.0
    args = (0.3, 0, ps, len(lens), max(lens), b.max_kv_len)
    want = torch.zeros(T, H * vdim, dtype=dt)
    ref.paged_attention(q, kp, vp, table, b.cu_q, b.kv_lens, b.token_req, want, *args, sink_values=sinks, distance=(r1, r2), chunk=chunk)
    got = torch.zeros(T, H * vdim, dtype=dt, device="cuda")
    ops.paged_attention(q.cuda(), kp.cuda(), vp.cuda(), table.cuda(), bg.cu_q, bg.kv_lens, bg.token_req, got, *args, ws=None,
                        min_q_len=1, sink_values=sinks.cuda(), distance=(r1.cuda(), r2.cuda()), chunk=chunk)
    close(got, want, dt, f"attention, stretches of {chunk}", 3e-2 if dt == torch.bfloat16 else 2e-5)
    if chunk == 0:
        # without the far key the last row's first head would read something else entirely
        kp2 = kp.clone()
        kp2[far, :, 1, :] = 0
        other = torch.zeros(T, H * vdim, dtype=dt)
        ref.paged_attention(q, kp2, vp, table, b.cu_q, b.kv_lens, b.token_req, other, *args, sink_values=sinks, distance=(r1, r2), chunk=0)
        assert (other[T - 1, :vdim].float() - want[T - 1, :vdim].float()).abs().max() > 0.05


@pytest.mark.parametrize("H,rank,rot,ps", [(3, 20, 6, 8), (8, 96, 16, 32), (4, 64, 16, 16), (2, 128, 32, 64)])
def test_attention_over_latent_rows_with_sinks(both, H, rank, rot, ps):
    ops, ref, dt = both
    lens, starts = [5, 1, 70, 2, 1], [0, 37, 13, 190, 500]
    b, table, pages = step_batch(lens, starts, [0, 1, 2, 3, 0], ps)
    bg = batches(b)[0].batch
    T, row = b.num_tokens, rank + rot
    q, pool = rnd(T, H, row, dtype=dt, scale=0.5, seed=1), rnd(pages, 1, ps, row, dtype=dt, seed=2)
    far = int(table[4, 1])
    pool[far, 0, 3, :] = (q[T - 1, 1, :].float() * 1.5).to(dt)     # one key far back stands out for the last row's second head
    sinks = rnd(H, seed=3)
    sinks[0] = 5.0
    args = (0.25, 0, ps, len(lens), max(lens), b.max_kv_len)
    want = torch.zeros(T, H * rank, dtype=dt)
    ref.paged_attention(q, pool, pool, table, b.cu_q, b.kv_lens, b.token_req, want, *args, value_dim=rank, sink_values=sinks)
    got = torch.zeros(T, H * rank, dtype=dt, device="cuda")
    pg = pool.cuda()
    ops.paged_attention(q.cuda(), pg, pg, table.cuda(), bg.cu_q, bg.kv_lens, bg.token_req, got, *args, ws=None, min_q_len=1,
                        value_dim=rank, sink_values=sinks.cuda())
    close(got, want, dt, "latent attention with sinks", 3e-2 if dt == torch.bfloat16 else 2e-5)


@pytest.mark.parametrize("T,E,K,top", [(19, 11, 48, 3), (1, 4, 200, 4), (300, 64, 128, 1), (7, 10, 176, 3)])
def test_router_over_all_experts(both, T, E, K, top):
    ops, ref, dt = both
    h, w = rnd(T, K, dtype=dt, seed=1), rnd(E, K, dtype=dt, scale=0.5, seed=2)
    ids, wts = torch.zeros(T, top, dtype=torch.int32), torch.zeros(T, top)
    ref.route_topk(h, w, None, top, ids, wts, score="softmax_all")
    ids_g, wts_g = torch.zeros(T, top, dtype=torch.int32, device="cuda"), torch.zeros(T, top, device="cuda")
    ops.route_topk(h.cuda(), w.cuda(), None, top, ids_g, wts_g, score="softmax_all")
    same = (ids_g.cpu() == ids)
    assert same.float().mean() > 0.98                                # (two experts within rounding of each other may swap)
    close(wts_g.cpu()[same], wts[same], torch.float32, "router weights", 1e-4)
    assert (wts_g.sum(-1) <= 1.0 + 1e-5).all()                       # shares of the whole softmax: not renormalized


# ---------------------------------------------------------------------------- the engine, replayed
def check(got, ref, dtype, what, name):
    """Per position, the largest difference as a fraction of the largest logit. 32-bit: every position
    within 2e-4 (sums in another order than the 64-bit plain model's). bfloat16: nine positions in ten
    within 0.05 and the median within 0.015, the rest finite: with sharpened random weights a router's
    close call or a sharp softmax turns the rounding of an input into a large change at a few positions,
    in the plain model itself; a fault of a kernel, a mask or a state shows at most positions."""
    scale = float(np.abs(ref).max())
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    err = np.abs(got - ref).max(-1) / scale
    helpers.OBSERVED[f"{name}/{dtype}"] = max(helpers.OBSERVED.get(f"{name}/{dtype}", 0.0), float(np.median(err)))
    if dtype == "float32":
        assert err.max() <= 2e-4, f"{what}: {err.max():.3e} of the largest logit at position {int(err.argmax())}"
        return
    over = int((err > 0.05).sum())
    assert over <= max(1, len(err) // 10), f"{what}: {over} of {len(err)} positions beyond 0.05 (largest {err.max():.3e})"
    assert np.median(err) <= 0.015, f"{what}: median {np.median(err):.3e}"


@pytest.fixture(scope="module", params=[(n, d) for n in CASES for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def run(request):
    name, dtype = request.param
    tr = TraceRunner(model_dir(name, STORE[dtype]), dtype, max_tokens=4 * up64(130), extra=["--page-size", "16"])
    yield name, dtype, tr
    assert tr.close() == 0


def test_whole(run):
    name, dtype, tr = run
    for n, seed in ((1, 1), (2, 2), (17, 3), (130, 4)):
        toks = random_tokens(name, n, seed)
        out = tr.step([("w", toks, range(n))], end=["w"])
        check(out, plain_logits(name, STORE[dtype], toks), dtype, f"whole, {n} tokens", name)


def test_prompt_then_token_by_token(run):
    name, dtype, tr = run
    toks = random_tokens(name, 120, 7)
    ref = plain_logits(name, STORE[dtype], toks)
    outs = [tr.step([("d", toks[:39], [38])])]
    for i in range(39, 120):                      # every stretch's edge of the configurations is passed by decoded tokens
        outs.append(tr.step([("d", [toks[i]], [0])], end=["d"] if i == 119 else []))
    check(np.concatenate(outs), ref[38:], dtype, "decode after a prompt", name)


def test_long_decoding_from_the_first_token(run):
    name, dtype, tr = run
    toks = random_tokens(name, 100, 9)
    ref = plain_logits(name, STORE[dtype], toks)
    got = np.concatenate([tr.step([("l", [t], [0])], end=["l"] if i == 99 else []) for i, t in enumerate(toks)])
    check(got[:4], ref[:4], dtype, "first tokens", name)
    check(got, ref, dtype, "long decoding", name)


def test_portions_down_to_two_tokens(run):
    name, dtype, tr = run
    toks = random_tokens(name, 118, 11)
    ref = plain_logits(name, STORE[dtype], toks)
    cuts = [7, 2, 19, 3, 2, 16, 2, 31, 1, 15, 2, 18]
    pos, outs = 0, []
    for i, c in enumerate(cuts):
        outs.append(tr.step([("p", toks[pos:pos + c], range(c))], end=["p"] if i == len(cuts) - 1 else []))
        pos += c
    assert pos == 118
    check(np.concatenate(outs), ref, dtype, "portions", name)


def test_mixed_requests_reusing_pages_and_slots(run):
    name, dtype, tr = run
    lens = [90, 33, 128, 21, 64, 2, 75]
    toks = [random_tokens(name, n, 20 + i) for i, n in enumerate(lens)]
    refs = [plain_logits(name, STORE[dtype], t) for t in toks]
    pool = 4 * up64(130) - 128
    fed, got = [0] * len(lens), [[] for _ in lens]
    live, waiting = [], list(range(len(lens)))
    rng = np.random.default_rng(1)
    most = 0
    while live or waiting:
        while waiting and len(live) < 4 and sum(up64(lens[i]) for i in live) + up64(lens[waiting[0]]) <= pool:
            live.append(waiting.pop(0))
        most = max(most, len(live))
        entries, ended = [], []
        active = [i for i in live if rng.random() > 0.15] or live[:1]        # now and then a request sits a step out
        for i in active:
            left = lens[i] - fed[i]
            n = 1 if left <= 12 else int(min(left - 12, rng.integers(2, 24)))
            entries.append((f"m{i}", toks[i][fed[i]:fed[i] + n], range(n)))
            if fed[i] + n == lens[i]:
                ended.append(f"m{i}")
        out = tr.step(entries, end=ended)
        row = 0
        for (_, t, _), i in zip(entries, active):
            got[i].append(out[row:row + len(t)])
            row += len(t)
            fed[i] += len(t)
            if fed[i] == lens[i]:
                live.remove(i)
    assert most == 4
    for i in range(len(lens)):
        check(np.concatenate(got[i]), refs[i], dtype, f"mixed, request {i}", name)


def test_every_way_of_cutting_gives_the_same_logits_in_32_bit(run):
    name, dtype, tr = run
    if dtype != "float32":
        pytest.skip("compared against the plain model in bfloat16")
    toks = random_tokens(name, 80, 31)
    whole = tr.step([("x", toks, range(80))], end=["x"])
    parts = [tr.step([("y", toks[:50], range(50))])]
    parts += [tr.step([("y", [t], [0])]) for t in toks[50:79]]
    parts.append(tr.step([("y", [toks[79]], [0])], end=["y"]))
    assert np.abs(np.concatenate(parts) - whole).max() <= 2e-5 * max(1.0, np.abs(whole).max())


def test_a_long_request_whose_early_tokens_reach_the_end():
    """700 tokens through stretches of 33 positions, a latent attention that reads everything and
    recurrences: the last logits follow the plain model in both dtypes, and they change with token 3."""
    name = "MD"
    toks = random_tokens(name, 700, 3)
    for dtype in ("float32", "bfloat16"):
        ref = plain_logits(name, STORE[dtype], toks)
        tr = TraceRunner(model_dir(name, STORE[dtype]), dtype, max_tokens=up64(700))
        tr.step([("a", toks[:300], [])])
        out = tr.step([("a", toks[300:], range(390, 400))], end=["a"])
        check(out, ref[690:], dtype, "the end of 700 tokens", name)
        if dtype == "float32":
            other = list(toks)
            other[3] = (toks[3] + 1) % CASES[name][0]["vocab"]
            alt = tr.step([("b", other, range(690, 700))], end=["b"])
            assert np.abs(alt - out).max() > 1e-4 * np.abs(out).max()
        assert tr.close() == 0


def test_the_edges_of_a_stretch_through_the_engine():
    """The one-layer model: changing a token just in front of a query's stretch leaves its logits as
    they were, bit for bit; the stretch's first token changes them. Once within a prompt portion, once
    decoded token by token behind a portion, so that the edge is passed by decoded tokens; the stretch
    (9 positions) ends inside a page of 16, and two stretches on at a page's border (position 63 | 64 is
    not one, 31 | 32 neither: the borders that matter are 27, 36, 45, ...)."""
    name, size = "MC", 9
    toks = random_tokens(name, 48, 1)
    tr = TraceRunner(model_dir(name), "float32", max_tokens=up64(64), extra=["--page-size", "16"])

    def last_decoded(t, rid, upto):
        tr.step([(rid, t[:25], [])])
        for i in range(25, upto):
            tr.step([(rid, [t[i]], [])])
        return tr.step([(rid, [t[upto]], [0])], end=[rid])[0]

    def last_in_portion(t, rid, upto):
        tr.step([(rid, t[:13], [])])
        return tr.step([(rid, t[13:upto + 1], [upto - 13])], end=[rid])[0]

    for k, last in enumerate((last_decoded, last_in_portion)):
        for upto in (39, 44, 47):                                   # the query's place in its stretch: 3, 8 (the last), 2
            first = upto // size * size
            base = last(toks, f"a{k}{upto}", upto)
            for j, same in ((first - 1, True), (first, upto == first and False), (upto, False)):
                t = list(toks)
                t[j] = (t[j] + 7) % 64
                diff = np.abs(last(t, f"b{k}{upto}{j}", upto) - base).max()
                assert (diff == 0.0) == same, f"query {upto}, token {j} changed: difference {diff}"
    assert tr.close() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype):
    from garuda_b200 import Engine, SamplingParams
    from tests.plain import midulorn_plain as mp
    name = "MB"
    cfg, w = CASES[name][0], weights(name, STORE[dtype])
    e = Engine(model_dir(name, STORE[dtype]), dtype=dtype, context=256, kv_tokens=1024, max_concurrent=4)
    assert e.model.graph_safe
    prompts = [random_tokens(name, n, 70 + n) for n in (5, 40, 1, 23, 64)]
    res = e.generate(prompts, SamplingParams.greedy(max_tokens=12))
    assert e.runner.graphs.replays > 0
    for p, r in zip(prompts, res):
        assert r.finish_reason == "length" and len(r.tokens) == 12
        seq = list(p)
        for tok in r.tokens:
            logits = mp.forward(cfg, w, seq)[-1]
            slack = (1e-4 if dtype == "float32" else 0.05) * float(np.abs(logits).max())
            assert logits[tok] >= float(logits.max()) - slack, f"token {tok} has logit {logits[tok]}, the best is {logits.max()}"
            seq.append(tok)


# ---------------------------------------------------------------------------- configurations drawn at random
def _random_config(rng):
    def pick(xs):
        return xs[int(rng.integers(0, len(xs)))]

    mixed_width = pick([(1, 48), (2, 32), (3, 16)])                 # layers with mixed values share (kv heads, value width)

    def attention():
        v_mix = pick([True, True, False])
        g, vdim = mixed_width if v_mix else (pick([1, 2, 3]), pick([8, 20, 32, 64, 128]))
        dim = pick([8, 12, 32, 64, 128])
        m = {"heads": g * pick([1, 2, 4]), "kv_heads": g, "dim": dim, "vdim": vdim, "scale": pick([0.5, 1.0, 2.0]) / dim ** 0.5}
        if pick([True, True, True, False]):
            m["conv"] = pick([1, 2, 3, 4, 7])
        if pick([True, True, True, False]):
            m["mask"] = {"size": pick([1, 5, 16, 33, 64, 100])}
        if v_mix:
            m["v_mix"] = True
        return {"type": "attention", "mixer": m}

    def latent():
        rot = pick([2, 8, 16, 32, 64])
        rank = pick([8, 20, 32, 64, 128, 256])
        return {"type": "latent_attention", "mixer": {
            "heads": pick([1, 2, 5, 8]), "dim": pick([8, 20, 32, 64]), "rot_dim": rot, "vdim": pick([8, 24, 64]), "kv_rank": rank,
            "scale": pick([0.1, 0.2, 0.4]), "rot": {"base": pick([100.0, 10000.0, 500000.0]), "dims": rot}}}

    def recurrence():
        return {"type": "mingru", "mixer": {"width": pick([8, 40, 128, 300])}}

    def mlp():
        kind = pick(["dense", "dense", "moe", "moe", None])
        if kind == "dense":
            return {"kind": "dense", "ff": pick([8, 24, 56, 128])}
        if kind == "moe":
            experts = pick([1, 2, 5, 12, 33])
            return {"kind": "moe", "expert": {"ff": pick([8, 24, 64])}, "router": {"experts": experts, "top": int(rng.integers(1, min(experts, 6) + 1))}}
        return None

    layers = [dict(pick([attention, attention, latent, recurrence])(), mlp=mlp()) for _ in range(pick([1, 2, 3, 5]))]
    return {"architecture": "Midulorn", "vocab": pick([50, 97, 300, 1000]), "width": pick([40, 64, 72, 136, 256]),
            "embedding": {"scale": pick([1.0, 3.0, 12.0])}, "norm": {"eps": pick([1e-5, 1e-6])},
            "postln_alpha": pick([1.0, 1.3, 2.0, 4.0]), "logit_scale": pick([1.0, 0.25, 0.5]), "layers": layers}


@pytest.mark.parametrize("seed", [2, 5, 11, 17])
def test_configurations_drawn_at_random(seed, tmp_path):
    from garuda_b200.weights import write_random_model
    from tests.plain import midulorn_plain as mp
    rng = np.random.default_rng(seed)
    for k in range(3):
        cfg = _random_config(rng)
        for dtype in ("float32", "bfloat16"):
            d = write_random_model(str(tmp_path / f"m{k}{dtype}"), cfg, seed * 10 + k, store_dtype=STORE[dtype], scale=SHARPEN)
            w = helpers.folder_weights(d)
            a, b = rng.integers(0, cfg["vocab"], 70).tolist(), rng.integers(0, cfg["vocab"], 45).tolist()
            ra, rb = mp.forward(cfg, w, a).astype(np.float32), mp.forward(cfg, w, b).astype(np.float32)
            tr = TraceRunner(d, dtype, max_tokens=2 * up64(70), extra=["--page-size", "16"])
            check(tr.step([("w", a, range(70))], end=["w"]), ra, dtype, f"seed {seed}.{k}: whole", "random")
            outs_a, outs_b = [tr.step([("a", a[:40], range(40)), ("b", b[:3], range(3))])], []
            outs_b.append(outs_a[0][40:])
            outs_a[0] = outs_a[0][:40]
            o = tr.step([("b", b[3:30], range(27)), ("a", a[40:42], range(2))])
            outs_b.append(o[:27])
            outs_a.append(o[27:])
            for i in range(15):
                o = tr.step([("a", [a[42 + i]], [0]), ("b", [b[30 + i]], [0])], end=["b"] if i == 14 else [])
                outs_a.append(o[:1])
                outs_b.append(o[1:])
            outs_a.append(tr.step([("a", a[57:], range(13))], end=["a"]))
            check(np.concatenate(outs_a), ra, dtype, f"seed {seed}.{k}: request a", "random")
            check(np.concatenate(outs_b), rb, dtype, f"seed {seed}.{k}: request b", "random")
            assert tr.close() == 0


def test_command_line_generates_with_sampling(tmp_path):
    """`garuda generate` on a folder of this design: greedy tokens are the plain model's, and a
    sampled run with a seed (temperature, top-k, top-p through the engine's sampler) repeats itself."""
    import json
    import os
    import subprocess
    import sys
    from tests.plain import midulorn_plain as mp
    name = "MA"
    d = model_dir(name)
    cfg = tmp_path / "config.toml"
    prompt = random_tokens(name, 11, 5)
    exe = [sys.executable, os.path.join(helpers.ROOT, "bin", "garuda")]

    def generate(sampling, *more):
        cfg.write_text(f'[model]\npath = "{d}"\ndtype = "float32"\ncontext = 128\n[memory]\npage_size = 16\n[sampling]\n{sampling}')
        out = subprocess.run(exe + ["--config", str(cfg), "generate", "--prompt-ids", ",".join(map(str, prompt)), *more],
                             capture_output=True, text=True)
        assert out.returncode == 0, out.stderr
        return json.loads(out.stdout.strip().splitlines()[-1])

    rec = generate("temperature = 0.0\nmax_tokens = 6\n")
    seq = list(prompt)
    for _ in range(6):
        seq.append(int(np.argmax(mp.forward(CASES[name][0], weights(name), seq)[-1])))
    assert rec["tokens"] == seq[len(prompt):] and rec["finish_reason"] == "length"
    a = generate("temperature = 0.9\ntop_k = 20\ntop_p = 0.9\nmax_tokens = 8\n", "--seed", "4")
    b = generate("temperature = 0.9\ntop_k = 20\ntop_p = 0.9\nmax_tokens = 8\n", "--seed", "4")
    assert a["tokens"] == b["tokens"] and len(a["tokens"]) == 8
