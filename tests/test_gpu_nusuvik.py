"""GPU tests of the Nusuvik family: the engine (model, page pool, scheduler, kernels) against the plain float64 restatement in
tests/nusuvik_oracle.py, on small random models of several shapes."""
import math

import pytest
import torch

from tests import nusuvik_oracle as O
from tests.hybrid_util import random_tokens, row_err
from tests.nusuvik_util import dense, latent_layer, make_config, make_weights, moe

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4   # float32 engine vs float64 oracle


def _engine(cfg, w, dtype=torch.float32, max_tokens=1024, **kw):
    from qserve_b200.engine import Engine
    from qserve_b200.hybrid import HybridDecoder
    from qserve_b200.modelcfg import ARCHITECTURES

    model = HybridDecoder(ARCHITECTURES[cfg["architecture"]](cfg), w, dtype, torch.device("cuda:0"))
    return Engine(model, max_tokens=max_tokens, **kw)


def _whole(eng, sid, toks):
    out = eng.step([(sid, toks, list(range(len(toks))))])
    eng.release(sid)
    return out


def _portions(eng, sid, toks, sizes):
    """Feed toks in portions of the given sizes (cycled), wanting every position."""
    outs, at, i = [], 0, 0
    while at < len(toks):
        n = min(sizes[i % len(sizes)], len(toks) - at)
        outs.append(eng.step([(sid, toks[at:at + n], list(range(n)))]))
        at, i = at + n, i + 1
    return torch.cat(outs)


STACK = [latent_layer(), latent_layer(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16, q_rank=12, mlp=moe()),
         latent_layer(heads=5, dim=6, rot_dim=10, vdim=12, kv_rank=14, q_rank=20, mlp=None), latent_layer(mlp=moe(experts=4, top=4, ff=16, groups=1, keep=1))]


def _bf16_close(got, want) -> bool:
    """bfloat16 engine against the float64 oracle through stacks with expert mixtures: rounding noise can turn a router's close call, which
    moves that row by much more than rounding; so the typical row must agree to rounding noise and only a few rows may be far off."""
    got, want = got.double().cpu(), want.double().cpu()
    e = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
    return float(e.median()) < 0.04 and int((e > 0.15).sum()) <= max(1, 0.1 * e.numel())


NO_EXPERTS = [STACK[0], latent_layer(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16, q_rank=12, mlp=dense(ff=24)), STACK[2]]   # no close calls to turn


def _rows_rel(got, want) -> float:
    """Largest RMS difference of a row relative to that row's own RMS (rows of very different sizes in one tensor)."""
    got, want = got.double().cpu(), want.double().cpu()
    return float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()).max())


def _raw():
    return torch.cuda.current_stream().cuda_stream


# ------------------------------------------------------------------------------------------------------------------------
# kernels alone
# ------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,width", [(1, 40), (2, 40), (2, 33), (2, 2048), (1, 1030)])
def test_stream_update_norm_kernel(dev, dtype, kind, width):
    """x += rows + rows + bias (rows fp32 or of the storage type, any of them absent), then the RMS or layer norm, and the joined row [x | x0]."""
    from qserve_b200._lib import check, lib

    g = torch.Generator().manual_seed(width + kind)
    T, dt = 6, 0 if dtype == torch.bfloat16 else 1
    x, x0 = torch.randn(T, width, generator=g) + 0.7, torch.randn(T, width, generator=g)
    gain, bias, ab = torch.randn(width, generator=g), torch.randn(width, generator=g), torch.randn(width, generator=g)
    for f1, f2, with2, with_b in ((True, False, True, True), (False, True, True, False), (False, False, False, True), (None, None, False, False)):
        a1 = torch.randn(T, width, generator=g).to(torch.float32 if f1 else dtype) if f1 is not None else None
        a2 = torch.randn(T, width, generator=g).to(torch.float32 if f2 else dtype) if with2 else None
        xd, h, cat = x.clone().to(dev), torch.zeros(T, width, dtype=dtype, device=dev), torch.zeros(T, 2 * width, dtype=dtype, device=dev)
        a1d, a2d = (a1.to(dev) if a1 is not None else None), (a2.to(dev) if a2 is not None else None)
        gd, bd, abd, x0d = gain.to(dev), bias.to(dev), ab.to(dev), x0.to(dev)
        ptr = lambda t: None if t is None else t.data_ptr()
        check(lib.qs_hyb_stream_update_norm(h.data_ptr(), cat.data_ptr(), xd.data_ptr(), x0d.data_ptr(), ptr(a1d), 1 if f1 else 0, ptr(a2d), 1 if f2 else 0,
                                            abd.data_ptr() if with_b else None, gd.data_ptr(), bd.data_ptr() if kind == 2 else None, kind, 1e-5, T, width,
                                            dt, _raw()))
        nx = x.double() + (a1.double() if a1 is not None else 0) + (a2.double() if a2 is not None else 0) + (ab.double() if with_b else 0)
        want = O.layer_norm(nx, gain.double(), bias.double(), 1e-5) if kind == 2 else O.unit_rms(nx, gain.double(), 1e-5)
        tol = 1e-5 if dtype == torch.float32 else 2.0 ** -8
        assert torch.allclose(xd.cpu().double(), nx, atol=1e-5, rtol=1e-6)
        assert row_err(h, want) < tol
        assert row_err(cat, torch.cat([nx, x0.double()], -1)) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("ff,in_stride", [(24, 24), (24, 67), (2048, 2048 + 512), (13, 13)])
def test_bias_gelu_and_softcap_kernels(dev, dtype, ff, in_stride):
    from qserve_b200._lib import check, lib

    g = torch.Generator().manual_seed(ff)
    T, dt = 5, 0 if dtype == torch.bfloat16 else 1
    z, b = (torch.randn(T, in_stride, generator=g) * 2).to(dtype), torch.randn(ff, generator=g)
    zd, bd, out = z.to(dev), b.to(dev), torch.zeros(T, ff + 3, dtype=dtype, device=dev)
    check(lib.qs_hyb_bias_gelu_tanh(out.data_ptr(), ff + 3, zd.data_ptr(), in_stride, bd.data_ptr(), T, ff, dt, _raw()))
    want = O.gelu_tanh(z[:, :ff].double() + b.double())
    assert row_err(out[:, :ff], want) < (1e-6 if dtype == torch.float32 else 2.0 ** -8)
    assert float(out[:, ff:].abs().max()) == 0.0
    x = torch.randn(1000, generator=g) * 30
    xd = x.to(dev)
    check(lib.qs_hyb_softcap(xd.data_ptr(), xd.numel(), 12.5, _raw()))
    assert torch.allclose(xd.cpu().double(), 12.5 * torch.tanh(x.double() / 12.5), atol=1e-5)


@pytest.mark.parametrize("T", [7, 700])
@pytest.mark.parametrize("experts,top,groups,keep,width", [(6, 2, 3, 2, 48), (8, 3, 2, 1, 40), (1, 1, 1, 1, 16), (64, 6, 8, 3, 256), (12, 12, 12, 12, 33),
                                                          (40, 3, 40, 3, 64), (9, 2, 3, 1, 20), (66, 5, 2, 2, 48)])
def test_grouped_sigmoid_router_kernel(dev, experts, top, groups, keep, width, T):
    from qserve_b200._lib import check, lib

    g = torch.Generator().manual_seed(experts + T)
    h, wr = torch.randn(T, width, generator=g), torch.randn(experts, width, generator=g) * 2.0 * width ** -0.5
    corr = torch.randn(experts, generator=g) * 0.5 - 0.3
    hd, wd, cd = h.to(dev), wr.to(dev), corr.to(dev)
    route, idx, wt = torch.zeros(T, experts, device=dev), torch.zeros(T, top, dtype=torch.int32, device=dev), torch.zeros(T, top, device=dev)
    check(lib.qs_hyb_moe_router(route.data_ptr(), idx.data_ptr(), wt.data_ptr(), hd.data_ptr(), wd.data_ptr(), T, width, experts, top, 1, cd.data_ptr(),
                                groups, keep, 1, _raw()))
    spec = {"router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}
    want_idx, want_w = O.route(spec, {"router": wr, "correction": corr}, "", h.double())
    assert torch.equal(idx.cpu().long(), want_idx)
    assert torch.allclose(wt.cpu().double(), want_w, atol=1e-6)
    assert torch.allclose(route.cpu().double(), torch.zeros(T, experts, dtype=torch.float64).scatter(1, want_idx, want_w), atol=1e-6)


def _latent_case(dev, dtype, H, K, R, lens, page=16, seed=0, needle=None):
    """Random query rows and a random pool; sequences of the given lengths whose last `q` positions are queries.  Returns what the kernels need
    and the direct answer [H, T, K]."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n, _ in lens) + 2
    pool = torch.randn(n_pages, page, K + R, generator=g).to(dtype)
    perm = torch.randperm(n_pages, generator=g).tolist()  # pages in no particular order
    max_blocks = max(-(-n // page) for n, _ in lens)
    table = torch.zeros(len(lens), max_blocks, dtype=torch.int32)
    slots, poss, at = [], [], 0
    for s, (n, nq) in enumerate(lens):
        k = -(-n // page)
        table[s, :k] = torch.tensor(perm[at:at + k], dtype=torch.int32)
        at += k
        slots += [s] * nq
        poss += list(range(n - nq, n))
    T = len(slots)
    qa = (torch.randn(T, H, K + R, generator=g) * 0.5).to(dtype)
    if needle is not None:  # one query row points at one far cell: the cell's direction, long enough to own the softmax
        t, h, key = needle
        s, pos = slots[t], key
        cell = pool[int(table[s, pos // page]), pos % page].float()
        qa[t, h] = (cell / cell.norm() * 40.0).to(dtype)
    scale = 1.0 / math.sqrt(K + R)
    want = torch.zeros(H, T, K, dtype=torch.float64)
    for t, (s, pos) in enumerate(zip(slots, poss)):
        cells = torch.stack([pool[int(table[s, j // page]), j % page] for j in range(pos + 1)]).double()
        p = torch.softmax(qa[t].double() @ cells.T * scale, -1)
        want[:, t] = p @ cells[:, :K]
    dv = lambda t: t.to(dev)
    return dv(qa), dv(pool), dv(torch.tensor(slots, dtype=torch.int32)), dv(torch.tensor(poss, dtype=torch.int32)), dv(table), max_blocks, T, scale, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,K,R", [(1, 8, 2), (3, 24, 8), (8, 64, 8), (5, 33, 0), (20, 40, 6), (2, 512, 64), (16, 128, 32), (9, 100, 4)])
def test_latent_attention_kernel(dev, dtype, H, K, R):
    """The plain kernel against the direct sum: several sequences in one launch, pages out of order, prompts and single tokens, lengths at and
    around page and tile borders."""
    from qserve_b200._lib import check, lib

    lens = [(1, 1), (16, 3), (17, 17), (33, 2), (64, 1), (65, 5), (200, 1), (129, 40)]
    qa, pool, slot, pos, table, mb, T, scale, want = _latent_case(dev, dtype, H, K, R, lens, seed=H + K)
    out = torch.zeros(H, T, K, dtype=dtype, device=dev)
    check(lib.qs_hyb_latent_attention(out.data_ptr(), qa.data_ptr(), pool.data_ptr(), slot.data_ptr(), pos.data_ptr(), table.data_ptr(), mb, T, H, K, R,
                                      scale, 16, 0, 0, None, 0 if dtype == torch.bfloat16 else 1, _raw()))
    assert _rows_rel(out, want) < (2e-5 if dtype == torch.float32 else 2.0 ** -7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("key", [0, 1, 15, 16, 31, 32, 63, 64, 500, 895, 896, 898])
def test_latent_attention_far_key(dev, dtype, key):
    """One query that points at one cell among 900: the answer is that cell's latent, wherever it lies (first cells, page and tile borders,
    the newest cells), for a decoded token and inside a prompt portion."""
    from qserve_b200._lib import check, lib

    H, K, R = 4, 32, 8
    for nq in (1, 70):
        n = 900
        t = nq - 1 if key >= n - nq else nq // 2  # a query that may see the key
        if n - nq + t < key:
            continue
        qa, pool, slot, pos, table, mb, T, scale, want = _latent_case(dev, dtype, H, K, R, [(n, nq), (40, 2)], seed=key, needle=(t, 2, key))
        out = torch.zeros(H, T, K, dtype=dtype, device=dev)
        check(lib.qs_hyb_latent_attention(out.data_ptr(), qa.data_ptr(), pool.data_ptr(), slot.data_ptr(), pos.data_ptr(), table.data_ptr(), mb, T, H, K,
                                          R, scale, 16, 0, 0, None, 0 if dtype == torch.bfloat16 else 1, _raw()))
        cell = pool[int(table[0, key // 16]), key % 16, :K].double().cpu()
        assert float((want[2, t] - cell).abs().max()) < 1e-2  # the case is what it claims: the direct answer is the cell
        assert float((out[2, t].double().cpu() - cell).abs().max()) < (1e-2 if dtype == torch.float32 else 3e-2)
        assert _rows_rel(out, want) < (2e-5 if dtype == torch.float32 else 2.0 ** -7)


@pytest.mark.parametrize("H,K,R", [(1, 32, 8), (8, 64, 40), (16, 128, 0), (20, 64, 24), (40, 256, 32), (128, 64, 8), (16, 512, 64), (3, 32, 40)])
def test_latent_attention_tensor_core_kernel(dev, H, K, R):
    """The tensor-core kernels (rows of a tile = (token, head) pairs; single tokens with their cells shared out over blocks) against the direct
    sum and against the plain kernel: long portions, short ones, single tokens, at page and tile borders, all in one launch."""
    from qserve_b200._lib import check, lib
    from qserve_b200.hybrid import StepBatch

    assert lib.qs_hyb_latent_attention_fast_supported(0, H, K, R) == 1
    lens = [(1, 1), (16, 16), (17, 1), (33, 2), (64, 1), (65, 15), (300, 1), (129, 40), (130, 70), (257, 64)]
    qa, pool, slot, pos, table, mb, T, scale, want = _latent_case(dev, torch.bfloat16, H, K, R, lens, seed=H + K)
    b = StepBatch.build([(s, n - nq, -1, [0] * nq) for s, (n, nq) in enumerate(lens)], table, dev)
    assert b.n_tiles > 0 and b.n_short > 0
    scratch = torch.zeros(int(lib.qs_hyb_latent_attention_scratch_floats(T, H, K)), device=dev)
    out = torch.zeros(H, T, K, dtype=torch.bfloat16, device=dev)
    ptr = lambda t: t.data_ptr()
    check(lib.qs_hyb_latent_attention_fast(ptr(out), ptr(qa), ptr(pool), ptr(b.tok_slot), ptr(b.tok_pos), ptr(table), mb, ptr(b.tile_entry), ptr(b.tile_row0),
                                           b.n_tiles, ptr(b.short_tokens), b.n_short, ptr(b.entry_start), ptr(b.entry_len), ptr(b.entry_slot),
                                           ptr(b.entry_pos0), T, ptr(scratch), H, K, R, scale, 16, 0, 0, None, 0, _raw()))
    assert torch.equal(b.tok_pos, pos) and torch.equal(b.tok_slot, slot)
    assert _rows_rel(out, want) < 2.0 ** -7
    plain = torch.zeros_like(out)
    check(lib.qs_hyb_latent_attention(ptr(plain), ptr(qa), ptr(pool), ptr(slot), ptr(pos), ptr(table), mb, T, H, K, R, scale, 16, 0, 0, None, 0, _raw()))
    assert _rows_rel(out, plain) < 2.0 ** -7


@pytest.mark.parametrize("key", [0, 1, 31, 32, 63, 64, 500, 895, 896, 898])
@pytest.mark.parametrize("window", [0, 200])
def test_latent_attention_tensor_core_far_key(dev, key, window):
    """One query that points at one cell among 900, on the tensor-core kernels: a decoded token (cells shared out over blocks) and a row inside
    a prompt portion.  With a window of 200 positions the cell is seen only from inside it, by both kernels alike."""
    from qserve_b200._lib import check, lib
    from qserve_b200.hybrid import StepBatch

    H, K, R, n = 4, 32, 8, 900
    for nq in (1, 70):
        t = nq - 1 if key >= n - nq else nq // 2
        qpos = n - nq + t
        if qpos < key:
            continue
        lens = [(n, nq), (40, 2)]
        qa, pool, slot, pos, table, mb, T, scale, want = _latent_case(dev, torch.bfloat16, H, K, R, lens, seed=key, needle=(t, 2, key))
        b = StepBatch.build([(s, m - q, -1, [0] * q) for s, (m, q) in enumerate(lens)], table, dev)
        scratch = torch.zeros(int(lib.qs_hyb_latent_attention_scratch_floats(T, H, K)), device=dev)
        out, plain = torch.zeros(H, T, K, dtype=torch.bfloat16, device=dev), torch.zeros(H, T, K, dtype=torch.bfloat16, device=dev)
        ptr = lambda x: x.data_ptr()
        check(lib.qs_hyb_latent_attention_fast(ptr(out), ptr(qa), ptr(pool), ptr(b.tok_slot), ptr(b.tok_pos), ptr(table), mb, ptr(b.tile_entry),
                                               ptr(b.tile_row0), b.n_tiles, ptr(b.short_tokens), b.n_short, ptr(b.entry_start), ptr(b.entry_len),
                                               ptr(b.entry_slot), ptr(b.entry_pos0), T, ptr(scratch), H, K, R, scale, 16, 0, window, None, 0, _raw()))
        check(lib.qs_hyb_latent_attention(ptr(plain), ptr(qa), ptr(pool), ptr(slot), ptr(pos), ptr(table), mb, T, H, K, R, scale, 16, 0, window, None, 0, _raw()))
        cell = pool[int(table[0, key // 16]), key % 16, :K].double().cpu()
        seen = window == 0 or key > qpos - window
        hit = float((out[2, t].double().cpu() - cell).abs().max()) < 3e-2
        assert hit == seen
        assert _rows_rel(out, plain) < 2.0 ** -7
        if window == 0:
            assert _rows_rel(out, want) < 2.0 ** -7


# ------------------------------------------------------------------------------------------------------------------------
# layers through the engine
# ------------------------------------------------------------------------------------------------------------------------
LAYERS = [
    latent_layer(mlp=None), latent_layer(heads=1, dim=4, rot_dim=2, vdim=6, kv_rank=5, q_rank=7, mlp=None),
    latent_layer(heads=8, dim=16, rot_dim=8, vdim=16, kv_rank=32, q_rank=24, mlp=None),
    latent_layer(heads=5, dim=20, rot_dim=12, vdim=4, kv_rank=9, q_rank=3, base=1e6, mlp=None),
    latent_layer(heads=2, dim=2, rot_dim=30, vdim=40, kv_rank=64, q_rank=64, mlp=None),
    latent_layer(heads=12, dim=8, rot_dim=4, vdim=8, kv_rank=130, q_rank=16, scale=0.5, mlp=None),
    latent_layer(heads=4, dim=16, rot_dim=16, vdim=16, kv_rank=16, q_rank=16, mlp=None),   # equal sizes everywhere
    latent_layer(heads=3, dim=12, rot_dim=0, vdim=8, kv_rank=20, q_rank=10, mlp=None),      # no rotated part at all
]


@pytest.mark.parametrize("layer", LAYERS, ids=lambda l: "x".join(str(v) for v in l["mixer"].values() if isinstance(v, int)))
def test_single_latent_layer(dev, layer):
    cfg = make_config([layer])
    w = make_weights(cfg, 2, sharp=3.0)
    toks = random_tokens(150, cfg["vocab"], 2)
    taps = []
    got = _engine(cfg, w).step([("a", toks, list(range(len(toks))))], tap=lambda r, x: taps.append(x.clone()))
    want, layers = O.forward(cfg, w, toks, return_layers=True)
    assert row_err(taps[0], layers[0]) < F32_TOL
    assert row_err(got, want) < F32_TOL


@pytest.mark.parametrize("spec", [dense(), dense(ff=1), dense(ff=300), moe(), moe(experts=1, top=1, ff=8, groups=1, keep=1),
                                  moe(experts=8, top=3, ff=16, groups=2, keep=1), moe(experts=9, top=9, ff=5, groups=9, keep=9),
                                  moe(experts=36, top=3, ff=24, groups=6, keep=2)],
                         ids=lambda s: s["kind"] + "-" + "-".join(str(v) for v in (s.get("router") or s).values() if isinstance(v, int)))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_beside_mixer(dev, spec, dtype):
    """Both branches read the one normed row; their sum meets the stream.  bfloat16 mixtures run on expert-sorted rows, fp32 ones stacked."""
    cfg = make_config([latent_layer(mlp=spec)], width=48)
    w = make_weights(cfg, 3)
    toks = random_tokens(120, cfg["vocab"], 3)
    taps = []
    got = _engine(cfg, w, dtype).step([("a", toks, list(range(len(toks))))], tap=lambda r, x: taps.append(x.clone()))
    want, layers = O.forward(cfg, w, toks, return_layers=True)
    if dtype == torch.float32:
        assert row_err(taps[0], layers[0]) < F32_TOL and row_err(got, want) < F32_TOL
    else:
        assert row_err(taps[0], layers[0]) < 0.02


@pytest.mark.parametrize("loop", [None, (0, 1, 1), (0, 2, 3), (1, 3, 2), (2, 4, 4), (3, 4, 2)])
def test_stack_and_loop(dev, loop):
    """Layer order and the loop: passes with their own caches, the projection of [stream; embedding output] at the start of every pass, also
    when layers come before the loop, and no loop at all."""
    cfg = make_config(STACK, loop=loop)
    w = make_weights(cfg, 4)
    toks = random_tokens(90, cfg["vocab"], 4)
    taps = []
    got = _engine(cfg, w).step([("a", toks, list(range(len(toks))))], tap=lambda r, x: taps.append(x.clone()))
    want, layers = O.forward(cfg, w, toks, return_layers=True)
    assert len(taps) == len(layers)
    for a, b in zip(taps, layers):
        assert row_err(a, b) < F32_TOL
    assert row_err(got, want) < F32_TOL
    assert float(got.abs().max()) <= cfg["logit_softcap"]


def test_without_pair_embedding_and_cap(dev):
    cfg = make_config(STACK[:2], bigram=None, cap=None, loop=(0, 2, 2))
    w = make_weights(cfg, 5)
    toks = random_tokens(60, cfg["vocab"], 5)
    assert row_err(_whole(_engine(cfg, w), "a", toks), O.forward(cfg, w, toks)) < F32_TOL


# ------------------------------------------------------------------------------------------------------------------------
# the cache: decoding, portions, batches, reuse
# ------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefill_against_token_by_token(dev, dtype):
    cfg = make_config(STACK, loop=(1, 3, 2))
    w = make_weights(cfg, 6, sharp=2.0)
    toks = random_tokens(140, cfg["vocab"], 6)
    want = O.forward(cfg, w, toks)
    eng = _engine(cfg, w, dtype)
    whole = _whole(eng, "a", toks)
    single = _portions(eng, "b", toks, [1])   # from the first token on: graph replay from the second
    eng.release("b")
    if dtype == torch.float32:
        assert row_err(whole, want) < F32_TOL and row_err(single, want) < F32_TOL
    else:
        assert _bf16_close(whole, want) and _bf16_close(single, want) and _bf16_close(single, whole)


@pytest.mark.parametrize("sizes", [[2], [3, 2, 7], [64], [63, 1, 65], [17, 100, 5, 2], [130, 2]])
def test_portions(dev, sizes):
    cfg = make_config(STACK, loop=(0, 2, 2))
    w = make_weights(cfg, 7, sharp=2.0)
    toks = random_tokens(210, cfg["vocab"], 7)
    eng = _engine(cfg, w, page_size=16)
    got = _portions(eng, "a", toks, sizes)
    assert row_err(got, O.forward(cfg, w, toks)) < F32_TOL


@pytest.mark.parametrize("dtype,stack", [(torch.float32, STACK), (torch.bfloat16, STACK), (torch.bfloat16, NO_EXPERTS)], ids=["f32", "bf16", "bf16-dense"])
def test_mixed_batches_with_reuse(dev, dtype, stack):
    """Unequal requests in one batch (portions beside single tokens) against each alone; four slots and a page pool that is far smaller than
    the sum of all requests, so that pages and slots are handed out again."""
    cfg = make_config(stack, loop=(1, 2, 3))
    w = make_weights(cfg, 8, sharp=2.0)
    lens = [70, 33, 120, 5, 64, 97, 18, 2]
    reqs = {f"r{i}": random_tokens(n, cfg["vocab"], 20 + i) for i, n in enumerate(lens)}
    eng = _engine(cfg, w, dtype, max_tokens=4 * 128, page_size=16)
    alone = {k: O.forward(cfg, w, v) for k, v in reqs.items()}
    fed = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    waiting, live, step = list(reqs), [], 0
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries = []
        for j, k in enumerate(live):
            left = len(reqs[k]) - fed[k]
            n = min(left, 1 if (step + j) % 3 == 0 and fed[k] > 0 else [29, 2, 64, 7][(step + j) % 4])
            entries.append((k, reqs[k][fed[k]:fed[k] + n], list(range(n))))
        out = eng.step(entries)
        r = 0
        for k, toks, want in entries:
            got[k].append(out[r:r + len(toks)])
            r += len(toks)
            fed[k] += len(toks)
        for k in [k for k in live if fed[k] == len(reqs[k])]:
            live.remove(k)
            eng.release(k)
        step += 1
    assert eng.cache.free_pages() == eng.cache.num_pages and len(eng.cache.seqs) == 0
    for k in reqs:
        g = torch.cat(got[k])
        if dtype == torch.float32:
            assert row_err(g, alone[k]) < F32_TOL, k
        elif stack is STACK:
            assert _bf16_close(g, alone[k]), k
        else:
            assert row_err(g, alone[k]) < 0.06, k


def test_long_decoding_and_graph_replay(dev):
    """Hundreds of single tokens through captured graphs against eager launches and the oracle; two sequences side by side."""
    cfg = make_config(STACK[:2], loop=(0, 1, 2))
    w = make_weights(cfg, 9, sharp=2.0)
    a, b = random_tokens(330, cfg["vocab"], 9), random_tokens(300, cfg["vocab"], 10)
    outs = {}
    for graphs in (True, False):
        eng = _engine(cfg, w, use_graphs=graphs, page_size=16)
        eng.step([("a", a[:30], []), ("b", b[:1], [])])
        rows = []
        for i in range(299):
            rows.append(eng.step([("a", a[30 + i:31 + i], [0]), ("b", b[1 + i:2 + i], [0])]))
        outs[graphs] = torch.stack(rows)
    assert torch.equal(outs[True], outs[False])
    wa, wb = O.forward(cfg, w, a[:329]), O.forward(cfg, w, b)
    assert row_err(outs[True][:, 0], wa[30:]) < F32_TOL and row_err(outs[True][:, 1], wb[1:]) < F32_TOL


@pytest.mark.parametrize("far", [0, 1, 15, 16, 17, 63, 64, 300])
def test_far_token_is_seen(dev, far):
    """A long prompt whose token at `far` (first cells, page borders, an earlier portion) is changed: the oracle's answer at the last positions
    moves by a small but definite amount, and the engine's distance to the right answer is a small fraction of that move -- in a prompt portion
    and for decoded tokens.  (One cell that owns the softmax is the kernel test above; here every cell has a small weight.)"""
    cfg = make_config([latent_layer(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, q_rank=24, mlp=None)], bigram=None)
    w = make_weights(cfg, 11)
    toks = random_tokens(420, cfg["vocab"], 11)
    other = list(toks)
    other[far] = (toks[far] + 1) % cfg["vocab"]
    want, moved = O.forward(cfg, w, toks), O.forward(cfg, w, other)
    effect = row_err(moved[-40:], want[-40:])
    assert effect > 2e-5
    eng = _engine(cfg, w, page_size=16)
    eng.step([("a", toks[:301], [])])
    part = eng.step([("a", toks[301:400], list(range(99)))])
    tail = torch.cat([eng.step([("a", [t], [0])]) for t in toks[400:]])
    assert row_err(part[-20:], want[380:400]) < 0.05 * row_err(moved[380:400], want[380:400])
    assert row_err(tail, want[400:]) < 0.05 * row_err(moved[400:], want[400:])


def test_tensor_core_path_through_engine(dev):
    """bfloat16 models whose sizes the tensor-core kernels take: whole prompts, portions, single tokens (graph replay) and a mixed batch through
    the engine, against the oracle and against the same engine kept on the plain kernel.  Prompt portions run on per-head keys and values laid
    out from the cached rows where the head sizes allow, else (and when told so) on tiles in the latent space; single tokens always there."""
    import qserve_b200.hybrid as hyb

    stack = [latent_layer(heads=4, dim=16, rot_dim=16, vdim=32, kv_rank=32, q_rank=24),           # prompt portions on per-head keys and values
             latent_layer(heads=20, dim=8, rot_dim=16, vdim=8, kv_rank=64, q_rank=32, mlp=None),  # sizes only the latent-space tiles take
             latent_layer(heads=3, dim=40, rot_dim=8, vdim=64, kv_rank=128, q_rank=16, mlp=None)]
    cfg = make_config(stack, loop=(0, 1, 2))
    w = make_weights(cfg, 13, sharp=2.0)
    a, b = random_tokens(200, cfg["vocab"], 13), random_tokens(90, cfg["vocab"], 14)
    wa, wb = O.forward(cfg, w, a), O.forward(cfg, w, b)
    runs = {}
    for impl in (None, "latent", "plain"):
        hyb.LATENT_IMPL = impl
        try:
            eng = _engine(cfg, w, torch.bfloat16, page_size=16)
            whole = _whole(eng, "w", a)
            parts = _portions(eng, "p", a, [70, 2, 33, 1, 1, 64])
            eng.release("p")
            ga, gb = [eng.step([("a", a[:100], list(range(100)))])], []
            for i in range(90):  # a portion of b beside single tokens of a, then both decode
                e = [("a", a[100 + i:101 + i], [0])] + ([("b", b[:40], list(range(40)))] if i == 0 else [("b", b[39 + i:40 + i], [0])] if i <= 50 else [])
                out = eng.step(e)
                ga.append(out[:1])
                if i <= 50:
                    gb.append(out[1:])
            runs[impl] = (whole, parts, torch.cat(ga), torch.cat(gb))
        finally:
            hyb.LATENT_IMPL = None
    for got, want in zip(runs[None], (wa, wa, wa[:190], wb)):
        assert row_err(got, want) < 0.06
    for impl in (None, "latent"):
        for f, p in zip(runs[impl], runs["plain"]):
            assert row_err(f, p) < 0.03


def test_generate_through_scheduler(dev):
    """Greedy generation through Engine.generate: admission, prompt chunks, decoding, retirement; against the oracle's argmax."""
    from qserve_b200.engine import SamplingParams

    cfg = make_config(STACK[:3], loop=(0, 2, 2), cap=6.0)
    w = make_weights(cfg, 12)
    prompts = [random_tokens(n, cfg["vocab"], 40 + n) for n in (5, 37, 1, 70, 12, 20)]
    eng = _engine(cfg, w, max_tokens=4 * 96, page_size=16, chunk=24, max_batch_tokens=48)
    outs = eng.generate(prompts, [SamplingParams(max_new_tokens=6)] * len(prompts))
    for p, o in zip(prompts, outs):
        assert o == O.greedy(cfg, w, p, 6)
    assert eng.cache.free_pages() == eng.cache.num_pages
