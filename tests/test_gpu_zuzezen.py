"""GPU tests of the Zuzezen family: the engine (model, page pool, state slots, scheduler, kernels) against the plain float64 restatement in
tests/zuzezen_oracle.py, on small random models of several shapes."""
import math

import pytest
import torch

from tests import zuzezen_oracle as O
from tests.hybrid_util import bf16_close, random_tokens, row_err
from tests.zuzezen_util import attention_layer, dense, gla_layer, latent_layer, make_config, make_weights

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


def _raw():
    return torch.cuda.current_stream().cuda_stream


def _bf(t):
    return t.to(torch.bfloat16).to(torch.float32)


STACK = [gla_layer(), latent_layer(), attention_layer(), latent_layer(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16, mlp=None),
         gla_layer(heads=2, dim=8, vdim=8, tau=3.0, mlp=dense(24))]


# ------------------------------------------------------------------------------------------------------------------------
# kernels alone
# ------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,add_f32,bias,scale", [(40, True, True, True), (33, False, False, True), (2048, True, False, False), (1030, False, True, True),
                                                      (44, True, True, False), (9000, True, True, True), (1301, True, False, True)])
def test_post_norm_update_kernel(dev, dtype, width, add_f32, bias, scale):
    from qserve_b200._lib import check, lib

    g = torch.Generator().manual_seed(width)
    T, dt = 9, 0 if dtype == torch.bfloat16 else 1
    x, y = torch.randn(T, width, generator=g), _bf(torch.randn(T, width, generator=g) * 3.0)
    w, ls, b = torch.randn(width, generator=g) * 0.3, torch.rand(width, generator=g), torch.randn(width, generator=g)
    yy = y.double() + (b.double() if bias else 0.0)
    want = x.double() + yy / torch.sqrt(yy.pow(2).mean(-1, keepdim=True) + 1e-5) * (1.0 + w.double()) * (ls.double() if scale else 1.0)
    xd, wd, lsd, bd = x.to(dev), w.to(dev), ls.to(dev), b.to(dev)
    yd = y.to(dev) if add_f32 else y.to(dev).to(dtype)
    h = torch.zeros(T, width, dtype=dtype, device=dev)
    check(lib.qs_hyb_post_norm_update(h.data_ptr(), xd.data_ptr(), yd.data_ptr(), 1 if add_f32 else 0, bd.data_ptr() if bias else None, wd.data_ptr(),
                                      lsd.data_ptr() if scale else None, 1.0, 1e-5, T, width, dt, _raw()))
    assert float((xd.double().cpu() - want).abs().max()) < 2e-5
    assert torch.equal(h, xd.to(dtype))   # the sublayers' copy is the stream rounded once
    x2 = x.to(dev)
    check(lib.qs_hyb_post_norm_update(None, x2.data_ptr(), yd.data_ptr(), 1 if add_f32 else 0, bd.data_ptr() if bias else None, wd.data_ptr(),
                                      lsd.data_ptr() if scale else None, 1.0, 1e-5, T, width, dt, _raw()))
    assert torch.equal(x2, xd)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("ff,in_stride,bias", [(24, 48, True), (24, 67, True), (2048, 4096 + 512, True), (13, 26, False), (1, 2, True)])
def test_bias_gated_act_kernel(dev, dtype, act, ff, in_stride, bias):
    from qserve_b200._lib import check, lib

    g = torch.Generator().manual_seed(ff + act)
    T, dt = 5, 0 if dtype == torch.bfloat16 else 1
    z = _bf(torch.randn(T, in_stride, generator=g) * 3.0)
    z[0, 0], z[0, min(1, ff - 1)] = -60.0, 40.0   # far tails of the activation
    b = torch.randn(2 * ff, generator=g) if bias else torch.zeros(2 * ff)
    a, u = z[:, :ff].double() + b[:ff].double(), z[:, ff:2 * ff].double() + b[ff:].double()
    fa = a * torch.sigmoid(a) if act == 1 else 0.5 * a * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (a + 0.044715 * a ** 3)))
    want = fa * u
    zd, bd = z.to(dev).to(dtype), b.to(dev)
    out = torch.zeros(T, ff + 3, dtype=dtype, device=dev)
    check(lib.qs_hyb_bias_gated_act(out.data_ptr(), ff + 3, zd.data_ptr(), in_stride, bd.data_ptr() if bias else None, T, ff, act, dt, _raw()))
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    assert float(((out[:, :ff].double().cpu() - want).abs() / (want.abs() + 1.0)).max()) < tol
    assert float(out[:, ff:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,Dv", [(1, 1, 1), (3, 12, 20), (2, 40, 72), (4, 64, 128), (2, 128, 64), (1, 200, 40), (2, 16, 8), (1, 30, 33), (1, 300, 16)])
def test_gated_linear_kernel(dev, dtype, H, D, Dv):
    """Runs of unequal length in one launch, some continuing from a state that an earlier launch left in their slot."""
    from qserve_b200._lib import check, lib

    g = torch.Generator().manual_seed(H * 1000 + D)
    dt, tau, eps = 0 if dtype == torch.bfloat16 else 1, 4.0, 1e-5
    hd, hv = H * D, H * Dv
    stride = 2 * hd + 2 * hv + 3
    norm_w, zb = 1.0 + 0.2 * torch.randn(Dv, generator=g), 1.5 + torch.randn(hd, generator=g)
    state = torch.zeros(4, H, D, Dv, device=dev)
    zbd, nwd = zb.to(dev), norm_w.to(dev)
    ref_state = {}

    def launch(entries):  # (slot, first position, tokens)
        T = sum(n for _, _, n in entries)
        proj, z = _bf(torch.randn(T, stride, generator=g)), torch.randn(T, hd, generator=g) * 2.0
        want = torch.zeros(T, hv, dtype=torch.float64)
        r = 0
        for slot, p0, n in entries:
            S = torch.zeros(H, D, Dv, dtype=torch.float64) if p0 == 0 else ref_state[slot]
            for t in range(r, r + n):
                row = proj[t].double()
                q, k = row[:hd].view(H, D) / math.sqrt(D), row[hd:2 * hd].view(H, D)
                v, gate = row[2 * hd:2 * hd + hv].view(H, Dv), row[2 * hd + hv:2 * hd + 2 * hv]
                a = torch.sigmoid(z[t].double() + zb.double()).pow(1.0 / tau).view(H, D)
                S = a[:, :, None] * S + k[:, :, None] * v[:, None, :]
                o = (S * q[:, :, None]).sum(1)
                o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * norm_w.double()
                want[t] = o.reshape(-1) * (gate * torch.sigmoid(gate))
            ref_state[slot] = S
            r += n
        es = torch.tensor([sum(e[2] for e in entries[:i]) for i in range(len(entries))], dtype=torch.int32, device=dev)
        el = torch.tensor([e[2] for e in entries], dtype=torch.int32, device=dev)
        sl = torch.tensor([e[0] for e in entries], dtype=torch.int32, device=dev)
        p0 = torch.tensor([e[1] for e in entries], dtype=torch.int32, device=dev)
        pd, zd = proj.to(dev).to(dtype), z.to(dev)
        prep, o_raw = torch.zeros(T, 3 * hd + hv, device=dev), torch.zeros(T, hv, device=dev)
        out = torch.zeros(T, hv + 2, dtype=dtype, device=dev)
        check(lib.qs_hyb_gated_linear(out.data_ptr(), hv + 2, prep.data_ptr(), o_raw.data_ptr(), pd.data_ptr(), stride, zd.data_ptr(), zbd.data_ptr(),
                                      tau, nwd.data_ptr(), state.data_ptr(), es.data_ptr(), el.data_ptr(), sl.data_ptr(), p0.data_ptr(), T,
                                      len(entries), H, D, Dv, eps, dt, _raw()))
        got = out[:, :hv].double().cpu()
        err = float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()).max())
        assert err < (1e-4 if dtype == torch.float32 else 2.0 ** -6)

    launch([(2, 0, 70), (0, 0, 1), (3, 0, 37)])
    launch([(0, 1, 1), (2, 70, 2), (1, 0, 5), (3, 37, 40)])   # slot 1 held nothing before: it must start from zero, not from what lies there
    state[1].normal_()
    ref_state.pop(1)
    launch([(1, 0, 3), (0, 2, 1)])
    for slot, S in ref_state.items():
        assert float((state[slot].double().cpu() - S).abs().max()) < 1e-3 * max(1.0, float(S.abs().max()))


# ------------------------------------------------------------------------------------------------------------------------
# every mechanism alone, through the engine
# ------------------------------------------------------------------------------------------------------------------------
LAYERS = [
    gla_layer(), gla_layer(heads=1, dim=1, vdim=1, tau=1.0, rank=1), gla_layer(heads=2, dim=40, vdim=16, tau=12.0, rank=8), gla_layer(heads=5, dim=7, vdim=33, rank=2),
    gla_layer(heads=2, dim=16, vdim=16, rank=16),   # equal sizes everywhere
    latent_layer(mlp=None), latent_layer(heads=1, dim=4, rot_dim=2, vdim=6, kv_rank=5, mlp=None),
    latent_layer(heads=8, dim=16, rot_dim=8, vdim=16, kv_rank=32, mlp=None), latent_layer(heads=5, dim=20, rot_dim=12, vdim=4, kv_rank=9, base=1e6, mlp=None),
    latent_layer(heads=2, dim=2, rot_dim=30, vdim=40, kv_rank=64, scaling=False, mlp=None),
    latent_layer(heads=4, dim=16, rot_dim=16, vdim=16, kv_rank=16, scale=0.5, mlp=None),   # equal sizes everywhere
    latent_layer(heads=3, dim=8, rot_dim=12, vdim=10, kv_rank=20, rot_dims=6, mlp=None),    # only half of the shared part is turned
    attention_layer(mlp=None), attention_layer(heads=1, kv_heads=1, dim=4, size=1, keep_first=0, mlp=None),
    attention_layer(heads=6, kv_heads=2, dim=10, size=40, keep_first=40, mlp=None), attention_layer(heads=3, kv_heads=3, dim=32, size=7, keep_first=1, mlp=None),
    attention_layer(heads=8, kv_heads=1, dim=16, size=0, keep_first=0, mlp=None),          # no window at all
    attention_layer(heads=2, kv_heads=2, dim=64, size=64, keep_first=70, scale=0.2, mlp=None),   # more kept positions than the window is wide
]


@pytest.mark.parametrize("layer", LAYERS, ids=lambda l: l["type"][:3] + "-" + "x".join(str(v) for v in l["mixer"].values() if isinstance(v, int)))
def test_single_layer(dev, layer):
    cfg = make_config([layer])
    w = make_weights(cfg, 2, sharp=3.0)
    toks = random_tokens(150, cfg["vocab"], 2)
    taps, layers = [], []
    got = _engine(cfg, w).step([("a", toks, list(range(len(toks))))], tap=lambda r, x: taps.append(x.clone()))
    want = O.forward(cfg, w, toks, layers)
    assert row_err(taps[0], layers[0]) < F32_TOL
    assert row_err(got, want) < F32_TOL


@pytest.mark.parametrize("ff", [56, 1, 300])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_after_mixer(dev, ff, dtype):
    cfg = make_config([gla_layer(mlp=dense(ff)), attention_layer(mlp=dense(ff))])
    w = make_weights(cfg, 3)
    toks = random_tokens(70, cfg["vocab"], 3)
    got = _whole(_engine(cfg, w, dtype), "a", toks)
    want = O.forward(cfg, w, toks)
    assert row_err(got, want) < F32_TOL if dtype == torch.float32 else bf16_close(got, want)


def test_stack_and_taps(dev):
    cfg = make_config(STACK, width=52, vocab=131, embed_scale=9.0)
    w = make_weights(cfg, 4, sharp=2.0)
    toks = random_tokens(120, cfg["vocab"], 4)
    taps, layers = [], []
    got = _engine(cfg, w).step([("a", toks, list(range(len(toks))))], tap=lambda r, x: taps.append(x.clone()))
    want = O.forward(cfg, w, toks, layers)
    assert len(taps) == len(layers) == len(STACK)
    for t, l in zip(taps, layers):
        assert row_err(t, l) < F32_TOL
    assert row_err(got, want) < F32_TOL


# ------------------------------------------------------------------------------------------------------------------------
# cuts, batches, reuse
# ------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefill_against_token_by_token(dev, dtype):
    cfg = make_config(STACK)
    w = make_weights(cfg, 6, sharp=2.0 if dtype == torch.float32 else 1.0)   # peaked maps multiply bfloat16's rounding noise layer by layer
    toks = random_tokens(140, cfg["vocab"], 6)
    want = O.forward(cfg, w, toks)
    eng = _engine(cfg, w, dtype)
    whole = _whole(eng, "a", toks)
    single = _portions(eng, "b", toks, [1])   # from the first token on: graph replay from the second
    eng.release("b")
    if dtype == torch.float32:
        assert row_err(whole, want) < F32_TOL and row_err(single, want) < F32_TOL
    else:
        assert bf16_close(whole, want) and bf16_close(single, want) and bf16_close(single, whole)


@pytest.mark.parametrize("sizes", [[2], [3, 2, 7], [64], [63, 1, 65], [17, 100, 5, 2], [130, 2], [23, 24, 25]])
def test_portions(dev, sizes):
    """Portions cut in the middle of pages (16) and of the window (24 wide, 3 kept)."""
    cfg = make_config(STACK)
    w = make_weights(cfg, 7, sharp=2.0)
    toks = random_tokens(210, cfg["vocab"], 7)
    eng = _engine(cfg, w, page_size=16)
    got = _portions(eng, "a", toks, sizes)
    assert row_err(got, O.forward(cfg, w, toks)) < F32_TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixed_batches_with_reuse(dev, dtype):
    """Unequal requests in one batch (portions beside single tokens) against each alone; four slots and a page pool that is far smaller than
    the sum of all requests, so that pages and slots are handed out again (a slot's old recurrent state must not leak into its next owner)."""
    cfg = make_config(STACK)
    w = make_weights(cfg, 8, sharp=2.0 if dtype == torch.float32 else 1.0)
    lens = [70, 33, 120, 5, 64, 97, 18, 2, 1, 50]
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
            if (step + j) % 5 == 4 and len(live) > 1:
                continue   # a live request may sit out a step
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
        assert row_err(g, alone[k]) < F32_TOL if dtype == torch.float32 else bf16_close(g, alone[k]), k


def test_long_decoding_and_graph_replay(dev):
    """Hundreds of single tokens through captured graphs against eager launches and the oracle; two sequences side by side.  The window
    (24 positions, 3 kept) passes over decoded tokens many times, and the recurrent states are carried through every step."""
    cfg = make_config(STACK[:3] + [gla_layer(heads=1, dim=5, vdim=6, tau=30.0)])
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


# ------------------------------------------------------------------------------------------------------------------------
# keys far away, at page borders, at the edges of the window and of the kept first positions
# ------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("far", [0, 1, 15, 16, 17, 63, 64, 300])
@pytest.mark.parametrize("kind", ["latent", "gla"])
def test_far_token_is_seen(dev, far, kind):
    """A long prompt whose token at `far` (first positions, page borders, an earlier portion) is changed: the oracle's answer at the last
    positions moves by a small but definite amount, and the engine's distance to the right answer is a small fraction of that move -- in a
    prompt portion and for decoded tokens."""
    layer = latent_layer(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, mlp=None) if kind == "latent" else gla_layer(heads=2, dim=16, vdim=16, tau=64.0)
    cfg = make_config([layer])
    w = make_weights(cfg, 11)
    if kind == "gla":
        w["l0.mix.a2.b"] += 3.0   # slow forgetting: a token 400 positions back still shows
    toks = random_tokens(420, cfg["vocab"], 11)
    other = list(toks)
    other[far] = (toks[far] + 1) % cfg["vocab"]
    want, moved = O.forward(cfg, w, toks), O.forward(cfg, w, other)
    assert row_err(moved[-40:], want[-40:]) > 2e-5
    eng = _engine(cfg, w, page_size=16)
    eng.step([("a", toks[:301], [])])
    part = eng.step([("a", toks[301:400], list(range(99)))])
    tail = torch.cat([eng.step([("a", [t], [0])]) for t in toks[400:]])
    assert row_err(part[-20:], want[380:400]) < 0.05 * row_err(moved[380:400], want[380:400])
    assert row_err(tail, want[400:]) < 0.05 * row_err(moved[400:], want[400:])


WINDOW, KEPT = 40, 5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("query", [130, 144, 191])   # in the middle of a page, at a page's first cell, at the last cell of a 64-key tile
def test_window_and_kept_edges(dev, dtype, decoded, query):
    """One attention layer: the logits at `query` depend on the token at position j exactly when j is inside the window or among the kept first
    positions.  Changing a visible token moves the oracle's answer and the float32 engine follows it; changing a hidden one (just outside the
    window, just past the kept positions) leaves the engine's answer bit for bit as it was, in either storage type.  In a prompt portion and
    for a token decoded alone."""
    cfg = make_config([attention_layer(heads=4, kv_heads=2, dim=16, size=WINDOW, keep_first=KEPT, mlp=None)])
    w = make_weights(cfg, 12)
    toks = random_tokens(query + 1, cfg["vocab"], 12)

    def at_query(seq):
        eng = _engine(cfg, w, dtype, page_size=16)
        if decoded:
            eng.step([("a", seq[:query], [])])
            return eng.step([("a", seq[query:], [0])])[0]
        eng.step([("a", seq[:100], [])])
        return eng.step([("a", seq[100:], [query - 100])])[0]   # a portion that starts inside an earlier window

    base, want = at_query(toks), O.forward(cfg, w, toks)[query]
    for j, seen in ((query - WINDOW + 1, True), (query - WINDOW, False), (KEPT - 1, True), (KEPT, False), (0, True), (query - 1, True), (query - WINDOW - 17, False)):
        other = list(toks)
        other[j] = (toks[j] + 7) % cfg["vocab"]
        moved, got = O.forward(cfg, w, other)[query], at_query(other)
        effect = float((moved - want).norm())
        if seen:
            assert effect > 1e-5 * float(want.norm()), j   # far keys pay the distance penalty; the flattest head still shows them
            if dtype == torch.float32 or effect > 1e-2 * float(want.norm()):   # bfloat16 rounds smaller moves away
                assert not torch.equal(got, base), j
            if dtype == torch.float32:
                assert float((got.double().cpu() - moved).norm()) < 0.2 * effect, j   # a missed key would leave the whole effect
        else:
            assert effect < 1e-12 and torch.equal(got, base), j


@pytest.mark.parametrize("dtype,impl", [(torch.float32, None), (torch.bfloat16, None), (torch.bfloat16, "plain")], ids=["f32", "bf16-tensor-core", "bf16-plain"])
@pytest.mark.parametrize("decoded", [False, True])
def test_attention_needles(dev, dtype, impl, decoded):
    """The attention mixer on hand-made projection rows: the probe token's query in the flattest head is a large multiple of ONE key's
    direction, so that key owns the softmax whenever it is visible and the head's output is that key's value (the key itself).  Needles at the
    window's edges, at the edges of the kept first positions, at page and tile borders, far away, and the probe's own position; the probe as
    the last row of a prompt portion (tiles on the tensor cores in bfloat16) and as a token of its own (the head-group kernel)."""
    import qserve_b200.hybrid as hyb
    from qserve_b200.hybrid import StepBatch, _stream

    H, G, D, probe = 8, 2, 64, 191
    cfg = make_config([attention_layer(heads=H, kv_heads=G, dim=D, size=WINDOW, keep_first=KEPT, scale=0.2, mlp=None)], width=16)
    eng = _engine(cfg, make_weights(cfg, 21), dtype, page_size=16)
    mixer, cache, dt = eng.model.layers[0].mixer, eng.cache, eng.model.dt
    mixer.bias.zero_()
    mixer.q_gain.fill_(10.0)
    mixer.k_gain.fill_(1.0)
    assert dtype != torch.bfloat16 or lib_fast_ok(mixer)
    g = torch.Generator().manual_seed(5)
    rows = _bf(torch.randn(probe + 1, mixer.in_features, generator=g))
    rows[:, mixer.col_g:] = 20.0   # gates wide open
    keys = rows[:, H * D + (G - 1) * D: H * D + G * D]   # the last key / value head, which the last (flattest) query head reads
    cut = probe if decoded else probe - 29
    hyb.ATTENTION_IMPL = impl
    try:
        for j, seen in ((probe - WINDOW + 1, True), (probe - WINDOW, False), (KEPT - 1, True), (KEPT, False), (0, True), (15, False), (16, False), (64, False),
                        (127, False), (128, False), (probe - WINDOW + 9, True), (160, True), (176, True), (probe - 1, True), (probe, True)):
            r = rows.clone()
            r[probe, (H - 1) * D: H * D] = keys[j]
            st = cache.admit("a")
            cache.reserve("a", probe + 1)
            table = cache.sync_block_table()
            scratch = torch.empty(max(1, eng.model.scratch_floats(probe + 1)), dtype=torch.float32, device=dev)
            for lo, hi in ((0, cut), (cut, probe + 1)):
                b = StepBatch.build([(st.slot, lo, -1, list(range(hi - lo)))], table, dev, cache.page_size)
                proj = r[lo:hi].to(dev).to(dtype).contiguous()
                out = torch.zeros(hi - lo, mixer.out_features, dtype=dtype, device=dev)
                mixer.run(proj, out, b, cache.runs[0], cache.page_size, scratch, dt, _stream(dev))
            cache.release("a")
            head = out[-1, (H - 1) * D:].double().cpu()
            hit = float((head - keys[j].double()).abs().max()) < 0.05 * float(keys[j].abs().max())
            assert hit == seen, (j, seen)
    finally:
        hyb.ATTENTION_IMPL = None


def lib_fast_ok(mixer) -> bool:
    from qserve_b200._lib import lib

    m = mixer.m
    return lib.qs_hyb_attention_fast_supported(0, m.heads, m.kv_heads, 1, m.dim, m.vdim, mixer.in_features) == 1


@pytest.mark.parametrize("n", [1, 2, 3, 6, 7])
def test_first_tokens(dev, n):
    """Sequences shorter than the kept positions and the window, whole and token by token."""
    cfg = make_config([attention_layer(size=4, keep_first=6), latent_layer(), gla_layer(mlp=dense(8))])
    w = make_weights(cfg, 13, sharp=2.0)
    toks = random_tokens(n, cfg["vocab"], 13)
    eng = _engine(cfg, w)
    want = O.forward(cfg, w, toks)
    assert row_err(_whole(eng, "a", toks), want) < F32_TOL
    assert row_err(_portions(eng, "b", toks, [1]), want) < F32_TOL


# ------------------------------------------------------------------------------------------------------------------------
# bfloat16 on the tensor-core kernels
# ------------------------------------------------------------------------------------------------------------------------
TC_LAYERS = [latent_layer(heads=4, dim=16, rot_dim=16, vdim=32, kv_rank=32),                 # prompt portions on per-head keys and values
             attention_layer(heads=8, kv_heads=2, dim=32, size=70, keep_first=9),
             latent_layer(heads=20, dim=8, rot_dim=16, vdim=8, kv_rank=64, mlp=None),        # sizes only the latent-space tiles take
             latent_layer(heads=3, dim=40, rot_dim=8, vdim=64, kv_rank=40, mlp=None),        # per-head portions, single tokens on the plain kernel
             attention_layer(heads=8, kv_heads=8, dim=64, size=33, keep_first=40, mlp=None),
             gla_layer(heads=2, dim=64, vdim=128, mlp=None)]


def _engine_runs(cfg, w, a, b):
    """Whole prompt, portions, and a mixed schedule (a portion of b beside single tokens of a, then both decode) in bfloat16."""
    eng = _engine(cfg, w, torch.bfloat16, page_size=16)
    whole = _whole(eng, "w", a)
    parts = _portions(eng, "p", a, [70, 2, 33, 1, 1, 64])
    eng.release("p")
    ga, gb = [eng.step([("a", a[:100], list(range(100)))])], []
    for i in range(90):
        e = [("a", a[100 + i:101 + i], [0])] + ([("b", b[:40], list(range(40)))] if i == 0 else [("b", b[39 + i:40 + i], [0])] if i <= 50 else [])
        out = eng.step(e)
        ga.append(out[:1])
        if i <= 50:
            gb.append(out[1:])
    return whole, parts, torch.cat(ga), torch.cat(gb)


@pytest.mark.parametrize("layer", range(len(TC_LAYERS)))
def test_tensor_core_paths_layer_by_layer(dev, layer):
    """bfloat16 layers whose sizes the tensor-core kernels take, one at a time (so that rounding noise is not multiplied by later layers):
    whole prompts, portions, single tokens (graph replay) and a mixed batch through the engine, against the oracle and against the same engine
    kept on the plain kernels.  Latent attention: prompt portions on per-head keys and values where the head sizes allow, else (and when told
    so) on tiles in the latent space, single tokens always there, all with the sink; attention: tiles for portions, head groups for single
    tokens, with the kept first positions, the distance bias and the head gate."""
    import qserve_b200.hybrid as hyb

    cfg = make_config([TC_LAYERS[layer]], width=64)
    w = make_weights(cfg, 14 + layer, sharp=2.0)
    a, b = random_tokens(200, cfg["vocab"], 14), random_tokens(90, cfg["vocab"], 15)
    wa, wb = O.forward(cfg, w, a), O.forward(cfg, w, b)
    runs = {}
    for impl in (None, "latent", "plain"):
        hyb.LATENT_IMPL = impl
        hyb.ATTENTION_IMPL = "plain" if impl == "plain" else None
        try:
            runs[impl] = _engine_runs(cfg, w, a, b)
        finally:
            hyb.LATENT_IMPL = hyb.ATTENTION_IMPL = None
    for impl in (None, "latent", "plain"):
        for got, want in zip(runs[impl], (wa, wa, wa[:190], wb)):
            assert row_err(got, want) < 0.06, impl
    for impl in (None, "latent"):
        for f, p in zip(runs[impl], runs["plain"]):
            assert row_err(f, p) < 0.03, impl


def test_tensor_core_paths_stack(dev):
    cfg = make_config(TC_LAYERS, width=64)
    w = make_weights(cfg, 14)
    a, b = random_tokens(200, cfg["vocab"], 14), random_tokens(90, cfg["vocab"], 15)
    wa, wb = O.forward(cfg, w, a), O.forward(cfg, w, b)
    for got, want in zip(_engine_runs(cfg, w, a, b), (wa, wa, wa[:190], wb)):
        assert bf16_close(got, want)


@pytest.mark.parametrize("sink", [-30.0, 0.0, 6.0])
def test_sink_on_every_latent_path(dev, sink):
    """A sink that outweighs every key, an ordinary one and a negligible one: the tensor-core paths against float32 on the plain kernel."""
    import qserve_b200.hybrid as hyb

    cfg = make_config([latent_layer(heads=4, dim=16, rot_dim=16, vdim=32, kv_rank=32, mlp=None)], width=48)
    w = make_weights(cfg, 15)
    w["l0.mix.sink"] = torch.full((4,), sink)
    toks = random_tokens(150, cfg["vocab"], 15)
    want = O.forward(cfg, w, toks)
    assert row_err(_portions(_engine(cfg, w, page_size=16), "a", toks, [100, 1]), want) < F32_TOL
    for impl in (None, "latent", "plain"):
        hyb.LATENT_IMPL = impl
        try:
            got = _portions(_engine(cfg, w, torch.bfloat16, page_size=16), "a", toks, [100, 1])
        finally:
            hyb.LATENT_IMPL = None
        assert row_err(got, want) < 0.05, impl


# ------------------------------------------------------------------------------------------------------------------------
# the framework's own entry points
# ------------------------------------------------------------------------------------------------------------------------
def test_generate_through_scheduler(dev):
    """Greedy generation through Engine.generate: admission, prompt chunks, decoding, retirement; against the oracle's argmax."""
    from qserve_b200.engine import SamplingParams

    cfg = make_config(STACK)
    w = make_weights(cfg, 16)
    prompts = [random_tokens(n, cfg["vocab"], 40 + n) for n in (5, 37, 1, 70, 12, 20)]
    eng = _engine(cfg, w, max_tokens=4 * 96, page_size=16, chunk=24, max_batch_tokens=48)
    outs = eng.generate(prompts, [SamplingParams(max_new_tokens=6)] * len(prompts))
    for p, o in zip(prompts, outs):
        assert o == O.greedy(cfg, w, p, 6)
    assert eng.cache.free_pages() == eng.cache.num_pages


def test_model_folder_and_trace_replay(dev, tmp_path):
    """config.json + model.safetensors on disk -> Engine.from_dir -> a replayed trace with portions, a request that sits out, and reuse."""
    import io
    import json
    import struct

    import numpy as np

    from qserve_b200.engine import Engine, replay_trace

    cfg = make_config(STACK[:3])
    w = {k: _bf(v) for k, v in make_weights(cfg, 17).items()}   # as the file holds them
    (tmp_path / "m").mkdir()
    (tmp_path / "out").mkdir()
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for k, v in w.items():
        raw = v.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    (tmp_path / "m" / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    a, b = random_tokens(50, cfg["vocab"], 17), random_tokens(9, cfg["vocab"], 18)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [29]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[:2], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[30:], "want": [0, 19]}, {"id": "b", "tokens": b[2:], "want": [6]}], "end": ["a", "b"]}]
    eng = Engine.from_dir(str(tmp_path / "m"), torch.float32, max_tokens=128, max_seqs=2, page_size=64)
    log = io.StringIO()
    assert replay_trace(eng, [json.dumps(s) for s in steps], str(tmp_path / "out"), log) == 3
    assert log.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
    wa, wb = O.forward(cfg, w, a), O.forward(cfg, w, b)
    got0 = torch.from_numpy(np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
    got2 = torch.from_numpy(np.fromfile(tmp_path / "out" / "2.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
    assert not (tmp_path / "out" / "1.f32").exists()
    assert row_err(got0, wa[29:30]) < F32_TOL and row_err(got2, torch.stack([wa[30], wa[49], wb[8]])) < F32_TOL
    assert eng.cache.free_pages() == eng.cache.num_pages
