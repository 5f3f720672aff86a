"""GPU tests of the Toderax family: the engine (model, cache / state manager, scheduler, kernels) against the plain float64 restatement in
tests/toderax_oracle.py, on small random models of several shapes."""
import math

import pytest
import torch

from tests import toderax_oracle as O
from tests.hybrid_util import bf16_close, random_tokens, row_err
from tests.toderax_util import gate_layer, make_config, make_weights, moe, pair_layer

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


MIXED = [gate_layer(), pair_layer(), pair_layer(heads=2, kv_heads=2, dim=8, vdim=8, chunk=7, r_heads=1, r_dim=8, r_vdim=24, rot_dims=4, mlp=None),
         gate_layer(heads=3, dim=20, vdim=8, mlp=moe(experts=3, top=3, ff=16, shared_ff=0))]


# ------------------------------------------------------------------------------------------------------------------------
# each mechanism alone
# ------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("streams,groups,width", [(0, 1, 48), (1, 1, 40), (3, 2, 48), (4, 6, 36), (8, 5, 35), (11, 4, 48)])
def test_embedding_streams_and_group_norm(dev, streams, groups, width):
    """No layers: the scaled embedding in every stream, their sum, the group-wise final norm."""
    cfg = make_config([], streams=streams, groups=groups, width=width, embed_scale=0.5 + streams)
    w = make_weights(cfg, 1)
    toks = random_tokens(40, cfg["vocab"], 1)
    assert row_err(_whole(_engine(cfg, w), "a", toks), O.forward(cfg, w, toks)) < F32_TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams,groups,width", [(1, 1, 40), (3, 2, 48), (8, 5, 35), (2, 1, 2560), (4, 16, 2048), (13, 3, 48), (16, 1, 30)])
def test_stream_norm_kernel(dev, dtype, streams, groups, width):
    """The streams' kernel alone against its formulas: pending write (fp32 or storage-type rows), read coefficients, sum, group-wise norm."""
    from qserve_b200._lib import check, lib

    g = torch.Generator().manual_seed(width + streams)
    T, dt = 5, 0 if dtype == torch.bfloat16 else 1
    s = torch.cuda.current_stream().cuda_stream
    x = torch.randn(T, streams, width, generator=g)
    mix, cout, cin = torch.randn(streams, streams, generator=g), torch.randn(streams, generator=g), torch.randn(streams, generator=g)
    gain = torch.randn(width, generator=g)
    for y_f32 in (True, False):
        y = torch.randn(T, width, generator=g).to(torch.float32 if y_f32 else dtype)
        xd, h, total = x.clone().to(dev), torch.zeros(T, width, dtype=dtype, device=dev), torch.zeros(T, width, device=dev)
        yd, md, od, cd, gd = y.to(dev), mix.to(dev), cout.to(dev), cin.to(dev), gain.to(dev)
        check(lib.qs_hyb_stream_norm(h.data_ptr(), total.data_ptr(), xd.data_ptr(), streams, yd.data_ptr(), 1 if y_f32 else 0, md.data_ptr(),
                                     od.data_ptr(), cd.data_ptr(), gd.data_ptr(), groups, 0.25, 1e-5, T, width, dt, s))
        nx = torch.einsum("st,bsw->btw", mix.double(), x.double()) + cout.double()[None, :, None] * y.double()[:, None, :]
        u = torch.einsum("s,bsw->bw", cin.double(), nx)
        assert torch.allclose(xd.cpu().double(), nx, atol=1e-4, rtol=1e-5)
        assert torch.allclose(total.cpu().double(), u, atol=1e-4, rtol=1e-5)
        assert row_err(h, O.group_norm(u, 0.25 + gain, groups, 1e-5)) < (1e-5 if dtype == torch.float32 else 2.0 ** -8)


@pytest.mark.parametrize("T", [9, 1029, 2050])
@pytest.mark.parametrize("experts,top,width", [(6, 2, 48), (1, 1, 16), (40, 40, 33), (64, 7, 2048), (5, 4, 8), (3, 2, 8200)])
def test_router_kernel(dev, experts, top, width, T):
    """One token per block (few tokens) and several tokens per block sharing the router rows (many tokens)."""
    from qserve_b200._lib import check, lib

    g = torch.Generator().manual_seed(experts)
    h, wr = torch.randn(T, width, generator=g), torch.randn(experts, width, generator=g) * width ** -0.5
    hd, wd = h.to(dev), wr.to(dev)
    route, idx, wt = torch.zeros(T, experts, device=dev), torch.zeros(T, top, dtype=torch.int32, device=dev), torch.zeros(T, top, device=dev)
    check(lib.qs_hyb_moe_router(route.data_ptr(), idx.data_ptr(), wt.data_ptr(), hd.data_ptr(), wd.data_ptr(), T, width, experts, top, 0,
                                None, 1, 1, 1, torch.cuda.current_stream().cuda_stream))
    score = torch.softmax(h.double() @ wr.double().T, -1)
    best = torch.topk(score, top, -1)
    assert torch.equal(idx.cpu().long(), best.indices)
    assert torch.allclose(wt.cpu().double(), best.values, atol=1e-6)
    assert torch.allclose(route.cpu().double(), torch.zeros_like(score).scatter(1, best.indices, best.values), atol=1e-6)


LAYERS = [
    gate_layer(mlp=None), gate_layer(heads=1, dim=40, vdim=8, mlp=None), gate_layer(heads=5, dim=4, vdim=72, mlp=None),
    gate_layer(heads=1, dim=128, vdim=32, mlp=None), gate_layer(heads=2, dim=130, vdim=4, mlp=None),
    gate_layer(heads=2, dim=128, vdim=72, mlp=None), gate_layer(heads=1, dim=64, vdim=136, mlp=None), gate_layer(heads=1, dim=100, vdim=66, mlp=None),
    gate_layer(heads=1, dim=300, vdim=12, mlp=None), gate_layer(heads=1, dim=512, vdim=8, mlp=None),
    pair_layer(heads=2, kv_heads=1, dim=16, vdim=16, chunk=20, r_heads=1, r_dim=260, r_vdim=12, rot_dims=64, mlp=None),
    pair_layer(heads=2, kv_heads=1, dim=16, vdim=16, chunk=33, r_heads=2, r_dim=128, r_vdim=64, rot_dims=64, mlp=None),
    pair_layer(heads=2, kv_heads=1, dim=16, vdim=16, chunk=0, r_heads=1, r_dim=64, r_vdim=130, rot_dims=64, mlp=None),
    pair_layer(mlp=None), pair_layer(heads=3, kv_heads=1, dim=20, vdim=12, chunk=0, r_heads=1, r_dim=8, r_vdim=40, rot_dims=8, mlp=None),
    pair_layer(heads=2, kv_heads=2, dim=64, vdim=160, chunk=64, r_heads=2, r_dim=64, r_vdim=16, rot_dims=32, mlp=None),
    pair_layer(heads=1, kv_heads=1, dim=8, vdim=8, chunk=1, r_heads=4, r_dim=24, r_vdim=8, rot_dims=2, mlp=None),
    pair_layer(heads=8, kv_heads=2, dim=16, vdim=32, chunk=100, r_heads=2, r_dim=128, r_vdim=32, rot_dims=128, base=1e6, mlp=None),
]


@pytest.mark.parametrize("layer", LAYERS, ids=lambda l: l["type"] + "-" + "x".join(str(v) for v in (l["mixer"].get("left") or l["mixer"]).values()
                                                                                 if isinstance(v, int)))
def test_single_mixer_layer(dev, layer):
    cfg = make_config([layer])
    w = make_weights(cfg, 2)
    toks = random_tokens(150, cfg["vocab"], 2)
    taps = []
    got = _engine(cfg, w).step([("a", toks, list(range(len(toks))))], tap=lambda r, x: taps.append(x.clone()))
    want, layers = O.forward(cfg, w, toks, return_layers=True)
    assert row_err(taps[0], layers[0]) < F32_TOL
    assert row_err(got, want) < F32_TOL


@pytest.mark.parametrize("spec", [moe(), moe(experts=1, top=1, ff=8, shared_ff=0), moe(experts=9, top=9, ff=5, shared_ff=64),
                                  moe(experts=33, top=1, ff=16, limit=0.3, shared_ff=7, shared_limit=5.0)],
                         ids=lambda s: "E%d-top%d" % (s["router"]["experts"], s["router"]["top"]))
def test_expert_mixture(dev, spec):
    cfg = make_config([gate_layer(mlp=spec)], streams=2)
    w = make_weights(cfg, 3)
    toks = random_tokens(120, cfg["vocab"], 3)
    taps = []
    got = _engine(cfg, w).step([("a", toks, list(range(len(toks))))], tap=lambda r, x: taps.append(x.clone()))
    want, layers = O.forward(cfg, w, toks, return_layers=True)
    assert row_err(taps[0], layers[0]) < F32_TOL
    assert row_err(got, want) < F32_TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("spec", [moe(experts=6, top=2, ff=24), moe(experts=16, top=4, ff=8, shared_ff=0), moe(experts=3, top=3, ff=40, shared_ff=8),
                                  moe(experts=70, top=5, ff=16)], ids=lambda s: "E%d-top%d" % (s["router"]["experts"], s["router"]["top"]))
def test_sorted_experts_equal_stacked_experts(dev, monkeypatch, dtype, spec):
    """The two ways to run the experts (sorted rows through grouped products; all experts stacked with zero weights for the unused) on the
    same inputs, in a batch large enough that every expert gets rows and in one where most get none."""
    from qserve_b200 import hybrid
    from qserve_b200.modelcfg import MoeConfig

    W, dt = 64, 1 if dtype == torch.float32 else 0
    c = MoeConfig(spec["router"]["experts"], spec["router"]["top"], spec["expert"]["ff"], spec["expert"]["limit"],
                  (spec.get("shared") or {}).get("ff", 0), (spec.get("shared") or {}).get("limit", 0.0))
    cfg = make_config([gate_layer(mlp=spec)], width=W)
    w = {k[len("l0.mlp."):]: v for k, v in make_weights(cfg, 14).items() if k.startswith("l0.mlp.")}
    s = torch.cuda.current_stream().cuda_stream
    ffs = {}
    for impl in ("sorted", "dense"):
        monkeypatch.setattr(hybrid, "MOE_IMPL", impl)
        ffs[impl] = hybrid.MoeFeedForward(c, w, W, dtype, dev)
        assert ffs[impl].impl == impl
    for T in (300, 1, 3):
        h = torch.randn(T, W, generator=torch.Generator().manual_seed(T)).to(dtype).to(dev)
        a, a32 = ffs["sorted"].run(h, dt, s)
        b, b32 = ffs["dense"].run(h, dt, s)
        assert a32 and not b32
        want = O.expert_mixture(h.double().cpu(), w, spec)
        if dtype == torch.float32:
            assert row_err(a, want) < 1e-5 and row_err(b, want) < 1e-5
        else:  # the same router choices (same kernel, same input); the two differ by where they round
            assert row_err(a, b) < 2e-2 and row_err(a, want) < 2e-2


@pytest.mark.parametrize("streams,groups", [(0, 1), (1, 3), (4, 2)])
def test_stack_of_layers(dev, streams, groups):
    cfg = make_config(MIXED, streams=streams, groups=groups)
    w = make_weights(cfg, 4)
    toks = random_tokens(90, cfg["vocab"], 4)
    taps = []
    got = _engine(cfg, w).step([("a", toks, list(range(len(toks))))], tap=lambda r, x: taps.append(x.clone()))
    want, layers = O.forward(cfg, w, toks, return_layers=True)
    assert len(taps) == layers.shape[0] == len(MIXED)
    for r, t in enumerate(taps):
        assert row_err(t, layers[r]) < F32_TOL, f"layer {r}"
    assert row_err(got, want) < F32_TOL


# expert choices are left out of the bfloat16 comparisons (every expert runs): a close call of the router may fall the other way in 16 bits
BF16 = [gate_layer(mlp=moe(experts=4, top=4)), pair_layer(mlp=moe(experts=4, top=4)),
        pair_layer(heads=8, kv_heads=2, dim=32, vdim=64, chunk=50, r_heads=2, r_dim=64, r_vdim=32, rot_dims=32, mlp=None),  # the tensor-core kernels' sizes
        gate_layer(heads=2, dim=64, vdim=16, mlp=moe(experts=2, top=2, ff=16, shared_ff=0))]


def test_bfloat16_engine_stays_within_rounding(dev):
    cfg = make_config(BF16)
    w = make_weights(cfg, 5)
    toks = random_tokens(200, cfg["vocab"], 5)
    assert bf16_close(_whole(_engine(cfg, w, torch.bfloat16), "a", toks), O.forward(cfg, w, toks))


# ------------------------------------------------------------------------------------------------------------------------
# the same logits however the tokens are cut, batched and placed
# ------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompt_then_token_by_token(dev, dtype):
    close = (lambda a, b: row_err(a, b) < F32_TOL) if dtype == torch.float32 else bf16_close
    layers = MIXED if dtype == torch.float32 else BF16
    cfg = make_config(layers)
    w = make_weights(cfg, 6)
    toks = random_tokens(200, cfg["vocab"], 6)
    want = O.forward(cfg, w, toks)
    eng = _engine(cfg, w, dtype)
    got = torch.cat([eng.step([("a", toks[:61], list(range(61)))]), _portions(eng, "a", toks[61:], [1])])
    assert close(got, want)
    eng.release("a")
    got = _portions(eng, "b", toks, [1])  # from the very first token on, one by one
    assert close(got, want)


@pytest.mark.parametrize("sizes", [[2], [3, 2, 64, 5], [63, 1, 65], [128, 7], [23, 1, 1]])
def test_portions_of_a_prompt(dev, sizes):
    cfg = make_config(MIXED)
    w = make_weights(cfg, 7)
    toks = random_tokens(197, cfg["vocab"], 7)
    assert row_err(_portions(_engine(cfg, w), "a", toks, sizes), O.forward(cfg, w, toks)) < F32_TOL


@pytest.mark.parametrize("sizes", [[1], [40, 1, 2, 70]])
def test_wide_states_in_long_and_short_runs(dev, sizes):
    """Head sizes for which long runs of tokens and single tokens take different thread layouts of the recurrence."""
    cfg = make_config([gate_layer(heads=2, dim=128, vdim=72, mlp=None),
                       pair_layer(heads=2, kv_heads=1, dim=16, vdim=16, chunk=33, r_heads=1, r_dim=64, r_vdim=130, rot_dims=64, mlp=None)])
    w = make_weights(cfg, 15)
    toks = random_tokens(120, cfg["vocab"], 15)
    assert row_err(_portions(_engine(cfg, w), "a", toks, sizes), O.forward(cfg, w, toks)) < F32_TOL


@pytest.mark.parametrize("dtype,layers", [(torch.float32, MIXED), (torch.bfloat16, BF16)], ids=["f32", "bf16"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(dev, dtype, layers):
    """Four live sequences at most, a pool that cannot hold all requests at once: pages and slots are handed out again, portions of some
    requests run beside single tokens of others, and every position must equal the request run alone."""
    cfg = make_config(layers)
    w = make_weights(cfg, 8)
    lens = [150, 70, 1, 33, 129, 64, 90]
    reqs = {f"r{i}": random_tokens(n, cfg["vocab"], 10 + i) for i, n in enumerate(lens)}
    want = {k: O.forward(cfg, w, v) for k, v in reqs.items()}
    eng = _engine(cfg, w, dtype, max_tokens=6 * 64, max_seqs=4)
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    waiting, live = list(reqs), []
    sizes = [2, 17, 1, 64, 5, 1, 1, 40]
    step = 0
    while waiting or live:
        def pages(k):
            return -(-len(reqs[k]) // 64)
        while waiting and len(live) < 4 and sum(pages(k) for k in live) + pages(waiting[0]) <= 6:
            live.append(waiting.pop(0))
        entries, ends = [], []
        for j, k in enumerate(live):
            if (step + j) % 5 == 4 and len(live) > 1:
                continue  # left out of this step
            n = min(sizes[(step + 3 * j) % len(sizes)], len(reqs[k]) - at[k])
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
        out = eng.step(entries)
        r = 0
        for k, t, _ in entries:
            got[k].append(out[r:r + len(t)])
            r += len(t)
            at[k] += len(t)
            if at[k] == len(reqs[k]):
                ends.append(k)
        for k in ends:
            eng.release(k)
            live.remove(k)
        step += 1
    assert eng.cache.free_pages() == 6 and len(eng.cache.slots) == 4
    for k in reqs:
        if dtype == torch.float32:
            assert row_err(torch.cat(got[k]), want[k]) < F32_TOL, k
        else:
            assert bf16_close(torch.cat(got[k]), want[k]), k
            alone = _whole(eng, "alone", reqs[k])  # the same kernels on the whole prompt: the batch changes nothing beyond rounding
            assert row_err(torch.cat(got[k]), alone) < 0.03, k


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_graph_replay_equals_eager_launches(dev, dtype):
    cfg = make_config(MIXED if dtype == torch.float32 else BF16)
    w = make_weights(cfg, 13)
    reqs = [random_tokens(n, cfg["vocab"], 30 + i) for i, n in enumerate([40, 90, 23, 70])]
    outs = []
    for graphs in (True, False):
        eng = _engine(cfg, w, dtype, max_tokens=5 * 64, max_seqs=3, use_graphs=graphs)
        got = []
        eng.step([(i, reqs[i][:20], []) for i in range(3)])
        for t in range(20, 23):
            got.append(eng.step([(i, reqs[i][t:t + 1], [0]) for i in range(3)]))
        eng.release(2)
        eng.step([(3, reqs[3][:50], [])])
        for t in range(23, 40):
            got.append(eng.step([(0, reqs[0][t:t + 1], [0]), (1, reqs[1][t:t + 1], [0]), (3, reqs[3][t + 27:t + 28], [0])]))
        assert bool(eng._graphs) == graphs
        outs.append(torch.cat(got))
    assert row_err(outs[0], outs[1]) < (1e-5 if dtype == torch.float32 else 2e-2)


def test_long_decoding(dev):
    cfg = make_config([gate_layer(), pair_layer(chunk=50)])
    w = make_weights(cfg, 9)
    toks = random_tokens(330, cfg["vocab"], 9)
    eng = _engine(cfg, w)
    eng.step([("a", toks[:10], [])])
    got = _portions(eng, "a", toks[10:], [1])
    assert row_err(got, O.forward(cfg, w, toks)[10:]) < F32_TOL


# ------------------------------------------------------------------------------------------------------------------------
# one key that matters: far back, at page borders, just inside and just outside the chunk -- in a prompt and when decoding
# ------------------------------------------------------------------------------------------------------------------------
def _needle_model(n_tokens, needle, chunk, dim=16, vdim=8, sink=0.0):
    """One side-by-side layer whose retention side is switched off (gain 0), one attention head, identity-like projections: the stream carries
    q | k | v directly.  The last token's query points along the key at `needle`; values are distinct per position."""
    width = 2 * dim + vdim
    layer = pair_layer(heads=1, kv_heads=1, dim=dim, vdim=vdim, chunk=chunk, scale=1.0, r_heads=1, r_dim=8, r_vdim=8, rot_dims=4, mlp=None)
    cfg = make_config([layer], vocab=n_tokens + 1, width=width, streams=0, groups=1, eps=1e-6, embed_scale=1.0)
    w = make_weights(cfg, 10)
    eye = torch.eye(width)
    w["l0.mix.left.q"], w["l0.mix.left.k"], w["l0.mix.left.v"] = eye[:dim].clone(), eye[dim:2 * dim].clone(), eye[2 * dim:].clone()
    for n, size in (("q.b", dim), ("k.b", dim), ("v.b", vdim)):
        w["l0.mix.left." + n] = torch.zeros(size)
    w["l0.mix.left.temp"], w["l0.mix.left.sink"] = torch.tensor([2.5]), torch.tensor([sink])
    w["l0.norm1"], w["l0.mix.right.out"] = torch.ones(width), torch.zeros(width)
    gen = torch.Generator().manual_seed(3)
    emb = torch.randn(n_tokens + 1, width, generator=gen)
    mark = torch.randn(dim, generator=gen) * 4.0
    unit = mark / mark.norm()
    emb[:, dim:2 * dim] -= (emb[:, dim:2 * dim] @ unit)[:, None] * unit[None, :]  # no other key has a part along the mark
    emb[n_tokens, :dim] = mark             # the query of the last token (vocab id n_tokens)
    emb[needle, dim:2 * dim] = mark        # the key of the needle (token id = its position)
    w["embed"] = emb.to(torch.bfloat16).float()
    toks = list(range(n_tokens - 1)) + [n_tokens]
    return cfg, w, toks


@pytest.mark.parametrize("chunk,needle,seen", [(0, 0, True), (0, 63, True), (0, 64, True), (0, 290, True), (100, 200, True), (100, 199, False),
                                                (100, 201, True), (100, 255, True), (100, 256, True), (100, 0, False), (100, 100, False),
                                                (64, 256, True), (64, 255, False), (299, 0, False), (300, 0, True), (150, 150, True), (150, 149, False)])
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_inside_or_outside_the_chunk(dev, chunk, needle, seen, decode):
    n = 300
    cfg, w, toks = _needle_model(n, needle, chunk)
    want = O.forward(cfg, w, toks)[-1:]
    # a needle the last token sees must matter, one outside its chunk must not: the oracle's answer moves, or stays, when the needle goes
    w2 = {k: v.clone() for k, v in w.items()}
    w2["embed"][needle, :] = w2["embed"][(needle + 1) % (n - 1), :]
    moved = row_err(O.forward(cfg, w2, toks)[-1:], want)
    assert moved > 50 * F32_TOL if seen else moved < 1e-9
    eng = _engine(cfg, w)
    if decode:
        eng.step([("a", toks[:-1], [])])
        got = eng.step([("a", toks[-1:], [0])])
    else:
        eng.step([("a", toks[:130], [])])
        got = eng.step([("a", toks[130:], [n - 131])])
    assert row_err(got, want) < F32_TOL


@pytest.mark.parametrize("chunk,needle,seen", [(0, 0, True), (100, 200, True), (100, 199, False), (64, 256, True), (64, 255, False), (300, 0, True),
                                                (150, 150, True), (150, 149, False)])
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_inside_or_outside_the_chunk_on_the_fast_kernels(dev, chunk, needle, seen, decode):
    """The same in bfloat16 with head sizes the tensor-core prompt and single-token kernels take."""
    n = 300
    cfg, w, toks = _needle_model(n, needle, chunk, dim=16, vdim=32)
    want = O.forward(cfg, w, toks)[-1:]
    eng = _engine(cfg, w, torch.bfloat16)
    if decode:
        eng.step([("a", toks[:-1], [])])
        got = eng.step([("a", toks[-1:], [0])])
    else:
        eng.step([("a", toks[:130], [])])
        got = eng.step([("a", toks[130:], [n - 131])])
    assert row_err(got, want) < 0.05


@pytest.mark.parametrize("shape", [(4, 2, 16, 32, 24, 0, True), (6, 3, 48, 96, 100, 0, True), (8, 2, 32, 64, 64, 0, False), (2, 1, 64, 128, 1, 0, True),
                                   (3, 3, 16, 256, 0, 37, True), (16, 1, 16, 32, 130, 50, True), (4, 4, 128, 128, 0, 0, True)],
                         ids=lambda s: "H%d-G%d-D%d-Dv%d-chunk%d-window%d-sink%d" % s)
def test_fast_attention_kernels_match_the_plain_kernel_with_masks_and_sinks(dev, shape):
    """Same bfloat16 inputs and cache through the tensor-core kernels and through the plain kernel, with chunks, windows and sinks: prompt
    portions with and without context, portions that cross chunk edges and end inside a page, short portions and single tokens in one batch."""
    from qserve_b200.hybrid import MultiMapAttentionMixer, StepBatch
    from qserve_b200.modelcfg import AttentionMixerConfig

    H, G, D, Dv, chunk, window, sink = shape
    m = AttentionMixerConfig(H, G, D, Dv, None, 2.0 * D ** -0.5, bias=True, qk_norm=True, head_temp=True, sink=sink, chunk=chunk, window=window)
    g = torch.Generator().manual_seed(5)
    r = lambda *s: torch.randn(*s, generator=g)
    w = {"q": r(H * D, 8), "k": r(G * D, 8), "v": r(G * Dv, 8), "o": r(8, H * Dv), "q.b": r(H * D), "k.b": r(G * D), "v.b": r(G * Dv),
         "temp": 1.0 + torch.rand(H, generator=g), "sink": r(H) + 2.0}
    mixer = MultiMapAttentionMixer(m, w, 1e-5, torch.bfloat16, dev)
    pages, page = 40, 64
    kpool = torch.zeros(pages, page, G, D, dtype=torch.bfloat16, device=dev)
    vpool = torch.zeros(pages, page, G, Dv, dtype=torch.bfloat16, device=dev)
    table = torch.randperm(pages, generator=g).to(torch.int32).view(4, 10).to(dev)
    steps = [[(0, 0, -1, [0] * 200), (1, 0, -1, [0] * 70), (2, 0, -1, [0] * 3), (3, 0, -1, [0] * 16)],
             [(0, 200, 0, [0] * 1), (1, 70, 0, [0] * 130), (2, 3, 0, [0] * 15), (3, 16, 0, [0] * 64)],
             [(0, 201, 0, [0] * 90), (1, 200, 0, [0] * 1), (2, 18, 0, [0] * 1), (3, 80, 0, [0] * 17)],
             [(0, 291, 0, [0] * 15), (1, 201, 0, [0] * 15), (2, 19, 0, [0] * 15), (3, 97, 0, [0] * 15)],
             [(0, 306, 0, [0] * 1), (3, 112, 0, [0] * 1)]]
    for entries in steps:
        b = StepBatch.build(entries, table, dev)
        T = b.n_tokens
        proj = (r(T, mixer.in_features) * 1.5).to(torch.bfloat16).to(dev)
        outs = []
        for fast in (True, False):
            p2, out = proj.clone(), torch.zeros(T, H * Dv, dtype=torch.bfloat16, device=dev)
            scratch = torch.empty(mixer.scratch_floats(T), dtype=torch.float32, device=dev) if fast else None
            mixer.run(p2, out, b, {"k": kpool, "v": vpool}, page, scratch, 0, torch.cuda.current_stream().cuda_stream)
            outs.append(out.float())
        torch.cuda.synchronize()
        d = (outs[0] - outs[1]).abs()
        assert float(d.max()) <= 2.0 ** -6 * float(outs[1].abs().max()) and float(d.mean()) < 1e-3 * float(outs[1].abs().mean())


def test_sink_takes_its_share(dev):
    """A large sink leaves the values little weight; the engine follows the oracle for small, moderate and large sinks."""
    outs = []
    for sink in (-20.0, 2.0, 12.0):
        cfg, w, toks = _needle_model(120, 60, 50, sink=sink)
        want = O.forward(cfg, w, toks)
        outs.append(want)
        assert row_err(_whole(_engine(cfg, w), "a", toks), want) < F32_TOL
    assert row_err(outs[0], outs[1]) > 50 * F32_TOL and row_err(outs[1], outs[2]) > 50 * F32_TOL


@pytest.mark.parametrize("kind", ["gate", "retention"])
def test_state_remembers_an_early_token(dev, kind):
    """A recurrent layer that forgets slowly: what the first token wrote is still read hundreds of tokens later, through portions and slots."""
    if kind == "gate":
        cfg = make_config([gate_layer(heads=2, dim=16, vdim=16, mlp=None)], streams=2)
        w = make_weights(cfg, 11)
        w["l0.mix.lower"] = torch.full((32,), 0.998046875)
    else:
        cfg = make_config([pair_layer(r_heads=2, r_dim=16, r_vdim=16, rot_dims=16, decay=[0.99951171875, 0.998046875], mlp=None)], streams=2)
        w = make_weights(cfg, 11)
        w["l0.mix.left.out"] = torch.zeros(cfg["width"])
    toks = random_tokens(400, cfg["vocab"], 11)
    want = O.forward(cfg, w, toks)
    other = list(toks)
    other[0] = (toks[0] + 1) % cfg["vocab"]
    assert row_err(O.forward(cfg, w, other)[-1:], want[-1:]) > 20 * F32_TOL
    eng = _engine(cfg, w)
    eng.step([("a", toks[:5], [])])
    eng.step([("a", toks[5:399], [])])
    assert row_err(eng.step([("a", toks[399:], [0])]), want[-1:]) < F32_TOL


# ------------------------------------------------------------------------------------------------------------------------
# generation through the engine's own entry point and scheduler
# ------------------------------------------------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler(dev):
    cfg = make_config(MIXED)
    w = make_weights(cfg, 12)
    prompts = [random_tokens(n, cfg["vocab"], 20 + i) for i, n in enumerate([5, 140, 33, 1, 70, 12])]
    from qserve_b200.engine import SamplingParams

    eng = _engine(cfg, w, max_tokens=7 * 64, max_seqs=3, max_batch_tokens=96, chunk=48)
    outs = eng.generate(prompts, [SamplingParams(max_new_tokens=8)] * len(prompts))
    assert eng.cache.free_pages() == 7 and len(eng.cache.slots) == 3
    for p, o in zip(prompts, outs):
        assert len(o) == 8
        seq = list(p)
        for tok in o:  # every chosen token is the oracle's argmax (up to ties within rounding)
            lg = O.forward(cfg, w, seq)[-1]
            assert lg[tok] >= lg.max() - 1e-3 * lg.abs().max(), (len(p), len(seq))
            seq.append(tok)
