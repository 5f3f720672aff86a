"""CPU tests of the Nusuvik family's host side: config parser and registry, run schedule and pass starts, cache storage, and the float64
restatement on cases worked out by hand."""
import math

import pytest
import torch

from tests import nusuvik_oracle as O
from tests.nusuvik_util import dense, latent_layer, make_config, make_weights, moe


def test_parser_and_registry():
    from qserve_b200.modelcfg import ARCHITECTURES, LatentAttentionMixerConfig, MlpConfig, MoeConfig

    cfg = make_config([latent_layer(), latent_layer(heads=1, dim=4, rot_dim=2, vdim=6, kv_rank=5, q_rank=7, mlp=moe()), latent_layer(mlp=None)],
                      loop=(1, 2, 3), cap=7.5)
    c = ARCHITECTURES["Nusuvik"](cfg)
    assert c.architecture == "Nusuvik" and c.block == "parallel" and c.shared_norm and c.norm_kind == "layer" and c.loop_in
    assert c.logit_softcap == 7.5 and c.norm_offset == 0.0 and c.pair_buckets == 47
    assert c.schedule() == [0, 1, 1, 1, 2] and c.pass_starts() == [1, 2, 3]
    m = c.layers[1].mixer
    assert isinstance(m, LatentAttentionMixerConfig) and (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank) == (1, 4, 2, 6, 5, 7)
    assert m.rot.layout == "half" and m.rot.dims == 2 and m.gate
    f0, f1 = c.layers[0].mlp, c.layers[1].mlp
    assert isinstance(f0, MlpConfig) and not f0.gated and f0.bias and f0.ff == 56
    assert isinstance(f1, MoeConfig) and f1.router == "sigmoid" and f1.correction and (f1.groups, f1.keep, f1.top) == (3, 2, 2)
    assert f1.limit == math.inf and f1.alpha == 1.0 and f1.up_shift == 0.0 and f1.shared_ff == 0
    assert c.layers[2].mlp is None


def test_defaults_without_loop_pair_and_cap():
    from qserve_b200.modelcfg import ARCHITECTURES

    c = ARCHITECTURES["Nusuvik"](make_config([latent_layer()], bigram=None, cap=None))
    assert not c.loop_in and c.pass_starts() == [] and c.schedule() == [0] and c.pair_buckets == 0 and c.logit_softcap == 0.0


@pytest.mark.parametrize("bad", [dict(experts=6, top=2, groups=4, keep=1), dict(experts=6, top=3, groups=3, keep=1), dict(experts=6, top=2, groups=3, keep=4)])
def test_parser_rejects_impossible_routers(bad):
    from qserve_b200.modelcfg import ARCHITECTURES

    with pytest.raises(ValueError):
        ARCHITECTURES["Nusuvik"](make_config([latent_layer(mlp=moe(**bad))]))


def test_other_families_keep_their_defaults():
    from qserve_b200.modelcfg import ARCHITECTURES
    from tests.hybrid_util import attention_layer, make_config as rizurax_config

    c = ARCHITECTURES["Rizurax"](rizurax_config([attention_layer()]))
    assert c.norm_kind == "rms" and not c.shared_norm and not c.loop_in and c.logit_softcap == 0.0
    assert c.layers[0].mlp.gated and not c.layers[0].mlp.bias


def test_cache_holds_one_latent_row_per_position():
    from qserve_b200.cache import HybridCache
    from qserve_b200.modelcfg import ARCHITECTURES

    c = ARCHITECTURES["Nusuvik"](make_config([latent_layer(kv_rank=24, rot_dim=8), latent_layer(kv_rank=10, rot_dim=2)], loop=(0, 1, 2)))
    cache = HybridCache(c, torch.float32, torch.device("cpu"), max_tokens=200, max_seqs=3, page_size=16)
    assert len(cache.runs) == 3  # a looped layer has a cache of its own per pass
    assert [tuple(r["c"].shape) for r in cache.runs] == [(13, 16, 32), (13, 16, 32), (13, 16, 12)]
    st = cache.admit("a")
    cache.reserve("a", 40)
    assert len(st.pages) == 3 and cache.free_pages() == 10
    cache.release("a")
    assert cache.free_pages() == 13 and cache.can_admit()


def test_oracle_router_by_hand():
    """4 experts in 2 groups, 1 group kept, 2 chosen.  Scores s = sigmoid(z); the correction lifts group 1 above group 0 although group 0 holds
    the largest score, so the winners come from group 1 and are weighted by their uncorrected scores."""
    W = 4
    w = {"router": torch.eye(4), "correction": torch.tensor([0.0, -0.9, 0.3, 0.2])}
    z = torch.tensor([[2.0, 0.0, 0.5, -0.5]], dtype=torch.float64)
    spec = {"router": {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}}}
    idx, wt = O.route(spec, w, "", z)
    s = torch.sigmoid(z[0])
    # group scores: (s0 + 0) + (s1 - 0.9) = 0.481, (s2 + 0.3) + (s3 + 0.2) = 1.500
    assert idx.tolist() == [[2, 3]]
    assert torch.allclose(wt[0], torch.stack([s[2], s[3]]) / (s[2] + s[3]))
    assert abs(float(wt.sum()) - 1.0) < 1e-12


def test_oracle_negative_choice_scores_do_not_beat_masked_groups():
    """All choice scores negative: experts of a dropped group must still lose (they count as minus infinity, not as zero)."""
    w = {"router": torch.eye(4), "correction": torch.tensor([-2.0, -2.1, -3.0, -3.1])}
    z = torch.zeros(1, 4, dtype=torch.float64)
    idx, _ = O.route({"router": {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}}}, w, "", z)
    assert sorted(idx[0].tolist()) == [0, 1]


def test_oracle_rotation_and_causality():
    v = torch.arange(12, dtype=torch.float64).view(2, 6)
    out = O.rotate_half(v, torch.tensor([0, 3]), 4, 10.0)
    assert torch.equal(out[0], v[0])  # position 0: no turn
    a = 3.0 * torch.tensor([1.0, 10.0 ** -0.5], dtype=torch.float64)
    assert torch.allclose(out[1, :2], v[1, :2] * torch.cos(a) - v[1, 2:4] * torch.sin(a))
    assert torch.allclose(out[1, 2:4], v[1, 2:4] * torch.cos(a) + v[1, :2] * torch.sin(a))
    assert torch.equal(out[1, 4:], v[1, 4:])
    # a later token never changes an earlier position's logits
    cfg = make_config([latent_layer(), latent_layer(mlp=moe())], loop=(0, 1, 2))
    w = make_weights(cfg, 5)
    toks = [3, 9, 1, 44, 7, 7, 20]
    full = O.forward(cfg, w, toks)
    assert torch.allclose(O.forward(cfg, w, toks[:4]), full[:4], atol=1e-12)
