"""CPU tests of the Zuzezen family's host side: config parser and registry, rotary frequencies, distance-bias slopes, cache storage, and the
float64 restatement on cases worked out by hand."""
import math

import pytest
import torch

from tests import zuzezen_oracle as O
from tests.zuzezen_util import attention_layer, dense, gla_layer, latent_layer, make_config, make_weights


def test_parser_and_registry():
    from qserve_b200.modelcfg import (ARCHITECTURES, AttentionMixerConfig, GatedLinearMixerConfig, LatentAttentionMixerConfig, MlpConfig)

    cfg = make_config([gla_layer(), latent_layer(heads=1, dim=4, rot_dim=2, vdim=6, kv_rank=5), attention_layer(heads=6, kv_heads=3, dim=8, size=9, keep_first=2),
                       gla_layer(heads=1, dim=7, vdim=3, tau=2.5, mlp=dense(9))], embed_scale=3.5)
    c = ARCHITECTURES["Zuzezen"](cfg)
    assert c.architecture == "Zuzezen" and c.block == "post" and c.layer_scale and c.norm_kind == "rms" and c.norm_offset == 1.0
    assert c.embed_scale == 3.5 and c.schedule() == [0, 1, 2, 3] and c.pair_buckets == 0 and c.logit_softcap == 0.0
    g = c.layers[0].mixer
    assert isinstance(g, GatedLinearMixerConfig) and (g.heads, g.dim, g.vdim, g.tau) == (3, 12, 20, 8.0) and c.layers[0].mlp is None
    m = c.layers[1].mixer
    assert isinstance(m, LatentAttentionMixerConfig) and (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank) == (1, 4, 2, 6, 5, 0)
    assert m.rot.layout == "interleaved" and m.rot.factor == 4.0 and m.sink and m.gate and m.gate_wide
    a = c.layers[2].mixer
    assert isinstance(a, AttentionMixerConfig) and (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.keep_first) == (6, 3, 8, 8, 9, 2)
    assert a.rot is None and a.bias and a.qk_norm and a.qk_gain and a.tied_values and a.head_gate and a.maps == 1 and not a.sink
    f = c.layers[3].mlp
    assert isinstance(f, MlpConfig) and f.gated and f.bias and f.act == "silu" and f.ff == 9


def test_parser_rejects_unknown_parts():
    from qserve_b200.modelcfg import ARCHITECTURES

    with pytest.raises(ValueError):
        ARCHITECTURES["Zuzezen"](make_config([{"type": "delta", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError):
        ARCHITECTURES["Zuzezen"](make_config([gla_layer(mlp={"kind": "moe", "ff": 8})]))
    bad = attention_layer()
    bad["mixer"]["vdim"] = bad["mixer"]["dim"] + 1   # values are the keys: one size
    with pytest.raises(ValueError):
        ARCHITECTURES["Zuzezen"](make_config([bad]))


def test_other_families_keep_their_defaults():
    from qserve_b200.modelcfg import ARCHITECTURES
    from tests.hybrid_util import attention_layer as rizurax_attention, make_config as rizurax_config

    c = ARCHITECTURES["Rizurax"](rizurax_config([rizurax_attention()]))
    a = c.layers[0].mixer
    assert c.block == "parallel" and not c.layer_scale
    assert not (a.keep_first or a.qk_gain or a.tied_values or a.head_gate) and a.distance_slope == 0.0 and a.slopes() is None
    assert c.layers[0].mlp.act == "gelu_tanh"


def test_slopes_halve_geometrically():
    from qserve_b200.modelcfg import ARCHITECTURES

    a = ARCHITECTURES["Zuzezen"](make_config([attention_layer(heads=4, kv_heads=1)])).layers[0].mixer
    assert a.slopes() == [0.25, 0.0625, 0.015625, 0.00390625]
    a = ARCHITECTURES["Zuzezen"](make_config([attention_layer(heads=3, kv_heads=3)])).layers[0].mixer
    assert a.slopes() == pytest.approx([2.0 ** (-8 / 3), 2.0 ** (-16 / 3), 2.0 ** -8])


@pytest.mark.parametrize("scaling", [None, {"factor": 4.0, "original": 48, "fast": 16.0, "slow": 2.0}, {"factor": 1.5, "original": 4096, "fast": 32.0, "slow": 1.0}])
def test_rotary_frequencies_match_the_restatement(scaling):
    from qserve_b200.modelcfg import _parse_rot

    rot = {"dims": 12, "base": 700.0}
    if scaling:
        rot["scaling"] = scaling
    r = _parse_rot(rot)
    cos, sin = O.rotary_table(rot, 6)
    f, amp = torch.tensor(r.inv_freq(), dtype=torch.float64), r.amplitude()
    ang = torch.arange(6, dtype=torch.float64)[:, None] * f[None, :]
    assert torch.allclose(cos, amp * torch.cos(ang), atol=1e-13) and torch.allclose(sin, amp * torch.sin(ang), atol=1e-13)
    if scaling:
        assert amp == pytest.approx(1.0 + 0.1 * math.log(scaling["factor"]))
        plain = [700.0 ** (-2.0 * i / 12) for i in range(6)]
        assert all(p / scaling["factor"] - 1e-15 <= x <= p + 1e-15 for x, p in zip(r.inv_freq(), plain))


def test_cache_storage_per_mixer():
    from qserve_b200.cache import HybridCache
    from qserve_b200.modelcfg import ARCHITECTURES

    c = ARCHITECTURES["Zuzezen"](make_config([gla_layer(heads=2, dim=6, vdim=10), latent_layer(kv_rank=10, rot_dim=2), attention_layer(heads=4, kv_heads=2, dim=8)]))
    cache = HybridCache(c, torch.float32, torch.device("cpu"), max_tokens=200, max_seqs=3, page_size=16)
    assert tuple(cache.runs[0]["state"].shape) == (3, 2, 6, 10) and cache.runs[0]["state"].dtype == torch.float32
    assert tuple(cache.runs[1]["c"].shape) == (13, 16, 12)
    assert tuple(cache.runs[2]["k"].shape) == (13, 16, 2, 8) and tuple(cache.runs[2]["v"].shape) == (13, 16, 2, 8)
    st = cache.admit("a")
    cache.reserve("a", 40)
    assert len(st.pages) == 3 and cache.free_pages() == 10
    cache.release("a")
    assert cache.free_pages() == 13 and cache.can_admit()


def test_oracle_rotation_by_hand():
    v = torch.arange(12, dtype=torch.float64).view(2, 6)
    cos, sin = O.rotary_table({"dims": 4, "base": 10.0}, 4)
    out = O.rotate_pairs(torch.stack([v[0], v[1]]), cos[[0, 3]], sin[[0, 3]])
    assert torch.equal(out[0], v[0])  # position 0: no turn
    a = 3.0 * torch.tensor([1.0, 10.0 ** -0.5], dtype=torch.float64)
    assert torch.allclose(out[1, 0:4:2], v[1, 0:4:2] * torch.cos(a) - v[1, 1:4:2] * torch.sin(a))
    assert torch.allclose(out[1, 1:4:2], v[1, 1:4:2] * torch.cos(a) + v[1, 0:4:2] * torch.sin(a))
    assert torch.equal(out[1, 4:], v[1, 4:])


def test_oracle_window_keeps_first_positions():
    """One head, identity-like weights: with a window of 2 that keeps position 0, the query at position 3 mixes the values of positions 0, 2
    and 3 only; moving position 1's input must not move its output, moving position 0's must."""
    cfg = make_config([attention_layer(heads=1, kv_heads=1, dim=4, size=2, keep_first=1, mlp=None)], width=4, vocab=9)
    w = make_weights(cfg, 1)
    m, mw = cfg["layers"][0]["mixer"], {k[7:]: v.double() for k, v in w.items() if k.startswith("l0.mix.")}
    h = torch.randn(4, 4, dtype=torch.float64, generator=torch.Generator().manual_seed(3))
    base = O.window_attention(h, m, mw, 1e-5)
    h1, h0 = h.clone(), h.clone()
    h1[1] += 1.0
    h0[0] += 1.0
    assert torch.allclose(O.window_attention(h1, m, mw, 1e-5)[3], base[3], atol=1e-13)
    assert not torch.allclose(O.window_attention(h0, m, mw, 1e-5)[3], base[3], atol=1e-6)


def test_oracle_sink_takes_weight_without_a_value():
    """A very large sink empties the head's output; a very small one leaves plain softmax."""
    cfg = make_config([latent_layer(heads=1, dim=4, rot_dim=2, vdim=3, kv_rank=5, mlp=None)], width=6, vocab=9)
    w = make_weights(cfg, 2)
    m, mw = cfg["layers"][0]["mixer"], {k[7:]: v.double() for k, v in w.items() if k.startswith("l0.mix.")}
    h = torch.randn(5, 6, dtype=torch.float64, generator=torch.Generator().manual_seed(4))
    mw["sink"] = torch.tensor([60.0], dtype=torch.float64)
    assert float(O.latent_attention(h, m, mw, 1e-5).abs().max()) < 1e-12
    mw["sink"] = torch.tensor([-60.0], dtype=torch.float64)
    lo = O.latent_attention(h, m, mw, 1e-5)
    mw["sink"] = torch.tensor([-80.0], dtype=torch.float64)
    assert torch.allclose(O.latent_attention(h, m, mw, 1e-5), lo, atol=1e-13) and float(lo.abs().max()) > 1e-3


def test_oracle_gated_linear_state_and_causality():
    """The recurrence can be cut anywhere when the state is carried; a later token never changes an earlier position's logits."""
    cfg = make_config([gla_layer(), latent_layer(), attention_layer(), gla_layer(mlp=dense(12))])
    w = make_weights(cfg, 5)
    toks = [3, 9, 1, 44, 7, 7, 20]
    full = O.forward(cfg, w, toks)
    assert torch.allclose(O.forward(cfg, w, toks[:4]), full[:4], atol=1e-12)
    m, mw = cfg["layers"][0]["mixer"], {k[7:]: v.double() for k, v in w.items() if k.startswith("l0.mix.")}
    h = torch.randn(6, cfg["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(6))
    # a decay of one (huge logits) and tau = 1 make the state a plain running sum: o_t = (sum_{s<=t} k_s v_s^T)^T q_t
    mw2 = dict(mw)
    mw2["a2.b"] = torch.full_like(mw["a2.b"], 40.0)
    mw2["norm"], mw2["g"], mw2["o"] = torch.ones_like(mw["norm"]), mw["g"], torch.eye(m["heads"] * m["vdim"], dtype=torch.float64)
    got = O.gated_linear(h, dict(m, tau=1.0), mw2, 0.0)
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ mw["q"].T).view(6, H, D) / math.sqrt(D)
    k, v = (h @ mw["k"].T).view(6, H, D), (h @ mw["v"].T).view(6, H, Dv)
    o = torch.stack([sum((q[t] * k[s]).sum(-1, keepdim=True) * v[s] for s in range(t + 1)) for t in range(6)])
    want = (o / o.pow(2).mean(-1, keepdim=True).sqrt()).reshape(6, -1) * O.silu(h @ mw["g"].T)
    assert torch.allclose(got, want, atol=1e-9)
