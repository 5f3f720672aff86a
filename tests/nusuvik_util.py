"""Helpers of the Nusuvik tests: small random models (config dict + weights under the design's tensor names)."""
import math

import torch


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, groups=3, keep=2):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}, "expert": {"ff": ff}}


def latent_layer(heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=24, q_rank=40, base=300.0, scale=None, mlp="default"):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}
    if rot_dim:
        m["rot"] = {"dims": rot_dim, "base": base}
    return {"type": "latent_attention", "mixer": m, "mlp": dense() if mlp == "default" else mlp}


def make_config(layers, vocab=83, width=44, loop=None, bigram=(47, 29, 3), eps=1e-5, cap=9.0):
    cfg = {"architecture": "Nusuvik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    if cap:
        cfg["logit_softcap"] = cap
    return cfg


def make_weights(cfg, seed=0, sharp=1.0):
    """Random weights, rounded to bfloat16 values (held as float32) so that every dtype sees the same numbers.  `sharp` scales the query
    up-projection: large values make the softmax maps peaked, so that a key wrongly seen or missed moves the output."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    bf = lambda t: t.to(torch.bfloat16).to(torch.float32)
    r = lambda *shape, s=1.0: bf(torch.randn(*shape, generator=g) * s)
    w = {"embed": r(cfg["vocab"], W), "head": r(cfg["vocab"], W, s=2.0 * W ** -0.5), "final.norm": 1.0 + r(W, s=0.2), "final.norm.b": r(W, s=0.2)}
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        w["bigram"] = r(bg["buckets"] + 1, W, s=0.5)
    if cfg.get("loop"):
        w["loop.in"] = r(W, 2 * W, s=W ** -0.5)
    for i, ly in enumerate(cfg["layers"]):
        p, m = f"l{i}.", ly["mixer"]
        w[p + "norm1"], w[p + "norm1.b"] = 1.0 + r(W, s=0.2), r(W, s=0.2)
        H, D, R, Dv, K, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        q = p + "mix."
        w[q + "dq"], w[q + "dq.norm"], w[q + "uq"] = r(Q, W, s=W ** -0.5), 1.0 + r(Q, s=0.2), r(H * (D + R), Q, s=sharp * 2.0 * Q ** -0.5)
        w[q + "dkv"], w[q + "dkv.norm"] = r(K + R, W, s=W ** -0.5), 1.0 + r(K, s=0.2)
        w[q + "uk"], w[q + "uv"] = r(H * D, K, s=2.0 * K ** -0.5), r(H * Dv, K, s=K ** -0.5)
        w[q + "g"], w[q + "o"] = r(H, W, s=2.0 * W ** -0.5), r(W, H * Dv, s=(H * Dv) ** -0.5)
        f = ly.get("mlp")
        if not f:
            continue
        q = p + "mlp."
        if f["kind"] == "dense":
            w[q + "up"], w[q + "up.b"] = r(f["ff"], W, s=W ** -0.5), r(f["ff"], s=0.3)
            w[q + "down"], w[q + "down.b"] = r(W, f["ff"], s=f["ff"] ** -0.5), r(W, s=0.3)
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            for e in range(E):
                w[f"{q}e{e}.gate"], w[f"{q}e{e}.up"], w[f"{q}e{e}.down"] = r(ff, W, s=2.0 * W ** -0.5), r(ff, W, s=2.0 * W ** -0.5), r(W, ff, s=ff ** -0.5)
            w[q + "router"] = r(E, W, s=3.0 * W ** -0.5)
            w[q + "correction"] = r(E, s=0.4)   # large enough to change the choice, and to make choice scores negative
    return w
