"""Helpers of the Zuzezen tests: small random models (config dict + weights under the design's tensor names)."""
import math

import torch


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def gla_layer(heads=3, dim=12, vdim=20, tau=8.0, rank=5, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp, "_rank": rank}


def latent_layer(heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=24, base=300.0, scaling=True, scale=None, mlp="default", rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}
    if rot_dim:
        m["rot"] = {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}   # rot_dims < rot_dim: the rest of the shared part is not turned
        if scaling:
            m["rot"]["scaling"] = {"factor": 4.0, "original": 48, "fast": 16.0, "slow": 2.0}
    return {"type": "latent_attention", "mixer": m, "mlp": dense() if mlp == "default" else mlp}


def attention_layer(heads=4, kv_heads=2, dim=16, size=24, keep_first=3, scale=None, mlp="default"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale if scale is not None else 1.5 / math.sqrt(dim)}
    if size:
        m["mask"] = {"size": size, "keep_first": keep_first}
    return {"type": "attention", "mixer": m, "mlp": dense() if mlp == "default" else mlp}


def make_config(layers, vocab=83, width=44, eps=1e-5, embed_scale=5.0):
    return {"architecture": "Zuzezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "layers": layers}


def make_weights(cfg, seed=0, sharp=1.0):
    """Random weights, rounded to bfloat16 values (held as float32) so that every dtype sees the same numbers.  `sharp` scales the query
    projections: large values make the softmax maps peaked, so that a key wrongly seen or missed moves the output.  A gla layer's
    "_rank" entry (which no parser reads) is the rank of its decay projection."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    bf = lambda t: t.to(torch.bfloat16).to(torch.float32)
    r = lambda *shape, s=1.0: bf(torch.randn(*shape, generator=g) * s)
    w = {"embed": r(cfg["vocab"], W, s=0.2), "head": r(cfg["vocab"], W, s=2.0 * W ** -0.5), "final.norm": r(W, s=0.2)}
    for i, ly in enumerate(cfg["layers"]):
        p, q, m = f"l{i}.", f"l{i}.mix.", ly["mixer"]
        w[p + "norm1"], w[p + "ls1"] = r(W, s=0.2), bf(0.5 + 0.5 * torch.rand(W, generator=g))
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        if ly["type"] == "gla":
            rank = ly.get("_rank", 5)
            w[q + "q"], w[q + "k"], w[q + "v"] = r(H * D, W, s=2.0 * W ** -0.5), r(H * D, W, s=W ** -0.5), r(H * Dv, W, s=W ** -0.5)
            w[q + "g"], w[q + "norm"] = r(H * Dv, W, s=W ** -0.5), 1.0 + r(Dv, s=0.2)
            w[q + "a1"], w[q + "a2"], w[q + "a2.b"] = r(rank, W, s=W ** -0.5), r(H * D, rank, s=2.0 * rank ** -0.5), 2.0 + r(H * D, s=1.5)
        elif ly["type"] == "latent_attention":
            R, K = m["rot_dim"], m["kv_rank"]
            w[q + "q"] = r(H * (D + R), W, s=sharp * 2.0 * W ** -0.5)
            w[q + "dkv"], w[q + "dkv.norm"] = r(K + R, W, s=W ** -0.5), 1.0 + r(K, s=0.2)
            w[q + "uk"], w[q + "uv"] = r(H * D, K, s=2.0 * K ** -0.5), r(H * Dv, K, s=K ** -0.5)
            w[q + "sink"], w[q + "g"] = r(H, s=1.0), r(H * Dv, W, s=2.0 * W ** -0.5)
        else:
            G = m["kv_heads"]
            w[q + "q"], w[q + "q.b"] = r(H * D, W, s=W ** -0.5), r(H * D, s=0.3)
            w[q + "k"], w[q + "k.b"] = r(G * D, W, s=W ** -0.5), r(G * D, s=0.3)
            w[q + "q.norm"], w[q + "k.norm"] = sharp * (1.0 + r(D, s=0.2)), 2.0 * (1.0 + r(D, s=0.2))
            w[q + "g"] = r(H, W, s=2.0 * W ** -0.5)
        w[q + "o"] = r(W, H * Dv, s=(H * Dv) ** -0.5)
        f = ly.get("mlp")
        if f:
            q = p + "mlp."
            w[p + "norm2"], w[p + "ls2"] = r(W, s=0.2), bf(0.5 + 0.5 * torch.rand(W, generator=g))
            w[q + "gate"], w[q + "gate.b"] = r(f["ff"], W, s=2.0 * W ** -0.5), r(f["ff"], s=0.3)
            w[q + "up"], w[q + "up.b"] = r(f["ff"], W, s=W ** -0.5), r(f["ff"], s=0.3)
            w[q + "down"], w[q + "down.b"] = r(W, f["ff"], s=f["ff"] ** -0.5), r(W, s=0.3)
    return w
