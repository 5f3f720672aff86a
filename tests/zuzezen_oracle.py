"""Plain float64 restatement of the Zuzezen family, one function per mechanism, for the tests.  Whole sequences only: no cache, no state
carried between calls, no batching -- the engine's paged / chunked / batched results are compared against this.

Notation: n tokens at positions 0 .. n-1, h the [n, width] input of a sublayer, weights under the design's tensor names (a mixer sees them
without the "<layer>.mix." prefix).  Linear weights are [out, in]."""
import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


# ---------------------------------------------------------------------------------------------------------------------------------
# rotary angles: plain frequencies base^(-2i/dims), optionally blended towards f / factor by a linear ramp over the pair index
# ---------------------------------------------------------------------------------------------------------------------------------
def rotary_table(rot, n):
    """cos and sin [n, dims / 2] (already times the amplitude) for positions 0 .. n-1."""
    dims, base = rot["dims"], rot["base"]
    freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        turns = lambda t: dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo, hi = max(math.floor(turns(sc["fast"])), 0), min(math.ceil(turns(sc["slow"])), dims - 1)
        for i in range(dims // 2):
            ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            freq[i] = (1.0 - ramp) * freq[i] + ramp * freq[i] / sc["factor"]
        amp = 1.0 + 0.1 * math.log(sc["factor"])
    ang = torch.arange(n, dtype=F64)[:, None] * torch.tensor(freq, dtype=F64)[None, :]
    return amp * torch.cos(ang), amp * torch.sin(ang)


def rotate_pairs(x, cos, sin):
    """x [n, ..., d]: neighbours (2i, 2i+1) of the first 2 * cos.shape[1] entries are turned by the position's angle; the rest passes."""
    out = x.clone()
    shape = (-1,) + (1,) * (x.dim() - 2)  # positions run along the first axis
    for i in range(cos.shape[1]):
        a, b, c, s = x[..., 2 * i], x[..., 2 * i + 1], cos[:, i].reshape(shape), sin[:, i].reshape(shape)
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


# ---------------------------------------------------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------------------------------------------------
def latent_attention(h, m, w, eps):
    """Keys and values of every head are linear images of one small normed latent per position; a second, rotated key part is shared by the
    heads.  Softmax with one extra denominator term per head (the sink)."""
    n, H, D, R, Dv, K = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w["q"].T).reshape(n, H, D + R)
    down = h @ w["dkv"].T
    latent = unit_rms(down[:, :K], eps) * w["dkv.norm"]
    k_shared = down[:, K:]
    q_rot = q[:, :, D:]
    if m.get("rot"):
        cos, sin = rotary_table(m["rot"], n)
        q_rot, k_shared = rotate_pairs(q_rot, cos, sin), rotate_pairs(k_shared, cos, sin)
    k_head = (latent @ w["uk"].T).reshape(n, H, D)
    v_head = (latent @ w["uv"].T).reshape(n, H, Dv)
    out = torch.zeros(n, H, Dv, dtype=F64)
    for head in range(H):
        for i in range(n):
            s = (k_head[: i + 1, head] @ q[i, head, :D] + k_shared[: i + 1] @ q_rot[i, head]) * m["scale"]
            top = max(float(s.max()), float(w["sink"][head]))
            e = torch.exp(s - top)
            out[i, head] = (e[:, None] * v_head[: i + 1, head]).sum(0) / (e.sum() + math.exp(float(w["sink"][head]) - top))
    out = out.reshape(n, H * Dv) * torch.sigmoid(h @ w["g"].T)
    return out @ w["o"].T


def window_attention(h, m, w, eps):
    """Grouped heads whose values are the keys as projected; unit-RMS q / k with gains; a linear distance penalty per head; a sliding window
    that keeps the sequence's first positions; one sigmoid gate per head."""
    n, H, G, D = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w["q"].T + w["q.b"]).reshape(n, H, D)
    k_raw = (h @ w["k"].T + w["k.b"]).reshape(n, G, D)
    q = unit_rms(q, eps) * w["q.norm"]
    k = unit_rms(k_raw, eps) * w["k.norm"]
    mask = m.get("mask") or {}
    size, first = mask.get("size", 0), mask.get("keep_first", 0)
    gate = torch.sigmoid(h @ w["g"].T)
    out = torch.zeros(n, H, D, dtype=F64)
    for head in range(H):
        grp = head // (H // G)
        slope = 2.0 ** (-8.0 * (head + 1) / H)
        for i in range(n):
            seen = torch.tensor([j for j in range(i + 1) if not size or i - j < size or j < first])
            s = (k[seen, grp] @ q[i, head]) * m["scale"] - slope * (i - seen).to(F64)
            p = torch.softmax(s, 0)
            out[i, head] = gate[i, head] * (p[:, None] * k_raw[seen, grp]).sum(0)
    return out.reshape(n, H * D) @ w["o"].T


def gated_linear(h, m, w, eps, state=None):
    """One [dim, vdim] matrix per head, decayed per key channel, written with k v^T, read with q."""
    n, H, D, Dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(n, H, D) / math.sqrt(D)
    k = (h @ w["k"].T).reshape(n, H, D)
    v = (h @ w["v"].T).reshape(n, H, Dv)
    decay = torch.sigmoid((h @ w["a1"].T) @ w["a2"].T + w["a2.b"]).pow(1.0 / m["tau"]).reshape(n, H, D)
    S = torch.zeros(H, D, Dv, dtype=F64) if state is None else state
    out = torch.zeros(n, H, Dv, dtype=F64)
    for t in range(n):
        S = decay[t, :, :, None] * S + k[t, :, :, None] * v[t, :, None, :]
        out[t] = (S * q[t, :, :, None]).sum(1)
    out = unit_rms(out, eps) * w["norm"]
    return (out.reshape(n, H * Dv) * silu(h @ w["g"].T)) @ w["o"].T


def feed_forward(h, w):
    return (silu(h @ w["gate"].T + w["gate.b"]) * (h @ w["up"].T + w["up.b"])) @ w["down"].T + w["down.b"]


MIXERS = {"latent_attention": latent_attention, "attention": window_attention, "gla": gated_linear}


# ---------------------------------------------------------------------------------------------------------------------------------
# the stack: a sublayer reads the stream; its output is normed (gains are offsets from one), scaled per channel and added
# ---------------------------------------------------------------------------------------------------------------------------------
def forward(cfg, weights, tokens, taps=None):
    """Logits [n, vocab] (float64) of a whole sequence.  taps: a list that receives the stream after every layer."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    for i, ly in enumerate(cfg["layers"]):
        p = f"l{i}."
        sub = lambda kind: {k[len(p) + len(kind) + 1:]: v for k, v in w.items() if k.startswith(p + kind + ".")}
        y = MIXERS[ly["type"]](x, ly["mixer"], sub("mix"), eps)
        x = x + unit_rms(y, eps) * (1.0 + w[p + "norm1"]) * w[p + "ls1"]
        if ly.get("mlp"):
            y = feed_forward(x, sub("mlp"))
            x = x + unit_rms(y, eps) * (1.0 + w[p + "norm2"]) * w[p + "ls2"]
        if taps is not None:
            taps.append(x.clone())
    return (unit_rms(x, eps) * (1.0 + w["final.norm"])) @ w["head"].T


def greedy(cfg, weights, prompt, n_new):
    """n_new tokens by argmax, re-running the whole sequence every time."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(cfg, weights, toks)[-1])))
    return toks[len(prompt):]
