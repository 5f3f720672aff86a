"""Plain float64 restatement of the Nusuvik design, one function per mechanism, for the tests.  It shares no code with qserve_b200: it
reads the config dict and a name -> tensor map directly and recomputes a whole sequence from scratch (no cache, no batching), with keys and
values of every head written out (the engine never forms them).

    x_t = E[tok_t] + B[(tok_{t-1} a + tok_t b) mod n]              (row n of B for t = 0);   x0 = x
    layer:   h = LN(x);   x <- x + mix(h) + ff(h)                  (one norm, both branches read it; ff may be absent)
    loop:    layers [start, stop) run `times` times; every pass begins with x <- W_in [x ; x0]
    logits = cap * tanh(W_head LN_final(x) / cap)
"""
import math

import torch

F64 = torch.float64


def layer_norm(x, gain, bias, eps):
    mu = x.mean(-1, keepdim=True)
    var = (x - mu).pow(2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * gain + bias


def unit_rms(x, gain, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def rotate_half(v, pos, dims, base):
    """v [T, ..., n]: entry i < dims/2 and entry i + dims/2 turn by pos * base^(-2i/dims); entries from `dims` on stay."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = pos.to(F64)[:, None] * freq[None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    while c.dim() < v.dim():
        c, s = c.unsqueeze(1), s.unsqueeze(1)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], -1)


def embed(cfg, w, tokens):
    x = w["embed"].to(F64)[tokens]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        rows = [bg["buckets"]] + [(tokens[i - 1] * bg["mul_prev"] + tokens[i] * bg["mul_cur"]) % bg["buckets"] for i in range(1, len(tokens))]
        x = x + w["bigram"].to(F64)[rows]
    return x


def latent_attention(m, w, p, h, eps, scores_out=None):
    """m: the mixer's config dict, p: tensor name prefix ('l<i>.mix.'), h [T, W]."""
    g = lambda n: w[p + n].to(F64)
    T = h.shape[0]
    H, D, R, Dv, K = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    rot = m.get("rot")
    turn = (lambda v: rotate_half(v, pos, rot["dims"], rot["base"])) if rot else (lambda v: v)
    q = (unit_rms(h @ g("dq").T, g("dq.norm"), eps) @ g("uq").T).view(T, H, D + R)
    down = h @ g("dkv").T
    c = unit_rms(down[:, :K], g("dkv.norm"), eps)
    k_shared = turn(down[:, K:])
    keys = (c @ g("uk").T).view(T, H, D)
    values = (c @ g("uv").T).view(T, H, Dv)
    s = torch.einsum("thd,uhd->htu", q[..., :D], keys) + torch.einsum("thr,ur->htu", turn(q[..., D:]), k_shared)
    s = s * m["scale"]
    s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), -math.inf)
    if scores_out is not None:
        scores_out.append(s)
    o = torch.einsum("htu,uhv->thv", torch.softmax(s, -1), values)
    o = o * torch.sigmoid(h @ g("g").T)[:, :, None]
    return o.reshape(T, H * Dv) @ g("o").T


def dense_ff(w, p, h):
    g = lambda n: w[p + n].to(F64)
    return gelu_tanh(h @ g("up").T + g("up.b")) @ g("down").T + g("down.b")


def route(spec, w, p, h):
    """Chosen experts [T, top] and their weights [T, top]."""
    r = spec["router"]
    E, top = r["experts"], r["top"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    G, keep = grp["count"], grp["keep"]
    score = torch.sigmoid(h @ w[p + "router"].to(F64).T)
    choice = score + w[p + "correction"].to(F64)
    per = E // G
    grouped = choice.view(-1, G, per)
    group_score = grouped.topk(min(2, per), -1).values.sum(-1)
    kept = torch.zeros_like(group_score, dtype=torch.bool).scatter(1, group_score.topk(keep, -1).indices, True)
    choice = grouped.masked_fill(~kept[:, :, None], -math.inf).reshape(-1, E)
    idx = choice.topk(top, -1).indices
    wt = score.gather(1, idx)
    return idx, wt / (wt.sum(-1, keepdim=True) + 1e-20)


def expert(w, p, h):
    g = lambda n: w[p + n].to(F64)
    a = h @ g("gate").T
    return (a * torch.sigmoid(a) * (h @ g("up").T)) @ g("down").T


def expert_mixture(spec, w, p, h):
    idx, wt = route(spec, w, p, h)
    out = torch.zeros_like(h)
    for e in range(spec["router"]["experts"]):
        use = (idx == e)
        rows = use.any(-1).nonzero().flatten()
        if rows.numel():
            out[rows] += (wt * use)[rows].sum(-1, keepdim=True) * expert(w, f"{p}e{e}.", h[rows])
    return out


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x = embed(cfg, w, tokens)
    x0 = x.clone()
    seen = []

    def layer(i, x):
        ly, p = cfg["layers"][i], f"l{i}."
        h = layer_norm(x, w[p + "norm1"].to(F64), w[p + "norm1.b"].to(F64), eps)
        y = latent_attention(ly["mixer"], w, p + "mix.", h, eps)
        if ly.get("mlp"):
            y = y + (dense_ff(w, p + "mlp.", h) if ly["mlp"]["kind"] == "dense" else expert_mixture(ly["mlp"], w, p + "mlp.", h))
        x = x + y
        seen.append(x.clone())
        return x

    n, lp = len(cfg["layers"]), cfg.get("loop")
    if lp:
        for i in range(lp["start"]):
            x = layer(i, x)
        for _ in range(lp["times"]):
            x = torch.cat([x, x0], -1) @ w["loop.in"].to(F64).T
            for i in range(lp["start"], lp["stop"]):
                x = layer(i, x)
        for i in range(lp["stop"], n):
            x = layer(i, x)
    else:
        for i in range(n):
            x = layer(i, x)
    logits = layer_norm(x, w["final.norm"].to(F64), w["final.norm.b"].to(F64), eps) @ w["head"].to(F64).T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, seen) if return_layers else logits


def greedy(cfg, w, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
