"""Architecture table of the benchmark models (pure Python: importing it does NOT load libqserve_b200.so, so the CPU
baseline arm of bench.py can use it without touching the product library).  Dimensions: SURVEY.md section 8."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ModelConfig:
    name: str
    hidden: int
    intermediate: int
    heads: int
    kv_heads: int
    layers: int
    vocab: int
    rope_theta: float
    eps: float = 1e-5
    head_dim: int = 128
    max_pos: int = 8192


MODELS = {
    "llama-3-8b": ModelConfig("Llama-3-8B", 4096, 14336, 32, 8, 32, 128256, 500000.0),
    "mistral-7b": ModelConfig("Mistral-7B", 4096, 14336, 32, 8, 32, 32000, 10000.0, max_pos=32768),
    "llama-2-7b": ModelConfig("Llama-2-7B", 4096, 11008, 32, 32, 32, 32000, 10000.0, max_pos=4096),
    "qwen1.5-72b": ModelConfig("Qwen1.5-72B", 8192, 24576, 64, 64, 80, 152064, 1000000.0, eps=1e-6, max_pos=32768),
    "tiny": ModelConfig("tiny-test", 512, 1024, 4, 2, 2, 1024, 10000.0),
}

PRECISIONS = ("w4a8kv4", "w4a8kv4-g128", "w8a8kv8", "w4a8kv8", "w8a8kv4")


# ------------------------------------------------------------------------------------------------------------------------
# Hybrid decoders described by a config.json: a list of layers, each with a sequence mixer (softmax attention over a paged cache or a
# recurrent layer with a per-sequence state) and an optional feed-forward.  Pure Python; the engine lives in qserve_b200.hybrid.
# ------------------------------------------------------------------------------------------------------------------------
import json
import math
import os
from typing import Callable, Dict, Optional, Tuple


@dataclass(frozen=True)
class RotaryConfig:
    """Rotary embedding on the first `dims` entries of a head; optional YaRN blend of the frequencies.  layout "interleaved" pairs entries
    (2i, 2i+1), "half" pairs entry i with entry i + dims/2."""
    dims: int
    base: float
    factor: Optional[float] = None   # None: no scaling
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0
    layout: str = "interleaved"

    def inv_freq(self):
        """Per-pair angular frequency (float64 list).  With scaling, pair i is blended between f_i and f_i / factor by a linear ramp whose
        ends are the pair indices that make `fast` and `slow` turns over the original context length."""
        half = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        if self.factor is None:
            return f
        turn = lambda t: self.dims * math.log(self.original / (2.0 * math.pi * t)) / (2.0 * math.log(self.base))
        lo = max(math.floor(turn(self.fast)), 0)
        hi = min(math.ceil(turn(self.slow)), self.dims - 1)
        out = []
        for i in range(half):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f[i] / self.factor * ramp + f[i] * (1.0 - ramp))
        return out

    def amplitude(self) -> float:
        return 1.0 if self.factor is None else 0.1 * math.log(self.factor) + 1.0


@dataclass(frozen=True)
class AttentionMixerConfig:
    """Causal softmax attention with `maps` score maps per head over shared values (2 = differential attention)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    rot: Optional[RotaryConfig]  # None: positions do not enter the scores
    scale: float
    maps: int = 1
    diff: float = 0.0        # differential attention: offset of lambda, and (1 - diff) scales the normalised head output
    head_norm: bool = False  # unit-RMS per head after the maps are combined
    # one map per head only:
    bias: bool = False       # q / k / v projections have biases (tensors q.b, k.b, v.b)
    qk_norm: bool = False    # q and k are brought to unit RMS per head before the scores
    head_temp: bool = False  # scores of head h are multiplied by the learned number temp[h]
    sink: bool = False       # the softmax denominator has one more term exp(sink[h]) without a value
    chunk: int = 0           # > 0: a query sees only keys of its own chunk of this many positions (counted from position 0)
    window: int = 0          # > 0: a query sees at most this many latest positions, its own included
    keep_first: int = 0      # with a window: the first keep_first positions of the sequence stay visible to every later query
    qk_gain: bool = False    # unit-RMS q / k are multiplied by learned gains of `dim` numbers shared by the heads (tensors q.norm, k.norm)
    tied_values: bool = False  # no value projection: a position's value is the key projection's output (bias included), taken ahead of the unit-RMS step
    distance_slope: float = 0.0  # > 0: slope_h (i - j) is taken off the score of query i and key j, slope_h = 2^(-distance_slope (h + 1) / heads)
    head_gate: bool = False  # head h's output is multiplied by sigmoid((W_g x)_h) (tensor g [heads, width])

    def slopes(self):
        """Per-head slope of the distance bias (float64 list), or None."""
        if self.distance_slope <= 0.0:
            return None
        return [2.0 ** (-self.distance_slope * (h + 1) / self.heads) for h in range(self.heads)]


@dataclass(frozen=True)
class GateRecurrenceMixerConfig:
    """HGRN2: per head a [dim, vdim] fp32 state, S <- diag(f) S + (1 - f) v^T with a forget gate f per row that never falls below a learned
    floor, read out with q = silu(.), unit RMS per head with a gain."""
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class RetentionMixerConfig:
    """Retention: per head a [dim, vdim] fp32 state, S <- decay_h S + k v^T, o = S^T q; rotary q / k, k scaled by dim^-1/2; unit-RMS heads
    times silu of an output gate."""
    heads: int
    dim: int
    vdim: int
    rot: Optional[RotaryConfig]
    decay: Tuple[float, ...]
    gated: bool = True


@dataclass(frozen=True)
class GatedLinearMixerConfig:
    """Gated linear attention: per head a [dim, vdim] fp32 state, S <- diag(a) S + k v^T with a decay per key channel
    a = sigmoid(z)^(1/tau), z a low-rank projection (rank `decay_rank`) of the mixer's input plus a bias; o = S^T q with q times dim^-1/2;
    unit-RMS heads with a gain shared by the heads, times silu of an output gate."""
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int


@dataclass(frozen=True)
class ParallelMixerConfig:
    """Two mixers side by side on the same input (tensors under left.* / right.*); each output is RMS-normed over the width with its own gain
    (left.out / right.out), the result is `scale` times their sum."""
    left: object
    right: object
    scale: float = 0.5


@dataclass(frozen=True)
class DeltaMixerConfig:
    """Gated delta rule: per head a [dim, vdim] fp32 state; short causal convolution of `conv` taps on q, k, v."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    unit_eps: float = 1e-6


@dataclass(frozen=True)
class LatentAttentionMixerConfig:
    """Causal softmax attention whose keys and values are linear images of a small latent row per position: only that row (`kv_rank` numbers,
    unit RMS times a gain) and one rotated key part of `rot_dim` numbers shared by all heads are cached.  Queries pass a latent of `q_rank`
    numbers (unit RMS times a gain; q_rank 0: queries are projected from the mixer's input directly, tensor q); a head's query has `dim`
    unrotated and `rot_dim` rotated numbers, its value `vdim`.  `gate`: the heads' outputs are multiplied by the sigmoid of a projection of
    the mixer's input, one number per head, or (`gate_wide`) one per output number.  `sink`: one more term exp(sink[h]) in head h's softmax
    denominator."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    rot: Optional[RotaryConfig]
    scale: float
    gate: bool = True
    chunk: int = 0
    window: int = 0
    gate_wide: bool = False
    sink: bool = False


@dataclass(frozen=True)
class MlpConfig:
    """Dense feed-forward.  gated: W_down(act(W_gate h) * W_up h); not gated: W_down act(W_up h).  bias: every projection has one.
    act: "gelu_tanh" or "silu"."""
    kind: str
    ff: int
    gated: bool = True
    bias: bool = False
    act: str = "gelu_tanh"


@dataclass(frozen=True)
class MoeConfig:
    """Mixture of experts: the `top` best of `experts` run per token; experts compute W_down(g sigmoid(alpha g) (u + up_shift)) with
    g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit) (limit = inf, alpha = 1, up_shift = 0: silu(W_gate h) * W_up h); optionally a
    shared expert for every token with its own size and limit.
    router "softmax": scores softmax over all experts, the winners weighted by their scores as they are.
    router "sigmoid": scores sigmoid(logit); the choice is made on score + a learned correction per expert (tensor `correction`), restricted
    to the `keep` best of `groups` equal groups of neighbouring experts (a group's score: the sum of its two largest choice scores); the
    winners are weighted by their scores divided by the winners' sum."""
    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: int = 0
    shared_limit: float = 0.0
    alpha: float = 1.702
    kind: str = "moe"
    up_shift: float = 1.0
    router: str = "softmax"
    correction: bool = False
    groups: int = 1
    keep: int = 1


@dataclass(frozen=True)
class HybridLayerConfig:
    type: str
    mixer: object
    mlp: Optional[MlpConfig]


@dataclass(frozen=True)
class HybridConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: Tuple[HybridLayerConfig, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    pair_buckets: int = 0    # 0: no (previous, current) pair embedding
    pair_mul_prev: int = 0
    pair_mul_cur: int = 0
    norm_offset: float = 1.0  # gains are stored as offsets from this value
    block: str = "parallel"   # "parallel": x += mixer(norm1 x) + ff(norm2 x);  "sequential": x += mixer(norm1 x), then x += ff(norm2 x);
                              # "post": x += ls1 norm1(mixer(x)), then x += ls2 norm2(ff(x)): the un-normed stream goes into a sublayer, what comes out is normed
    streams: int = 0          # sequential blocks: > 0 = that many residual streams with hyper-connection coefficients (tensors hc1.*, hc2.*)
    norm_groups: int = 1      # RMS norms work on this many equal consecutive parts of the width, each with its own statistic
    embed_scale: float = 1.0
    norm_kind: str = "rms"    # "layer": (x - mean) / sqrt(var + eps) * w + b with plain gains (tensor <norm>) and biases (tensor <norm>.b)
    shared_norm: bool = False  # parallel blocks: the mixer and the feed-forward read ONE normed row (norm1; there is no norm2)
    loop_in: bool = False     # before the first layer of every pass of the loop: x <- W [x; x0] (tensor loop.in [W, 2 W], x0 the embedding output)
    logit_softcap: float = 0.0  # > 0: logits <- cap * tanh(logits / cap)
    layer_scale: bool = False   # "post" blocks: a normed sublayer output is multiplied per channel by a learned row (tensors ls1, ls2)

    def schedule(self):
        """Layer index of every layer RUN: layers loop_start .. loop_stop-1 run loop_times times in a row (same weights, own cache / state)."""
        n = len(self.layers)
        return list(range(self.loop_start)) + list(range(self.loop_start, self.loop_stop)) * self.loop_times + list(range(self.loop_stop, n))

    def pass_starts(self):
        """Indices into schedule() of the runs that begin a pass of the loop."""
        span = self.loop_stop - self.loop_start
        return [self.loop_start + k * span for k in range(self.loop_times)] if span > 0 else []


def _parse_rot(r: dict) -> RotaryConfig:
    sc = r.get("scaling")
    if sc:
        return RotaryConfig(int(r["dims"]), float(r["base"]), float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
    return RotaryConfig(int(r["dims"]), float(r["base"]))


def parse_rizurax(c: dict) -> HybridConfig:
    """Rizurax: parallel layers (mixer and feed-forward read the same stream), mixers `attention` (differential, two maps per head, unit-RMS
    heads) and `delta` (gated delta rule), hashed pair embedding, a looped span of layers."""
    layers = []
    for ly in c["layers"]:
        m = ly["mixer"]
        if ly["type"] == "attention":
            mixer = AttentionMixerConfig(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), _parse_rot(m["rot"]), float(m["scale"]),
                                         maps=2, diff=float(m["diff"]), head_norm=True)
        elif ly["type"] == "delta":
            mixer = DeltaMixerConfig(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m["conv"]))
        else:
            raise ValueError(f"unknown mixer type {ly['type']!r}")
        mlp = ly.get("mlp")
        if mlp is not None and mlp.get("kind") != "dense":
            raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(HybridLayerConfig(ly["type"], mixer, MlpConfig("dense", int(mlp["ff"])) if mlp is not None else None))
    lp = c.get("loop") or {}
    bg = (c.get("embedding") or {}).get("bigram") or {}
    return HybridConfig("Rizurax", int(c["vocab"]), int(c["width"]), float(c["norm"]["eps"]), tuple(layers),
                        int(lp.get("start", 0)), int(lp.get("stop", 0)), int(lp.get("times", 1)),
                        int(bg.get("buckets", 0)), int(bg.get("mul_prev", 0)), int(bg.get("mul_cur", 0)))


def parse_toderax(c: dict) -> HybridConfig:
    """Toderax: sequential blocks on `streams` residual streams (hyper-connections), group-wise RMS norms with plain gains, a scaled
    embedding; mixers `hgrn2` (gate recurrence) and `parallel` (chunked softmax attention with a sink beside retention); mixture-of-experts
    feed-forward with a shared expert."""
    layers = []
    for ly in c["layers"]:
        m = ly["mixer"]
        if ly["type"] == "hgrn2":
            mixer = GateRecurrenceMixerConfig(int(m["heads"]), int(m["dim"]), int(m["vdim"]))
        elif ly["type"] == "parallel":
            a, r = m["left"], m["right"]
            left = AttentionMixerConfig(int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"]), None, float(a["scale"]), bias=True,
                                        qk_norm=True, head_temp=True, sink=True, chunk=int((a.get("mask") or {}).get("size", 0)))
            rot = r.get("rot")
            right = RetentionMixerConfig(int(r["heads"]), int(r["dim"]), int(r["vdim"]),
                                         RotaryConfig(int(rot["dims"]), float(rot["base"]), layout="half") if rot else None,
                                         tuple(float(d) for d in r["decay"]))
            if len(right.decay) != right.heads:
                raise ValueError("retention needs one decay per head")
            mixer = ParallelMixerConfig(left, right)
        else:
            raise ValueError(f"unknown mixer type {ly['type']!r}")
        mlp = ly.get("mlp")
        ff = None
        if mlp is not None:
            if mlp.get("kind") != "moe":
                raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
            sh = mlp.get("shared") or {}
            ff = MoeConfig(int(mlp["router"]["experts"]), int(mlp["router"]["top"]), int(mlp["expert"]["ff"]), float(mlp["expert"]["limit"]),
                           int(sh.get("ff", 0)), float(sh.get("limit", 0.0)))
        layers.append(HybridLayerConfig(ly["type"], mixer, ff))
    norm = c["norm"]
    return HybridConfig("Toderax", int(c["vocab"]), int(c["width"]), float(norm["eps"]), tuple(layers), norm_offset=0.0, block="sequential",
                        streams=int(c.get("streams", 0)), norm_groups=int(norm.get("groups", 1)),
                        embed_scale=float((c.get("embedding") or {}).get("scale", 1.0)))


def parse_nusuvik(c: dict) -> HybridConfig:
    """Nusuvik: parallel layers with ONE layer norm (gain and bias) that both the mixer and the feed-forward read; mixer `latent_attention`
    (latent queries, a cached key/value latent with a shared rotated key part, a sigmoid gate per head); feed-forwards dense (gelu_tanh between
    two biased projections) or a mixture of experts (sigmoid scores, a correction for the choice, groups of experts, silu-gated experts);
    hashed pair embedding; a looped span of layers whose every pass starts with a projection of [stream; embedding output]; final layer norm
    and a tanh cap on the logits."""
    layers = []
    for ly in c["layers"]:
        m = ly["mixer"]
        if ly["type"] == "latent_attention":
            r = m.get("rot")
            rot = RotaryConfig(int(r["dims"]), float(r["base"]), layout="half") if r else None
            mixer = LatentAttentionMixerConfig(int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]), int(m["q_rank"]),
                                               rot, float(m["scale"]))
            if rot is not None and (rot.dims > mixer.rot_dim or rot.dims % 2):
                raise ValueError("latent attention rotates an even number of at most rot_dim entries")
        else:
            raise ValueError(f"unknown mixer type {ly['type']!r}")
        mlp = ly.get("mlp")
        if mlp is None:
            ff = None
        elif mlp.get("kind") == "dense":
            ff = MlpConfig("dense", int(mlp["ff"]), gated=False, bias=True)
        elif mlp.get("kind") == "moe":
            r = mlp["router"]
            g = r.get("groups") or {}
            ff = MoeConfig(int(r["experts"]), int(r["top"]), int(mlp["expert"]["ff"]), math.inf, alpha=1.0, up_shift=0.0, router="sigmoid",
                           correction=True, groups=int(g.get("count", 1)), keep=int(g.get("keep", g.get("count", 1))))
            if ff.experts % ff.groups or not 1 <= ff.keep <= ff.groups or not 1 <= ff.top <= ff.keep * (ff.experts // ff.groups):
                raise ValueError("router: groups must divide the experts, 1 <= keep <= groups, top <= experts of the kept groups")
        else:
            raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(HybridLayerConfig(ly["type"], mixer, ff))
    lp = c.get("loop") or {}
    bg = (c.get("embedding") or {}).get("bigram") or {}
    return HybridConfig("Nusuvik", int(c["vocab"]), int(c["width"]), float(c["norm"]["eps"]), tuple(layers),
                        int(lp.get("start", 0)), int(lp.get("stop", 0)), int(lp.get("times", 1)),
                        int(bg.get("buckets", 0)), int(bg.get("mul_prev", 0)), int(bg.get("mul_cur", 0)), norm_offset=0.0,
                        norm_kind="layer", shared_norm=True, loop_in=bool(lp), logit_softcap=float(c.get("logit_softcap") or 0.0))


def parse_zuzezen(c: dict) -> HybridConfig:
    """Zuzezen: post-norm blocks (a sublayer takes the un-normed stream; its output is RMS-normed with a gain kept as an offset from one, scaled per
    channel and added), a scaled embedding; mixers `latent_attention` (queries projected directly, interleaved rotary pairs with YaRN
    frequencies on the shared rotated part, a sink, a sigmoid gate per output number), `attention` (grouped heads without a value
    projection, biased q / k with unit RMS and gains, a linear distance bias, a sliding window that keeps the first positions, a sigmoid
    gate per head) and `gla` (gated linear attention); dense silu-gated feed-forwards with biases."""
    layers = []
    for ly in c["layers"]:
        m = ly["mixer"]
        if ly["type"] == "latent_attention":
            rot = _parse_rot(m["rot"]) if m.get("rot") else None
            mixer = LatentAttentionMixerConfig(int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]), 0, rot,
                                               float(m["scale"]), gate=True, gate_wide=True, sink=True)
            if rot is not None and (rot.dims > mixer.rot_dim or rot.dims % 2):
                raise ValueError("latent attention rotates an even number of at most rot_dim entries")
        elif ly["type"] == "attention":
            mk = m.get("mask") or {}
            window = int(mk.get("size", 0))
            keep = int(mk.get("keep_first", 0)) if window > 0 else 0   # without a window every earlier position is visible anyway
            mixer = AttentionMixerConfig(int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"])), None,
                                         float(m["scale"]), bias=True, qk_norm=True, window=window, keep_first=keep, qk_gain=True,
                                         tied_values=True, distance_slope=8.0, head_gate=True)
            if mixer.vdim != mixer.dim:
                raise ValueError("attention whose values are its keys needs vdim == dim")
        elif ly["type"] == "gla":
            mixer = GatedLinearMixerConfig(int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"]), int(m.get("decay_rank", 0)))
        else:
            raise ValueError(f"unknown mixer type {ly['type']!r}")
        mlp = ly.get("mlp")
        if mlp is not None and mlp.get("kind") != "dense":
            raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(HybridLayerConfig(ly["type"], mixer, MlpConfig("dense", int(mlp["ff"]), gated=True, bias=True, act="silu") if mlp is not None else None))
    return HybridConfig("Zuzezen", int(c["vocab"]), int(c["width"]), float(c["norm"]["eps"]), tuple(layers), norm_offset=1.0, block="post",
                        embed_scale=float((c.get("embedding") or {}).get("scale", 1.0)), layer_scale=True)


# config.json "architecture" -> parser.  The quantised Llama-family models of MODELS are built by qserve_b200.decode.DecodeRunner.
ARCHITECTURES: Dict[str, Callable[[dict], HybridConfig]] = {"Rizurax": parse_rizurax, "Toderax": parse_toderax, "Nusuvik": parse_nusuvik,
                                                                 "Zuzezen": parse_zuzezen}


def read_model_config(model_dir: str) -> HybridConfig:
    """Parse `<model_dir>/config.json` with the parser its "architecture" names."""
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    arch = c.get("architecture")
    if arch not in ARCHITECTURES:
        raise ValueError(f"unknown architecture {arch!r}; known: {sorted(ARCHITECTURES)}")
    return ARCHITECTURES[arch](c)
