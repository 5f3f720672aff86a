"""Unquantised hybrid decoders over the library's kernels (csrc/hybrid.cu): a stack of layers, each a sequence mixer (attention over the
paged cache, or a recurrent layer over a state slot) beside an optional feed-forward, on an fp32 residual stream.

The model is assembled from a `HybridConfig` (qserve_b200.modelcfg): mixers are looked up in `MIXERS` and feed-forwards in `FEED_FORWARDS`
by config type, so another design reuses them with other constants.  Layers are "parallel" blocks (mixer and feed-forward read the same
stream and their output projections are one product), "sequential" blocks (mixer, then feed-forward) on one or several residual streams
with learned read / write / mixing coefficients, or "post" blocks (mixer, then feed-forward, each taking the un-normed stream and normed on the
way back, with a learned scale per channel).  A forward pass takes a `StepBatch` -- the flat batch a scheduler step has put together (portions of
prompts beside single decoded tokens) -- and the `HybridCache`; there is no other forward path: whole prompts, portions and decoding
all go through `HybridDecoder.forward`.

Matrix products are cuBLAS through torch (as the quantised models' lm_head is); everything else is this library's kernels.  With
`dtype=torch.float32` every product runs in true fp32 (TF32 off).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

import ctypes

from ._lib import AttnExtra, check, lib
from .cache import HybridCache
from .modelcfg import (AttentionMixerConfig, DeltaMixerConfig, GatedLinearMixerConfig, GateRecurrenceMixerConfig, HybridConfig,
                       LatentAttentionMixerConfig, MlpConfig, MoeConfig, ParallelMixerConfig, RetentionMixerConfig)

_DT = {torch.bfloat16: 0, torch.float32: 1}
_NORM_KIND = {"rms": 1, "layer": 2}      # QS_NORM_RMS, QS_NORM_LAYER
_ROUTER_MODE = {"softmax": 0, "sigmoid": 1}  # QS_ROUTER_SOFTMAX, QS_ROUTER_SIGMOID_GROUPS
_ACT = {"gelu_tanh": 0, "silu": 1}           # QS_ACT_GELU_TANH, QS_ACT_SILU
_ROT_LAYOUT = {"interleaved": 0, "half": 1}
_F32_OUT = [None]  # whether torch.mm takes out_dtype on this build (found at first use)


def _mm_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a @ b with an fp32 result (the accumulator as it is, where the library offers it; else the storage type's rounding widened)."""
    if a.dtype == torch.float32:
        return torch.mm(a, b)
    if _F32_OUT[0] is None:
        try:
            torch.mm(a[:1], b, out_dtype=torch.float32)
            _F32_OUT[0] = True
        except (TypeError, RuntimeError):
            _F32_OUT[0] = False
    if _F32_OUT[0]:
        try:
            return torch.mm(a, b, out_dtype=torch.float32)
        except RuntimeError:  # a shape or stride this form of the product does not take
            pass
    return torch.mm(a, b).float()


def _pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """`w` with zero rows added up to a multiple: projection rows whose stride keeps 16-byte alignment in bfloat16 (the tensor-core attention
    kernels load queries 16 bytes at a time straight from the rows of the mixer's one input product)."""
    pad = (-w.shape[0]) % multiple
    return w if pad == 0 else torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], 0)


def _stream(dev: torch.device):
    return torch._C._cuda_getCurrentRawStream(dev.index if dev.index is not None else torch.cuda.current_device())


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


@dataclass
class StepBatch:
    """Device-side description of one step's flat token batch.  Row t of every activation belongs to token t."""
    n_tokens: int
    n_entries: int
    tokens: torch.Tensor       # int32 [T]
    prev: torch.Tensor         # int32 [T] previous token of the same sequence, -1 for a sequence's first token
    tok_slot: torch.Tensor     # int32 [T] slot (= block-table row) of the token's sequence
    tok_pos: torch.Tensor      # int32 [T] position in its sequence
    tok_entry: torch.Tensor    # int32 [T] index of its entry
    entry_start: torch.Tensor  # int32 [E] first row of the entry
    entry_len: torch.Tensor    # int32 [E]
    entry_slot: torch.Tensor   # int32 [E]
    entry_pos0: torch.Tensor   # int32 [E] position of the entry's first token
    block_table: torch.Tensor  # int32 [slots, max_blocks]
    # attention work lists: entries of at least TILE_MIN tokens are cut into tiles of TILE_ROWS query rows, the other tokens run one by one
    n_tiles: int = 0
    n_long: int = 0
    n_short: int = 0
    tile_entry: Optional[torch.Tensor] = None    # int32 [n_tiles] entry of the tile
    tile_row0: Optional[torch.Tensor] = None     # int32 [n_tiles] first row of the tile within its entry
    long_tokens: Optional[torch.Tensor] = None   # int32 [n_long] rows covered by tiles
    short_tokens: Optional[torch.Tensor] = None  # int32 [n_short] all other rows

    # entries of at least TILE_MIN tokens, when `build` is told the page size: their sequences' pages so far, numbered in one run, so that a
    # mixer can lay out per-step copies of what those pages hold (page i of the run is the sequence's page ctx_src[i]; ctx_table is a block
    # table into the run)
    n_ctx_pages: int = 0
    ctx_src: Optional[torch.Tensor] = None     # int64 [n_ctx_pages] page of the pool
    ctx_table: Optional[torch.Tensor] = None   # int32 [slots, max_blocks]

    TILE_MIN = 16
    TILE_ROWS = 64

    @staticmethod
    def pack(entries: Sequence[tuple]):
        """Host side of a batch: one int32 tensor holding every table, and the sizes (T, E, tiles, long rows, short rows) that say where.
        entries: (slot, first position, previous token or -1, token list) per sequence, in batch order."""
        T = sum(len(e[3]) for e in entries)
        E = len(entries)
        tiles = [(i, r0) for i, e in enumerate(entries) if len(e[3]) >= StepBatch.TILE_MIN for r0 in range(0, len(e[3]), StepBatch.TILE_ROWS)]
        nt = len(tiles)
        host = torch.empty(6 * T + 4 * E + 2 * nt, dtype=torch.int32)
        tok, prev, slot, pos, ent, lists = (host[i * T:(i + 1) * T] for i in range(6))
        es, el, eslot, ep0 = (host[6 * T + i * E: 6 * T + (i + 1) * E] for i in range(4))
        r, longs, shorts = 0, [], []
        for i, (s, p0, last, toks) in enumerate(entries):
            n = len(toks)
            if n == 0:
                raise ValueError("an entry of a step must bring at least one token")
            tt = torch.as_tensor(toks, dtype=torch.int32)
            tok[r:r + n] = tt
            prev[r] = last
            prev[r + 1:r + n] = tt[:-1]
            slot[r:r + n] = s
            pos[r:r + n] = torch.arange(p0, p0 + n, dtype=torch.int32)
            ent[r:r + n] = i
            es[i], el[i], eslot[i], ep0[i] = r, n, s, p0
            (longs if n >= StepBatch.TILE_MIN else shorts).extend(range(r, r + n))
            r += n
        lists[:] = torch.tensor(longs + shorts, dtype=torch.int32)
        if nt:
            host[6 * T + 4 * E:] = torch.tensor([t[0] for t in tiles] + [t[1] for t in tiles], dtype=torch.int32)
        return host, (T, E, nt, len(longs), len(shorts))

    @staticmethod
    def view(d: torch.Tensor, sizes: tuple, block_table: torch.Tensor) -> "StepBatch":
        """The batch over a device copy `d` of a packed host tensor."""
        T, E, nt, n_long, n_short = sizes
        v = [d[i * T:(i + 1) * T] for i in range(5)] + [d[6 * T + i * E: 6 * T + (i + 1) * E] for i in range(4)]
        o = 6 * T + 4 * E
        return StepBatch(T, E, *v, block_table, nt, n_long, n_short, d[o:o + nt], d[o + nt:o + 2 * nt], d[5 * T:5 * T + n_long], d[5 * T + n_long:6 * T])

    @staticmethod
    def build(entries: Sequence[tuple], block_table: torch.Tensor, device: torch.device, page_size: int = 0) -> "StepBatch":
        host, sizes = StepBatch.pack(entries)
        if device.type == "cuda":
            host = host.pin_memory()
        b = StepBatch.view(host.to(device, non_blocking=True), sizes, block_table)
        if page_size > 0:
            slots, idx = [], []
            for s, p0, _, toks in entries:
                if len(toks) >= StepBatch.TILE_MIN:
                    n = -(-(p0 + len(toks)) // page_size)
                    slots += [s] * n
                    idx += range(n)
            if slots:
                cs, ci = torch.tensor(slots, dtype=torch.int64).to(device), torch.tensor(idx, dtype=torch.int64).to(device)
                b.n_ctx_pages = len(slots)
                b.ctx_src = block_table[cs, ci].to(torch.int64)
                b.ctx_table = torch.zeros_like(block_table)
                b.ctx_table[cs, ci] = torch.arange(len(slots), dtype=block_table.dtype, device=device)
        return b


# ------------------------------------------------------------------------------------------------------------------------
# mixers
# ------------------------------------------------------------------------------------------------------------------------
class _Mixer:
    """What the decoder needs of a sequence mixer: `w_in` [in_features, W] (one product makes the mixer's projection rows), `run` (projection
    rows -> head outputs [T, out_features], through the mixer's cache or state), `w_out` [W, out_features]."""

    def place_out(self, st) -> None:
        """Keep the output projection on the device (blocks that do not fold it into a product of their own)."""
        self.w_out = st(self.w_out)

    def project(self, cat: torch.Tensor, dt: int, stream):
        """Head outputs -> the mixer's output rows [T, W]; returns (rows, rows are fp32)."""
        return torch.mm(cat, self.w_out.t()), False


class MultiMapAttentionMixer(_Mixer):
    """Causal softmax attention over the paged cache with `maps` score maps per head sharing the values; maps = 2 is differential attention:
    o = a1 - lambda a2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, then unit RMS per head and a factor (1 - diff).
    With one map: optional projection biases, unit-RMS q / k (with gains shared by the heads), a learned temperature per head (folded into the
    prepared query), a sink term in the denominator, a mask by chunks of positions and / or a window that may keep the sequence's first
    positions visible, a linear distance bias per head, values tied to the key projection's raw output (no value projection), and a sigmoid gate per head
    (its logits are the last `heads` columns of the mixer's projection rows)."""

    def __init__(self, m: AttentionMixerConfig, w: Dict[str, torch.Tensor], eps: float, dtype, device):
        self.m, self.eps = m, eps
        assert m.heads % m.kv_heads == 0
        f32 = lambda t: t.to(torch.float32).to(device).contiguous()
        self.general = m.rot is None or m.rot.layout != "interleaved" or m.bias or m.qk_norm or m.head_temp or m.tied_values
        plus = m.sink or m.keep_first or m.distance_slope > 0.0 or m.head_gate or m.qk_gain
        if (self.general or plus) and m.maps != 1:
            raise ValueError("biases, unit-RMS q / k, head temperatures, sinks, kept first positions, distance biases, tied values, head gates and "
                             "non-interleaved rotations need one score map per head")
        if m.keep_first and (m.window <= 0 or m.chunk):
            raise ValueError("kept first positions go with a window and no chunks")
        if m.tied_values and m.vdim != m.dim:
            raise ValueError("values tied to the keys need vdim == dim")
        if m.qk_gain and not m.qk_norm:
            raise ValueError("q / k gains belong to the unit-RMS q / k")
        parts = ["q", "k"] + ([] if m.tied_values else ["v"])
        self.bias = f32(torch.cat([w[n + ".b"] for n in parts], 0)) if m.bias else None
        self.q_gain, self.k_gain = (f32(w["q.norm"]), f32(w["k.norm"])) if m.qk_gain else (None, None)
        if m.qk_gain and (self.q_gain.numel() != m.dim or self.k_gain.numel() != m.dim):
            raise ValueError("q / k gains have `dim` numbers")
        sl = m.slopes()
        self.slopes = torch.tensor(sl, dtype=torch.float64).to(torch.float32).to(device) if sl is not None else None
        self.temp = f32(w["temp"]) if m.head_temp else None
        self.sinks = f32(w["sink"]) if m.sink else None
        for t, n in ((self.temp, "temp"), (self.sinks, "sink")):
            if t is not None and t.numel() != m.heads:
                raise ValueError(f"attention weight {n} must have one number per head")
        self.col_g = (m.heads + m.kv_heads) * m.maps * m.dim + (0 if m.tied_values else m.kv_heads * m.vdim)
        self.in_features = self.col_g + (m.heads if m.head_gate else 0)
        self.out_features = m.heads * m.vdim
        rows_of = {"q": m.heads * m.maps * m.dim, "k": m.kv_heads * m.maps * m.dim, "v": m.kv_heads * m.vdim, "g": m.heads}
        parts += ["g"] if m.head_gate else []
        for name in parts:
            if w[name].shape[0] != rows_of[name]:
                raise ValueError(f"attention weight {name}: {tuple(w[name].shape)} does not have {rows_of[name]} rows")
        self.w_in = _pad_rows(torch.cat([w[n] for n in parts], 0)).to(device=device, dtype=dtype).contiguous()
        self.in_features = self.w_in.shape[0]
        self.w_out = w["o"]
        self.inv_freq = torch.tensor(m.rot.inv_freq(), dtype=torch.float64).to(torch.float32).to(device) if m.rot is not None else None
        self.amp = float(m.rot.amplitude()) if m.rot is not None else 1.0
        if self.general and self.amp != 1.0:
            raise ValueError("scaled rotary frequencies are only built for the interleaved layout")
        if self.bias is not None and self.bias.numel() != self.col_g:
            raise ValueError("attention biases do not match the projections")
        if m.maps == 2:
            d = lambda a, b: float((w[a].double() * w[b].double()).sum())
            self.lam = math.exp(d("lq1", "lk1")) - math.exp(d("lq2", "lk2")) + m.diff
            self.out_scale = 1.0 - m.diff
        else:
            self.lam, self.out_scale = 0.0, 1.0

    def scratch_floats(self, tokens: int) -> int:
        # per-map outputs of the tiled prompt kernel and the key shares of the single-token kernel
        return int(lib.qs_hyb_attention_scratch_floats(tokens, self.m.heads, self.m.kv_heads, self.m.maps, self.m.vdim))

    def run(self, proj: torch.Tensor, out: torch.Tensor, b: StepBatch, run_cache: dict, page_size: int, scratch, dt: int, stream) -> None:
        m = self.m
        fast = scratch is not None and ATTENTION_IMPL != "plain" and \
            lib.qs_hyb_attention_fast_supported(dt, m.heads, m.kv_heads, m.maps, m.dim, m.vdim, proj.stride(0)) == 1
        extra = None
        if m.keep_first or self.slopes is not None or m.head_gate:
            gate = proj.data_ptr() + self.col_g * proj.element_size() if m.head_gate else None
            extra = ctypes.byref(AttnExtra(m.keep_first, _p(self.slopes), gate, proj.stride(0)))
        if self.general:
            check(lib.qs_hyb_qk_prepare_append(proj.data_ptr(), proj.stride(0), _p(self.bias), _p(self.temp), _p(b.tok_slot), _p(b.tok_pos),
                                               _p(b.block_table), b.block_table.shape[1], run_cache["k"].data_ptr(), run_cache["v"].data_ptr(),
                                               _p(self.inv_freq), 1 if m.rot is not None and m.rot.layout == "half" else 0,
                                               m.rot.dims if m.rot is not None else 0, 1 if m.qk_norm else 0, self.eps, b.n_tokens, m.heads,
                                               m.kv_heads, m.dim, m.vdim, page_size, _p(self.q_gain), _p(self.k_gain), 1 if m.tied_values else 0,
                                               dt, stream))
        else:
            check(lib.qs_hyb_rope_append(proj.data_ptr(), proj.stride(0), _p(b.tok_slot), _p(b.tok_pos), _p(b.block_table), b.block_table.shape[1],
                                         run_cache["k"].data_ptr(), run_cache["v"].data_ptr(), self.inv_freq.data_ptr(), self.amp, b.n_tokens,
                                         m.heads, m.kv_heads, m.maps, m.dim, m.vdim, m.rot.dims, page_size, dt, stream))
        if fast:
            # prompt portions as 64-row tiles on the tensor cores, single tokens and short portions with a head group as the tile's rows
            check(lib.qs_hyb_attention_fast(out.data_ptr(), out.stride(0), proj.data_ptr(), proj.stride(0), run_cache["k"].data_ptr(),
                                            run_cache["v"].data_ptr(), _p(b.tok_slot), _p(b.tok_pos), _p(b.block_table), b.block_table.shape[1],
                                            _p(b.tile_entry), _p(b.tile_row0), b.n_tiles, _p(b.long_tokens), b.n_long, _p(b.short_tokens), b.n_short,
                                            _p(b.entry_start), _p(b.entry_len), _p(b.entry_slot), _p(b.entry_pos0), scratch.data_ptr(), m.heads,
                                            m.kv_heads, m.maps, m.dim, m.vdim, m.scale, self.lam, self.out_scale, self.eps,
                                            1 if m.head_norm else 0, page_size, m.chunk, m.window, _p(self.sinks), extra, dt, stream))
            return
        check(lib.qs_hyb_attention(out.data_ptr(), out.stride(0), proj.data_ptr(), proj.stride(0), run_cache["k"].data_ptr(),
                                   run_cache["v"].data_ptr(), _p(b.tok_slot), _p(b.tok_pos), _p(b.block_table), b.block_table.shape[1],
                                   b.n_tokens, m.heads, m.kv_heads, m.maps, m.dim, m.vdim, m.scale, self.lam, self.out_scale, self.eps,
                                   1 if m.head_norm else 0, page_size, m.chunk, m.window, _p(self.sinks), extra, dt, stream))


ATTENTION_IMPL = None  # tests: "plain" keeps the attention on the CUDA-core kernel


class GatedDeltaMixer(_Mixer):
    """Gated delta rule with short convolutions; the state and the convolution's last inputs live in the sequence's slot."""

    def __init__(self, m: DeltaMixerConfig, w: Dict[str, torch.Tensor], eps: float, dtype, device):
        self.m, self.eps = m, eps
        assert m.heads % m.kv_heads == 0
        qk, hv = m.kv_heads * m.dim, m.heads * m.vdim
        for name, rows in (("q", qk), ("k", qk), ("v", hv), ("g", hv), ("b", m.heads), ("a", m.heads)):
            if w[name].shape[0] != rows:
                raise ValueError(f"delta weight {name}: {tuple(w[name].shape)} does not have {rows} rows")
        self.in_features = 2 * qk + 2 * hv + 2 * m.heads
        self.out_features = hv
        self.w_in = torch.cat([w["q"], w["k"], w["v"], w["g"], w["b"], w["a"]], 0).to(device=device, dtype=dtype).contiguous()
        self.w_out = w["o"]
        f32 = lambda t: t.to(torch.float32).to(device).contiguous()
        self.conv_w = f32(torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]], 0))
        if self.conv_w.shape[1] != m.conv:
            raise ValueError("convolution weights do not have `conv` taps")
        self.a_log, self.dt_bias, self.norm_w = f32(w["A_log"]), f32(w["dt_bias"]), f32(w["norm"])
        self.prep_width = 2 * qk + hv + 2 * m.heads

    def scratch_floats(self, tokens: int) -> int:
        return tokens * (self.prep_width + self.out_features)

    def run(self, proj: torch.Tensor, out: torch.Tensor, b: StepBatch, run_cache: dict, page_size: int, scratch: torch.Tensor, dt: int, stream) -> None:
        m, T = self.m, b.n_tokens
        prep = scratch[: T * self.prep_width]
        o_raw = scratch[T * self.prep_width: T * (self.prep_width + self.out_features)]
        check(lib.qs_hyb_gated_delta(out.data_ptr(), out.stride(0), prep.data_ptr(), o_raw.data_ptr(), proj.data_ptr(), proj.stride(0),
                                     self.conv_w.data_ptr(), run_cache["conv"].data_ptr(), run_cache["state"].data_ptr(), self.a_log.data_ptr(),
                                     self.dt_bias.data_ptr(), self.norm_w.data_ptr(), _p(b.tok_entry), _p(b.tok_pos), _p(b.entry_start),
                                     _p(b.entry_len), _p(b.entry_slot), _p(b.entry_pos0), T, b.n_entries, m.heads, m.kv_heads, m.dim, m.vdim,
                                     m.conv, m.unit_eps, self.eps, dt, stream))


class GateRecurrenceMixer(_Mixer):
    """HGRN2: q = silu(W_q h), forget gate f = lower + (1 - lower) sigmoid(W_f h + b) per head and row, S <- diag(f) S + (1 - f) v^T, o = S^T q,
    unit RMS per head with a gain shared by the heads.  The fp32 state lives in the sequence's slot."""

    def __init__(self, m: GateRecurrenceMixerConfig, w: Dict[str, torch.Tensor], eps: float, dtype, device):
        self.m, self.eps = m, eps
        hd, hv = m.heads * m.dim, m.heads * m.vdim
        for name, rows in (("q", hd), ("f", hd), ("v", hv)):
            if w[name].shape[0] != rows:
                raise ValueError(f"gate recurrence weight {name}: {tuple(w[name].shape)} does not have {rows} rows")
        self.in_features, self.out_features = 2 * hd + hv, hv
        self.w_in = torch.cat([w["q"], w["f"], w["v"]], 0).to(device=device, dtype=dtype).contiguous()
        self.w_out = w["o"]
        f32 = lambda t: t.to(torch.float32).to(device).contiguous()
        self.f_bias, self.lower, self.norm_w = f32(w["f.b"]), f32(w["lower"]), f32(w["norm"])
        if self.f_bias.numel() != hd or self.lower.numel() != hd or self.norm_w.numel() != m.vdim:
            raise ValueError("gate recurrence: f.b and lower have heads * dim entries, norm has vdim")

    def scratch_floats(self, tokens: int) -> int:
        return tokens * (self.in_features + self.out_features)

    def run(self, proj, out, b: StepBatch, run_cache: dict, page_size: int, scratch: torch.Tensor, dt: int, stream) -> None:
        m, T = self.m, b.n_tokens
        prep = scratch[: T * self.in_features]
        o_raw = scratch[T * self.in_features: T * (self.in_features + self.out_features)]
        check(lib.qs_hyb_gate_recurrence(out.data_ptr(), out.stride(0), prep.data_ptr(), o_raw.data_ptr(), proj.data_ptr(), proj.stride(0),
                                         self.f_bias.data_ptr(), self.lower.data_ptr(), self.norm_w.data_ptr(), run_cache["state"].data_ptr(),
                                         _p(b.entry_start), _p(b.entry_len), _p(b.entry_slot), _p(b.entry_pos0), T, b.n_entries, m.heads, m.dim,
                                         m.vdim, self.eps, dt, stream))


class RetentionMixer(_Mixer):
    """Retention: S <- decay_h S + k v^T, o = S^T q with rotary q / k (k times dim^-1/2 after the rotation), unit-RMS heads times silu of an
    output gate.  The fp32 state lives in the sequence's slot."""

    def __init__(self, m: RetentionMixerConfig, w: Dict[str, torch.Tensor], eps: float, dtype, device):
        self.m, self.eps = m, eps
        hd, hv = m.heads * m.dim, m.heads * m.vdim
        names = (("q", hd), ("k", hd), ("v", hv)) + ((("g", hv),) if m.gated else ())
        for name, rows in names:
            if w[name].shape[0] != rows:
                raise ValueError(f"retention weight {name}: {tuple(w[name].shape)} does not have {rows} rows")
        self.in_features, self.out_features = sum(r for _, r in names), hv
        self.prep_width = 2 * hd + hv
        self.w_in = torch.cat([w[n] for n, _ in names], 0).to(device=device, dtype=dtype).contiguous()
        self.w_out = w["o"]
        if m.rot is not None and (m.rot.layout != "half" or m.rot.factor is not None):
            raise ValueError("retention rotates pairs (i, i + dims/2) with unscaled frequencies")
        self.inv_freq = torch.tensor(m.rot.inv_freq(), dtype=torch.float64).to(torch.float32).to(device) if m.rot is not None else None
        self.decay = torch.tensor(m.decay, dtype=torch.float64).to(torch.float32).to(device)

    def scratch_floats(self, tokens: int) -> int:
        return tokens * (self.prep_width + self.out_features)

    def run(self, proj, out, b: StepBatch, run_cache: dict, page_size: int, scratch: torch.Tensor, dt: int, stream) -> None:
        m, T = self.m, b.n_tokens
        prep = scratch[: T * self.prep_width]
        o_raw = scratch[T * self.prep_width: T * (self.prep_width + self.out_features)]
        check(lib.qs_hyb_retention(out.data_ptr(), out.stride(0), prep.data_ptr(), o_raw.data_ptr(), proj.data_ptr(), proj.stride(0),
                                   self.decay.data_ptr(), _p(self.inv_freq), m.rot.dims if m.rot is not None else 0, float(m.dim) ** -0.5,
                                   1 if m.gated else 0, run_cache["state"].data_ptr(), _p(b.tok_pos), _p(b.entry_start), _p(b.entry_len),
                                   _p(b.entry_slot), _p(b.entry_pos0), T, b.n_entries, m.heads, m.dim, m.vdim, self.eps, dt, stream))


class GatedLinearMixer(_Mixer):
    """Gated linear attention: S <- diag(a) S + k v^T, o = S^T q with q times dim^-1/2 and a decay per head and key channel
    a = sigmoid(W_a2 (W_a1 h) + b)^(1/tau) (the low-rank projection's first factor is part of the mixer's one input product, its second an fp32
    product of its own; decay, state and read-out are fp32); unit-RMS heads with a gain shared by the heads, times silu of an output gate.
    The fp32 state lives in the sequence's slot."""

    def __init__(self, m: GatedLinearMixerConfig, w: Dict[str, torch.Tensor], eps: float, dtype, device):
        self.m, self.eps = m, eps
        hd, hv = m.heads * m.dim, m.heads * m.vdim
        rank = w["a1"].shape[0]
        if m.decay_rank and rank != m.decay_rank:
            raise ValueError(f"gated linear attention: a1 has {rank} rows, the configuration says {m.decay_rank}")
        for name, rows in (("q", hd), ("k", hd), ("v", hv), ("g", hv), ("a2", hd)):
            if w[name].shape[0] != rows:
                raise ValueError(f"gated linear attention weight {name}: {tuple(w[name].shape)} does not have {rows} rows")
        if w["a2"].shape[1] != rank or w["a2.b"].numel() != hd or w["norm"].numel() != m.vdim:
            raise ValueError("gated linear attention: a2 is [heads * dim, rank], a2.b has heads * dim entries, norm has vdim")
        self.col_a = 2 * hd + 2 * hv
        self.in_features, self.out_features = self.col_a + rank, hv
        self.prep_width = 3 * hd + hv
        self.w_in = torch.cat([w["q"], w["k"], w["v"], w["g"], w["a1"]], 0).to(device=device, dtype=dtype).contiguous()
        self.w_a2 = w["a2"].to(device=device, dtype=dtype).contiguous()
        self.w_out = w["o"]
        f32 = lambda t: t.to(torch.float32).to(device).contiguous()
        self.a_bias, self.norm_w = f32(w["a2.b"]), f32(w["norm"])

    def scratch_floats(self, tokens: int) -> int:
        return tokens * (self.prep_width + self.out_features)

    def run(self, proj, out, b: StepBatch, run_cache: dict, page_size: int, scratch: torch.Tensor, dt: int, stream) -> None:
        m, T = self.m, b.n_tokens
        prep = scratch[: T * self.prep_width]
        o_raw = scratch[T * self.prep_width: T * (self.prep_width + self.out_features)]
        z = _mm_f32(proj[:, self.col_a:], self.w_a2.t())  # decay logits [T, heads * dim], fp32 from here on
        check(lib.qs_hyb_gated_linear(out.data_ptr(), out.stride(0), prep.data_ptr(), o_raw.data_ptr(), proj.data_ptr(), proj.stride(0), z.data_ptr(),
                                      self.a_bias.data_ptr(), m.tau, self.norm_w.data_ptr(), run_cache["state"].data_ptr(), _p(b.entry_start),
                                      _p(b.entry_len), _p(b.entry_slot), _p(b.entry_pos0), T, b.n_entries, m.heads, m.dim, m.vdim, self.eps, dt, stream))


class LatentAttentionMixer(_Mixer):
    """Latent attention: c_q = unit_rms(W_dq h) g_q, q = W_uq c_q (per head `dim` unrotated and `rot_dim` rotated numbers); [c | k_rot] =
    [unit_rms((W_dkv h)[:kv_rank]) g_kv | rotate((W_dkv h)[kv_rank:])] is all the cache holds per position.  Scores
    (q_nope . W_uk c + q_rot . k_rot) * scale are formed as (W_uk^T q_nope) . c + q_rot . k_rot: the key up-projection is applied to the
    query (a batched product over the heads), every head scores the cached rows as they lie in memory, the weighted sum of the latents goes
    through the value up-projection W_uv (another batched product), and a sigmoid gate of the mixer's input scales each head (or, gate_wide,
    each output number).  With q_rank 0 there is no query latent: q = W_q h is part of the one input product.  A sink adds exp(sink[h]) to head
    h's softmax denominators."""

    def __init__(self, m: LatentAttentionMixerConfig, w: Dict[str, torch.Tensor], eps: float, dtype, device):
        self.m, self.eps = m, eps
        H, D, R, Dv, K, Q = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank
        HQ, NG = H * (D + R), (H * Dv if m.gate_wide else H)
        names = ((("dq", Q), ("uq", HQ)) if Q else (("q", HQ),)) + (("dkv", K + R), ("uk", H * D), ("uv", H * Dv)) + ((("g", NG),) if m.gate else ())
        for name, rows in names:
            if w[name].shape[0] != rows:
                raise ValueError(f"latent attention weight {name}: {tuple(w[name].shape)} does not have {rows} rows")
        if w["uk"].shape[1] != K or w["uv"].shape[1] != K or w["dkv.norm"].numel() != K or (Q and (w["uq"].shape[1] != Q or w["dq.norm"].numel() != Q)):
            raise ValueError("latent attention: up-projections and gains do not match q_rank / kv_rank")
        st = lambda t: t.to(device=device, dtype=dtype).contiguous()
        f32 = lambda t: t.to(torch.float32).to(device).contiguous()
        # one product makes [query latent (or, without one, the queries) | key/value latent, rotated key part | gate logits]
        NQ = Q if Q else HQ
        self.col_q, self.col_kv, self.col_g = 0, NQ, NQ + K + R
        self.in_features = NQ + K + R + (NG if m.gate else 0)
        self.out_features = H * Dv
        self.w_in = st(_pad_rows(torch.cat([w["dq"] if Q else w["q"], w["dkv"]] + ([w["g"]] if m.gate else []), 0)))
        self.in_features = self.w_in.shape[0]
        self.w_uq = st(w["uq"]) if Q else None
        self.w_uk = st(w["uk"]).view(H, D, K)                                   # q_lat[h] = q_nope[h] @ w_uk[h]
        self.w_uv = st(w["uv"].reshape(H, Dv, K).transpose(1, 2))               # [H, K, Dv]: values[h] = o_lat[h] @ w_uv[h]
        self.w_out = w["o"]
        # prompt portions: keys [W_uk,h c | k_rot] and values W_uv,h c of every head are laid out per step from the cached rows (one product
        # each; the identity block passes the shared rotated part into every head's key), and the per-head tile kernels run on them
        aug = torch.zeros((H, D + R, K + R), dtype=torch.float32)
        aug[:, :D, :K] = w["uk"].to(torch.float32).reshape(H, D, K)
        aug[:, D:, K:] = torch.eye(R)
        self.w_keys = st(aug.reshape(H * (D + R), K + R))
        self.w_values = st(w["uv"])
        self.per_head_ok = lib.qs_hyb_attention_fast_supported(_DT[dtype], H, H, 1, D + R, Dv, HQ if Q else self.in_features) == 1
        self.gain_q, self.gain_kv = f32(w["dq.norm"]) if Q else None, f32(w["dkv.norm"])
        self.inv_freq = torch.tensor(m.rot.inv_freq(), dtype=torch.float64).to(torch.float32).to(device) if m.rot is not None else None
        self.rot_dims = m.rot.dims if m.rot is not None else 0
        self.rot_layout = _ROT_LAYOUT[m.rot.layout] if m.rot is not None else 0
        self.amp = float(m.rot.amplitude()) if m.rot is not None else 1.0
        self.sinks = f32(w["sink"]) if m.sink else None
        if self.sinks is not None and self.sinks.numel() != H:
            raise ValueError("latent attention: the sink has one number per head")

    def scratch_floats(self, tokens: int) -> int:
        per_head = int(lib.qs_hyb_attention_scratch_floats(tokens, self.m.heads, self.m.heads, 1, self.m.vdim)) if self.per_head_ok else 0
        return max(int(lib.qs_hyb_latent_attention_scratch_floats(tokens, self.m.heads, self.m.kv_rank)), per_head)

    def run(self, proj: torch.Tensor, out: torch.Tensor, b: StepBatch, run_cache: dict, page_size: int, scratch, dt: int, stream) -> None:
        m, T, dev = self.m, b.n_tokens, proj.device
        H, D, R, Dv, K, Q = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank
        pool = run_cache["c"]
        cq = torch.empty((T, Q), dtype=proj.dtype, device=dev) if Q else None
        check(lib.qs_hyb_latent_prepare(_p(cq), proj.data_ptr(), proj.stride(0), self.col_q, self.col_kv, _p(self.gain_q),
                                        self.gain_kv.data_ptr(), _p(self.inv_freq), self.rot_dims, _p(b.tok_slot), _p(b.tok_pos), _p(b.block_table),
                                        b.block_table.shape[1], pool.data_ptr(), T, Q, K, R, page_size, self.eps, self.rot_layout, self.amp, dt, stream))
        q = torch.mm(cq, self.w_uq.t()) if Q else proj[:, :H * (D + R)]          # [T, H (D + R)]
        fast = scratch is not None and LATENT_IMPL != "plain" and lib.qs_hyb_latent_attention_fast_supported(dt, H, K, R) == 1
        # portions of at least StepBatch.TILE_MIN tokens: per-head keys and values (less arithmetic per score than the K + R numbers of a cell);
        # single tokens and short portions: queries taken to the latent, scored against the cells as they lie
        per_head = scratch is not None and self.per_head_ok and LATENT_IMPL not in ("plain", "latent") and b.n_tiles > 0 and b.n_ctx_pages > 0
        latent = not per_head or b.n_short > 0
        qa = olat = ov = otok = None
        if latent:
            qlat = torch.bmm(q.unflatten(1, (H, D + R))[:, :, :D].transpose(0, 1), self.w_uk)  # [H, T, K]
            qa = torch.empty((T, H, K + R), dtype=proj.dtype, device=dev)
        check(lib.qs_hyb_latent_query(_p(qa), qlat.data_ptr() if latent else None, q.data_ptr(), q.stride(0), _p(self.inv_freq), self.rot_dims,
                                      _p(b.tok_pos), T, H, D, K, R, 1 if per_head else 0, self.rot_layout, self.amp, dt, stream))
        if per_head:
            cells = pool.index_select(0, b.ctx_src).view(-1, K + R)
            keys, values = torch.mm(cells, self.w_keys.t()), torch.mm(cells[:, :K], self.w_values.t())
            otok = torch.empty((T, H * Dv), dtype=proj.dtype, device=dev)
            check(lib.qs_hyb_attention_fast(otok.data_ptr(), otok.stride(0), q.data_ptr(), q.stride(0), keys.data_ptr(), values.data_ptr(), _p(b.tok_slot),
                                            _p(b.tok_pos), b.ctx_table.data_ptr(), b.ctx_table.shape[1], _p(b.tile_entry), _p(b.tile_row0), b.n_tiles,
                                            _p(b.long_tokens), b.n_long, None, 0, _p(b.entry_start), _p(b.entry_len), _p(b.entry_slot), _p(b.entry_pos0),
                                            scratch.data_ptr(), H, H, 1, D + R, Dv, m.scale, 0.0, 1.0, self.eps, 0, page_size, m.chunk, m.window,
                                            _p(self.sinks), None, dt, stream))
        if latent:
            olat = torch.empty((H, T, K), dtype=proj.dtype, device=dev)
            if fast:
                check(lib.qs_hyb_latent_attention_fast(olat.data_ptr(), qa.data_ptr(), pool.data_ptr(), _p(b.tok_slot), _p(b.tok_pos), _p(b.block_table),
                                                       b.block_table.shape[1], _p(b.tile_entry), _p(b.tile_row0), 0 if per_head else b.n_tiles,
                                                       _p(b.short_tokens), b.n_short, _p(b.entry_start), _p(b.entry_len), _p(b.entry_slot),
                                                       _p(b.entry_pos0), T, scratch.data_ptr(), H, K, R, m.scale, page_size, m.chunk, m.window,
                                                       _p(self.sinks), dt, stream))
            else:
                check(lib.qs_hyb_latent_attention(olat.data_ptr(), qa.data_ptr(), pool.data_ptr(), _p(b.tok_slot), _p(b.tok_pos), _p(b.block_table),
                                                  b.block_table.shape[1], T, H, K, R, m.scale, page_size, m.chunk, m.window, _p(self.sinks), dt, stream))
            ov = torch.bmm(olat, self.w_uv)                                      # [H, T, Dv]
        check(lib.qs_hyb_latent_gate_out(out.data_ptr(), out.stride(0), _p(ov), _p(otok), otok.stride(0) if per_head else 0, _p(b.tok_entry),
                                         _p(b.entry_len), StepBatch.TILE_MIN if latent else 1, proj.data_ptr() if m.gate else None, proj.stride(0),
                                         self.col_g, T, H, Dv, 1 if m.gate_wide else 0, dt, stream))


LATENT_IMPL = None  # tests: "plain" keeps the latent attention on the CUDA-core kernel, "latent" keeps prompt portions on the latent-space tiles


class ParallelMixer(_Mixer):
    """Two mixers on the same input: one product makes both projection rows, each runs on its part, and the result is
    scale (norm(W_o,left heads_left) gain_left + norm(W_o,right heads_right) gain_right) with plain RMS norms over the width."""

    def __init__(self, m: ParallelMixerConfig, w: Dict[str, torch.Tensor], eps: float, dtype, device):
        self.m, self.eps = m, eps
        sub = lambda side: {k[len(side) + 1:]: t for k, t in w.items() if k.startswith(side + ".") and k != side + ".out"}
        self.left = MIXERS[type(m.left)](m.left, sub("left"), eps, dtype, device)
        self.right = MIXERS[type(m.right)](m.right, sub("right"), eps, dtype, device)
        self.in_features = self.left.in_features + self.right.in_features
        self.out_features = self.left.out_features + self.right.out_features
        self.w_in = torch.cat([self.left.w_in, self.right.w_in], 0).contiguous()
        del self.left.w_in, self.right.w_in
        f32 = lambda t: t.to(torch.float32).to(device).contiguous()
        self.gain_left, self.gain_right = f32(w["left.out"]), f32(w["right.out"])

    def scratch_floats(self, tokens: int) -> int:
        return max(self.left.scratch_floats(tokens), self.right.scratch_floats(tokens))  # they run one after the other

    def place_out(self, st) -> None:
        self.left.place_out(st)
        self.right.place_out(st)

    def run(self, proj, out, b: StepBatch, run_cache: dict, page_size: int, scratch, dt: int, stream) -> None:
        a, oa = self.left.in_features, self.left.out_features
        self.left.run(proj[:, :a], out[:, :oa], b, run_cache["left"], page_size, scratch, dt, stream)
        self.right.run(proj[:, a:], out[:, oa:], b, run_cache["right"], page_size, scratch, dt, stream)

    def project(self, cat: torch.Tensor, dt: int, stream):
        oa = self.left.out_features
        yl, fl = self.left.project(cat[:, :oa], dt, stream)
        yr, fr = self.right.project(cat[:, oa:], dt, stream)
        if fl or fr:
            raise NotImplementedError("side-by-side mixers whose own outputs are fp32 rows")
        T, W = yl.shape
        y = torch.empty((T, W), dtype=torch.float32, device=cat.device)
        check(lib.qs_hyb_branch_norm_mean(y.data_ptr(), yl.data_ptr(), yr.data_ptr(), self.gain_left.data_ptr(), self.gain_right.data_ptr(),
                                          self.m.scale, self.eps, T, W, dt, stream))
        return y, True


MIXERS = {AttentionMixerConfig: MultiMapAttentionMixer, DeltaMixerConfig: GatedDeltaMixer, GateRecurrenceMixerConfig: GateRecurrenceMixer,
          RetentionMixerConfig: RetentionMixer, ParallelMixerConfig: ParallelMixer, LatentAttentionMixerConfig: LatentAttentionMixer,
          GatedLinearMixerConfig: GatedLinearMixer}


# ------------------------------------------------------------------------------------------------------------------------
# feed-forwards of sequential blocks
# ------------------------------------------------------------------------------------------------------------------------
MOE_IMPL = None  # tests: force "sorted" or "dense"; None picks by storage type and sizes


class MoeFeedForward:
    """Mixture of experts with an optional shared expert.  The router (fp32 logits; softmax scores, or sigmoid scores with a correction and
    groups of experts; the best `top`) is one kernel.  Two ways to run the experts:

    "sorted": the (token, chosen expert) pairs are sorted by expert on the device (every expert's rows in token order), the tokens' rows are
              gathered in that order, two grouped matrix products (one group per expert) make gate | up and the down projection, and a kernel
              sums a token's experts with their router scores in fp32, beside the shared expert's dense products.  Only chosen experts compute.
    "dense":  the gate / up rows of all experts (and the shared one) are stacked into ONE pair of products; the activation kernel weights an
              expert's columns with the token's router score for it (exact zeros for experts the token does not use), and the stacked down
              projection sums the weighted experts in its fp32 accumulation.  Exact in every storage type and for every size.
    bfloat16 models whose sizes suit the grouped product (width and expert size multiples of 8) run "sorted", all others "dense"."""

    def __init__(self, c: MoeConfig, w: Dict[str, torch.Tensor], width: int, dtype, device):
        self.c, self.width = c, width
        st = lambda t: t.to(device=device, dtype=dtype).contiguous()
        experts = [f"e{e}" for e in range(c.experts)]
        names = experts + (["shared"] if c.shared_ff else [])
        for n in names:
            ff = c.shared_ff if n == "shared" else c.ff
            for part, shape in (("gate", (ff, width)), ("up", (ff, width)), ("down", (width, ff))):
                if tuple(w[f"{n}.{part}"].shape) != shape:
                    raise ValueError(f"expert weight {n}.{part}: {tuple(w[f'{n}.{part}'].shape)} is not {shape}")
        self.impl = MOE_IMPL or ("sorted" if dtype == torch.bfloat16 and width % 8 == 0 and c.ff % 8 == 0 else "dense")
        if self.impl == "sorted":
            self.w_gu = st(torch.stack([torch.cat([w[f"{n}.gate"], w[f"{n}.up"]], 0) for n in experts]))  # [E, 2 ff, W]
            self.w_dn = st(torch.stack([w[f"{n}.down"] for n in experts]))                               # [E, W, ff]
            if c.shared_ff:
                self.w_sh_in = st(torch.cat([w["shared.gate"], w["shared.up"]], 0))
                self.w_sh_dn = st(w["shared.down"])
            self.work = torch.empty(int(lib.qs_hyb_moe_plan_work_ints(c.experts)), dtype=torch.int32, device=device)
        elif self.impl == "dense":
            self.F = c.experts * c.ff + c.shared_ff
            self.w_in = st(torch.cat([w[f"{n}.gate"] for n in names] + [w[f"{n}.up"] for n in names], 0))  # [2 F, W]
            self.w_down = st(torch.cat([w[f"{n}.down"] for n in names], 1))                               # [W, F]
        else:
            raise ValueError(f"unknown expert implementation {self.impl!r}")
        self.w_router = w["router"].to(torch.float32).to(device).contiguous()
        if tuple(self.w_router.shape) != (c.experts, width):
            raise ValueError("router weight is not [experts, width]")
        if c.router not in _ROUTER_MODE:
            raise ValueError(f"unknown router {c.router!r}")
        self.correction = w["correction"].to(torch.float32).to(device).contiguous() if c.correction else None
        if self.correction is not None and self.correction.numel() != c.experts:
            raise ValueError("the router's correction has one number per expert")

    def run(self, h: torch.Tensor, dt: int, stream):
        """h [T, W] (storage type) -> (rows [T, W], rows are fp32)."""
        c, T, W = self.c, h.shape[0], h.shape[1]
        dev = h.device
        route = torch.empty((T, c.experts), dtype=torch.float32, device=dev)
        top_idx = torch.empty((T, c.top), dtype=torch.int32, device=dev)
        top_w = torch.empty((T, c.top), dtype=torch.float32, device=dev)
        check(lib.qs_hyb_moe_router(route.data_ptr(), top_idx.data_ptr(), top_w.data_ptr(), h.data_ptr(), self.w_router.data_ptr(), T, W, c.experts,
                                    c.top, _ROUTER_MODE[c.router], _p(self.correction), c.groups, c.keep, dt, stream))
        if self.impl == "dense":
            gu = torch.mm(h, self.w_in.t())
            act = torch.empty((T, self.F), dtype=h.dtype, device=dev)
            check(lib.qs_hyb_moe_act(act.data_ptr(), gu.data_ptr(), route.data_ptr(), T, c.experts, c.ff, c.limit, c.shared_ff, c.shared_limit, c.alpha,
                                     c.up_shift, dt, stream))
            return torch.mm(act, self.w_down.t()), False
        n = T * c.top
        ends = torch.empty(c.experts, dtype=torch.int32, device=dev)
        row_of = torch.empty(n, dtype=torch.int32, device=dev)
        src = torch.empty(n, dtype=torch.int32, device=dev)
        check(lib.qs_hyb_moe_plan(ends.data_ptr(), row_of.data_ptr(), src.data_ptr(), self.work.data_ptr(), top_idx.data_ptr(), T, c.experts, c.top,
                                  stream))
        xs = torch.empty((n, W), dtype=h.dtype, device=dev)
        check(lib.qs_hyb_moe_gather(xs.data_ptr(), h.data_ptr(), src.data_ptr(), n, W, dt, stream))
        gu = torch.nn.functional.grouped_mm(xs, self.w_gu.transpose(-2, -1), offs=ends)
        act = torch.empty((n, c.ff), dtype=h.dtype, device=dev)
        check(lib.qs_hyb_moe_act(act.data_ptr(), gu.data_ptr(), None, n, 0, 0, 0.0, c.ff, c.limit, c.alpha, c.up_shift, dt, stream))
        rows = torch.nn.functional.grouped_mm(act, self.w_dn.transpose(-2, -1), offs=ends)
        shared = None
        if c.shared_ff:
            gs = torch.mm(h, self.w_sh_in.t())
            sa = torch.empty((T, c.shared_ff), dtype=h.dtype, device=dev)
            check(lib.qs_hyb_moe_act(sa.data_ptr(), gs.data_ptr(), None, T, 0, 0, 0.0, c.shared_ff, c.shared_limit, c.alpha, c.up_shift, dt, stream))
            shared = torch.mm(sa, self.w_sh_dn.t())
        y = torch.empty((T, W), dtype=torch.float32, device=dev)
        check(lib.qs_hyb_moe_combine(y.data_ptr(), rows.data_ptr(), _p(shared), row_of.data_ptr(), top_w.data_ptr(), T, c.top, W, dt, stream))
        return y, True


class DenseFeedForward:
    """W_down (act(W_gate h + b_gate) * (W_up h + b_up)) [+ b_down], act gelu_tanh or silu.  The down projection's bias (`out_bias`) is left
    to the block, which adds it where it takes the rows."""

    def __init__(self, c: MlpConfig, w: Dict[str, torch.Tensor], width: int, dtype, device):
        st = lambda t: t.to(device=device, dtype=dtype).contiguous()
        if not c.gated:
            raise NotImplementedError("a dense feed-forward without a gate, outside a parallel block")
        if c.act not in _ACT:
            raise ValueError(f"unknown activation {c.act!r}")
        if tuple(w["gate"].shape) != (c.ff, width) or tuple(w["up"].shape) != (c.ff, width) or tuple(w["down"].shape) != (width, c.ff):
            raise ValueError("dense feed-forward: the projections do not match ff x width")
        self.ff, self.act = c.ff, _ACT[c.act]
        self.w_in, self.w_down = st(torch.cat([w["gate"], w["up"]], 0)), st(w["down"])
        self.in_bias = self.out_bias = None
        if c.bias:
            self.in_bias = torch.cat([w["gate.b"], w["up.b"]], 0).to(torch.float32).to(device).contiguous()
            self.out_bias = w["down.b"].to(torch.float32).to(device).contiguous()
            if self.in_bias.numel() != 2 * c.ff or self.out_bias.numel() != width:
                raise ValueError("dense feed-forward: the biases do not match their projections")

    def run(self, h: torch.Tensor, dt: int, stream):
        gu = torch.mm(h, self.w_in.t())
        act = torch.empty((h.shape[0], self.ff), dtype=h.dtype, device=h.device)
        if self.in_bias is None and self.act == 0:
            check(lib.qs_hyb_gelu_tanh_mul(act.data_ptr(), act.stride(0), gu.data_ptr(), h.shape[0], self.ff, dt, stream))
        else:
            check(lib.qs_hyb_bias_gated_act(act.data_ptr(), act.stride(0), gu.data_ptr(), gu.stride(0), _p(self.in_bias), h.shape[0], self.ff, self.act, dt,
                                            stream))
        return _mm_f32(act, self.w_down.t()), True


FEED_FORWARDS = {MoeConfig: MoeFeedForward, MlpConfig: DenseFeedForward}


@dataclass
class _Hyper:
    """Coefficients of one sublayer's connection to the residual streams: read (`cin` [s]), write (`cout` [s]) and mix [from, to]."""
    cin: torch.Tensor
    cout: torch.Tensor
    mix: torch.Tensor


# ------------------------------------------------------------------------------------------------------------------------
# the decoder
# ------------------------------------------------------------------------------------------------------------------------
class _Layer:
    def __init__(self, mixer, norm1, norm2, w_mlp_in, w_out, ff, hc1=None, hc2=None):
        self.mixer, self.norm1, self.norm2, self.w_mlp_in, self.w_out, self.ff = mixer, norm1, norm2, w_mlp_in, w_out, ff
        self.hc1, self.hc2 = hc1, hc2
        # parallel blocks: norm biases (layer norms), a dense feed-forward folded into the block's products (ff columns, gated or not, biases of
        # its projections), or a feed-forward that runs by itself beside the mixer (mixture of experts)
        self.norm1_b = self.norm2_b = self.mlp_in_bias = self.out_bias = self.side_ff = None
        self.w_all_in = None  # mixer and feed-forward input projections stacked (blocks whose branches read one normed row)
        self.gated = True
        self.ls1 = self.ls2 = None  # post-norm blocks: per-channel scales of the normed sublayer outputs


class HybridDecoder:
    """Two block forms (HybridConfig.block):

    "parallel":   x <- x + (mixer(norm1 x) + ff(norm2 x)) per layer run, both branches of the same x; the two output projections are ONE
                  product: [mixer heads | ff activation] @ [W_o | W_down]^T, so the sum of the branches is accumulated in fp32 inside the GEMM.
    "sequential": x <- x + mixer(norm1 x), then x <- x + ff(norm2 x), on `streams` residual streams [T, streams, W] whose read, write and
                  mixing coefficients belong to the sublayer (one stream with coefficients 1 is the plain residual).  A sublayer's write to
                  the streams happens inside the next sublayer's norm kernel.
    "post":       x <- x + ls1 norm1(mixer(x)), then x <- x + ls2 norm2(ff(x)): a sublayer takes the un-normed stream (its storage-type copy is
                  written by the kernel that lands the previous sublayer), and its fp32 output rows are normed, scaled per channel and
                  added in one kernel."""

    def __init__(self, cfg: HybridConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None):
        if dtype not in _DT:
            raise ValueError("dtype must be torch.bfloat16 or torch.float32")
        self.cfg, self.dtype, self.dt = cfg, dtype, _DT[dtype]
        self.device = dev = device or torch.device("cuda", torch.cuda.current_device())
        if dev.type != "cuda":
            raise RuntimeError("qserve_b200 has no CPU path: HybridDecoder needs a CUDA device")
        if dtype == torch.float32:
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
        st = lambda t: t.to(device=dev, dtype=dtype).contiguous()
        f32 = lambda t: t.to(torch.float32).to(dev).contiguous()
        W = cfg.width
        if tuple(weights["embed"].shape) != (cfg.vocab, W) or tuple(weights["head"].shape) != (cfg.vocab, W):
            raise ValueError("embed / head do not match vocab x width")
        self.embed = st(weights["embed"])
        self.pair = st(weights["bigram"]) if cfg.pair_buckets > 0 else None
        if self.pair is not None and self.pair.shape[0] != cfg.pair_buckets + 1:
            raise ValueError("the pair table must have buckets + 1 rows")
        self.head = st(weights["head"])
        self.final_norm = f32(weights["final.norm"])
        self.layers: List[_Layer] = []
        if cfg.block not in ("parallel", "sequential", "post"):
            raise ValueError(f"unknown block form {cfg.block!r}")
        self.n_streams = max(cfg.streams, 1) if cfg.block == "sequential" else 1
        one = torch.ones(1, dtype=torch.float32, device=dev)

        def hyper(pre: str) -> _Hyper:
            if cfg.streams <= 0:
                return _Hyper(one, one, one)
            h = _Hyper(f32(weights[pre + "in"]), f32(weights[pre + "out"]), f32(weights[pre + "mix"]))
            if h.cin.numel() != cfg.streams or h.cout.numel() != cfg.streams or tuple(h.mix.shape) != (cfg.streams, cfg.streams):
                raise ValueError(f"{pre}*: hyper-connection coefficients do not match {cfg.streams} streams")
            return h

        for i, ly in enumerate(cfg.layers):
            pre = f"l{i}."
            mw = {k[len(pre) + 4:]: v for k, v in weights.items() if k.startswith(pre + "mix.")}
            mixer = MIXERS[type(ly.mixer)](ly.mixer, mw, cfg.eps, dtype, dev)
            if cfg.block == "post":
                mixer.place_out(st)
                ff = norm2 = None
                if ly.mlp is not None:
                    fw = {k[len(pre) + 4:]: v for k, v in weights.items() if k.startswith(pre + "mlp.")}
                    ff, norm2 = FEED_FORWARDS[type(ly.mlp)](ly.mlp, fw, W, dtype, dev), f32(weights[pre + "norm2"])
                layer = _Layer(mixer, f32(weights[pre + "norm1"]), norm2, None, None, ff)
                if cfg.layer_scale:
                    layer.ls1 = f32(weights[pre + "ls1"])
                    layer.ls2 = f32(weights[pre + "ls2"]) if ff is not None else None
                for t in (layer.norm1, layer.norm2, layer.ls1, layer.ls2):
                    if t is not None and t.numel() != W:
                        raise ValueError(f"{pre}: norm gains and layer scales have `width` numbers")
                self.layers.append(layer)
                continue
            if cfg.block == "sequential":
                mixer.place_out(st)
                ff, norm2, hc2 = None, None, None
                if ly.mlp is not None:
                    fw = {k[len(pre) + 4:]: v for k, v in weights.items() if k.startswith(pre + "mlp.")}
                    ff = FEED_FORWARDS[type(ly.mlp)](ly.mlp, fw, W, dtype, dev)
                    if getattr(ff, "out_bias", None) is not None:
                        raise NotImplementedError("a biased dense feed-forward on hyper-connected streams")
                    norm2, hc2 = f32(weights[pre + "norm2"]), hyper(pre + "hc2.")
                self.layers.append(_Layer(mixer, f32(weights[pre + "norm1"]), norm2, None, None, ff, hyper(pre + "hc1."), hc2))
                continue
            outs = [mixer.w_out]
            w_mlp_in, norm2, ff = None, None, 0
            dense = isinstance(ly.mlp, MlpConfig)
            if dense:  # folded: its activation sits beside the mixer's heads as input of ONE output product
                ff = ly.mlp.ff
                w_mlp_in = st(torch.cat([weights[pre + "mlp.gate"], weights[pre + "mlp.up"]], 0) if ly.mlp.gated else weights[pre + "mlp.up"])
                if tuple(w_mlp_in.shape) != ((2 if ly.mlp.gated else 1) * ff, W) or tuple(weights[pre + "mlp.down"].shape) != (W, ff):
                    raise ValueError(f"{pre}mlp: the projections do not match ff x width")
                outs.append(weights[pre + "mlp.down"])
            if ly.mlp is not None and not cfg.shared_norm:
                norm2 = f32(weights[pre + "norm2"])
            w_out = st(torch.cat(outs, 1))  # [W, heads*vdim + ff]
            del mixer.w_out
            layer = _Layer(mixer, f32(weights[pre + "norm1"]), norm2, w_mlp_in, w_out, ff)
            if cfg.norm_kind == "layer":
                layer.norm1_b = f32(weights[pre + "norm1.b"])
                layer.norm2_b = f32(weights[pre + "norm2.b"]) if norm2 is not None else None
            if dense:
                layer.gated = ly.mlp.gated
                if ly.mlp.bias:
                    if ly.mlp.gated:
                        layer.mlp_in_bias = f32(torch.cat([weights[pre + "mlp.gate.b"], weights[pre + "mlp.up.b"]], 0))
                    else:
                        layer.mlp_in_bias = f32(weights[pre + "mlp.up.b"])
                    layer.out_bias = f32(weights[pre + "mlp.down.b"])
                    if layer.mlp_in_bias.numel() != w_mlp_in.shape[0] or layer.out_bias.numel() != W:
                        raise ValueError(f"{pre}mlp: the biases do not match their projections")
                if ly.mlp.gated and ly.mlp.bias:
                    raise NotImplementedError("a gated dense feed-forward with biases")
            elif ly.mlp is not None:
                fw = {k[len(pre) + 4:]: v for k, v in weights.items() if k.startswith(pre + "mlp.")}
                layer.side_ff = FEED_FORWARDS[type(ly.mlp)](ly.mlp, fw, W, dtype, dev)
            if dense and cfg.shared_norm and not ly.mlp.gated:
                layer.w_all_in = torch.cat([mixer.w_in, w_mlp_in], 0).contiguous()
                del mixer.w_in
                layer.w_mlp_in = None
            self.layers.append(layer)
        if cfg.norm_kind not in _NORM_KIND:
            raise ValueError(f"unknown norm {cfg.norm_kind!r}")
        if cfg.norm_kind == "layer" and (cfg.block != "parallel" or cfg.norm_offset != 0.0 or cfg.norm_groups != 1):
            raise NotImplementedError("layer norms are built for parallel blocks with plain gains")
        self.final_norm_b = f32(weights["final.norm.b"]) if cfg.norm_kind == "layer" else None
        self.loop_in = None
        if cfg.loop_in and cfg.pass_starts():
            self.loop_in = st(weights["loop.in"])
            if tuple(self.loop_in.shape) != (W, 2 * W):
                raise ValueError("loop.in must be [width, 2 width]")
        self.schedule = cfg.schedule()
        self._scratch: Optional[torch.Tensor] = None

    @classmethod
    def from_dir(cls, model_dir: str, dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None) -> "HybridDecoder":
        import os

        from .checkpoint import read_safetensors
        from .modelcfg import read_model_config

        return cls(read_model_config(model_dir), read_safetensors(os.path.join(model_dir, "model.safetensors")), dtype, device)

    def new_cache(self, max_tokens: int, max_seqs: int = 4, page_size: int = 64) -> HybridCache:
        return HybridCache(self.cfg, self.dtype, self.device, max_tokens, max_seqs, page_size)

    # ----------------------------------------------------------------------------------------------------------------
    def scratch_floats(self, tokens: int) -> int:
        return max((ly.mixer.scratch_floats(tokens) for ly in self.layers), default=0)

    def forward(self, b: StepBatch, cache: HybridCache, tap=None, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Residual stream [T, W] fp32 after the last layer run.  `tap(run_index, x)` (debugging / tests) sees it after every run.
        `scratch` (fp32, at least scratch_floats(T)): the caller's own work space, e.g. one that a captured CUDA graph keeps."""
        cfg, dev, dt, T, W = self.cfg, self.device, self.dt, b.n_tokens, self.cfg.width
        s = _stream(dev)
        x = torch.empty((T, self.n_streams, W) if cfg.block == "sequential" else (T, W), dtype=torch.float32, device=dev)
        check(lib.qs_hyb_embed(x.data_ptr(), _p(b.tokens), _p(b.prev), self.embed.data_ptr(), _p(self.pair), T, W, cfg.pair_buckets,
                               cfg.pair_mul_prev, cfg.pair_mul_cur, cfg.embed_scale, self.n_streams, dt, s))
        if scratch is None:
            need = self.scratch_floats(T)
            if need and (self._scratch is None or self._scratch.numel() < need):
                self._scratch = torch.empty(need, dtype=torch.float32, device=dev)
            scratch = self._scratch
        if cfg.block == "sequential":
            return self._forward_sequential(x, b, cache, tap, scratch, s)
        if cfg.block == "post":
            return self._forward_post(x, b, cache, tap, scratch, s)
        return self._forward_parallel(x, b, cache, tap, scratch, s)

    def _land(self, x, pending, s, out_h=None, w=None, bias=None, cat_out=None, x0=None) -> None:
        """x <- x + the pending sublayer outputs (rows, rows are fp32, second rows, they are fp32, a bias row); then the norm of x into out_h and /
        or [x | x0] into cat_out."""
        a1, f1, a2, f2, ab = pending if pending is not None else (None, False, None, False, None)
        check(lib.qs_hyb_stream_update_norm(_p(out_h), _p(cat_out), x.data_ptr(), _p(x0), _p(a1), 1 if f1 else 0, _p(a2), 1 if f2 else 0, _p(ab), _p(w),
                                            _p(bias), _NORM_KIND[self.cfg.norm_kind] if out_h is not None else 0, self.cfg.eps, x.shape[0],
                                            self.cfg.width, self.dt, s))

    def _forward_parallel(self, x, b: StepBatch, cache: HybridCache, tap, scratch, s) -> torch.Tensor:
        cfg, dev, dt, T, W = self.cfg, self.device, self.dt, b.n_tokens, self.cfg.width
        h1 = torch.empty((T, W), dtype=self.dtype, device=dev)
        h2 = h1 if cfg.shared_norm else torch.empty((T, W), dtype=self.dtype, device=dev)
        starts = set(cfg.pass_starts()) if self.loop_in is not None else set()
        x0 = x.clone() if starts else None  # the embedding output, read again at the start of every pass
        # the outputs of the previous layer still to be added to the stream: they land inside the next kernel that reads it (one pass over x)
        pending = None
        for run, li in enumerate(self.schedule):
            ly = self.layers[li]
            if run in starts:  # x <- W_in [x; x0]
                xin = torch.empty((T, 2 * W), dtype=self.dtype, device=dev)
                self._land(x, pending, s, cat_out=xin, x0=x0)
                pending = None
                x = _mm_f32(xin, self.loop_in.t())
            has_ff = ly.ff > 0 or ly.side_ff is not None
            plain = pending is None or (pending[2] is None and pending[4] is None and not pending[1])
            if cfg.norm_kind == "rms" and not cfg.shared_norm and plain:
                check(lib.qs_hyb_rms_norm(h1.data_ptr(), _p(h2) if has_ff else None, x.data_ptr(), _p(pending[0]) if pending else None,
                                          ly.norm1.data_ptr(), _p(ly.norm2), cfg.norm_offset, cfg.eps, T, W, dt, s))
            else:
                self._land(x, pending, s, out_h=h1, w=ly.norm1, bias=ly.norm1_b)
                if has_ff and not cfg.shared_norm:
                    self._land(x, None, s, out_h=h2, w=ly.norm2, bias=ly.norm2_b)
            if ly.w_all_in is not None:
                # one product for the mixer's projections and the feed-forward's: both read the same normed row
                both = torch.mm(h1, ly.w_all_in.t())
                proj, gu = both[:, :ly.mixer.in_features], both[:, ly.mixer.in_features:]
            else:
                proj = torch.mm(h1, ly.mixer.w_in.t())
                gu = torch.mm(h2, ly.w_mlp_in.t()) if ly.ff else None
            cat = torch.empty((T, ly.mixer.out_features + ly.ff), dtype=self.dtype, device=dev)
            ly.mixer.run(proj, cat[:, :ly.mixer.out_features] if ly.ff else cat, b, cache.runs[run], cache.page_size, scratch, dt, s)
            if ly.ff:
                act = cat.data_ptr() + ly.mixer.out_features * cat.element_size()
                if ly.gated:
                    check(lib.qs_hyb_gelu_tanh_mul(act, cat.stride(0), gu.data_ptr(), T, ly.ff, dt, s))
                else:
                    check(lib.qs_hyb_bias_gelu_tanh(act, cat.stride(0), gu.data_ptr(), gu.stride(0), _p(ly.mlp_in_bias), T, ly.ff, dt, s))
            upd = torch.mm(cat, ly.w_out.t())
            side, side32 = ly.side_ff.run(h2, dt, s) if ly.side_ff is not None else (None, False)
            pending = (upd, False, side, side32, ly.out_bias)
            if tap is not None:  # observers want the stream after every run: add right away
                self._land(x, pending, s)
                pending = None
                tap(run, x)
        if pending is not None:
            self._land(x, pending, s)
        return x

    def _stream_norm(self, out_h, out_sum, x, pending, cin, w, s) -> None:
        """Land the pending sublayer write (rows, rows are fp32, its connection) in the streams, then read them: the norm of sum_s cin[s] x_s
        into out_h and / or that sum itself (cin None: the plain sum) into out_sum."""
        cfg = self.cfg
        y, y32, hc = pending if pending is not None else (None, False, None)
        check(lib.qs_hyb_stream_norm(_p(out_h), _p(out_sum), x.data_ptr(), self.n_streams, _p(y), 1 if y32 else 0, _p(hc.mix) if hc else None,
                                     _p(hc.cout) if hc else None, _p(cin), _p(w), cfg.norm_groups, cfg.norm_offset, cfg.eps, x.shape[0], cfg.width,
                                     self.dt, s))

    def _forward_sequential(self, x, b: StepBatch, cache: HybridCache, tap, scratch, s) -> torch.Tensor:
        dev, dt, T, W = self.device, self.dt, b.n_tokens, self.cfg.width
        pending = None  # the last sublayer's write to the streams, still to land
        h = torch.empty((T, W), dtype=self.dtype, device=dev)
        for run, li in enumerate(self.schedule):
            ly = self.layers[li]
            self._stream_norm(h, None, x, pending, ly.hc1.cin, ly.norm1, s)
            proj = torch.mm(h, ly.mixer.w_in.t())
            cat = torch.empty((T, ly.mixer.out_features), dtype=self.dtype, device=dev)
            ly.mixer.run(proj, cat, b, cache.runs[run], cache.page_size, scratch, dt, s)
            y, y32 = ly.mixer.project(cat, dt, s)
            pending = (y, y32, ly.hc1)
            if ly.ff is not None:
                self._stream_norm(h, None, x, pending, ly.hc2.cin, ly.norm2, s)
                pending = (*ly.ff.run(h, dt, s), ly.hc2)
            if tap is not None:  # observers want the streams' sum after every run
                total = torch.empty((T, W), dtype=torch.float32, device=dev)
                self._stream_norm(None, total, x, pending, None, None, s)
                pending = None
                tap(run, total)
        total = torch.empty((T, W), dtype=torch.float32, device=dev)
        self._stream_norm(None, total, x, pending, None, None, s)
        return total

    def _forward_post(self, x, b: StepBatch, cache: HybridCache, tap, scratch, s) -> torch.Tensor:
        cfg, dev, dt, T, W = self.cfg, self.device, self.dt, b.n_tokens, self.cfg.width
        # the sublayers' input: the fp32 stream as it is with fp32 storage, else its storage-type copy, which every landing kernel renews
        if self.dtype == torch.float32:
            h, h_ptr = x, None
        else:
            h = torch.empty((T, W), dtype=self.dtype, device=dev)
            h_ptr = h.data_ptr()
            check(lib.qs_hyb_cast_rows(h_ptr, x.data_ptr(), T * W, dt, s))
        for run, li in enumerate(self.schedule):
            ly = self.layers[li]
            proj = torch.mm(h, ly.mixer.w_in.t())
            cat = torch.empty((T, ly.mixer.out_features), dtype=self.dtype, device=dev)
            ly.mixer.run(proj, cat, b, cache.runs[run], cache.page_size, scratch, dt, s)
            y = _mm_f32(cat, ly.mixer.w_out.t())
            check(lib.qs_hyb_post_norm_update(h_ptr, x.data_ptr(), y.data_ptr(), 1, None, ly.norm1.data_ptr(), _p(ly.ls1), cfg.norm_offset, cfg.eps, T, W, dt, s))
            if ly.ff is not None:
                y, y32 = ly.ff.run(h, dt, s)
                check(lib.qs_hyb_post_norm_update(h_ptr, x.data_ptr(), y.data_ptr(), 1 if y32 else 0, _p(getattr(ly.ff, "out_bias", None)),
                                                  ly.norm2.data_ptr(), _p(ly.ls2), cfg.norm_offset, cfg.eps, T, W, dt, s))
            if tap is not None:
                tap(run, x)
        return x

    def logits(self, x_rows: torch.Tensor) -> torch.Tensor:
        """Final norm and vocabulary projection of the given stream rows -> fp32 [n, vocab]."""
        n, W = x_rows.shape
        x_rows = x_rows.contiguous()
        h = torch.empty((n, W), dtype=self.dtype, device=self.device)
        if self.cfg.block == "sequential":
            check(lib.qs_hyb_stream_norm(h.data_ptr(), None, x_rows.data_ptr(), 1, None, 0, None, None, None, self.final_norm.data_ptr(),
                                         self.cfg.norm_groups, self.cfg.norm_offset, self.cfg.eps, n, W, self.dt, _stream(self.device)))
            return torch.mm(h, self.head.t()).float()
        s = _stream(self.device)
        if self.cfg.norm_kind == "rms":
            check(lib.qs_hyb_rms_norm(h.data_ptr(), None, x_rows.data_ptr(), None, self.final_norm.data_ptr(), None, self.cfg.norm_offset, self.cfg.eps, n,
                                      W, self.dt, s))
        else:
            self._land(x_rows, None, s, out_h=h, w=self.final_norm, bias=self.final_norm_b)
        out = _mm_f32(h, self.head.t()) if self.cfg.logit_softcap > 0.0 or self.cfg.block == "post" else torch.mm(h, self.head.t()).float()
        if self.cfg.logit_softcap > 0.0:
            check(lib.qs_hyb_softcap(out.data_ptr(), out.numel(), self.cfg.logit_softcap, s))
        return out


def random_weights(cfg: HybridConfig, seed: int = 0, device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random weights of the design's tensor names and shapes (benchmarks and smoke tests: there is no network for checkpoints), scaled so
    that activations stay O(1)."""
    g = torch.Generator(device=device or "cpu")
    g.manual_seed(seed)
    W = cfg.width

    def r(*shape, s=1.0):
        return (torch.randn(*shape, generator=g, device=device) * s).to(dtype)

    def mixer_weights(p: str, m) -> None:
        if isinstance(m, ParallelMixerConfig):
            mixer_weights(p + "left.", m.left)
            mixer_weights(p + "right.", m.right)
            w[p + "left.out"], w[p + "right.out"] = 1.0 + r(W, s=0.1), 1.0 + r(W, s=0.1)
            return
        H, D, Dv = m.heads, m.dim, m.vdim
        if isinstance(m, LatentAttentionMixerConfig):
            K, Q, R = m.kv_rank, m.q_rank, m.rot_dim
            if Q:
                w[p + "dq"], w[p + "dq.norm"], w[p + "uq"] = r(Q, W, s=W ** -0.5), 1.0 + r(Q, s=0.1), r(H * (D + R), Q, s=Q ** -0.5)
            else:
                w[p + "q"] = r(H * (D + R), W, s=W ** -0.5)
            w[p + "dkv"], w[p + "dkv.norm"] = r(K + R, W, s=W ** -0.5), 1.0 + r(K, s=0.1)
            w[p + "uk"], w[p + "uv"] = r(H * D, K, s=K ** -0.5), r(H * Dv, K, s=K ** -0.5)
            if m.gate:
                w[p + "g"] = r(H * Dv if m.gate_wide else H, W, s=W ** -0.5)
            if m.sink:
                w[p + "sink"] = r(H, s=0.5)
        elif isinstance(m, GatedLinearMixerConfig):
            rank = m.decay_rank or 16
            w[p + "q"], w[p + "k"], w[p + "v"], w[p + "g"] = r(H * D, W, s=W ** -0.5), r(H * D, W, s=W ** -0.5), r(H * Dv, W, s=W ** -0.5), r(H * Dv, W, s=W ** -0.5)
            w[p + "a1"], w[p + "a2"], w[p + "a2.b"], w[p + "norm"] = r(rank, W, s=W ** -0.5), r(H * D, rank, s=rank ** -0.5), 2.0 + r(H * D, s=0.5), 1.0 + r(Dv, s=0.1)
        elif isinstance(m, AttentionMixerConfig):
            G = m.kv_heads
            w[p + "q"], w[p + "k"] = r(H * m.maps * D, W, s=W ** -0.5), r(G * m.maps * D, W, s=W ** -0.5)
            if not m.tied_values:
                w[p + "v"] = r(G * Dv, W, s=W ** -0.5)
            if m.qk_gain:
                w[p + "q.norm"], w[p + "k.norm"] = 1.0 + r(D, s=0.1), 1.0 + r(D, s=0.1)
            if m.head_gate:
                w[p + "g"] = r(H, W, s=W ** -0.5)
            if m.maps == 2:
                for n in ("lq1", "lk1", "lq2", "lk2"):
                    w[p + n] = r(D, s=0.1)
            if m.bias:
                w[p + "q.b"], w[p + "k.b"] = r(H * D, s=0.1), r(G * D, s=0.1)
                if not m.tied_values:
                    w[p + "v.b"] = r(G * Dv, s=0.1)
            if m.head_temp:
                w[p + "temp"] = 1.0 + r(H, s=0.1)
            if m.sink:
                w[p + "sink"] = r(H, s=0.5)
        elif isinstance(m, DeltaMixerConfig):
            G = m.kv_heads
            w[p + "q"], w[p + "k"], w[p + "v"] = r(G * D, W, s=W ** -0.5), r(G * D, W, s=W ** -0.5), r(H * Dv, W, s=W ** -0.5)
            for n, c in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                w[p + f"{n}.conv"] = r(c, m.conv, s=0.5)
            w[p + "b"], w[p + "a"], w[p + "g"] = r(H, W, s=W ** -0.5), r(H, W, s=W ** -0.5), r(H * Dv, W, s=W ** -0.5)
            w[p + "A_log"], w[p + "dt_bias"], w[p + "norm"] = r(H, s=0.5), r(H, s=0.5), 1.0 + r(Dv, s=0.1)
        elif isinstance(m, GateRecurrenceMixerConfig):
            w[p + "q"], w[p + "f"], w[p + "v"] = r(H * D, W, s=W ** -0.5), r(H * D, W, s=W ** -0.5), r(H * Dv, W, s=W ** -0.5)
            w[p + "f.b"], w[p + "lower"], w[p + "norm"] = r(H * D, s=0.5), torch.sigmoid(r(H * D).float()).to(dtype), 1.0 + r(Dv, s=0.1)
        elif isinstance(m, RetentionMixerConfig):
            w[p + "q"], w[p + "k"], w[p + "v"] = r(H * D, W, s=W ** -0.5), r(H * D, W, s=W ** -0.5), r(H * Dv, W, s=W ** -0.5)
            if m.gated:
                w[p + "g"] = r(H * Dv, W, s=W ** -0.5)
        else:
            raise TypeError(type(m))
        w[p + "o"] = r(W, H * Dv, s=(H * Dv) ** -0.5)

    gain = (lambda: 1.0 + r(W, s=0.1)) if cfg.norm_offset == 0.0 else (lambda: r(W, s=0.1))
    w = {"embed": r(cfg.vocab, W), "head": r(cfg.vocab, W, s=W ** -0.5), "final.norm": gain()}
    layer_norm = cfg.norm_kind == "layer"
    if layer_norm:
        w["final.norm.b"] = r(W, s=0.1)
    if cfg.loop_in:
        w["loop.in"] = r(W, 2 * W, s=(2 * W) ** -0.5)
    if cfg.pair_buckets:
        w["bigram"] = r(cfg.pair_buckets + 1, W, s=0.5)
    for i, ly in enumerate(cfg.layers):
        p = f"l{i}."
        w[p + "norm1"] = gain()
        mixer_weights(p + "mix.", ly.mixer)
        if layer_norm:
            w[p + "norm1.b"] = r(W, s=0.1)
        if ly.mlp is not None:
            if not cfg.shared_norm:
                w[p + "norm2"] = gain()
                if layer_norm:
                    w[p + "norm2.b"] = r(W, s=0.1)
            if isinstance(ly.mlp, MoeConfig):
                c = ly.mlp
                for n in [f"e{e}" for e in range(c.experts)] + (["shared"] if c.shared_ff else []):
                    ff = c.shared_ff if n == "shared" else c.ff
                    w[f"{p}mlp.{n}.gate"], w[f"{p}mlp.{n}.up"], w[f"{p}mlp.{n}.down"] = r(ff, W, s=W ** -0.5), r(ff, W, s=W ** -0.5), r(W, ff, s=ff ** -0.5)
                w[p + "mlp.router"] = r(c.experts, W, s=W ** -0.5)
                if c.correction:
                    w[p + "mlp.correction"] = r(c.experts, s=0.1)
            else:
                w[p + "mlp.up"], w[p + "mlp.down"] = r(ly.mlp.ff, W, s=W ** -0.5), r(W, ly.mlp.ff, s=ly.mlp.ff ** -0.5)
                if ly.mlp.gated:
                    w[p + "mlp.gate"] = r(ly.mlp.ff, W, s=W ** -0.5)
                if ly.mlp.bias:
                    w[p + "mlp.up.b"], w[p + "mlp.down.b"] = r(ly.mlp.ff, s=0.1), r(W, s=0.1)
                    if ly.mlp.gated:
                        w[p + "mlp.gate.b"] = r(ly.mlp.ff, s=0.1)
        if cfg.layer_scale:
            w[p + "ls1"] = 0.5 + r(W, s=0.05)
            if ly.mlp is not None:
                w[p + "ls2"] = 0.5 + r(W, s=0.05)
        if cfg.streams > 0:
            ns = cfg.streams
            for q in (1, 2) if ly.mlp is not None else (1,):
                w[f"{p}hc{q}.in"] = (torch.full((ns,), 1.0 / ns, device=device) + torch.randn(ns, generator=g, device=device) * 0.05).to(dtype)
                w[f"{p}hc{q}.out"] = (1.0 + torch.randn(ns, generator=g, device=device) * 0.05).to(dtype)
                w[f"{p}hc{q}.mix"] = (torch.eye(ns, device=device) + torch.randn(ns, ns, generator=g, device=device) * 0.02).to(dtype)
    return w
