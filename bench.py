#!/usr/bin/env python
"""bench.py -- tokens/s of the Llama-3-8B W4A8KV4 decode step (batch 64, ctx 1024) on B200 in the driver's JSON contract,
with the per-kernel roofline, the reference's own GPU kernels on the same box, the reference's unmodified model code over
this backend, the tensor-parallel 72B record and the CPU baseline.

  python bench.py --gpus N --steps K --warmup W                 our sm_100a kernels behind the qserve_backend API
  python bench.py --impl reference --gpus N --steps K ...       the reference's CPU path (torch-CPU dequant-then-matmul restatement,
                                                                oracle/cpu_baseline.py) on the host cores; each step = a bounded sample
  python bench.py --impl reference-gpu --steps K ...            the reference's UNMODIFIED CUDA kernels (oracle/_ref, legacy mma.sync
                                                                compiled for sm_100a) driven through the same op sequence / buffers

A "step" is one decode step of the whole model for `batch` sequences (one new token each).  N > 1: the headline is N
data-parallel replicas of the 8B model (it fits one GPU: no collective on the data path), and the `tp` record of the same line
is Qwen1.5-72B (BASELINE config 5, all 80 layers) tensor-parallel over the N GPUs with NCCL all-reduces.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "tokens/s Llama-3-8B W4A8KV4 decode b64"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--precision", default="w4a8kv4")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=None, help="debug only: truncating the model invalidates the number")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip the reference-GPU-kernel block (oracle/_ref)")
    ap.add_argument("--no-refmodel", action="store_true", help="skip the block that runs the reference's unmodified model code over this backend")
    ap.add_argument("--no-tp", action="store_true", help="skip the Qwen1.5-72B tensor-parallel record")
    ap.add_argument("--tp-model", default="qwen1.5-72b")
    ap.add_argument("--tp-layers", type=int, default=None, help="debug only")
    ap.add_argument("--tp-only", action="store_true", help="print only the tensor-parallel record (tuning runs)")
    ap.add_argument("--tp-allreduce", default="peer", choices=["peer", "nccl"], help="TP record: all-reduce fused into add+norm+quant over peer memory, or NCCL")
    ap.add_argument("--tp-timeout", type=float, default=420.0, help="N > 1: seconds after which the tensor-parallel side record is abandoned (the headline line is still printed)")
    ap.add_argument("--tp-exact", action="store_true", help="TP record with the bit-exact parity rule (global per-token amax) instead of the throughput mode")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="eager launches instead of CUDA-graph replay")
    ap.add_argument("--no-fused", action="store_true", help="use exactly the reference op sequence (no fused add+norm / silu+quant extensions)")
    ap.add_argument("--kernel-reps", type=int, default=5)
    ap.add_argument("--hybrid", action="store_true", help="instead of the default workload: prefill and decode throughput of the Rizurax hybrid decoder "
                    "(random weights) at layer sizes of real models, beside the Llama-style W4A8KV4 runner at equal size; prints one JSON line")
    ap.add_argument("--toderax", action="store_true", help="instead of the default workload: prefill and decode throughput of the Toderax decoder "
                    "(hyper-connection streams, gate recurrence, chunked sink attention beside retention, mixture of experts; random weights) at "
                    "layer sizes of real models, beside the Rizurax hybrid decoder at equal size; prints one JSON line")
    ap.add_argument("--nusuvik", action="store_true", help="instead of the default workload: prefill and decode throughput of the Nusuvik decoder "
                    "(latent attention over a cache of latent rows, one layer norm per parallel block, dense and grouped-sigmoid expert "
                    "feed-forwards, loop input projection; random weights) at layer sizes of real models, beside the Rizurax hybrid decoder at "
                    "equal size; prints one JSON line")
    ap.add_argument("--zuzezen", action="store_true", help="instead of the default workload: prefill and decode throughput of the Zuzezen decoder "
                    "(post-norm blocks, gated linear attention, windowed attention with tied values and a distance bias, latent attention with a "
                    "sink; random weights) at layer sizes of real models, beside the Rizurax hybrid decoder at equal size and its like kernels "
                    "in the other designs; prints one JSON line")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------------------
# shared by all arms: the workload description (identical `config` on every arm) and the algorithmic bytes
# ------------------------------------------------------------------------------------------------------------
def model_cfg(name):
    from qserve_b200.modelcfg import MODELS  # pure Python: does not load the CUDA library

    return MODELS[name]


def weight_bytes(cfg, precision, tp=1):
    D, H, I = cfg.head_dim, cfg.hidden, cfg.intermediate
    per = 1.0 if precision.startswith("w8a8") else 0.5
    q, kv = cfg.heads * D // tp, max(1, cfg.kv_heads // tp) * D
    elems = (q + 2 * kv) * H + H * q + 2 * (I // tp) * H + H * (I // tp)
    return int(elems * per)


def kv_bytes_per_layer(cfg, precision, batch, ctx, tp=1):
    """codes + scale/zero of K and V for ctx tokens + q in / o out (unique bytes)."""
    bits = 4 if "kv4" in precision else 8
    D, Hkv, Hq = cfg.head_dim, max(1, cfg.kv_heads // tp), cfg.heads // tp
    return batch * Hkv * ctx * D * bits // 8 * 2 + batch * Hkv * ctx * 8 + 4 * batch * Hq * D


def step_bytes(cfg, precision, batch, ctx, layers=None, tp=1):
    L = layers if layers is not None else cfg.layers
    return L * (weight_bytes(cfg, precision, tp) + kv_bytes_per_layer(cfg, precision, batch, ctx, tp)) + 2 * cfg.vocab * cfg.hidden


def make_config(args, world):
    cfg = model_cfg(args.model)
    L = cfg.layers if args.layers is None else args.layers
    sb = step_bytes(cfg, args.precision, args.batch, args.ctx, L)
    return {"workload": f"{cfg.name} {args.precision} decode batch={args.batch} ctx={args.ctx} ({L} layers + final norm + fp16 lm_head + greedy sampling)",
            "precision": args.precision, "batch": args.batch, "ctx": args.ctx, "layers": L, "parallelism": f"dp{world}",
            "l2": f"per-step working set {sb / 1e9:.2f} GB (weights + KV pages + lm_head) >> 126 MB L2: inputs larger than L2, no flush needed"}


def metric_name(args):
    cfg = model_cfg(args.model)
    return METRIC if (args.model, args.precision, args.batch) == ("llama-3-8b", "w4a8kv4", 64) else f"tokens/s {cfg.name} {args.precision} decode b{args.batch}"


# ------------------------------------------------------------------------------------------------------------
# clocks during the timed region (B200_PROFILING.md: clocks line)
# ------------------------------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index: int):
        self.samples, self.reasons, self._stop = [], set(), threading.Event()
        self.max_mhz = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nv:
            self.t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self.nv:
            self.t.join(timeout=1)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def ncu_traffic(kernel: str):
    """dram bytes per launch of `kernel` from the newest committed ncu capture summary (profiles/rNN_ncu_traffic.json)."""
    import glob
    files = sorted(glob.glob(os.path.join(ROOT, "profiles", "r*_ncu_traffic.json")))
    if not files:
        return None
    d = json.load(open(files[-1])).get(kernel)
    return None if not d else int(d["dram_bytes_read"]) + int(d["dram_bytes_write"])


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (B200_PROFILING.md)"


# ------------------------------------------------------------------------------------------------------------
# arm: --impl reference  (CPU port of the reference path on the host cores; every step = one bounded sample)
# ------------------------------------------------------------------------------------------------------------
def reference_arm(args, rank: int):
    """The reference's CPU path on the host cores (kind = "port": the reference has no CPU code of its own).
    A step is a BOUNDED SAMPLE of the workload: one of the model's decoder layers (4 W4A8 GEMMs at M = batch: unpack + dequant +
    fp32 matmul; KV4 attention: dequant + fp32 SDPA) on inputs prepared once; the fp16 lm_head is timed once before the steps.
    tokens/s = batch / (layers x mean layer time + lm_head time).  Exactly --steps steps are timed after --warmup warm-up steps."""
    if rank != 0:
        return
    from oracle import cpu_baseline as cb  # the ONLY place besides tests/ and smoke() that executes oracle/ code

    cfg = model_cfg(args.model)
    threads = os.cpu_count() or 1
    sample = cb.LayerSample(cfg.hidden, cfg.intermediate, cfg.heads, cfg.kv_heads, args.batch, args.ctx, threads)
    t_lm = cb.lm_head_sample(cfg.hidden, cfg.vocab, args.batch, threads)
    for _ in range(args.warmup):
        sample.run()
    t0 = time.perf_counter()
    runs = [sample.run() for _ in range(args.steps)]
    wall = time.perf_counter() - t0
    layer_s = sum(r["layer_s"] for r in runs) / len(runs)
    mean = lambda k: sum(r[k] for r in runs) / len(runs)
    L = cfg.layers if args.layers is None else args.layers
    v = args.batch / (L * layer_s + t_lm)
    desc = (f"{args.steps} timed step(s) after {args.warmup} warm-up; each step = 1 of {L} decoder layers of the workload (4 W4A8 GEMMs at M={args.batch}: "
            f"unpack+dequant+fp32 matmul; KV4 attention B={args.batch} ctx={args.ctx}: dequant+fp32 SDPA) on inputs prepared once; fp16 lm_head timed once "
            f"({t_lm:.2f} s); tokens/s = batch / ({L} x {layer_s:.2f} s + lm_head)")
    line = {
        "impl": "reference", "metric": metric_name(args), "value": v, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * wall / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
        "config": make_config(args, args.gpus),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc, "layer_s": layer_s, "lm_head_s": t_lm,
                         "dequant_s": mean("dequant_s"), "matmul_s": mean("matmul_s"), "attention_s": mean("attention_s"),
                         "full_step_s_extrapolated": L * layer_s + t_lm},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------
# per-kernel timing (ours and the reference kernels go through the SAME function: only the OpSet differs)
# ------------------------------------------------------------------------------------------------------------
def time_kernel(fn, reps: int, stream, graph: bool = True):
    """Seconds per launch of the launches `fn()` issues (it returns their number).  graph=True: the launches are captured ONCE into a
    CUDA graph and the graph is replayed -- the host (ctypes marshalling, ~5-8 us per call, more than the short kernels themselves) is out of
    the timed region and the number is the device-side cost of a launch in a dependent chain, as in the captured decode step.
    graph=False (the reference extensions: their GEMMs launch on the legacy default stream and cannot be captured): eager back-to-back."""
    import torch

    fn()  # warm (attributes, workspaces)
    torch.cuda.synchronize()
    g = None
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            n_per = fn()
        run = g.replay
        run()
    else:
        n_per = None
        run = fn
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    n = 0
    for _ in range(reps):
        r = run()
        n += n_per if graph else r
    e1.record(stream)
    torch.cuda.synchronize()
    del g
    return e0.elapsed_time(e1) * 1e-3 / n  # seconds per launch


def kernel_table(run, reps, hbm_gbs, prefill: bool = True, fused_ops: bool = True, graph: bool = True):
    """Per-kernel launch duration and achieved HBM bandwidth, timed live with CUDA events on the launching stream (graph replay of the
    launch loop: see time_kernel).  Each timed
    loop walks the weights / KV pages of ALL layers (3.5 GB / 2.4 GB >> 126 MB L2), so every launch streams from HBM.
    `run.ops` decides whose kernels run (this library or the reference's)."""
    import torch

    stream = torch.cuda.current_stream()
    M, cfg, ops, L = run.batch, run.cfg, run.ops, run.L
    H, D = cfg.hidden, cfg.head_dim
    out = {}

    def gemm_bytes(lin):  # M*K + N*K/2 + 2*M*N + scales
        return M * lin.K + lin.weight_bytes() + 2 * M * lin.N + 4 * lin.N + 4 * M

    for name, xq, buf in (("qkv", run.q_hidden, run.qkv_buf), ("o", run.q_attn, run.out_buf), ("gate_up", run.q_hidden, run.gate_up_buf),
                          ("down", run.q_mlp, run.out_buf)):
        def fn(name=name, xq=xq, buf=buf):
            for ly in run.layers:
                ly[name](xq, run.q_scale, run.q_sum, buf)
            return len(run.layers)
        t = time_kernel(fn, reps, stream, graph)
        lin = run.layers[0][name]
        b = gemm_bytes(lin)
        out[f"gemm_{name}"] = {"M": M, "N": lin.N, "K": lin.K, "us": t * 1e6, "bytes": b, "GBps": b / t / 1e9, "frac": b / t / 1e9 / hbm_gbs,
                               "int8_TOPS": 2.0 * M * lin.N * lin.K / t / 1e12, "launches_per_step": L}

    q, k, v = run.qkv_buf.split([run.q_size, run.kv_size, run.kv_size], dim=-1)
    q, k, v = q.reshape(M, run.Hq, D), k.reshape(M, run.Hkv, D), v.reshape(M, run.Hkv, D)

    def attn():
        for li in range(L):
            ops.fused_attention.single_query_attention(q, k, v, run.block_tables[li], run.context_lens, None, min(8192, cfg.max_pos), 64, run.size_per_token,
                                                       run.max_seq_len, D, cfg.rope_theta, True, run.kv_bits == 4, True)
        return L
    t = time_kernel(attn, reps, stream, graph)
    b = run.kv_bytes_per_step() // L
    out["attention"] = {"B": M, "Hq": run.Hq, "Hkv": run.Hkv, "ctx": run.ctx, "us": t * 1e6, "bytes": b, "GBps": b / t / 1e9, "frac": b / t / 1e9 / hbm_gbs,
                        "launches_per_step": L}

    # the small ops of the reference sequence (latency-bound at M = 64; bytes = what they read + write)
    x = torch.randn((M, H), device=run.dev).half()
    gu = run.gate_up_buf
    attn_out = torch.randn((M, run.q_size), device=run.dev).half()
    nrep = 64

    def small(name, fn, nbytes, per_step):
        def loop():
            for _ in range(nrep):
                fn()
            return nrep
        t = time_kernel(loop, max(1, reps // 2), stream, graph)
        out[name] = {"us": t * 1e6, "bytes": nbytes, "GBps": nbytes / t / 1e9, "frac": nbytes / t / 1e9 / hbm_gbs, "launches_per_step": per_step}

    gam = run.layers[0]["ln1"]
    if run.act_sum:
        small("norm_quant", lambda: ops.layernorm_ops.rms_norm_general_fuse_sum(run.q_hidden, x, gam, run.q_sum, run.q_scale, cfg.eps, True), 3 * M * H, 2 * L)
        small("quant_attn_out", lambda: ops.fused_kernels.invoke_quant_fuse_sum(run.q_attn, attn_out, run.q_sum, run.q_scale), 3 * M * run.q_size, L)
        small("quant_mlp", lambda: ops.fused_kernels.invoke_quant_fuse_sum(run.q_mlp, run.mlp_act, run.q_sum, run.q_scale), 3 * M * run.Iloc, L)
    else:
        small("norm_quant", lambda: ops.layernorm_ops.rms_norm_general(run.q_hidden, x, gam, run.q_scale, cfg.eps, True), 3 * M * H, 2 * L)
        small("quant_attn_out", lambda: ops.fused_kernels.invoke_quant(run.q_attn, attn_out, run.q_scale), 3 * M * run.q_size, L)
        small("quant_mlp", lambda: ops.fused_kernels.invoke_quant(run.q_mlp, run.mlp_act, run.q_scale), 3 * M * run.Iloc, L)
    small("silu_and_mul", lambda: ops.activation_ops.silu_and_mul(run.mlp_act, gu), 6 * M * run.Iloc, L)
    if fused_ops:
        from qserve_b200 import backend as ext
        qsum = run.q_sum if run.act_sum else None
        nxt = torch.empty_like(x)
        small("add_norm_quant(fused)", lambda: ext.add_rms_norm_general(run.q_hidden, nxt, x, run.out_buf, gam, qsum, run.q_scale, cfg.eps), 7 * M * H, 2 * L)
        small("silu_mul_quant(fused)", lambda: ext.silu_and_mul_quant(run.q_mlp, gu, qsum, run.q_scale), 5 * M * run.Iloc, L)

        def attn_q():
            for li in range(L):
                ext.single_query_attention_quant(q, k, v, run.block_tables[li], run.context_lens, min(8192, cfg.max_pos), 64, run.size_per_token, run.max_seq_len,
                                                 D, cfg.rope_theta, run.kv_bits == 4, True, run.q_attn, run.q_scale, qsum)
            return L
        t = time_kernel(attn_q, reps, stream, graph)
        out["attention_quant(fused)"] = {"us": t * 1e6, "bytes": b, "GBps": b / t / 1e9, "frac": b / t / 1e9 / hbm_gbs, "launches_per_step": L}

    if prefill:
        # prefill-sized GEMM (tensor-pipe bound, SURVEY.md 8d "GEMM INT8-TC util"): 4096 tokens through gate_up_proj
        Mp = 4096
        lin = run.layers[0]["gate_up"]
        xq = torch.randint(-127, 128, (Mp, lin.K), dtype=torch.int8, device=run.dev)
        sc = torch.full((Mp,), 0.01, dtype=torch.half, device=run.dev)
        sm = torch.zeros((Mp,), dtype=torch.half, device=run.dev)
        big = torch.empty((Mp, lin.N), dtype=torch.half, device=run.dev)

        def pf():
            for ly in run.layers[:4]:
                ly["gate_up"](xq, sc, sm, big)
            return min(4, len(run.layers))
        t = time_kernel(pf, max(2, reps // 2), stream, graph)
        opsn = 2.0 * Mp * lin.N * lin.K
        out["gemm_prefill_gate_up"] = {"M": Mp, "N": lin.N, "K": lin.K, "us": t * 1e6, "int8_TOPS": opsn / t / 1e12,
                                       "frac_of_nominal_int8_dense": opsn / t / 1e12 / 4500.0, "frac_of_measured_umma_i8_peak": opsn / t / 1e12 / 4760.0,
                                       "bound": "tensor (INT8 dense: nominal 4.5 POP/s; measured tcgen05 kind::i8 issue peak 4.76 POP/s, tools/ubench/umma.cu)"}
        del big
        if fused_ops:  # (this repo's table only: the reference-gpu arm reuses kernel_table for the reference extensions)
            # prompt-phase attention: BASELINE config 3's prompt batch, 8 x ctx tokens, causal; flash-attn (the third-party
            # kernel the reference calls, a library) is timed beside it when the image has it
            from qserve_b200 import backend as _be
            cfg = run.cfg
            n_p, plen = 8, run.ctx
            qkv = torch.randn(n_p * plen, (cfg.heads + 2 * cfg.kv_heads) * 128, device=run.dev).half()
            q, k, v = qkv.split([cfg.heads * 128, cfg.kv_heads * 128, cfg.kv_heads * 128], dim=-1)
            q, k, v = q.reshape(-1, cfg.heads, 128), k.reshape(-1, cfg.kv_heads, 128), v.reshape(-1, cfg.kv_heads, 128)
            cu = torch.arange(0, (n_p + 1) * plen, plen, dtype=torch.int32, device=run.dev)
            flops = n_p * 4.0 * 128 * cfg.heads * plen * (plen + 1) / 2
            impls = {"qserve_b200": _be.flash_attn_varlen_func}
            try:
                from flash_attn import flash_attn_varlen_func as _fa
                impls["flash_attn"] = _fa
            except Exception:  # noqa: BLE001
                pass
            rec = {"prompts": n_p, "prompt_len": plen, "heads": cfg.heads, "kv_heads": cfg.kv_heads, "causal_flops": flops,
                   "bound": "tensor (fp16 dense: nominal 2.25 PFLOP/s)"}
            for name, fn in impls.items():
                def pa(fn=fn):
                    fn(q, k, v, cu, cu, plen, plen, dropout_p=0.0, causal=True)
                    return 1
                t = time_kernel(pa, max(2, reps // 2), stream, graph)
                rec[f"us_{name}" if name != "qserve_b200" else "us"] = t * 1e6
                rec[f"TFLOPS_{name}" if name != "qserve_b200" else "TFLOPS"] = flops / t / 1e12
            rec["frac_of_nominal_fp16_dense"] = rec["TFLOPS"] / 2250.0
            out["prefill_attention"] = rec
    return out


def roofline_from(kern, hbm_gbs, peak_src, fused: bool):
    """The dominant kernel FUNCTION of the step by measured time share: launches per step x isolated launch duration, with all
    launch shapes of one template instantiation aggregated (the four M = 64 GEMM shapes are ONE instantiation of gemm_kernel)."""
    gemm_keys = [k for k in ("gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down") if k in kern]
    attn_key = "attention_quant(fused)" if fused and "attention_quant(fused)" in kern else "attention"
    groups = {"gemm_kernel (W4A8/W8A8 tcgen05 GEMM, all four decode shapes: one template instantiation)": gemm_keys,
              "decode_attention_kernel (KV4/KV8 paged single-query attention)": [attn_key]}
    small = [k for k in (("add_norm_quant(fused)", "silu_mul_quant(fused)") if fused else ("norm_quant", "quant_attn_out", "quant_mlp", "silu_and_mul")) if k in kern]
    step_us = sum(kern[k]["us"] * kern[k]["launches_per_step"] for ks in groups.values() for k in ks) + sum(kern[k]["us"] * kern[k]["launches_per_step"] for k in small)
    best, share = None, {}
    for name, ks in groups.items():
        t = sum(kern[k]["us"] * kern[k]["launches_per_step"] for k in ks)
        share[name] = t / step_us
        if best is None or t > best[1]:
            best = (name, t, ks)
    name, t_us, ks = best
    launches = sum(kern[k]["launches_per_step"] for k in ks)
    bytes_step = sum(kern[k]["bytes"] * kern[k]["launches_per_step"] for k in ks)
    achieved = bytes_step / (t_us * 1e-6) / 1e9
    traffic = None
    parts = [ncu_traffic(k if k != "attention_quant(fused)" else "attention") for k in ks]
    if all(p is not None for p in parts):
        traffic = sum(p * kern[k]["launches_per_step"] for p, k in zip(parts, ks)) / launches
    return {"bound": "hbm", "kernel": name, "selection": "largest share of the step's kernel time (launches per step x measured launch duration)",
            "time_share_of_step_kernels": share[name], "time_shares": share,
            "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs, "peak_source": peak_src,
            "algorithmic_bytes": bytes_step / launches, "us_per_launch": t_us / launches, "launches_per_step": launches,
            "traffic": traffic, "traffic_unit": "dram bytes per launch, averaged over the launch shapes (ncu --set full)",
            "by_launch_shape": {k: {"us": kern[k]["us"], "frac": kern[k]["frac"], "bytes": kern[k]["bytes"]} for k in ks}}


# ------------------------------------------------------------------------------------------------------------
# arm: --impl reference-gpu  (the reference's own CUDA kernels on this B200: the "legacy mma.sync on B200" row)
# ------------------------------------------------------------------------------------------------------------
def reference_gpu_arm(args):
    import torch

    from oracle import refmods  # the reference itself (compiled unmodified by oracle/build_ref.py); this arm exists to time it
    from qserve_b200.decode import DecodeRunner, OpSet

    names = {"layernorm_ops": "layernorm_ops", "fused_kernels": "fused_kernels", "activation_ops": "activation_ops", "fused_attention": "fused_attention",
             "qgemm_chn": "qgemm_w4a8_per_chn", "qgemm_grp": "qgemm_w4a8_per_group", "qgemm_w8": "qgemm_w8a8"}
    mods = {k: refmods.load(v) for k, v in names.items()}
    missing = [names[k] for k, m in mods.items() if m is None]
    if missing:
        print(json.dumps({"impl": "reference-gpu", "unavailable": f"oracle/_ref lacks {missing} (oracle/build_ref.py needs /root/reference)"}), flush=True)
        return
    assert torch.cuda.is_available()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = model_cfg(args.model)
    run = DecodeRunner(args.model, args.precision, args.batch, args.ctx, dev, layers=args.layers, fused=False, ops=OpSet(**mods))
    hbm_gbs, _ = peaks()
    stream = torch.cuda.current_stream()  # the reference GEMMs launch on the legacy default stream (gemm_cuda.cu:53): stay on it
    tok = torch.randint(0, cfg.vocab, (args.batch,), device=dev)
    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            run.tokens_out.copy_(run.forward(tok))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(args.steps):
            run.tokens_out.copy_(run.forward(tok))
        e1.record(stream)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        ms = e0.elapsed_time(e1) / args.steps
        kern = kernel_table(run, args.kernel_reps, hbm_gbs, prefill=True, fused_ops=False, graph=False)
    seq = ("gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down", "attention", "norm_quant", "quant_attn_out", "quant_mlp", "silu_and_mul")
    kern_ms = sum(kern[k]["us"] * kern[k]["launches_per_step"] for k in seq) * 1e-3
    line = {"impl": "reference-gpu", "metric": metric_name(args), "value": args.batch / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
            "config": make_config(args, 1),
            "what": "the reference's UNMODIFIED CUDA kernels (kernels/csrc/**, legacy mma.sync / CUDA-core attention) compiled for sm_100a by oracle/build_ref.py, driven "
                    "through the reference op sequence of LlamaDecoderLayer.forward on the same buffers; eager launches (the reference GEMMs use the legacy "
                    "default stream and cannot be graph-captured), so `value` includes host launch overhead; `kernel_ms_per_step` is the GPU-time-only lower bound",
            "host_ms_per_step": 1000.0 * wall / args.steps,
            "kernel_ms_per_step": kern_ms, "tokens_per_s_kernel_time_only": args.batch / (kern_ms * 1e-3 + 0.25e-3),
            "kernels": kern, "gpu_launches": run.launches_per_step * args.steps}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------
# block: the reference's unmodified Python model code over this backend (eager / graph decode, config-3 prefill + decode)
# ------------------------------------------------------------------------------------------------------------
def refmodel_block(run, args, steps: int):
    import torch

    from qserve_b200 import refmodel
    from qserve_b200.decode import DecodeRunner

    if refmodel.locate_reference() is None:
        return {"unavailable": "reference Python package not found (baseline/_ref is installed by __graft_entry__.build() where /root/reference exists)"}
    out = {"what": "qserve.modeling.models.llama_w4a8_unpad.LlamaForCausalLM (the reference's own layer / model classes, unmodified, from baseline/_ref) with "
                   "qserve_backend = this repo; synthetic weights shared with the DecodeRunner"}
    stream = torch.cuda.current_stream()

    def timed(fn, n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n, 1000.0 * (time.perf_counter() - t0) / n

    def decode_numbers(ref, r, tag):
        tok = torch.randint(0, r.cfg.vocab, (r.batch,), device=r.dev)
        for _ in range(3):
            ref.decode_tokens(tok)
        ms, host_ms = timed(lambda: ref.decode_tokens(tok), steps)
        out[f"{tag}_eager"] = {"tokens_per_s": r.batch / (ms * 1e-3), "ms_per_step": ms, "host_ms_per_step": host_ms,
                               "note": "eager Python loop of the reference model: what a drop-in user of qserve_benchmark.py gets"}
        # the same unmodified forward captured in a CUDA graph (the ops are stream-ordered and allocation-free apart from torch's own)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            ref.decode_tokens(tok)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            ref.decode_tokens(tok)
        for _ in range(3):
            g.replay()
        ms, _ = timed(g.replay, steps)
        out[f"{tag}_graph"] = {"tokens_per_s": r.batch / (ms * 1e-3), "ms_per_step": ms}
        del g

    ref = refmodel.RefModel(run)
    decode_numbers(ref, run, "decode")
    del ref
    # BASELINE config 3: Llama-3-8B g128, a prompt step (in-place RoPE + KV4 quant/append + flash_attn_varlen_func inside the reference
    # layer code, llama_w4a8_unpad.py:203-242) followed by decode steps over the pages it wrote
    try:
        r3 = DecodeRunner(args.model, "w4a8kv4-g128", args.batch, args.ctx, run.dev, layers=args.layers, fused=False, seed=3)
        ref3 = refmodel.RefModel(r3)
        n_prompts, plen = 8, args.ctx
        lens = [plen] * n_prompts
        toks = torch.randint(0, r3.cfg.vocab, (n_prompts * plen,), device=r3.dev)
        meta = ref3.prefill_metadata(lens)
        per_impl = {}
        for impl in ("flash_attn", "qserve_b200"):  # the prompt attention behind the reference layer's flash_attn_varlen_func call
            ref3.use_prefill_attention(impl)
            for _ in range(2):
                ref3.prefill_logits(toks, lens, meta)
            per_impl[impl] = timed(lambda: ref3.prefill_logits(toks, lens, meta), 3)
        ms, host_ms = per_impl["qserve_b200"]
        out["config3_prefill"] = {"prompts": n_prompts, "prompt_len": plen, "tokens": n_prompts * plen, "ms_per_step": ms, "host_ms_per_step": host_ms,
                                  "tokens_per_s": n_prompts * plen / (ms * 1e-3), "int8_TOPS_gemm_only": 2.0 * n_prompts * plen * weight_bytes(r3.cfg, "w4a8", 1) * 2 * r3.L / (ms * 1e-3) / 1e12,
                                  "prompt_attention": "qserve_b200 tcgen05 kernel (qs_prefill_attention)",
                                  "ms_per_step_with_flash_attn": per_impl["flash_attn"][0],
                                  "tokens_per_s_with_flash_attn": n_prompts * plen / (per_impl["flash_attn"][0] * 1e-3)}
        decode_numbers(ref3, r3, "config3_decode")
        pf, dg = out["config3_prefill"], out["config3_decode_graph"]
        # in-flight batching round: one prompt step admits 8 sequences, then the batch decodes until they finish 512 tokens (qserve_benchmark protocol 1024 in / 512 out)
        out["config3_ifb_round"] = {"what": f"1 prompt step ({n_prompts} x {plen} tokens) + {args.batch // n_prompts} decode steps at batch {args.batch} per admitted group, "
                                            "steady state of 1024-in/512-out in-flight batching: generated tokens/s",
                                    "tokens_per_s": (n_prompts * 512) / ((pf["ms_per_step"] + 512 * dg["ms_per_step"] * n_prompts / args.batch) * 1e-3)}
        del ref3, r3
    except Exception as e:  # noqa: BLE001
        out["config3_error"] = repr(e)
    return out


# ------------------------------------------------------------------------------------------------------------
# block: BASELINE config 5 -- Qwen1.5-72B W4A8KV4, all 80 layers, tensor parallel over the N GPUs of the run (TP = 1 at N = 1)
# ------------------------------------------------------------------------------------------------------------
def tp_block(args, rank, world, dev, hbm_gbs):
    import torch
    import torch.distributed as dist

    from qserve_b200.decode import DecodeRunner

    cfg = model_cfg(args.tp_model)
    want_peer = args.tp_allreduce == "peer" and world > 1 and not args.tp_exact
    peer_err = None
    if want_peer:
        # symmetric memory needs CUDA VMM handle exchange between the ranks: agree on success before building the model on it
        ok = torch.ones(1, device=dev)
        try:
            from qserve_b200 import backend as _b
            probe = _b.PeerContext(8, 128, dev, dist.group.WORLD)
            del probe
        except Exception as e:  # noqa: BLE001
            ok.zero_()
            peer_err = repr(e)[:300]
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        want_peer = bool(ok.item() > 0)
    run = DecodeRunner(args.tp_model, "w4a8kv4", args.batch, args.ctx, dev, tp_rank=rank, tp_size=world, seed=rank, layers=args.tp_layers,
                       fused=True, tp_exact=args.tp_exact, tp_peer=want_peer)
    run.capture()
    step_fn = run.step
    stream = torch.cuda.current_stream()
    steps = max(5, min(args.steps, 20))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(3):
        step_fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step_fn()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1) / steps
    ar_us = None
    if world > 1:
        buf = torch.zeros((args.batch, cfg.hidden), dtype=torch.half, device=dev)
        for _ in range(5):
            dist.all_reduce(buf)
        barrier()
        e0.record(stream)
        for _ in range(200):
            dist.all_reduce(buf)
        e1.record(stream)
        barrier()
        ar_us = e0.elapsed_time(e1) * 1e3 / 200
        t = torch.tensor([ms, ar_us], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ar_us = t.tolist()
    L = run.L
    sb = step_bytes(cfg, "w4a8kv4", args.batch, args.ctx, L, world)
    rec = {"model": cfg.name, "precision": "w4a8kv4", "batch": args.batch, "ctx": args.ctx, "layers": L, "tp": world, "steps": steps,
           "quant_mode": "exact (global per-token amax, SURVEY 8e parity rule)" if args.tp_exact else "throughput (per-rank local amax)",
           "tokens_per_s": args.batch / (ms * 1e-3), "ms_per_step": ms, "per_rank_hbm_bytes_per_step": sb,
           "per_rank_hbm_frac": sb / (ms * 1e-3) / 1e9 / hbm_gbs,
           "allreduce": None if world == 1 else {"calls_per_step": 2 * L, "message_bytes": args.batch * cfg.hidden * 2, "us_per_call_isolated": ar_us,
                                                 "ms_per_step_isolated": 2 * L * ar_us * 1e-3,
                                                 "nvlink_bytes_algorithmic_per_step": 2 * L * args.batch * cfg.hidden * 2 * 2 * (world - 1) // world,
                                                 "us_per_call_isolated_is": "NCCL all-reduce of the same message, back to back, for reference",
                                                 "backend": ("fused into add+norm+quant: flag exchange + 128-bit peer loads over NVLink symmetric memory (qs_add_rms_norm_general_peer), no NCCL on the data path"
                                                             if run.tp_peer else "NCCL all-reduce inside the captured CUDA graph")},
           "peer_fallback_reason": peer_err,
           "note": "efficiency vs TP=1 = this tokens_per_s / (N x the tp=1 record of the --gpus 1 line); 36 GB of W4 weights fit one GPU, TP is for throughput"}
    run.graph = None
    del run
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------------------------------------------------
# --hybrid: the unquantised hybrid decoder (differential attention + gated delta rule) beside the closest existing model
# ------------------------------------------------------------------------------------------------------------
HYBRID_SIZES = {  # name: width, heads, kv heads, head size (per map / value), feed-forward, vocab
    "w2048": (2048, 16, 4, 128, 8192, 32000),
    "w4096": (4096, 32, 8, 128, 14336, 32000),
}


def hybrid_block(args):
    """Prefill (4 prompts x 2048 tokens in one step) and decode (64 sequences at 1024 tokens of context) of a four-layer stack attention |
    delta | attention | delta with a feed-forward in every layer, captured in CUDA graphs (device time of the step, host excluded), and the
    kernels of the design timed one by one with their algorithmic bytes / flops against the measured copy and bf16 GEMM peaks.  Beside it,
    at equal width / heads / feed-forward: the Llama-style W4A8KV4 decode step and the kernels that play the same parts there."""
    import torch

    from qserve_b200 import backend
    from qserve_b200._lib import check, lib
    from qserve_b200.decode import MODELS, DecodeRunner
    from qserve_b200.engine import Engine
    from qserve_b200.hybrid import HybridDecoder, StepBatch, random_weights
    from qserve_b200.modelcfg import AttentionMixerConfig, DeltaMixerConfig, HybridConfig, HybridLayerConfig, MlpConfig, ModelConfig, RotaryConfig

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm_gbs, peak_src = peaks()[0], peaks()[1] if len(peaks()) > 1 else "measured"
    try:
        tflops = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    except (OSError, KeyError, ValueError):
        tflops = 1590.0
    stream = torch.cuda.current_stream()
    reps = max(3, args.kernel_reps)
    B, CTX, NP, LP = 64, 1024, 4, 2048
    out = {"metric": "hybrid decoder throughput (tokens/s, random weights, bf16, 4 layers)", "unit": "tokens/s", "impl": "ours", "dtype": "bf16",
           "data": "synthetic", "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": tflops}, "sizes": {}}
    for name, (W, H, G, D, FF, V) in HYBRID_SIZES.items():
        att = AttentionMixerConfig(H, G, D, D, RotaryConfig(D // 2, 1e6, 4.0, 4096, 32.0, 1.0), D ** -0.5, maps=2, diff=0.5, head_norm=True)
        dlt = DeltaMixerConfig(H, G, D, D, 4)
        cfg = HybridConfig("Rizurax", V, W, 1e-5, tuple(HybridLayerConfig(t, m, MlpConfig("dense", FF)) for t, m in
                                                       (("attention", att), ("delta", dlt), ("attention", att), ("delta", dlt))),
                           pair_buckets=4093, pair_mul_prev=131, pair_mul_cur=11)
        model = HybridDecoder(cfg, random_weights(cfg, 0, dev), torch.bfloat16, dev)
        eng = Engine(model, max_tokens=B * (CTX + 64), max_seqs=B)
        g = torch.Generator().manual_seed(0)
        rec = {}
        with torch.no_grad():
            # ---- prefill: NP prompts of LP tokens in one step
            prompts = [torch.randint(0, V, (LP,), generator=g).tolist() for _ in range(NP)]
            for i, p in enumerate(prompts):
                eng.cache.admit(("p", i)); eng.cache.reserve(("p", i), LP)
            rows = [(eng.cache.seqs[("p", i)].slot, 0, -1, p) for i, p in enumerate(prompts)]
            pb = StepBatch.build(rows, eng.cache.sync_block_table(), dev)
            t = time_kernel(lambda: (model.forward(pb, eng.cache), 1)[1], reps, stream)
            rec["prefill"] = {"tokens": NP * LP, "ms": t * 1e3, "tokens_per_s": NP * LP / t}
            kern = {}
            ly_a, ly_d = model.layers[0], model.layers[1]
            T = NP * LP
            proj_a = torch.randn(T, ly_a.mixer.in_features, device=dev).to(torch.bfloat16)
            proj_d = torch.randn(T, ly_d.mixer.in_features, device=dev).to(torch.bfloat16)
            cat = torch.empty(T, H * D + FF, dtype=torch.bfloat16, device=dev)
            scratch = torch.empty(max(ly_d.mixer.scratch_floats(T), ly_a.mixer.scratch_floats(T)), dtype=torch.float32, device=dev)
            s = torch.cuda.current_stream().cuda_stream
            raw = lambda: torch._C._cuda_getCurrentRawStream(0)
            ta = time_kernel(lambda: (ly_a.mixer.run(proj_a, cat, pb, eng.cache.runs[0], 64, scratch, 0, raw()), 1)[1], reps, stream)
            flops = H * NP * (LP * (LP + 1) // 2) * (2 * 2 * D + 2 * 2 * D)
            kern["attention_prefill(rope+append+attention)"] = {"us": ta * 1e6, "tflops": flops / ta / 1e12, "frac_of_measured_bf16_peak": flops / ta / 1e12 / tflops}
            td = time_kernel(lambda: (ly_d.mixer.run(proj_d, cat, pb, eng.cache.runs[1], 64, scratch, 0, raw()), 1)[1], reps, stream)
            kern["delta_prefill(conv+scan+gate)"] = {"us": td * 1e6, "tokens_per_s": T / td}
            x = torch.randn(T, W, device=dev)
            h1, h2 = torch.empty(T, W, dtype=torch.bfloat16, device=dev), torch.empty(T, W, dtype=torch.bfloat16, device=dev)
            upd = torch.zeros(T, W, dtype=torch.bfloat16, device=dev)
            # as the engine runs it: the stream takes the previous layer's update (bf16 in, fp32 in and out) and leaves two normalised bf16 rows
            tn = time_kernel(lambda: (check(lib.qs_hyb_rms_norm(h1.data_ptr(), h2.data_ptr(), x.data_ptr(), upd.data_ptr(), ly_a.norm1.data_ptr(),
                                                                 ly_a.norm2.data_ptr(), 1.0, 1e-5, T, W, 0, raw())), 1)[1], reps, stream)
            kern["add_rms_norm_dual"] = {"us": tn * 1e6, "frac_of_measured_hbm": T * W * 14 / tn / 1e9 / hbm_gbs}
            del upd
            gu = torch.randn(T, 2 * FF, device=dev).to(torch.bfloat16)
            tg = time_kernel(lambda: (check(lib.qs_hyb_gelu_tanh_mul(cat.data_ptr(), cat.stride(0), gu.data_ptr(), T, FF, 0, raw())), 1)[1], reps, stream)
            kern["gelu_tanh_mul"] = {"us": tg * 1e6, "frac_of_measured_hbm": T * FF * 6 / tg / 1e9 / hbm_gbs}
            for i in range(NP):
                eng.release(("p", i))
            # ---- decode: B sequences with CTX tokens of context, one token each
            for i in range(B):
                eng.cache.admit(("d", i)); eng.cache.reserve(("d", i), CTX + 1)
            rows = [(eng.cache.seqs[("d", i)].slot, CTX, 5, [int(torch.randint(0, V, (1,), generator=g))]) for i in range(B)]
            db = StepBatch.build(rows, eng.cache.sync_block_table(), dev)
            t = time_kernel(lambda: (model.logits(model.forward(db, eng.cache)), 1)[1], reps * 4, stream)
            rec["decode"] = {"batch": B, "ctx": CTX, "ms": t * 1e3, "tokens_per_s": B / t}
            ta = time_kernel(lambda: (ly_a.mixer.run(proj_a[:B], cat[:B], db, eng.cache.runs[0], 64, scratch, 0, raw()), 1)[1], reps * 4, stream)
            kvb = B * (CTX + 1) * G * (2 * D + D) * 2
            kern["attention_decode(rope+append+attention)"] = {"us": ta * 1e6, "frac_of_measured_hbm": kvb / ta / 1e9 / hbm_gbs}
            td = time_kernel(lambda: (ly_d.mixer.run(proj_d[:B], cat[:B], db, eng.cache.runs[1], 64, scratch, 0, raw()), 1)[1], reps * 4, stream)
            kern["delta_decode(conv+scan+gate)"] = {"us": td * 1e6, "frac_of_measured_hbm": B * H * D * D * 8 / td / 1e9 / hbm_gbs}
            rec["kernels"] = kern
        del eng, model
        torch.cuda.empty_cache()
        # ---- the closest existing model at equal size: Llama-style W4A8KV4 (4 layers), decode step and its attention kernels
        key = "bench-" + name
        MODELS[key] = ModelConfig(key, W, FF, H, G, 4, V, 1e6, head_dim=D)
        with torch.no_grad():
            run = DecodeRunner(key, "w4a8kv4", B, CTX, dev)
            run.capture()
            t = time_kernel(lambda: (run.step(), 1)[1], reps * 4, stream, graph=False)
            peer = {"decode": {"batch": B, "ctx": CTX, "ms": t * 1e3, "tokens_per_s": B / t}}
            run.qkv_buf.normal_()
            ta = time_kernel(lambda: (run._attention(0), 1)[1], reps * 4, stream)
            peer["attention_decode_kv4"] = {"us": ta * 1e6, "frac_of_measured_hbm": run.kv_bytes_per_step() / run.L / ta / 1e9 / hbm_gbs}
            T = NP * LP
            xh, dl = torch.randn(T, W, device=dev).half(), torch.randn(T, W, device=dev).half()
            qo, ho = torch.empty(T, W, dtype=torch.int8, device=dev), torch.empty(T, W, dtype=torch.float16, device=dev)
            qs_, sc = torch.empty(T, dtype=torch.float16, device=dev), torch.empty(T, dtype=torch.float16, device=dev)
            gam = torch.ones(W, dtype=torch.float16, device=dev)
            tn = time_kernel(lambda: (backend.add_rms_norm_general(qo, ho, xh, dl, gam, qs_, sc, 1e-5), 1)[1], reps, stream)
            peer["add_rms_norm_quant"] = {"us": tn * 1e6, "frac_of_measured_hbm": T * W * 7 / tn / 1e9 / hbm_gbs}
            guh = torch.randn(T, 2 * FF, device=dev).half()
            qm = torch.empty(T, FF, dtype=torch.int8, device=dev)
            tg = time_kernel(lambda: (backend.silu_and_mul_quant(qm, guh, qs_, sc), 1)[1], reps, stream)
            peer["silu_and_mul_quant"] = {"us": tg * 1e6, "frac_of_measured_hbm": T * FF * 5 / tg / 1e9 / hbm_gbs}
            del xh, dl, qo, ho, guh, qm
            q = torch.randn(NP * LP, H, D, device=dev).half()
            k = torch.randn(NP * LP, G, D, device=dev).half()
            cu = torch.arange(0, NP * LP + 1, LP, dtype=torch.int32, device=dev)
            tp = time_kernel(lambda: (backend.flash_attn_varlen_func(q, k, k, cu, cu, LP, LP, 0.0, None, True), 1)[1], reps, stream)
            fl = H * NP * (LP * (LP + 1) // 2) * 4 * D
            peer["attention_prefill_fp16"] = {"us": tp * 1e6, "tflops": fl / tp / 1e12, "frac_of_measured_bf16_peak": fl / tp / 1e12 / tflops}
            del run
        torch.cuda.empty_cache()
        rec["llama_w4a8kv4_equal_size"] = peer
        out["sizes"][name] = rec
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------------------------
# --toderax: the Toderax decoder beside the closest existing model (the Rizurax hybrid decoder) at equal size
# ------------------------------------------------------------------------------------------------------------
def toderax_block(args):
    """Prefill (4 prompts x 2048 tokens in one step) and decode (64 sequences at 1024 tokens of context) of a four-layer stack
    gate recurrence | attention + retention | gate recurrence | attention + retention with a mixture of experts (32 experts, 8 per token, plus a
    shared expert; the experts a token runs hold as many weights as the other model's feed-forward) in every layer, on 2 residual streams.
    Whole steps are captured in CUDA graphs (device time, host excluded); the design's kernels are timed one by one with their algorithmic
    bytes / flops against the measured copy and bf16 GEMM peaks.  Beside it: the Rizurax stack (attention | delta | attention | delta, dense
    feed-forward) at equal width / heads / head size, and the kernels that play the same parts there."""
    import torch

    from qserve_b200._lib import check, lib
    from qserve_b200.engine import Engine
    from qserve_b200.hybrid import HybridDecoder, StepBatch, random_weights
    from qserve_b200.modelcfg import (AttentionMixerConfig, DeltaMixerConfig, GateRecurrenceMixerConfig, HybridConfig, HybridLayerConfig, MlpConfig,
                                      MoeConfig, ParallelMixerConfig, RetentionMixerConfig, RotaryConfig)

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm_gbs = peaks()[0]
    try:
        tflops = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    except (OSError, KeyError, ValueError):
        tflops = 1590.0
    stream = torch.cuda.current_stream()
    reps = max(3, args.kernel_reps)
    raw = lambda: torch._C._cuda_getCurrentRawStream(0)
    B, CTX, NP, LP, NS, NG, E, TOP = 64, 1024, 4, 2048, 2, 8, 32, 8
    out = {"metric": "Toderax decoder throughput (tokens/s, random weights, bf16, 4 layers)", "unit": "tokens/s", "impl": "ours", "dtype": "bf16",
           "data": "synthetic", "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": tflops}, "sizes": {}}

    def steps(model, eng, V, g):
        """Prefill and decode step times of a model; returns (record, prefill batch, decode batch)."""
        prompts = [torch.randint(0, V, (LP,), generator=g).tolist() for _ in range(NP)]
        for i, p_ in enumerate(prompts):
            eng.cache.admit(("p", i)); eng.cache.reserve(("p", i), LP)
        pb = StepBatch.build([(eng.cache.seqs[("p", i)].slot, 0, -1, p_) for i, p_ in enumerate(prompts)], eng.cache.sync_block_table(), dev)
        t = time_kernel(lambda: (model.forward(pb, eng.cache), 1)[1], reps, stream)
        rec = {"prefill": {"tokens": NP * LP, "ms": t * 1e3, "tokens_per_s": NP * LP / t}}
        for i in range(B):
            eng.cache.admit(("d", i)); eng.cache.reserve(("d", i), CTX + 1)
        db = StepBatch.build([(eng.cache.seqs[("d", i)].slot, CTX, 5, [int(torch.randint(0, V, (1,), generator=g))]) for i in range(B)],
                             eng.cache.sync_block_table(), dev)
        t = time_kernel(lambda: (model.logits(model.forward(db, eng.cache)), 1)[1], reps * 4, stream)
        rec["decode"] = {"batch": B, "ctx": CTX, "ms": t * 1e3, "tokens_per_s": B / t}
        return rec, pb, db

    def mixer_times(mixer, run_cache, pb, db, T):
        proj = torch.randn(T, mixer.in_features, device=dev).to(torch.bfloat16)
        cat = torch.empty(T, mixer.out_features, dtype=torch.bfloat16, device=dev)
        scratch = torch.empty(max(1, mixer.scratch_floats(T)), dtype=torch.float32, device=dev)
        tp = time_kernel(lambda: (mixer.run(proj, cat, pb, run_cache, 64, scratch, 0, raw()), 1)[1], reps, stream)
        td = time_kernel(lambda: (mixer.run(proj[:B], cat[:B], db, run_cache, 64, scratch, 0, raw()), 1)[1], reps * 4, stream)
        return tp, td

    for name, (W, H, G, D, FF, V) in HYBRID_SIZES.items():
        T = NP * LP
        chunk = LP  # a prompt is one chunk and a decoded token sees its whole context: the same score work as the other model's causal attention
        att = AttentionMixerConfig(H, G, D, D, None, D ** -0.5, bias=True, qk_norm=True, head_temp=True, sink=True, chunk=chunk)
        ret = RetentionMixerConfig(H // 2, D, D, RotaryConfig(D, 1e6, layout="half"), tuple(1.0 - 2.0 ** (-5 - 5 * i / (H // 2)) for i in range(H // 2)))
        par = ParallelMixerConfig(att, ret)
        gate = GateRecurrenceMixerConfig(H, D, D)
        moe = MoeConfig(E, TOP, FF // TOP, 7.0, FF // TOP, 7.0)
        cfg = HybridConfig("Toderax", V, W, 1e-5, tuple(HybridLayerConfig(t, m, moe) for t, m in
                                                       (("hgrn2", gate), ("parallel", par), ("hgrn2", gate), ("parallel", par))),
                           norm_offset=0.0, block="sequential", streams=NS, norm_groups=NG, embed_scale=4.0)
        g = torch.Generator().manual_seed(0)
        rec = {}
        with torch.no_grad():
            model = HybridDecoder(cfg, random_weights(cfg, 0, dev), torch.bfloat16, dev)
            eng = Engine(model, max_tokens=B * (CTX + 64) + NP * LP, max_seqs=B + NP)
            rec, pb, db = steps(model, eng, V, g)
            kern = {}
            ly_g, ly_p = model.layers[0], model.layers[1]
            tp, td = mixer_times(ly_p.mixer.left, eng.cache.runs[1]["left"], pb, db, T)
            flops = H * NP * (LP * (LP + 1) // 2) * 4 * D
            kern["attention_prefill(prepare+append+attention)"] = {"us": tp * 1e6, "tflops": flops / tp / 1e12, "frac_of_measured_bf16_peak": flops / tp / 1e12 / tflops}
            kern["attention_decode(prepare+append+attention)"] = {"us": td * 1e6, "frac_of_measured_hbm": B * (CTX + 1) * G * 2 * D * 2 / td / 1e9 / hbm_gbs}
            tp, td = mixer_times(ly_g.mixer, eng.cache.runs[0], pb, db, T)
            kern["gate_recurrence_prefill(prepare+scan+norm)"] = {"us": tp * 1e6, "tokens_per_s": T / tp, "heads": H}
            kern["gate_recurrence_decode(prepare+scan+norm)"] = {"us": td * 1e6, "frac_of_measured_hbm": B * H * D * D * 8 / td / 1e9 / hbm_gbs}
            tp, td = mixer_times(ly_p.mixer.right, eng.cache.runs[1]["right"], pb, db, T)
            kern["retention_prefill(rotate+scan+gate)"] = {"us": tp * 1e6, "tokens_per_s": T / tp, "heads": H // 2}
            kern["retention_decode(rotate+scan+gate)"] = {"us": td * 1e6, "frac_of_measured_hbm": B * (H // 2) * D * D * 8 / td / 1e9 / hbm_gbs}
            # the streams' kernel as the engine runs it: a pending bf16 write lands in the fp32 streams, one normalised bf16 row leaves
            x = torch.randn(T, NS, W, device=dev)
            h1, upd = torch.empty(T, W, dtype=torch.bfloat16, device=dev), torch.zeros(T, W, dtype=torch.bfloat16, device=dev)
            hc = ly_g.hc2
            tn = time_kernel(lambda: (check(lib.qs_hyb_stream_norm(h1.data_ptr(), None, x.data_ptr(), NS, upd.data_ptr(), 0, hc.mix.data_ptr(),
                                                                   hc.cout.data_ptr(), hc.cin.data_ptr(), ly_g.norm2.data_ptr(), NG, 0.0, 1e-5, T, W, 0,
                                                                   raw())), 1)[1], reps, stream)
            kern[f"stream_write_read_group_norm({NS} streams)"] = {"us": tn * 1e6, "frac_of_measured_hbm": T * W * (NS * 8 + 4) / tn / 1e9 / hbm_gbs}
            ya, yb, y32 = torch.randn(T, W, device=dev).bfloat16(), torch.randn(T, W, device=dev).bfloat16(), torch.empty(T, W, device=dev)
            tb = time_kernel(lambda: (check(lib.qs_hyb_branch_norm_mean(y32.data_ptr(), ya.data_ptr(), yb.data_ptr(), ly_p.mixer.gain_left.data_ptr(),
                                                                        ly_p.mixer.gain_right.data_ptr(), 0.5, 1e-5, T, W, 0, raw())), 1)[1], reps, stream)
            kern["branch_norm_mean"] = {"us": tb * 1e6, "frac_of_measured_hbm": T * W * 8 / tb / 1e9 / hbm_gbs}
            del x, upd, ya, yb, y32
            # the feed-forward: useful flops are those of the experts a token runs and the shared expert
            h = torch.randn(T, W, device=dev).to(torch.bfloat16)
            ffl = 2 * 3 * W * (TOP * moe.ff + moe.shared_ff)
            for label, hh, r_ in (("prefill", h, reps), ("decode", h[:B].contiguous(), reps * 4)):
                tm = time_kernel(lambda: (ly_g.ff.run(hh, 0, raw()), 1)[1], r_, stream)
                n = hh.shape[0]
                kern[f"moe_feed_forward_{label}(router+sort+gather+4 products+act+combine)"] = {
                    "us": tm * 1e6, "tflops": n * ffl / tm / 1e12, "frac_of_measured_bf16_peak": n * ffl / tm / 1e12 / tflops,
                    "weights_frac_of_measured_hbm": 3 * W * (min(E, n * TOP) * moe.ff + moe.shared_ff) * 2 / tm / 1e9 / hbm_gbs}
            route, ti, tw = torch.empty(T, E, device=dev), torch.empty(T, TOP, dtype=torch.int32, device=dev), torch.empty(T, TOP, device=dev)
            tr = time_kernel(lambda: (check(lib.qs_hyb_moe_router(route.data_ptr(), ti.data_ptr(), tw.data_ptr(), h.data_ptr(), ly_g.ff.w_router.data_ptr(),
                                                                  T, W, E, TOP, 0, None, 1, 1, 0, raw())), 1)[1], reps, stream)
            kern["moe_router"] = {"us": tr * 1e6, "frac_of_measured_hbm": T * W * 2 / tr / 1e9 / hbm_gbs}
            gu = torch.randn(T * TOP, 2 * moe.ff, device=dev).to(torch.bfloat16)
            act = torch.empty(T * TOP, moe.ff, dtype=torch.bfloat16, device=dev)
            ta = time_kernel(lambda: (check(lib.qs_hyb_moe_act(act.data_ptr(), gu.data_ptr(), None, T * TOP, 0, 0, 0.0, moe.ff, 7.0, 1.702, 1.0, 0, raw())), 1)[1],
                             reps, stream)
            kern["moe_clamped_activation"] = {"us": ta * 1e6, "frac_of_measured_hbm": T * TOP * moe.ff * 6 / ta / 1e9 / hbm_gbs}
            rec["kernels"] = kern
            del eng, model, h, gu, act
        torch.cuda.empty_cache()
        # ---- the closest existing model at equal size: Rizurax (differential attention | gated delta rule, dense feed-forward)
        ratt = AttentionMixerConfig(H, G, D, D, RotaryConfig(D // 2, 1e6, 4.0, 4096, 32.0, 1.0), D ** -0.5, maps=2, diff=0.5, head_norm=True)
        rdlt = DeltaMixerConfig(H, G, D, D, 4)
        rcfg = HybridConfig("Rizurax", V, W, 1e-5, tuple(HybridLayerConfig(t, m, MlpConfig("dense", FF)) for t, m in
                                                        (("attention", ratt), ("delta", rdlt), ("attention", ratt), ("delta", rdlt))),
                            pair_buckets=4093, pair_mul_prev=131, pair_mul_cur=11)
        with torch.no_grad():
            model = HybridDecoder(rcfg, random_weights(rcfg, 0, dev), torch.bfloat16, dev)
            eng = Engine(model, max_tokens=B * (CTX + 64) + NP * LP, max_seqs=B + NP)
            peer, pb, db = steps(model, eng, V, g)
            kern = {}
            tp, td = mixer_times(model.layers[0].mixer, eng.cache.runs[0], pb, db, T)
            flops = H * NP * (LP * (LP + 1) // 2) * 8 * D
            kern["attention_prefill(rope+append+attention, 2 maps)"] = {"us": tp * 1e6, "tflops": flops / tp / 1e12, "frac_of_measured_bf16_peak": flops / tp / 1e12 / tflops}
            kern["attention_decode(rope+append+attention, 2 maps)"] = {"us": td * 1e6, "frac_of_measured_hbm": B * (CTX + 1) * G * 3 * D * 2 / td / 1e9 / hbm_gbs}
            tp, td = mixer_times(model.layers[1].mixer, eng.cache.runs[1], pb, db, T)
            kern["delta_prefill(conv+scan+gate)"] = {"us": tp * 1e6, "tokens_per_s": T / tp, "heads": H}
            kern["delta_decode(conv+scan+gate)"] = {"us": td * 1e6, "frac_of_measured_hbm": B * H * D * D * 8 / td / 1e9 / hbm_gbs}
            ly = model.layers[0]
            x = torch.randn(T, W, device=dev)
            h1, h2 = torch.empty(T, W, dtype=torch.bfloat16, device=dev), torch.empty(T, W, dtype=torch.bfloat16, device=dev)
            upd = torch.zeros(T, W, dtype=torch.bfloat16, device=dev)
            tn = time_kernel(lambda: (check(lib.qs_hyb_rms_norm(h1.data_ptr(), h2.data_ptr(), x.data_ptr(), upd.data_ptr(), ly.norm1.data_ptr(),
                                                                 ly.norm2.data_ptr(), 1.0, 1e-5, T, W, 0, raw())), 1)[1], reps, stream)
            kern["add_rms_norm_dual"] = {"us": tn * 1e6, "frac_of_measured_hbm": T * W * 14 / tn / 1e9 / hbm_gbs}
            del x, upd
            # its feed-forward as the engine runs it: gate | up product, gelu-tanh gate, down product (here without the attention half of the row)
            w_dn = torch.randn(W, FF, device=dev).to(torch.bfloat16)
            for label, hh, r_ in (("prefill", h1, reps), ("decode", h1[:B].contiguous(), reps * 4)):
                n = hh.shape[0]
                cat = torch.empty(n, FF, dtype=torch.bfloat16, device=dev)

                def ffn():
                    gu_ = torch.mm(hh, ly.w_mlp_in.t())
                    check(lib.qs_hyb_gelu_tanh_mul(cat.data_ptr(), cat.stride(0), gu_.data_ptr(), n, FF, 0, raw()))
                    torch.mm(cat, w_dn.t())
                    return 1
                tm = time_kernel(ffn, r_, stream)
                kern[f"dense_feed_forward_{label}(2 products+act)"] = {"us": tm * 1e6, "tflops": n * 6 * W * FF / tm / 1e12,
                                                                      "frac_of_measured_bf16_peak": n * 6 * W * FF / tm / 1e12 / tflops,
                                                                      "weights_frac_of_measured_hbm": 3 * W * FF * 2 / tm / 1e9 / hbm_gbs}
            gu = torch.randn(T, 2 * FF, device=dev).to(torch.bfloat16)
            cat = torch.empty(T, FF, dtype=torch.bfloat16, device=dev)
            tg = time_kernel(lambda: (check(lib.qs_hyb_gelu_tanh_mul(cat.data_ptr(), cat.stride(0), gu.data_ptr(), T, FF, 0, raw())), 1)[1], reps, stream)
            kern["gelu_tanh_mul"] = {"us": tg * 1e6, "frac_of_measured_hbm": T * FF * 6 / tg / 1e9 / hbm_gbs}
            peer["kernels"] = kern
            del eng, model, gu, cat, h1, h2, w_dn
        torch.cuda.empty_cache()
        rec["rizurax_equal_size"] = peer
        out["sizes"][name] = rec
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------------------------
# --nusuvik: the Nusuvik decoder beside the closest existing model (the Rizurax hybrid decoder) at equal size
# ------------------------------------------------------------------------------------------------------------
def nusuvik_block(args):
    """Prefill (4 prompts x 2048 tokens in one step) and decode (64 sequences at 1024 tokens of context) of a four-layer stack of latent
    attention layers (key/value latent 512 + 64 rotated numbers per position, query latent 3/4 of the width, head size 128 + 64 rotated,
    value size 128) with feed-forwards dense | experts | dense | experts (32 experts in 4 groups of which 2 are kept, 8 per token, expert
    size = feed-forward / 8), the first two layers a loop that runs twice.  Whole steps are captured in CUDA graphs (device time); the
    design's kernels are timed one by one with their algorithmic bytes / flops against the measured copy and bf16 GEMM peaks.  Beside it:
    the Rizurax stack (attention | delta | attention | delta, dense feed-forward) at equal width / heads / head size, the kernels that play
    the same parts there, and the softmax-routed expert mixture of the Toderax design at equal expert sizes."""
    import torch

    from qserve_b200._lib import check, lib
    from qserve_b200.engine import Engine
    from qserve_b200.hybrid import FEED_FORWARDS, HybridDecoder, StepBatch, random_weights
    from qserve_b200.modelcfg import (AttentionMixerConfig, DeltaMixerConfig, HybridConfig, HybridLayerConfig, LatentAttentionMixerConfig, MlpConfig,
                                      MoeConfig, RotaryConfig)

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm_gbs = peaks()[0]
    try:
        tflops = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    except (OSError, KeyError, ValueError):
        tflops = 1590.0
    stream = torch.cuda.current_stream()
    reps = max(3, args.kernel_reps)
    raw = lambda: torch._C._cuda_getCurrentRawStream(0)
    B, CTX, NP, LP, E, TOP, KR, R = 64, 1024, 4, 2048, 32, 8, 512, 64
    out = {"metric": "Nusuvik decoder throughput (tokens/s, random weights, bf16, 4 layers of which 2 run twice)", "unit": "tokens/s", "impl": "ours",
           "dtype": "bf16", "data": "synthetic", "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": tflops}, "sizes": {}}

    def steps(model, eng, V, g):
        prompts = [torch.randint(0, V, (LP,), generator=g).tolist() for _ in range(NP)]
        for i, p_ in enumerate(prompts):
            eng.cache.admit(("p", i)); eng.cache.reserve(("p", i), LP)
        pb = StepBatch.build([(eng.cache.seqs[("p", i)].slot, 0, -1, p_) for i, p_ in enumerate(prompts)], eng.cache.sync_block_table(), dev,
                             eng.cache.page_size)
        t = time_kernel(lambda: (model.forward(pb, eng.cache), 1)[1], reps, stream)
        rec = {"prefill": {"tokens": NP * LP, "ms": t * 1e3, "tokens_per_s": NP * LP / t}}
        for i in range(B):
            eng.cache.admit(("d", i)); eng.cache.reserve(("d", i), CTX + 1)
        db = StepBatch.build([(eng.cache.seqs[("d", i)].slot, CTX, 5, [int(torch.randint(0, V, (1,), generator=g))]) for i in range(B)],
                             eng.cache.sync_block_table(), dev)
        t = time_kernel(lambda: (model.logits(model.forward(db, eng.cache)), 1)[1], reps * 4, stream)
        rec["decode"] = {"batch": B, "ctx": CTX, "ms": t * 1e3, "tokens_per_s": B / t}
        return rec, pb, db

    def mixer_times(mixer, run_cache, pb, db, T):
        proj = torch.randn(T, mixer.in_features, device=dev).to(torch.bfloat16)
        cat = torch.empty(T, mixer.out_features, dtype=torch.bfloat16, device=dev)
        scratch = torch.empty(max(1, mixer.scratch_floats(T)), dtype=torch.float32, device=dev)
        tp = time_kernel(lambda: (mixer.run(proj, cat, pb, run_cache, 64, scratch, 0, raw()), 1)[1], reps, stream)
        td = time_kernel(lambda: (mixer.run(proj[:B], cat[:B], db, run_cache, 64, scratch, 0, raw()), 1)[1], reps * 4, stream)
        return tp, td

    def ff_times(ff, h, label_fn, kern, useful_flops, weight_bytes):
        for label, hh, r_ in (("prefill", h, reps), ("decode", h[:B].contiguous(), reps * 4)):
            tm = time_kernel(lambda: (ff.run(hh, 0, raw()), 1)[1], r_, stream)
            n = hh.shape[0]
            kern[label_fn(label)] = {"us": tm * 1e6, "tflops": n * useful_flops / tm / 1e12, "frac_of_measured_bf16_peak": n * useful_flops / tm / 1e12 / tflops,
                                     "weights_frac_of_measured_hbm": weight_bytes(n) / tm / 1e9 / hbm_gbs}

    for name, (W, H, G, D, FF, V) in HYBRID_SIZES.items():
        T, pairs = NP * LP, NP * (LP * (LP + 1) // 2)
        lat = LatentAttentionMixerConfig(H, D, R, D, KR, 3 * W // 4, RotaryConfig(R, 1e6, layout="half"), (D + R) ** -0.5)
        moe = MoeConfig(E, TOP, FF // TOP, math.inf, alpha=1.0, up_shift=0.0, router="sigmoid", correction=True, groups=4, keep=2)
        dense = MlpConfig("dense", FF, gated=False, bias=True)
        cfg = HybridConfig("Nusuvik", V, W, 1e-5, tuple(HybridLayerConfig("latent_attention", lat, f) for f in (dense, moe, dense, moe)),
                           0, 2, 2, 4093, 131, 11, norm_offset=0.0, norm_kind="layer", shared_norm=True, loop_in=True, logit_softcap=30.0)
        g = torch.Generator().manual_seed(0)
        with torch.no_grad():
            model = HybridDecoder(cfg, random_weights(cfg, 0, dev), torch.bfloat16, dev)
            eng = Engine(model, max_tokens=B * (CTX + 64) + NP * LP, max_seqs=B + NP)
            rec, pb, db = steps(model, eng, V, g)
            kern = {}
            mx = model.layers[0].mixer
            tp, td = mixer_times(mx, eng.cache.runs[0], pb, db, T)
            # useful work: scores and weighted values of heads of size (D + R) and D; executed: the same over the latent's K + R and K numbers
            useful, executed = H * pairs * 2 * (D + R + D), H * pairs * 2 * (KR + R + KR)
            kern["latent_attention_prefill(norms+append+q up+rotate+keys and values of every head+per-head tile attention+gate)"] = {
                "us": tp * 1e6, "tflops": useful / tp / 1e12, "frac_of_measured_bf16_peak": useful / tp / 1e12 / tflops}
            import qserve_b200.hybrid as hyb_mod
            hyb_mod.LATENT_IMPL = "latent"
            try:
                tl, _ = mixer_times(mx, eng.cache.runs[0], pb, db, T)
            finally:
                hyb_mod.LATENT_IMPL = None
            kern["latent_attention_prefill, kept in the latent space(norms+append+q up+key up+rotate+latent tiles+value up+gate)"] = {
                "us": tl * 1e6, "useful_tflops": useful / tl / 1e12, "executed_tflops": executed / tl / 1e12,
                "frac_of_measured_bf16_peak_useful": useful / tl / 1e12 / tflops, "frac_of_measured_bf16_peak_executed": executed / tl / 1e12 / tflops}
            kern["latent_attention_decode(the same)"] = {"us": td * 1e6, "frac_of_measured_hbm": B * (CTX + 1) * (KR + R) * 2 / td / 1e9 / hbm_gbs}
            # the attention kernels alone
            qa = torch.randn(T, H, KR + R, device=dev).to(torch.bfloat16)
            ol = torch.empty(H, T, KR, dtype=torch.bfloat16, device=dev)
            scratch = torch.empty(max(1, mx.scratch_floats(T)), dtype=torch.float32, device=dev)
            pool = eng.cache.runs[0]["c"]

            def attn(b_, n):
                check(lib.qs_hyb_latent_attention_fast(ol.data_ptr(), qa.data_ptr(), pool.data_ptr(), b_.tok_slot.data_ptr(), b_.tok_pos.data_ptr(),
                                                       b_.block_table.data_ptr(), b_.block_table.shape[1], b_.tile_entry.data_ptr(), b_.tile_row0.data_ptr(),
                                                       b_.n_tiles, b_.short_tokens.data_ptr(), b_.n_short, b_.entry_start.data_ptr(), b_.entry_len.data_ptr(),
                                                       b_.entry_slot.data_ptr(), b_.entry_pos0.data_ptr(), n, scratch.data_ptr(), H, KR, R, lat.scale, 64, 0, 0,
                                                       None, 0, raw()))
                return 1
            ta = time_kernel(lambda: attn(pb, T), reps, stream)
            kern["latent_tile_kernel_prefill"] = {"us": ta * 1e6, "useful_tflops": useful / ta / 1e12, "executed_tflops": executed / ta / 1e12,
                                                  "frac_of_measured_bf16_peak_useful": useful / ta / 1e12 / tflops,
                                                  "frac_of_measured_bf16_peak_executed": executed / ta / 1e12 / tflops}
            ta = time_kernel(lambda: attn(db, B), reps * 4, stream)
            kern["latent_tile_kernel_decode(+merge)"] = {"us": ta * 1e6, "frac_of_measured_hbm": B * (CTX + 1) * (KR + R) * 2 / ta / 1e9 / hbm_gbs}
            # the same kernel on 8 times the context, over a pool of its own: a step's cells (600 MB) exceed L2 several times over
            LONG = 8 * CTX
            big = torch.randn(B * LONG // 64, 64, KR + R, device=dev).to(torch.bfloat16)
            lt = torch.arange(B * LONG // 64, dtype=torch.int32, device=dev).view(B, LONG // 64).contiguous()
            lb = StepBatch.build([(i, LONG - 1, 5, [1]) for i in range(B)], lt, dev)

            def attn_long():
                check(lib.qs_hyb_latent_attention_fast(ol.data_ptr(), qa.data_ptr(), big.data_ptr(), lb.tok_slot.data_ptr(), lb.tok_pos.data_ptr(),
                                                       lt.data_ptr(), lt.shape[1], None, None, 0, lb.short_tokens.data_ptr(), lb.n_short, None, None, None,
                                                       None, B, scratch.data_ptr(), H, KR, R, lat.scale, 64, 0, 0, None, 0, raw()))
                return 1
            ta = time_kernel(attn_long, reps * 2, stream)
            kern[f"latent_tile_kernel_decode(+merge), context {LONG}"] = {"us": ta * 1e6, "frac_of_measured_hbm": B * LONG * (KR + R) * 2 / ta / 1e9 / hbm_gbs}
            del big, lt, lb
            del qa, ol
            ly = model.layers[0]
            x = torch.randn(T, W, device=dev)
            h1, upd = torch.empty(T, W, dtype=torch.bfloat16, device=dev), torch.zeros(T, W, dtype=torch.bfloat16, device=dev)
            tn = time_kernel(lambda: (check(lib.qs_hyb_stream_update_norm(h1.data_ptr(), None, x.data_ptr(), None, upd.data_ptr(), 0, None, 0,
                                                                          ly.out_bias.data_ptr(), ly.norm1.data_ptr(), ly.norm1_b.data_ptr(), 2, 1e-5, T, W,
                                                                          0, raw())), 1)[1], reps, stream)
            kern["add_bias_layer_norm"] = {"us": tn * 1e6, "frac_of_measured_hbm": T * W * 12 / tn / 1e9 / hbm_gbs}
            gu = torch.randn(T, FF, device=dev).to(torch.bfloat16)
            cat = torch.empty(T, FF, dtype=torch.bfloat16, device=dev)
            tg = time_kernel(lambda: (check(lib.qs_hyb_bias_gelu_tanh(cat.data_ptr(), FF, gu.data_ptr(), FF, ly.mlp_in_bias.data_ptr(), T, FF, 0, raw())), 1)[1],
                             reps, stream)
            kern["bias_gelu_tanh"] = {"us": tg * 1e6, "frac_of_measured_hbm": T * FF * 4 / tg / 1e9 / hbm_gbs}
            del x, upd, gu, cat
            h = torch.randn(T, W, device=dev).to(torch.bfloat16)
            ffl = 2 * 3 * W * TOP * moe.ff
            wb = lambda n: 3 * W * min(E, n * TOP) * moe.ff * 2
            ff_times(model.layers[1].side_ff, h, lambda l: f"expert_feed_forward_{l}(grouped sigmoid router+sort+gather+2 grouped products+act+combine)", kern, ffl, wb)
            ff1 = model.layers[1].side_ff
            route, ti, tw = torch.empty(T, E, device=dev), torch.empty(T, TOP, dtype=torch.int32, device=dev), torch.empty(T, TOP, device=dev)
            for mode, label in ((1, "router_sigmoid_groups"), (0, "router_softmax(the other design's)")):
                tr = time_kernel(lambda: (check(lib.qs_hyb_moe_router(route.data_ptr(), ti.data_ptr(), tw.data_ptr(), h.data_ptr(), ff1.w_router.data_ptr(),
                                                                      T, W, E, TOP, mode, ff1.correction.data_ptr(), 4, 2, 0, raw())), 1)[1], reps, stream)
                kern[label] = {"us": tr * 1e6, "frac_of_measured_hbm": T * W * 2 / tr / 1e9 / hbm_gbs}
            # the like feed-forward of the closest design with experts: softmax router, clamped activation, no shared expert, equal sizes
            tmoe = MoeConfig(E, TOP, FF // TOP, 7.0)
            tw_ = {k[len("l1.mlp."):]: v for k, v in random_weights(cfg, 1, dev).items() if k.startswith("l1.mlp.")}
            ff_times(FEED_FORWARDS[MoeConfig](tmoe, tw_, W, torch.bfloat16, dev), h, lambda l: f"expert_feed_forward_{l}(softmax router, clamped activation: the other design's)",
                     kern, ffl, wb)
            rec["kernels"] = kern
            del eng, model, h, tw_, pool, scratch
        torch.cuda.empty_cache()
        # ---- the closest existing model at equal size: Rizurax (differential attention | gated delta rule, dense feed-forward)
        ratt = AttentionMixerConfig(H, G, D, D, RotaryConfig(D // 2, 1e6, 4.0, 4096, 32.0, 1.0), D ** -0.5, maps=2, diff=0.5, head_norm=True)
        rdlt = DeltaMixerConfig(H, G, D, D, 4)
        rcfg = HybridConfig("Rizurax", V, W, 1e-5, tuple(HybridLayerConfig(t, m, MlpConfig("dense", FF)) for t, m in
                                                        (("attention", ratt), ("delta", rdlt), ("attention", ratt), ("delta", rdlt))),
                            pair_buckets=4093, pair_mul_prev=131, pair_mul_cur=11)
        with torch.no_grad():
            model = HybridDecoder(rcfg, random_weights(rcfg, 0, dev), torch.bfloat16, dev)
            eng = Engine(model, max_tokens=B * (CTX + 64) + NP * LP, max_seqs=B + NP)
            peer, pb, db = steps(model, eng, V, g)
            kern = {}
            tp, td = mixer_times(model.layers[0].mixer, eng.cache.runs[0], pb, db, T)
            flops = H * pairs * 8 * D
            kern["attention_prefill(rope+append+attention, 2 maps)"] = {"us": tp * 1e6, "tflops": flops / tp / 1e12, "frac_of_measured_bf16_peak": flops / tp / 1e12 / tflops}
            kern["attention_decode(rope+append+attention, 2 maps)"] = {"us": td * 1e6, "frac_of_measured_hbm": B * (CTX + 1) * G * 3 * D * 2 / td / 1e9 / hbm_gbs}
            ly = model.layers[0]
            x = torch.randn(T, W, device=dev)
            h1, h2 = torch.empty(T, W, dtype=torch.bfloat16, device=dev), torch.empty(T, W, dtype=torch.bfloat16, device=dev)
            upd = torch.zeros(T, W, dtype=torch.bfloat16, device=dev)
            tn = time_kernel(lambda: (check(lib.qs_hyb_rms_norm(h1.data_ptr(), h2.data_ptr(), x.data_ptr(), upd.data_ptr(), ly.norm1.data_ptr(),
                                                                 ly.norm2.data_ptr(), 1.0, 1e-5, T, W, 0, raw())), 1)[1], reps, stream)
            kern["add_rms_norm_dual"] = {"us": tn * 1e6, "frac_of_measured_hbm": T * W * 14 / tn / 1e9 / hbm_gbs}
            gu = torch.randn(T, 2 * FF, device=dev).to(torch.bfloat16)
            cat = torch.empty(T, FF, dtype=torch.bfloat16, device=dev)
            tg = time_kernel(lambda: (check(lib.qs_hyb_gelu_tanh_mul(cat.data_ptr(), cat.stride(0), gu.data_ptr(), T, FF, 0, raw())), 1)[1], reps, stream)
            kern["gelu_tanh_mul"] = {"us": tg * 1e6, "frac_of_measured_hbm": T * FF * 6 / tg / 1e9 / hbm_gbs}
            peer["kernels"] = kern
            del eng, model, gu, cat, h1, h2, x, upd
        torch.cuda.empty_cache()
        rec["rizurax_equal_size"] = peer
        out["sizes"][name] = rec
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------------------------
# --zuzezen: the Zuzezen decoder beside the closest existing model (the Rizurax hybrid decoder) at equal size
# ------------------------------------------------------------------------------------------------------------
def zuzezen_block(args):
    """Prefill (4 prompts x 2048 tokens in one step) and decode (64 sequences at 1024 tokens of context) of a five-layer Zuzezen stack gla |
    latent attention | attention | latent attention | gla (the attention layers with a feed-forward) beside a four-layer Rizurax stack at equal
    width, head geometry and feed-forward size; then each Zuzezen kernel beside its like kernel of another design at equal size: the
    windowed attention (window 1024, 4 kept positions, distance bias, head gate, tied values) beside one-map sink attention whose chunk
    spans the same keys, the gated-linear scan beside the gate recurrence on the same scan kernel, latent attention with a sink and direct
    queries beside the one with a query latent, the post-norm landing kernel beside the add + norm kernel, the biased silu gate beside the
    gelu gate."""
    import torch

    from qserve_b200._lib import check, lib
    from qserve_b200.engine import Engine
    from qserve_b200.hybrid import MIXERS, HybridDecoder, StepBatch, random_weights
    from qserve_b200.modelcfg import (AttentionMixerConfig, DeltaMixerConfig, GatedLinearMixerConfig, GateRecurrenceMixerConfig, HybridConfig,
                                      HybridLayerConfig, LatentAttentionMixerConfig, MlpConfig, RotaryConfig)

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm_gbs = peaks()[0]
    try:
        tflops = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    except (OSError, KeyError, ValueError):
        tflops = 1590.0
    stream = torch.cuda.current_stream()
    reps = max(3, args.kernel_reps)
    raw = lambda: torch._C._cuda_getCurrentRawStream(0)
    B, CTX, NP, LP, KR, R, WIN, KEEP = 64, 1024, 4, 2048, 512, 64, 1024, 4
    out = {"metric": "Zuzezen decoder throughput (tokens/s, random weights, bf16, 5 layers)", "unit": "tokens/s", "impl": "ours",
           "dtype": "bf16", "data": "synthetic", "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": tflops}, "sizes": {}}

    def steps(model, eng, V, g):
        prompts = [torch.randint(0, V, (LP,), generator=g).tolist() for _ in range(NP)]
        for i, p_ in enumerate(prompts):
            eng.cache.admit(("p", i)); eng.cache.reserve(("p", i), LP)
        pb = StepBatch.build([(eng.cache.seqs[("p", i)].slot, 0, -1, p_) for i, p_ in enumerate(prompts)], eng.cache.sync_block_table(), dev,
                             eng.cache.page_size)
        t = time_kernel(lambda: (model.forward(pb, eng.cache), 1)[1], reps, stream)
        rec = {"prefill": {"tokens": NP * LP, "ms": t * 1e3, "tokens_per_s": NP * LP / t}}
        for i in range(B):
            eng.cache.admit(("d", i)); eng.cache.reserve(("d", i), CTX + 1)
        db = StepBatch.build([(eng.cache.seqs[("d", i)].slot, CTX, 5, [int(torch.randint(0, V, (1,), generator=g))]) for i in range(B)],
                             eng.cache.sync_block_table(), dev)
        t = time_kernel(lambda: (model.logits(model.forward(db, eng.cache)), 1)[1], reps * 4, stream)
        rec["decode"] = {"batch": B, "ctx": CTX, "ms": t * 1e3, "tokens_per_s": B / t}
        return rec, pb, db

    def mixer_times(mixer, run_cache, pb, db, T):
        proj = torch.randn(T, mixer.in_features, device=dev).to(torch.bfloat16)
        cat = torch.empty(T, mixer.out_features, dtype=torch.bfloat16, device=dev)
        scratch = torch.empty(max(1, mixer.scratch_floats(T)), dtype=torch.float32, device=dev)
        tp = time_kernel(lambda: (mixer.run(proj, cat, pb, run_cache, 64, scratch, 0, raw()), 1)[1], reps, stream)
        td = time_kernel(lambda: (mixer.run(proj[:B], cat[:B], db, run_cache, 64, scratch, 0, raw()), 1)[1], reps * 4, stream)
        return tp, td

    def lone_mixer(mcfg, W, seed):
        """A mixer of another design with random weights, and storage for it in a cache of its own."""
        c1 = HybridConfig("bench", 8, W, 1e-5, (HybridLayerConfig("m", mcfg, None),))
        w = {k[len("l0.mix."):]: v for k, v in random_weights(c1, seed, dev).items() if k.startswith("l0.mix.")}
        return MIXERS[type(mcfg)](mcfg, w, 1e-5, torch.bfloat16, dev)

    for name, (W, H, G, D, FF, V) in HYBRID_SIZES.items():
        T = NP * LP
        gla = GatedLinearMixerConfig(H, D, D, 8.0, 32)
        lat = LatentAttentionMixerConfig(H, D, R, D, KR, 0, RotaryConfig(R, 1e6, 4.0, 4096, 32.0, 1.0), (D + R) ** -0.5, gate=True, gate_wide=True, sink=True)
        att = AttentionMixerConfig(H, G, D, D, None, D ** -0.5, bias=True, qk_norm=True, window=WIN, keep_first=KEEP, qk_gain=True, tied_values=True,
                                   distance_slope=8.0, head_gate=True)
        ffc = MlpConfig("dense", FF, gated=True, bias=True, act="silu")
        cfg = HybridConfig("Zuzezen", V, W, 1e-5, tuple(HybridLayerConfig(t, m, f) for t, m, f in
                                                        (("gla", gla, None), ("latent_attention", lat, ffc), ("attention", att, ffc),
                                                         ("latent_attention", lat, ffc), ("gla", gla, None))),
                           norm_offset=1.0, block="post", embed_scale=8.0, layer_scale=True)
        g = torch.Generator().manual_seed(0)
        with torch.no_grad():
            model = HybridDecoder(cfg, random_weights(cfg, 0, dev), torch.bfloat16, dev)
            eng = Engine(model, max_tokens=B * (CTX + 64) + NP * LP, max_seqs=B + NP)
            rec, pb, db = steps(model, eng, V, g)
            kern = {}
            # keys a query sees: the window (or all earlier positions while the prompt is shorter), and the kept first positions
            pairs_win = NP * sum(min(i + 1, WIN) + (min(KEEP, i + 1 - WIN) if i + 1 > WIN else 0) for i in range(LP))
            pairs_all = NP * (LP * (LP + 1) // 2)
            seen_dec = min(CTX + 1, WIN) + (min(KEEP, CTX + 1 - WIN) if CTX + 1 > WIN else 0)
            tp, td = mixer_times(model.layers[2].mixer, eng.cache.runs[2], pb, db, T)
            kern["window_attention_prefill(bias+unit rms+gains+append, tiles with window / kept positions / distance bias, head gate)"] = {
                "us": tp * 1e6, "tflops": H * pairs_win * 4 * D / tp / 1e12, "frac_of_measured_bf16_peak": H * pairs_win * 4 * D / tp / 1e12 / tflops}
            kern["window_attention_decode(the same, head groups)"] = {"us": td * 1e6, "frac_of_measured_hbm": B * seen_dec * G * 2 * D * 2 / td / 1e9 / hbm_gbs}
            tp, td = mixer_times(model.layers[0].mixer, eng.cache.runs[0], pb, db, T)
            state_bytes = B * H * D * D * 4 * 2
            kern["gated_linear_prefill(decay product+prepare+scan+norm and gate)"] = {"us": tp * 1e6, "tokens_per_s": T / tp,
                                                                                      "state_updates_gflops": T * H * D * D * 4 / tp / 1e9}
            kern["gated_linear_decode(the same)"] = {"us": td * 1e6, "state_frac_of_measured_hbm": state_bytes / td / 1e9 / hbm_gbs}
            tp, td = mixer_times(model.layers[1].mixer, eng.cache.runs[1], pb, db, T)
            useful = H * pairs_all * 2 * (D + R + D)
            kern["latent_attention_prefill(norm+rotate+append+keys and values of every head+per-head tile attention with sink+wide gate)"] = {
                "us": tp * 1e6, "tflops": useful / tp / 1e12, "frac_of_measured_bf16_peak": useful / tp / 1e12 / tflops}
            kern["latent_attention_decode(norm+rotate+append+key up+latent tiles with sink+value up+wide gate)"] = {
                "us": td * 1e6, "frac_of_measured_hbm": B * (CTX + 1) * (KR + R) * 2 / td / 1e9 / hbm_gbs}
            ly = model.layers[1]
            x = torch.randn(T, W, device=dev)
            y = torch.randn(T, W, device=dev)
            h1 = torch.empty(T, W, dtype=torch.bfloat16, device=dev)
            tn = time_kernel(lambda: (check(lib.qs_hyb_post_norm_update(h1.data_ptr(), x.data_ptr(), y.data_ptr(), 1, ly.ff.out_bias.data_ptr(), ly.norm2.data_ptr(),
                                                                         ly.ls2.data_ptr(), 1.0, 1e-5, T, W, 0, raw())), 1)[1], reps, stream)
            kern["post_norm_update(fp32 rows in, bias, norm, layer scale, residual, bf16 copy)"] = {"us": tn * 1e6, "frac_of_measured_hbm": T * W * 14 / tn / 1e9 / hbm_gbs}
            gu = torch.randn(T, 2 * FF, device=dev).to(torch.bfloat16)
            cat = torch.empty(T, FF, dtype=torch.bfloat16, device=dev)
            tg = time_kernel(lambda: (check(lib.qs_hyb_bias_gated_act(cat.data_ptr(), FF, gu.data_ptr(), 2 * FF, ly.ff.in_bias.data_ptr(), T, FF, 1, 0, raw())), 1)[1],
                             reps, stream)
            kern["bias_silu_mul"] = {"us": tg * 1e6, "frac_of_measured_hbm": T * FF * 6 / tg / 1e9 / hbm_gbs}
            # ---- like kernels of the other designs at equal size, on this engine's batches
            like = {}
            sink_att = lone_mixer(AttentionMixerConfig(H, G, D, D, None, D ** -0.5, bias=True, qk_norm=True, head_temp=True, sink=True, chunk=WIN), W, 1)
            store = eng.cache.mixer_storage(sink_att.m)
            tp, td = mixer_times(sink_att, store, pb, db, T)
            pairs_chunk = NP * sum(i % WIN + 1 for i in range(LP))
            like["sink_attention_prefill(one map, chunks of the window's size)"] = {
                "us": tp * 1e6, "tflops": H * pairs_chunk * 4 * D / tp / 1e12, "frac_of_measured_bf16_peak": H * pairs_chunk * 4 * D / tp / 1e12 / tflops}
            like["sink_attention_decode"] = {"us": td * 1e6, "frac_of_measured_hbm": B * (CTX % WIN + 1) * G * 2 * D * 2 / td / 1e9 / hbm_gbs}
            del store
            full_att = lone_mixer(AttentionMixerConfig(H, G, D, D, None, D ** -0.5, bias=True, qk_norm=True, head_temp=True, sink=True), W, 1)
            store = eng.cache.mixer_storage(full_att.m)
            tp, td = mixer_times(full_att, store, pb, db, T)
            like["sink_attention_prefill(one map, no mask)"] = {
                "us": tp * 1e6, "tflops": H * pairs_all * 4 * D / tp / 1e12, "frac_of_measured_bf16_peak": H * pairs_all * 4 * D / tp / 1e12 / tflops}
            like["sink_attention_decode(no mask)"] = {"us": td * 1e6, "frac_of_measured_hbm": B * (CTX + 1) * G * 2 * D * 2 / td / 1e9 / hbm_gbs}
            del store
            gate = lone_mixer(GateRecurrenceMixerConfig(H, D, D), W, 2)
            store = eng.cache.mixer_storage(gate.m)
            tp, td = mixer_times(gate, store, pb, db, T)
            like["gate_recurrence_prefill(prepare+scan+norm)"] = {"us": tp * 1e6, "tokens_per_s": T / tp, "state_updates_gflops": T * H * D * D * 4 / tp / 1e9}
            like["gate_recurrence_decode"] = {"us": td * 1e6, "state_frac_of_measured_hbm": state_bytes / td / 1e9 / hbm_gbs}
            del store
            qlat = lone_mixer(LatentAttentionMixerConfig(H, D, R, D, KR, 3 * W // 4, RotaryConfig(R, 1e6, layout="half"), (D + R) ** -0.5), W, 3)
            store = eng.cache.mixer_storage(qlat.m)
            tp, td = mixer_times(qlat, store, pb, db, T)
            like["latent_attention_prefill(query latent, no sink, head gate)"] = {
                "us": tp * 1e6, "tflops": useful / tp / 1e12, "frac_of_measured_bf16_peak": useful / tp / 1e12 / tflops}
            like["latent_attention_decode(query latent, no sink, head gate)"] = {"us": td * 1e6, "frac_of_measured_hbm": B * (CTX + 1) * (KR + R) * 2 / td / 1e9 / hbm_gbs}
            del store
            h2 = torch.empty(T, W, dtype=torch.bfloat16, device=dev)
            upd = torch.zeros(T, W, dtype=torch.bfloat16, device=dev)
            tn = time_kernel(lambda: (check(lib.qs_hyb_rms_norm(h1.data_ptr(), h2.data_ptr(), x.data_ptr(), upd.data_ptr(), ly.norm1.data_ptr(),
                                                                 ly.norm2.data_ptr(), 1.0, 1e-5, T, W, 0, raw())), 1)[1], reps, stream)
            like["add_rms_norm_dual"] = {"us": tn * 1e6, "frac_of_measured_hbm": T * W * 14 / tn / 1e9 / hbm_gbs}
            tg = time_kernel(lambda: (check(lib.qs_hyb_gelu_tanh_mul(cat.data_ptr(), cat.stride(0), gu.data_ptr(), T, FF, 0, raw())), 1)[1], reps, stream)
            like["gelu_tanh_mul"] = {"us": tg * 1e6, "frac_of_measured_hbm": T * FF * 6 / tg / 1e9 / hbm_gbs}
            rec["kernels"], rec["like_kernels_of_other_designs"] = kern, like
            del eng, model, x, y, h1, h2, upd, gu, cat, sink_att, full_att, gate, qlat
        torch.cuda.empty_cache()
        # ---- the closest existing model at equal size: Rizurax (differential attention | gated delta rule, dense feed-forward)
        ratt = AttentionMixerConfig(H, G, D, D, RotaryConfig(D // 2, 1e6, 4.0, 4096, 32.0, 1.0), D ** -0.5, maps=2, diff=0.5, head_norm=True)
        rdlt = DeltaMixerConfig(H, G, D, D, 4)
        rcfg = HybridConfig("Rizurax", V, W, 1e-5, tuple(HybridLayerConfig(t, m, MlpConfig("dense", FF)) for t, m in
                                                        (("attention", ratt), ("delta", rdlt), ("attention", ratt), ("delta", rdlt))),
                            pair_buckets=4093, pair_mul_prev=131, pair_mul_cur=11)
        with torch.no_grad():
            model = HybridDecoder(rcfg, random_weights(rcfg, 0, dev), torch.bfloat16, dev)
            eng = Engine(model, max_tokens=B * (CTX + 64) + NP * LP, max_seqs=B + NP)
            peer, _, _ = steps(model, eng, V, g)
            del eng, model
        torch.cuda.empty_cache()
        rec["rizurax_equal_size"] = peer
        out["sizes"][name] = rec
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------------------------
def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if args.hybrid:
        if rank == 0:
            hybrid_block(args)
        return
    if args.toderax:
        if rank == 0:
            toderax_block(args)
        return
    if args.nusuvik:
        if rank == 0:
            nusuvik_block(args)
        return
    if args.zuzezen:
        if rank == 0:
            zuzezen_block(args)
        return
    if args.impl == "reference-gpu":
        if rank == 0:
            reference_gpu_arm(args)
        return

    import torch
    import torch.distributed as dist

    assert torch.cuda.is_available(), "bench.py needs a CUDA device: qserve_b200 has no CPU path (use --impl reference for the CPU baseline)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from qserve_b200 import backend
    from qserve_b200.decode import DecodeRunner

    backend.set_pdl(not args.no_pdl)
    cfg = model_cfg(args.model)
    if args.tp_only:
        with torch.no_grad():
            rec = tp_block(args, rank, world, dev, peaks()[0])
        if rank == 0:
            print(json.dumps({"tp": rec}), flush=True)
        sys.stdout.flush()
        if world > 1:
            dist.barrier()
            os._exit(0)
        return
    run = DecodeRunner(args.model, args.precision, args.batch, args.ctx, dev, seed=rank, layers=args.layers, fused=not args.no_fused)
    hbm_gbs, peak_src = peaks()

    # ---- pinned host buffers for the end-to-end leg ------------------------------------------------------
    tok_host = torch.randint(0, cfg.vocab, (args.batch,), dtype=torch.int64).pin_memory()
    out_host = torch.zeros(args.batch, dtype=torch.int64).pin_memory()
    run.tokens_in.copy_(tok_host)
    if args.no_graph:
        with torch.no_grad():
            for _ in range(2):
                run.tokens_out.copy_(run.forward(run.tokens_in))
        step = lambda: run.tokens_out.copy_(run.forward(run.tokens_in))
    else:
        run.capture()
        step = run.step
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            step()
        if os.environ.get("QS_PROFILE_STEP"):  # ncu --profile-from-start off: exactly one eager step between profiler start / stop
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            run.tokens_out.copy_(run.forward(run.tokens_in))
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        # ---- device-resident timing: exactly K steps, CUDA events, max over ranks -------------------------
        barrier()
        with ClockSampler(local_rank) as clk:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(args.steps):
                step()
            e1.record(stream)
            barrier()
        ms_dev = e0.elapsed_time(e1)
        # ---- end to end: host tokens in (pinned) -> H2D -> step -> D2H sampled tokens (pinned), every step ----
        barrier()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record(stream)
        for _ in range(args.steps):
            run.tokens_in.copy_(tok_host, non_blocking=True)
            step()
            out_host.copy_(run.tokens_out, non_blocking=True)
            stream.synchronize()          # the engine consumes the sampled tokens on the host every step (llm_engine.py:595)
            tok_host.copy_(out_host)      # feed them back, as the generation loop does
        e3.record(stream)
        barrier()
        ms_e2e = e2.elapsed_time(e3)

    if world > 1:
        t = torch.tensor([ms_dev, ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_dev, ms_e2e = t.tolist()
    tokens_per_step = args.batch * world
    value = tokens_per_step * args.steps / (ms_dev * 1e-3)
    e2e_value = tokens_per_step * args.steps / (ms_e2e * 1e-3)
    launches_per_step = run.launches_per_step

    kern, refm, cpu, ref_gpu = None, None, None, None
    if rank == 0:
        with torch.no_grad():
            kern = kernel_table(run, args.kernel_reps, hbm_gbs)
        if world == 1 and not args.no_refmodel:
            try:
                refm = refmodel_block(run, args, max(5, min(args.steps, 20)))
            except Exception as e:  # noqa: BLE001  (a broken side block must not lose the headline)
                refm = {"error": repr(e)}
    # free the 8B replica before the 72B record
    run.graph = None
    del run
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    fused = not args.no_fused
    clocks = clk.summary()

    def make_line(tp_rec):
        """The result line (rank 0).  Built from the data-parallel measurement alone, so that a failure of the tensor-parallel side record at
        N > 1 can still be reported next to a valid headline."""
        roof = roofline_from(kern, hbm_gbs, peak_src, fused)
        sb = step_bytes(cfg, args.precision, args.batch, args.ctx, args.layers)
        line = {
            "metric": metric_name(args), "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "s8", "data": "synthetic", "config": make_config(args, world),
            "run": {"graph": not args.no_graph, "pdl": not args.no_pdl, "fused_small_ops": fused,
                    "timing": "CUDA events on the launching stream, barrier + synchronize on both sides, max over ranks"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": args.batch * 8 * world, "d2h_bytes_per_step": args.batch * 8 * world,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": roof,
            "kernels": kern,
            "step_hbm_frac": (sb / (ms_dev / args.steps * 1e-3)) / 1e9 / hbm_gbs,
        }
        if tp_rec is not None:
            line["tp"] = tp_rec
        return line

    tp_rec = None
    if not args.no_tp and (args.model, args.precision) == ("llama-3-8b", "w4a8kv4"):
        import threading

        tp_done = threading.Event()

        def bail(why):
            # N > 1 and the tensor-parallel record failed or hangs on some rank: the data-parallel headline is complete and valid -- print it with
            # the error and leave without touching the (possibly wedged) communicator again
            if rank == 0:
                print(json.dumps(make_line({"error": why})), flush=True)
            sys.stdout.flush()
            os._exit(0)

        def watchdog():
            if not tp_done.wait(args.tp_timeout):
                bail(f"tensor-parallel record did not finish within {args.tp_timeout} s")

        if world > 1:
            dist.barrier()  # rank 0 has just spent seconds on the kernel table: enter the collective phase together
            threading.Thread(target=watchdog, daemon=True).start()
        try:
            with torch.no_grad():
                tp_rec = tp_block(args, rank, world, dev, hbm_gbs)
        except Exception as e:  # noqa: BLE001
            tp_rec = {"error": repr(e)}
            if world > 1:
                if rank != 0:
                    time.sleep(5)  # give rank 0 a moment to fail on its own (it prints); otherwise its watchdog prints
                bail(repr(e)[:400])
        tp_done.set()

    def finish():
        # do not let a slow communicator teardown keep the launcher alive after the result line is out
        sys.stdout.flush()
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()
            os._exit(0)

    if world > 1:
        dist.barrier()
    if rank != 0:
        finish()
        return

    if world == 1 and not args.no_ref_gpu:
        # the reference's own CUDA kernels on this box, same shapes / harness, in a separate process (keeps this arm's process free of oracle/_ref)
        try:
            cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference-gpu", "--steps", str(max(5, min(args.steps, 10))), "--warmup", "3",
                   "--model", args.model, "--precision", args.precision, "--batch", str(args.batch), "--ctx", str(args.ctx), "--kernel-reps", "3"]
            if args.layers is not None:
                cmd += ["--layers", str(args.layers)]
            res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
            lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
            ref_gpu = json.loads(lines[-1]) if lines else {"error": (res.stderr or res.stdout)[-400:]}
        except Exception as e:  # noqa: BLE001
            ref_gpu = {"error": repr(e)}
    if world == 1 and not args.no_cpu_baseline:
        from oracle import cpu_baseline as cb

        threads = os.cpu_count() or 1
        sample = cb.LayerSample(cfg.hidden, cfg.intermediate, cfg.heads, cfg.kv_heads, args.batch, args.ctx, threads)
        t_lm = cb.lm_head_sample(cfg.hidden, cfg.vocab, args.batch, threads)
        sample.run()
        rs = [sample.run() for _ in range(3)]
        layer_s = sum(r["layer_s"] for r in rs) / len(rs)
        v = args.batch / (cfg.layers * layer_s + t_lm)
        cpu = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"3 timed runs (after 1 warm-up) of 1 of {cfg.layers} decoder layers (4 W4A8 GEMMs M={args.batch} + KV4 attention B={args.batch} ctx={args.ctx}) on "
                         f"torch-CPU dequant-then-matmul + fp16 lm_head once, extrapolated x{cfg.layers}; {layer_s:.2f} s/layer, lm_head {t_lm:.2f} s"}

    line = make_line(tp_rec)
    if refm is not None:
        line["refmodel"] = refm
    if ref_gpu is not None:
        keep = {k: ref_gpu[k] for k in ("value", "unit", "ms_per_step", "host_ms_per_step", "kernel_ms_per_step", "tokens_per_s_kernel_time_only", "what",
                                        "unavailable", "error") if k in ref_gpu}
        if "kernels" in ref_gpu:
            keep["kernel_us"] = {k: v["us"] for k, v in ref_gpu["kernels"].items()}
            keep["speedup_per_kernel"] = {k: ref_gpu["kernels"][k]["us"] / kern[k]["us"] for k in ref_gpu["kernels"] if k in kern}
            keep["speedup_step_vs_reference_eager"] = value / ref_gpu["value"]
            keep["speedup_step_vs_reference_kernel_time_only"] = value / ref_gpu["tokens_per_s_kernel_time_only"]
        line["ref_gpu"] = keep
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    finish()


if __name__ == "__main__":
    main()
