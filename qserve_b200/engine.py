"""Serving engine of the hybrid decoders: requests, a continuous-batching scheduler with chunked prompts, the step function, sampling.

Shape follows the reference's engine (qserve/serve/engine.py: add_request / step loop; qserve/core/scheduler.py: running before
waiting, admission while blocks are free; qserve/sampling_params.py; qserve/modeling/layers/sampler.py), re-cut for a flat token batch:
one step runs single decoded tokens of some sequences beside portions of other sequences' prompts in the same kernels.

`Engine.step` is the only way tokens reach the model: `generate` drives it through the `Scheduler`, and a trace replay (`replay_trace`,
bin/trace_run) drives it with the batches a trace dictates.
"""
from __future__ import annotations

import json
import os
import sys
from collections import deque
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .cache import HybridCache, OutOfPages
from .hybrid import HybridDecoder, StepBatch


@dataclass
class SamplingParams:
    """temperature 0 = greedy; top_k 0 = off; top_p 1 = off (qserve/sampling_params.py)."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    max_new_tokens: int = 16
    stop_token_ids: Tuple[int, ...] = ()


@dataclass
class Request:
    id: object
    prompt: List[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    output: List[int] = field(default_factory=list)
    fed: int = 0            # tokens of prompt + output already run through the model
    finished: bool = False

    def pending(self) -> List[int]:
        """Tokens known but not yet run: the rest of the prompt, or the last sampled token."""
        return (self.prompt + self.output)[self.fed:]


def sample(logits: torch.Tensor, params: Sequence[SamplingParams], generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Next token per row of fp32 logits [n, vocab]: argmax for temperature 0, otherwise temperature / top-k / top-p sampling."""
    out = torch.argmax(logits, dim=-1)
    for i, p in enumerate(params):
        if p.temperature <= 0.0:
            continue
        row = logits[i] / p.temperature
        if p.top_k > 0:
            kth = torch.topk(row, min(p.top_k, row.numel())).values[-1]
            row = torch.where(row < kth, torch.full_like(row, float("-inf")), row)
        probs = torch.softmax(row, -1)
        if p.top_p < 1.0:
            sp, idx = torch.sort(probs, descending=True)
            keep = torch.cumsum(sp, 0) - sp < p.top_p
            probs = torch.zeros_like(probs).scatter(0, idx, sp * keep)
            probs = probs / probs.sum()
        out[i] = torch.multinomial(probs, 1, generator=generator)[0]
    return out


class Scheduler:
    """Continuous batching: every running sequence gets its pending tokens (one when decoding, a portion of at most `chunk` tokens of a
    prompt), oldest first, within `max_batch_tokens`; waiting requests are admitted while a state slot and pages are free."""

    def __init__(self, cache: HybridCache, max_batch_tokens: int = 2048, chunk: int = 512):
        self.cache, self.max_batch_tokens, self.chunk = cache, max_batch_tokens, chunk
        self.waiting: deque = deque()
        self.running: List[Request] = []

    def add(self, req: Request) -> None:
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def schedule(self) -> List[Tuple[Request, List[int]]]:
        budget, free = self.max_batch_tokens, self.cache.free_pages()
        batch: List[Tuple[Request, List[int]]] = []

        def take(req: Request) -> bool:
            nonlocal budget, free
            st = self.cache.seqs[req.id]
            room = (len(st.pages) + free) * self.cache.page_size - st.length  # positions the pages that are left can hold
            toks = req.pending()[: max(0, min(self.chunk, budget, room))]
            if not toks:
                return False
            free -= self.cache.pages_needed(req.id, len(toks))
            budget -= len(toks)
            batch.append((req, toks))
            return True

        for req in self.running:
            if budget <= 0:
                break
            take(req)
        while self.waiting and budget > 0 and self.cache.can_admit() and free > 0:
            req = self.waiting.popleft()
            self.cache.admit(req.id)
            self.running.append(req)
            take(req)
        if not batch and self.running:
            raise OutOfPages("no running sequence can advance: the page pool is too small for the live requests")
        return batch

    def retire(self, req: Request) -> None:
        self.running.remove(req)
        self.cache.release(req.id)


class Engine:
    def __init__(self, model: HybridDecoder, max_tokens: int = 4096, max_seqs: int = 4, page_size: int = 64, max_batch_tokens: int = 2048,
                 chunk: int = 512, seed: int = 0, use_graphs: bool = True):
        self.model = model
        # steps that only decode (one token per sequence, none at its first position) replay a CUDA graph captured per batch size: the
        # launches of a step cost more host time than its kernels take
        self.use_graphs = use_graphs
        self._graphs: Dict[int, dict] = {}
        self.cache = model.new_cache(max_tokens, max_seqs, page_size)
        self.scheduler = Scheduler(self.cache, max_batch_tokens, chunk)
        self.generator = torch.Generator(device=model.device)
        self.generator.manual_seed(seed)
        self.steps = 0

    @classmethod
    def from_dir(cls, model_dir: str, dtype: torch.dtype = torch.bfloat16, **kw) -> "Engine":
        return cls(HybridDecoder.from_dir(model_dir, dtype), **kw)

    # ----------------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, entries: Sequence[Tuple[object, Sequence[int], Sequence[int]]], tap=None) -> torch.Tensor:
        """Run one batch: per entry (sequence id, its next tokens, indices among them whose logits are wanted).  A sequence is admitted at
        its first entry.  Returns fp32 logits [wanted, vocab] in entry order."""
        cache = self.cache
        rows, want_rows, r = [], [], 0
        for sid, toks, want in entries:
            if sid not in cache.seqs:
                cache.admit(sid)
            cache.reserve(sid, len(toks))
        for sid, toks, want in entries:
            st = cache.seqs[sid]
            rows.append((st.slot, st.length, st.last_token, list(toks)))
            want_rows += [r + int(w) for w in want]
            r += len(toks)
        table = cache.sync_block_table()
        graphed = self.use_graphs and tap is None and all(len(r[3]) == 1 and r[1] > 0 for r in rows)
        if graphed:
            all_logits = self._decode_step(rows, table)
            graphed = all_logits is not None
        if not graphed:
            x = self.model.forward(StepBatch.build(rows, table, self.model.device, cache.page_size), cache, tap)
        for sid, toks, _ in entries:
            st = cache.seqs[sid]
            st.length += len(toks)
            st.last_token = int(toks[-1])
        self.steps += 1
        if not want_rows:
            return torch.empty((0, self.model.cfg.vocab), dtype=torch.float32, device=self.model.device)
        idx = torch.tensor(want_rows, dtype=torch.int64, device=self.model.device)
        if graphed:
            return all_logits.index_select(0, idx)
        return self.model.logits(x.index_select(0, idx))

    def _decode_step(self, rows, table) -> Optional[torch.Tensor]:
        """Replay (capture at first use) the graph of a decode-only step of len(rows) sequences; returns the logits of all rows, or None if
        capture failed (the step then runs eagerly and graphs stay off)."""
        n, dev = len(rows), self.model.device
        host, sizes = StepBatch.pack(rows)
        g = self._graphs.get(n)
        if g is None:
            g = {"host": torch.empty_like(host).pin_memory(), "dev": torch.empty(host.numel(), dtype=torch.int32, device=dev), "sizes": sizes,
                 "scratch": torch.empty(max(1, self.model.scratch_floats(n)), dtype=torch.float32, device=dev)}
            g["batch"] = StepBatch.view(g["dev"], sizes, table)
            g["host"].copy_(host)
            g["dev"].copy_(g["host"], non_blocking=True)
            graph = torch.cuda.CUDAGraph()
            try:
                torch.cuda.synchronize(dev)
                with torch.cuda.graph(graph):
                    g["logits"] = self.model.logits(self.model.forward(g["batch"], self.cache, None, g["scratch"]))
            except RuntimeError as e:
                print(f"[qserve_b200] CUDA-graph capture of the decode step failed, running eagerly: {e}", file=sys.stderr)
                self.use_graphs = False
                return None
            g["graph"] = graph
            self._graphs[n] = g
        else:
            assert g["sizes"] == sizes
            torch.cuda.current_stream(dev).synchronize()  # the previous replay has consumed the pinned staging copy
            g["host"].copy_(host)
            g["dev"].copy_(g["host"], non_blocking=True)
        g["graph"].replay()
        return g["logits"]

    def release(self, seq_id) -> None:
        self.cache.release(seq_id)

    # ----------------------------------------------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[Sequence[SamplingParams]] = None) -> List[List[int]]:
        """Continuous-batched generation of all prompts; returns the new tokens per prompt."""
        params = list(params) if params is not None else [SamplingParams() for _ in prompts]
        reqs = [Request(("gen", self.steps, i), list(p), params[i]) for i, p in enumerate(prompts)]
        for rq in reqs:
            if not rq.prompt:
                raise ValueError("empty prompt")
            self.scheduler.add(rq)
        while self.scheduler.has_work():
            batch = self.scheduler.schedule()
            entries, samplers = [], []
            for rq, toks in batch:
                last = rq.fed + len(toks) == len(rq.prompt) + len(rq.output)  # the portion ends at the newest token: sample after it
                entries.append((rq.id, toks, [len(toks) - 1] if last else []))
                if last:
                    samplers.append(rq)
            logits = self.step(entries)
            for rq, toks in batch:
                rq.fed += len(toks)
            if samplers:
                nxt = sample(logits, [rq.params for rq in samplers], self.generator).tolist()
                for rq, tok in zip(samplers, nxt):
                    rq.output.append(int(tok))
                    if len(rq.output) >= rq.params.max_new_tokens or tok in rq.params.stop_token_ids:
                        rq.finished = True
                        self.scheduler.retire(rq)
        return [rq.output for rq in reqs]


# --------------------------------------------------------------------------------------------------------------------
def replay_trace(engine: Engine, lines: Iterable[str], out_dir: str, log=sys.stdout) -> int:
    """Feed the batches of a trace through `engine.step`.  One JSON object per line:
    {"step": n, "entries": [{"id": ..., "tokens": [...], "want": [...]}], "end": [ids]}; writes <out_dir>/<n>.f32 (little-endian fp32
    [wanted, vocab]) for steps that want logits, prints `done <n>` after every step."""
    n_steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", []) if e.get("tokens")]
        logits = engine.step(entries) if entries else None
        if logits is not None and logits.shape[0] > 0:
            data = logits.to(torch.float32).cpu().contiguous().numpy().astype("<f4", copy=False).tobytes()
            tmp = os.path.join(out_dir, f".{rec['step']}.f32.part")
            with open(tmp, "wb") as f:
                f.write(data)
            os.replace(tmp, os.path.join(out_dir, f"{rec['step']}.f32"))
        elif logits is not None:
            torch.cuda.synchronize(engine.model.device)
        for sid in rec.get("end", []):
            if sid in engine.cache.seqs:
                engine.release(sid)
        print(f"done {rec['step']}", file=log, flush=True)
        n_steps += 1
    return n_steps
