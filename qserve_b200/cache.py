"""Cache and state manager of the hybrid decoders: one pool of key/value pages shared by all sequences, and a fixed number of
state slots (one per live sequence) for what a recurrent layer carries from token to token.

* Pages hold `page_size` positions.  A sequence owns a list of pages (its block-table row); page ids are valid in every attention layer
  run's K and V pool, as in the reference's block manager (qserve/core/block_manager.py: one block table per sequence, all layers).
* A slot holds, per recurrent layer run, the fp32 state (and, for the delta rule, the convolution's last inputs); the slot index is also the
  block-table row.  Two mixers side by side keep their storage side by side ("left" / "right").
* Released pages and slots go back to LIFO free lists and are handed out again first: nothing is cleared on release, a recurrent layer
  starts a sequence (position 0) from zero by itself and attention never reads beyond a sequence's own length.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List

import torch

from .modelcfg import (AttentionMixerConfig, DeltaMixerConfig, GatedLinearMixerConfig, GateRecurrenceMixerConfig, HybridConfig,
                       LatentAttentionMixerConfig, ParallelMixerConfig, RetentionMixerConfig)


class OutOfPages(RuntimeError):
    pass


class OutOfSlots(RuntimeError):
    pass


class FreeList:
    """LIFO pool of integer ids."""

    def __init__(self, n: int):
        self.n = n
        self._free = list(range(n - 1, -1, -1))

    def __len__(self) -> int:
        return len(self._free)

    def take(self) -> int:
        return self._free.pop()

    def give(self, i: int) -> None:
        assert 0 <= i < self.n and i not in self._free, f"id {i} released twice"
        self._free.append(i)


@dataclass
class SequenceState:
    slot: int
    pages: List[int] = field(default_factory=list)
    length: int = 0          # positions held in the cache / folded into the state
    last_token: int = -1     # previous token (for the pair embedding); -1 before the first


class HybridCache:
    def __init__(self, cfg: HybridConfig, dtype: torch.dtype, device: torch.device, max_tokens: int, max_seqs: int = 4, page_size: int = 64):
        self.cfg, self.dtype, self.device, self.page_size, self.max_seqs = cfg, dtype, device, page_size, max_seqs
        self.num_pages = max(1, -(-max_tokens // page_size))
        self.pages = FreeList(self.num_pages)
        self.slots = FreeList(max_seqs)
        self.seqs: Dict[object, SequenceState] = {}
        self.max_blocks = self.num_pages  # one sequence may hold the whole pool
        self.block_table_host = torch.zeros((max_seqs, self.max_blocks), dtype=torch.int32).pin_memory() if device.type == "cuda" else \
            torch.zeros((max_seqs, self.max_blocks), dtype=torch.int32)
        self.block_table = torch.zeros((max_seqs, self.max_blocks), dtype=torch.int32, device=device)
        self._table_dirty = True
        # per layer RUN (a looped layer has one cache / state per pass)
        self.runs = [self.mixer_storage(cfg.layers[li].mixer) for li in cfg.schedule()]

    def mixer_storage(self, m) -> dict:
        """What one run of a mixer keeps between steps: pages for an attention layer (keys and values, or the latent rows of a latent
        attention), a slot-indexed fp32 state for a recurrent one, both (under "left" / "right") for two mixers side by side."""
        dtype, device, page_size, max_seqs = self.dtype, self.device, self.page_size, self.max_seqs
        if isinstance(m, AttentionMixerConfig):
            return {"k": torch.zeros((self.num_pages, page_size, m.kv_heads, m.maps * m.dim), dtype=dtype, device=device),
                    "v": torch.zeros((self.num_pages, page_size, m.kv_heads, m.vdim), dtype=dtype, device=device)}
        if isinstance(m, LatentAttentionMixerConfig):
            # one row per position for all heads: the key/value latent and the rotated key part they share
            return {"c": torch.zeros((self.num_pages, page_size, m.kv_rank + m.rot_dim), dtype=dtype, device=device)}
        if isinstance(m, DeltaMixerConfig):
            c = 2 * m.kv_heads * m.dim + m.heads * m.vdim
            return {"state": torch.zeros((max_seqs, m.heads, m.dim, m.vdim), dtype=torch.float32, device=device),
                    "conv": torch.zeros((max_seqs, max(m.conv - 1, 1), c), dtype=torch.float32, device=device)}
        if isinstance(m, (GateRecurrenceMixerConfig, RetentionMixerConfig, GatedLinearMixerConfig)):
            return {"state": torch.zeros((max_seqs, m.heads, m.dim, m.vdim), dtype=torch.float32, device=device)}
        if isinstance(m, ParallelMixerConfig):
            return {"left": self.mixer_storage(m.left), "right": self.mixer_storage(m.right)}
        raise TypeError(type(m))

    # ----------------------------------------------------------------------------------------------------------------
    def admit(self, seq_id) -> SequenceState:
        if seq_id in self.seqs:
            raise KeyError(f"sequence {seq_id!r} is already live")
        if not len(self.slots):
            raise OutOfSlots(f"all {self.max_seqs} state slots are in use")
        st = SequenceState(slot=self.slots.take())
        self.seqs[seq_id] = st
        return st

    def can_admit(self) -> bool:
        return len(self.slots) > 0

    def pages_needed(self, seq_id, new_tokens: int) -> int:
        st = self.seqs[seq_id]
        return max(0, -(-(st.length + new_tokens) // self.page_size) - len(st.pages))

    def reserve(self, seq_id, new_tokens: int) -> None:
        """Make room for `new_tokens` more positions of the sequence."""
        st = self.seqs[seq_id]
        need = self.pages_needed(seq_id, new_tokens)
        if need > len(self.pages):
            raise OutOfPages(f"{need} pages needed, {len(self.pages)} of {self.num_pages} free")
        for _ in range(need):
            p = self.pages.take()
            self.block_table_host[st.slot, len(st.pages)] = p
            st.pages.append(p)
            self._table_dirty = True

    def release(self, seq_id) -> None:
        st = self.seqs.pop(seq_id)
        for p in reversed(st.pages):
            self.pages.give(p)
        self.slots.give(st.slot)

    def sync_block_table(self) -> torch.Tensor:
        if self._table_dirty:
            self.block_table.copy_(self.block_table_host)  # blocking: the host table changes again before the next step
            self._table_dirty = False
        return self.block_table

    def free_pages(self) -> int:
        return len(self.pages)
