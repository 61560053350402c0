"""Block-paged KV caches whose decode-step device work runs on this library's
kernels — the host-side mirror of the reference's cache layer.

    KVCacheSpec        cache/kv_cache.py:71-109         (fields used by the paged caches)
    BlockAllocator     cache/block_allocator.py:40-162  (LIFO free list, reference counts)
    BlockTable         cache/block_allocator.py:165-229 (blocks, length, version)
    PagedKVCache       cache/paged_cache.py:57-566      (fp16 pools, page bounds)
    Int8PagedKVCache   cache/int8_paged_cache.py:143-1028 (int8 pools, fp32 scales,
                       fp16 K residual, deferred finalize)

Same storage layout (`[num_blocks, 16, H, D]` pools per layer, `[max_batch,
max_pages]` int32 block tables at capacity width, persistent decode buffers
whose addresses never change), same call order (`advance` outside a captured
graph, `write` and attention inside), same invariants (every K page but a
sequence's last is in the INT8 pool, the last is exact in the residual;
shared prefix blocks are full and read-only).

What is different is the hot part: `write()` for one token per sequence is one
launch (`ls_kv_append_fp16` / `ls_int8_decode_write`), INT8 page finalisation
is one launch per layer (`ls_int8_finalize_blocks`) instead of a dozen torch
ops, and `advance()` stages the step's indices and new block ids in pinned host
memory and ships them with one copy. Prefill writes (more than one token per
sequence) are set-up, not the hot path; they reuse the same kernels row by row.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from latentserve_b200 import fused_elementwise as fe
from latentserve_b200 import int8_write as iw
from latentserve_b200 import kv_write

_EPS = 1e-8


class OutOfBlocks(RuntimeError):
    """The pool cannot supply the blocks asked for: backpressure, not a crash."""


@dataclass
class KVCacheSpec:
    num_layers: int
    num_kv_heads: int
    head_dim: int
    max_seq_len: int
    max_batch_size: int
    dtype: torch.dtype = torch.float16
    device: str = "cuda"


class BlockAllocator:
    """Fixed pool of block ids with reference counts; most recently freed
    block is handed out first."""

    def __init__(self, num_blocks: int, block_size: int):
        if num_blocks <= 0 or block_size <= 0:
            raise ValueError("num_blocks and block_size must be positive")
        self.num_blocks, self.block_size = num_blocks, block_size
        self._free = list(range(num_blocks - 1, -1, -1))
        self._refs = [0] * num_blocks

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_blocks - len(self._free)

    def blocks_for_tokens(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_size)

    def allocate(self, n: int) -> list[int]:
        if n > len(self._free):
            raise OutOfBlocks(f"need {n} blocks, {len(self._free)} free of {self.num_blocks}")
        out = [self._free.pop() for _ in range(n)]
        for b in out:
            self._refs[b] = 1
        return out

    def incref(self, blocks) -> None:
        for b in blocks:
            if self._refs[b] <= 0:
                raise ValueError(f"increfing block {b} that is not allocated")
            self._refs[b] += 1

    def free(self, blocks) -> None:
        for b in blocks:
            if self._refs[b] <= 0:
                raise ValueError(f"freeing block {b} that is not allocated")
            self._refs[b] -= 1
            if self._refs[b] == 0:
                self._free.append(b)

    def ref_count(self, block: int) -> int:
        return self._refs[block]

    def reset(self) -> None:
        self._free = list(range(self.num_blocks - 1, -1, -1))
        self._refs = [0] * self.num_blocks


class BlockTable:
    """One sequence: its physical blocks in logical order, its length, and a
    version that changes whenever the block list does."""

    def __init__(self, allocator: BlockAllocator):
        self.allocator = allocator
        self.blocks: list[int] = []
        self.length = 0
        self.version = 0

    def append(self, num_tokens: int) -> None:
        need = self.allocator.blocks_for_tokens(self.length + num_tokens) - len(self.blocks)
        if need > 0:
            self.blocks.extend(self.allocator.allocate(need))
            self.version += 1
        self.length += num_tokens

    def slot(self, position: int) -> int:
        if not 0 <= position < self.length:
            raise IndexError(f"position {position} beyond length {self.length}")
        bs = self.allocator.block_size
        return self.blocks[position // bs] * bs + position % bs

    def free(self) -> None:
        self.allocator.free(self.blocks)
        self.blocks, self.length = [], 0
        self.version += 1


class _PagedBase:
    """Bookkeeping shared by the two caches: tables, active set, and the
    persistent device buffers a decode step reads."""

    def __init__(self, spec: KVCacheSpec, block_size: int, num_blocks: Optional[int]):
        if block_size != 16 or spec.head_dim != 128:
            raise ValueError("the sm_100a kernels need block_size 16 and head_dim 128")
        self.spec, self.block_size = spec, block_size
        self.device = torch.device(spec.device)
        if self.device.type != "cuda":
            raise RuntimeError("latentserve_b200 caches live on a CUDA device; there is no CPU path")
        per_seq = -(-spec.max_seq_len // block_size)
        self.num_blocks = num_blocks if num_blocks is not None else per_seq * spec.max_batch_size
        self.allocator = BlockAllocator(self.num_blocks, block_size)
        mb = spec.max_batch_size
        self.tables = [BlockTable(self.allocator) for _ in range(mb)]
        self._active = list(range(mb))
        self._active_range: Optional[int] = None       # n when the active set is known to be range(n)
        self._decode_slots: list = []
        self._capacity_pages = max(1, per_seq)
        dev = self.device
        # The tables, flat, with one spare element behind them: the slot a step's table
        # patches of sequences that gained no block are aimed at (see _grow).
        self._block_tables_flat = torch.zeros(mb * self._capacity_pages + 16, dtype=torch.int32, device=dev)
        self._block_tables_buf = self._block_tables_flat[: mb * self._capacity_pages].view(mb, self._capacity_pages)
        self._patches: list = []                    # (row, page, block) gained by this advance()
        # Everything a decode step ships lives in ONE device buffer -- lengths and residual
        # rows (int32), write slots, residual slots and the pages to finalise (int64), and the
        # blocks the sequences gained this step as patches of their table rows (whole rows
        # are copied only when a slot changes hands) -- of which the kernels' inputs are typed views, filled by one
        # asynchronous copy per advance() from one of two pinned host images (the
        # reference makes several small blocking copies per step,
        # cache/paged_cache.py:252-273,337-360). An event per image keeps the host from
        # rewriting an image whose copy has not run yet.
        off_i64 = -(-(8 * mb) // 16) * 16
        off_state = off_i64 + 32 * mb               # int32 [4]: pages to finalise, arrivals, padding
        off_patch = off_state + 16                  # int64 [mb] flat table indices, then int32 [mb] block ids
        self._step_bytes = off_patch + 12 * mb
        self._step_dev = torch.zeros(self._step_bytes, dtype=torch.uint8, device=dev)

        def views(buf):
            return (buf[: 4 * mb].view(torch.int32), buf[4 * mb: 8 * mb].view(torch.int32),
                    buf[off_i64: off_i64 + 8 * mb].view(torch.int64),
                    buf[off_i64 + 8 * mb: off_i64 + 16 * mb].view(torch.int64),
                    buf[off_i64 + 16 * mb: off_i64 + 24 * mb].view(torch.int64),
                    buf[off_i64 + 24 * mb: off_i64 + 32 * mb].view(torch.int64),
                    buf[off_state: off_state + 16].view(torch.int32),
                    buf[off_patch: off_patch + 8 * mb].view(torch.int64),
                    buf[off_patch + 8 * mb: off_patch + 12 * mb].view(torch.int32))

        (self._seq_lens_buf, self._res_rows_buf, slots_dev, self._k_res_idx_buf, self._fin_rows_buf,
         self._fin_ids_buf, self._fin_state_buf, self._patch_idx_buf, self._patch_val_buf) = views(self._step_dev)
        self._write_slots_buf = slots_dev.view(mb, 1)
        self._step_host = [torch.zeros(self._step_bytes, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self._step_np = [tuple(v.numpy() for v in views(h)) for h in self._step_host]
        self._step_events: list = [None, None]
        self._step_next, self._step_open = 0, None
        self._table_state: list = [None] * mb
        self._block_tables = self._seq_lens_tensor = self._write_slots = None
        self._prefill_slots: Optional[torch.Tensor] = None
        self._decode_slot_vec: Optional[torch.Tensor] = None      # [b] view of the decode slots

    # -- state ---------------------------------------------------------
    @property
    def seq_lens(self) -> list[int]:
        return [self.tables[i].length for i in self._active]

    @property
    def max_len(self) -> int:
        return max((self.tables[i].length for i in self._active), default=0)

    def active_slots(self) -> list[int]:
        return list(self._active)

    def set_active(self, slots: Sequence[int]) -> None:
        slots = list(slots)
        self._active_range = None
        if len(set(slots)) != len(slots) or any(not 0 <= s < len(self.tables) for s in slots):
            raise ValueError(f"bad active set {slots}")
        self._active = slots

    def can_admit(self, num_tokens: int) -> bool:
        return self.allocator.blocks_for_tokens(num_tokens) <= self.allocator.num_free

    def free_sequence(self, index: int) -> None:
        self.tables[index].free()

    def attach_prefix(self, index: int, blocks: Sequence[int], num_tokens: int) -> None:
        """Start sequence `index` on already-written, full, shared blocks."""
        table = self.tables[index]
        if table.length or table.blocks:
            raise ValueError(f"slot {index} is not empty")
        if num_tokens != len(blocks) * self.block_size:
            raise ValueError("a cached prefix is a whole number of full blocks")
        self.allocator.incref(blocks)
        table.blocks, table.length = list(blocks), num_tokens
        table.version += 1

    def block_tables_tensor(self, batch_size: Optional[int] = None) -> torch.Tensor:
        if self._block_tables is None:
            raise RuntimeError("call advance() before block_tables_tensor()")
        return self._block_tables if batch_size is None else self._block_tables[:batch_size]

    def seq_lens_tensor(self, batch_size: Optional[int] = None) -> torch.Tensor:
        if self._seq_lens_tensor is None:
            raise RuntimeError("call advance() before seq_lens_tensor()")
        return self._seq_lens_tensor if batch_size is None else self._seq_lens_tensor[:batch_size]

    # -- per-step staging ------------------------------------------------
    def _activate(self, batch_size, slots) -> None:
        """`set_active` for advance(): skipped when the request is the active set already
        (every step of a steady decode loop)."""
        if slots is not None:
            if list(slots) != self._active:
                self.set_active(slots)
        elif batch_size is not None:
            if self._active_range != batch_size:
                self.set_active(range(batch_size))
                self._active_range = batch_size

    def _grow(self, n: int, batch_size, slots):
        self._activate(batch_size, slots)
        active = self._active
        if n == 1:
            # One pass: previous length, a new block where the token opens a page, the
            # token's flat slot.
            bs, tables, alloc = self.block_size, self.tables, self.allocator
            starts, slot_list = [], []
            state, cap, patches = self._table_state, self._capacity_pages, self._patches
            for row, i in enumerate(active):
                t = tables[i]
                length, blocks = t.length, t.blocks
                need = -(-(length + 1) // bs) - len(blocks)
                if need > 0:
                    # A sequence whose row on the device is current gains its block as a
                    # patch of that row (one entry of the step's staging copy) instead of
                    # a copy of the whole row.
                    current = need == 1 and state[row] == (i, t.version) and len(blocks) < cap
                    try:
                        got = alloc.allocate(need)
                    except OutOfBlocks:
                        # Rows patched so far go back to a whole-row copy next time.
                        for prow, _, _ in patches:
                            state[prow] = None
                        patches.clear()
                        raise
                    blocks.extend(got)
                    t.version += 1
                    if current:
                        patches.append((row, len(blocks) - 1, blocks[-1]))
                        state[row] = (i, t.version)
                slot_list.append(blocks[length // bs] * bs + length % bs)
                t.length = length + 1
                starts.append(length)
            self._decode_slots = slot_list
            return active, starts
        starts = [self.tables[i].length for i in active]
        for i in active:
            self.tables[i].append(n)
        return active, starts

    def _ship_tables(self, active: list[int]) -> None:
        """Block-table rows that changed, and every active length."""
        for row, i in enumerate(active):
            t = self.tables[i]
            state = (i, t.version)
            if self._table_state[row] != state:
                if len(t.blocks) > self._capacity_pages:
                    for prow, _, _ in self._patches:     # unshipped: whole-row copies next time
                        self._table_state[prow] = None
                    self._patches.clear()
                    raise RuntimeError(f"sequence in slot {i} needs {len(t.blocks)} pages, past the "
                                       f"cache's capacity of {self._capacity_pages}")
                if t.blocks:
                    # A fresh (pageable) host row each time, so the copy completes on the
                    # host before the row can change: only rows whose block list changed.
                    src = torch.tensor(t.blocks, dtype=torch.int32)
                    self._block_tables_buf[row, : len(t.blocks)].copy_(src)
                self._table_state[row] = state
        b = len(active)
        stage = self._stage()
        stage[0][:b] = [self.tables[i].length for i in active]
        patches = self._patches
        if patches:
            # Rows without a patch aim at the spare element behind the tables.
            cap = self._capacity_pages
            stage[7][:b] = len(self.tables) * cap
            for row, page, blk in patches:
                stage[7][row] = row * cap + page
                stage[8][row] = blk
        self._flush_stage()
        if patches:
            # Behind the staging copy on the stream, ahead of the step's kernels.
            self._block_tables_flat.index_copy_(0, self._patch_idx_buf[:b], self._patch_val_buf[:b])
            patches.clear()
        self._block_tables = self._block_tables_buf[:b]
        self._seq_lens_tensor = self._seq_lens_buf[:b]

    def _stage(self):
        """Host image being filled for this advance(): numpy views (lens, res_rows,
        slots, res_idx, fin_rows, fin_ids, fin_state, patch_idx, patch_val). Opened on first use; starts as a copy of the last one shipped,
        so fields an advance() does not touch keep their values."""
        if self._step_open is None:
            i = self._step_next
            if self._step_events[i] is not None:
                self._step_events[i].synchronize()
            self._step_host[i].copy_(self._step_host[1 - i])
            self._step_open = i
        return self._step_np[self._step_open]

    def _flush_stage(self) -> None:
        i = self._step_open
        if i is None:
            return
        self._step_dev.copy_(self._step_host[i], non_blocking=True)
        if self._step_events[i] is None:
            self._step_events[i] = torch.cuda.Event()
        self._step_events[i].record()
        self._step_next, self._step_open = 1 - i, None

    def _slot_vec(self, slots: torch.Tensor, b: int) -> torch.Tensor:
        """The first b decode slots as a vector (the view made once per advance)."""
        vec = self._decode_slot_vec
        if vec is not None and slots is self._write_slots and vec.shape[0] >= b:
            return vec
        return slots[:b, 0]

    def _ship_decode_slots(self, active, starts) -> None:
        b = len(active)
        self._stage()[2][:b] = self._decode_slots          # computed by _grow
        self._write_slots = self._write_slots_buf[:b]
        self._decode_slot_vec = self._write_slots_buf[:b, 0]


class PagedKVCache(_PagedBase):
    """fp16 block-paged KV cache."""

    def __init__(self, spec: KVCacheSpec, block_size: int = 16, num_blocks: Optional[int] = None):
        super().__init__(spec, block_size, num_blocks)
        shape = (self.num_blocks, block_size, spec.num_kv_heads, spec.head_dim)
        self.k_pool = [torch.zeros(shape, dtype=spec.dtype, device=self.device)
                       for _ in range(spec.num_layers)]
        self.v_pool = [torch.zeros(shape, dtype=spec.dtype, device=self.device)
                       for _ in range(spec.num_layers)]
        self._flat_k = [t.view(-1, spec.num_kv_heads, spec.head_dim) for t in self.k_pool]
        self._flat_v = [t.view(-1, spec.num_kv_heads, spec.head_dim) for t in self.v_pool]
        self._bounds_on = False
        self.kmin: list = []
        self.kmax: list = []
        self.fused_append = False

    def enable_fused_append(self) -> None:
        """Let a decode step's append ride on the attention launch: `write()` of one
        token per sequence launches nothing and leaves the rows for the next
        `paged_decode_attention` call on that layer's pools, whose kernel takes the
        newest row from them and stores them to the pools (`ls_paged_decode_append_fp16`):
        one launch per layer instead of two. For callers that follow every `write()`
        with the layer's attention call, as `GQAAttention.forward` does
        (model/attention/gqa.py:267, 283-344); rows nobody attended are appended by the
        next `advance()`. Not used while page bounds are kept (the sparse indexer needs
        the append kernel's bounds update)."""
        self.fused_append = True

    def _flush_deferred_appends(self) -> None:
        from latentserve_b200 import paged_decode as pd

        if not self.fused_append:
            return
        for layer, pool in enumerate(self.k_pool):
            pending = pd.take_pending_append(pool)
            if pending is not None and self._write_slots is not None:
                k, v = pending
                kv_write.append_fp16(k, v, self._slot_vec(self._write_slots, k.shape[0]), self._flat_k[layer],
                                     self._flat_v[layer], None, None, self.block_size)

    def reset(self) -> None:
        """Free every sequence; storage and buffer addresses stay."""
        for t in self.tables:
            if t.blocks:
                t.free()
        self._table_state = [None] * len(self.tables)
        self._patches.clear()
        self._active = list(range(len(self.tables)))
        self._active_range = None

    def shareable_blocks(self, index: int) -> int:
        return self.tables[index].length // self.block_size

    def advance(self, n: int, batch_size: Optional[int] = None,
                slots: Optional[Sequence[int]] = None) -> None:
        self._flush_deferred_appends()              # rows of the last step nobody attended
        active, starts = self._grow(n, batch_size, slots)
        if n == 1:
            self._ship_decode_slots(active, starts)
            self._prefill_slots = None
        else:
            self._prefill_slots = torch.tensor(
                [[self.tables[i].slot(p) for p in range(s, s + n)] for i, s in zip(active, starts)],
                dtype=torch.int64, device=self.device)
            self._write_slots = self._prefill_slots
            self._decode_slot_vec = None
        self._ship_tables(active)

    def write(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor, start_pos: int = 0) -> None:
        """k, v [B, kv_heads, n, head_dim] -> the pools, at the slots `advance` reserved."""
        b, h, n, d = k.shape
        slots = self._write_slots
        if slots is None or slots.shape[0] < b or slots.shape[1] != n:
            raise RuntimeError("call advance(n, batch_size) before write()")
        kmin = self.kmin[layer_idx] if self._bounds_on else None
        kmax = self.kmax[layer_idx] if self._bounds_on else None
        if n == 1:
            if self.fused_append and not self._bounds_on and b == len(self._active):
                from latentserve_b200 import paged_decode as pd
                from latentserve_b200 import paged_decode_cuda as pdc

                if pdc.append_rows_ok(k, v, k):
                    pd.defer_append(self.k_pool[layer_idx], k, v)
                    return
            kv_write.append_fp16(k, v, self._slot_vec(slots, b), self._flat_k[layer_idx],
                                 self._flat_v[layer_idx], kmin, kmax, self.block_size)
            return
        # Prefill: the same kernel, one launch per position (bounds stay exact
        # because positions are written in order).
        for j in range(n):
            kv_write.append_fp16(k[:, :, j], v[:, :, j], slots[:b, j].contiguous(),
                                 self._flat_k[layer_idx], self._flat_v[layer_idx], kmin, kmax,
                                 self.block_size)

    def rope_write(self, layer_idx: int, qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                   positions: torch.Tensor, q_out: torch.Tensor, q_heads: int) -> None:
        """One decode token per sequence, from the fused QKV projection row: rotate
        q into `q_out`, rotate k and append it with v at the slots `advance(1)`
        reserved (and update the page bounds) — one launch."""
        b = qkv.shape[0]
        slots = self._write_slots
        if slots is None or slots.shape[0] < b or slots.shape[1] != 1:
            raise RuntimeError("call advance(1, batch_size) before rope_write()")
        kmin = self.kmin[layer_idx] if self._bounds_on else None
        kmax = self.kmax[layer_idx] if self._bounds_on else None
        fe.rope_append_fp16(qkv, cos, sin, positions, self._slot_vec(slots, b), q_out, self._flat_k[layer_idx],
                            self._flat_v[layer_idx], kmin, kmax, q_heads, self.spec.num_kv_heads,
                            self.block_size)

    def qkv_rope_write(self, layer_idx: int, x: torch.Tensor, w: torch.Tensor, bias, cos: torch.Tensor,
                       sin: torch.Tensor, positions: torch.Tensor, q_out: torch.Tensor, q_heads: int, *,
                       norm_weight=None, row_sumsq=None, eps: float = 1e-6) -> None:
        """`rope_write` with the fused QKV projection in front of it, in one launch
        (decode batches of up to 32 rows): x [B, hidden] is (normalised and)
        multiplied by w [(q_heads + 2 kv_heads) * 128, hidden] + bias, then rotated
        and appended exactly as `rope_write` does with the projection's output."""
        from latentserve_b200 import projections as pj

        b = x.shape[0]
        slots = self._write_slots
        if slots is None or slots.shape[0] < b or slots.shape[1] != 1:
            raise RuntimeError("call advance(1, batch_size) before qkv_rope_write()")
        kmin = self.kmin[layer_idx] if self._bounds_on else None
        kmax = self.kmax[layer_idx] if self._bounds_on else None
        pj.qkv_rope_append(x, w, bias, cos, sin, positions, self._slot_vec(slots, b), q_out,
                           self._flat_k[layer_idx], self._flat_v[layer_idx], kmin, kmax, q_heads,
                           self.spec.num_kv_heads, norm_weight=norm_weight, row_sumsq=row_sumsq, eps=eps)

    def rewind(self, length: int, slots: Optional[Sequence[int]] = None) -> None:
        """Shorten the active sequences (or `slots`) back to `length` tokens, keeping
        their blocks: growing again reuses the same blocks and slots and overwrites the
        tokens past `length` (cache/paged_cache.py:275-303 in the reference). The page the
        rewind lands in gets its bounds recomputed over the rows that remain. Host-side
        set-up, not the hot path: the next `advance()` ships the new lengths."""
        bs = self.block_size
        for i in (self._active if slots is None else slots):
            table = self.tables[i]
            if not 0 <= length <= table.length:
                raise ValueError(f"cannot rewind slot {i} from {table.length} to {length}")
            table.length = length
            if self._bounds_on and length % bs:
                blk, rows = table.blocks[length // bs], length % bs
                for layer in range(len(self.k_pool)):
                    self.kmin[layer][blk] = self.k_pool[layer][blk, :rows].amin(dim=0)
                    self.kmax[layer][blk] = self.k_pool[layer][blk, :rows].amax(dim=0)
        if self._block_tables is not None:                  # lengths as the kernels see them
            active = self._active
            self._stage()[0][:len(active)] = [self.tables[i].length for i in active]
            self._flush_stage()

    def enable_page_bounds(self) -> None:
        """Keep each block's per-channel min / max of K for the sparse indexer.
        Bounds of blocks already written are rebuilt over their written rows."""
        if self._bounds_on:
            return
        nb, _, h, d = self.k_pool[0].shape
        self.kmin = [torch.zeros(nb, h, d, dtype=self.spec.dtype, device=self.device)
                     for _ in self.k_pool]
        self.kmax = [torch.zeros_like(t) for t in self.kmin]
        self._bounds_on = True
        bs = self.block_size
        # Whole pool at once over all 16 rows, then the partly filled last page
        # of each sequence again over its written rows only.
        partial = [(t.blocks[(t.length - 1) // bs], t.length - (t.length - 1) // bs * bs)
                   for t in self.tables if t.length % bs]
        for layer in range(len(self.k_pool)):
            self.kmin[layer].copy_(self.k_pool[layer].amin(dim=1))
            self.kmax[layer].copy_(self.k_pool[layer].amax(dim=1))
            for blk, rows in partial:
                self.kmin[layer][blk] = self.k_pool[layer][blk, :rows].amin(dim=0)
                self.kmax[layer][blk] = self.k_pool[layer][blk, :rows].amax(dim=0)

    def page_bounds(self, layer_idx: int):
        return (self.kmin[layer_idx], self.kmax[layer_idx]) if self._bounds_on else None


class Int8PagedKVCache(_PagedBase):
    """INT8 block-paged KV cache: V quantised per (token, head) on write; K
    quantised per (block, head, channel) when its 16-token page completes, the
    still-filling page held exact in an fp16 residual per sequence slot."""

    def __init__(self, spec: KVCacheSpec, block_size: int = 16, num_blocks: Optional[int] = None,
                 asymmetric: bool = False):
        super().__init__(spec, block_size, num_blocks)
        nb, h, d, mb = self.num_blocks, spec.num_kv_heads, spec.head_dim, spec.max_batch_size
        dev, layers = self.device, range(spec.num_layers)
        self.asymmetric = asymmetric
        self.k_qmax = self.v_qmax = 127
        self.k_levels = self.v_levels = 255
        self.k_offset = self.v_offset = 128
        # K side: one tensor per kind with the layers stacked (the per-layer tensors the
        # kernels take are its slices), so a completed page is finalised in every layer by
        # one launch.
        nl = spec.num_layers
        self._k_pool_all = torch.zeros(nl, nb, block_size, h, d, dtype=torch.int8, device=dev)
        self._k_scale_all = torch.ones(nl, nb, h, d, dtype=torch.float32, device=dev)
        self._k_zero_all = torch.zeros(nl, nb, h, d, dtype=torch.float32, device=dev) if asymmetric else None
        self.k_pool = [self._k_pool_all[i] for i in layers]
        self.v_pool = [torch.zeros(nb, block_size, h, d, dtype=torch.int8, device=dev) for _ in layers]
        self.k_scale_pool = [self._k_scale_all[i] for i in layers]
        self.v_scale_pool = [torch.ones(nb, block_size, h, dtype=torch.float32, device=dev)
                             for _ in layers]
        self.k_zero_pool = [self._k_zero_all[i] for i in layers] if asymmetric else []
        self.v_zero_pool = [torch.zeros_like(t) for t in self.v_scale_pool] if asymmetric else []
        self._flat_v = [t.view(-1, h, d) for t in self.v_pool]
        self._flat_v_scale = [t.view(-1, h) for t in self.v_scale_pool]
        self._flat_v_zero = [t.view(-1, h) for t in self.v_zero_pool]
        self._k_res_all = torch.zeros(nl, mb, block_size, h, d, dtype=spec.dtype, device=dev)
        self._k_residual = [self._k_res_all[i] for i in layers]
        self._k_res_flat = [r.view(mb * block_size, h, d) for r in self._k_residual]
        self._res_rows = None
        self._bounds_on = False         # page bounds of the exact fp16 K, for INT8 + sparse (an extension)
        self.kmin: list = []
        self.kmax: list = []
        self._fin = [0] * mb            # K pages already quantised, per slot (all layers at once)
        self.deferred_finalize = True   # the only mode: a page is finalised in the step after it filled up
        self.finalize_in_step = False   # see enable_finalize_in_step()

    def reset(self) -> None:
        for t in self.tables:
            if t.blocks:
                t.free()
        self._table_state = [None] * len(self.tables)
        self._patches.clear()
        self._active = list(range(len(self.tables)))
        self._active_range = None
        self._fin = [0] * len(self.tables)

    def free_sequence(self, index: int) -> None:
        super().free_sequence(index)
        self._fin[index] = 0

    def shareable_blocks(self, index: int) -> int:
        """Full blocks whose K is final in the pool (quantised), safe to share."""
        return self._fin[index]

    def attach_prefix(self, index: int, blocks: Sequence[int], num_tokens: int) -> None:
        super().attach_prefix(index, blocks, num_tokens)
        self._fin[index] = len(blocks)

    def residual(self, layer_idx: int) -> torch.Tensor:
        return self._k_residual[layer_idx]

    def enable_page_bounds(self) -> None:
        """Keep each block's per-channel min / max of the exact fp16 K (as the fp16
        cache does) so that the sparse indexer can run over an INT8 cache. Must be
        switched on while the cache is empty: finalised pages no longer hold exact K."""
        if self._bounds_on:
            return
        if any(t.length for t in self.tables):
            raise RuntimeError("enable_page_bounds() on an INT8 cache must precede the first write")
        nb, _, h, d = self.k_pool[0].shape
        self.kmin = [torch.zeros(nb, h, d, dtype=self.spec.dtype, device=self.device)
                     for _ in range(self.spec.num_layers)]
        self.kmax = [torch.zeros_like(t) for t in self.kmin]
        self._bounds_on = True

    def page_bounds(self, layer_idx: int):
        return (self.kmin[layer_idx], self.kmax[layer_idx]) if self._bounds_on else None

    def residual_rows_tensor(self, batch_size: Optional[int] = None) -> torch.Tensor:
        if self._res_rows is None:
            raise RuntimeError("residual rows exist only after a decode advance(1)")
        return self._res_rows if batch_size is None else self._res_rows[:batch_size]

    def _quant_consts(self) -> dict:
        return dict(eps=_EPS, qmax=float(self.k_qmax), levels=float(self.k_levels),
                    offset=float(self.k_offset))

    def _collect_pending(self, seqs: Sequence[int]) -> int:
        """The page each of `seqs` completed since its last finalisation (at most one
        per sequence: the residual holds one) into the step's staging image; returns
        how many there are. `_launch_finalize` quantises them, in every layer, once
        the image is on the device."""
        bs = self.block_size
        rows, ids = [], []
        for s in seqs:
            done = self.tables[s].length // bs
            pending = done - self._fin[s]
            if pending <= 0:
                continue
            if pending > 1:
                raise RuntimeError(f"sequence in slot {s} has {pending} unquantized blocks; the "
                                   "residual holds one, so the earlier ones are already lost")
            rows.append(s)
            ids.append(self.tables[s].blocks[done - 1])
            self._fin[s] = done
        if rows:
            stage = self._stage()
            stage[4][: len(rows)] = rows
            stage[5][: len(rows)] = ids
        return len(rows)

    def _launch_finalize(self, count: int) -> None:
        iw.finalize_layers(self._k_res_all, self._fin_rows_buf, self._fin_ids_buf, count,
                           self._k_pool_all, self._k_scale_all, self._k_zero_all,
                           **self._quant_consts())

    def enable_finalize_in_step(self) -> None:
        """Move page finalisation out of `advance()` and into the step itself: the
        first write of a step (`write` / `rope_write` for layer 0) starts with one
        launch of a fixed grid that finalises, in every layer, the pages `advance()`
        listed in the staged image -- their number is read on the device -- before
        anything overwrites the residual. `advance()` then launches nothing: its
        device work is the one staged copy. Meant for a captured decode step (the
        launch becomes the graph's first INT8 node); the reference runs these ops
        eagerly in `advance()`, between replays (cache/int8_paged_cache.py:443-446).
        Contract of this mode: every `advance()` is followed by a step that writes
        layer 0 before the next `advance()` -- what a decode loop does. The kernel
        consumes the list once, so replaying a step without a new `advance()` is
        harmless."""
        self.finalize_in_step = True

    def _finalize_in_step(self) -> None:
        iw.finalize_pending(self._k_res_all, self._fin_rows_buf, self._fin_ids_buf, self._fin_state_buf,
                            self._k_pool_all, self._k_scale_all, self._k_zero_all,
                            **self._quant_consts())

    def advance(self, n: int, batch_size: Optional[int] = None,
                slots: Optional[Sequence[int]] = None) -> None:
        self._activate(batch_size, slots)
        # Pages completed by the previous step are still whole in the residual: they are
        # quantised below, after this step's staging copy and before anything writes the
        # residual again.
        pending = self._collect_pending(self._active)
        active, starts = self._grow(n, None, None)
        self._starts = starts
        if n == 1:
            b, bs = len(active), self.block_size
            self._ship_decode_slots(active, starts)
            stage = self._stage()
            stage[3][:b] = [i * bs + st % bs for i, st in zip(active, starts)]
            stage[1][:b] = active
            self._res_rows = self._res_rows_buf[:b]
            self._prefill_slots = None
        else:
            self._prefill_slots = torch.tensor(
                [[self.tables[i].slot(p) for p in range(s, s + n)] for i, s in zip(active, starts)],
                dtype=torch.int64, device=self.device)
            self._write_slots = self._prefill_slots
            self._decode_slot_vec = None
        if self.finalize_in_step:
            state = self._stage()[6]
            state[0], state[1] = pending, 0
        self._ship_tables(active)
        if not self.finalize_in_step:
            self._launch_finalize(pending)

    def rope_write(self, layer_idx: int, qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                   positions: torch.Tensor, q_out: torch.Tensor, q_heads: int) -> None:
        """As PagedKVCache.rope_write: rotated q out, rotated K into the residual,
        V quantised on write, one launch."""
        b = qkv.shape[0]
        slots = self._write_slots
        if slots is None or slots.shape[0] < b or slots.shape[1] != 1:
            raise RuntimeError("call advance(1, batch_size) before rope_write()")
        if self.finalize_in_step and layer_idx == 0:
            self._finalize_in_step()
        fe.rope_append_int8(qkv, cos, sin, positions, self._slot_vec(slots, b), self._k_res_idx_buf[:b], q_out,
                            self._flat_v[layer_idx], self._flat_v_scale[layer_idx],
                            self._flat_v_zero[layer_idx] if self.asymmetric else None,
                            self._k_res_flat[layer_idx], q_heads, self.spec.num_kv_heads,
                            asym=self.asymmetric, eps=_EPS, qmax=float(self.v_qmax),
                            levels=float(self.v_levels), offset=float(self.v_offset),
                            kmin=self.kmin[layer_idx] if self._bounds_on else None,
                            kmax=self.kmax[layer_idx] if self._bounds_on else None)

    def write(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor, start_pos: int = 0) -> None:
        b, h, n, d = k.shape
        slots = self._write_slots
        if slots is None or slots.shape[0] < b or slots.shape[1] != n:
            raise RuntimeError("call advance(n, batch_size) before write()")
        if self.finalize_in_step and layer_idx == 0:
            self._finalize_in_step()
        if self._bounds_on:                       # bounds of the rows as given (exact fp16 K)
            for j in range(n):
                kv_write.update_bounds_only(k[:, :, j], self._slot_vec(slots, b) if n == 1 else
                                            slots[:b, j].contiguous(), self.kmin[layer_idx],
                                            self.kmax[layer_idx], self.block_size)
        zero = self._flat_v_zero[layer_idx] if self.asymmetric else None
        consts = dict(asym=self.asymmetric, eps=_EPS, qmax=float(self.v_qmax),
                      levels=float(self.v_levels), offset=float(self.v_offset))
        if n == 1:
            iw.decode_write(k, v, self._slot_vec(slots, b), self._k_res_idx_buf[:b], self._flat_v[layer_idx],
                            self._flat_v_scale[layer_idx], zero, self._k_res_flat[layer_idx], **consts)
            return
        # Prefill (set-up path): token by token through the same two kernels,
        # finalising a sequence's page as soon as a position completes it.
        bs = self.block_size
        active, starts = self._active[:b], self._starts[:b]
        for j in range(n):
            res_idx = torch.tensor([i * bs + (s + j) % bs for i, s in zip(active, starts)],
                                   dtype=torch.int64, device=self.device)
            iw.decode_write(k[:, :, j:j + 1], v[:, :, j:j + 1], slots[:b, j].contiguous(), res_idx,
                            self._flat_v[layer_idx], self._flat_v_scale[layer_idx], zero,
                            self._k_res_flat[layer_idx], **consts)
            rows = [i for i, s in zip(active, starts) if (s + j + 1) % bs == 0]
            if rows:
                ids = [self.tables[i].blocks[(s + j) // bs] for i, s in zip(active, starts)
                       if (s + j + 1) % bs == 0]
                iw.finalize_blocks(self._k_residual[layer_idx],
                                   torch.tensor(rows, dtype=torch.int64, device=self.device),
                                   torch.tensor(ids, dtype=torch.int64, device=self.device),
                                   self.k_pool[layer_idx], self.k_scale_pool[layer_idx],
                                   self.k_zero_pool[layer_idx] if self.asymmetric else None,
                                   **self._quant_consts())
        if layer_idx == self.spec.num_layers - 1:
            for i, s in zip(active, starts):
                self._fin[i] = (s + n) // bs
