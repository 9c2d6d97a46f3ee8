"""Host side of one paged-layout step: from the scheduler's view of a batch to the store entries LayerState.store consumes.

This is the part of the reference's vLLM metadata builder that feeds the store and the prefill-with-context path
(GAACMetadataBuilder.build, gaac/vllm/backend.py:205-254), without vLLM: plain numpy on the host arrays a scheduler has
(query_start_loc, num_computed_tokens), plus the small amount of device plumbing around it (block ids looked up from the slot
mapping, a pinned staging ring so the upload never blocks the host, persistent device buffers for CUDA-graph replay).

Vocabulary: a batch has R requests; request r contributes the query tokens [qsl[r], qsl[r+1]) of the step's flat K/V tensors and
had `start[r]` tokens in the cache before the step.  A store entry = (block id, first row of the step's K/V tensors, first
position inside the 16-token block, number of rows): one per (request, block) pair the step writes into.
"""
from __future__ import annotations
import numpy as np
import torch

BLOCK = 16


def _segments(counts: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """For counts [n0, n1, ...]: (owner, rank) of every element of the concatenation - owner = index of its segment, rank = its
    position inside the segment."""
    counts = np.asarray(counts, dtype=np.int64)
    total = int(counts.sum())
    owner = np.repeat(np.arange(counts.size, dtype=np.int64), counts)
    first = np.cumsum(counts) - counts
    return owner, np.arange(total, dtype=np.int64) - first[owner]


def build_entries(query_start_loc, num_computed_tokens) -> np.ndarray:
    """Store entries of one step -> int32 [E, 4] = (row, row, offset in block, rows).  Column 0 repeats the first K/V row of the
    entry; resolve_blocks replaces it by the physical block id (the block a token lives in is slot_mapping[row] // 16, and the
    slot mapping is a device tensor).  query_start_loc: [R+1] cumulative query lengths; num_computed_tokens: [R] tokens already
    cached per request.  Requests with no query tokens produce no entry.  (gaac/vllm/backend.py:208-219)"""
    qsl = np.asarray(query_start_loc, dtype=np.int64)
    R = qsl.size - 1
    start = np.asarray(num_computed_tokens, dtype=np.int64)[:R]
    qlen = qsl[1:] - qsl[:-1]
    end = start + qlen                                           # tokens in the cache after the step
    first_blk = start // BLOCK
    n_blk = np.where(qlen > 0, (end - 1) // BLOCK - first_blk + 1, 0)
    req, k = _segments(n_blk)
    blk = first_blk[req] + k                                     # logical block of the entry
    lo = np.maximum(start[req], blk * BLOCK)                     # first and one-past-last token position the entry covers
    hi = np.minimum(end[req], (blk + 1) * BLOCK)
    row = qsl[req] + (lo - start[req])
    return np.stack([row, row, lo - blk * BLOCK, hi - lo], axis=1).astype(np.int32)


def resolve_blocks(ent: torch.Tensor, slot_mapping: torch.Tensor) -> torch.Tensor:
    """Fill column 0 of device entries with the physical block of each entry's first token (in place; returns ent)."""
    ent[:, 0] = (slot_mapping[ent[:, 1].long()] // BLOCK).to(torch.int32)
    return ent


def build_context_pairs(num_computed_tokens, query_lens) -> dict:
    """Prefill requests that already have tokens in the cache (prefix hits, chunked prefill) attend over context + new tokens; the
    context is expanded from the paged buffer into flat scratch K/V by LayerState.decode_blocks.  For prefill requests with
    `num_computed_tokens` cached and `query_lens` new tokens each, returns
      pairs   int32 [P, 3]  (logical block of the request, first scratch row, valid rows): map column 0 through the block table
      owner   int64 [P]     prefill request of each pair
      cu_k    int32 [n+1]   scratch row where each request starts (context rows first, then its new tokens)
      slots   int64 [T]     scratch row of every new token, in batch order
      rows, max_k           scratch rows in all, longest (context + new) length
    (gaac/vllm/backend.py:243-253)"""
    ctx = np.asarray(num_computed_tokens, dtype=np.int64)
    new = np.asarray(query_lens, dtype=np.int64)
    total = ctx + new
    row0 = np.concatenate([[0], np.cumsum(total)])               # scratch row where request i starts
    owner, k = _segments((ctx + BLOCK - 1) // BLOCK)             # one pair per context block
    valid = np.minimum(BLOCK, ctx[owner] - k * BLOCK)
    pairs = np.stack([k, row0[owner] + k * BLOCK, valid], axis=1).astype(np.int32)
    t_owner, t_k = _segments(new)
    slots = row0[t_owner] + ctx[t_owner] + t_k
    return dict(pairs=pairs, owner=owner, cu_k=row0.astype(np.int32), slots=slots.astype(np.int64), rows=int(row0[-1]), max_k=int(total.max()) if total.size else 0)


class EntryUploader:
    """Device buffers and pinned staging for the per-step entries of pure-decode batches (gaac/vllm/backend.py:193-200, 220-224).

    Kernels captured in CUDA graphs read the entries from fixed addresses, so the entries of every step are copied into ONE
    persistent device buffer; rows beyond the step's entries are marked inactive (block -1, which the store kernel skips).  The
    copy goes through a ring of pinned host buffers: a pageable host-to-device copy would stall the host until the GPU has
    drained, and a single pinned buffer could be overwritten by the next step before the copy engine has read it."""

    def __init__(self, max_entries: int, n_kv: int, device, ring: int = 16):
        self.max_entries, self.n_kv, self.device = max_entries, n_kv, torch.device(device)
        pin = self.device.type == "cuda"
        self.ent = torch.zeros(max_entries, 4, dtype=torch.int32, device=device)
        self.ent[:, 0] = -1
        self.freeq = torch.empty(max_entries * 2 * n_kv, dtype=torch.int32, device=device)
        self._stage = torch.zeros(ring, max_entries, 4, dtype=torch.int32, pin_memory=pin)
        self._next = 0

    def upload(self, ent_cpu: np.ndarray, slot_mapping: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """(entries [E, 4] on the device, free-queue scratch [E * 2 * n_kv]).  Batches larger than the persistent buffer (prefill
        steps) get fresh tensors, as they are never replayed from a graph."""
        E = ent_cpu.shape[0]
        if E > self.max_entries:
            ent = torch.from_numpy(np.ascontiguousarray(ent_cpu)).to(self.device)
            freeq = torch.empty(E * 2 * self.n_kv, dtype=torch.int32, device=self.device)
        else:
            stage = self._stage[self._next, :E]
            self._next = (self._next + 1) % self._stage.shape[0]
            stage.copy_(torch.from_numpy(np.ascontiguousarray(ent_cpu)))
            ent = self.ent[:E]
            ent.copy_(stage, non_blocking=True)
            self.ent[E:, 0].fill_(-1)
            freeq = self.freeq[:E * 2 * self.n_kv]
        if slot_mapping is not None:
            resolve_blocks(ent, slot_mapping)
        return ent, freeq
