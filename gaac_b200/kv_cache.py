"""Serving cache of one attention layer in the slot layout (drop-in for gaac/kv_cache.py).

A slot is the storage of one sequence: n_kv cache heads, each with room for `capacity` tokens.  Tokens live in two places:
whole 16-token tiles in compressed form, and the 0..15 tokens that do not fill a tile yet as plain BF16 rows (the tail).  The
decode step appends one token per batch row; the append that completes a tail turns it into a compressed tile on the device
and adds the tile's escape bytes to the head's escape stream.  Nothing in a decode step (append, attention) talks to the host,
so the step can be captured in a CUDA graph; batch rows find their slot through a device tensor, and a row whose slot is -1 is
left alone (its attention output is zero).  The exponent bases come either from an offline calibration ([n_kv, 128] tables
shared by all sequences) or, when none are given, from each sequence's own prompt at prefill time (one table row per cache
head).

Buffer shapes, field names and the byte accounting follow gaac/kv_cache.py:99-146 because callers and the attention launcher
read them; the device work goes through libgaac_b200.so.
"""
from __future__ import annotations
import torch
from . import _lib
from .codec import Codec, Page, D, T, CB, bases_from_hist, exponent_hist
from .encoder import TileEncoder
from .kernel import _ext, choose_nsplit, choose_nsplit_sm100

TAIL = T                       # rows of the raw tail buffer of a head
TILE_MAX_ESC = 1280            # a tile whose 256 groups are all raw has 256 * 5 escape bytes
_OVER_READ = 8                 # the readers may touch up to 8 bytes behind the last escape byte of a head


def _round_up_tokens(n: int) -> int:
    return -(-n // T) * T


class _Store:
    """What one kind ('k' or 'v') keeps for H cache heads (gaac/kv_cache.py:99-119): sign/mantissa bytes, codes, tag words and
    tile offsets per head, one escape stream of ovf_cap bytes per head inside `ovf`, the raw tails, and the base tables."""

    def __init__(self, kind, H, cap, ovf_cap, base3, base4, dev):
        self.kind, self.H = kind, H
        self.base3, self.base4 = base3, base4
        u8 = dict(dtype=torch.uint8, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        self.sm = torch.zeros(H, cap * D, **u8)
        self.codes = torch.zeros(H, cap * CB, **u8)
        self.flags = torch.zeros(H, cap, **i32)
        self.tile_off = torch.zeros(H, cap // T, **i32)
        self.ovf_used = torch.zeros(H, **i32)
        self.tail = torch.zeros(H, TAIL, D, dtype=torch.bfloat16, device=dev)
        self.enc = TileEncoder(kind, dev)
        self._set_escape_stream(torch.zeros(H * ovf_cap, **u8), ovf_cap)

    def _set_escape_stream(self, ovf, ovf_cap):
        self.ovf, self.ovf_cap = ovf, ovf_cap
        self.head_start = torch.arange(self.H + 1, dtype=torch.int32, device=ovf.device) * ovf_cap

    def grow(self, ovf_cap):
        """Give every head an escape stream of ovf_cap bytes, keeping what is stored."""
        wider = torch.zeros(self.H, ovf_cap, dtype=torch.uint8, device=self.ovf.device)
        wider[:, :self.ovf_cap].copy_(self.ovf.view(self.H, self.ovf_cap))
        self._set_escape_stream(wider.view(-1), ovf_cap)

    def c_store(self) -> _lib.Store:
        p = lambda t: t.data_ptr()
        return _lib.Store(p(self.sm), p(self.codes), p(self.flags), p(self.tile_off), p(self.ovf), p(self.ovf_used), p(self.tail), p(self.base3), p(self.base4))


class CompressedKVCache:
    def __init__(self, n_slots: int, n_kv: int, capacity: int, bases: dict | None = None,
                 ovf_bytes_per_tile: int = 128, device="cuda"):
        """capacity: tokens a sequence may hold (rounded up to whole tiles).  bases: {'k3','k4','v3','v4'} -> uint8 [n_kv, 128],
        or None to calibrate every sequence on its own prompt.  ovf_bytes_per_tile: escape bytes reserved per tile of capacity."""
        if torch.device(device).type != "cuda":
            raise RuntimeError("CompressedKVCache needs a CUDA device: gaac_b200 has no CPU path")
        _lib.lib()
        self.n_slots, self.n_kv = n_slots, n_kv
        self.cap = _round_up_tokens(capacity)
        self.H = n_slots * n_kv
        self.per_sequence_bases = bases is None
        ovf_cap = (self.cap // T) * ovf_bytes_per_tile + _OVER_READ
        tables = {}
        for key in ("k3", "k4", "v3", "v4"):
            if self.per_sequence_bases:
                tables[key] = torch.zeros(self.H, D, dtype=torch.uint8, device=device)           # filled per sequence by prefill
            else:
                tables[key] = bases[key].to(device, torch.uint8).reshape(n_kv, D).contiguous()
        self.k = _Store("k", self.H, self.cap, ovf_cap, tables["k3"], tables["k4"], device)
        self.v = _Store("v", self.H, self.cap, ovf_cap, tables["v3"], tables["v4"], device)
        self.S = torch.zeros(self.H, dtype=torch.int32, device=device)                           # tokens in compressed tiles, per head
        self.tail_len = torch.zeros(self.H, dtype=torch.int32, device=device)                    # tokens in the raw tail, per head
        self.append_errors = torch.zeros(1, dtype=torch.int32, device=device)                    # tiles an append refused for lack of escape room
        self._scratch = None                                                                     # escape slots of the prefill in flight (grown on demand)
        self._slot_status = torch.zeros(n_slots, 4, dtype=torch.int32, device=device)           # per slot: what its last prefill reported
        self._pending, self._pending_bytes = {}, 0                                                # prefills whose host check is still due: slot -> (tokens, escape slots)
        self.pending_scratch_limit = 1 << 30                                                      # bytes of escape slots kept for unchecked prefills before a check is forced
        self.growable = True                                                                     # False: the buffers may not move (their addresses are baked into CUDA graphs)

    @staticmethod
    def bytes_per_slot(n_kv: int, capacity: int, ovf_bytes_per_tile: int = 128, per_sequence_bases: bool = True) -> int:
        """Device bytes one slot costs, the figure an engine divides its memory budget by (gaac/kv_cache.py:142-146)."""
        cap = _round_up_tokens(capacity)
        tiles = cap // T
        payload = cap * (D + CB + 4)                                   # sign/mantissa + codes + tag word per token
        escapes = tiles * ovf_bytes_per_tile + _OVER_READ
        counters = tiles * 4 + 8                                       # tile offsets; head_start and ovf_used entries
        tail = TAIL * D * 2
        own_bases = 2 * D if per_sequence_bases else 0
        one_kind_one_head = payload + escapes + counters + tail + own_bases
        return 2 * n_kv * one_kind_one_head + 8 * n_kv                 # K and V; the token and tail counters of the heads

    def _heads(self, slot: int) -> slice:
        return slice(slot * self.n_kv, (slot + 1) * self.n_kv)

    # ------------------------------------------------------------------ prefill
    def prefill(self, slot: int, k: torch.Tensor, v: torch.Tensor, check: bool = True):
        """Put a prompt's K and V ([L, n_kv, 128] bf16, one row per token as the model produces them) into `slot`: whole tiles
        compressed, the remainder into the tail.  Replaces whatever the slot held.  (gaac/kv_cache.py:149-169)
        One library call (encode of both kinds straight from the token-major rows, offsets, the copy into the heads' escape
        streams, tails, counters) and ONE host read afterwards (the status words): the copy never writes past a head's share, so
        the check can follow it.  Only when a head's stream was too small are the streams enlarged and the copy (not the
        encode) repeated.
        check=False puts the host read off: the call returns as soon as its kernels are queued and keeps the prompt's escape
        slots (160 B per token and kv head) until settle_prefills() - which append, attention, decompress, check_capacity
        and stats call first - reads the status words of all such prefills in one go and repairs the slots whose streams were
        too small.  A step that prefills several prompts then waits for the GPU once, not once per prompt."""
        L = k.shape[0]
        assert L <= self.cap, f"sequence of {L} tokens exceeds the cache capacity {self.cap}"
        assert 0 <= slot < self.n_slots
        hs = self._heads(slot)
        k, v = self._token_rows(k), self._token_rows(v)
        if self.per_sequence_bases and L:
            for st, x in ((self.k, k), (self.v, v)):
                rows = x if x.is_contiguous() else x.contiguous()                                 # the histogram reads [L, n_kv * 128] rows
                st.base3[hs], st.base4[hs] = bases_from_hist(exponent_hist(rows, self.n_kv), self.n_kv)
        need = _lib.lib().gaac_cache_prefill_scratch_bytes(L, self.n_kv)
        if check:
            self.settle_prefills()
            if self._scratch is None or self._scratch.numel() < need:
                self._scratch = torch.empty(need, dtype=torch.uint8, device=k.device)
            scratch, status = self._scratch, self._slot_status[slot]
        else:
            old = self._pending.pop(slot, None)
            if old is not None:
                self._pending_bytes -= old[1].numel()
            if self._pending_bytes + need > self.pending_scratch_limit:
                self.settle_prefills()
            scratch, status = torch.empty(need, dtype=torch.uint8, device=k.device), self._slot_status[slot]
        self._prefill_launch(slot, L, k, v, scratch, status, copy_only=0)
        if not check:
            self._pending[slot] = (L, scratch)
            self._pending_bytes += need
            return
        short_k, used_k, short_v, used_v = status.tolist()                                         # the one host synchronisation
        # room for these tiles and for one more worst-case tile, which an append may add before the next check_capacity
        wanted = max(used_k, used_v) + TILE_MAX_ESC + _OVER_READ
        if wanted > self.k.ovf_cap:
            self._grow(wanted)
        if short_k or short_v:
            self._prefill_launch(slot, L, None, None, scratch, status, copy_only=1)

    def _prefill_launch(self, slot, L, k, v, scratch, status, copy_only: int):
        dev = self.S.device
        _lib.check(_lib.lib().gaac_cache_prefill(self.k.c_store(), self.v.c_store(), _lib.ptr(k), _lib.ptr(v), L, _lib.row_stride(k) if k is not None else self.n_kv * D,
                                                 slot, self.n_kv, self.tail_len.data_ptr(), self.S.data_ptr(), self.cap, self.k.ovf_cap, self.k.base3.shape[0],
                                                 scratch.data_ptr(), scratch.numel(), status.data_ptr(), copy_only, _lib.stream_ptr(dev)), "gaac_cache_prefill")

    def settle_prefills(self):
        """Host check of every prefill made with check=False: one read of their status words; the escape streams grow when one
        of them (plus a worst-case tile) no longer fits, and the slots whose escape bytes did not fit get theirs copied again
        from the escape slots kept since the prefill."""
        if not self._pending:
            return
        pending, self._pending, self._pending_bytes = self._pending, {}, 0
        slots = list(pending)
        words = self._slot_status[torch.tensor(slots, dtype=torch.long, device=self.S.device)].tolist()
        wanted = max(max(w[1], w[3]) for w in words) + TILE_MAX_ESC + _OVER_READ
        if wanted > self.k.ovf_cap:
            try:
                self._grow(wanted)
            except RuntimeError:                     # the streams may not move: the prefills stay unsettled, and every later call says so again
                self._pending, self._pending_bytes = pending, sum(p[1].numel() for p in pending.values())
                raise
        for slot, w in zip(slots, words):
            if w[0] or w[2]:
                L, scratch = pending[slot]
                self._prefill_launch(slot, L, None, None, scratch, self._slot_status[slot], copy_only=1)

    @staticmethod
    def _token_rows(x: torch.Tensor) -> torch.Tensor:
        """x [L, n_kv, 128] as the library reads it: unit stride over channels, heads 128 elements apart, 16-byte aligned rows; a
        slice of a larger token-major tensor passes as it is, anything else is copied."""
        if not x.is_cuda:
            raise RuntimeError("CompressedKVCache needs CUDA tensors: gaac_b200 has no CPU path")
        ok = x.dtype == torch.bfloat16 and x.dim() == 3 and x.shape[2] == D and x.stride(2) == 1 and (x.shape[1] == 1 or x.stride(1) == D) and \
            (x.shape[0] <= 1 or (x.stride(0) >= x.shape[1] * D and x.stride(0) % 8 == 0)) and x.data_ptr() % 16 == 0
        if ok and x.shape[0] <= 1:
            return x.contiguous()
        return x if ok else x.to(torch.bfloat16).contiguous()

    # ------------------------------------------------------------------ decode step
    def append(self, slots: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
        """One new token for every batch row: slots int32 [B] (-1: skip the row), k / v [B, n_kv, 128] bf16.  A single kernel
        launch that also advances the counters; safe inside a CUDA graph.  (gaac/kv_cache.py:172-181)"""
        B = slots.numel()
        if B == 0:
            return
        self.settle_prefills()
        k, v = k.contiguous(), v.contiguous()
        rc = _lib.lib().gaac_append_kv(self.k.c_store(), self.v.c_store(), k.data_ptr(), v.data_ptr(), slots.data_ptr(), B, self.n_kv,
                                       self.tail_len.data_ptr(), self.S.data_ptr(), self.cap, self.k.ovf_cap, self.k.base3.shape[0],
                                       self.append_errors.data_ptr(), _lib.stream_ptr(k.device))
        _lib.check(rc, "gaac_append_kv")

    def attention(self, q: torch.Tensor, slots: torch.Tensor, scale: float, max_len: int | None = None, nsplit: int | None = None, out_f32=None):
        """q [B, n_q, 128] bf16, row b attending over slot slots[b] -> [B, n_q, 128] bf16; rows with slot -1 come back as
        zeros.  max_len (longest sequence in the batch, the capacity when omitted) only steers the split count.
        (gaac/kv_cache.py:183-192)"""
        B, n_q, _ = q.shape
        self.settle_prefills()
        if nsplit is None:
            nsplit = choose_nsplit_sm100(B, self.n_kv, max_len or self.cap)
        K, V = self.k, self.v
        out = _ext().gaac_attn_launch(K.sm, K.codes, K.flags, K.tile_off, K.ovf, K.head_start, K.base3, K.base4,
                                      V.sm, V.codes, V.flags, V.tile_off, V.ovf, V.head_start, V.base3, V.base4,
                                      q.reshape(B * n_q, D).contiguous(), slots, n_q, self.n_kv, self.S, self.cap, scale, nsplit,
                                      K.tail, V.tail, self.tail_len, TAIL, out_f32=out_f32)
        return out.view(B, n_q, D)

    # ------------------------------------------------------------------ housekeeping
    def max_escape_bytes(self) -> torch.Tensor:
        """Fullest escape stream over all heads and both kinds (a device scalar)."""
        return torch.maximum(self.k.ovf_used.max(), self.v.ovf_used.max())

    def check_capacity(self, used: int | None = None):
        """Keep one worst-case tile of escape room free in every head.  A head completes at most one tile per 16 decode steps, so
        calling this every 16 steps (or more often) means an append never runs out of room.  `used`: the caller's own reading of
        max_escape_bytes(), to save the device read.  (gaac/kv_cache.py:198-203)"""
        self.settle_prefills()
        if used is None:
            used = int(self.max_escape_bytes())
        wanted = used + TILE_MAX_ESC + _OVER_READ
        if wanted > self.k.ovf_cap:
            self._grow(wanted)

    def _grow(self, need: int):
        if not self.growable:
            raise RuntimeError(f"escape stream needs {need} B per head but holds {self.k.ovf_cap} B and CUDA graphs are captured; "
                               "raise gaac_ovf_bytes_per_tile or calibrate the exponent bases on representative prompts")
        new_cap = max(2 * self.k.ovf_cap, need + 4096 + 7) // 8 * 8       # at least double, so growth is rare
        for st in (self.k, self.v):
            st.grow(new_cap)

    def decompress(self, slot: int) -> tuple[torch.Tensor, torch.Tensor]:
        """The slot's K and V back as BF16 [L, n_kv, 128], bit for bit what went in: decoded tiles followed by the tail.
        (gaac/kv_cache.py:211-226)"""
        self.settle_prefills()
        hs = self._heads(slot)
        n_comp, n_tail = int(self.S[hs.start]), int(self.tail_len[hs.start])
        result = []
        for st in (self.k, self.v):
            pieces = [st.tail[hs, :n_tail]]
            if n_comp:
                own_rows = st.base3.shape[0] != self.n_kv
                b3 = st.base3[hs] if own_rows else st.base3
                b4 = st.base4[hs] if own_rows else st.base4
                view = Page(st.sm[hs], st.codes[hs], st.flags[hs], None, st.ovf, st.head_start[hs.start:hs.stop + 1], st.tile_off[hs],
                            b3, b4, self.n_kv, n_comp, self.n_kv, st.kind)
                pieces.insert(0, Codec.decode(view))
            result.append(torch.cat(pieces, 1).transpose(0, 1).contiguous())
        return result[0], result[1]

    def stats(self) -> dict:
        """Bytes the stored tokens occupy (tiles, escapes, tag words, tile offsets, raw tails) against their size as plain BF16.
        (gaac/kv_cache.py:228-234)"""
        self.settle_prefills()
        comp_tokens, tail_tokens = int(self.S.sum()), int(self.tail_len.sum())                 # summed over heads
        escapes = int(self.k.ovf_used.sum()) + int(self.v.ovf_used.sum())
        per_kind = comp_tokens * (D + CB + 4) + (comp_tokens // T) * 4 + tail_tokens * D * 2
        used = 2 * per_kind + escapes
        plain = 2 * (comp_tokens + tail_tokens) * D * 2
        return dict(tokens=(comp_tokens + tail_tokens) // max(1, self.n_kv), bytes_used=used, bf16_bytes=plain, ratio=plain / max(1, used))
