"""Tile encoder on the CUDA library: one warp per (head, 16-token tile), bit-identical to the reference codec.

Mirror of gaac/encoder.py.  `encode_tiles` writes sign/mantissa, code and tag bytes in the kernel's fragment order and leaves each
tile's escape bytes in a bounded scratch slot (1280 B worst case); `compact` turns the per-tile byte counts into tile offsets and
packs the slots into each head's escape stream.  `encode_into` chains the two on the device with no host round trip in
between (the escape stream is caller-sized and the copy into it is bounded); `encode` builds a whole Page with it and reads the
exact size once at the end.
"""
from __future__ import annotations
import torch
from . import _lib
from .codec import Codec, Page, D, T, CB, perm, storage_index, row_offsets

SLOT = 1280


class TileEncoder:
    def __init__(self, kind: str, device="cuda"):
        self.kind = kind
        self.device = device
        # index tables kept for callers that read them (the kernels do not need them)
        self.perm = perm(kind).to(torch.int32)
        self._slots = None

    @property
    def inv_sm(self):
        si, _ = storage_index(self.kind, "cpu")
        inv = torch.empty_like(si); inv[si] = torch.arange(si.numel())
        return inv.to(torch.int32)

    @property
    def inv_cd(self):
        _, ci = storage_index(self.kind, "cpu")
        inv = torch.empty_like(ci); inv[ci] = torch.arange(ci.numel())
        return inv.to(torch.int32)

    def _scratch(self, n: int, dev):
        if self._slots is None or self._slots.numel() < n or self._slots.device != dev:
            self._slots = torch.empty(n, dtype=torch.uint8, device=dev)
        return self._slots

    def encode_tiles(self, x, base3, base4, sm, cd, flags, S, S_pad, n_kv, bidx=None) -> torch.Tensor:
        """Encode x [H, S_in, D] (tiles 0..ceil(S/16)-1) into sm/cd/flags with token stride S_pad; escape bytes stay in the
        scratch slots.  Returns tile_bytes int32 [H, ntiles]; finish with compact().  (gaac/encoder.py:94-102)"""
        if not x.is_cuda:
            raise RuntimeError("TileEncoder needs CUDA tensors: gaac_b200 has no CPU path")
        H = x.shape[0]; ntiles = (S + T - 1) // T; dev = x.device
        x = x.contiguous()
        slots = self._scratch(H * ntiles * SLOT, dev)
        tile_bytes = torch.empty(H, ntiles, dtype=torch.int32, device=dev)
        if H == 0 or ntiles == 0:
            return tile_bytes
        _lib.check(_lib.lib().gaac_encode_tiles(
            x.data_ptr(), H, S, x.shape[1], S_pad, base3.data_ptr(), base4.data_ptr(), _lib.ptr(bidx), n_kv, 0 if self.kind == "k" else 1,
            sm.data_ptr(), cd.data_ptr(), flags.data_ptr(), slots.data_ptr(), tile_bytes.data_ptr(), _lib.stream_ptr(dev)), "gaac_encode_tiles")
        return tile_bytes

    def tile_offsets(self, tile_bytes) -> tuple[torch.Tensor, torch.Tensor]:
        """(tile_off int32 [H, ntiles], head_bytes int32 [H]): exclusive prefix of tile_bytes per head and its total."""
        H, ntiles = tile_bytes.shape
        tile_off = torch.empty_like(tile_bytes); head_bytes = torch.zeros(H, dtype=torch.int32, device=tile_bytes.device)
        if H and ntiles:
            _lib.check(_lib.lib().gaac_compact(None, tile_bytes.data_ptr(), H, ntiles, None, None, tile_off.data_ptr(), ntiles,
                                               head_bytes.data_ptr(), None, 0, 0, None, _lib.stream_ptr(tile_bytes.device)), "gaac_compact")
        return tile_off, head_bytes

    def compact(self, tile_bytes, head_start, ovf, flags=None, S=0, S_pad=0, ovf_off=None) -> torch.Tensor:
        """Pack the scratch slots into ovf at head_start[h] + tile_off[h, t]; returns tile_off int32 [H, ntiles].
        (gaac/encoder.py:104-109)  With flags / S / S_pad / ovf_off the per-row escape offsets are written too."""
        H, ntiles = tile_bytes.shape
        tile_off = torch.empty_like(tile_bytes)
        if H and ntiles:
            head_start = head_start.contiguous()
            _lib.check(_lib.lib().gaac_compact(self._slots.data_ptr(), tile_bytes.data_ptr(), H, ntiles, head_start.data_ptr(), ovf.data_ptr(),
                                               tile_off.data_ptr(), ntiles, None, _lib.ptr(flags), S, S_pad, _lib.ptr(ovf_off),
                                               _lib.stream_ptr(tile_bytes.device)), "gaac_compact")
        return tile_off

    # ------------------------------------------------------------------ whole encode without a host round trip
    GUESS_BYTES_PER_TILE = 128          # first guess for the escape stream of a Page (measured mean on model-like data: 30-60 B)

    def _status(self, dev) -> torch.Tensor:
        st = getattr(self, "_status_word", None)
        if st is None or st.device != dev:
            self._status_word = st = torch.zeros(1, dtype=torch.int32, device=dev)
        return st

    def encode_into(self, x: torch.Tensor, base3, base4, n_kv: int, sm, cd, flags, tile_off, ovf, *, S: int | None = None, S_pad: int | None = None,
                    head_start=None, head_base=None, head_cap: int = 0, head_bytes=None, ovf_off=None, bidx=None, zero_pad: int = 8, status=None):
        """Encode x [H, S_in, D] (its first S tokens) into caller-owned buffers: four kernel launches, no host synchronisation, so
        it can sit inside a CUDA graph (the serving path).  sm / cd / flags: [H, S_pad*..] rows as in a Page; tile_off int32
        [H, ntiles] contiguous, written.  Escape bytes go to `ovf`:
          packed   - head after head; head_start int32 [H+1] is written (head_start[H] = all bytes); bounded by ovf.numel()
          per head - head h at ovf + head_base[h] (int32 [H], given) with at most head_cap bytes; head_bytes int32 [H] is written
        Returns (status, retry): status = device int32 whose bit 0 is set when the room did not suffice (those tiles' escape bytes
        were not written; head_start / head_bytes are exact all the same); retry(ovf, head_base=None, head_cap=0) repeats only the
        copy into a larger buffer.  zero_pad bytes of read padding are kept free behind every head (per head) or written as zeros
        behind the last head (packed).  status: the int32 word to use (zero on entry); by default one kept by the encoder."""
        if not x.is_cuda:
            raise RuntimeError("TileEncoder needs CUDA tensors: gaac_b200 has no CPU path")
        H, S_in, _ = x.shape
        S = S_in if S is None else S
        S_pad = sm.shape[1] // D if S_pad is None else S_pad
        ntiles = (S + T - 1) // T
        dev = x.device
        x = x.contiguous()
        assert tile_off.stride(0) == ntiles or H == 1, "tile_off rows must be ntiles apart"
        L = _lib.lib(); st = _lib.stream_ptr(dev)
        slots = self._scratch(H * ntiles * SLOT, dev)
        work = torch.empty(H * ntiles + 2 * H + 1, dtype=torch.int32, device=dev)
        tile_bytes = work[:H * ntiles]
        hb = head_bytes if head_bytes is not None else work[H * ntiles:H * ntiles + H]
        hs = head_start if head_start is not None else work[H * ntiles + H:]
        if status is None: status = self._status(dev)
        _lib.check(L.gaac_encode_begin(x.data_ptr(), H, S, S_in, S_pad, base3.data_ptr(), base4.data_ptr(), _lib.ptr(bidx), n_kv, 0 if self.kind == "k" else 1,
                                       sm.data_ptr(), cd.data_ptr(), flags.data_ptr(), slots.data_ptr(), tile_bytes.data_ptr(), tile_off.data_ptr(),
                                       hb.data_ptr(), hs.data_ptr(), st), "gaac_encode_begin")

        def copy(ovf, head_base=head_base, head_cap=head_cap):
            per_head = head_base is not None
            _lib.check(L.gaac_compact_copy(slots.data_ptr(), tile_bytes.data_ptr(), H, ntiles, (head_base if per_head else hs).data_ptr(), ovf.data_ptr(),
                                           tile_off.data_ptr(), ntiles, flags.data_ptr(), S, S_pad, _lib.ptr(ovf_off), 0 if per_head else zero_pad,
                                           0 if per_head else ovf.numel(), (head_cap - zero_pad) if per_head else 0, status.data_ptr(), _lib.stream_ptr(dev)),
                       "gaac_compact_copy")
            return status
        copy(ovf)
        return status, copy

    def encode(self, codec: Codec, x: torch.Tensor) -> Page:
        """x: [H, S, D] bf16 -> Page, bit-identical to the reference Codec.encode(x, kind).  (gaac/encoder.py:111-123)
        Everything is launched into an escape buffer of GUESS_BYTES_PER_TILE bytes per tile; ONE host read at the end (the total and
        the status word) cuts the stream to its exact size, as the reference's is.  When the guess was too small the copy alone is
        repeated into a buffer of the exact size."""
        if not x.is_cuda:
            raise RuntimeError("TileEncoder needs CUDA tensors: gaac_b200 has no CPU path")
        H, S, _ = x.shape; dev = x.device
        S_pad = (S + T - 1) // T * T
        ntiles = S_pad // T
        sm = torch.empty(H, S_pad * D, dtype=torch.uint8, device=dev)
        cd = torch.empty(H, S_pad * CB, dtype=torch.uint8, device=dev)
        flags = torch.empty(H, S_pad, dtype=torch.int32, device=dev)          # every row of every tile is written, padded rows as 0
        meta = torch.zeros(H * ntiles + H + 2, dtype=torch.int32, device=dev)                     # tile offsets | head_start [H+1] | the call's status word
        tile_off, head_start, status = meta[:H * ntiles].view(H, ntiles), meta[H * ntiles:H * ntiles + H + 1], meta[-1:]
        ovf_off = torch.empty(H, S, dtype=torch.int32, device=dev)
        if H == 0 or ntiles == 0:
            return Page(sm, cd, flags, ovf_off, torch.zeros(8, dtype=torch.uint8, device=dev), head_start, tile_off, codec.base3, codec.base4, H, S, codec.n_kv, self.kind)
        cap = H * ntiles * self.GUESS_BYTES_PER_TILE + 8
        ovf = torch.empty(cap, dtype=torch.uint8, device=dev)
        _, retry = self.encode_into(x, codec.base3, codec.base4, codec.n_kv, sm, cd, flags, tile_off, ovf, S=S, S_pad=S_pad, head_start=head_start, ovf_off=ovf_off,
                                    status=status)
        total, st = meta[-2:].tolist()                                                            # the one host synchronisation: all bytes, status word
        if st:                                                                                    # the guess was too small: now the size is known
            ovf = torch.empty(total + 8, dtype=torch.uint8, device=dev)
            retry(ovf)
        elif cap != total + 8:
            ovf = ovf[:total + 8].clone()
        return Page(sm, cd, flags, ovf_off, ovf, head_start, tile_off, codec.base3, codec.base4, H, S, codec.n_kv, self.kind)
