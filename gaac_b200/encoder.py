"""Tile encoder on the CUDA library: one warp per (head, 16-token tile), bit-identical to the reference codec.

Mirror of gaac/encoder.py.  `encode_tiles` writes sign/mantissa, code and tag bytes in the kernel's fragment order and
leaves each tile's escape bytes in a bounded scratch slot (1280 B worst case); `compact` turns the per-tile byte counts into
tile offsets and packs the slots into each head's escape stream.
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

    def encode(self, codec: Codec, x: torch.Tensor) -> Page:
        """x: [H, S, D] bf16 -> Page, bit-identical to the reference Codec.encode(x, kind).  (gaac/encoder.py:111-123)"""
        if not x.is_cuda:
            raise RuntimeError("TileEncoder needs CUDA tensors: gaac_b200 has no CPU path")
        H, S, _ = x.shape; dev = x.device
        S_pad = (S + T - 1) // T * T
        ntiles = S_pad // T
        x = x.contiguous()
        L = _lib.lib(); st = _lib.stream_ptr(dev)
        # every buffer whose size is known is allocated before the one host synchronisation, so the GPU never waits for the host
        sm = torch.empty(H, S_pad * D, dtype=torch.uint8, device=dev)
        cd = torch.empty(H, S_pad * CB, dtype=torch.uint8, device=dev)
        flags = torch.empty(H, S_pad, dtype=torch.int32, device=dev)          # every row of every tile is written, padded rows as 0
        meta = torch.empty(2 * H * ntiles + 2 * H + 1, dtype=torch.int32, device=dev)
        tile_bytes, tile_off = meta[:H * ntiles].view(H, ntiles), meta[H * ntiles:2 * H * ntiles].view(H, ntiles)
        head_bytes, head_start = meta[2 * H * ntiles:2 * H * ntiles + H], meta[2 * H * ntiles + H:]
        ovf_off = torch.empty(H, S, dtype=torch.int32, device=dev)
        if H == 0 or ntiles == 0:
            head_start.zero_()
            return Page(sm, cd, flags, ovf_off, torch.zeros(8, dtype=torch.uint8, device=dev), head_start, tile_off, codec.base3, codec.base4, H, S, codec.n_kv, self.kind)
        slots = self._scratch(H * ntiles * SLOT, dev)
        _lib.check(L.gaac_encode_begin(x.data_ptr(), H, S, x.shape[1], S_pad, codec.base3.data_ptr(), codec.base4.data_ptr(), None, codec.n_kv,
                                       0 if self.kind == "k" else 1, sm.data_ptr(), cd.data_ptr(), flags.data_ptr(), slots.data_ptr(),
                                       tile_bytes.data_ptr(), tile_off.data_ptr(), head_bytes.data_ptr(), head_start.data_ptr(), st), "gaac_encode_begin")
        ovf = torch.empty(int(head_start[-1]) + 8, dtype=torch.uint8, device=dev)     # host sync: sizes the escape stream exactly, as the reference does
        _lib.check(L.gaac_compact_copy(slots.data_ptr(), tile_bytes.data_ptr(), H, ntiles, head_start.data_ptr(), ovf.data_ptr(), tile_off.data_ptr(), ntiles,
                                       flags.data_ptr(), S, S_pad, ovf_off.data_ptr(), 8, st), "gaac_compact_copy")
        return Page(sm, cd, flags, ovf_off, ovf, head_start, tile_off, codec.base3, codec.base4, H, S, codec.n_kv, self.kind)
