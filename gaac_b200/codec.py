"""Lossless BF16 KV format (GAAC tiles): calibration, encoder and bit-exact decoder on the B200 CUDA library.

Mirror of the reference module gaac/codec.py (same names, tensor layouts and Page fields); the arithmetic runs in
libgaac_b200.so.  Format (gaac/codec.py:1-18): a BF16 value is split into its sign+mantissa byte (stored as is) and its
8-bit exponent, which is coded against a per-(kv head, channel) base: 3-bit code inside the calibrated 8-wide window; groups
of 8 stored positions that do not fit are promoted as a whole to a 16-wide window (one escape byte) or to raw exponents (five
escape bytes), recorded in a 2-bit tag per group.  Storage order inside a 16-token tile is the m16n8k16 fragment order.
"""
from __future__ import annotations
from dataclasses import dataclass
import torch
from . import _lib

D = 128     # head dim
T = 16      # tokens per tile
GS = 8      # elements per group
CB = D * 3 // 8   # code bytes per token row


def perm_k(D: int = D) -> torch.Tensor:
    """K storage order (gaac/codec.py:29-36): stored position 32j + 4s + q holds channel 16s + 2j + (0, 1, 8, 9)[q]."""
    j, s, q = torch.meshgrid(torch.arange(4), torch.arange(8), torch.arange(4), indexing="ij")
    return (16 * s + 2 * j + torch.tensor([0, 1, 8, 9])[q]).reshape(-1).to(torch.long)


def perm_v(D: int = D) -> torch.Tensor:
    """V storage order (gaac/codec.py:39-45): stored position 16r + n holds channel 8n + r."""
    r, n = torch.meshgrid(torch.arange(8), torch.arange(16), indexing="ij")
    return (8 * n + r).reshape(-1).to(torch.long)


def perm(kind: str) -> torch.Tensor:
    return perm_k() if kind == "k" else perm_v()


def storage_index(kind: str, dev) -> tuple[torch.Tensor, torch.Tensor]:
    """(sm_idx [T*D], code_idx [T*CB]): storage byte -> token-major byte inside one tile (gaac/codec.py:52-67)."""
    lane = torch.arange(32)
    if kind == "k":
        o = torch.arange(2).view(2, 1, 1)
        tok = 8 * o + (lane >> 2).view(1, 32, 1)
        j = (lane & 3).view(1, 32, 1)
        sm = tok * D + 32 * j + torch.arange(32).view(1, 1, 32)
        cd = tok * CB + 12 * j + torch.arange(12).view(1, 1, 12)
    else:
        j, r = (lane & 3).view(32, 1, 1), (lane >> 2).view(32, 1, 1)
        tok = torch.stack([2 * j, 2 * j + 1, 2 * j + 8, 2 * j + 9], 1).view(32, 4, 1)
        sm = tok * D + 16 * r + torch.arange(16).view(1, 1, 16)
        cd = tok * CB + 6 * r + torch.arange(6).view(1, 1, 6)
    return sm.reshape(-1).to(dev), cd.reshape(-1).to(dev)


def _cuda(x: torch.Tensor, what: str) -> torch.Tensor:
    if not x.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor: gaac_b200 has no CPU path")
    return x


def exponent_hist(x: torch.Tensor, n_kv: int) -> torch.Tensor:
    """x: [..., n_kv, D] bf16 (token-major) -> int64 [n_kv*D, 256] exponent histogram (gaac/codec.py:80-84)."""
    x = _cuda(x, "x").contiguous()
    n_ch = n_kv * D
    hist = torch.zeros(n_ch, 256, dtype=torch.int64, device=x.device)
    N = x.numel() // n_ch
    if N:
        _lib.check(_lib.lib().gaac_exponent_hist(x.data_ptr(), N, n_ch, hist.data_ptr(), _lib.stream_ptr(x.device)), "gaac_exponent_hist")
    return hist


def bases_from_hist(hist: torch.Tensor, n_kv: int) -> tuple[torch.Tensor, torch.Tensor]:
    """hist: [n_kv*D, 256] exponent counts -> (base3, base4) uint8 [n_kv, D]: start of the densest 8- / 16-wide window,
    first maximum wins (gaac/codec.py:70-77)."""
    hist = _cuda(hist, "hist").to(torch.int64).contiguous()
    n = hist.shape[0]
    b3 = torch.empty(n, dtype=torch.uint8, device=hist.device); b4 = torch.empty_like(b3)
    _lib.check(_lib.lib().gaac_bases_from_hist(hist.data_ptr(), n, b3.data_ptr(), b4.data_ptr(), _lib.stream_ptr(hist.device)), "gaac_bases_from_hist")
    return b3.view(n_kv, D), b4.view(n_kv, D)


@dataclass
class Page:
    """One kind (K or V) of H heads, every head S tokens long, in compressed form.  Field set and layouts as in
    gaac/codec.py:87-102.  Token rows are padded to whole tiles (S_pad = 16 * ceil(S / 16)); inside a tile the bytes are in the
    order the attention kernel's fragments want them (storage_index).

      sm, codes        uint8 [H, S_pad*128], [H, S_pad*48]   sign+mantissa byte and 3-bit code of every element
      flags            int32 [H, S_pad]                      one tag word per token row, 2 bits per group; padding rows are 0
      ovf              uint8 [n + 8]                         the escape bytes of all heads back to back, 8 spare bytes behind
      ovf_head_start   int32 [H + 1]                         where each head's escape bytes begin in ovf
      tile_off         int32 [H, S_pad/16]                   where each tile's escape bytes begin inside its head's share
      ovf_off          int32 [H, S]                          the same per token row (only the reference's torch decoder reads it)
      base3, base4     uint8 [n_kv, 128]                     the exponent window starts the codes are relative to
    """
    sm: torch.Tensor
    codes: torch.Tensor
    flags: torch.Tensor
    ovf_off: torch.Tensor
    ovf: torch.Tensor
    ovf_head_start: torch.Tensor
    tile_off: torch.Tensor
    base3: torch.Tensor
    base4: torch.Tensor
    H: int
    S: int
    n_kv: int
    kind: str                     # 'k' or 'v'

    @property
    def nbytes(self) -> int:
        """Bytes that have to be read to use the Page: per token 128 + 48 + 4, the escape bytes, 4 per tile for its offset
        (gaac/codec.py:104-108; the two small base tables are left out there as well)."""
        escapes = int(self.ovf_head_start[-1] - self.ovf_head_start[0])
        tiles = (self.S + T - 1) // T
        return self.H * (self.S * (D + CB + 4) + tiles * 4) + escapes

    @property
    def ratio(self) -> float:
        """BF16 bytes of the same tokens divided by nbytes."""
        return self.H * self.S * D * 2 / self.nbytes


class Codec:
    """Holds the exponent bases of n_kv kv heads and turns [H, S, 128] bf16 into a Page and back (gaac/codec.py:115-218).
    Encoding and decoding produce the reference's bytes, computed by the CUDA kernels."""

    def __init__(self, n_kv: int, device: str = "cuda"):
        self.n_kv, self.device = n_kv, device
        self.base3 = self.base4 = None

    def _as_table(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.device, torch.uint8).reshape(self.n_kv, D).contiguous()

    def calibrate(self, sample: torch.Tensor) -> "Codec":
        """Pick the bases from sample [H, n_tokens, 128] bf16; H may be a multiple of n_kv, head h then counts for kv head h % n_kv."""
        groups = sample.shape[0] // self.n_kv
        token_major = sample.to(self.device).reshape(groups, self.n_kv, -1, D).permute(0, 2, 1, 3)     # [groups, n_tokens, n_kv, 128]
        self.base3, self.base4 = bases_from_hist(exponent_hist(token_major, self.n_kv), self.n_kv)
        return self

    def set_bases(self, base3: torch.Tensor, base4: torch.Tensor) -> "Codec":
        """Use given tables (any shape with n_kv*128 entries).  Values must leave room for the window: base3 <= 248, base4 <= 240."""
        self.base3, self.base4 = self._as_table(base3), self._as_table(base4)
        return self

    def encode(self, x: torch.Tensor, kind: str) -> Page:
        """x: [H, S, D] bf16 -> Page."""
        from .encoder import TileEncoder
        return TileEncoder(kind, self.device).encode(self, x.to(self.device))

    @staticmethod
    def decode(page: Page) -> torch.Tensor:
        """Bit-exact reconstruction: Page -> [H, S, D] bf16."""
        sm = _cuda(page.sm, "page.sm")
        H, S = page.H, page.S
        out = torch.empty(H, S, D, dtype=torch.bfloat16, device=sm.device)
        if H == 0 or S == 0:
            return out
        S_pad = page.sm.shape[1] // D
        nb = page.base3.shape[0]
        bidx = None
        if nb != page.n_kv:                          # one base row per head (per-sequence calibration)
            bidx = (torch.arange(H, device=sm.device, dtype=torch.int32) % nb).contiguous()
        _lib.check(_lib.lib().gaac_decode_page(
            page.sm.data_ptr(), page.codes.data_ptr(), page.flags.data_ptr(), page.tile_off.data_ptr(), _lib.row_stride(page.tile_off),
            page.ovf.data_ptr(), page.ovf_head_start.data_ptr(), page.base3.data_ptr(), page.base4.data_ptr(), _lib.ptr(bidx),
            page.n_kv, 0 if page.kind == "k" else 1, H, S, S_pad, out.data_ptr(), _lib.stream_ptr(sm.device)), "gaac_decode_page")
        return out


def row_offsets(flags: torch.Tensor, S: int) -> torch.Tensor:
    """Row offsets within each head's escape stream from the tag words (gaac/codec.py:221-225)."""
    f = flags[:, :S].to(torch.int64) & 0xFFFFFFFF
    odd = (f >> 1) & 0x55555555
    even = f & 0x55555555
    def popc(v):
        v = (v & 0x33333333) + ((v >> 2) & 0x33333333)
        v = (v + (v >> 4)) & 0x0F0F0F0F
        return (v * 0x01010101 >> 24) & 0xFF
    rb = popc(even) + 4 * popc(odd)
    return (torch.cumsum(rb, 1) - rb).to(torch.int32).contiguous()
