"""Compressed KV cache of one attention layer for serving, slot layout (mirror of gaac/kv_cache.py).

Each sequence owns a slot = n_kv cache heads with a fixed token capacity.  A head holds compressed 16-token tiles plus a raw
BF16 tail of 0..15 tokens; when a decode step fills the tail, the tile is compressed in place and its escape bytes are
appended to the head's escape stream.  All decode-step work (append + attention) runs on the device with no host
synchronisation and is CUDA-graph capturable: batch rows reach their slot through a device slot map, rows with slot -1 are
skipped.  Exponent bases are either calibrated per model ([n_kv, D] tables) or per sequence from its own prompt at prefill
([n_slots*n_kv, D] tables).
"""
from __future__ import annotations
import torch
from . import _lib
from .codec import Codec, Page, D, T, CB, row_offsets
from .encoder import TileEncoder
from .kernel import _ext, choose_nsplit, choose_nsplit_sm100

TAIL = 16
TILE_MAX_ESC = 1280    # worst-case escape bytes of one 16-token tile (all 256 groups raw)


class _Store:
    """Compressed buffers of one kind ('k' or 'v') for H cache heads (gaac/kv_cache.py:99-119)."""
    def __init__(self, kind, H, cap, ovf_cap, base3, base4, dev):
        self.kind, self.H, self.ovf_cap = kind, H, ovf_cap
        self.sm = torch.zeros(H, cap * D, dtype=torch.uint8, device=dev)
        self.codes = torch.zeros(H, cap * CB, dtype=torch.uint8, device=dev)
        self.flags = torch.zeros(H, cap, dtype=torch.int32, device=dev)
        self.tile_off = torch.zeros(H, cap // T, dtype=torch.int32, device=dev)
        self.ovf = torch.zeros(H * ovf_cap, dtype=torch.uint8, device=dev)
        self.head_start = (torch.arange(H + 1, device=dev, dtype=torch.int32) * ovf_cap).contiguous()
        self.ovf_used = torch.zeros(H, dtype=torch.int32, device=dev)
        self.tail = torch.zeros(H, TAIL, D, dtype=torch.bfloat16, device=dev)
        self.base3, self.base4 = base3, base4
        self.enc = TileEncoder(kind, dev)

    def grow(self, ovf_cap):
        new = torch.zeros(self.H * ovf_cap, dtype=torch.uint8, device=self.ovf.device)
        new.view(self.H, ovf_cap)[:, :self.ovf_cap] = self.ovf.view(self.H, self.ovf_cap)
        self.ovf, self.ovf_cap = new, ovf_cap
        self.head_start = (torch.arange(self.H + 1, device=new.device, dtype=torch.int32) * ovf_cap).contiguous()

    def c_store(self) -> _lib.Store:
        return _lib.Store(self.sm.data_ptr(), self.codes.data_ptr(), self.flags.data_ptr(), self.tile_off.data_ptr(), self.ovf.data_ptr(),
                          self.ovf_used.data_ptr(), self.tail.data_ptr(), self.base3.data_ptr(), self.base4.data_ptr())


class CompressedKVCache:
    def __init__(self, n_slots: int, n_kv: int, capacity: int, bases: dict | None = None,
                 ovf_bytes_per_tile: int = 128, device="cuda"):
        """capacity: max tokens per sequence; bases: {'k3','k4','v3','v4'} uint8 [n_kv, D] (None = per-sequence calibration);
        ovf_bytes_per_tile: escape-stream reservation per 16-token tile."""
        if not torch.device(device).type == "cuda":
            raise RuntimeError("CompressedKVCache needs a CUDA device: gaac_b200 has no CPU path")
        _lib.lib()
        self.n_slots, self.n_kv = n_slots, n_kv
        self.cap = (capacity + T - 1) // T * T
        self.H = H = n_slots * n_kv
        self.per_sequence_bases = bases is None
        NB = H if bases is None else n_kv
        def table(key):
            if bases is None: return torch.zeros(NB, D, dtype=torch.uint8, device=device)
            return bases[key].to(device, torch.uint8).reshape(n_kv, D).contiguous()
        ovf_cap = (self.cap // T) * ovf_bytes_per_tile + 8
        self.k = _Store("k", H, self.cap, ovf_cap, table("k3"), table("k4"), device)
        self.v = _Store("v", H, self.cap, ovf_cap, table("v3"), table("v4"), device)
        self.S = torch.zeros(H, dtype=torch.int32, device=device)          # compressed tokens per head
        self.tail_len = torch.zeros(H, dtype=torch.int32, device=device)
        self.growable = True       # set False once CUDA graphs captured the buffer addresses

    @staticmethod
    def bytes_per_slot(n_kv: int, capacity: int, ovf_bytes_per_tile: int = 128, per_sequence_bases: bool = True) -> int:
        """gaac/kv_cache.py:142-146."""
        cap = (capacity + T - 1) // T * T
        per_head = cap * (D + CB + 4) + (cap // T) * 4 + (cap // T) * ovf_bytes_per_tile + 8 + 8 + TAIL * D * 2 + (2 * D if per_sequence_bases else 0)
        return 2 * n_kv * per_head + 8 * n_kv

    # ------------------------------------------------------------------ prefill
    def prefill(self, slot: int, k: torch.Tensor, v: torch.Tensor):
        """Store a sequence's prompt K/V ([L, n_kv, D] bf16, token-major as produced by the model) in `slot`.
        (gaac/kv_cache.py:149-169)"""
        L = k.shape[0]
        assert L <= self.cap, f"sequence of {L} tokens exceeds the cache capacity {self.cap}"
        h0, h1 = slot * self.n_kv, (slot + 1) * self.n_kv
        Sf = L // T * T
        for st, x in ((self.k, k), (self.v, v)):
            xh = x.transpose(0, 1).contiguous()                                # [n_kv, L, D]
            if self.per_sequence_bases:
                c = Codec(self.n_kv, x.device).calibrate(xh)
                st.base3[h0:h1] = c.base3; st.base4[h0:h1] = c.base4
            st.ovf_used[h0:h1] = 0
            if Sf:
                bidx = (torch.arange(h0, h1, device=x.device, dtype=torch.int32) % st.base3.shape[0]).contiguous()
                tb = st.enc.encode_tiles(xh[:, :Sf], st.base3, st.base4, st.sm[h0:h1], st.codes[h0:h1], st.flags[h0:h1], Sf, self.cap, self.n_kv, bidx=bidx)
                _, head_bytes = st.enc.tile_offsets(tb)
                need = int(head_bytes.max()) + TILE_MAX_ESC + 8        # headroom for the next decode tile before check_capacity runs
                if need > st.ovf_cap: self._grow(need)
                st.tile_off[h0:h1, :Sf // T] = st.enc.compact(tb, st.head_start[h0:h1 + 1], st.ovf)
                st.ovf_used[h0:h1] = head_bytes
            if L > Sf: st.tail[h0:h1, :L - Sf] = xh[:, Sf:]
        self.S[h0:h1] = Sf; self.tail_len[h0:h1] = L - Sf

    # ------------------------------------------------------------------ decode step
    def append(self, slots: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
        """One new token per batch row: slots int32 [B] (-1 = skip), k/v [B, n_kv, D] bf16.  One launch, graph-safe.
        (gaac/kv_cache.py:172-181)"""
        k, v = k.contiguous(), v.contiguous()
        K, V = self.k, self.v
        B = slots.numel()
        if B == 0: return
        _lib.check(_lib.lib().gaac_append_kv(K.c_store(), V.c_store(), k.data_ptr(), v.data_ptr(), slots.data_ptr(), B, self.n_kv,
                                             self.tail_len.data_ptr(), self.S.data_ptr(), self.cap, K.ovf_cap, K.base3.shape[0],
                                             _lib.stream_ptr(k.device)), "gaac_append_kv")

    def attention(self, q: torch.Tensor, slots: torch.Tensor, scale: float, max_len: int | None = None, nsplit: int | None = None, out_f32=None):
        """q: [B, n_q, D] bf16 (row b attends over slot slots[b]) -> [B, n_q, D] bf16.  (gaac/kv_cache.py:183-192)"""
        B, n_q, _ = q.shape
        if nsplit is None: nsplit = choose_nsplit_sm100(B, self.n_kv, max_len or self.cap)
        K, V = self.k, self.v
        out = _ext().gaac_attn_launch(K.sm, K.codes, K.flags, K.tile_off, K.ovf, K.head_start, K.base3, K.base4,
                                      V.sm, V.codes, V.flags, V.tile_off, V.ovf, V.head_start, V.base3, V.base4,
                                      q.reshape(B * n_q, D).contiguous(), slots, n_q, self.n_kv, self.S, self.cap, scale, nsplit,
                                      K.tail, V.tail, self.tail_len, TAIL, out_f32=out_f32)
        return out.view(B, n_q, D)

    # ------------------------------------------------------------------ housekeeping
    def max_escape_bytes(self) -> torch.Tensor:
        return torch.maximum(self.k.ovf_used.max(), self.v.ovf_used.max())

    def check_capacity(self, used: int | None = None):
        """Call at least once every 16 decode steps: each head finalizes at most one tile in 16 steps, so keeping one
        worst-case tile of headroom makes the escape streams overflow-proof between checks.  (gaac/kv_cache.py:198-203)"""
        used = int(self.max_escape_bytes()) if used is None else used
        if used + TILE_MAX_ESC + 8 > self.k.ovf_cap: self._grow(used + TILE_MAX_ESC + 8)

    def _grow(self, need: int):
        if not self.growable:
            raise RuntimeError(f"escape stream needs {need} B per head but holds {self.k.ovf_cap} B and CUDA graphs are captured; "
                               "raise gaac_ovf_bytes_per_tile or calibrate the exponent bases on representative prompts")
        cap = max(2 * self.k.ovf_cap, need + 4096 + 7) // 8 * 8
        self.k.grow(cap); self.v.grow(cap)

    def decompress(self, slot: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Bit-exact BF16 K/V of `slot` ([L, n_kv, D] each) from the compressed tiles + raw tail.  (gaac/kv_cache.py:211-226)"""
        h0, h1 = slot * self.n_kv, (slot + 1) * self.n_kv
        S, tl_ = int(self.S[h0]), int(self.tail_len[h0])
        out = []
        for st in (self.k, self.v):
            parts = []
            if S:
                per_seq = st.base3.shape[0] != self.n_kv
                b3, b4 = (st.base3[h0:h1], st.base4[h0:h1]) if per_seq else (st.base3, st.base4)
                pg = Page(st.sm[h0:h1], st.codes[h0:h1], st.flags[h0:h1], None,
                          st.ovf, st.head_start[h0:h1 + 1], st.tile_off[h0:h1], b3, b4, self.n_kv, S, self.n_kv, st.kind)
                parts.append(Codec.decode(pg))
            parts.append(st.tail[h0:h1, :tl_])
            out.append(torch.cat(parts, 1).transpose(0, 1).contiguous())
        return out[0], out[1]

    def stats(self) -> dict:
        """Bytes in use (compressed tiles + escapes + metadata + raw tails) vs the BF16 bytes of the same tokens.
        (gaac/kv_cache.py:228-234)"""
        S = int(self.S.sum()); tl_ = int(self.tail_len.sum())
        esc = int(self.k.ovf_used.sum() + self.v.ovf_used.sum())
        used = 2 * (S * (D + CB + 4) + (S // T) * 4 + tl_ * D * 2) + esc
        bf16 = 2 * (S + tl_) * D * 2
        return dict(tokens=(S + tl_) // max(1, self.n_kv), bytes_used=used, bf16_bytes=bf16, ratio=bf16 / max(1, used))
