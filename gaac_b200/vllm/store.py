"""Store path of the paged layout (mirror of gaac/vllm/store.py): writes new K/V tokens into the compressed block buffer.

Block (16 tokens, all n_kv heads, K and V) = 2*n_kv tile slots of TS bytes, slot t = 2*kvh + kind; physical tile
p = block*(2*n_kv) + t.  Entry e (built on the host) = (block id, first token row of this step in the K/V tensors, block
offset of that row, number of new rows).
  * block not full after this step -> new rows go to the raw side pool RAW[r] (popped from a per-layer free stack when the
                                      block starts), MT[p] = ~r
  * block completes this step      -> the 16 rows are compressed into the block's tile slot when the escape bytes fit the
                                      slot (MT[p] = p, raw tile released) or kept raw (MT[p] = ~r)
Pops happen only in the store kernel, pushes only in the free kernel that follows it.
"""
from __future__ import annotations
import torch
from .. import _lib

D = 128
SM_OFF, CD_OFF, FL_OFF, OVF_OFF = 0, 2048, 2816, 2880   # byte layout of a tile slot; TS = OVF_OFF + OVF_SLOT


class LayerState:
    """Per-layer device state outside the block buffer: raw side pool, mode table, free stack, bases (gaac/vllm/store.py:177-203)."""

    def __init__(self, num_blocks: int, n_kv: int, raw_tiles: int, bases: dict, ovf_slot: int, device):
        if torch.device(device).type != "cuda":
            raise RuntimeError("LayerState needs a CUDA device: gaac_b200 has no CPU path")
        _lib.lib()
        self.n_kv, self.ovf_slot, self.TS = n_kv, ovf_slot, OVF_OFF + ovf_slot
        assert self.TS % 16 == 0, "OVF_SLOT must be a multiple of 16"
        self.mt = torch.arange(num_blocks * 2 * n_kv, dtype=torch.int32, device=device)          # every tile starts 'compressed at itself'
        self.raw = torch.zeros(raw_tiles, 16, D, dtype=torch.bfloat16, device=device)
        self.stack = torch.arange(raw_tiles, dtype=torch.int32, device=device); self.top = torch.tensor([raw_tiles], dtype=torch.int32, device=device)
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        self.b3k, self.b4k, self.b3v, self.b4v = (bases[k].to(device).to(torch.uint8).contiguous() for k in ("k3", "k4", "v3", "v4"))

    @property
    def bases(self):
        return (self.b3k, self.b4k, self.b3v, self.b4v)

    def c_state(self, buf: torch.Tensor) -> _lib.Paged:
        return _lib.Paged(buf.data_ptr(), self.raw.data_ptr(), self.mt.data_ptr(), self.stack.data_ptr(), self.top.data_ptr(), self.err.data_ptr(),
                          self.b3k.data_ptr(), self.b4k.data_ptr(), self.b3v.data_ptr(), self.b4v.data_ptr(), self.n_kv, self.TS, self.ovf_slot)

    def store(self, key: torch.Tensor, value: torch.Tensor, buf: torch.Tensor, ent: torch.Tensor, freeq: torch.Tensor):
        """key/value: [num_tokens, n_kv, D] bf16 (or int16 views of them); buf: uint8 flat block buffer; ent: int32 [E,4] =
        (blk, tok0, off0, n); freeq: int32 [E*2*n_kv] scratch.  (gaac/vllm/store.py:204-213)"""
        E = ent.shape[0]
        if E == 0: return
        assert key.stride(-1) == 1 and value.stride(-1) == 1
        assert (key.shape[1] == 1 or key.stride(1) == D) and (value.shape[1] == 1 or value.stride(1) == D)
        _lib.check(_lib.lib().gaac_paged_store(self.c_state(buf), key.data_ptr(), value.data_ptr(), key.stride(0), value.stride(0),
                                               ent.data_ptr(), E, freeq.data_ptr(), _lib.stream_ptr(buf.device)), "gaac_paged_store")

    def decode_blocks(self, buf: torch.Tensor, pairs: torch.Tensor, sk: torch.Tensor, sv: torch.Tensor):
        """pairs: int32 [P,3] (block, first scratch row, valid rows); sk/sv: flat scratch K/V [rows, n_kv, D] bf16 (written).
        (gaac/vllm/store.py:215-221)"""
        P = pairs.shape[0]
        if P == 0: return
        assert sk.stride(0) == self.n_kv * D and sv.stride(0) == self.n_kv * D
        _lib.check(_lib.lib().gaac_paged_decode_blocks(self.c_state(buf), pairs.data_ptr(), P, sk.data_ptr(), sv.data_ptr(), sk.stride(0),
                                                       _lib.stream_ptr(buf.device)), "gaac_paged_decode_blocks")

    def release_blocks(self, blocks: torch.Tensor):
        """blocks: int32 [F] block ids whose content is dead (freed without prefix caching).  (gaac/vllm/store.py:223-227)"""
        F = blocks.shape[0]
        if F == 0: return
        st = _lib.Paged(self.raw.data_ptr(), self.raw.data_ptr(), self.mt.data_ptr(), self.stack.data_ptr(), self.top.data_ptr(), self.err.data_ptr(),
                        self.b3k.data_ptr(), self.b4k.data_ptr(), self.b3v.data_ptr(), self.b4v.data_ptr(), self.n_kv, self.TS, self.ovf_slot)
        _lib.check(_lib.lib().gaac_paged_release(st, blocks.data_ptr(), F, _lib.stream_ptr(blocks.device)), "gaac_paged_release")
