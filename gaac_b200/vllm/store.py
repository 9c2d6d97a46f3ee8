"""Writing new K/V tokens into the paged block buffer (drop-in for gaac/vllm/store.py).

The serving engine owns one flat uint8 buffer per layer, cut into 16-token blocks.  A block has one tile slot of TS bytes for
every (kv head, kind): slot index inside the block t = 2*kvh + kind (kind 0 = K, 1 = V), so tile slot p = block*2*n_kv + t sits
at byte p*TS.  What the engine tells the store per decode or prefill step is a list of entries, one per touched block:
(block id, row of the step's K/V tensors where this block's new tokens start, position inside the block where they go, how many).

Two cases per tile slot.  A block that is still filling keeps its rows as plain BF16 in a tile of a side pool (`raw`); the
pool tile is taken from a free stack the first time the block is written, and the mode table remembers it as mt[p] = ~r.  A block
that the step completes is compressed: if the tile's escape bytes fit the slot's escape area the tile goes into its slot,
mt[p] = p again, and the pool tile goes back on the stack; if they do not fit the tile simply stays in the pool for good.
Pool tiles are popped only by the store kernel and pushed back only by the kernel launched right behind it, so the two never
race on the stack.  A pop from an empty stack is counted in `err` instead of trapping.
"""
from __future__ import annotations
import torch
from .. import _lib

D = 128
SM_OFF, CD_OFF, FL_OFF, OVF_OFF = 0, 2048, 2816, 2880   # where sign/mantissa, codes, tag words and escapes start inside a tile slot; TS = OVF_OFF + ovf_slot


class LayerState:
    """Everything of one layer that lives outside the block buffer (gaac/vllm/store.py:177-203): the side pool of raw tiles, the
    mode table, the free stack with its top index, the error counter and the four base tables."""

    def __init__(self, num_blocks: int, n_kv: int, raw_tiles: int, bases: dict, ovf_slot: int, device):
        if torch.device(device).type != "cuda":
            raise RuntimeError("LayerState needs a CUDA device: gaac_b200 has no CPU path")
        _lib.lib()
        self.n_kv, self.ovf_slot, self.TS = n_kv, ovf_slot, OVF_OFF + ovf_slot
        assert self.TS % 16 == 0, "OVF_SLOT must be a multiple of 16"
        i32 = dict(dtype=torch.int32, device=device)
        n_slots = num_blocks * 2 * n_kv
        self.mt = torch.arange(n_slots, **i32)                                   # mt[p] == p: nothing of the block is in the pool
        self.raw = torch.zeros(raw_tiles, 16, D, dtype=torch.bfloat16, device=device)
        self.stack = torch.arange(raw_tiles, **i32)                              # all pool tiles free
        self.top = torch.full((1,), raw_tiles, **i32)
        self.err = torch.zeros(1, **i32)
        self.b3k, self.b4k, self.b3v, self.b4v = (bases[name].to(device).to(torch.uint8).contiguous() for name in ("k3", "k4", "v3", "v4"))

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
        _lib.check(_lib.lib().gaac_paged_store(self.c_state(buf), key.data_ptr(), value.data_ptr(), _lib.row_stride(key), _lib.row_stride(value),
                                               ent.data_ptr(), E, freeq.data_ptr(), _lib.stream_ptr(buf.device)), "gaac_paged_store")

    def decode_blocks(self, buf: torch.Tensor, pairs: torch.Tensor, sk: torch.Tensor, sv: torch.Tensor):
        """pairs: int32 [P,3] (block, first scratch row, valid rows); sk/sv: flat scratch K/V [rows, n_kv, D] bf16 (written).
        (gaac/vllm/store.py:215-221)"""
        P = pairs.shape[0]
        if P == 0: return
        assert _lib.row_stride(sk) == self.n_kv * D and _lib.row_stride(sv) == self.n_kv * D
        _lib.check(_lib.lib().gaac_paged_decode_blocks(self.c_state(buf), pairs.data_ptr(), P, sk.data_ptr(), sv.data_ptr(), _lib.row_stride(sk),
                                                       _lib.stream_ptr(buf.device)), "gaac_paged_decode_blocks")

    def release_blocks(self, blocks: torch.Tensor):
        """blocks: int32 [F] block ids whose content is dead (freed without prefix caching).  (gaac/vllm/store.py:223-227)"""
        F = blocks.shape[0]
        if F == 0: return
        st = _lib.Paged(self.raw.data_ptr(), self.raw.data_ptr(), self.mt.data_ptr(), self.stack.data_ptr(), self.top.data_ptr(), self.err.data_ptr(),
                        self.b3k.data_ptr(), self.b4k.data_ptr(), self.b3v.data_ptr(), self.b4v.data_ptr(), self.n_kv, self.TS, self.ovf_slot)
        _lib.check(_lib.lib().gaac_paged_release(st, blocks.data_ptr(), F, _lib.stream_ptr(blocks.device)), "gaac_paged_release")
