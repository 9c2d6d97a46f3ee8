"""Decode attention over the paged block buffer, head_dim 128 (mirror of gaac/vllm/paged_kernel.py).

Block (16 tokens, all n_kv heads, K and V) = 2*n_kv tile slots of TS bytes each, slot t = 2*kvh + kind:
  [0,2048) sign/mantissa (fragment order) | [2048,2816) 3-bit codes | [2816,2880) 16 x u32 row tags | [2880,TS) escape slot.
Mode table MT[p]: p itself -> compressed in the slot; ~r -> raw bf16 tile r of the side pool (the sequence's still-filling
block, or a finalized tile whose escapes did not fit the slot).  Block table, mode table, raw tiles and compressed tiles are
all read by the one fused kernel: there is no decompression pass.
"""
from __future__ import annotations
import torch
from .. import _lib
from ..kernel import workspace, choose_nsplit_sm100


def choose_nsplit(B, n_kv, S, target_ctas=96, min_tok=512, cap=48):
    """The reference's heuristic verbatim (gaac/vllm/paged_kernel.py:291-293)."""
    return min(max(1, target_ctas // (B * n_kv)), max(1, S // min_tok), cap)


def paged_attention(q, out, buf, raw, mt, bt, seq_lens, bases, TS, n_q, n_kv, nsplit=None, out_f32=None):
    """q: [B, n_q, 128] bf16 contiguous; out: [B, n_q*128] bf16 (written); buf: uint8 flat block buffer; raw: [Pr,16,128] bf16;
    mt: int32 [num_blocks*2*n_kv]; bt: int32 [B, max_blocks]; seq_lens: int32 [B]; bases: (b3k,b4k,b3v,b4v) uint8 [n_kv,128].
    (gaac/vllm/paged_kernel.py:296-301; the softmax scale is 1/sqrt(128) as there.)  nsplit=None picks the B200 split count
    for a ragged batch whose longest row fills the block table; an explicit nsplit is honoured as given."""
    B = q.shape[0]; D = q.shape[-1]
    G = n_q // max(1, n_kv)
    if not (1 <= G <= 8): raise RuntimeError("G must be 1..8")
    if TS % 16: raise RuntimeError("tile stride must be a multiple of 16")
    if not q.is_cuda: raise RuntimeError("gaac_b200 attention needs CUDA tensors: there is no CPU path")
    if nsplit is None: nsplit = choose_nsplit_sm100(B, n_kv, bt.shape[1] * 16, ragged=True)
    st = _lib.Paged(buf.data_ptr(), raw.data_ptr(), mt.data_ptr(), None, None, None,
                    bases[0].data_ptr(), bases[1].data_ptr(), bases[2].data_ptr(), bases[3].data_ptr(), n_kv, TS, TS - 2880)
    ws = workspace(q.device, B, n_q, nsplit)
    _lib.check(_lib.lib().gaac_paged_decode_attn(st, bt.data_ptr(), _lib.row_stride(bt), seq_lens.data_ptr(), q.data_ptr(), B, n_q, 1.0 / (D ** 0.5), int(nsplit),
                                                 ws.data_ptr(), ws.numel(), out.data_ptr(), _lib.ptr(out_f32), _lib.stream_ptr(q.device)), "gaac_paged_decode_attn")
    return out
