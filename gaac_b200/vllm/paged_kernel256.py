"""Decode attention over the paged block buffer, head_dim 256 (mirror of gaac/vllm/paged_kernel256.py).

A 256-dim head is stored as two 128-dim half-heads in neighbouring tile slots of a block, each half-head with its own exponent
bases: the store (LayerState with n_kv = 2 * kv heads), the block decoder and the bases all work on half-heads, only this
kernel puts the halves together.  In the kernel two warps share one stream of tiles, one per half: each rebuilds its half of the K
tile, the two partial scores meet in shared memory, both warps run the same softmax step and each accumulates the 128 output
dimensions of its half of V.
"""
from __future__ import annotations
import torch
from .. import _lib
from ..kernel import workspace, choose_nsplit_sm100


def paged_attention256(q, out, buf, raw, mt, bt, seq_lens, bases, TS, n_q, n_kv, nsplit=None, scale=None, out_f32=None):
    """q: [B, n_q, 256] bf16 contiguous; out: [B, n_q*256] bf16 (written); n_kv: 256-dim kv heads; bases: (b3k, b4k, b3v, b4v) uint8
    [2*n_kv, 128], one row per half-head; the other arguments as paged_attention.  scale defaults to 1/sqrt(256).
    (gaac/vllm/paged_kernel256.py:299-305)"""
    B = q.shape[0]
    G = n_q // max(1, n_kv)
    if q.shape[-1] != 256: raise RuntimeError("head_dim must be 256")
    if not (1 <= G <= 8 and G * n_kv == n_q): raise RuntimeError("GQA group size must be 1..8")
    if TS % 16: raise RuntimeError("tile stride must be a multiple of 16")
    if not q.is_cuda: raise RuntimeError("gaac_b200 attention needs CUDA tensors: there is no CPU path")
    if nsplit is None: nsplit = choose_nsplit_sm100(B, n_kv, bt.shape[1] * 16, ragged=True)
    st = _lib.Paged(buf.data_ptr(), raw.data_ptr(), mt.data_ptr(), None, None, None,
                    bases[0].data_ptr(), bases[1].data_ptr(), bases[2].data_ptr(), bases[3].data_ptr(), 2 * n_kv, TS, TS - 2880)
    ws = workspace(q.device, B, 2 * n_q, nsplit)
    _lib.check(_lib.lib().gaac_paged_decode_attn256(st, bt.data_ptr(), _lib.row_stride(bt), seq_lens.data_ptr(), q.data_ptr(), B, n_q,
                                                    float(scale) if scale is not None else 256 ** -0.5, int(nsplit), ws.data_ptr(), ws.numel(),
                                                    out.data_ptr(), _lib.ptr(out_f32), _lib.stream_ptr(q.device)), "gaac_paged_decode_attn256")
    return out
