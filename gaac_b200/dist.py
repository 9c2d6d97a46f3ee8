"""Multi-GPU partitioning of the compressed-KV decode path (one process per GPU, torch.distributed).

The reference runs compressed KV on a single GPU (nanovllm/config.py:37 asserts tensor_parallel_size == 1); this module is
what a multi-GPU deployment of the same path needs:

  * shard_sequences / shard_heads: batched decode and kv-head sharding - independent shards, no collective on the path;
  * split_context + ContextSplitAttention: batch-1 long context - every rank attends over its contiguous, tile-aligned token
    range and writes an un-normalised partial (m, l, acc[128]) per query head; the partials are all-gathered (NCCL over
    NVLink on GPUs) and merged with the split-merge algebra of gaac/kernel.py:281-294.
"""
from __future__ import annotations
import torch
import torch.distributed as dist

T = 16


def shard_sequences(seq_lens, world: int) -> list[list[int]]:
    """Sequence indices per rank, balanced by token count (longest first onto the lightest rank)."""
    order = sorted(range(len(seq_lens)), key=lambda i: -int(seq_lens[i]))
    load = [0] * world
    out: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i); load[r] += int(seq_lens[i])
    return [sorted(x) for x in out]


def shard_heads(n_kv: int, world: int, rank: int) -> range:
    """KV heads of `rank` (contiguous, as even as possible).  Query heads kvh*G .. kvh*G+G-1 go with their kv head."""
    base, extra = divmod(n_kv, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def split_context(S: int, world: int, rank: int) -> tuple[int, int]:
    """Token range [lo, hi) of `rank`: contiguous, aligned to 16-token tiles; the ragged end belongs to the last rank."""
    tiles = (S + T - 1) // T
    lo, hi = tiles * rank // world, tiles * (rank + 1) // world
    return lo * T, min(hi * T, S)


def merge_partials(part: torch.Tensor, group=None, combine_fn=None, out_f32: torch.Tensor | None = None) -> torch.Tensor:
    """part: [n_heads, 130] fp32 (m in natural-log units, l, acc[128]) of this rank -> merged output [n_heads, 128] on every rank.
    combine_fn(pm, pl, pa) merges [n_heads, world] / [n_heads, world, 128]; default: the CUDA merge kernel (gaac_combine)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        gathered = part.unsqueeze(0)
    else:
        gathered = torch.empty(world * part.shape[0], *part.shape[1:], dtype=part.dtype, device=part.device)   # concatenated along dim 0
        dist.all_gather_into_tensor(gathered, part.contiguous(), group=group)
        gathered = gathered.view(world, *part.shape)
    if combine_fn is None:
        from .kernel import combine_parts
        return combine_parts(gathered.contiguous(), out_f32=out_f32)          # one launch on the gathered buffer as it is
    g = gathered.permute(1, 0, 2)                                   # [n_heads, world, 130]
    return combine_fn(g[:, :, 0].contiguous(), g[:, :, 1].contiguous(), g[:, :, 2:].contiguous())


class PeerExchange:
    """Receive buffers of all ranks, mapped into every rank (peer memory over NVLink), for the fused partial exchange: the
    attention kernel stores its partial rows into every rank's buffer as 8-byte entries (value + exchange number), and either
    the same launch (fused) or gaac_exchange_merge waits for all ranks' rows and merges them.  Built on torch's symmetric
    memory (one rendezvous at construction) with NVLink multicast binding switched off (plain peer loads and stores only);
    raises when the mapping is unavailable, and the caller falls back to the NCCL all-gather.
    n_heads = B * n_q rows per exchange at most.  (`groups` is accepted for callers written against the flag-based exchange
    and ignored.)"""

    def __init__(self, n_heads: int, device, group=None, groups: int | None = None):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")      # before the first rendezvous of the process
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.n_heads = n_heads
        self._buf = symm.empty(self._layout(self.world, self.n_heads), dtype=torch.uint8, device=device)
        self._buf.zero_()
        self._hdl = symm.rendezvous(self._buf, group)
        ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        self._setup(ptrs, device)
        torch.cuda.synchronize(device)
        dist.barrier(group)                                     # every rank's buffer is zero before anyone pushes

    @staticmethod
    def _layout(world: int, n_heads: int) -> int:
        """Bytes of a receive buffer: 2 x world x n_heads rows of 130 eight-byte entries."""
        return (2 * world * n_heads * 130 * 8 + 255) // 256 * 256

    def _setup(self, ptrs, device):
        from . import _lib
        self._recv = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self._state = torch.zeros(3, dtype=torch.int32, device=device)                     # exchange number, ticket, err
        self.x = _lib.Exchange(self._recv.data_ptr(), self._state.data_ptr(), self._state.data_ptr() + 4,
                               self._state.data_ptr() + 8, self.rank, self.world, self.n_heads)

    @classmethod
    def local(cls, bufs, rank: int, n_heads: int, groups: int | None = None):
        """An exchange whose 'ranks' are buffers on one GPU (uint8 tensors made by local_buffer): lets one process run the ranks
        one after the other in stream order.  Only the last rank to push may use the fused launch (everything it waits for is
        there already); the others push and merge with separate launches."""
        self = cls.__new__(cls)
        self.world, self.rank, self.n_heads = len(bufs), rank, n_heads
        self._buf = bufs[rank]
        self._setup([b.data_ptr() for b in bufs], bufs[rank].device)
        return self

    @classmethod
    def local_buffer(cls, world: int, n_heads: int, device, groups: int | None = None) -> torch.Tensor:
        return torch.zeros(cls._layout(world, n_heads), dtype=torch.uint8, device=device)

    def merge(self, groups: int | None = None, out_f32: torch.Tensor | None = None, n_heads: int | None = None) -> torch.Tensor:
        """Launch the wait-and-merge kernel on the current stream (after a push-only launch); returns [n_heads, 128] bf16."""
        from . import _lib
        n_heads = self.n_heads if n_heads is None else n_heads
        out = torch.empty(n_heads, 128, dtype=torch.bfloat16, device=self._state.device)
        _lib.check(_lib.lib().gaac_exchange_merge(self.x, n_heads, out.data_ptr(), _lib.ptr(out_f32),
                                                  _lib.stream_ptr(self._state.device)), "gaac_exchange_merge")
        return out

    def error(self) -> bool:
        """True when a wait ran out (a peer never delivered); reads the device flag, so it synchronises."""
        return bool(self._state[2].item())


class ContextSplitAttention:
    """Batch-1 decode attention with the context split across the ranks of a process group.

    Every rank holds the Pages of its own token range (kp, vp: kinds 'k' / 'v', H = n_kv heads).  __call__(q) attends over the
    local range and merges the ranks' partials; every rank returns the full [n_q, 128] output."""

    def __init__(self, kp, vp, n_q: int, scale: float | None = None, nsplit: int | None = None, group=None, exchange: str = "auto", fused: bool = True):
        """exchange: 'p2p' = partial rows pushed by the attention kernel into peer memory (PeerExchange), 'nccl' = NCCL
        all-gather + merge kernel, 'auto' = p2p when the symmetric-memory rendezvous succeeds, else nccl.  fused (p2p only):
        the attention launch also waits for the other ranks and merges (one launch per layer); it needs the whole grid
        resident, so it is dropped when n_kv * nsplit exceeds the SM count."""
        from .kernel import choose_nsplit_sm100, SM_COUNT_B200
        self.kp, self.vp, self.n_q, self.group = kp, vp, n_q, group
        self.n_kv = kp.H
        self.peer = None
        if exchange in ("auto", "p2p") and dist.is_initialized() and dist.get_world_size(group) > 1 and kp.sm.is_cuda:
            try:
                self.peer = PeerExchange(n_q, kp.sm.device, group, groups=self.n_kv)
            except Exception:
                if exchange == "p2p":
                    raise
        self.scale = scale if scale is not None else 128 ** -0.5
        self.nsplit = nsplit or choose_nsplit_sm100(1, self.n_kv, max(kp.S, 1))
        self.fused = fused and self.n_kv * self.nsplit <= SM_COUNT_B200
        self._part = torch.empty(n_q, 130, dtype=torch.float32, device=kp.sm.device)

    def partial(self, q: torch.Tensor) -> torch.Tensor:
        from .kernel import _pages_call
        _pages_call(q.reshape(1, self.n_q, 128), self.kp, self.vp, 1, self.n_q, self.n_kv, self.scale, self.nsplit, part=self._part)
        return self._part

    def __call__(self, q: torch.Tensor, out_f32: torch.Tensor | None = None) -> torch.Tensor:
        if self.peer is None:
            return merge_partials(self.partial(q), self.group, out_f32=out_f32)
        from .kernel import _pages_call
        q3 = q.reshape(1, self.n_q, 128)
        if self.fused:
            out = torch.empty(self.n_q, 128, dtype=torch.bfloat16, device=q.device)
            _pages_call(q3, self.kp, self.vp, 1, self.n_q, self.n_kv, self.scale, self.nsplit, out=out, out_f32=out_f32, exchange=self.peer.x, fused=True)
            return out
        _pages_call(q3, self.kp, self.vp, 1, self.n_q, self.n_kv, self.scale, self.nsplit, exchange=self.peer.x)
        return self.peer.merge(self.n_kv, out_f32=out_f32)
