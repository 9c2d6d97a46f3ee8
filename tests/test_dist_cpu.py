"""Multi-rank host logic on CPU: world_size-2 gloo process group, partials all-gathered and merged; sharding helpers.
The merge function is injected (the oracle's), so no GPU and no CUDA library call is involved."""
import os, socket
import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from oracle import gaac_oracle as O
from gaac_b200 import dist as gd


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); return s.getsockname()[1]


def _partial(q16, k16, v16, scale):
    """(m, l, acc) of one token range in fp64 -> [n_q, 130] float32.  k16/v16 [L, n_kv, D]."""
    n_q, n_kv = q16.shape[0], k16.shape[1]; G = n_q // n_kv
    out = np.zeros((n_q, 130), np.float32)
    for h in range(n_q):
        k, v = O.bf16_to_f64(k16[:, h // G]), O.bf16_to_f64(v16[:, h // G])
        if k.shape[0] == 0:
            out[h, 0] = -np.inf; continue
        s = (k @ O.bf16_to_f64(q16[h])) * scale
        m = s.max(); p = np.exp(s - m)
        out[h, 0], out[h, 1], out[h, 2:] = m, p.sum(), p @ v
    return out


def _worker(rank, world, port, S, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n_kv, G = 2, 4
    k16 = O.kv_like(n_kv, S, 1).transpose(1, 0, 2); v16 = O.kv_like(n_kv, S, 2).transpose(1, 0, 2)
    rng = np.random.default_rng(3)
    q16 = O.f32_to_bf16((rng.standard_normal((n_kv * G, 128)) * 0.1).astype(np.float32))
    lo, hi = gd.split_context(S, world, rank)
    part = torch.from_numpy(_partial(q16, k16[lo:hi], v16[lo:hi], 128 ** -0.5))
    combine = lambda pm, pl, pa: torch.from_numpy(O.combine_partials(pm.numpy(), pl.numpy(), pa.numpy()))
    out = gd.merge_partials(part, combine_fn=combine).numpy()
    ref = O.attention_ref(q16, k16, v16, 128 ** -0.5)
    ret[rank] = float(np.abs(out - ref).max() / max(1.0, np.abs(ref).max()))
    dist.destroy_process_group()


@pytest.mark.parametrize("S", [40, 1000])          # 40 tokens: rank 0 gets 1 tile, rank 1 the ragged rest
def test_context_split_merge_two_ranks(S):
    world, port = 2, _free_port()
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, port, S, ret), nprocs=world, join=True)
    assert len(ret) == world and max(ret.values()) < 1e-5, dict(ret)


def test_split_context_covers_everything_tile_aligned():
    for S in (0, 5, 16, 333, 65536, 131072):
        for world in (1, 2, 4, 8):
            r = [gd.split_context(S, world, k) for k in range(world)]
            assert r[0][0] == 0 and r[-1][1] == S
            for a, b in zip(r, r[1:]):
                assert a[1] == b[0] and a[1] % 16 == 0
            assert max(hi - lo for lo, hi in r) - min(hi - lo for lo, hi in r) <= 16 + 15


def test_shard_sequences_balances_tokens():
    rng = np.random.default_rng(0)
    lens = rng.integers(4096, 65537, 16).tolist()
    for world in (1, 2, 4, 8):
        sh = gd.shard_sequences(lens, world)
        assert sorted(i for s in sh for i in s) == list(range(16))
        load = [sum(lens[i] for i in s) for s in sh]
        assert max(load) <= sum(lens) / world + max(lens)


def test_shard_heads():
    for n_kv, world in ((8, 8), (8, 4), (8, 3), (2, 4)):
        hs = [list(gd.shard_heads(n_kv, world, r)) for r in range(world)]
        assert sorted(h for x in hs for h in x) == list(range(n_kv))
        assert max(len(x) for x in hs) - min(len(x) for x in hs) <= 1
