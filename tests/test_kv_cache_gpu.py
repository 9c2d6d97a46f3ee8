"""Slot cache (layout A) on the GPU: prefill, append, attention with tails and padded rows, CUDA-graph decode step, and byte
parity with the fixtures produced by the reference.  Cases follow the reference's tests/test_kv_cache.py:32-86."""
import numpy as np
import pytest
from common import golden, sha, to_bf16_cuda, bits, assert_attention_close
from oracle import gaac_oracle as O

pytestmark = pytest.mark.gpu
N_KV, G, SCALE = 4, 4, 128 ** -0.5


def _tok(x16):                 # [n_kv, L, D] -> token-major [L, n_kv, D]
    return np.ascontiguousarray(x16.transpose(1, 0, 2))


def _bases(seed):
    import torch
    k, v = _tok(O.kv_like(N_KV, 4096, seed)), _tok(O.kv_like(N_KV, 4096, seed + 1))
    k3, k4 = O.bases_from_hist(O.exponent_hist_fast(k, N_KV), N_KV); v3, v4 = O.bases_from_hist(O.exponent_hist_fast(v, N_KV), N_KV)
    return {n: torch.from_numpy(a) for n, a in (("k3", k3), ("k4", k4), ("v3", v3), ("v4", v4))}


def _check(cache, hist, slots_l, q16):
    import torch
    slots = torch.tensor(slots_l, dtype=torch.int32, device="cuda")
    o32 = torch.empty(len(slots_l), N_KV * G, 128, dtype=torch.float32, device="cuda")
    out = cache.attention(to_bf16_cuda(q16), slots, SCALE, out_f32=o32)
    for b, s in enumerate(slots_l):
        if s < 0:
            assert out[b].abs().max().item() == 0
            continue
        k, v = hist[s]
        ref, _ = assert_attention_close(o32[b].cpu().numpy(), q16[b], k, v, SCALE, (b, s))
        assert np.abs(out[b].float().cpu().numpy() - ref).max() <= 2e-2 * np.abs(ref).max() + 1e-3
        dk, dv = cache.decompress(s)
        assert np.array_equal(bits(dk), k) and np.array_equal(bits(dv), v)


@pytest.mark.parametrize("static_bases", [True, False])
def test_slots_prefill_append(static_bases):
    from gaac_b200 import CompressedKVCache
    import torch
    cache = CompressedKVCache(n_slots=4, n_kv=N_KV, capacity=1024, bases=_bases(10) if static_bases else None)
    lens = {0: 37, 2: 500, 3: 16}
    hist = {}
    for s, L in lens.items():
        k, v = _tok(O.kv_like(N_KV, L, 20 + s)), _tok(O.kv_like(N_KV, L, 40 + s))
        cache.prefill(s, to_bf16_cuda(k), to_bf16_cuda(v)); hist[s] = (k, v)
    rng = np.random.default_rng(0)
    for step in range(40):
        slots_l = [3, 0, 2, -1] if step % 3 else [2, 3, -1, 0]
        slots = torch.tensor(slots_l, dtype=torch.int32, device="cuda")
        k = O.f32_to_bf16((rng.standard_normal((4, N_KV, 128)) * 0.5).astype(np.float32))
        v = O.f32_to_bf16((rng.standard_normal((4, N_KV, 128)) * 0.5).astype(np.float32))
        cache.append(slots, to_bf16_cuda(k), to_bf16_cuda(v))
        for b, s in enumerate(slots_l):
            if s >= 0: hist[s] = (np.concatenate([hist[s][0], k[b:b + 1]]), np.concatenate([hist[s][1], v[b:b + 1]]))
        if step % 16 == 15: cache.check_capacity()
        if step % 13 == 0 or step == 39:
            q16 = O.f32_to_bf16((rng.standard_normal((4, N_KV * G, 128)) * 0.1).astype(np.float32))
            _check(cache, hist, slots_l, q16)
    st = cache.stats()
    assert st["tokens"] == sum(h[0].shape[0] for h in hist.values()) and st["ratio"] > 1.0
    k, v = _tok(O.kv_like(N_KV, 64, 99)), _tok(O.kv_like(N_KV, 64, 98))      # slot reuse
    cache.prefill(0, to_bf16_cuda(k), to_bf16_cuda(v)); hist[0] = (k, v)
    _check(cache, hist, [0], O.f32_to_bf16((rng.standard_normal((1, N_KV * G, 128)) * 0.1).astype(np.float32)))


@pytest.mark.parametrize("mode", ["static", "perseq"])
def test_cache_bytes_match_reference_fixture(mode):
    """Same prefill + 30 appends as the fixture script ran through the reference; every buffer byte-identical."""
    import torch
    from gaac_b200 import CompressedKVCache
    g = golden("slot_cache")
    bases = {b: torch.from_numpy(g[f"bases_{b}"]) for b in ("k3", "k4", "v3", "v4")} if mode == "static" else None
    cache = CompressedKVCache(n_slots=2, n_kv=2, capacity=96, bases=bases)
    cache.prefill(1, to_bf16_cuda(g[f"{mode}_prefill_k"]), to_bf16_cuda(g[f"{mode}_prefill_v"]))
    slots = torch.tensor([1, -1], dtype=torch.int32, device="cuda")
    kn, vn = g[f"{mode}_new_k"], g[f"{mode}_new_v"]
    for step in range(kn.shape[0]):
        cache.append(slots, to_bf16_cuda(kn[step]), to_bf16_cuda(vn[step]))
    assert np.array_equal(cache.S.cpu().numpy(), g[f"{mode}_S"]) and np.array_equal(cache.tail_len.cpu().numpy(), g[f"{mode}_tail_len"])
    for nm, st in (("k", cache.k), ("v", cache.v)):
        assert st.ovf_cap == int(g[f"{mode}_{nm}_ovf_cap"])
        for f in ("sm", "codes", "flags", "tile_off", "ovf", "ovf_used", "base3", "base4"):
            assert sha(getattr(st, f).cpu().numpy()) == str(g[f"{mode}_{nm}_{f}_sha"]), (nm, f)
        tl = int(cache.tail_len[2])
        assert np.array_equal(bits(st.tail)[:, :tl], g[f"{mode}_{nm}_tail"][:, :tl])
    s = cache.stats()
    assert [s["tokens"], s["bytes_used"], s["bf16_bytes"]] == g[f"{mode}_stats"].tolist()
    assert [CompressedKVCache.bytes_per_slot(2, 96), CompressedKVCache.bytes_per_slot(8, 1000, 64, False)] == g["bytes_per_slot"].tolist()


def test_cuda_graph_decode_step():
    """append + attention captured in one CUDA graph, 20 replays (tests/test_kv_cache.py:59-86)."""
    import torch
    from gaac_b200 import CompressedKVCache
    cache = CompressedKVCache(n_slots=2, n_kv=N_KV, capacity=512, bases=_bases(11))
    k0, v0 = _tok(O.kv_like(N_KV, 200, 5)), _tok(O.kv_like(N_KV, 200, 6))
    cache.prefill(1, to_bf16_cuda(k0), to_bf16_cuda(v0))
    slots = torch.tensor([1, -1], dtype=torch.int32, device="cuda")
    q = torch.zeros(2, N_KV * G, 128, dtype=torch.bfloat16, device="cuda")
    kn = torch.zeros(2, N_KV, 128, dtype=torch.bfloat16, device="cuda"); vn = torch.zeros_like(kn)
    def step():
        cache.append(slots, kn, vn); return cache.attention(q, slots, SCALE, max_len=512)
    s = torch.cuda.Stream(); s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):          # warm up outside capture, on a padded batch
        slots.fill_(-1); step()
    torch.cuda.current_stream().wait_stream(s)
    cache.growable = False
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = step()
    slots.copy_(torch.tensor([1, -1], dtype=torch.int32))
    hk, hv = k0, v0
    rng = np.random.default_rng(3)
    for _ in range(20):
        k = O.f32_to_bf16((rng.standard_normal((2, N_KV, 128)) * 0.5).astype(np.float32)); v = O.f32_to_bf16((rng.standard_normal((2, N_KV, 128)) * 0.5).astype(np.float32))
        q16 = O.f32_to_bf16((rng.standard_normal((2, N_KV * G, 128)) * 0.1).astype(np.float32))
        kn.copy_(to_bf16_cuda(k)); vn.copy_(to_bf16_cuda(v)); q.copy_(to_bf16_cuda(q16))
        g.replay(); torch.cuda.synchronize()
        hk, hv = np.concatenate([hk, k[:1]]), np.concatenate([hv, v[:1]])
        ref = O.attention_ref(q16[0], hk, hv, SCALE)
        assert np.abs(out[0].float().cpu().numpy() - ref).max() <= 2e-2 * np.abs(ref).max() + 1e-3
        assert out[1].abs().max().item() == 0
    dk, dv = cache.decompress(1)
    assert np.array_equal(bits(dk), hk) and np.array_equal(bits(dv), hv)


def test_capacity_and_growth_rules():
    import torch
    from gaac_b200 import CompressedKVCache
    cache = CompressedKVCache(n_slots=1, n_kv=2, capacity=64, bases=None, ovf_bytes_per_tile=16)
    rng = np.random.default_rng(4)
    junk = rng.integers(0, 65536, (64, 2, 128)).astype(np.uint16)
    junk = np.where(((junk >> 7) & 0xFF) == 0xFF, junk & ~np.uint16(0x4000), junk)
    cache.prefill(0, to_bf16_cuda(junk), to_bf16_cuda(junk))             # forces the escape stream to grow
    assert cache.k.ovf_cap >= 4 * 1280
    dk, dv = cache.decompress(0)
    assert np.array_equal(bits(dk), junk) and np.array_equal(bits(dv), junk)
    with pytest.raises(AssertionError):
        cache.prefill(0, to_bf16_cuda(np.zeros((65, 2, 128), np.uint16)), to_bf16_cuda(np.zeros((65, 2, 128), np.uint16)))
    cache.growable = False
    with pytest.raises(RuntimeError, match="escape stream"):
        cache.check_capacity(used=cache.k.ovf_cap)


def test_append_never_writes_outside_a_heads_escape_share():
    """A cache whose escape streams are far too small for the data (random bit patterns: 1280 escape bytes per tile against 8 reserved)
    and a caller that never runs check_capacity: the appends that complete a tile must refuse it instead of writing into the next
    head's share.  The refused tiles are counted, the head's counters stay where they were, and a neighbouring slot filled with
    ordinary data still decompresses bit for bit."""
    import torch
    from gaac_b200 import CompressedKVCache
    cache = CompressedKVCache(n_slots=3, n_kv=2, capacity=256, bases=_bases2(), ovf_bytes_per_tile=8)
    good_k, good_v = _tok(O.kv_like(2, 37, 5)), _tok(O.kv_like(2, 37, 6))
    for s in (0, 2):
        cache.prefill(s, to_bf16_cuda(good_k), to_bf16_cuda(good_v))                  # may grow the streams: that is prefill's job
    cap_before = cache.k.ovf_cap
    cache.growable = False
    rng = np.random.default_rng(3)
    slots = torch.tensor([1], dtype=torch.int32, device="cuda")
    for step in range(160):                                                       # ten tiles' worth of junk into slot 1: 12.8 KB of escapes per head
        junk = rng.integers(0, 65536, (1, 2, 128)).astype(np.uint16)
        junk = np.where(((junk >> 7) & 0xFF) >= 0x86, junk & ~np.uint16(0x4000), junk)
        cache.append(slots, to_bf16_cuda(junk), to_bf16_cuda(junk))
    torch.cuda.synchronize()
    stored_tiles = int(cache.S[2]) // 16                                          # head 2 = first head of slot 1
    assert int(cache.append_errors) > 0 and 0 < stored_tiles < 10                 # the stream filled up; the tiles after that were refused
    assert cache.k.ovf_cap == cap_before
    assert int(cache.k.ovf_used.max()) + 8 <= cache.k.ovf_cap and int(cache.v.ovf_used.max()) + 8 <= cache.v.ovf_cap
    for s in (0, 2):
        dk, dv = cache.decompress(s)
        assert np.array_equal(bits(dk), good_k) and np.array_equal(bits(dv), good_v)


def _bases2():
    import torch
    k, v = _tok(O.kv_like(2, 2048, 11)), _tok(O.kv_like(2, 2048, 12))
    k3, k4 = O.bases_from_hist(O.exponent_hist_fast(k, 2), 2); v3, v4 = O.bases_from_hist(O.exponent_hist_fast(v, 2), 2)
    return {n: torch.from_numpy(a) for n, a in (("k3", k3), ("k4", k4), ("v3", v3), ("v4", v4))}


@pytest.mark.parametrize("static_bases", [True, False])
def test_prefill_reads_token_major_rows_in_place(static_bases):
    """prefill takes the prompt as the model produces it: a span of a larger token-major tensor (row stride n_kv*128, no copy),
    a QKV-style buffer whose rows are wider than n_kv*128, a transposed view (copied by the wrapper); lengths 0, 5, 16, 33 and
    one that fills the capacity.  Every slot decompresses to exactly what went in and attends correctly."""
    from gaac_b200 import CompressedKVCache
    import torch
    cap = 256
    cache = CompressedKVCache(n_slots=7, n_kv=N_KV, capacity=cap, bases=_bases(11) if static_bases else None)
    lens = [5, 16, 33, cap]
    total = sum(lens)
    k_all, v_all = _tok(O.kv_like(N_KV, total, 71)), _tok(O.kv_like(N_KV, total, 72))
    kd, vd = to_bf16_cuda(k_all), to_bf16_cuda(v_all)
    hist, at = {}, 0
    for s, L in enumerate(lens):                                             # spans of one flat batch tensor, as a prefill step has them
        cache.prefill(s, kd[at:at + L], vd[at:at + L]); hist[s] = (k_all[at:at + L], v_all[at:at + L]); at += L
    # rows inside a wider buffer: [L, 3 * n_kv, 128], the K heads in the middle third
    L = 40
    wide = torch.zeros(L, 3 * N_KV, 128, dtype=torch.bfloat16, device="cuda")
    k5, v5 = _tok(O.kv_like(N_KV, L, 73)), _tok(O.kv_like(N_KV, L, 74))
    wide[:, N_KV:2 * N_KV] = to_bf16_cuda(k5); wide[:, 2 * N_KV:] = to_bf16_cuda(v5)
    cache.prefill(4, wide[:, N_KV:2 * N_KV], wide[:, 2 * N_KV:]); hist[4] = (k5, v5)
    # a head-major tensor viewed token-major (strides the library does not read directly)
    k6, v6 = O.kv_like(N_KV, 21, 75), O.kv_like(N_KV, 21, 76)
    cache.prefill(5, to_bf16_cuda(k6).transpose(0, 1), to_bf16_cuda(v6).transpose(0, 1)); hist[5] = (_tok(k6), _tok(v6))
    # a one-token prompt: torch reports an arbitrary stride for its only row
    k7, v7 = _tok(O.kv_like(N_KV, 1, 78)), _tok(O.kv_like(N_KV, 1, 79))
    cache.prefill(6, to_bf16_cuda(k7), to_bf16_cuda(v7)); hist[6] = (k7, v7)
    for s, (k, v) in hist.items():
        dk, dv = cache.decompress(s)
        assert np.array_equal(bits(dk), k) and np.array_equal(bits(dv), v), s
    rng = np.random.default_rng(3)
    q16 = O.f32_to_bf16((rng.standard_normal((7, N_KV * G, 128)) * 0.1).astype(np.float32))
    _check(cache, hist, [0, 1, 2, 3, 4, 5, 6], q16)
    # an empty prompt empties the slot
    cache.prefill(2, kd[:0], vd[:0])
    assert int(cache.S[2 * N_KV]) == 0 and int(cache.tail_len[2 * N_KV]) == 0 and int(cache.k.ovf_used[2 * N_KV]) == 0


def test_unchecked_prefills_are_settled_in_one_go():
    """prefill(check=False) for a batch of prompts, among them one whose escape bytes overflow the heads' streams (random bit
    patterns: every group raw): nothing is read back until the first call that needs the cache (here attention), which grows
    the streams once and repairs the overflowed slot from the escape slots kept since its prefill."""
    from gaac_b200 import CompressedKVCache
    import torch
    cache = CompressedKVCache(n_slots=5, n_kv=N_KV, capacity=512, bases=_bases(12), ovf_bytes_per_tile=64)
    cap0 = cache.k.ovf_cap
    rng = np.random.default_rng(8)
    hist = {}
    for s, L in ((0, 100), (1, 512), (3, 17)):
        k, v = _tok(O.kv_like(N_KV, L, 80 + s)), _tok(O.kv_like(N_KV, L, 90 + s))
        cache.prefill(s, to_bf16_cuda(k), to_bf16_cuda(v), check=False); hist[s] = (k, v)
    junk_k = rng.integers(0, 1 << 16, (300, N_KV, 128)).astype(np.uint16); junk_k[(junk_k & 0x7F80) == 0x7F80] = 0      # no Inf / NaN patterns
    junk_v = rng.integers(0, 1 << 16, (300, N_KV, 128)).astype(np.uint16); junk_v[(junk_v & 0x7F80) == 0x7F80] = 0
    cache.prefill(2, to_bf16_cuda(junk_k), to_bf16_cuda(junk_v), check=False)
    k, v = _tok(O.kv_like(N_KV, 40, 85)), _tok(O.kv_like(N_KV, 40, 95))
    cache.prefill(3, to_bf16_cuda(k), to_bf16_cuda(v), check=False); hist[3] = (k, v)       # the same slot again before any check
    assert len(cache._pending) == 4 and cache.k.ovf_cap == cap0
    q16 = O.f32_to_bf16((rng.standard_normal((3, N_KV * G, 128)) * 0.1).astype(np.float32))
    _check(cache, hist, [0, 1, 3], q16)                                     # attention settles the pending prefills first
    assert not cache._pending and cache.k.ovf_cap > cap0
    dk, dv = cache.decompress(2)
    assert np.array_equal(bits(dk), junk_k) and np.array_equal(bits(dv), junk_v)
    # a checked prefill and appends afterwards behave as ever
    slots = torch.tensor([0, 2], dtype=torch.int32, device="cuda")
    k1 = O.f32_to_bf16((rng.standard_normal((2, N_KV, 128)) * 0.5).astype(np.float32)); v1 = O.f32_to_bf16((rng.standard_normal((2, N_KV, 128)) * 0.5).astype(np.float32))
    cache.append(slots, to_bf16_cuda(k1), to_bf16_cuda(v1))
    hist[0] = (np.concatenate([hist[0][0], k1[0:1]]), np.concatenate([hist[0][1], v1[0:1]]))
    dk, dv = cache.decompress(0)
    assert np.array_equal(bits(dk), hist[0][0]) and np.array_equal(bits(dv), hist[0][1])
    assert int(cache.append_errors) == 0


def test_ragged_slots_in_a_grid_larger_than_the_gpu():
    """Seven batch rows over slots of very different lengths (one padding row, two equal ones) with 8 splits: 7 x 4 x 8 = 224
    CTAs, more than the GPU holds at once, so late CTAs start while early ones are merging.  A second call with another row-to-slot
    map reuses the workspace."""
    from gaac_b200 import CompressedKVCache
    import torch
    cache = CompressedKVCache(n_slots=6, n_kv=N_KV, capacity=1024, bases=_bases(13))
    lens = {0: 37, 1: 500, 2: 16, 3: 1000, 4: 500, 5: 5}
    hist = {}
    for s, L in lens.items():
        k, v = _tok(O.kv_like(N_KV, L, 120 + s)), _tok(O.kv_like(N_KV, L, 140 + s))
        cache.prefill(s, to_bf16_cuda(k), to_bf16_cuda(v), check=False); hist[s] = (k, v)
    rng = np.random.default_rng(4)
    for slots_l in ([5, 3, -1, 0, 1, 4, 2], [3, 3, 1, -1, 5, 0, 4]):
        slots = torch.tensor(slots_l, dtype=torch.int32, device="cuda")
        q16 = O.f32_to_bf16((rng.standard_normal((7, N_KV * G, 128)) * 0.1).astype(np.float32))
        o32 = torch.empty(7, N_KV * G, 128, dtype=torch.float32, device="cuda")
        out = cache.attention(to_bf16_cuda(q16), slots, SCALE, nsplit=8, out_f32=o32)
        for b, s in enumerate(slots_l):
            if s < 0:
                assert out[b].abs().max().item() == 0
                continue
            assert_attention_close(o32[b].cpu().numpy(), q16[b], hist[s][0], hist[s][1], SCALE, (b, s))
