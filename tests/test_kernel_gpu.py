"""Fused decode attention against the fp64 oracle (cases of the reference's tests/test_kernel.py:6-19 and more)."""
import numpy as np
import pytest
from common import golden, to_bf16_cuda, bits, assert_attention_close
from oracle import gaac_oracle as O

pytestmark = pytest.mark.gpu
SCALE = 128 ** -0.5


def _pages(k16, v16, n_kv):
    from gaac_b200 import Codec, TileEncoder
    k, v = to_bf16_cuda(k16), to_bf16_cuda(v16)
    ck, cv = Codec(n_kv).calibrate(k), Codec(n_kv).calibrate(v)
    return TileEncoder("k").encode(ck, k), TileEncoder("v").encode(cv, v)


def _check(out, out32, q16, k16, v16, B, n_kv, scale):
    """out bf16 [B, n_q, D], out32 fp32 (same shape); k16/v16 [B*n_kv, S, D]."""
    o16, o32 = bits(out), out32.cpu().numpy()
    for b in range(B):
        kb = k16[b * n_kv:(b + 1) * n_kv].transpose(1, 0, 2); vb = v16[b * n_kv:(b + 1) * n_kv].transpose(1, 0, 2)
        ref, _ = assert_attention_close(o32[b], q16[b], kb, vb, scale, b)          # fp32 result: max(2e-3, 2^-12 sum p|v|) per element
        mag = np.abs(ref).max()
        assert np.array_equal(o16[b], O.f32_to_bf16(o32[b]))                      # the bf16 output is the rounded fp32 result
        err16 = np.abs(O.bf16_to_f64(o16[b]) - ref).max()
        assert err16 <= 2e-2 * mag + 1e-3, (b, err16, mag)                        # the reference's own bound


@pytest.mark.parametrize("B,n_kv,G", [(1, 8, 4), (2, 4, 8), (3, 2, 1), (1, 8, 2), (1, 2, 6), (2, 1, 3)])
@pytest.mark.parametrize("S", [16, 333, 4096])
def test_attention_matches_reference(B, n_kv, G, S):
    import torch
    from gaac_b200 import attention
    k16, v16 = O.kv_like(B * n_kv, S, seed=3), O.kv_like(B * n_kv, S, seed=4)
    kp, vp = _pages(k16, v16, n_kv)
    rng = np.random.default_rng(S + G)
    q16 = O.f32_to_bf16((rng.standard_normal((B, n_kv * G, 128)) * 0.1).astype(np.float32))
    q = to_bf16_cuda(q16)
    for nsplit in (None, 1, 3):
        o32 = torch.empty(B, n_kv * G, 128, dtype=torch.float32, device="cuda")
        out = attention(q, kp, vp, SCALE, nsplit=nsplit, out_f32=o32)
        _check(out, o32, q16, k16, v16, B, n_kv, SCALE)


@pytest.mark.parametrize("tag", ["2_4_50", "1_8_333", "2_1_16"])
def test_attention_matches_reference_fixture(tag):
    """Inputs and fp32 outputs produced by the reference's own test formula (tests/common.py:15-22)."""
    import torch
    from gaac_b200 import attention
    g = golden("attention")
    n_kv, G, S = (int(t) for t in tag.split("_"))
    q16, k16, v16 = g[f"q_{tag}"], g[f"k_{tag}"], g[f"v_{tag}"]             # k/v [S, n_kv, D]
    kh, vh = np.ascontiguousarray(k16.transpose(1, 0, 2)), np.ascontiguousarray(v16.transpose(1, 0, 2))
    kp, vp = _pages(kh, vh, n_kv)
    o32 = torch.empty(1, n_kv * G, 128, dtype=torch.float32, device="cuda")
    out = attention(to_bf16_cuda(q16[None]), kp, vp, SCALE, out_f32=o32)
    ref = g[f"o_{tag}"]                                                    # fp32 output of the reference's own formula
    oref, _ = assert_attention_close(o32[0].cpu().numpy(), q16, k16, v16, SCALE, tag)
    assert np.abs(oref - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max())    # the oracle agrees with the reference's formula
    assert np.abs(out[0].float().cpu().numpy() - ref).max() <= 2e-2 * np.abs(ref).max() + 1e-3


def test_attention_long_escape_tiles_and_default_scale():
    """Tiles whose escapes exceed the staged window (random bit patterns: 1280 B per tile) and scale=None."""
    import torch
    from gaac_b200 import attention, Codec, TileEncoder
    rng = np.random.default_rng(5)
    S, n_kv = 200, 2
    k16, v16 = O.kv_like(n_kv, S, seed=7), O.kv_like(n_kv, S, seed=8)
    junk = rng.integers(0, 65536, (n_kv, 48, 128)).astype(np.uint16)
    junk = np.where(((junk >> 7) & 0xFF) >= 0x86, junk & ~np.uint16(0x4000), junk)      # keep magnitudes moderate, no Inf/NaN
    k16[:, 64:112] = junk; v16[:, 32:80] = junk
    kp, vp = _pages(k16, v16, n_kv)
    q16 = O.f32_to_bf16((rng.standard_normal((1, 8, 128)) * 0.05).astype(np.float32))
    o32 = torch.empty(1, 8, 128, dtype=torch.float32, device="cuda")
    out = attention(to_bf16_cuda(q16), kp, vp, out_f32=o32)
    assert_attention_close(o32[0].cpu().numpy(), q16[0], k16.transpose(1, 0, 2), v16.transpose(1, 0, 2), SCALE)
    assert np.isfinite(out.float().cpu().numpy()).all()


def test_combine_matches_oracle():
    import torch
    from gaac_b200.kernel import combine
    rng = np.random.default_rng(1)
    pm = rng.standard_normal((6, 5)).astype(np.float32) * 3; pm[2, 1] = -np.inf; pm[4, :] = -np.inf
    pl = rng.random((6, 5)).astype(np.float32) + 0.1; pl[4, :] = 0
    pa = rng.standard_normal((6, 5, 128)).astype(np.float32)
    o32 = torch.empty(6, 128, dtype=torch.float32, device="cuda")
    out = combine(torch.from_numpy(pm).cuda(), torch.from_numpy(pl).cuda(), torch.from_numpy(pa).cuda(), out_f32=o32)
    ref = O.combine_partials(pm, pl, pa)
    assert np.abs(o32.cpu().numpy() - ref).max() < 1e-5
    assert (out[4] == 0).all()


def test_partial_mode_equals_full_attention():
    """Context split: two halves attended separately as partials (m, l, acc) and merged with combine == one call."""
    import torch
    from gaac_b200 import attention, Codec, TileEncoder
    from gaac_b200.kernel import _ext, combine
    n_kv, G, S = 2, 4, 2048
    k16, v16 = O.synth_kv("k", n_kv, S, 1), O.synth_kv("v", n_kv, S, 1)
    k, v = to_bf16_cuda(k16), to_bf16_cuda(v16)
    ck, cv = Codec(n_kv).calibrate(k), Codec(n_kv).calibrate(v)
    rng = np.random.default_rng(2)
    q16 = O.f32_to_bf16(rng.standard_normal((1, n_kv * G, 128)).astype(np.float32))
    q = to_bf16_cuda(q16)
    parts = []
    for lo, hi in ((0, 1024), (1024, 2048)):
        kp, vp = TileEncoder("k").encode(ck, k[:, lo:hi].contiguous()), TileEncoder("v").encode(cv, v[:, lo:hi].contiguous())
        part = torch.empty(n_kv * G, 130, dtype=torch.float32, device="cuda")
        slots = torch.arange(1, dtype=torch.int32, device="cuda"); SL = torch.full((n_kv,), hi - lo, dtype=torch.int32, device="cuda")
        e = torch.empty(0, dtype=torch.int32, device="cuda"); eq = torch.empty(0, dtype=torch.bfloat16, device="cuda")
        _ext().gaac_attn_launch(kp.sm, kp.codes, kp.flags, kp.tile_off, kp.ovf, kp.ovf_head_start, kp.base3, kp.base4,
                                vp.sm, vp.codes, vp.flags, vp.tile_off, vp.ovf, vp.ovf_head_start, vp.base3, vp.base4,
                                q.reshape(-1, 128), slots, n_kv * G, n_kv, SL, hi - lo, SCALE, 4, eq, eq, e, 0, partial=part)
        parts.append(part)
    allp = torch.stack(parts, 1)                                   # [n_q, 2, 130]
    o32 = torch.empty(n_kv * G, 128, dtype=torch.float32, device="cuda")
    combine(allp[:, :, 0].contiguous(), allp[:, :, 1].contiguous(), allp[:, :, 2:].contiguous(), out_f32=o32)
    assert_attention_close(o32.cpu().numpy(), q16[0], k16.transpose(1, 0, 2), v16.transpose(1, 0, 2), SCALE)
    # the packed form (what an all-gather of the ranks' partials holds) merges to the same values in one launch
    from gaac_b200.kernel import combine_parts
    o32b = torch.empty_like(o32)
    outb = combine_parts(torch.stack(parts, 0).contiguous(), out_f32=o32b)
    assert torch.equal(o32b, o32) and outb.shape == (n_kv * G, 128)


def _half_pages(n_kv, S, seed):
    import torch
    from gaac_b200 import Codec, TileEncoder
    k16, v16 = O.synth_kv("k", n_kv, S, seed), O.synth_kv("v", n_kv, S, seed)
    k, v = to_bf16_cuda(k16), to_bf16_cuda(v16)
    ck, cv = Codec(n_kv).calibrate(k), Codec(n_kv).calibrate(v)
    halves = []
    for lo, hi in ((0, S // 2), (S // 2, S)):
        halves.append((TileEncoder("k").encode(ck, k[:, lo:hi].contiguous()), TileEncoder("v").encode(cv, v[:, lo:hi].contiguous()), hi - lo))
    return k16, v16, halves


def test_peer_exchange_two_ranks_on_one_gpu():
    """Cross-GPU exchange with both ranks' buffers on one GPU, run in stream order so that no launch ever waits for a later
    one: rank 0 pushes only, rank 1 runs the fused launch (push, wait, merge: rank 0's rows are there already), then rank 0
    merges with the separate kernel.  Four exchanges in a row use both buffer parities; the third one goes through the slot-map
    entry points instead of the Pages entry, and the (row, kv head) group count changes for the last."""
    import torch
    from gaac_b200.kernel import _ext, _pages_call
    from gaac_b200.dist import PeerExchange
    n_kv, G, S = 2, 4, 2048
    n_q = n_kv * G
    k16, v16, halves = _half_pages(n_kv, S, 3)
    k16b, v16b, halves_b = _half_pages(1, 512, 4)                               # a second cache with one kv head: one flag group
    bufs = [PeerExchange.local_buffer(2, n_q, "cuda", groups=n_kv) for _ in range(2)]
    xs = [PeerExchange.local(bufs, r, n_q, groups=n_kv) for r in range(2)]
    slots = torch.zeros(1, dtype=torch.int32, device="cuda")
    e = torch.empty(0, dtype=torch.int32, device="cuda"); eq = torch.empty(0, dtype=torch.bfloat16, device="cuda")
    rng = np.random.default_rng(5)
    for step in range(4):
        hv, kk, vv, nkv = (halves, k16, v16, n_kv) if step < 3 else (halves_b, k16b, v16b, 1)
        nq = nkv * G
        q16 = O.f32_to_bf16(rng.standard_normal((1, nq, 128)).astype(np.float32))
        q = to_bf16_cuda(q16)
        o32 = [torch.empty(nq, 128, dtype=torch.float32, device="cuda") for _ in range(2)]
        outs = [None, None]
        for r, (kp, vp, n) in enumerate(hv):
            if step == 2:
                SL = torch.full((nkv,), n, dtype=torch.int32, device="cuda")
                outs[r] = _ext().gaac_attn_launch(kp.sm, kp.codes, kp.flags, kp.tile_off, kp.ovf, kp.ovf_head_start, kp.base3, kp.base4,
                                                  vp.sm, vp.codes, vp.flags, vp.tile_off, vp.ovf, vp.ovf_head_start, vp.base3, vp.base4,
                                                  q.reshape(-1, 128), slots, nq, nkv, SL, n, SCALE, 4, eq, eq, e, 0, exchange=xs[r].x, fused=(r == 1),
                                                  out_f32=o32[r] if r == 1 else None)
            elif r == 0:
                _pages_call(q, kp, vp, 1, nq, nkv, SCALE, 4, exchange=xs[0].x)
            else:
                outs[1] = torch.empty(nq, 128, dtype=torch.bfloat16, device="cuda")
                _pages_call(q, kp, vp, 1, nq, nkv, SCALE, 4, out=outs[1], out_f32=o32[1], exchange=xs[1].x, fused=True)
        outs[0] = xs[0].merge(nkv, out_f32=o32[0], n_heads=nq)
        for r in range(2):
            assert_attention_close(o32[r].cpu().numpy(), q16[0], kk.transpose(1, 0, 2), vv.transpose(1, 0, 2), SCALE, (step, r))
            assert not xs[r].error()
        assert torch.equal(o32[0], o32[1]) and torch.equal(outs[0].view(-1), outs[1].view(-1))
    assert int(xs[0]._state[0]) == 4 and int(xs[1]._state[0]) == 4               # both ranks counted four exchanges


@pytest.mark.parametrize("world", [4, 8])
def test_peer_exchange_many_ranks_on_one_gpu(world):
    """The same stream-ordered emulation with 4 and 8 ranks, uneven context parts (the last rank gets the remainder, one rank an
    empty part): ranks 0..world-2 push only, the last rank runs the fused launch after them (all rows are there already), the
    others merge with the separate kernel.  Every rank must produce the same output, bit for bit."""
    import torch
    from gaac_b200 import Codec, TileEncoder
    from gaac_b200.kernel import _pages_call
    from gaac_b200.dist import PeerExchange
    n_kv, G, S = 2, 4, 16 * 131
    n_q = n_kv * G
    k16, v16 = O.synth_kv("k", n_kv, S, 21), O.synth_kv("v", n_kv, S, 21)
    k, v = to_bf16_cuda(k16), to_bf16_cuda(v16)
    ck, cv = Codec(n_kv).calibrate(k), Codec(n_kv).calibrate(v)
    cuts = [0] + [16 * int(round(131 * (r + 1) / world * (0.7 if r % 2 else 1.2))) for r in range(world - 1)]
    cuts = sorted(min(c, S) for c in cuts) + [S]
    cuts[2] = cuts[1]                                                            # rank 1 holds no tokens at all
    parts = []
    for r in range(world):
        lo, hi = cuts[r], cuts[r + 1]
        if hi > lo:
            parts.append((TileEncoder("k").encode(ck, k[:, lo:hi].contiguous()), TileEncoder("v").encode(cv, v[:, lo:hi].contiguous())))
        else:
            parts.append(None)
    bufs = [PeerExchange.local_buffer(world, n_q, "cuda", groups=n_kv) for _ in range(world)]
    xs = [PeerExchange.local(bufs, r, n_q, groups=n_kv) for r in range(world)]
    rng = np.random.default_rng(9)
    empty = (TileEncoder("k").encode(ck, k[:, :0].contiguous()), TileEncoder("v").encode(cv, v[:, :0].contiguous()))
    for step in range(3):
        q16 = O.f32_to_bf16(rng.standard_normal((1, n_q, 128)).astype(np.float32))
        q = to_bf16_cuda(q16)
        o32 = [torch.empty(n_q, 128, dtype=torch.float32, device="cuda") for _ in range(world)]
        for r in range(world):
            kp, vp = parts[r] if parts[r] is not None else empty
            if r < world - 1:
                _pages_call(q, kp, vp, 1, n_q, n_kv, SCALE, 3, exchange=xs[r].x)
            else:
                _pages_call(q, kp, vp, 1, n_q, n_kv, SCALE, 3, out=torch.empty(n_q, 128, dtype=torch.bfloat16, device="cuda"), out_f32=o32[r], exchange=xs[r].x, fused=True)
        for r in range(world - 1):
            xs[r].merge(n_kv, out_f32=o32[r], n_heads=n_q)
        assert_attention_close(o32[0].cpu().numpy(), q16[0], k16.transpose(1, 0, 2), v16.transpose(1, 0, 2), SCALE, step)
        for r in range(world):
            assert not xs[r].error()
            assert torch.equal(o32[r], o32[0]), (step, r)


def test_peer_exchange_wait_runs_out():
    """A merge whose peers never push gives up after its bounded wait: error flag set, output zero, GPU still usable; and the
    exchange after it works again (flags carry the exchange number, so a lost exchange does not shift the later ones)."""
    import torch
    from gaac_b200.kernel import _pages_call
    from gaac_b200.dist import PeerExchange
    n_kv, G = 2, 4
    n_q = n_kv * G
    k16, v16, halves = _half_pages(n_kv, 512, 6)
    bufs = [PeerExchange.local_buffer(2, n_q, "cuda", groups=n_kv) for _ in range(2)]
    xs = [PeerExchange.local(bufs, r, n_q, groups=n_kv) for r in range(2)]
    out = xs[0].merge(n_kv)                                                     # nobody pushed: exchange 1 is lost on rank 0
    assert xs[0].error()
    assert (out == 0).all()
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
    xs[1]._state[0] = 1                                                         # rank 1 gave up on exchange 1 as well
    q16 = O.f32_to_bf16(np.random.default_rng(8).standard_normal((1, n_q, 128)).astype(np.float32))
    q = to_bf16_cuda(q16)
    _pages_call(q, halves[0][0], halves[0][1], 1, n_q, n_kv, SCALE, 2, exchange=xs[0].x)
    o32 = torch.empty(n_q, 128, dtype=torch.float32, device="cuda")
    _pages_call(q, halves[1][0], halves[1][1], 1, n_q, n_kv, SCALE, 2, out=torch.empty(n_q, 128, dtype=torch.bfloat16, device="cuda"), out_f32=o32,
                exchange=xs[1].x, fused=True)
    assert_attention_close(o32.cpu().numpy(), q16[0], k16.transpose(1, 0, 2), v16.transpose(1, 0, 2), SCALE)
    assert not xs[1].error()


def test_copy_wait_error_word_stays_clear():
    """The kernel's waits on its own bulk copies are bounded and report through an error word in the workspace: it must be
    zero after ordinary calls (long context, many splits)."""
    import torch
    from gaac_b200 import attention, Codec, TileEncoder
    from gaac_b200.kernel import workspace_error
    n_kv, G, S = 2, 4, 8192
    k16, v16 = O.synth_kv("k", n_kv, S, 9), O.synth_kv("v", n_kv, S, 9)
    k, v = to_bf16_cuda(k16), to_bf16_cuda(v16)
    ck, cv = Codec(n_kv).calibrate(k), Codec(n_kv).calibrate(v)
    kp, vp = TileEncoder("k").encode(ck, k), TileEncoder("v").encode(cv, v)
    q = to_bf16_cuda(O.f32_to_bf16(np.random.default_rng(3).standard_normal((1, n_kv * G, 128)).astype(np.float32)))
    for nsplit in (1, 7, 16):
        attention(q, kp, vp, nsplit=nsplit)
    torch.cuda.synchronize()
    assert not workspace_error(q.device, 1, n_kv * G)


def _fp64_attention_on_gpu(q, k, v, n_kv, G, scale):
    """(reference, sum_i p_i |v_i|) in float64 on the GPU: q [n_kv*G, 128], k / v [n_kv, L, 128] bf16."""
    import torch
    qd = q.double().view(n_kv, G, 128)
    s = torch.einsum("hgd,htd->hgt", qd, k.double()) * scale
    p = torch.softmax(s, -1)
    vd = v.double()
    return torch.einsum("hgt,htd->hgd", p, vd).reshape(n_kv * G, 128), torch.einsum("hgt,htd->hgd", p, vd.abs()).reshape(n_kv * G, 128)


@pytest.mark.parametrize("S", [2048, 65536, 131072])
@pytest.mark.parametrize("outliers", [False, True])
def test_attention_full_size_contexts(S, outliers):
    """32 query / 8 kv heads over 2048, 65536 and 131072 tokens of the benchmark generator, default split count.  The codec is
    lossless, so the float64 reference is computed on the GPU from the original BF16 tensors.  Without the generator's forced
    outliers (no element multiplied by 2^4 or 2^7) the fp32 result is held to a plain 2e-3 max-abs; with them to
    max(2e-3, 2^-12 * sum_i p_i |v_i|) per element.  A single-split run must meet the same bound (split merge)."""
    import torch
    from gaac_b200 import attention, Codec, TileEncoder
    from gaac_b200.synth import synth_kv
    n_kv, G = 8, 4
    fr = dict(raw_frac=0.002, four_frac=0.10) if outliers else dict(raw_frac=0.0, four_frac=0.0)
    k, v = synth_kv("k", n_kv, S, 41, "cuda", **fr), synth_kv("v", n_kv, S, 41, "cuda", **fr)
    ck, cv = Codec(n_kv).calibrate(k[:, :2048]), Codec(n_kv).calibrate(v[:, :2048])
    kp, vp = TileEncoder("k").encode(ck, k), TileEncoder("v").encode(cv, v)
    q = torch.randn(1, n_kv * G, 128, generator=torch.Generator(device="cuda").manual_seed(5), device="cuda").to(torch.bfloat16)
    o32 = torch.empty(1, n_kv * G, 128, dtype=torch.float32, device="cuda")
    out = attention(q, kp, vp, SCALE, out_f32=o32)
    ref, ref_abs = _fp64_attention_on_gpu(q[0], k, v, n_kv, G, SCALE)
    bound = torch.clamp(ref_abs * 2.0 ** -12, min=2e-3)
    err = (o32[0].double() - ref).abs()
    assert bool((err <= bound).all()), float((err / bound).max())
    if not outliers:
        assert float(err.max()) <= 2e-3, float(err.max())
    assert torch.equal(out[0], o32[0].to(torch.bfloat16))
    o1 = torch.empty_like(o32)
    attention(q, kp, vp, SCALE, nsplit=1, out_f32=o1)
    err1 = (o1[0].double() - ref).abs()
    assert bool((err1 <= bound).all()) and (outliers or float(err1.max()) <= 2e-3)


@pytest.mark.parametrize("B,n_kv,G,S,nsplit", [(1, 1, 4, 65536, None), (1, 1, 8, 65536, 296), (1, 2, 4, 40000, 74), (64, 2, 2, 4096, 4), (5, 8, 1, 9000, 33)])
def test_attention_many_splits_and_many_rows(B, n_kv, G, S, nsplit):
    """Split counts far beyond the usual 18 (one kv head over 128 CTAs, the most the cost model picks, 296 = two CTAs per SM's
    worth; more splits than tiles per warp would allow evenly) and many-row batches that run in several waves, against the
    float64 reference computed on the GPU; ranges that leave whole CTAs without a tile must not disturb the merge."""
    import torch
    from gaac_b200 import attention, Codec, TileEncoder
    from gaac_b200.synth import synth_kv
    from gaac_b200.kernel import choose_nsplit_sm100, workspace_error
    k, v = synth_kv("k", B * n_kv, S, 43, "cuda"), synth_kv("v", B * n_kv, S, 43, "cuda")
    ck, cv = Codec(n_kv).calibrate(k[:n_kv, :2048]), Codec(n_kv).calibrate(v[:n_kv, :2048])
    kp, vp = TileEncoder("k").encode(ck, k), TileEncoder("v").encode(cv, v)
    q = torch.randn(B, n_kv * G, 128, generator=torch.Generator(device="cuda").manual_seed(6), device="cuda").to(torch.bfloat16)
    o32 = torch.empty(B, n_kv * G, 128, dtype=torch.float32, device="cuda")
    if nsplit is None:
        assert choose_nsplit_sm100(B, n_kv, S) == 128
    out = attention(q, kp, vp, SCALE, nsplit=nsplit, out_f32=o32)
    for b in range(B):
        ref, ref_abs = _fp64_attention_on_gpu(q[b], k[b * n_kv:(b + 1) * n_kv], v[b * n_kv:(b + 1) * n_kv], n_kv, G, SCALE)
        bound = torch.clamp(ref_abs * 2.0 ** -12, min=2e-3)
        err = (o32[b].double() - ref).abs()
        assert bool((err <= bound).all()), (b, float((err / bound).max()))
    assert torch.equal(out, o32.to(torch.bfloat16))
    assert not workspace_error("cuda")


def test_workspace_is_shared_by_calls_of_different_shapes():
    """One stream, one cached workspace: a small call (1 row, 32 query heads, 8 splits) leaves its partials behind, then a call
    with more (row, kv head) groups than the first one had counters runs on the same buffer.  The header of the workspace has a
    fixed size, so the second call's counters never sit on the first call's partials."""
    import torch
    from gaac_b200 import attention, Codec, TileEncoder
    from gaac_b200.kernel import workspace_error
    rng = np.random.default_rng(12)
    for B, n_kv, G, S, nsplit in ((1, 8, 4, 2048, 8), (16, 8, 1, 256, 2), (1, 8, 4, 2048, 3), (3, 2, 8, 700, 5)):
        k16, v16 = O.synth_kv("k", B * n_kv, S, 50 + B), O.synth_kv("v", B * n_kv, S, 50 + B)
        k, v = to_bf16_cuda(k16), to_bf16_cuda(v16)
        kp, vp = TileEncoder("k").encode(Codec(n_kv).calibrate(k), k), TileEncoder("v").encode(Codec(n_kv).calibrate(v), v)
        q16 = O.f32_to_bf16(rng.standard_normal((B, n_kv * G, 128)).astype(np.float32))
        o32 = torch.full((B, n_kv * G, 128), float("nan"), dtype=torch.float32, device="cuda")
        out = attention(to_bf16_cuda(q16), kp, vp, SCALE, nsplit=nsplit, out_f32=o32)
        _check(out, o32, q16, k16, v16, B, n_kv, SCALE)
    assert not workspace_error("cuda")
