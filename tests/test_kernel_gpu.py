"""Fused decode attention against the fp64 oracle (cases of the reference's tests/test_kernel.py:6-19 and more)."""
import numpy as np
import pytest
from common import golden, to_bf16_cuda, bits, attn_tol
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
        ref = O.attention_ref(q16[b], kb, vb, scale)
        mag = np.abs(ref).max()
        err32 = np.abs(o32[b] - ref).max()
        assert err32 <= attn_tol(ref, vb), (b, err32, mag)                        # fp32 result: 2e-3 max-abs at unit scale
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
    ref = g[f"o_{tag}"]
    assert np.abs(o32[0].cpu().numpy() - ref).max() <= attn_tol(ref, v16)
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
    ref = O.attention_ref(q16[0], k16.transpose(1, 0, 2), v16.transpose(1, 0, 2), SCALE)
    assert np.abs(o32[0].cpu().numpy() - ref).max() <= attn_tol(ref, v16)
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
    ref = O.attention_ref(q16[0], k16.transpose(1, 0, 2), v16.transpose(1, 0, 2), SCALE)
    assert np.abs(o32.cpu().numpy() - ref).max() <= attn_tol(ref, v16)
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
    """Fused exchange (gaac_decode_attn_push + gaac_exchange_merge) with both ranks' buffers on one GPU: every push is launched
    before any merge, so no kernel ever waits for another launch.  Three exchanges in a row use both buffer parities."""
    import torch
    from gaac_b200.kernel import _ext
    from gaac_b200.dist import PeerExchange
    n_kv, G, S = 2, 4, 2048
    n_q = n_kv * G
    k16, v16, halves = _half_pages(n_kv, S, 3)
    bufs = [PeerExchange.local_buffer(2, n_q, "cuda") for _ in range(2)]
    xs = [PeerExchange.local(bufs, r, n_q) for r in range(2)]
    slots = torch.zeros(1, dtype=torch.int32, device="cuda")
    e = torch.empty(0, dtype=torch.int32, device="cuda"); eq = torch.empty(0, dtype=torch.bfloat16, device="cuda")
    rng = np.random.default_rng(5)
    for step in range(3):
        q16 = O.f32_to_bf16(rng.standard_normal((1, n_q, 128)).astype(np.float32))
        q = to_bf16_cuda(q16)
        for r, (kp, vp, n) in enumerate(halves):
            SL = torch.full((n_kv,), n, dtype=torch.int32, device="cuda")
            _ext().gaac_attn_launch(kp.sm, kp.codes, kp.flags, kp.tile_off, kp.ovf, kp.ovf_head_start, kp.base3, kp.base4,
                                    vp.sm, vp.codes, vp.flags, vp.tile_off, vp.ovf, vp.ovf_head_start, vp.base3, vp.base4,
                                    q.reshape(-1, 128), slots, n_q, n_kv, SL, n, SCALE, 4, eq, eq, e, 0, exchange=xs[r].x)
        o32 = [torch.empty(n_q, 128, dtype=torch.float32, device="cuda") for _ in range(2)]
        outs = [xs[r].merge(n_kv, out_f32=o32[r]) for r in range(2)]
        ref = O.attention_ref(q16[0], k16.transpose(1, 0, 2), v16.transpose(1, 0, 2), SCALE)
        for r in range(2):
            assert np.abs(o32[r].cpu().numpy() - ref).max() <= attn_tol(ref, v16)
            assert not xs[r].error()
        assert torch.equal(o32[0], o32[1]) and torch.equal(outs[0], outs[1])


def test_peer_exchange_wait_runs_out():
    """A merge whose peers never push gives up after its bounded wait: error flag set, output zero, GPU still usable."""
    import torch
    from gaac_b200.dist import PeerExchange
    n_q = 8
    bufs = [PeerExchange.local_buffer(2, n_q, "cuda") for _ in range(2)]
    x = PeerExchange.local(bufs, 0, n_q)
    out = x.merge(2)
    assert x.error()
    assert (out == 0).all()
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


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


@pytest.mark.parametrize("S", [65536, 131072])
def test_attention_full_size_contexts(S):
    """BASELINE config 1 (65536 tokens) and config 3 (131072 tokens) shapes: 32 query / 8 kv heads, synthetic KV of the benchmark
    generator, default split count.  The codec is lossless, so the fp64 reference is computed on the GPU from the original BF16
    tensors; the split merge is also checked against a single-split run (same result within the same tolerance)."""
    import torch
    from gaac_b200 import attention, Codec, TileEncoder
    from gaac_b200.synth import synth_kv
    n_kv, G = 8, 4
    k, v = synth_kv("k", n_kv, S, 41, "cuda"), synth_kv("v", n_kv, S, 41, "cuda")
    ck, cv = Codec(n_kv).calibrate(k[:, :2048]), Codec(n_kv).calibrate(v[:, :2048])
    kp, vp = TileEncoder("k").encode(ck, k), TileEncoder("v").encode(cv, v)
    q = torch.randn(1, n_kv * G, 128, generator=torch.Generator(device="cuda").manual_seed(5), device="cuda").to(torch.bfloat16)
    o32 = torch.empty(1, n_kv * G, 128, dtype=torch.float32, device="cuda")
    out = attention(q, kp, vp, SCALE, out_f32=o32)
    qd = q[0].double().view(n_kv, G, 128)
    s = torch.einsum("hgd,htd->hgt", qd, k.double()) * SCALE
    ref = torch.einsum("hgt,htd->hgd", torch.softmax(s, -1), v.double()).reshape(n_kv * G, 128)
    tol = 2e-3 * max(1.0, float(ref.abs().max()), float(v.float().abs().max()))
    assert float((o32[0].double() - ref).abs().max()) <= tol
    assert torch.equal(out[0], o32[0].to(torch.bfloat16))
    o1 = torch.empty_like(o32)
    attention(q, kp, vp, SCALE, nsplit=1, out_f32=o1)
    assert float((o1[0].double() - ref).abs().max()) <= tol
