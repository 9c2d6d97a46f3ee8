"""Bit-exact check of the BF16 rebuild that runs INSIDE the fused attention kernels.

The attention kernels decode compressed tiles straight into tensor-core fragments; nothing of the rebuilt K and V is normally
visible except through a softmax-weighted sum, where one wrong exponent among millions of elements would drown.  The library
therefore carries a second instantiation of the same kernels (gaac_debug_*_rebuild) that also writes every fragment word it
rebuilt to memory.  Here those words are compared bit for bit with what was encoded, over everything the kernels distinguish:
the three tiers, tiles whose escape bytes exceed the staged window (read from global memory instead), every byte phase of a
head's escape stream against the 16-byte copy granule, the raw BF16 tail of the slot layout with 1, 7 and 15 rows, and in the
paged layout small and large escape slots, finalized tiles that stayed raw, and the still-filling block.
"""
import numpy as np
import pytest
from common import to_bf16_cuda, bits, assert_attention_close
from oracle import gaac_oracle as O

pytestmark = pytest.mark.gpu
SCALE = 128 ** -0.5
SENTINEL = 0x7FC1            # a NaN pattern no input contains: rows the kernel must not write keep it


def _junk_tiles(rng, n_heads, n_tok):
    """Random bit patterns (every group raw: 1280 escape bytes per tile), Inf/NaN and huge magnitudes removed."""
    junk = rng.integers(0, 65536, (n_heads, n_tok, 128)).astype(np.uint16)
    return np.where(((junk >> 7) & 0xFF) >= 0x86, junk & ~np.uint16(0x4000), junk)


def _rebuild_pages(kp, vp, q16, B, n_kv, G, nsplit):
    """Run the debug instantiation over two Pages -> (k_rebuilt, v_rebuilt) uint16 [B*n_kv, S_pad + 16, 128], fp32 output."""
    import torch
    from gaac_b200 import _lib
    from gaac_b200.kernel import _page_side, workspace
    n_q, S, S_pad = n_kv * G, kp.S, kp.sm.shape[1] // 128
    rows = S_pad + 16
    kr = torch.full((B * n_kv, rows, 128), SENTINEL, dtype=torch.int16, device="cuda"); vr = kr.clone()
    out = torch.empty(B, n_q, 128, dtype=torch.bfloat16, device="cuda"); o32 = torch.empty(B, n_q, 128, dtype=torch.float32, device="cuda")
    ws = workspace(torch.device("cuda"), B, n_q, nsplit)
    q = to_bf16_cuda(q16)
    rc = _lib.lib().gaac_debug_decode_attn_rebuild(_page_side(kp), _page_side(vp), q.data_ptr(), None, B, n_q, n_kv, None, S, S_pad,
                                                   SCALE, nsplit, None, 0, kp.base3.size(0), ws.data_ptr(), ws.numel(), out.data_ptr(), o32.data_ptr(),
                                                   kr.data_ptr(), vr.data_ptr(), rows, _lib.stream_ptr(torch.device("cuda")))
    assert rc == 0, rc
    torch.cuda.synchronize()
    return kr.cpu().numpy().view(np.uint16), vr.cpu().numpy().view(np.uint16), o32


def _assert_rebuilt(got, want16, S, what):
    """got [H, rows, 128] against the encoder's input want16 [H, S, 128]; rows >= S must be untouched."""
    bad = np.argwhere(got[:, :S] != want16)
    assert bad.size == 0, (what, "first mismatch (head, token, channel)", bad[0].tolist(), hex(int(got[tuple(bad[0])])), hex(int(want16[tuple(bad[0])])))
    assert (got[:, S:] == SENTINEL).all(), (what, "rows beyond the sequence were written")


@pytest.mark.parametrize("B,n_kv,G,S,nsplit", [(1, 2, 4, 1000, 3), (2, 2, 8, 333, 1), (1, 8, 4, 4096, 6), (3, 1, 1, 16, 1)])
def test_rebuild_inside_attention_is_bit_exact_all_tiers(B, n_kv, G, S, nsplit):
    import torch
    from gaac_b200 import Codec, TileEncoder
    rng = np.random.default_rng(S + G)
    k16, v16 = O.synth_kv("k", B * n_kv, S, 3, raw_frac=0.01, four_frac=0.2), O.synth_kv("v", B * n_kv, S, 4, raw_frac=0.01, four_frac=0.2)
    if S >= 333:                                           # two stretches of random bit patterns: their tiles overflow the staged window
        k16[:, 64:128] = _junk_tiles(rng, B * n_kv, 64); v16[:, 32:80] = _junk_tiles(rng, B * n_kv, 48)
    k, v = to_bf16_cuda(k16), to_bf16_cuda(v16)
    kp, vp = TileEncoder("k").encode(Codec(n_kv).calibrate(k), k), TileEncoder("v").encode(Codec(n_kv).calibrate(v), v)
    shares = O.tier_shares(kp.flags.cpu().numpy(), S)
    assert min(shares) > 0, shares                          # all three tiers occur
    q16 = O.f32_to_bf16((rng.standard_normal((B, n_kv * G, 128)) * 0.05).astype(np.float32))
    kr, vr, o32 = _rebuild_pages(kp, vp, q16, B, n_kv, G, nsplit)
    _assert_rebuilt(kr, k16, S, "K"); _assert_rebuilt(vr, v16, S, "V")
    for b in range(B):                                     # the debug instantiation computes the same attention
        assert_attention_close(o32[b].cpu().numpy(), q16[b], k16[b * n_kv:(b + 1) * n_kv].transpose(1, 0, 2), v16[b * n_kv:(b + 1) * n_kv].transpose(1, 0, 2), SCALE, b)


def test_rebuild_at_every_phase_of_the_escape_stream():
    """The escape window of a tile is copied from the 16-byte boundary below its first byte.  Shift the heads' escape bytes by
    0..15 bytes (head_start moves, the bytes stay the same) so that every alignment of a head's stream occurs."""
    import torch
    from gaac_b200 import Codec, TileEncoder
    n_kv, G, S = 2, 4, 512
    rng = np.random.default_rng(1)
    k16, v16 = O.synth_kv("k", n_kv, S, 13, raw_frac=0.02, four_frac=0.3), O.synth_kv("v", n_kv, S, 14, raw_frac=0.02, four_frac=0.3)
    k, v = to_bf16_cuda(k16), to_bf16_cuda(v16)
    kp, vp = TileEncoder("k").encode(Codec(n_kv).calibrate(k), k), TileEncoder("v").encode(Codec(n_kv).calibrate(v), v)
    q16 = O.f32_to_bf16((rng.standard_normal((1, n_kv * G, 128)) * 0.05).astype(np.float32))
    ovf_k, ovf_v, hs_k, hs_v = kp.ovf, vp.ovf, kp.ovf_head_start, vp.ovf_head_start
    for pad in range(16):
        for pg, ovf, hs in ((kp, ovf_k, hs_k), (vp, ovf_v, hs_v)):
            pg.ovf = torch.cat([torch.full((pad,), 0xEE, dtype=torch.uint8, device="cuda"), ovf]).contiguous()
            pg.ovf_head_start = (hs + pad).contiguous()
            if hasattr(pg, "_attn_side"): del pg._attn_side
        kr, vr, _ = _rebuild_pages(kp, vp, q16, 1, n_kv, G, 2)
        _assert_rebuilt(kr, k16, S, ("K", pad)); _assert_rebuilt(vr, v16, S, ("V", pad))


@pytest.mark.parametrize("tail", [1, 7, 15])
def test_rebuild_slot_cache_with_tail(tail):
    """Slot layout through the serving cache: compressed tiles of three sequences (one with per-sequence padding row -1) plus
    raw BF16 tails of `tail` rows, read through the slot map and the per-head length tables."""
    import torch
    from gaac_b200 import CompressedKVCache, _lib
    from gaac_b200.kernel import _side, workspace
    n_kv, G, n_slots = 2, 4, 3
    cache = CompressedKVCache(n_slots=n_slots, n_kv=n_kv, capacity=512)
    hist = {}
    for s, L in ((0, 64 + tail), (2, 160 + tail)):
        k16 = np.ascontiguousarray(O.synth_kv("k", n_kv, L, 20 + s, raw_frac=0.01).transpose(1, 0, 2))
        v16 = np.ascontiguousarray(O.synth_kv("v", n_kv, L, 30 + s, raw_frac=0.01).transpose(1, 0, 2))
        cache.prefill(s, to_bf16_cuda(k16), to_bf16_cuda(v16)); hist[s] = (k16, v16)
    slots_l = [2, -1, 0]
    B, n_q, rows = len(slots_l), n_kv * G, 512 + 16
    slots = torch.tensor(slots_l, dtype=torch.int32, device="cuda")
    q16 = O.f32_to_bf16((np.random.default_rng(tail).standard_normal((B, n_q, 128)) * 0.05).astype(np.float32))
    kr = torch.full((B * n_kv, rows, 128), SENTINEL, dtype=torch.int16, device="cuda"); vr = kr.clone()
    out = torch.empty(B, n_q, 128, dtype=torch.bfloat16, device="cuda")
    K, V = cache.k, cache.v
    sk = _side(K.sm, K.codes, K.flags, K.tile_off, K.ovf, K.head_start, K.base3, K.base4, K.tail)
    sv = _side(V.sm, V.codes, V.flags, V.tile_off, V.ovf, V.head_start, V.base3, V.base4, V.tail)
    ws = workspace(torch.device("cuda"), B, n_q, 2)
    q = to_bf16_cuda(q16)
    rc = _lib.lib().gaac_debug_decode_attn_rebuild(sk, sv, q.data_ptr(), slots.data_ptr(), B, n_q, n_kv, cache.S.data_ptr(), 0, cache.cap,
                                                   SCALE, 2, cache.tail_len.data_ptr(), 16, K.base3.shape[0], ws.data_ptr(), ws.numel(), out.data_ptr(), None,
                                                   kr.data_ptr(), vr.data_ptr(), rows, _lib.stream_ptr(torch.device("cuda")))
    assert rc == 0, rc
    torch.cuda.synchronize()
    kr, vr = kr.cpu().numpy().view(np.uint16), vr.cpu().numpy().view(np.uint16)
    for b, s in enumerate(slots_l):
        got_k, got_v = kr[b * n_kv:(b + 1) * n_kv], vr[b * n_kv:(b + 1) * n_kv]
        if s < 0:
            assert (got_k == SENTINEL).all() and (got_v == SENTINEL).all() and float(out[b].abs().max()) == 0.0
            continue
        k16, v16 = hist[s]
        _assert_rebuilt(got_k, k16.transpose(1, 0, 2), k16.shape[0], ("K", s)); _assert_rebuilt(got_v, v16.transpose(1, 0, 2), v16.shape[0], ("V", s))


@pytest.mark.parametrize("ovf_slot,adv,gen", [(128, 3, {}), (16, 0, dict(raw_frac=0.0, four_frac=0.004)), (128, 0, dict(raw_frac=0.02, four_frac=0.3))])
def test_rebuild_paged_layout(ovf_slot, adv, gen):
    """Paged layout: compressed slots with a 128-byte and a 16-byte escape area, finalized tiles that stayed raw (escapes did not
    fit, or adversarial bit patterns) and the filling block of every sequence, all read through block table and mode table."""
    import torch
    from gaac_b200 import _lib
    from gaac_b200.kernel import workspace
    from test_paged_gpu import _build_paged
    n_kv, G = 2, 4
    seq_lens = [16, 37, 333, 1000, 5]
    st, buf, bt, ks, vs = _build_paged(seq_lens, n_kv, 256, seed=21 + ovf_slot, adversarial_every=adv, ovf_slot=ovf_slot, raw_tiles=512, **gen)
    assert int(st.err) == 0                                           # the raw pool was large enough for every tile that stayed raw
    mt = st.mt.cpu().numpy()
    full_tiles = sum(L // 16 for L in seq_lens) * 2 * n_kv
    n_raw_final = int((mt < 0).sum()) - sum(1 for L in seq_lens if L % 16) * 2 * n_kv
    assert 0 < n_raw_final < full_tiles or (ovf_slot == 128 and adv == 0), (n_raw_final, full_tiles)     # both kinds of finalized tile occur
    B, n_q, rows = len(seq_lens), n_kv * G, 1024
    q16 = O.f32_to_bf16((np.random.default_rng(2).standard_normal((B, n_q, 128)) * 0.05).astype(np.float32))
    kr = torch.full((B * n_kv, rows, 128), SENTINEL, dtype=torch.int16, device="cuda"); vr = kr.clone()
    out = torch.empty(B, n_q * 128, dtype=torch.bfloat16, device="cuda")
    sl = torch.tensor(seq_lens, dtype=torch.int32, device="cuda")
    q = to_bf16_cuda(q16)
    for nsplit in (1, 3):
        kr.fill_(SENTINEL); vr.fill_(SENTINEL)
        ws = workspace(torch.device("cuda"), B, n_q, nsplit)
        rc = _lib.lib().gaac_debug_paged_decode_attn_rebuild(st.c_state(buf), bt.data_ptr(), bt.stride(0), sl.data_ptr(), q.data_ptr(), B, n_q,
                                                             SCALE, nsplit, ws.data_ptr(), ws.numel(), out.data_ptr(), None, kr.data_ptr(), vr.data_ptr(), rows,
                                                             _lib.stream_ptr(torch.device("cuda")))
        assert rc == 0, rc
        torch.cuda.synchronize()
        gk, gv = kr.cpu().numpy().view(np.uint16), vr.cpu().numpy().view(np.uint16)
        for b, L in enumerate(seq_lens):
            _assert_rebuilt(gk[b * n_kv:(b + 1) * n_kv], ks[b].transpose(1, 0, 2), L, ("K", b, nsplit))
            _assert_rebuilt(gv[b * n_kv:(b + 1) * n_kv], vs[b].transpose(1, 0, 2), L, ("V", b, nsplit))
