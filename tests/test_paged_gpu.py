"""Paged layout (layout B) on the GPU: store / release / block decode against the fixtures produced by the reference's
Triton kernels, and the fused paged attention against the fp64 oracle (the reference has no tests for this layout)."""
import numpy as np
import pytest
from common import golden, sha, to_bf16_cuda, bits, assert_attention_close
from oracle import gaac_oracle as O

pytestmark = pytest.mark.gpu


def _bases_t():
    import torch
    go = golden("slot_cache")
    return {b: torch.from_numpy(go[f"bases_{b}"]) for b in ("k3", "k4", "v3", "v4")}


def test_store_release_decode_match_reference_fixture():
    import torch
    from gaac_b200.vllm.store import LayerState, OVF_OFF
    g = golden("paged_store")
    n_kv, num_blocks, ovf_slot = 2, 8, 128
    TS = OVF_OFF + ovf_slot
    st = LayerState(num_blocks, n_kv, raw_tiles=12, bases=_bases_t(), ovf_slot=ovf_slot, device="cuda")
    buf = torch.zeros(num_blocks * 2 * n_kv * TS, dtype=torch.uint8, device="cuda")
    k, v = to_bf16_cuda(g["k"]), to_bf16_cuda(g["v"])
    for ent in g["steps"]:
        ent = torch.from_numpy(ent[ent[:, 0] >= 0]).cuda()
        freeq = torch.empty(ent.shape[0] * 2 * n_kv, dtype=torch.int32, device="cuda")
        st.store(k.view(torch.int16), v.view(torch.int16), buf, ent, freeq)
    # the order in which concurrent programs pop raw tiles is free: compare content, counts and the compressed bytes
    mt, mt_ref = st.mt.cpu().numpy(), g["mt"]
    assert np.array_equal(mt < 0, mt_ref < 0) and np.array_equal(mt[mt >= 0], mt_ref[mt_ref >= 0])
    assert int(st.top) == int(g["top"][0]) and int(st.err) == int(g["err"][0])
    raws = -mt[mt < 0] - 1
    assert len(set(raws.tolist())) == raws.size and set(raws.tolist()).isdisjoint(set(st.stack.cpu().numpy()[:int(st.top)].tolist()))
    assert sha(buf.cpu().numpy()) == str(g["buf_sha"])
    pairs = torch.tensor([[3, 0, 16], [5, 16, 16], [1, 32, 13]], dtype=torch.int32, device="cuda")
    sk = torch.zeros(45, n_kv, 128, dtype=torch.bfloat16, device="cuda"); sv = torch.zeros_like(sk)
    st.decode_blocks(buf, pairs, sk, sv)
    assert np.array_equal(bits(sk), g["k"]) and np.array_equal(bits(sv), g["v"])
    ent = torch.tensor([[1, 0, 13, 3]], dtype=torch.int32, device="cuda"); freeq = torch.empty(2 * n_kv, dtype=torch.int32, device="cuda")
    st.store(to_bf16_cuda(g["k2"]), to_bf16_cuda(g["v2"]), buf, ent, freeq)
    st.release_blocks(torch.tensor([5], dtype=torch.int32, device="cuda"))
    assert np.array_equal(st.mt.cpu().numpy(), g["mt_final"])             # all raw tiles are back: the table is deterministic again
    assert int(st.top) == int(g["top_final"][0]) and int(st.err) == 0
    assert sorted(st.stack.cpu().numpy()[:int(st.top)].tolist()) == sorted(g["stack_final"][:int(g["top_final"][0])].tolist())
    assert sha(buf.cpu().numpy()) == str(g["buf_final_sha"])


def test_raw_pool_exhaustion_counts_errors():
    import torch
    from gaac_b200.vllm.store import LayerState, OVF_OFF
    n_kv = 1
    st = LayerState(4, n_kv, raw_tiles=1, bases={k_: torch.zeros(1, 128, dtype=torch.uint8) for k_ in ("k3", "k4", "v3", "v4")}, ovf_slot=16, device="cuda")
    buf = torch.zeros(4 * 2 * (OVF_OFF + 16), dtype=torch.uint8, device="cuda")
    x = to_bf16_cuda(O.kv_like(1, 4, 1).transpose(1, 0, 2))
    ent = torch.tensor([[0, 0, 0, 4]], dtype=torch.int32, device="cuda"); freeq = torch.empty(2, dtype=torch.int32, device="cuda")
    st.store(x, x, buf, ent, freeq)            # K and V of block 0 both want a raw tile, the pool holds one
    assert int(st.err) == 1 and int(st.top) == -1


def _build_paged(seq_lens, n_kv, num_blocks, seed, adversarial_every=0, ovf_slot=128, raw_tiles=None, **gen):
    """Store sequences of the given lengths through the paged store (whole prompt at once) -> (state, buf, bt, k16s, v16s).
    gen: raw_frac / four_frac of the synthetic generator."""
    import torch
    from gaac_b200.vllm.store import LayerState, OVF_OFF
    rng = np.random.default_rng(seed)
    TS = OVF_OFF + ovf_slot
    cal_k, cal_v = O.synth_kv("k", n_kv, 2048, seed, **gen), O.synth_kv("v", n_kv, 2048, seed, **gen)
    k3, k4 = O.calibrate(cal_k, n_kv); v3, v4 = O.calibrate(cal_v, n_kv)
    bases = {n: torch.from_numpy(a) for n, a in (("k3", k3), ("k4", k4), ("v3", v3), ("v4", v4))}
    st = LayerState(num_blocks, n_kv, raw_tiles=raw_tiles or len(seq_lens) * 2 * n_kv + 64, bases=bases, ovf_slot=ovf_slot, device="cuda")
    buf = torch.zeros(num_blocks * 2 * n_kv * TS, dtype=torch.uint8, device="cuda")
    perm = rng.permutation(num_blocks)
    max_blocks = (max(seq_lens) + 15) // 16
    bt = np.zeros((len(seq_lens), max_blocks), np.int32)
    ks, vs, used = [], [], 0
    for i, L in enumerate(seq_lens):
        # same generator, same per-channel scales as the calibration sample (seed selects the scales)
        k16 = O.synth_kv("k", n_kv, 2048 + L, seed, **gen)[:, 2048:]; v16 = O.synth_kv("v", n_kv, 2048 + L, seed, **gen)[:, 2048:]
        k16 = np.ascontiguousarray(np.roll(k16, i * 7, axis=1)); v16 = np.ascontiguousarray(np.roll(v16, i * 11, axis=1))
        nb = (L + 15) // 16
        blocks = perm[used:used + nb]; used += nb
        bt[i, :nb] = blocks
        if adversarial_every:
            for t in range(0, nb - 1, adversarial_every):
                junk = rng.integers(0, 65536, (16, 128)).astype(np.uint16)
                k16[(i + t) % n_kv, t * 16:(t + 1) * 16] = np.where(((junk >> 7) & 0xFF) >= 0x84, junk & ~np.uint16(0x4000), junk)
        kt, vt = np.ascontiguousarray(k16.transpose(1, 0, 2)), np.ascontiguousarray(v16.transpose(1, 0, 2))
        ent = np.array([[blocks[t], t * 16, 0, min(16, L - t * 16)] for t in range(nb)], np.int32)
        freeq = torch.empty(nb * 2 * n_kv, dtype=torch.int32, device="cuda")
        st.store(to_bf16_cuda(kt), to_bf16_cuda(vt), buf, torch.from_numpy(ent).cuda(), freeq)
        ks.append(kt); vs.append(vt)
    return st, buf, torch.from_numpy(bt).cuda(), ks, vs


@pytest.mark.parametrize("n_kv,G,adv", [(2, 4, 0), (2, 4, 3), (1, 8, 5), (4, 1, 0), (2, 6, 2)])
def test_paged_attention_matches_oracle(n_kv, G, adv):
    import torch
    from gaac_b200.vllm.paged_kernel import paged_attention
    seq_lens = [16, 37, 333, 1000, 5]
    st, buf, bt, ks, vs = _build_paged(seq_lens, n_kv, 256, seed=n_kv * 10 + G, adversarial_every=adv)
    assert int(st.err) == 0
    if adv: assert int((st.mt < 0).sum()) > len(seq_lens)              # some finalized tiles stayed raw
    B, n_q = len(seq_lens), n_kv * G
    rng = np.random.default_rng(1)
    q16 = O.f32_to_bf16((rng.standard_normal((B, n_q, 128)) * 0.3).astype(np.float32))
    sl = torch.tensor(seq_lens, dtype=torch.int32, device="cuda")
    for nsplit in (1, 4):
        out = torch.empty(B, n_q * 128, dtype=torch.bfloat16, device="cuda")
        o32 = torch.empty(B, n_q, 128, dtype=torch.float32, device="cuda")
        paged_attention(to_bf16_cuda(q16), out, buf, st.raw, st.mt, bt, sl, st.bases, st.TS, n_q, n_kv, nsplit, out_f32=o32)
        for b in range(B):
            ref, _ = assert_attention_close(o32[b].cpu().numpy(), q16[b], ks[b], vs[b], 128 ** -0.5, (b, nsplit))
            mag = np.abs(ref).max()
            assert np.abs(out[b].view(n_q, 128).float().cpu().numpy() - ref).max() <= 2e-2 * mag + 1e-3


def test_paged_attention_rows_handed_out_longest_first():
    """Grids larger than the GPU (here 7 rows x 4 kv heads x 8 splits = 224 CTAs) number their CTAs by row length, longest row
    first (a small sort launch in front of the attention kernel): ragged lengths with ties, a one-token row and the longest row
    last in batch order must give the same results as ever; a second call with other lengths reuses the workspace."""
    import torch
    from gaac_b200.vllm.paged_kernel import paged_attention
    n_kv, G = 4, 2
    seq_lens = [300, 16, 1, 300, 47, 640, 1500]
    st, buf, bt, ks, vs = _build_paged(seq_lens, n_kv, 512, seed=77, adversarial_every=4)
    assert int(st.err) == 0
    B, n_q = len(seq_lens), n_kv * G
    rng = np.random.default_rng(2)
    for lens in (seq_lens, [250, 16, 1, 300, 30, 100, 777]):              # the second set: prefixes of the stored sequences
        q16 = O.f32_to_bf16((rng.standard_normal((B, n_q, 128)) * 0.3).astype(np.float32))
        sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
        out = torch.empty(B, n_q * 128, dtype=torch.bfloat16, device="cuda")
        o32 = torch.empty(B, n_q, 128, dtype=torch.float32, device="cuda")
        paged_attention(to_bf16_cuda(q16), out, buf, st.raw, st.mt, bt, sl, st.bases, st.TS, n_q, n_kv, 8, out_f32=o32)
        for b in range(B):
            assert_attention_close(o32[b].cpu().numpy(), q16[b], ks[b][:lens[b]], vs[b][:lens[b]], 128 ** -0.5, (b, lens[b]))
        assert torch.equal(out.view(B, n_q, 128), o32.to(torch.bfloat16))


def test_paged_incremental_decode_steps():
    """Append one token per sequence per step through the store (finalising blocks that fill) and attend after each step."""
    import torch
    from gaac_b200.vllm.paged_kernel import paged_attention
    n_kv, G = 2, 4
    seq_lens = [30, 47, 16]
    st, buf, bt, ks, vs = _build_paged(seq_lens, n_kv, 64, seed=5)
    used_blocks = set(bt.cpu().numpy().reshape(-1).tolist())
    spare = [b for b in range(64) if b not in used_blocks]
    bt = torch.cat([bt, torch.zeros(3, 2, dtype=torch.int32, device="cuda")], 1)
    rng = np.random.default_rng(2)
    lens = list(seq_lens)
    all_k = O.synth_kv("k", n_kv, 2048 + 60, 5)[:, 2048:].transpose(1, 0, 2)           # [60, n_kv, D], same channel scales as the bases
    all_v = O.synth_kv("v", n_kv, 2048 + 60, 5)[:, 2048:].transpose(1, 0, 2)
    for step in range(20):
        new_k = np.ascontiguousarray(all_k[3 * step:3 * step + 3]); new_v = np.ascontiguousarray(all_v[3 * step:3 * step + 3])
        ent = []
        for i in range(3):
            off = lens[i] % 16
            if off == 0:
                bt[i, lens[i] // 16] = spare.pop()
            ent.append([int(bt[i, lens[i] // 16]), i, off, 1])
            ks[i] = np.concatenate([ks[i], new_k[i:i + 1]]); vs[i] = np.concatenate([vs[i], new_v[i:i + 1]]); lens[i] += 1
        freeq = torch.empty(3 * 2 * n_kv, dtype=torch.int32, device="cuda")
        st.store(to_bf16_cuda(new_k), to_bf16_cuda(new_v), buf, torch.tensor(ent, dtype=torch.int32, device="cuda"), freeq)
        q16 = O.f32_to_bf16((rng.standard_normal((3, n_kv * G, 128)) * 0.3).astype(np.float32))
        out = torch.empty(3, n_kv * G * 128, dtype=torch.bfloat16, device="cuda")
        o32 = torch.empty(3, n_kv * G, 128, dtype=torch.float32, device="cuda")
        paged_attention(to_bf16_cuda(q16), out, buf, st.raw, st.mt, bt, torch.tensor(lens, dtype=torch.int32, device="cuda"), st.bases, st.TS, n_kv * G, n_kv, 2, out_f32=o32)
        for b in range(3):
            assert_attention_close(o32[b].cpu().numpy(), q16[b], ks[b], vs[b], 128 ** -0.5, (step, b))
    assert int(st.err) == 0
    # raw tiles in use = one per (sequence, kv head, kind) with a filling block
    filling = sum(1 for L in lens if L % 16)
    assert int((st.mt < 0).sum()) == filling * 2 * n_kv


def test_step_metadata_feeds_store_and_attention():
    """The host-side step metadata (build_entries, EntryUploader: gaac/vllm/backend.py:205-224 restated) drives the GPU store over a
    chunked prefill, a whole-prompt prefill and decode steps; afterwards every block decodes to what was written and paged
    attention over the result matches the oracle."""
    import torch
    from gaac_b200.vllm import metadata as M
    from gaac_b200.vllm.store import LayerState, OVF_OFF
    from gaac_b200.vllm.paged_kernel import paged_attention
    n_kv, G, num_blocks, ovf_slot = 2, 4, 64, 128
    TS = OVF_OFF + ovf_slot
    cal_k, cal_v = O.synth_kv("k", n_kv, 512, 3), O.synth_kv("v", n_kv, 512, 3)
    k3, k4 = O.calibrate(cal_k, n_kv); v3, v4 = O.calibrate(cal_v, n_kv)
    st = LayerState(num_blocks, n_kv, raw_tiles=32, bases={n: torch.from_numpy(a) for n, a in (("k3", k3), ("k4", k4), ("v3", v3), ("v4", v4))}, ovf_slot=ovf_slot, device="cuda")
    buf = torch.zeros(num_blocks * 2 * n_kv * TS, dtype=torch.uint8, device="cuda")
    up = M.EntryUploader(max_entries=8, n_kv=n_kv, device="cuda")
    rng = np.random.default_rng(1)
    blocks = rng.permutation(num_blocks)
    table = {0: blocks[0:8], 1: blocks[8:16], 2: blocks[16:24]}
    cached = {0: 0, 1: 0, 2: 0}
    hist = {r: (np.zeros((0, n_kv, 128), np.uint16), np.zeros((0, n_kv, 128), np.uint16)) for r in table}
    stream = {r: (np.roll(O.synth_kv("k", n_kv, 512 + 120, 3)[:, 512:].transpose(1, 0, 2), r, axis=0), np.roll(O.synth_kv("v", n_kv, 512 + 120, 3)[:, 512:].transpose(1, 0, 2), r, axis=0)) for r in table}
    for step in [{0: 20, 1: 37}, {0: 13, 2: 16}] + [{0: 1, 1: 1, 2: 1}] * 30:
        reqs = sorted(step)
        qsl = np.concatenate([[0], np.cumsum([step[r] for r in reqs])])
        key = np.concatenate([stream[r][0][cached[r]:cached[r] + step[r]] for r in reqs]); val = np.concatenate([stream[r][1][cached[r]:cached[r] + step[r]] for r in reqs])
        slot_mapping = np.concatenate([table[r][(cached[r] + np.arange(step[r])) // 16] * 16 + (cached[r] + np.arange(step[r])) % 16 for r in reqs])
        ent, freeq = up.upload(M.build_entries(qsl, [cached[r] for r in reqs]), torch.from_numpy(slot_mapping).cuda())
        st.store(to_bf16_cuda(key), to_bf16_cuda(val), buf, ent, freeq)
        for i, r in enumerate(reqs):
            hist[r] = (np.concatenate([hist[r][0], key[qsl[i]:qsl[i + 1]]]), np.concatenate([hist[r][1], val[qsl[i]:qsl[i + 1]]]))
            cached[r] += step[r]
    assert int(st.err) == 0
    # every block decodes to what was written
    L = [cached[r] for r in sorted(table)]
    rows0 = np.concatenate([[0], np.cumsum([(l + 15) // 16 * 16 for l in L])])
    pairs = [[int(table[r][b]), int(rows0[i] + 16 * b), min(16, L[i] - 16 * b)] for i, r in enumerate(sorted(table)) for b in range((L[i] + 15) // 16)]
    sk = torch.zeros(int(rows0[-1]), n_kv, 128, dtype=torch.bfloat16, device="cuda"); sv = torch.zeros_like(sk)
    st.decode_blocks(buf, torch.tensor(pairs, dtype=torch.int32, device="cuda"), sk, sv)
    for i, r in enumerate(sorted(table)):
        assert np.array_equal(bits(sk)[rows0[i]:rows0[i] + L[i]], hist[r][0]) and np.array_equal(bits(sv)[rows0[i]:rows0[i] + L[i]], hist[r][1])
    # and attention over the stored blocks
    n_q = n_kv * G
    bt = torch.tensor(np.stack([table[r] for r in sorted(table)]).astype(np.int32), device="cuda")
    q16 = O.f32_to_bf16((rng.standard_normal((3, n_q, 128)) * 0.3).astype(np.float32))
    out = torch.empty(3, n_q * 128, dtype=torch.bfloat16, device="cuda"); o32 = torch.empty(3, n_q, 128, dtype=torch.float32, device="cuda")
    paged_attention(to_bf16_cuda(q16), out, buf, st.raw, st.mt, bt, torch.tensor(L, dtype=torch.int32, device="cuda"), st.bases, st.TS, n_q, n_kv, out_f32=o32)
    for i, r in enumerate(sorted(table)):
        assert_attention_close(o32[i].cpu().numpy(), q16[i], hist[r][0], hist[r][1], 128 ** -0.5, r)
