"""Generate the golden fixtures in this directory by running the REFERENCE implementation on CPU.

Usage (needs the reference checkout; the fixtures themselves are committed, so tests never need it):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/GAAC [--only-tables]

What runs: the reference torch codec (gaac/codec.py) on CPU tensors, and the reference Triton kernels
(gaac/encoder.py, gaac/kv_cache.py, gaac/vllm/store.py) under the Triton interpreter, on small seeded inputs.
Inputs are stored in the fixtures, so nothing depends on a random-number stream being reproducible.
Large outputs are stored as SHA-256 digests; small ones in full.
"""
from __future__ import annotations
import hashlib, os, sys
os.environ.setdefault("TRITON_INTERPRET", "1")
import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def sha(a) -> str:
    a = np.ascontiguousarray(a)
    return hashlib.sha256(a.tobytes()).hexdigest()


def u16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def kv_like(H, S, seed, outliers=1e-3, scale_seed=None):
    """tests/common.py:4-12 of the reference on a CPU generator; scale_seed fixes the per-channel scales across calls
    (so bases calibrated on one sample fit another, as they do for a real model)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    scale = torch.exp2(torch.rand(1, 1, 128, generator=g) * 8 - 4)
    if scale_seed is not None:
        scale = torch.exp2(torch.rand(1, 1, 128, generator=torch.Generator().manual_seed(scale_seed)) * 8 - 4)
    x = torch.randn(H, S, 128, generator=g) * scale
    m = torch.rand(H, S, 128, generator=g) < outliers
    return torch.where(m, x * 1e4, x).to(torch.bfloat16)


def page_fields(pg):
    n = int(pg.ovf_head_start[-1])
    return dict(sm=pg.sm.numpy(), codes=pg.codes.numpy(), flags=pg.flags.numpy(), ovf_off=pg.ovf_off.numpy(),
                ovf=pg.ovf[:n].numpy(), ovf_head_start=pg.ovf_head_start.numpy(), tile_off=pg.tile_off.numpy())


def tables_and_calibration(ref_root: str):
    """tables.npz: the reference's index tables (gaac/codec.py:29-67, gaac/encoder.py:84-88), row_offsets on a tag-word sample,
    and a calibration case with its input: exponent histogram, bases, BaseCollector over two steps."""
    sys.path.insert(0, ref_root)
    from gaac import TileEncoder, BaseCollector
    from gaac.codec import perm_k, perm_v, perm, storage_index, exponent_hist, bases_from_hist, row_offsets
    out = {"perm_k": perm_k().numpy(), "perm_v": perm_v().numpy()}
    for kind in "kv":
        si, ci = storage_index(kind, "cpu")
        out[f"storage_sm_{kind}"], out[f"storage_cd_{kind}"] = si.numpy(), ci.numpy()
        te = TileEncoder(kind, device="cpu")
        out[f"enc_perm_{kind}"], out[f"enc_inv_sm_{kind}"], out[f"enc_inv_cd_{kind}"] = te.perm.numpy(), te.inv_sm.numpy(), te.inv_cd.numpy()
        assert torch.equal(perm(kind), perm_k() if kind == "k" else perm_v())
    g = torch.Generator(device="cpu").manual_seed(11)
    tag = torch.tensor([0, 1, 3], dtype=torch.int64)[torch.randint(0, 3, (3, 48, 16), generator=g)]
    flags = (tag << (2 * torch.arange(16))).sum(-1)
    flags = torch.where(flags >= 2 ** 31, flags - 2 ** 32, flags).to(torch.int32)
    out["ro_flags"], out["ro_offsets"] = flags.numpy(), row_offsets(flags, 41).numpy()
    n_kv = 2
    x = kv_like(4, 300, seed=5)                                          # [H, T, D], head h -> kv head h % n_kv
    xt = x.reshape(2, n_kv, -1, 128).permute(0, 2, 1, 3).contiguous()    # token-major [., T, n_kv, D]
    hist = exponent_hist(xt, n_kv)
    b3, b4 = bases_from_hist(hist, n_kv)
    out["cal_x"], out["cal_hist"], out["cal_base3"], out["cal_base4"] = u16(x), hist.numpy(), b3.numpy(), b4.numpy()
    col = BaseCollector()
    k1, v1, k2, v2 = (kv_like(n_kv, 200, seed=s).transpose(0, 1).contiguous() for s in (6, 7, 8, 9))      # [N, n_kv, D]
    col.observe(0, k1, v1); col.observe(0, k2, v2); col.observe(3, k2, v1)
    bases = col.bases()
    for i, t in enumerate((k1, v1, k2, v2)): out[f"col_in_{i}"] = u16(t)
    for layer in (0, 3):
        for name in ("k3", "k4", "v3", "v4"): out[f"col_{layer}_{name}"] = bases[layer][name].numpy()
    np.savez_compressed(os.path.join(HERE, "tables.npz"), **out)
    print("tables.npz written to", HERE)


def main(ref_root: str):
    sys.path.insert(0, ref_root)
    import gaac
    from gaac import Codec, TileEncoder, CompressedKVCache
    from gaac.codec import exponent_hist, bases_from_hist
    from gaac.vllm.store import LayerState, OVF_OFF
    torch.manual_seed(0)

    # ------------------------------------------------------------------ 1. codec: reference torch encoder + Triton encoder
    out = {}
    n_kv, H = 2, 4
    calib = kv_like(H, 2048, seed=1)
    codec = Codec(n_kv, device="cpu").calibrate(calib)
    out["codec_base3"], out["codec_base4"] = codec.base3.numpy(), codec.base4.numpy()
    out["calib_hist_sha"] = np.array(sha(exponent_hist(calib.reshape(H // n_kv, n_kv, -1, 128).permute(0, 2, 1, 3), n_kv).numpy()))
    for S in (16, 100, 333):
        x = kv_like(H, S, seed=2 + S)
        out[f"codec_x_{S}"] = u16(x)
        for kind in "kv":
            ref = codec.encode(x, kind)
            fast = TileEncoder(kind, device="cpu").encode(codec, x)
            fr, ff = page_fields(ref), page_fields(fast)
            for f in fr:
                assert np.array_equal(fr[f], ff[f]), (S, kind, f)
            assert torch.equal(Codec.decode(ref).view(torch.int16), x.view(torch.int16))
            for f, a in fr.items():
                if S == 16:
                    out[f"codec_{kind}_{S}_{f}"] = a
                else:
                    out[f"codec_{kind}_{S}_{f}_sha"] = np.array(sha(a))
            out[f"codec_{kind}_{S}_nbytes"] = np.array(ref.nbytes)
    # adversarial: uniformly random bit patterns without NaN/Inf (tests/test_codec.py:22-29)
    g = torch.Generator().manual_seed(5)
    xa = torch.randint(-32768, 32767, (2, 48, 128), dtype=torch.int16, generator=g)
    xa = torch.where(((xa >> 7) & 0xFF) == 0xFF, xa & ~0x4000, xa).view(torch.bfloat16)
    ca = Codec(2, device="cpu").calibrate(xa)
    pa = ca.encode(xa, "k")
    assert torch.equal(Codec.decode(pa).view(torch.int16), xa.view(torch.int16))
    out["adv_x"] = u16(xa); out["adv_base3"] = ca.base3.numpy(); out["adv_base4"] = ca.base4.numpy()
    for f, a in page_fields(pa).items():
        out[f"adv_{f}_sha"] = np.array(sha(a))
    out["adv_nbytes"] = np.array(pa.nbytes)
    np.savez_compressed(os.path.join(HERE, "codec.npz"), **out)

    # ------------------------------------------------------------------ 2. slot cache (layout A): prefill + appends
    out = {}
    tok = lambda x: x.transpose(0, 1).contiguous()
    n_kv = 2
    kc, vc = tok(kv_like(n_kv, 1024, 11, scale_seed=7)), tok(kv_like(n_kv, 1024, 12, scale_seed=8))
    k3, k4 = bases_from_hist(exponent_hist(kc, n_kv), n_kv); v3, v4 = bases_from_hist(exponent_hist(vc, n_kv), n_kv)
    bases = dict(k3=k3, k4=k4, v3=v3, v4=v4)
    for b in bases:
        out[f"bases_{b}"] = bases[b].numpy()
    for mode in ("static", "perseq"):
        cache = CompressedKVCache(n_slots=2, n_kv=n_kv, capacity=96, bases=bases if mode == "static" else None, device="cpu")
        k, v = tok(kv_like(n_kv, 37, 13, scale_seed=7)), tok(kv_like(n_kv, 37, 14, scale_seed=8))
        cache.prefill(1, k, v)
        slots = torch.tensor([1, -1], dtype=torch.int32)
        g = torch.Generator().manual_seed(15)
        kn_all = (torch.randn(30, 2, n_kv, 128, generator=g) * 0.5).to(torch.bfloat16)
        vn_all = (torch.randn(30, 2, n_kv, 128, generator=g) * 0.5).to(torch.bfloat16)
        for step in range(30):
            cache.append(slots, kn_all[step], vn_all[step])
        dk, dv = cache.decompress(1)
        hk, hv = torch.cat([k, kn_all[:, 0]]), torch.cat([v, vn_all[:, 0]])
        assert torch.equal(dk.view(torch.int16), hk.view(torch.int16)) and torch.equal(dv.view(torch.int16), hv.view(torch.int16))
        out[f"{mode}_prefill_k"], out[f"{mode}_prefill_v"] = u16(k), u16(v)
        out[f"{mode}_new_k"], out[f"{mode}_new_v"] = u16(kn_all), u16(vn_all)
        out[f"{mode}_S"], out[f"{mode}_tail_len"] = cache.S.numpy(), cache.tail_len.numpy()
        for nm, st in (("k", cache.k), ("v", cache.v)):
            out[f"{mode}_{nm}_ovf_cap"] = np.array(st.ovf_cap)
            for f in ("sm", "codes", "flags", "tile_off", "ovf", "ovf_used", "base3", "base4"):
                out[f"{mode}_{nm}_{f}_sha"] = np.array(sha(getattr(st, f).numpy()))
            out[f"{mode}_{nm}_tail"] = u16(st.tail)
            out[f"{mode}_{nm}_ovf_used"] = st.ovf_used.numpy()
        out[f"{mode}_stats"] = np.array([cache.stats()[k_] for k_ in ("tokens", "bytes_used", "bf16_bytes")], dtype=np.int64)
    out["bytes_per_slot"] = np.array([CompressedKVCache.bytes_per_slot(2, 96), CompressedKVCache.bytes_per_slot(8, 1000, 64, False)], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "slot_cache.npz"), **out)

    # ------------------------------------------------------------------ 3. paged store (layout B)
    out = {}
    n_kv, num_blocks, ovf_slot = 2, 8, 128
    TS = OVF_OFF + ovf_slot
    st = LayerState(num_blocks, n_kv, raw_tiles=12, bases=bases, ovf_slot=ovf_slot, device="cpu")
    buf = torch.zeros(num_blocks * 2 * n_kv * TS, dtype=torch.uint8)
    L = 45
    k, v = tok(kv_like(n_kv, L, 21, scale_seed=7)), tok(kv_like(n_kv, L, 22, scale_seed=8))
    # make block 5's K tile of head 0 incompressible into the slot: random bit patterns -> raw fallback
    g = torch.Generator().manual_seed(23)
    junk = torch.randint(-32768, 32767, (16, 128), dtype=torch.int16, generator=g)
    junk = torch.where(((junk >> 7) & 0xFF) == 0xFF, junk & ~0x4000, junk).view(torch.bfloat16)
    k[16:32, 0] = junk
    steps = [
        [[3, 0, 0, 16], [5, 16, 0, 16], [1, 32, 0, 8]],        # prefill 40 tokens into blocks 3, 5, 1 (1 is filling)
        [[1, 40, 8, 1]], [[1, 41, 9, 1]], [[1, 42, 10, 1]], [[1, 43, 11, 1]], [[1, 44, 12, 1]],
    ]
    for si, ent_l in enumerate(steps):
        ent = torch.tensor(ent_l, dtype=torch.int32)
        freeq = torch.empty(ent.shape[0] * 2 * n_kv, dtype=torch.int32)
        st.store(k.view(torch.int16), v.view(torch.int16), buf, ent, freeq)
    out["k"], out["v"] = u16(k), u16(v)
    out["steps"] = np.array([e + [[-1, 0, 0, 0]] * (3 - len(e)) for e in steps], dtype=np.int32)
    out["mt"], out["top"], out["err"] = st.mt.numpy().copy(), st.top.numpy().copy(), st.err.numpy().copy()   # copies: the tensors are mutated below
    out["stack"] = st.stack.numpy().copy()
    out["buf_sha"] = np.array(sha(buf.numpy())); out["raw_sha"] = np.array(sha(u16(st.raw)))
    pairs = torch.tensor([[3, 0, 16], [5, 16, 16], [1, 32, 13]], dtype=torch.int32)
    sk = torch.zeros(L, n_kv, 128, dtype=torch.bfloat16); sv = torch.zeros_like(sk)
    st.decode_blocks(buf, pairs, sk, sv)
    assert torch.equal(sk.view(torch.int16), k.view(torch.int16)) and torch.equal(sv.view(torch.int16), v.view(torch.int16))
    # finish block 1 (3 more tokens), then release block 5
    k2, v2 = tok(kv_like(n_kv, 3, 24, scale_seed=7)), tok(kv_like(n_kv, 3, 25, scale_seed=8))
    ent = torch.tensor([[1, 0, 13, 3]], dtype=torch.int32); freeq = torch.empty(2 * n_kv, dtype=torch.int32)
    st.store(k2.view(torch.int16), v2.view(torch.int16), buf, ent, freeq)
    st.release_blocks(torch.tensor([5], dtype=torch.int32))
    out["k2"], out["v2"] = u16(k2), u16(v2)
    out["mt_final"], out["top_final"], out["err_final"] = st.mt.numpy(), st.top.numpy(), st.err.numpy()
    out["stack_final"] = st.stack.numpy()
    out["buf_final_sha"] = np.array(sha(buf.numpy()))
    np.savez_compressed(os.path.join(HERE, "paged_store.npz"), **out)

    # ------------------------------------------------------------------ 4. attention: the reference test's fp32 formula
    out = {}
    def ref_attention(q, k, v, scale):   # tests/common.py:15-22
        n_q, n_kv = q.shape[0], k.shape[1]
        G = n_q // n_kv
        kk = k.float().repeat_interleave(G, 1).transpose(0, 1); vv = v.float().repeat_interleave(G, 1).transpose(0, 1)
        p = torch.softmax((kk @ q.float().unsqueeze(-1)).squeeze(-1) * scale, -1)
        return (p.unsqueeze(1) @ vv).squeeze(1)
    g = torch.Generator().manual_seed(31)
    for n_kv, G, S in ((2, 4, 50), (1, 8, 333), (2, 1, 16)):
        k, v = tok(kv_like(n_kv, S, 32 + S)), tok(kv_like(n_kv, S, 33 + S))
        q = (torch.randn(n_kv * G, 128, generator=g) * 0.1).to(torch.bfloat16)
        o = ref_attention(q, k, v, 128 ** -0.5)
        tag = f"{n_kv}_{G}_{S}"
        out[f"q_{tag}"], out[f"k_{tag}"], out[f"v_{tag}"], out[f"o_{tag}"] = u16(q), u16(k), u16(v), o.numpy()
    out["choose_nsplit"] = np.array([[B, nk, S, gaac.choose_nsplit(B, nk, S)] for B, nk, S in
                                     ((1, 8, 65536), (1, 8, 131072), (64, 8, 32768), (16, 8, 4096), (1, 2, 100), (3, 2, 5000))], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **out)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    root = args[0] if args else os.environ.get("GAAC_REFERENCE", "")
    if "--only-tables" not in sys.argv:
        main(root)
    tables_and_calibration(root)
