"""The numpy oracle against fixtures produced by the reference implementation itself (tests/golden/make_golden.py)."""
import numpy as np
import pytest
from common import golden, sha
from oracle import gaac_oracle as O

PAGE_FIELDS = ("sm", "codes", "flags", "ovf_off", "ovf", "ovf_head_start", "tile_off")


def _check_page(pg, g, prefix, full):
    n = int(pg["ovf_head_start"][-1])
    for f in PAGE_FIELDS:
        a = pg[f][:n] if f == "ovf" else pg[f]
        if full:
            assert np.array_equal(a, g[f"{prefix}_{f}"]), f
        else:
            assert sha(a) == str(g[f"{prefix}_{f}_sha"]), f


@pytest.mark.parametrize("kind", ["k", "v"])
@pytest.mark.parametrize("S", [16, 100, 333])
def test_encode_matches_reference(kind, S):
    g = golden("codec")
    x = g[f"codec_x_{S}"]
    pg = O.encode(x, g["codec_base3"], g["codec_base4"], kind, 2)
    _check_page(pg, g, f"codec_{kind}_{S}", full=(S == 16))
    assert O.page_nbytes(pg) == int(g[f"codec_{kind}_{S}_nbytes"])
    assert np.array_equal(O.decode(pg), x)
    assert np.array_equal(O.row_offsets(pg["flags"], S), pg["ovf_off"])


def test_calibration_matches_reference():
    g = golden("codec")
    # same generator as the fixture script is not needed: bases are checked through the adversarial case below,
    # whose calibration sample is its own input
    x = g["adv_x"]
    b3, b4 = O.calibrate(x, 2)
    assert np.array_equal(b3, g["adv_base3"]) and np.array_equal(b4, g["adv_base4"])
    h_slow = O.exponent_hist(x.reshape(1, 2, -1, 128).transpose(0, 2, 1, 3)[:, :8], 2)
    h_fast = O.exponent_hist_fast(x.reshape(1, 2, -1, 128).transpose(0, 2, 1, 3)[:, :8], 2)
    assert np.array_equal(h_slow, h_fast)


def test_adversarial_matches_reference():
    g = golden("codec")
    x = g["adv_x"]
    pg = O.encode(x, g["adv_base3"], g["adv_base4"], "k", 2)
    _check_page(pg, g, "adv", full=False)
    assert O.page_nbytes(pg) == int(g["adv_nbytes"])
    assert np.array_equal(O.decode(pg), x)
    assert O.page_nbytes(pg) <= x.size * 2 + 2 * 48 * 5 * 2      # never expands beyond raw + metadata (tests/test_codec.py:29)


@pytest.mark.parametrize("mode", ["static", "perseq"])
def test_slot_cache_model_matches_reference(mode):
    g = golden("slot_cache")
    n_kv, n_slots, cap = 2, 2, 96
    H = n_slots * n_kv
    k0, v0 = g[f"{mode}_prefill_k"], g[f"{mode}_prefill_v"]          # [L, n_kv, D]
    kn, vn = g[f"{mode}_new_k"], g[f"{mode}_new_v"]                  # [steps, B, n_kv, D]
    for nm, x0, xn in (("k", k0, kn), ("v", v0, vn)):
        ovf_cap = int(g[f"{mode}_{nm}_ovf_cap"])
        xh = np.ascontiguousarray(x0.transpose(1, 0, 2))
        if mode == "static":
            b3, b4 = g[f"bases_{nm}3"].copy(), g[f"bases_{nm}4"].copy()
        else:
            b3, b4 = np.zeros((H, 128), np.uint8), np.zeros((H, 128), np.uint8)
            c3, c4 = O.calibrate(xh, n_kv)
            b3[2:4], b4[2:4] = c3, c4
        m = O.SlotCacheModel(nm, H, cap, ovf_cap, b3, b4)
        m.prefill(2, xh)
        for step in range(xn.shape[0]):
            for kvh in range(n_kv):
                m.append(2 + kvh, xn[step, 0, kvh])
        assert np.array_equal(m.S, g[f"{mode}_S"]) and np.array_equal(m.tail_len, g[f"{mode}_tail_len"])
        assert np.array_equal(m.ovf_used, g[f"{mode}_{nm}_ovf_used"])
        for f in ("sm", "codes", "flags", "tile_off", "ovf", "ovf_used", "base3", "base4"):
            assert sha(getattr(m, f)) == str(g[f"{mode}_{nm}_{f}_sha"]), (nm, f)
        tl = int(m.tail_len[2])
        assert np.array_equal(m.tail[:, :tl], g[f"{mode}_{nm}_tail"][:, :tl])


def test_paged_store_model_matches_reference():
    g = golden("paged_store")
    go = golden("slot_cache")
    bases = {b: go[f"bases_{b}"] for b in ("k3", "k4", "v3", "v4")}
    m = O.PagedStoreModel(8, 2, 12, bases, 128)
    k, v = g["k"], g["v"]
    for ent in g["steps"]:
        m.store(k, v, ent[ent[:, 0] >= 0])
    assert np.array_equal(m.mt, g["mt"]) and len(m.stack) == int(g["top"][0]) and m.err == int(g["err"][0])
    assert np.array_equal(np.array(m.stack), g["stack"][:len(m.stack)])
    assert sha(m.buf) == str(g["buf_sha"]) and sha(m.raw) == str(g["raw_sha"])
    assert (m.mt[5 * 4 + 0] < 0) and (m.mt[3 * 4:4 * 4] >= 0).all()            # the junk K tile stayed raw
    for blk, row0, nv in ((3, 0, 16), (5, 16, 16), (1, 32, 13)):
        for kvh in range(2):
            assert np.array_equal(m.decode_tile(blk, kvh, "k")[:nv], k[row0:row0 + nv, kvh])
            assert np.array_equal(m.decode_tile(blk, kvh, "v")[:nv], v[row0:row0 + nv, kvh])
    m.store(g["k2"], g["v2"], np.array([[1, 0, 13, 3]]))
    m.release_blocks([5])
    assert np.array_equal(m.mt, g["mt_final"]) and len(m.stack) == int(g["top_final"][0]) and m.err == int(g["err_final"][0])
    assert np.array_equal(np.array(m.stack), g["stack_final"][:len(m.stack)])
    assert sha(m.buf) == str(g["buf_final_sha"])


@pytest.mark.parametrize("tag", ["2_4_50", "1_8_333", "2_1_16"])
def test_attention_oracle_matches_reference_formula(tag):
    g = golden("attention")
    o = O.attention_ref(g[f"q_{tag}"], g[f"k_{tag}"], g[f"v_{tag}"], 128 ** -0.5)
    ref = g[f"o_{tag}"]
    assert np.abs(o - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max())       # fp64 vs the reference's fp32 formula


def test_choose_nsplit_matches_reference():
    for B, nk, S, ns in golden("attention")["choose_nsplit"]:
        assert O.choose_nsplit(int(B), int(nk), int(S)) == int(ns)


def test_combine_equals_unsplit_attention():
    rng = np.random.default_rng(0)
    q = O.f32_to_bf16(rng.standard_normal((4, 128)).astype(np.float32))
    k = O.kv_like(1, 200, 3).transpose(1, 0, 2); v = O.kv_like(1, 200, 4).transpose(1, 0, 2)
    full = O.attention_ref(q, k, v, 0.1)
    pm, pl, pa = [], [], []
    for lo, hi in ((0, 64), (64, 64), (64, 200)):      # includes an empty split (m = -inf)
        kk, vv = O.bf16_to_f64(k[lo:hi, 0]), O.bf16_to_f64(v[lo:hi, 0])
        s = (O.bf16_to_f64(q) @ kk.T) * 0.1
        m = s.max(-1) if hi > lo else np.full(4, -np.inf)
        p = np.exp(s - m[:, None]) if hi > lo else np.zeros((4, 0))
        pm.append(m); pl.append(p.sum(-1)); pa.append(p @ vv)
    o = O.combine_partials(np.stack(pm, -1), np.stack(pl, -1), np.stack(pa, -2))
    assert np.abs(o - full).max() < 1e-9
