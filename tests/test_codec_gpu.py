"""CUDA encoder / decoder / calibration against the oracle and the reference-generated fixtures (bit-exact).
Cases follow the reference's tests/test_codec.py:6-29."""
import numpy as np
import pytest
from common import golden, sha, to_bf16_cuda, bits, page_to_dict, assert_pages_equal
from oracle import gaac_oracle as O

pytestmark = pytest.mark.gpu


def _codec(b3, b4, n_kv):
    import torch
    from gaac_b200 import Codec
    return Codec(n_kv).set_bases(torch.from_numpy(b3), torch.from_numpy(b4))


@pytest.mark.parametrize("kind", ["k", "v"])
@pytest.mark.parametrize("S", [16, 100, 333])
def test_encoder_matches_reference_fixture(kind, S):
    from gaac_b200 import TileEncoder, Codec
    g = golden("codec")
    x16 = g[f"codec_x_{S}"]
    codec = _codec(g["codec_base3"], g["codec_base4"], 2)
    x = to_bf16_cuda(x16)
    pg = TileEncoder(kind).encode(codec, x)
    d = page_to_dict(pg)
    n = d["n_esc"]
    for f in ("sm", "codes", "flags", "ovf_off", "ovf_head_start", "tile_off"):
        if S == 16:
            assert np.array_equal(d[f], g[f"codec_{kind}_{S}_{f}"]), f
        else:
            assert sha(d[f]) == str(g[f"codec_{kind}_{S}_{f}_sha"]), f
    assert (np.array_equal(d["ovf"][:n], g[f"codec_{kind}_{S}_ovf"]) if S == 16 else sha(d["ovf"][:n]) == str(g[f"codec_{kind}_{S}_ovf_sha"]))
    assert pg.nbytes == int(g[f"codec_{kind}_{S}_nbytes"])
    assert np.array_equal(bits(Codec.decode(pg)), x16)
    pg2 = codec.encode(x, kind)                       # Codec.encode runs the same kernels
    assert_pages_equal(page_to_dict(pg2), d)


@pytest.mark.parametrize("kind", ["k", "v"])
@pytest.mark.parametrize("S", [16, 100, 1024])
def test_encoder_matches_oracle_and_roundtrips(kind, S):
    """n_kv = 4, H = 8, calibration on a different-seed sample so all tiers occur (tests/test_codec.py:6-19)."""
    from gaac_b200 import TileEncoder, Codec
    n_kv = 4
    calib16, x16 = O.kv_like(2 * n_kv, 2048, seed=1), O.kv_like(2 * n_kv, S, seed=2)
    codec = Codec(n_kv).calibrate(to_bf16_cuda(calib16))
    b3, b4 = O.calibrate(calib16, n_kv)
    assert np.array_equal(codec.base3.cpu().numpy(), b3) and np.array_equal(codec.base4.cpu().numpy(), b4)
    pg = TileEncoder(kind).encode(codec, to_bf16_cuda(x16))
    ref = O.encode(x16, b3, b4, kind, n_kv)
    assert_pages_equal(page_to_dict(pg), ref)
    assert abs(pg.ratio - O.page_ratio(ref)) < 1e-12
    assert np.array_equal(bits(Codec.decode(pg)), x16)


def test_adversarial_never_expands_beyond_raw():
    """Uniformly random bit patterns: lossless, at most raw size + metadata (tests/test_codec.py:22-29)."""
    from gaac_b200 import TileEncoder, Codec
    g = golden("codec")
    x16 = g["adv_x"]
    x = to_bf16_cuda(x16)
    codec = Codec(2).calibrate(x)
    assert np.array_equal(codec.base3.cpu().numpy(), g["adv_base3"]) and np.array_equal(codec.base4.cpu().numpy(), g["adv_base4"])
    pg = TileEncoder("k").encode(codec, x)
    d = page_to_dict(pg)
    for f in ("sm", "codes", "flags", "ovf_off", "ovf_head_start", "tile_off"):
        assert sha(d[f]) == str(g[f"adv_{f}_sha"]), f
    assert sha(d["ovf"][:d["n_esc"]]) == str(g["adv_ovf_sha"])
    assert np.array_equal(bits(Codec.decode(pg)), x16)
    assert pg.nbytes <= x.numel() * 2 + 2 * 48 * 5 * 2
    rng = np.random.default_rng(9)
    y16 = rng.integers(0, 65536, (4, 256, 128)).astype(np.uint16)
    y16 = np.where(((y16 >> 7) & 0xFF) == 0xFF, y16 & ~np.uint16(0x4000), y16)
    y = to_bf16_cuda(y16)
    c2 = Codec(4).calibrate(y)
    for kind in "kv":
        p2 = TileEncoder(kind).encode(c2, y)
        assert np.array_equal(bits(Codec.decode(p2)), y16)
        assert p2.nbytes <= y.numel() * 2 + 4 * 256 * 5


def test_calibration_kernels_match_oracle():
    import torch
    from gaac_b200.codec import exponent_hist, bases_from_hist
    x16 = O.synth_kv("k", 6, 5000, seed=3)                            # [H, T, D] -> token-major [T, n_kv, D]
    xt = np.ascontiguousarray(x16.transpose(1, 0, 2))
    h = exponent_hist(to_bf16_cuda(xt), 6)
    href = O.exponent_hist_fast(xt, 6)
    assert np.array_equal(h.cpu().numpy(), href)
    b3, b4 = bases_from_hist(h, 6)
    r3, r4 = O.bases_from_hist(href, 6)
    assert np.array_equal(b3.cpu().numpy(), r3) and np.array_equal(b4.cpu().numpy(), r4)
    flat = torch.zeros(128, 256, dtype=torch.int64, device="cuda")     # ties: the first maximum wins
    flat[1, 200:] = 7; flat[2, 37] = 1; flat[3, 255] = 5
    t3, t4 = bases_from_hist(flat, 1)
    o3, o4 = O.bases_from_hist(flat.cpu().numpy(), 1)
    assert np.array_equal(t3.cpu().numpy(), o3) and np.array_equal(t4.cpu().numpy(), o4)
    assert t3[0, 0] == 0 and t3[0, 1] == 200 and t4[0, 3] == 240


def test_base_collector_matches_oracle(tmp_path):
    import torch
    from gaac_b200 import BaseCollector
    col = BaseCollector()
    hk = hv = 0
    for step in range(3):
        k16 = np.ascontiguousarray(O.synth_kv("k", 2, 300, seed=10 + step).transpose(1, 0, 2))
        v16 = np.ascontiguousarray(O.synth_kv("v", 2, 300, seed=20 + step).transpose(1, 0, 2))
        col.observe(0, to_bf16_cuda(k16), to_bf16_cuda(v16))
        hk = hk + O.exponent_hist_fast(k16, 2); hv = hv + O.exponent_hist_fast(v16, 2)
    b = col.bases()[0]
    k3, k4 = O.bases_from_hist(hk, 2); v3, v4 = O.bases_from_hist(hv, 2)
    for nm, ref in (("k3", k3), ("k4", k4), ("v3", v3), ("v4", v4)):
        assert b[nm].dtype == torch.uint8 and b[nm].device.type == "cpu" and np.array_equal(b[nm].numpy(), ref)
    assert col.save(str(tmp_path / "bases.pt")) == 1
    assert set(torch.load(str(tmp_path / "bases.pt"))[0]) == {"k3", "k4", "v3", "v4"}


def test_calibration_and_collector_match_reference_fixture():
    """Histogram kernel, window search and BaseCollector against outputs of the reference's exponent_hist / bases_from_hist /
    BaseCollector (tests/golden/tables.npz)."""
    import torch
    from gaac_b200 import BaseCollector, Codec
    from gaac_b200.codec import exponent_hist, bases_from_hist
    g = golden("tables")
    x = to_bf16_cuda(g["cal_x"])
    xt = x.reshape(2, 2, -1, 128).permute(0, 2, 1, 3).contiguous()
    hist = exponent_hist(xt, 2)
    assert hist.dtype == torch.int64 and np.array_equal(hist.cpu().numpy(), g["cal_hist"])
    b3, b4 = bases_from_hist(hist, 2)
    assert np.array_equal(b3.cpu().numpy(), g["cal_base3"]) and np.array_equal(b4.cpu().numpy(), g["cal_base4"])
    c = Codec(2).calibrate(x)
    assert np.array_equal(c.base3.cpu().numpy(), g["cal_base3"]) and np.array_equal(c.base4.cpu().numpy(), g["cal_base4"])
    k1, v1, k2, v2 = (to_bf16_cuda(g[f"col_in_{i}"]) for i in range(4))
    col = BaseCollector()
    col.observe(0, k1, v1); col.observe(0, k2, v2); col.observe(3, k2, v1)
    got = col.bases()
    assert sorted(got) == [0, 3]
    for layer in (0, 3):
        for name in ("k3", "k4", "v3", "v4"):
            assert np.array_equal(got[layer][name].numpy(), g[f"col_{layer}_{name}"]), (layer, name)


def test_full_size_roundtrip_property():
    """[8, 65536, 128] per kind: round trip bit-exact on the GPU, ratio and tier shares against the oracle on a 4096-token slice."""
    import torch
    from gaac_b200 import TileEncoder, Codec
    for kind in "kv":
        x16 = O.synth_kv(kind, 8, 65536, seed=0)
        x = to_bf16_cuda(x16)
        codec = Codec(8).calibrate(x[:, :2048])
        pg = TileEncoder(kind).encode(codec, x)
        assert torch.equal(Codec.decode(pg).view(torch.int16), x.view(torch.int16))
        assert 1.37 < pg.ratio < 1.42
        t0, t1, t2 = O.tier_shares(pg.flags.cpu().numpy(), 65536)
        assert 0.78 < t0 < 0.88 and 0.10 < t1 < 0.20 and 0.001 < t2 < 0.015
        b3, b4 = codec.base3.cpu().numpy(), codec.base4.cpu().numpy()
        ref = O.encode(np.ascontiguousarray(x16[:, :4096]), b3, b4, kind, 8)
        d = page_to_dict(pg)
        assert np.array_equal(d["flags"][:, :4096], ref["flags"]) and np.array_equal(d["tile_off"][:, :256], ref["tile_off"])
        assert np.array_equal(d["sm"][:, :4096 * 128], ref["sm"]) and np.array_equal(d["codes"][:, :4096 * 48], ref["codes"])
