"""Index tables, row offsets and calibration against values produced by the reference (tests/golden/tables.npz, written by
tests/golden/make_golden.py from gaac/codec.py:29-84,221-225, gaac/encoder.py:84-88 and gaac/calibration.py): the Python tables
this package exports for callers, and the oracle's own."""
import numpy as np
import torch
from common import golden, sha
from oracle import gaac_oracle as O


def test_exported_permutations_and_storage_order_match_reference():
    from gaac_b200 import codec, TileEncoder
    g = golden("tables")
    assert np.array_equal(codec.perm_k().numpy(), g["perm_k"]) and np.array_equal(codec.perm_v().numpy(), g["perm_v"])
    assert np.array_equal(O.perm_k(), g["perm_k"]) and np.array_equal(O.perm_v(), g["perm_v"])
    for kind in "kv":
        assert np.array_equal(codec.perm(kind).numpy(), g[f"perm_{kind}"])
        si, ci = codec.storage_index(kind, "cpu")
        assert np.array_equal(si.numpy(), g[f"storage_sm_{kind}"]) and np.array_equal(ci.numpy(), g[f"storage_cd_{kind}"])
        osi, oci = O.storage_index(kind)
        assert np.array_equal(osi, g[f"storage_sm_{kind}"]) and np.array_equal(oci, g[f"storage_cd_{kind}"])
        te = TileEncoder(kind, device="cpu")                           # the tables need no device
        assert te.perm.dtype == torch.int32 and np.array_equal(te.perm.numpy(), g[f"enc_perm_{kind}"])
        assert te.inv_sm.dtype == torch.int32 and np.array_equal(te.inv_sm.numpy(), g[f"enc_inv_sm_{kind}"])
        assert te.inv_cd.dtype == torch.int32 and np.array_equal(te.inv_cd.numpy(), g[f"enc_inv_cd_{kind}"])


def test_row_offsets_match_reference():
    from gaac_b200.codec import row_offsets
    g = golden("tables")
    got = row_offsets(torch.from_numpy(g["ro_flags"]), 41)
    assert got.dtype == torch.int32 and np.array_equal(got.numpy(), g["ro_offsets"])
    assert np.array_equal(O.row_offsets(g["ro_flags"], 41), g["ro_offsets"])


def test_oracle_histogram_and_bases_match_reference():
    g = golden("tables")
    x = g["cal_x"]                                                     # [H = 4, T, D], head h counts for kv head h % 2
    xt = np.ascontiguousarray(x.reshape(2, 2, -1, 128).transpose(0, 2, 1, 3))
    for hist in (O.exponent_hist(xt, 2), O.exponent_hist_fast(xt, 2)):
        assert hist.dtype == np.int64 and np.array_equal(hist, g["cal_hist"])
    b3, b4 = O.bases_from_hist(g["cal_hist"], 2)
    assert np.array_equal(b3, g["cal_base3"]) and np.array_equal(b4, g["cal_base4"])
    c3, c4 = O.calibrate(x, 2)
    assert np.array_equal(c3, g["cal_base3"]) and np.array_equal(c4, g["cal_base4"])


def test_oracle_histogram_matches_reference_digest_of_the_codec_fixture():
    """codec.npz keeps the SHA-256 of the reference's exponent histogram of its calibration sample.  The sample itself comes from
    torch's CPU generator (as in the fixture script); the bases derived from it are in the fixture too, which tells whether the
    generator still produces the same stream: if it does, the oracle's histogram must hash to the stored digest."""
    g = golden("codec")
    gen = torch.Generator(device="cpu").manual_seed(1)
    scale = torch.exp2(torch.rand(1, 1, 128, generator=gen) * 8 - 4)
    x = torch.randn(4, 2048, 128, generator=gen) * scale
    m = torch.rand(4, 2048, 128, generator=gen) < 1e-3
    calib = torch.where(m, x * 1e4, x).to(torch.bfloat16)
    x16 = calib.view(torch.int16).numpy().view(np.uint16)
    b3, b4 = O.calibrate(x16, 2)
    if not (np.array_equal(b3, g["codec_base3"]) and np.array_equal(b4, g["codec_base4"])):
        import pytest
        pytest.skip("torch's CPU random stream differs from the one the fixture was made with")
    xt = np.ascontiguousarray(x16.reshape(2, 2, -1, 128).transpose(0, 2, 1, 3))
    assert sha(O.exponent_hist_fast(xt, 2)) == str(g["calib_hist_sha"])
