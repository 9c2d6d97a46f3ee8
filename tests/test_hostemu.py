"""Lane-level encode / decode functions of the CUDA kernels (gaac_b200/csrc/gaac_tile.h) compiled for the host and checked
against the oracle tile by tile, all three tiers and random bit patterns included."""
import ctypes, os, subprocess, tempfile
import numpy as np
import pytest
from oracle import gaac_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def emu():
    so = os.path.join(tempfile.mkdtemp(prefix="gaac_emu_"), "libtile_emul.so")
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-shared", "-fPIC", "-o", so, os.path.join(ROOT, "tests", "hostemu", "tile_emul.cpp")])
    return ctypes.CDLL(so)


def P(a):
    return a.ctypes.data_as(ctypes.c_void_p)


@pytest.mark.parametrize("trial", range(24))
def test_tile_encode_decode_matches_oracle(emu, trial):
    kind = "kv"[trial % 2]
    rng = np.random.default_rng(trial)
    if trial < 16:
        x = O.synth_kv(kind, 1, 16, trial, raw_frac=0.05, four_frac=0.3)
        b3, b4 = O.calibrate(O.synth_kv(kind, 1, 512, trial), 1)
    else:
        x = rng.integers(0, 65536, (1, 16, 128)).astype(np.uint16)
        b3 = rng.integers(0, 249, (1, 128)).astype(np.uint8); b4 = rng.integers(0, 241, (1, 128)).astype(np.uint8)
    nvalid = 16 if trial % 5 else 11
    pg = O.encode(np.ascontiguousarray(x[:, :nvalid]), b3, b4, kind, 1)
    sm = np.zeros(2048, np.uint8); cd = np.zeros(768, np.uint8); fl = np.zeros(16, np.uint32); esc = np.zeros(1288, np.uint8)
    tot = emu.emu_encode_tile(trial % 2, P(x), nvalid, P(b3), P(b4), P(sm), P(cd), P(fl), P(esc))
    n = int(pg["ovf_head_start"][-1])
    assert tot == n
    assert np.array_equal(sm, pg["sm"][0]) and np.array_equal(cd, pg["codes"][0])
    assert np.array_equal(fl.view(np.int32), pg["flags"][0]) and np.array_equal(esc[:n], pg["ovf"][:n])
    out = np.zeros((16, 128), np.uint16)
    emu.emu_decode_tile(trial % 2, P(sm), P(cd), P(fl), P(esc), P(b3), P(b4), P(out))
    assert np.array_equal(out[:nvalid], x[0, :nvalid])
    for shift in (0, 1, 3):                          # the table-driven decoder reads raw payloads as aligned words: try every alignment
        buf = np.zeros(1288 + 16, np.uint8).view(np.uint8)
        base = (-buf.ctypes.data) % 4 + shift
        buf[base:base + 1288] = esc
        out2 = np.zeros((16, 128), np.uint16)
        emu.emu_decode_tile_lut(trial % 2, P(sm), P(cd), P(fl), ctypes.c_void_p(buf.ctypes.data + base), P(b3), P(b4), P(out2))
        assert np.array_equal(out2[:nvalid], x[0, :nvalid]), shift
