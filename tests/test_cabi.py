"""The C-ABI library: it loads, exports every symbol the header declares, and rejects bad arguments without touching a GPU."""
import ctypes, os, re
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from gaac_b200 import build, _lib
    build.build()
    return _lib.lib()


def test_header_symbols_are_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "gaac_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = sorted(set(re.findall(r"\b(gaac_[a-z0-9_]+)\s*\(", hdr)))
    assert len(names) >= 16
    for n in names:
        assert hasattr(lib, n), n


def test_status_strings(lib):
    assert lib.gaac_status_string(0) == b"ok"
    for s in range(1, 6):
        assert len(lib.gaac_status_string(s)) > 4
    assert lib.gaac_abi_version() == 4


def test_bad_arguments_are_rejected_before_any_launch(lib):
    from gaac_b200 import _lib
    z = ctypes.c_void_p(0)
    assert lib.gaac_encode_tiles(z, 1, 16, 16, 16, z, z, z, 1, 0, z, z, z, z, z, z) == 1
    assert lib.gaac_compact(z, z, 1, 1, z, z, z, 1, z, z, 0, 0, z, z) == 1
    assert lib.gaac_head_prefix(z, 1, z, z) == 1
    assert lib.gaac_decode_page(z, z, z, z, 1, z, z, z, z, z, 1, 0, 1, 16, 16, z, z) == 1
    assert lib.gaac_exponent_hist(z, 1, 128, z, z) == 1
    assert lib.gaac_combine(z, z, z, 1, 1, z, z, z) == 1
    assert lib.gaac_attn_workspace_bytes(0, 32, 4) == 0
    assert lib.gaac_attn_workspace_bytes(1, 32, 4) >= 4 * 32 * 4 * 130
    fake = ctypes.c_void_p(0x1000)      # never dereferenced: the checks below fail first
    side = _lib.Side(0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 64, 0x1000, 0x1000, None)
    # GQA group of 9 is unsupported; n_q not a multiple of n_kv too
    assert lib.gaac_decode_attn(side, side, fake, fake, 1, 9, 1, fake, 16, 0.1, 1, None, 0, 1, fake, 1 << 20, fake, None, None) == 2
    assert lib.gaac_decode_attn(side, side, fake, fake, 1, 6, 4, fake, 16, 0.1, 1, None, 0, 1, fake, 1 << 20, fake, None, None) == 2
    # S_pad must be a multiple of 16; workspace must be large enough; sm must be 16-byte aligned
    assert lib.gaac_decode_attn(side, side, fake, fake, 1, 8, 2, fake, 17, 0.1, 1, None, 0, 1, fake, 1 << 20, fake, None, None) == 1
    assert lib.gaac_decode_attn(side, side, fake, fake, 1, 8, 2, fake, 16, 0.1, 4, None, 0, 1, fake, 64, fake, None, None) == 5
    bad = _lib.Side(0x1008, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 64, 0x1000, 0x1000, None)
    assert lib.gaac_decode_attn(bad, side, fake, fake, 1, 8, 2, fake, 16, 0.1, 1, None, 0, 1, fake, 1 << 20, fake, None, None) == 3
    # workspace layout: a 64 KiB header whatever the shape, so calls of different shapes can share one workspace
    assert lib.gaac_attn_workspace_header_bytes(1, 32) == lib.gaac_attn_workspace_header_bytes(64, 64) == 65536
    assert lib.gaac_attn_workspace_header_bytes(4096, 8) > 65536
    assert lib.gaac_attn_workspace_bytes(2, 8, 3) == 65536 + 2 * 256 + 48 * 128 * 4 + 256           # header, pm, pl, pa, row order
    # the Pages entry wants exactly one destination; the fused exchange wants an output
    x = _lib.Exchange(0x1000, 0x1000, 0x1000, 0x1000, 0, 2, 64)
    assert lib.gaac_decode_attn_pages(side, side, fake, 1, 8, 2, 16, 16, 0.1, 1, 2, fake, 1 << 20, None, None, None, None, 0, None) == 1
    assert lib.gaac_decode_attn_pages(side, side, fake, 1, 8, 2, 16, 16, 0.1, 1, 2, fake, 1 << 20, fake, None, fake, None, 0, None) == 1
    assert lib.gaac_decode_attn_pages(side, side, fake, 1, 8, 2, 16, 16, 0.1, 1, 2, fake, 1 << 20, None, None, None, x, 1, None) == 1
    assert lib.gaac_decode_attn_pages(side, side, fake, 1, 8, 2, 32, 16, 0.1, 1, 2, fake, 1 << 20, fake, None, None, None, 0, None) == 1     # S > S_pad
    small = _lib.Exchange(0x1000, 0x1000, 0x1000, 0x1000, 0, 2, 4)                                                  # rows_cap 4 < B*n_q
    assert lib.gaac_decode_attn_pages(side, side, fake, 1, 8, 2, 16, 16, 0.1, 1, 2, fake, 1 << 20, None, None, None, small, 0, None) == 1
    assert lib.gaac_exchange_merge(x, 65, fake, None, None) == 1                                                     # more heads than rows_cap
    assert lib.gaac_exchange_merge(x, 8, None, None, None) == 1                                                      # no output
    assert lib.gaac_debug_decode_attn_rebuild(side, side, fake, None, 1, 8, 2, None, 16, 16, 0.1, 1, None, 0, 2, fake, 1 << 20, fake, None, None, fake, 32, None) == 1
    pg = _lib.Paged(0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 2, 3000, 120)
    assert lib.gaac_paged_decode_attn(pg, fake, 4, fake, fake, 1, 8, 0.1, 1, fake, 1 << 20, fake, None, None) == 2     # TS % 16
    odd = _lib.Paged(0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 3, 3008, 128)
    assert lib.gaac_paged_decode_attn256(odd, fake, 4, fake, fake, 1, 8, 0.1, 1, fake, 1 << 22, fake, None, None) == 2   # half-heads come in pairs
    two = _lib.Paged(0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 2, 3008, 128)
    assert lib.gaac_paged_decode_attn256(two, fake, 4, fake, fake, 1, 9, 0.1, 1, fake, 1 << 22, fake, None, None) == 2   # group of 9
    assert lib.gaac_paged_decode_attn256(two, fake, 4, fake, fake, 1, 4, 0.1, 2, fake, 1024, fake, None, None) == 5      # workspace for 2 * n_q heads


def test_missing_library_fails_loudly(monkeypatch):
    from gaac_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libgaac_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()


def test_cpu_tensors_are_refused():
    import torch
    from gaac_b200 import Codec, TileEncoder
    x = torch.zeros(2, 16, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        TileEncoder("k").encode_tiles(x, None, None, None, None, None, 16, 16, 2)
    with pytest.raises(RuntimeError, match="no CPU path"):
        from gaac_b200.codec import exponent_hist
        exponent_hist(x, 2)


def test_split_count_heuristics():
    """choose_nsplit keeps the reference's values; choose_nsplit_sm100 fills 148 SMs in one wave for few rows, bounds the
    tiles per warp from below, and switches to the wave model / ragged rule when the rows alone exceed half the SMs."""
    from gaac_b200.kernel import choose_nsplit, choose_nsplit_sm100
    assert choose_nsplit(1, 8, 65536) == 12 and choose_nsplit(16, 8, 65536) == 1 and choose_nsplit(1, 8, 1024) == 2   # gaac/kernel.py:340-342
    assert choose_nsplit_sm100(1, 8, 65536) == 18           # 144 CTAs
    assert choose_nsplit_sm100(1, 8, 8192) == 16            # at least two tiles per warp
    assert choose_nsplit_sm100(1, 1, 100) == 1
    assert choose_nsplit_sm100(64, 1, 32768) == 9           # four full waves of ranges whose metadata fits the staged table
    assert choose_nsplit_sm100(64, 2, 32768) == 8           # 1024 CTAs = 6.9 waves of 256-tile ranges (measured best of 1, 2, 4, 8, 15)
    assert choose_nsplit_sm100(1, 1, 65536) == 128          # two tiles per warp
    assert choose_nsplit_sm100(16, 8, 65536, ragged=True) == 8
    assert choose_nsplit_sm100(256, 8, 4096) == 1
