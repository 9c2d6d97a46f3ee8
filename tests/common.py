"""Shared helpers of the test-suite (fixtures follow the reference's tests/common.py)."""
import hashlib, os
import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def sha(a) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


# ---- torch <-> numpy bf16 bit patterns (imported lazily so CPU-only collection stays light)
def to_bf16_cuda(x16: np.ndarray):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x16).view(np.int16)).cuda().view(torch.bfloat16)


def bits(t) -> np.ndarray:
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def page_to_dict(pg) -> dict:
    """gaac_b200.Page -> the oracle's dict form."""
    n = int(pg.ovf_head_start[-1])
    return dict(sm=pg.sm.cpu().numpy(), codes=pg.codes.cpu().numpy(), flags=pg.flags.cpu().numpy(), ovf_off=pg.ovf_off.cpu().numpy(),
                ovf=pg.ovf.cpu().numpy(), ovf_head_start=pg.ovf_head_start.cpu().numpy(), tile_off=pg.tile_off.cpu().numpy(),
                base3=pg.base3.cpu().numpy(), base4=pg.base4.cpu().numpy(), H=pg.H, S=pg.S, n_kv=pg.n_kv, kind=pg.kind, n_esc=n)


def assert_pages_equal(got: dict, ref: dict):
    n = int(ref["ovf_head_start"][-1])
    for f in ("sm", "codes", "flags", "ovf_off", "ovf_head_start", "tile_off"):
        assert np.array_equal(got[f], ref[f]), f
    assert np.array_equal(got["ovf"][:n], ref["ovf"][:n]), "ovf"
    assert got["ovf"].size == n + 8


def attn_tol(ref: np.ndarray, v16: np.ndarray) -> float:
    """Bound on |fp32 result - fp64 reference|: 2e-3 max-abs at unit scale.  The kernel rounds the softmax weights to BF16
    before the PV product (as the reference kernel does, gaac/kernel.py:178), a relative error of 2^-9 = 1.95e-3 per weight,
    so the bound scales with the largest |v| attended over when that exceeds 1."""
    vmax = float(np.abs((v16.astype(np.uint32) << 16).view(np.float32)).max()) if v16.size else 0.0
    return 2e-3 * max(1.0, float(np.abs(ref).max()), vmax)
