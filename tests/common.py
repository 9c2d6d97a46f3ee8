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


def assert_attention_close(o32: np.ndarray, q16: np.ndarray, k16: np.ndarray, v16: np.ndarray, scale: float, what=""):
    """fp32 attention result against the float64 oracle, element by element: |o32 - ref| <= max(2e-3, 2^-12 * sum_i p_i |v_i|)
    (oracle.attention_bound).  q16 [n_q, D], k16 / v16 [L, n_kv, D] BF16 bit patterns.  Returns (ref, worst error / bound)."""
    from oracle import gaac_oracle as O
    ref, ref_abs = O.attention_ref(q16, k16, v16, scale, with_abs=True)
    err = np.abs(np.asarray(o32, dtype=np.float64) - ref)
    bound = O.attention_bound(ref_abs)
    worst = float((err / bound).max()) if err.size else 0.0
    assert worst <= 1.0, (what, "max |err| / bound", worst, "max |err|", float(err.max()))
    return ref, worst
