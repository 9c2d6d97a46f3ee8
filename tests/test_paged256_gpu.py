"""Paged decode attention for head_dim 256 (two 128-dim half-heads per head, gaac/vllm/paged_kernel256.py) against the float64
oracle.  The store, the block table and the mode table are those of the 128-dim tests with twice as many (half-)heads; the
reference has no test for this kernel."""
import numpy as np
import pytest
from common import to_bf16_cuda, assert_attention_close
from oracle import gaac_oracle as O
from test_paged_gpu import _build_paged

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_kv,G,adv", [(1, 4, 0), (2, 2, 3), (1, 8, 0), (2, 1, 4), (1, 6, 2)])
def test_paged_attention256_matches_oracle(n_kv, G, adv):
    import torch
    from gaac_b200.vllm.paged_kernel256 import paged_attention256
    from gaac_b200.kernel import workspace_error
    seq_lens = [16, 37, 333, 1000, 5]
    st, buf, bt, ks, vs = _build_paged(seq_lens, 2 * n_kv, 256, seed=n_kv * 10 + G, adversarial_every=adv)     # 2 * n_kv half-heads
    assert int(st.err) == 0
    if adv: assert int((st.mt < 0).sum()) > len(seq_lens) * 2 * 2 * n_kv      # some finalized tiles stayed raw
    B, n_q = len(seq_lens), n_kv * G
    rng = np.random.default_rng(1)
    q16 = O.f32_to_bf16((rng.standard_normal((B, n_q, 256)) * 0.3).astype(np.float32))
    sl = torch.tensor(seq_lens, dtype=torch.int32, device="cuda")
    for nsplit in (1, 4, None):
        out = torch.empty(B, n_q * 256, dtype=torch.bfloat16, device="cuda")
        o32 = torch.full((B, n_q, 256), float("nan"), dtype=torch.float32, device="cuda")
        paged_attention256(to_bf16_cuda(q16), out, buf, st.raw, st.mt, bt, sl, st.bases, st.TS, n_q, n_kv, nsplit, out_f32=o32)
        for b in range(B):
            k256 = ks[b].reshape(seq_lens[b], n_kv, 256); v256 = vs[b].reshape(seq_lens[b], n_kv, 256)          # half-heads 2h, 2h+1 = dims 0-127, 128-255 of head h
            ref, _ = assert_attention_close(o32[b].cpu().numpy(), q16[b], k256, v256, 256 ** -0.5, (b, nsplit))
            assert np.abs(out[b].view(n_q, 256).float().cpu().numpy() - ref).max() <= 2e-2 * np.abs(ref).max() + 1e-3
    assert not workspace_error("cuda")


def test_paged_attention256_rejects_bad_shapes():
    import torch
    from gaac_b200.vllm.paged_kernel256 import paged_attention256
    z = torch.zeros(16, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="head_dim"):
        paged_attention256(torch.zeros(1, 4, 128, dtype=torch.bfloat16, device="cuda"), z, z, z, z, z, z, (z, z, z, z), 3008, 4, 1)
    with pytest.raises(RuntimeError, match="group size"):
        paged_attention256(torch.zeros(1, 9, 256, dtype=torch.bfloat16, device="cuda"), z, z, z, z, z, z, (z, z, z, z), 3008, 9, 1)
