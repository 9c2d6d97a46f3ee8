"""The allocation-free attention entry point (gaac_decode_attn_static) against the regular one, straight through the C ABI.

Some callers cannot give the library a workspace: their HBM is fully reserved by a cache pool, or their host forbids
allocator calls on the hot path.  For them the library carries a fixed device array; this test calls that entry point twice
in a row (the array keeps the previous call's contents, so the second call checks that stale state does no harm) and
compares each result with gaac_decode_attn fed a fresh caller workspace.  The file sorts last so a run that stops at the
first failure has already run everything else."""
import ctypes as C
import numpy as np
import pytest
from common import to_bf16_cuda, assert_attention_close
from oracle import gaac_oracle as O

pytestmark = pytest.mark.gpu


def _side(p, _lib):
    return _lib.Side(p.sm.data_ptr(), p.codes.data_ptr(), p.flags.data_ptr(), p.tile_off.data_ptr(), p.ovf.data_ptr(),
                     p.ovf_head_start.data_ptr(), p.ovf.numel(), p.base3.data_ptr(), p.base4.data_ptr(), None)


def test_static_workspace_entry_matches_regular_entry_twice():
    """Two calls in a row at one shape, then a third with more rows, kv heads and query heads on the same array."""
    import torch
    from gaac_b200 import Codec, TileEncoder, _lib
    L = _lib.lib()
    cap = L.gaac_static_workspace_bytes()
    assert cap == 8 << 20
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(0)
    for call, (B, n_kv, G, S, nsplit) in enumerate(((2, 2, 4, 1000, 5), (2, 2, 4, 1000, 5), (5, 4, 8, 333, 3))):
        n_q = n_kv * G
        assert L.gaac_attn_workspace_bytes(B, n_q, nsplit) <= cap
        k16, v16 = O.synth_kv("k", B * n_kv, S, 11), O.synth_kv("v", B * n_kv, S, 11)
        k, v = to_bf16_cuda(k16), to_bf16_cuda(v16)
        kp = TileEncoder("k").encode(Codec(n_kv).calibrate(k), k); vp = TileEncoder("v").encode(Codec(n_kv).calibrate(v), v)
        K, V = _side(kp, _lib), _side(vp, _lib)
        slots = torch.arange(B, dtype=torch.int32, device="cuda"); SL = torch.full((B * n_kv,), S, dtype=torch.int32, device="cuda")
        q16 = O.f32_to_bf16((rng.standard_normal((B, n_q, 128)) * (0.3 + call)).astype(np.float32))
        q = to_bf16_cuda(q16)
        out_s = torch.empty(B, n_q, 128, dtype=torch.bfloat16, device="cuda"); f32_s = torch.empty(B, n_q, 128, dtype=torch.float32, device="cuda")
        rc = L.gaac_decode_attn_static(K, V, q.data_ptr(), slots.data_ptr(), B, n_q, n_kv, SL.data_ptr(), kp.sm.shape[1] // 128, 128 ** -0.5, nsplit,
                                       None, 0, n_kv, out_s.data_ptr(), f32_s.data_ptr(), stream)
        assert rc == 0, L.gaac_status_string(rc)
        ws = torch.zeros(L.gaac_attn_workspace_bytes(B, n_q, nsplit), dtype=torch.uint8, device="cuda")
        out_r = torch.empty_like(out_s); f32_r = torch.empty_like(f32_s)
        rc = L.gaac_decode_attn(K, V, q.data_ptr(), slots.data_ptr(), B, n_q, n_kv, SL.data_ptr(), kp.sm.shape[1] // 128, 128 ** -0.5, nsplit,
                                None, 0, n_kv, ws.data_ptr(), ws.numel(), out_r.data_ptr(), f32_r.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        for b in range(B):
            kb = k16[b * n_kv:(b + 1) * n_kv].transpose(1, 0, 2); vb = v16[b * n_kv:(b + 1) * n_kv].transpose(1, 0, 2)
            ref, _ = assert_attention_close(f32_s[b].cpu().numpy(), q16[b], kb, vb, 128 ** -0.5, call)
            # the two entry points run the same kernel; tiles reach the warps in a different order from run to run, so the
            # results agree to fp32 accumulation noise, far inside the tolerance of the tests
            assert np.abs(f32_s[b].cpu().numpy() - f32_r[b].cpu().numpy()).max() <= 1e-4 * max(1.0, np.abs(ref).max()), call
            assert np.abs(out_s[b].float().cpu().numpy() - out_r[b].float().cpu().numpy()).max() <= 2e-2 * np.abs(ref).max() + 1e-3, call
    err = C.c_int32(-1)
    assert L.gaac_static_workspace_error(C.byref(err), 0, stream) == 0 and err.value == 0      # no bounded wait ran out


def test_static_workspace_entry_rejects_oversized_requests():
    from gaac_b200 import _lib
    L = _lib.lib()
    fake = C.c_void_p(0x1000)
    side = _lib.Side(0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 64, 0x1000, 0x1000, None)
    B, n_q, nsplit = 64, 64, 64                      # 64*64*64*130*4 B = 136 MB of partials: far beyond the 8 MiB array
    assert L.gaac_attn_workspace_bytes(B, n_q, nsplit) > L.gaac_static_workspace_bytes()
    assert L.gaac_decode_attn_static(side, side, fake, fake, B, n_q, 8, fake, 16, 0.1, nsplit, None, 0, 8, fake, None, None) == 5
