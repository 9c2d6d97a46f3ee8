"""Drop-in proof against the reference's own host code (needs the unmodified reference package under baseline/_ref, which
travels with the repository to the GPU box but is not part of it; the tests are skipped where it is absent).

1. The reference package with ONLY its native module swapped: `gaac.kernel._ext` is replaced by `gaac_b200.kernel._ext`, then
   the reference's own `gaac.attention` (gaac/kernel.py:345-359) and `gaac.kv_cache.CompressedKVCache` (gaac/kv_cache.py:149-192,
   its Triton prefill / append kernels included) run over the B200 launcher.
2. The reference's engine-side caller with the whole package swapped: `nanovllm.layers.attention.Attention.forward`
   (nanovllm/layers/attention.py:59-96) is imported unmodified with `gaac` aliased to `gaac_b200`, prefills two sequences in one
   step, then decodes through ONE captured CUDA graph with a padded batch row (slot -1) and the 16-step capacity check of
   nanovllm/engine/model_runner.py:268-273.
"""
import os, sys
import numpy as np
import pytest
from common import to_bf16_cuda, bits, assert_attention_close
from oracle import gaac_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "gaac")), reason="reference package not installed under baseline/_ref")]
SCALE = 128 ** -0.5


def _forget(prefixes):
    for name in [m for m in sys.modules if any(m == p or m.startswith(p + ".") for p in prefixes)]:
        del sys.modules[name]


@pytest.fixture
def reference_importable():
    """The reference's packages importable for the duration of one test, and forgotten afterwards."""
    _forget(["gaac", "nanovllm"])
    sys.path.insert(0, REF)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    try:
        yield
    finally:
        sys.path.remove(REF)
        _forget(["gaac", "nanovllm"])


def _tok(x16):                 # [n_kv, L, D] -> token-major [L, n_kv, D]
    return np.ascontiguousarray(x16.transpose(1, 0, 2))


def test_reference_host_code_over_the_b200_launcher(reference_importable, monkeypatch):
    import torch
    import gaac as ref
    import gaac.kernel, gaac.kv_cache
    import gaac_b200.kernel as ours
    assert "baseline/_ref" in ref.__file__.replace(os.sep, "/")
    # the one-function swap a maintainer of the reference would make (both names refer to the same function there)
    monkeypatch.setattr(ref.kernel, "_ext", ours._ext)
    monkeypatch.setattr(ref.kv_cache, "_ext", ours._ext)
    n_kv, G = 2, 4
    rng = np.random.default_rng(0)
    # ---- reference attention() over Pages made by the reference's own encoder
    for B, S in ((1, 1000), (2, 333)):
        k16, v16 = O.synth_kv("k", B * n_kv, S, 61), O.synth_kv("v", B * n_kv, S, 62)
        k, v = to_bf16_cuda(k16), to_bf16_cuda(v16)
        kp = ref.TileEncoder("k", device="cuda").encode(ref.Codec(n_kv, device="cuda").calibrate(k), k)
        vp = ref.TileEncoder("v", device="cuda").encode(ref.Codec(n_kv, device="cuda").calibrate(v), v)
        q16 = O.f32_to_bf16((rng.standard_normal((B, n_kv * G, 128)) * 0.3).astype(np.float32))
        out = ref.attention(to_bf16_cuda(q16), kp, vp)                      # the reference's entry point, default scale and split count
        assert out.shape == (B, n_kv * G, 128) and out.dtype == torch.bfloat16
        for b in range(B):
            want = O.attention_ref(q16[b], _tok(k16[b * n_kv:(b + 1) * n_kv]), _tok(v16[b * n_kv:(b + 1) * n_kv]), SCALE)
            assert np.abs(out[b].float().cpu().numpy() - want).max() <= 2e-2 * np.abs(want).max() + 1e-3        # the reference's own bound
    # ---- the reference's slot cache: its Triton prefill and append, our attention
    cache = ref.CompressedKVCache(n_slots=3, n_kv=n_kv, capacity=512, device="cuda")
    hist = {}
    for s, L in ((0, 45), (2, 200)):
        k16, v16 = _tok(O.synth_kv("k", n_kv, L, 70 + s)), _tok(O.synth_kv("v", n_kv, L, 80 + s))
        cache.prefill(s, to_bf16_cuda(k16), to_bf16_cuda(v16)); hist[s] = (k16, v16)
    slots_l = [2, -1, 0]
    slots = torch.tensor(slots_l, dtype=torch.int32, device="cuda")
    for step in range(20):
        k1 = O.f32_to_bf16((rng.standard_normal((3, n_kv, 128)) * 0.5).astype(np.float32)); v1 = O.f32_to_bf16((rng.standard_normal((3, n_kv, 128)) * 0.5).astype(np.float32))
        cache.append(slots, to_bf16_cuda(k1), to_bf16_cuda(v1))
        for b, s in enumerate(slots_l):
            if s >= 0: hist[s] = (np.concatenate([hist[s][0], k1[b:b + 1]]), np.concatenate([hist[s][1], v1[b:b + 1]]))
        if step % 16 == 15: cache.check_capacity()
        q16 = O.f32_to_bf16((rng.standard_normal((3, n_kv * G, 128)) * 0.3).astype(np.float32))
        out = cache.attention(to_bf16_cuda(q16), slots, SCALE)
        for b, s in enumerate(slots_l):
            if s < 0:
                assert float(out[b].abs().max()) == 0.0
                continue
            want = O.attention_ref(q16[b], hist[s][0], hist[s][1], SCALE)
            assert np.abs(out[b].float().cpu().numpy() - want).max() <= 2e-2 * np.abs(want).max() + 1e-3, (step, b)


def test_nanovllm_attention_layer_with_the_package_swapped(reference_importable):
    import torch
    import gaac_b200
    import gaac_b200.codec, gaac_b200.encoder, gaac_b200.kernel, gaac_b200.kv_cache, gaac_b200.calibration
    sys.modules["gaac"] = gaac_b200
    for m in ("codec", "encoder", "kernel", "kv_cache", "calibration"):
        sys.modules["gaac." + m] = sys.modules["gaac_b200." + m]
    from gaac import CompressedKVCache                                      # what nanovllm/engine/model_runner.py:131 imports
    assert CompressedKVCache is gaac_b200.CompressedKVCache
    pytest.importorskip("flash_attn")
    from nanovllm.layers.attention import Attention                        # the reference's layer, unmodified
    from nanovllm.utils.context import set_context, reset_context
    n_kv, G = 2, 4
    n_q = n_kv * G
    attn = Attention(n_q, 128, SCALE, n_kv)
    attn.gaac = CompressedKVCache(n_slots=4, n_kv=n_kv, capacity=512, device="cuda")
    rng = np.random.default_rng(1)
    # ---- prefill: two prompts in one step (nanovllm/layers/attention.py:83-93)
    lens, slots_of = [37, 100], [0, 2]
    k16 = np.concatenate([_tok(O.synth_kv("k", n_kv, L, 90 + i)) for i, L in enumerate(lens)]); v16 = np.concatenate([_tok(O.synth_kv("v", n_kv, L, 95 + i)) for i, L in enumerate(lens)])
    q16 = O.f32_to_bf16((rng.standard_normal((sum(lens), n_q, 128)) * 0.3).astype(np.float32))
    cu = torch.tensor([0, lens[0], sum(lens)], dtype=torch.int32, device="cuda")
    set_context(True, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens), prefill_spans=[(0, 0, lens[0]), (2, lens[0], sum(lens))])
    o = attn(to_bf16_cuda(q16), to_bf16_cuda(k16), to_bf16_cuda(v16))
    reset_context()
    assert o.shape == (sum(lens), n_q, 128)
    hist = {0: (k16[:lens[0]], v16[:lens[0]]), 2: (k16[lens[0]:], v16[lens[0]:])}
    for s in slots_of:
        dk, dv = attn.gaac.decompress(s)
        assert np.array_equal(bits(dk), hist[s][0]) and np.array_equal(bits(dv), hist[s][1])
    # ---- decode through one captured CUDA graph, batch of 3 rows with one padding row (model_runner.py:262-273, 277-318)
    bs = 3
    slots_l = [2, 0, -1]
    q_s = torch.zeros(bs, n_q, 128, dtype=torch.bfloat16, device="cuda"); k_s = torch.zeros(bs, n_kv, 128, dtype=torch.bfloat16, device="cuda"); v_s = torch.zeros_like(k_s)
    kv_slots = torch.tensor(slots_l, dtype=torch.int32, device="cuda")

    def feed():
        q1 = O.f32_to_bf16((rng.standard_normal((bs, n_q, 128)) * 0.3).astype(np.float32))
        k1 = O.f32_to_bf16((rng.standard_normal((bs, n_kv, 128)) * 0.5).astype(np.float32)); v1 = O.f32_to_bf16((rng.standard_normal((bs, n_kv, 128)) * 0.5).astype(np.float32))
        q_s.copy_(to_bf16_cuda(q1)); k_s.copy_(to_bf16_cuda(k1)); v_s.copy_(to_bf16_cuda(v1))
        for b, s in enumerate(slots_l):
            if s >= 0: hist[s] = (np.concatenate([hist[s][0], k1[b:b + 1]]), np.concatenate([hist[s][1], v1[b:b + 1]]))
        return q1

    def check(out, q1, step):
        for b, s in enumerate(slots_l):
            if s < 0:
                assert float(out[b].abs().max()) == 0.0
                continue
            want = O.attention_ref(q1[b], hist[s][0], hist[s][1], SCALE)
            assert np.abs(out[b].float().cpu().numpy() - want).max() <= 2e-2 * np.abs(want).max() + 1e-3, (step, b)

    set_context(False, kv_slots=kv_slots, max_seqlen_k=512)
    q1 = feed()
    check(attn(q_s, k_s, v_s), q1, "warm-up")                              # the engine's eager warm-up step
    attn.gaac.growable = False                                             # model_runner.py:317-318: addresses are baked into the graph
    q1 = feed()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_s = attn(q_s, k_s, v_s)
    # the capture itself does not run the step; replay it once for the inputs fed above
    graph.replay(); check(out_s, q1, "first replay")
    for step in range(1, 40):
        q1 = feed()
        graph.replay()
        check(out_s, q1, step)
        if step % 16 == 0:                                                 # the engine's cadence: one host read every 16 decode steps
            attn.gaac.check_capacity(int(attn.gaac.max_escape_bytes()))
    reset_context()
    for s in slots_of:
        dk, dv = attn.gaac.decompress(s)
        assert np.array_equal(bits(dk), hist[s][0]) and np.array_equal(bits(dv), hist[s][1])
    assert int(attn.gaac.append_errors) == 0
