"""Time the UNMODIFIED reference package on this GPU, beside gaac_b200, on the headline workload of bench.py (batch 1, 32 q / 8 kv heads, 65536 tokens).

The reference is installed, as it is, under baseline/_ref (`pip install --no-deps --target baseline/_ref <reference checkout>`)
and its JIT extension `gaac_attn_v1` is prebuilt for sm_100a under baseline/_ref/_torch_ext by build_reference.py, so
that nothing is compiled with nvcc on the GPU box; its Triton encoder compiles there in seconds.  Both directories are
git-ignored.  This script runs the reference through its own public API (Codec.calibrate, TileEncoder.encode, attention) and
prints one JSON line: microseconds per layer of its CUDA kernel (its own nsplit heuristic, and the best of a small sweep),
milliseconds per encode of its Triton encoder, and live parity checks against gaac_b200 on the same tensors (encoder output,
attention over the reference's Pages, and the slot cache after prefill + appends).
bench.py runs it in a child process as a side measurement; it is not part of any timed region of gaac_b200.
"""
import json, os, sys, time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _extension_dir() -> str:
    """The prebuilt extension's directory, spelled as it was when it was built (see build_reference.py)."""
    ext = os.path.join(REF, "_torch_ext")
    try:
        built_as = open(os.path.join(ext, "BUILD_DIR")).read().strip()
        if built_as and os.path.realpath(built_as) == os.path.realpath(ext):
            ext = built_as
    except OSError:
        pass
    return ext


def _preload_extension(ref_kernel, name: str = "gaac_attn_v1") -> bool:
    """Hand a prebuilt extension to the reference's loader cache (gaac/kernel.py:329-337 and gaac/vllm/paged_kernel.py:282-288
    keep the loaded module in `_mod`).
    torch's JIT loader would rebuild it (over a minute of nvcc) because a copied tree does not keep the file times ninja logged;
    the library is the reference's own kernel, compiled from its own source by its own build step, only that step is not
    repeated.  Returns False (and the reference then builds it itself) when the library is not there or does not load."""
    so = os.path.join(os.environ["TORCH_EXTENSIONS_DIR"], name, name + ".so")
    try:
        import importlib.machinery, importlib.util
        import torch  # noqa: F401  (the extension links against libtorch)
        loader = importlib.machinery.ExtensionFileLoader(name, so)
        mod = importlib.util.module_from_spec(importlib.util.spec_from_loader(name, loader))
        loader.exec_module(mod)
        ref_kernel._mod = mod
        return True
    except Exception:
        return False


os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
os.environ.setdefault("TORCH_EXTENSIONS_DIR", _extension_dir())
sys.path.insert(0, REF)
sys.path.insert(1, os.path.dirname(HERE))

N_Q, N_KV, CTX, HEAD_DIM, N_SETS = 32, 8, 65536, 128, 4


def main():
    import torch
    import gaac as ref                                           # the reference package
    import gaac_b200 as ours
    from gaac_b200.synth import synth_kv
    dev = torch.device("cuda", 0)
    scale = HEAD_DIM ** -0.5
    out = {"reference_version": getattr(ref, "__version__", "0.1.0")}
    sets, enc_ms = [], []
    for i in range(N_SETS):
        k = synth_kv("k", N_KV, CTX, seed=100 + i, device=dev); v = synth_kv("v", N_KV, CTX, seed=100 + i, device=dev)
        ck, cv = ref.Codec(N_KV, device=dev).calibrate(k[:, :2048]), ref.Codec(N_KV, device=dev).calibrate(v[:, :2048])
        tk, tv = ref.TileEncoder("k", device=dev), ref.TileEncoder("v", device=dev)
        kp, vp = tk.encode(ck, k), tv.encode(cv, v)              # first call compiles the Triton kernels
        if i == 0:
            for _ in range(3): tk.encode(ck, k)
            torch.cuda.synchronize()
            for _ in range(9):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); tk.encode(ck, k); b.record(); torch.cuda.synchronize(); enc_ms.append(a.elapsed_time(b))
            # encoder parity, full size: gaac_b200's encoder on the same tensor and bases
            oc = ours.Codec(N_KV, dev); oc.set_bases(ck.base3, ck.base4)
            op = ours.TileEncoder("k", dev).encode(oc, k)
            out["encoder_bit_identical"] = bool(all(torch.equal(getattr(op, f), getattr(kp, f)) for f in ("sm", "codes", "flags", "tile_off", "ovf_head_start"))
                                                and torch.equal(op.ovf[:int(op.ovf_head_start[-1])], kp.ovf[:int(kp.ovf_head_start[-1])]))
        sets.append((kp, vp)); del k, v
    out["triton_encode_ms"] = sorted(enc_ms)[len(enc_ms) // 2]
    out["triton_encode_blocks_per_s"] = N_KV * (CTX // 16) / (out["triton_encode_ms"] * 1e-3)
    q = torch.randn(1, N_Q, HEAD_DIM, generator=torch.Generator(device=dev).manual_seed(7), device=dev).to(torch.bfloat16)

    def timed(fn, n=200, warm=20):
        for i in range(warm): fn(i)
        torch.cuda.synchronize(); ts = []
        for i in range(n):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(i); b.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(b) * 1e3)
        return sorted(ts)[len(ts) // 2]

    t0 = time.time()
    import gaac.kernel as ref_kernel
    out["extension_preloaded"] = _preload_extension(ref_kernel)
    o_ref = ref.attention(q, *sets[0], scale=scale)              # loads (or builds) the reference's CUDA extension
    torch.cuda.synchronize()
    out["extension_load_s"] = time.time() - t0
    o_ours = ours.attention(q, *sets[0], scale=scale)            # gaac_b200 reading the reference's Pages: the drop-in claim
    out["attn_max_abs_diff_vs_gaac_b200"] = float((o_ref.float() - o_ours.float()).abs().max())
    ns0 = ref.choose_nsplit(1, N_KV, CTX)
    res = {}
    for ns in sorted({ns0, 18, 36, 48}):
        res[ns] = timed(lambda i: ref.attention(q, *sets[i % N_SETS], scale=scale, nsplit=ns))
    out["attn_us_by_nsplit"] = res
    out["attn_us_own_nsplit"] = res[ns0]; out["own_nsplit"] = ns0
    out["attn_us_best"] = min(res.values())
    out["gaac_b200_us_same_protocol"] = timed(lambda i: ours.attention(q, *sets[i % N_SETS], scale=scale))
    out.update(slot_cache_parity(torch, ref, ours, dev))
    out.update(paged_store_parity(torch, ref, ours, dev))
    out.update(paged_attention_timing(torch, ref, dev, timed))
    print(json.dumps(out), flush=True)


def paged_attention_timing(torch, ref, dev, timed) -> dict:
    """The reference's paged kernel (gaac_vpaged + gaac_combine2) and ours on the same block buffer: 16 ragged sequences as in
    bench.py --workload paged16, stored once (the stores are byte-identical, see paged_store_parity)."""
    import numpy as np
    from gaac_b200.synth import synth_kv
    try:
        import gaac.vllm.paged_kernel as rpk
        from gaac_b200.vllm.store import LayerState, OVF_OFF
        from gaac_b200.vllm.paged_kernel import paged_attention as our_paged
        from gaac_b200.kernel import choose_nsplit_sm100
        if not _preload_extension(rpk, "gaac_vpaged128_v1"):
            return {"paged_attn_unavailable": "the reference's paged extension is not prebuilt"}
        n_kv, G, B = 8, 4, 16
        rng = np.random.default_rng(0)
        lens = [int(l) // 16 * 16 + int(t) for l, t in zip(rng.integers(4096, 65537, B), rng.integers(0, 16, B))]
        num_blocks = sum((l + 15) // 16 for l in lens) + 1024
        ck = ref.Codec(n_kv, device=dev).calibrate(synth_kv("k", n_kv, 2048, 7, dev)); cv = ref.Codec(n_kv, device=dev).calibrate(synth_kv("v", n_kv, 2048, 7, dev))
        st = LayerState(num_blocks, n_kv, raw_tiles=B * 2 * n_kv + 4096, ovf_slot=128, device=dev, bases={"k3": ck.base3, "k4": ck.base4, "v3": cv.base3, "v4": cv.base4})
        buf = torch.zeros(num_blocks * 2 * n_kv * (OVF_OFF + 128), dtype=torch.uint8, device=dev)
        perm = rng.permutation(num_blocks); used = 0
        bt = np.zeros((B, (max(lens) + 15) // 16), np.int32)
        for i, L in enumerate(lens):
            k = synth_kv("k", n_kv, L, 7, dev).transpose(0, 1).contiguous(); v = synth_kv("v", n_kv, L, 7, dev).transpose(0, 1).contiguous()
            nb = (L + 15) // 16
            blocks = perm[used:used + nb]; used += nb; bt[i, :nb] = blocks
            ent = np.array([[blocks[t], t * 16, 0, min(16, L - t * 16)] for t in range(nb)], np.int32)
            st.store(k, v, buf, torch.from_numpy(ent).to(dev), torch.empty(nb * 2 * n_kv, dtype=torch.int32, device=dev))
        btd = torch.from_numpy(bt).to(dev); sl = torch.tensor(lens, dtype=torch.int32, device=dev)
        q = torch.randn(B, n_kv * G, 128, generator=torch.Generator(device=dev).manual_seed(2), device=dev).to(torch.bfloat16)
        o_r = torch.empty(B, n_kv * G * 128, dtype=torch.bfloat16, device=dev); o_o = torch.empty_like(o_r)
        ns0 = rpk.choose_nsplit(B, n_kv, max(lens))
        res = {ns: timed(lambda i: rpk.paged_attention(q, o_r, buf, st.raw, st.mt, btd, sl, st.bases, st.TS, n_kv * G, n_kv, ns), n=20, warm=3) for ns in sorted({ns0, 4, 8, 16})}
        rpk.paged_attention(q, o_r, buf, st.raw, st.mt, btd, sl, st.bases, st.TS, n_kv * G, n_kv, 8)
        ns_o = choose_nsplit_sm100(B, n_kv, bt.shape[1] * 16, ragged=True)
        us_o = timed(lambda i: our_paged(q, o_o, buf, st.raw, st.mt, btd, sl, st.bases, st.TS, n_kv * G, n_kv, ns_o), n=20, warm=3)
        return {"paged_attn_us_by_nsplit": res, "paged_attn_us_own_nsplit": res[ns0], "paged_own_nsplit": ns0, "paged_attn_us_best": min(res.values()),
                "paged_gaac_b200_us": us_o, "paged_attn_max_abs_diff_vs_gaac_b200": float((o_r.float() - o_o.float()).abs().max())}
    except Exception as e:
        return {"paged_attn_error": repr(e)[:300]}


def paged_store_parity(torch, ref, ours, dev) -> dict:
    """The paged store of both packages fed with the same entries (three prompts stored block by block, then 24 decode steps of one
    token per sequence, so filling blocks pass through raw tiles and are finalised): the block buffers must be byte-identical, the
    mode tables must agree on which tiles are compressed (raw tile numbers may differ: the pop order of concurrent programs is
    free), and decoding every block back through each package's own decoder must give the same BF16 rows."""
    from gaac_b200.synth import synth_kv
    try:
        from gaac.vllm.store import LayerState as RefState, OVF_OFF
        from gaac_b200.vllm.store import LayerState as OurState
        n_kv, num_blocks, ovf_slot = 4, 96, 128
        TS = OVF_OFF + ovf_slot
        cal_k, cal_v = synth_kv("k", n_kv, 2048, 700, dev), synth_kv("v", n_kv, 2048, 700, dev)
        ck, cv = ref.Codec(n_kv, device=dev).calibrate(cal_k), ref.Codec(n_kv, device=dev).calibrate(cal_v)
        bases = {"k3": ck.base3, "k4": ck.base4, "v3": cv.base3, "v4": cv.base4}
        rs, os_ = RefState(num_blocks, n_kv, 64, bases, ovf_slot, dev), OurState(num_blocks, n_kv, 64, bases, ovf_slot, dev)
        rbuf = torch.zeros(num_blocks * 2 * n_kv * TS, dtype=torch.uint8, device=dev); obuf = torch.zeros_like(rbuf)
        lens, blocks, nxt = [150, 33, 64], [], 0
        for i, L in enumerate(lens):
            k = synth_kv("k", n_kv, L, 700, dev).transpose(0, 1).contiguous(); v = synth_kv("v", n_kv, L, 700, dev).transpose(0, 1).contiguous()
            nb = (L + 15) // 16
            bl = list(range(nxt, nxt + nb + 2)); nxt += nb + 2; blocks.append(bl)
            ent = torch.tensor([[bl[t], t * 16, 0, min(16, L - t * 16)] for t in range(nb)], dtype=torch.int32, device=dev)
            for st, buf in ((rs, rbuf), (os_, obuf)):
                st.store(k.view(torch.int16), v.view(torch.int16), buf, ent, torch.empty(nb * 2 * n_kv, dtype=torch.int32, device=dev))
        g = torch.Generator(device=dev).manual_seed(11)
        for step in range(24):
            k = (torch.randn(3, n_kv, 128, generator=g, device=dev) * cal_k[:, :3].transpose(0, 1).float().abs().clamp(min=0.05)).to(torch.bfloat16)
            v = (torch.randn(3, n_kv, 128, generator=g, device=dev) * cal_v[:, :3].transpose(0, 1).float().abs().clamp(min=0.05)).to(torch.bfloat16)
            ent = torch.tensor([[blocks[i][lens[i] // 16], i, lens[i] % 16, 1] for i in range(3)], dtype=torch.int32, device=dev)
            for st, buf in ((rs, rbuf), (os_, obuf)):
                st.store(k.view(torch.int16), v.view(torch.int16), buf, ent, torch.empty(3 * 2 * n_kv, dtype=torch.int32, device=dev))
            lens = [l + 1 for l in lens]
        torch.cuda.synchronize()
        same = bool(torch.equal(rbuf, obuf) and torch.equal(rs.mt < 0, os_.mt < 0) and torch.equal(rs.mt[rs.mt >= 0], os_.mt[os_.mt >= 0])
                    and int(rs.top) == int(os_.top) and int(rs.err) == int(os_.err) == 0)
        pairs, row = [], 0
        for i, L in enumerate(lens):
            for t in range((L + 15) // 16):
                pairs.append([blocks[i][t], row, min(16, L - t * 16)]); row += 16
        pairs = torch.tensor(pairs, dtype=torch.int32, device=dev)
        rk = torch.zeros(row, n_kv, 128, dtype=torch.bfloat16, device=dev); rv = torch.zeros_like(rk); ok = torch.zeros_like(rk); ov = torch.zeros_like(rk)
        rs.decode_blocks(rbuf, pairs, rk, rv); os_.decode_blocks(obuf, pairs, ok, ov)
        same = same and torch.equal(rk.view(torch.int16), ok.view(torch.int16)) and torch.equal(rv.view(torch.int16), ov.view(torch.int16))
        return {"paged_store_bit_identical": bool(same), "paged_raw_tiles_in_use": int((os_.mt < 0).sum())}
    except Exception as e:
        return {"paged_store_bit_identical": None, "paged_store_error": repr(e)[:300]}


def slot_cache_parity(torch, ref, ours, dev) -> dict:
    """The slot cache of both packages fed with the same prompts and the same decode steps (per-sequence calibration, prefill of
    two sequences of different length, 40 appended tokens each, so tiles are finalised on the way): every compressed buffer must
    be byte-identical, and both attentions over their own cache must agree."""
    from gaac_b200.synth import synth_kv
    try:
        n_kv, n_q, cap = 4, 16, 512
        rc, oc = ref.CompressedKVCache(2, n_kv, cap, device=dev), ours.CompressedKVCache(2, n_kv, cap, device=dev)
        for slot, L in ((0, 200), (1, 77)):
            k = synth_kv("k", n_kv, L, 900 + slot, dev).transpose(0, 1).contiguous(); v = synth_kv("v", n_kv, L, 900 + slot, dev).transpose(0, 1).contiguous()
            rc.prefill(slot, k, v); oc.prefill(slot, k, v)
        slots = torch.tensor([0, 1], dtype=torch.int32, device=dev)
        g = torch.Generator(device=dev).manual_seed(3)
        for step in range(40):
            k = (torch.randn(2, n_kv, 128, generator=g, device=dev) * 2).to(torch.bfloat16); v = torch.randn(2, n_kv, 128, generator=g, device=dev).to(torch.bfloat16)
            rc.append(slots, k, v); oc.append(slots, k, v)
        torch.cuda.synchronize()
        same = bool(torch.equal(rc.S, oc.S) and torch.equal(rc.tail_len, oc.tail_len))
        for a, b in ((rc.k, oc.k), (rc.v, oc.v)):
            used = int(a.ovf_used.max())
            same = same and all(torch.equal(getattr(a, f), getattr(b, f)) for f in ("sm", "codes", "flags", "tile_off", "ovf_used", "base3", "base4"))
            same = same and torch.equal(a.ovf.view(a.H, -1)[:, :used], b.ovf.view(b.H, -1)[:, :used])
            for h in range(a.H):
                n = int(rc.tail_len[h])
                same = same and torch.equal(a.tail[h, :n], b.tail[h, :n])
        q = torch.randn(2, n_q, 128, generator=g, device=dev).to(torch.bfloat16)
        o_r = rc.attention(q, slots, 128 ** -0.5); o_o = oc.attention(q, slots, 128 ** -0.5)
        return {"slot_cache_bit_identical": same, "slot_cache_attn_max_abs_diff": float((o_r.float() - o_o.float()).abs().max())}
    except Exception as e:                                      # a side check must not lose the timings above
        return {"slot_cache_bit_identical": None, "slot_cache_error": repr(e)[:200]}


if __name__ == "__main__":
    main()
