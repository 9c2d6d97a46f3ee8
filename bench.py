"""Benchmark of the GAAC hot path on B200: fused decode attention over the compressed KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ctx64k|ctx128k|paged16|batch64]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Headline workload `ctx64k` (synthetic, see gaac_b200/synth.py): decode attention, batch 1, 32 query heads / 8 KV heads (GQA 4),
head_dim 128, 65536-token context, KV fully encoded into the slot layout with a 0-token tail, softmax scale 1/sqrt(128).
A STEP is one decode step of a 32-layer model: 32 attention layers back to back, replayed from CUDA graphs of 16 layers, rotating
over several independent KV sets whose total size exceeds the L2 cache, so every layer streams its compressed bytes from HBM.
`value` is microseconds per LAYER (step time / 32), device-timed with inputs resident in HBM.  With N > 1 GPUs the context is
split into N contiguous token ranges (strong scaling): each rank attends over its range, pushes its per-head partials
(m, l, acc) into every rank's memory over NVLink from the attention kernel's epilogue, waits for the others in the same launch
and merges; an NCCL all-gather + merge kernel is the fallback.

Other workloads print one line each in the same format:
  ctx128k  32 layers x 131072 tokens, context split over the ranks; value = milliseconds per 32-layer decode step
  paged16  16 ragged sequences (4096..65536 tokens) in the paged layout, sharded by sequence; a step = append one token per
           sequence through the store (blocks that fill are encoded) + paged attention
  batch64  64 sequences x 32768 tokens, kv heads sharded over the ranks; a step = append + attention of one layer; also a
           prefill-encode pass through CompressedKVCache.prefill and the encoder's rate on a whole layer
One JSON line on stdout (rank 0).  `e2e` is the same metric fed from pinned host memory with the results read back.
"""
from __future__ import annotations
import argparse, json, os, subprocess, sys, threading, time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_Q, N_KV, HEAD_DIM = 32, 8, 128
N_SETS = 4                         # independent KV sets rotated over ("layers"): 4 x ~193 MB compressed > 126 MB of L2
SCALE = HEAD_DIM ** -0.5
LAYERS_PER_STEP = 32               # a decode step of a 32-layer model
LAYERS_PER_GRAPH = 16              # layers captured in one CUDA graph; a step replays two of them
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_attn_kernel launch at the 65536-token workload, from the ncu capture
# summarised in profiles/ (scaled by tokens for other context lengths: the traffic is proportional to the tiles read)
NCU_TRAFFIC_BYTES_64K = 197.1e6


def workload_text(ctx: int) -> str:
    return f"decode attention, batch 1, {N_Q} q heads / {N_KV} kv heads (GQA {N_Q // N_KV}), head_dim {HEAD_DIM}, {ctx}-token context, slot layout, 0-token tail"


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs (read-only query)."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int, period_ms: int = 50):
        self.index, self.period_ms, self.rows, self.proc = index, period_ms, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True); self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try: self.proc.wait(timeout=5)
            except Exception: pass

    def summary(self, t_from: float | None = None, t_to: float | None = None) -> dict:
        rows = [r for t, r in self.rows if (t_from is None or t >= t_from) and (t_to is None or t <= t_to)]
        mhz = sorted(int(r[0]) for r in rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(mhz)}


class Ranks:
    """One process per GPU: rank / world from the launcher's environment, NCCL process group when N > 1."""

    def __init__(self, args):
        import torch
        self.torch = torch
        self.world = int(os.environ.get("WORLD_SIZE", "1")); self.rank = int(os.environ.get("RANK", "0")); self.local = int(os.environ.get("LOCAL_RANK", "0"))
        assert self.world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE {self.world}: launch with torch.distributed.run"
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import datetime
            import torch.distributed as dist
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")          # plain peer loads/stores only
            dist.init_process_group("nccl", device_id=self.dev, timeout=datetime.timedelta(seconds=90))     # fail fast instead of hanging
            self.dist = dist

    def barrier(self):
        if self.dist: self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if not self.dist: return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t)

    def min_over_ranks(self, x: int) -> int:
        if not self.dist: return x
        t = self.torch.tensor([x], dtype=self.torch.int32, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return int(t)

    def finish(self):
        """Leave.  With N > 1 the process group is torn down in the ordinary way (every graph that could hold one of its kernels has
        been released by then); a watchdog ends the process if the teardown has not returned after 20 s, so that a stuck
        communicator cannot hold N GPUs until the launcher's own limit."""
        sys.stdout.flush(); sys.stderr.flush()
        if not self.dist: return
        self.barrier()
        threading.Timer(20.0, lambda: os._exit(0)).start()
        try:
            self.dist.destroy_process_group()
        finally:
            sys.stdout.flush(); sys.stderr.flush()
            os._exit(0)


def keep_busy(launch, R, seconds: float = 0.6) -> int:
    """Untimed launches of the step's dominant kernel for about `seconds`, run right before a timed region inside the
    clock-sampling window: the clock record then shows the GPU under this load (a region of a few milliseconds would fall
    between two samples).  Every rank runs the same count.  Returns the number of launches."""
    import torch
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(4): launch()
    b.record(); torch.cuda.synchronize()
    n = int(R.max_over_ranks(float(max(1, min(20000, int(seconds / max(a.elapsed_time(b) / 4e3, 1e-5)))))))
    for _ in range(n): launch()
    return n


# ------------------------------------------------------------------------------------------------ reference arm (CPU)
class CpuPath:
    """The reference's CPU path for this workload - decode the compressed cache (gaac/codec.py:186-218) and run softmax
    attention on the decoded KV - restated in numpy (oracle/), run on a bounded sample and scaled to the full layer.  Used only
    when the reference package itself did not travel with the repository."""

    def __init__(self, sample_heads: int, sample_tokens: int, threads: int, ctx: int):
        import numpy as np
        from oracle import gaac_oracle as O
        self.np, self.O, self.threads, self.heads = np, O, threads, sample_heads
        self.G = N_Q // N_KV
        rng = np.random.default_rng(0)
        k16, v16 = O.synth_kv("k", sample_heads, sample_tokens, 0), O.synth_kv("v", sample_heads, sample_tokens, 0)
        kb3, kb4 = O.calibrate(k16[:, :2048], sample_heads); vb3, vb4 = O.calibrate(v16[:, :2048], sample_heads)
        self.q16 = O.f32_to_bf16(rng.standard_normal((sample_heads * self.G, HEAD_DIM)).astype(np.float32))
        chunk = max(256, (sample_tokens // max(1, threads)) // 16 * 16)
        self.pages = []
        for h in range(sample_heads):
            for t0 in range(0, sample_tokens, chunk):
                sl = slice(t0, t0 + chunk)
                self.pages.append((h, O.encode(k16[h:h + 1, sl], kb3[h:h + 1], kb4[h:h + 1], "k", 1), O.encode(v16[h:h + 1, sl], vb3[h:h + 1], vb4[h:h + 1], "v", 1)))
        self.frac = (sample_heads * sample_tokens) / (N_KV * ctx)
        self.sample = f"{sample_heads} of {N_KV} kv heads x {sample_tokens} of {ctx} tokens (codec decode + softmax attention), time scaled by {1 / self.frac:.0f}"

    def _work(self, item):
        np, O = self.np, self.O
        h, kp, vp = item
        k = O.bf16_to_f64(O.decode(kp)[0]).astype(np.float32); v = O.bf16_to_f64(O.decode(vp)[0]).astype(np.float32)
        q = O.bf16_to_f64(self.q16[h * self.G:(h + 1) * self.G]).astype(np.float32)
        s = (q @ k.T) * SCALE
        m = s.max(-1)
        p = np.exp(s - m[:, None])
        return h, m, p.sum(-1), p @ v

    def step_us_per_layer(self) -> float:
        from concurrent.futures import ThreadPoolExecutor
        np, O = self.np, self.O
        t = time.perf_counter()
        with ThreadPoolExecutor(self.threads) as ex:
            parts = list(ex.map(self._work, self.pages))
        for h in range(self.heads):                   # merge the chunks of each head (same algebra as the split merge)
            ph = [p for p in parts if p[0] == h]
            O.combine_partials(np.stack([p[1] for p in ph], -1), np.stack([p[2] for p in ph], -1), np.stack([p[3] for p in ph], -2))
        return (time.perf_counter() - t) / self.frac * 1e6


class RefCpuPath:
    """The reference's own CPU path, run from the unmodified package installed under baseline/_ref: `Codec.decode` of the
    compressed K and V (gaac/codec.py:186-218) followed by torch's scaled_dot_product_attention on the decoded BF16 KV
    (the comparison of examples/attention.py:27-32 on the host), all host threads.  sample_heads / sample_tokens equal to the
    workload's = the whole layer, nothing scaled."""

    def __init__(self, sample_heads: int, sample_tokens: int, threads: int, ctx: int):
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "gaac")):
            raise FileNotFoundError("reference package not installed under baseline/_ref")
        if ref_dir not in sys.path: sys.path.insert(0, ref_dir)
        import torch
        import gaac as ref
        from gaac_b200.synth import synth_kv
        torch.set_num_threads(threads)
        self.torch, self.ref, self.heads = torch, ref, sample_heads
        k = synth_kv("k", sample_heads, sample_tokens, 0, device="cpu"); v = synth_kv("v", sample_heads, sample_tokens, 0, device="cpu")
        ck = ref.Codec(sample_heads, device="cpu").calibrate(k[:, :2048]); cv = ref.Codec(sample_heads, device="cpu").calibrate(v[:, :2048])
        self.kp, self.vp = ck.encode(k, "k"), cv.encode(v, "v")
        G = N_Q // N_KV
        self.q = torch.randn(1, sample_heads * G, 1, HEAD_DIM, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
        self.frac = (sample_heads * sample_tokens) / (N_KV * ctx)
        whole = sample_heads == N_KV and sample_tokens == ctx
        self.sample = (f"the whole layer: {N_KV} kv heads x {ctx} tokens (reference Codec.decode on CPU + torch SDPA), nothing scaled" if whole else
                       f"{sample_heads} of {N_KV} kv heads x {sample_tokens} of {ctx} tokens (reference Codec.decode on CPU + torch SDPA), time scaled by {1 / self.frac:.0f}")

    def step_us_per_layer(self) -> float:
        torch, F = self.torch, self.torch.nn.functional
        t = time.perf_counter()
        k = self.ref.Codec.decode(self.kp); v = self.ref.Codec.decode(self.vp)                   # [H, S, 128] bf16
        F.scaled_dot_product_attention(self.q, k.unsqueeze(0), v.unsqueeze(0), scale=SCALE, enable_gqa=True)
        return (time.perf_counter() - t) / self.frac * 1e6


def make_cpu_path(sample_heads: int, sample_tokens: int, threads: int, ctx: int):
    """(path, kind): the reference's own CPU code when its package travelled with the repository, else the oracle's restatement."""
    try:
        return RefCpuPath(sample_heads, sample_tokens, threads, ctx), "reference"
    except Exception as e:
        print(f"reference CPU path unavailable ({type(e).__name__}: {e}); timing the oracle port", file=sys.stderr, flush=True)
        return CpuPath(min(sample_heads, 1), min(sample_tokens, 16384), threads, ctx), "port"


def cpu_path_within(budget_s: float, calls: int, threads: int, ctx: int):
    """The largest CPU sample whose `calls` calls fit the time budget: the whole layer first, then 1 kv head x 16384 tokens,
    then 1 x 4096.  Returns (path, kind, seconds of the first call)."""
    for heads, tokens in ((N_KV, ctx), (1, 16384), (1, 4096)):
        cpu, kind = make_cpu_path(heads, tokens, threads, ctx)
        t = time.perf_counter(); cpu.step_us_per_layer(); t = time.perf_counter() - t
        if t * calls <= budget_s or (heads, tokens) == (1, 4096):
            return cpu, kind, t
    raise AssertionError


def run_reference(args):
    """The reference arm: the reference's CPU implementation of the path on this box's host cores, the same metric and config."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ctx = 131072 if args.workload == "ctx128k" else 65536
    threads = os.cpu_count() or 1
    cpu, kind, _ = cpu_path_within(150.0, args.steps + args.warmup, threads, ctx)
    for _ in range(args.warmup): cpu.step_us_per_layer()
    vals = [cpu.step_us_per_layer() for _ in range(args.steps)]
    us = sum(vals) / len(vals)
    metric, unit, value = ("decode_attn_us_per_layer_64k_ctx", "us/layer", us) if ctx == 65536 else ("decode_attn_ms_per_32_layer_step_128k_ctx", "ms/step", us * LAYERS_PER_STEP / 1e3)
    line = {"impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16" if kind == "reference" else "f32", "data": "synthetic",
            "config": {"workload": workload_text(ctx), "step": ("a timed step of this arm is ONE layer call (ms_per_step is its time); us/layer needs no scaling" if ctx == 65536 else
                                "a timed step of this arm is ONE layer call (ms_per_step is its time); the 32-layer value is 32 times that"),
                       "path": ("CPU: the unmodified reference package (baseline/_ref): Codec.decode + torch scaled_dot_product_attention" if kind == "reference"
                                else "CPU: numpy restatement (oracle/) of the reference codec decode + softmax attention")},
            "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": kind, "sample": cpu.sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ batch-1 long context (headline)
def run_context(args, ctx: int):
    import torch
    from gaac_b200 import Codec, TileEncoder, _lib, attention
    from gaac_b200.kernel import _pages_call, choose_nsplit_sm100, combine_parts
    from gaac_b200.synth import synth_kv
    R = Ranks(args)
    torch, dev, world, rank = R.torch, R.dev, R.world, R.rank
    _lib.lib()
    headline = ctx == 65536

    # ---- this rank's share of the context: contiguous, tile aligned
    tiles = ctx // 16
    t_lo, t_hi = tiles * rank // world, tiles * (rank + 1) // world
    S_loc = (t_hi - t_lo) * 16
    g = torch.Generator(device=dev).manual_seed(7)
    q = torch.randn(1, N_Q, HEAD_DIM, generator=g, device=dev).to(torch.bfloat16)
    sets, parity_ref = [], None
    for i in range(N_SETS):
        k = synth_kv("k", N_KV, ctx, seed=100 + i, device=dev); v = synth_kv("v", N_KV, ctx, seed=100 + i, device=dev)
        ck, cv = Codec(N_KV, dev).calibrate(k[:, :2048]), Codec(N_KV, dev).calibrate(v[:, :2048])
        kp = TileEncoder("k", dev).encode(ck, k[:, t_lo * 16:t_hi * 16].contiguous()); vp = TileEncoder("v", dev).encode(cv, v[:, t_lo * 16:t_hi * 16].contiguous())
        sets.append((kp, vp))
        if i == 0:                       # float64 reference of set 0 over the WHOLE context (the codec is lossless), and sum p|v| for the bound
            s = torch.einsum("hgd,htd->hgt", q[0].double().view(N_KV, N_Q // N_KV, HEAD_DIM), k.double()) * SCALE
            p = torch.softmax(s, -1); vd = v.double()
            parity_ref = (torch.einsum("hgt,htd->hgd", p, vd).reshape(N_Q, HEAD_DIM), torch.einsum("hgt,htd->hgd", p, vd.abs()).reshape(N_Q, HEAD_DIM))
            del s, p, vd
        del k, v
    comp_bytes = sum(kp.nbytes + vp.nbytes for kp, vp in sets) / N_SETS
    algo_bytes = comp_bytes + 2 * N_Q * HEAD_DIM * 2                                   # + q + out (bf16)
    bf16_bytes = 2 * N_KV * S_loc * HEAD_DIM * 2
    nsplit = choose_nsplit_sm100(1, N_KV, S_loc)

    # N > 1: the partials travel by plain stores from the attention kernel's epilogue into every rank's receive buffer (peer
    # memory) and the same launch waits and merges; NCCL all-gather + merge kernel when the peer mapping cannot be set up.
    peer, exchange_mode = None, "none"
    part = torch.empty(N_Q, 130, dtype=torch.float32, device=dev)
    gathered = torch.empty(world * N_Q, 130, dtype=torch.float32, device=dev)
    if world > 1:
        exchange_mode = "nccl all-gather + merge kernel"
        ok = 0
        if not args.nccl_exchange:
            try:
                from gaac_b200.dist import PeerExchange
                peer = PeerExchange(N_Q, dev, groups=N_KV); ok = 1
            except Exception as e:
                print(f"[rank {rank}] peer exchange unavailable: {type(e).__name__}: {e}", file=sys.stderr, flush=True)
        if R.min_over_ranks(ok) == 1:
            exchange_mode = ("partials pushed into peer memory by the attention kernel (NVLink stores); " +
                             ("a separate wait-and-merge kernel" if args.two_kernel_exchange else "the same launch waits for the other ranks and merges"))
        else:
            peer = None
    fused = peer is not None and not args.two_kernel_exchange

    def layer(i, qq, out=None, out_f32=None):
        """One attention layer over KV set i; qq [1, N_Q, 128]; returns (and, when given, fills) the [N_Q, 128] bf16 output."""
        kp, vp = sets[i % N_SETS]
        if world == 1:
            return attention(qq, kp, vp, scale=SCALE, nsplit=nsplit, out_f32=out_f32, out=out)                 # the call a user makes
        if out is None: out = torch.empty(N_Q, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        if fused:
            _pages_call(qq, kp, vp, 1, N_Q, N_KV, SCALE, nsplit, out=out, out_f32=out_f32, exchange=peer.x, fused=True)
            return out
        if peer is not None:
            _pages_call(qq, kp, vp, 1, N_Q, N_KV, SCALE, nsplit, exchange=peer.x)
            o = peer.merge(N_KV, out_f32=out_f32); out.copy_(o); return out
        _pages_call(qq, kp, vp, 1, N_Q, N_KV, SCALE, nsplit, part=part)
        R.dist.all_gather_into_tensor(gathered, part)
        o = combine_parts(gathered.view(world, N_Q, 130), out_f32=out_f32); out.copy_(o); return out

    launches_per_layer = 1 if (world == 1 or fused) else 2     # ours: attention (+ the merge kernel); NCCL's own kernel is not counted

    for i in range(max(3, args.warmup)):
        layer(i, q)
    R.barrier()
    # ---- parity of this very set-up: fp32 result of layer 0 against the float64 reference of the whole context
    o32 = torch.empty(N_Q, HEAD_DIM, dtype=torch.float32, device=dev)
    layer(0, q, out_f32=o32.view(1, N_Q, HEAD_DIM) if world == 1 else o32)
    torch.cuda.synchronize()
    err = (o32.double() - parity_ref[0]).abs()
    bound = torch.clamp(parity_ref[1] * 2.0 ** -12, min=2e-3)
    parity = {"max_abs_err_fp32": float(err.max()), "bound": "max(2e-3, 2^-12 * sum_i p_i |v_i|) per element", "worst_err_over_bound": float((err / bound).max()),
              "within_2e-3_flat": bool(float(err.max()) <= 2e-3), "reference": "float64 softmax attention over the original BF16 K/V of KV set 0, whole context"}
    del parity_ref

    if args.profile:                                            # the command to run under ncu: a few eager layers, nothing else
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for i in range(args.steps):
            ev[i][0].record(); layer(i, q); ev[i][1].record()
        torch.cuda.synchronize()
        ts = sorted(a.elapsed_time(b) for a, b in ev)
        if rank == 0: print(json.dumps({"profile_run": True, "kernel_us_median": ts[len(ts) // 2] * 1e3, "nsplit": nsplit, "parity": parity}), flush=True)
        R.finish()
        return

    # ---- CUDA graphs: the launch path of a decode loop, which the reference's serving engine also captures.  One graph holds
    # LAYERS_PER_GRAPH consecutive layers (the kernels carry programmatic-dependent-launch edges, so a layer's CTAs become
    # resident while the previous layer's split merge is finishing); a step replays LAYERS_PER_STEP / LAYERS_PER_GRAPH of them.
    g_half, launch_mode = None, "eager"
    if not args.no_graph:
        try:
            g_half = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_half):
                keep = [layer(i, q) for i in range(LAYERS_PER_GRAPH)]
            launch_mode = f"cuda graph replay, {LAYERS_PER_GRAPH} layers per graph"
        except Exception as e:                                                          # capture unsupported: the same on every rank
            g_half = None; launch_mode = f"eager (graph capture failed: {type(e).__name__})"
        R.barrier()

    def run_steps(n):
        for _ in range(n):
            if g_half is not None:
                for _ in range(LAYERS_PER_STEP // LAYERS_PER_GRAPH): g_half.replay()
            else:
                for i in range(LAYERS_PER_STEP): layer(i, q)

    warm = max(3, args.warmup)
    run_steps(warm)
    R.barrier()
    # how many steps keep the GPU busy for about 0.7 s: they run, untimed, right before the timed region so that the clock sampler
    # sees the loaded state that the timed steps run in (the timed region itself can be shorter than one sampling period)
    t_probe = time.perf_counter(); run_steps(2); torch.cuda.synchronize(); t_probe = (time.perf_counter() - t_probe) / 2
    preload = int(R.max_over_ranks(float(max(1, int(0.7 / max(t_probe, 1e-5))))))
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(R.local) as clk:
        R.barrier()
        c_from = time.perf_counter()
        run_steps(preload)
        R.barrier()
        t0.record()
        run_steps(args.steps)
        t1.record()
        R.barrier()
        c_to = time.perf_counter()
    total_ms = R.max_over_ranks(t0.elapsed_time(t1))
    ms_per_step = total_ms / args.steps
    us_per_layer = ms_per_step * 1e3 / LAYERS_PER_STEP

    # ---- one layer at a time.  (1) the kernel's own duration: the same 16-layer graph captured with the programmatic dependent
    # launch switched off, so that every layer starts only after its predecessor has finished entirely; time / layers.  (2) the
    # protocol of the reference's own measurement (examples/attention.py:36-44): event-bracketed single eager calls with a
    # synchronise in between, which adds the host's launch path to every call.
    lib = _lib.lib()
    iso_us, g_iso = None, None
    if not args.no_graph:
        try:
            lib.gaac_set_launch_overlap(0)
            R.barrier()
            g_iso = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_iso):
                keep_iso = [layer(i, q) for i in range(LAYERS_PER_GRAPH)]
        except Exception as e:
            g_iso = None
            print(f"serialised graph capture failed ({type(e).__name__})", file=sys.stderr, flush=True)
        finally:
            lib.gaac_set_launch_overlap(1)
    if g_iso is not None:
        for _ in range(3): g_iso.replay()
        R.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20): g_iso.replay()
        b.record(); torch.cuda.synchronize()
        iso_us = R.max_over_ranks(a.elapsed_time(b) * 1e3 / (20 * LAYERS_PER_GRAPH))
    per_call = []
    for i in range(10): layer(i, q)
    R.barrier()
    for i in range(60):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); layer(i, q); b.record(); torch.cuda.synchronize(); per_call.append(a.elapsed_time(b) * 1e3)
    per_call.sort()
    per_call_us = R.max_over_ranks(per_call[len(per_call) // 2])
    if iso_us is None: iso_us = per_call_us

    # ---- end to end: one step = the 32 layers' queries from pinned host memory, 32 attention calls through the public API, the 32
    # results back in pinned host memory, one synchronise; captured as one CUDA graph and replayed (falls back to eager)
    q_host = q.expand(LAYERS_PER_STEP, N_Q, HEAD_DIM).contiguous().cpu().pin_memory()
    out_host = torch.empty(LAYERS_PER_STEP, N_Q, HEAD_DIM, dtype=torch.bfloat16).pin_memory()
    q_dev = torch.empty(LAYERS_PER_STEP, N_Q, HEAD_DIM, dtype=torch.bfloat16, device=dev)
    out_dev = torch.empty(LAYERS_PER_STEP, N_Q, HEAD_DIM, dtype=torch.bfloat16, device=dev)

    def e2e_body():
        q_dev.copy_(q_host, non_blocking=True)
        for l in range(LAYERS_PER_STEP):
            layer(l, q_dev[l:l + 1], out=out_dev[l])
        out_host.copy_(out_dev, non_blocking=True)
    e2e_mode, g_e2e = "eager", None
    for _ in range(2):
        e2e_body(); torch.cuda.synchronize()
    if not args.no_graph and (world == 1 or peer is not None):
        try:
            R.barrier()
            g_e2e = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_e2e):
                e2e_body()
            e2e_mode = "one CUDA graph per step (copy in, 32 attention calls, copy out)"
        except Exception as e:
            g_e2e = None
            print(f"e2e graph capture failed ({type(e).__name__}); timing the eager step", file=sys.stderr, flush=True)
    def e2e_step():
        if g_e2e is not None: g_e2e.replay()
        else: e2e_body()
        torch.cuda.synchronize()
    for _ in range(3): e2e_step()
    R.barrier()
    tb = time.perf_counter()
    for _ in range(args.steps): e2e_step()
    R.barrier()
    e2e_us = R.max_over_ranks((time.perf_counter() - tb) / args.steps * 1e6 / LAYERS_PER_STEP)
    e2e_ok = bool(torch.isfinite(out_host.float()).all())

    extras = {}
    if rank == 0 and world == 1 and headline and not args.no_side:
        extras = side_measurements(torch, dev, sets, q, args, layer, ctx)
    if rank == 0:
        peak, which = measured_peak_gbs()
        achieved = algo_bytes / (iso_us * 1e-6) / 1e9
        if headline:
            metric, unit, value = "decode_attn_us_per_layer_64k_ctx", "us/layer", us_per_layer
            e2e_value = e2e_us
        else:
            metric, unit, value = "decode_attn_ms_per_32_layer_step_128k_ctx", "ms/step", ms_per_step
            e2e_value = e2e_us * LAYERS_PER_STEP / 1e3
        line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": warm + 2 + preload,
                "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": workload_text(ctx), "step": f"one decode step of a {LAYERS_PER_STEP}-layer model = {LAYERS_PER_STEP} attention layers; us/layer = step time / {LAYERS_PER_STEP}",
                           "l2": f"layers rotate over {N_SETS} KV sets ({comp_bytes * N_SETS / 1e6:.0f} MB compressed per rank) larger than L2",
                           "nsplit": nsplit, "tokens_per_rank": S_loc, "launch": launch_mode,
                           "launch_overlap": f"programmatic dependent launch, {LAYERS_PER_GRAPH} back-to-back attention layers per graph: a layer's CTAs become resident while the previous layer's split merge finishes",
                           "preload": f"{preload} identical untimed steps run right before the timed region inside the clock-sampling window",
                           "parallelism": "single GPU" if world == 1 else f"context split x{world}; {exchange_mode}"},
                "us_per_layer": us_per_layer, "us_per_layer_isolated": iso_us, "us_per_call_eager": per_call_us,
                "hbm_gbs_compressed": world * algo_bytes / (us_per_layer * 1e-6) / 1e9,
                "bf16_equiv_gbs": world * bf16_bytes / (us_per_layer * 1e-6) / 1e9,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES_64K * S_loc / 65536,
                             "peak_source": which, "algorithmic_bytes_per_launch": algo_bytes, "kernel_us": iso_us,
                             "kernel_us_is": "one layer of a 16-layer graph replayed with launch overlap switched off: each launch starts after its predecessor has finished entirely (N > 1: including the wait for the other ranks)",
                             "frac_pipelined": algo_bytes / (us_per_layer * 1e-6) / 1e9 / peak, "frac_of_8TBs_nominal": achieved / 8000.0},
                "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": q_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2,
                        "us_per_layer": e2e_us, "mode": e2e_mode, "results_finite": e2e_ok},
                "parity": parity,
                "gpu_launches": launches_per_layer * LAYERS_PER_STEP * args.steps, "clocks": clk.summary(c_from, c_to)}
        if peer is not None: line["config"]["exchange_wait_ran_out"] = peer.error()
        line.update(extras)
        print(json.dumps(line), flush=True)
    # release everything that holds kernels of the process group before it is torn down
    g_half = g_e2e = g_iso = None
    R.finish()


def side_measurements(torch, dev, sets, q, args, layer, ctx) -> dict:
    """Numbers reported beside the headline (outside its timed region): the CPU baseline on a bounded sample, the encoder's
    throughput, a library BF16-KV decode (flash-attn / SDPA) at the same shape under BOTH protocols used for our kernel, and the
    reference's own CUDA kernel on this GPU."""
    from gaac_b200 import Codec, TileEncoder
    from gaac_b200.synth import synth_kv
    out = {}
    threads = os.cpu_count() or 1
    try:
        cpu, kind, t_first = cpu_path_within(25.0, 4, threads, ctx)
        tb, vals = time.perf_counter(), []
        while time.perf_counter() - tb < max(10.0, 2.5 * t_first) and len(vals) < 50: vals.append(cpu.step_us_per_layer())
        out["cpu_baseline"] = {"value": sum(vals) / len(vals), "unit": "us/layer", "cores": threads, "kind": kind, "sample": cpu.sample + f", mean of {len(vals)} runs"}
        del cpu
    except Exception as e:
        out["cpu_baseline"] = {"value": None, "unit": "us/layer", "cores": threads, "kind": "port", "sample": f"failed: {e!r}"}
    # encoder: 8 x 65536 tokens per kind
    try:
        enc = {}
        for kind in "kv":
            x = synth_kv(kind, N_KV, ctx, seed=55, device=dev)
            codec = Codec(N_KV, dev).calibrate(x[:, :2048]); te = TileEncoder(kind, dev)
            xs = [x, x.clone(), x.clone()]
            for i in range(3): te.encode(codec, xs[i % 3])
            torch.cuda.synchronize(); ts = []
            for i in range(9):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); pg = te.encode(codec, xs[i % 3]); b.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(b))
            ms = sorted(ts)[len(ts) // 2]
            enc[kind] = {"ms": ms, "blocks_per_s": N_KV * (ctx // 16) / (ms * 1e-3), "gbs_in_plus_out": (x.numel() * 2 + pg.nbytes) / (ms * 1e-3) / 1e9, "ratio": pg.ratio}
            del x, xs
        out["encode"] = enc
    except Exception as e:                                   # side number only
        out["encode"] = {"error": repr(e)}
    # library BF16-KV decode at the same shape (context, not our kernel), timed exactly as our kernel is:
    #   per_call: event-bracketed single calls with a synchronise between (the reference's protocol, examples/attention.py:36-44)
    #   graph:    LAYERS_PER_GRAPH calls over the rotating KV sets captured in a CUDA graph, replayed, divided by the layers
    try:
        k = torch.randn(N_SETS, 1, ctx, N_KV, HEAD_DIM, device=dev).to(torch.bfloat16); v = torch.randn_like(k)
        qq = q.view(1, 1, N_Q, HEAD_DIM)
        try:
            from flash_attn import flash_attn_with_kvcache
            f = lambda i: flash_attn_with_kvcache(qq, k[i % N_SETS], v[i % N_SETS], softmax_scale=SCALE, causal=True); name = "flash_attn_with_kvcache"
            f(0)
        except Exception:
            import torch.nn.functional as F
            f = lambda i: F.scaled_dot_product_attention(qq.transpose(1, 2), k[i % N_SETS].transpose(1, 2), v[i % N_SETS].transpose(1, 2), scale=SCALE, enable_gqa=True); name = "sdpa"

        def per_call(fn, n=60):
            for i in range(10): fn(i)
            torch.cuda.synchronize(); ts = []
            for i in range(n):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); fn(i); b.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(b))
            return sorted(ts)[len(ts) // 2] * 1e3

        def graphed(fn, reps=40):
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                keep = [fn(i) for i in range(LAYERS_PER_GRAPH)]
            for _ in range(5): gr.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps): gr.replay()
            b.record(); torch.cuda.synchronize()
            return a.elapsed_time(b) * 1e3 / (reps * LAYERS_PER_GRAPH)
        lib = {"name": name, "us_per_call": per_call(f)}
        try: lib["us_graph_replay"] = graphed(f)
        except Exception as e: lib["us_graph_replay"] = None; lib["graph_error"] = repr(e)[:200]
        ours = {"us_per_call": per_call(lambda i: layer(i, q)), "us_graph_replay": graphed(lambda i: layer(i, q))}
        lib["us"] = lib["us_per_call"]
        out["bf16_kv_decode_library"] = lib
        out["vs_bf16_kv_decode_library"] = {"ours": ours, "speedup_per_call": lib["us_per_call"] / ours["us_per_call"],
                                            "speedup_graph_replay": (lib["us_graph_replay"] / ours["us_graph_replay"]) if lib.get("us_graph_replay") else None,
                                            "target": 1.3, "note": "like-for-like pairs only: both arms per call, or both arms replayed from a 16-layer CUDA graph"}
        del k, v
    except Exception as e:
        out["bf16_kv_decode_library"] = {"error": repr(e)}
    # the reference's own CUDA kernel and Triton encoder on this GPU (unmodified package under baseline/_ref, child process)
    out["reference_cuda_kernel"] = reference_kernel_side_number()
    return out


def reference_kernel_side_number() -> dict:
    script = os.path.join(ROOT, "baseline", "run_reference_kernel.py")
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "gaac")):
        return {"unavailable": "the reference package is not installed under baseline/_ref on this box"}
    try:
        r = subprocess.run([sys.executable, script], capture_output=True, text=True, timeout=300)
        lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
        if r.returncode != 0 or not lines:
            return {"unavailable": f"reference run failed (rc {r.returncode}): " + (r.stderr.strip().splitlines() or ["no output"])[-1][:300]}
        return json.loads(lines[-1])
    except subprocess.TimeoutExpired:
        return {"unavailable": "reference run did not finish in 300 s"}
    except Exception as e:
        return {"unavailable": repr(e)}


# ------------------------------------------------------------------------------------------------ paged batched decode, sharded by sequence
def run_paged16(args):
    """16 sequences with contexts uniform in [4096, 65536] (+ a 0..15-token filling block), 32 q / 8 kv heads, paged layout, block
    table = a seeded random permutation of the rank's share of a 2^20-block pool.  Sequences are sharded over the ranks by tokens
    (no collective on the path).  A step appends one token per sequence through the store (a block that fills is encoded) and
    runs paged attention; time = max over ranks."""
    import numpy as np
    import torch
    from gaac_b200 import Codec
    from gaac_b200.dist import shard_sequences
    from gaac_b200.kernel import choose_nsplit_sm100
    from gaac_b200.synth import synth_kv
    from gaac_b200.vllm.store import LayerState, OVF_OFF
    from gaac_b200.vllm.paged_kernel import paged_attention
    R = Ranks(args)
    dev, world, rank = R.dev, R.world, R.rank
    n_kv, G, B_all, ovf_slot = 8, 4, 16, 128
    n_q, TS = n_kv * G, OVF_OFF + ovf_slot
    rng = np.random.default_rng(0)
    lens_all = [int(l) // 16 * 16 + int(t) for l, t in zip(rng.integers(4096, 65537, B_all), rng.integers(0, 16, B_all))]
    shard_world, shard_rank = (int(x) for x in args.shard.split("/")[::-1]) if args.shard else (world, rank)
    mine = shard_sequences(lens_all, shard_world)[shard_rank]
    lens0 = [lens_all[i] for i in mine]
    B = len(lens0)
    warm = max(3, args.warmup)
    T_steps = warm + 2 * args.steps + 24                                        # steps of new tokens prepared up front
    pool_blocks = args.pool_blocks // world
    need_blocks = sum((L + T_steps + 15) // 16 for L in lens0)
    assert need_blocks <= pool_blocks, "pool too small for this rank's sequences"
    cal_k, cal_v = synth_kv("k", n_kv, 2048, 7, dev), synth_kv("v", n_kv, 2048, 7, dev)
    ck, cv = Codec(n_kv, dev).calibrate(cal_k), Codec(n_kv, dev).calibrate(cal_v)
    st = LayerState(pool_blocks, n_kv, raw_tiles=max(1, B) * 2 * n_kv + 4096, ovf_slot=ovf_slot, device=dev,
                    bases={"k3": ck.base3.cpu(), "k4": ck.base4.cpu(), "v3": cv.base3.cpu(), "v4": cv.base4.cpu()})
    buf = torch.zeros(pool_blocks * 2 * n_kv * TS, dtype=torch.uint8, device=dev)
    perm = np.random.default_rng(1000 + rank).permutation(pool_blocks).astype(np.int32)
    max_blocks = max([(L + T_steps + 15) // 16 for L in lens0] + [1])
    bt = np.zeros((max(B, 1), max_blocks), np.int32); used = 0
    new_k = torch.empty(T_steps, max(B, 1), n_kv, 128, dtype=torch.bfloat16, device=dev); new_v = torch.empty_like(new_k)
    for i, L in enumerate(lens0):
        nb_all = (L + T_steps + 15) // 16
        bt[i, :nb_all] = perm[used:used + nb_all]; used += nb_all
        kk = synth_kv("k", n_kv, L + T_steps, 7, dev).transpose(0, 1).contiguous(); vv = synth_kv("v", n_kv, L + T_steps, 7, dev).transpose(0, 1).contiguous()
        nb = (L + 15) // 16
        ent = np.array([[bt[i, t], t * 16, 0, min(16, L - t * 16)] for t in range(nb)], np.int32)
        st.store(kk, vv, buf, torch.from_numpy(ent).to(dev), torch.empty(nb * 2 * n_kv, dtype=torch.int32, device=dev))     # the prompt, through the store
        new_k[:, i] = kk[L:L + T_steps]; new_v[:, i] = vv[L:L + T_steps]
        del kk, vv
    btd = torch.from_numpy(bt).to(dev)
    ent_all = np.zeros((T_steps, max(B, 1), 4), np.int32); sl_all = np.zeros((T_steps, max(B, 1)), np.int32)
    for s in range(T_steps):
        for i, L in enumerate(lens0):
            cur = L + s
            ent_all[s, i] = (bt[i, cur // 16], i, cur % 16, 1); sl_all[s, i] = cur + 1
    ent_d, sl_d = torch.from_numpy(ent_all).to(dev), torch.from_numpy(sl_all).to(dev)
    freeq = torch.empty(max(B, 1) * 2 * n_kv, dtype=torch.int32, device=dev)
    q = torch.randn(max(B, 1), n_q, 128, device=dev).to(torch.bfloat16)
    out = torch.empty(max(B, 1), n_q * 128, dtype=torch.bfloat16, device=dev)
    ns = args.nsplit or choose_nsplit_sm100(max(B, 1), n_kv, max(lens0 + [16]), ragged=True, total_tokens=sum(lens0))

    def attend(s):
        paged_attention(q, out, buf, st.raw, st.mt, btd, sl_d[s], st.bases, TS, n_q, n_kv, ns)

    def step(s):
        if B == 0: return
        st.store(new_k[s], new_v[s], buf, ent_d[s], freeq)
        attend(s)

    def algo_bytes_at(s) -> float:
        """Algorithmic bytes of the attention launch of step s: slot payload + the escape bytes in use per compressed tile, 256 B
        per row of the filling block, 4 B per mode-table entry and per block-table entry, q and out."""
        if B == 0: return 0.0
        lens = [L + s + 1 for L in lens0]
        full, part_rows = sum(L // 16 for L in lens), sum(L % 16 for L in lens)
        blocks = sum((L + 15) // 16 for L in lens)
        return full * 2 * n_kv * (2880 + esc_mean) + part_rows * 2 * n_kv * 256 + blocks * (2 * n_kv * 4 + 4) + 2 * B * n_q * 128 * 2
    # mean escape bytes per compressed tile, from the tag words of a sample of this rank's tiles
    esc_mean = 0.0
    if B:
        ids = torch.from_numpy(bt[0, :min(lens0[0] // 16, 2048)].astype(np.int64)).to(dev)
        slots_ = (ids[:, None] * (2 * n_kv) + torch.arange(2 * n_kv, device=dev)[None, :]).reshape(-1)
        fl = buf.view(-1, TS)[slots_, 2816:2880].contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        pc = lambda x: sum(((x >> b) & 1) for b in range(32))
        esc_mean = float((pc(fl & 0x55555555) + 4 * pc(fl & 0xAAAAAAAA)).sum() / slots_.numel())

    s = 0
    for _ in range(warm): step(s); s += 1
    R.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(R.local) as clk:
        R.barrier(); c_from = time.perf_counter()
        preload = 0 if args.profile else keep_busy(lambda: attend(s - 1) if B else None, R)     # the attention launch of the last step, repeated
        t0.record()
        s_first = s
        for _ in range(args.steps): step(s); s += 1
        t1.record()
        R.barrier(); c_to = time.perf_counter()
    ms_per_step = R.max_over_ranks(t0.elapsed_time(t1) / args.steps)
    if args.profile:                                            # the command to run under ncu: warm-up and timed steps, nothing else
        if rank == 0: print(json.dumps({"profile_run": True, "workload": "paged16", "us_per_step": ms_per_step * 1e3, "nsplit": ns}), flush=True)
        R.finish()
        return
    # the attention launch alone (events around it), and the store alone
    ka, ks_ = [], []
    for _ in range(20):
        if B == 0: break
        a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        a.record(); st.store(new_k[s], new_v[s], buf, ent_d[s], freeq); b.record(); attend(s); c.record(); torch.cuda.synchronize()
        ks_.append(a.elapsed_time(b) * 1e3); ka.append(b.elapsed_time(c) * 1e3); s += 1
    attn_us = sorted(ka)[len(ka) // 2] if ka else 0.0
    store_us = sorted(ks_)[len(ks_) // 2] if ks_ else 0.0
    # end to end: this step's new K/V rows, entries, lengths and queries from pinned host memory, the outputs back
    hk, hv = new_k[s:s + args.steps].cpu().pin_memory(), new_v[s:s + args.steps].cpu().pin_memory()
    he, hs_, hq = ent_d[s:s + args.steps].cpu().pin_memory(), sl_d[s:s + args.steps].cpu().pin_memory(), q.cpu().pin_memory()
    ho = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    dk, dv, de, ds, dq = torch.empty_like(new_k[0]), torch.empty_like(new_v[0]), torch.empty_like(ent_d[0]), torch.empty_like(sl_d[0]), torch.empty_like(q)
    def e2e_step(i):
        dk.copy_(hk[i], non_blocking=True); dv.copy_(hv[i], non_blocking=True); de.copy_(he[i], non_blocking=True); ds.copy_(hs_[i], non_blocking=True); dq.copy_(hq, non_blocking=True)
        if B:
            st.store(dk, dv, buf, de, freeq)
            paged_attention(dq, out, buf, st.raw, st.mt, btd, ds, st.bases, TS, n_q, n_kv, ns)
        ho.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
    R.barrier()
    tb = time.perf_counter()
    for i in range(args.steps): e2e_step(i)
    R.barrier()
    e2e_us = R.max_over_ranks((time.perf_counter() - tb) / args.steps * 1e6)
    err_count = int(st.err)
    tokens_all = sum(lens_all)
    nbytes = algo_bytes_at(s_first + args.steps // 2)
    tot_bytes = R.max_over_ranks(0.0)                                            # keeps the ranks in step; the sum comes below
    if R.dist:
        t = torch.tensor([nbytes], dtype=torch.float64, device=dev); R.dist.all_reduce(t); tot_bytes = float(t)
    else:
        tot_bytes = nbytes
    if rank == 0:
        peak, which = measured_peak_gbs()
        achieved = nbytes / max(attn_us, 1e-9) / 1e3
        line = {"metric": "paged_decode_step_us_16_seqs", "value": ms_per_step * 1e3, "unit": "us/step", "n_gpus": world, "steps": args.steps, "warmup": warm,
                "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"paged batched decode: {B_all} sequences, contexts 4096..65536 (+0..15 filling tokens, {tokens_all} tokens in all), {n_q} q / {n_kv} kv heads, head_dim 128, "
                                       f"16-token blocks, block table = random permutation of a {args.pool_blocks}-block pool; step = store of one token per sequence (blocks that fill are encoded) + paged attention, one layer",
                           "l2": f"rank 0 streams {nbytes / 1e6:.0f} MB of compressed tiles per step, larger than L2", "nsplit": ns,
                           "parallelism": "single GPU" if world == 1 else f"sequences sharded over {world} GPUs by tokens, no collective on the path", "sequences_rank0": B, "launch": "eager",
                           "preload": f"{preload} untimed attention launches right before the timed region, inside the clock-sampling window"},
                "attention_us_rank0": attn_us, "store_us_rank0": store_us, "raw_pool_errors": err_count,
                "hbm_gbs_compressed": tot_bytes / (ms_per_step * 1e-3) / 1e9,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None, "peak_source": which,
                             "algorithmic_bytes_per_launch": nbytes, "kernel_us": attn_us, "kernel": "decode_attn_kernel<paged> of rank 0, events around the launch"},
                "e2e": {"value": e2e_us, "unit": "us/step", "h2d_bytes_per_step": int(hk[0].numel() * 2 * 2 + he[0].numel() * 4 + hs_[0].numel() * 4 + hq.numel() * 2), "d2h_bytes_per_step": int(ho.numel() * 2)},
                "gpu_launches": 3 * args.steps, "clocks": clk.summary(c_from, c_to)}
        print(json.dumps(line), flush=True)
    R.finish()


# ------------------------------------------------------------------------------------------------ large batch, kv heads sharded
def run_batch64(args):
    """64 sequences x 32768 tokens, 64 q / 8 kv heads (GQA 8), kv heads sharded over the ranks (no collective on the attention
    path).  Decode step of one layer = CompressedKVCache.append + attention, alternating between two layer caches so that every
    step streams from HBM.  Prefill-encode: `prefill_layers` layers x 64 sequences through CompressedKVCache.prefill (the call an
    engine makes, one sequence at a time), and the encoder's own rate on a whole layer's [64*n_kv, 32768, 128] tensor."""
    import torch
    from gaac_b200 import Codec, CompressedKVCache, TileEncoder
    from gaac_b200.dist import shard_heads
    from gaac_b200.synth import synth_kv
    R = Ranks(args)
    dev, world, rank = R.dev, R.world, R.rank
    B, S, G, n_kv_all, n_layers_model = 64, 32768, 8, 8, 64
    heads = shard_heads(n_kv_all, world, rank)
    n_kv = len(heads)
    n_q = n_kv * G
    warm = max(3, args.warmup)
    assert n_kv >= 1, "more ranks than kv heads"
    # four distinct sequences' K/V of this rank's heads, token-major as a model produces them
    seqs = []
    for i in range(4):
        k = synth_kv("k", n_kv_all, S, 300 + i, dev)[heads.start:heads.stop].transpose(0, 1).contiguous()
        v = synth_kv("v", n_kv_all, S, 300 + i, dev)[heads.start:heads.stop].transpose(0, 1).contiguous()
        seqs.append((k, v))
    ck = Codec(n_kv, dev).calibrate(seqs[0][0][:2048].transpose(0, 1)); cv = Codec(n_kv, dev).calibrate(seqs[0][1][:2048].transpose(0, 1))
    bases = {"k3": ck.base3, "k4": ck.base4, "v3": cv.base3, "v4": cv.base4}
    caches = [CompressedKVCache(n_slots=B, n_kv=n_kv, capacity=S + 1024, bases=bases, device=dev) for _ in range(2)]
    # ---- prefill-encode pass through the cache API
    def prefill_layer(cache, check=False):
        for slot in range(B):
            cache.prefill(slot, *seqs[slot % 4], check=check)
        cache.settle_prefills()
    prefill_layer(caches[0]); prefill_layer(caches[1])                           # warm-up; both caches end up full
    torch.cuda.synchronize()
    def time_prefill(check):
        R.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tb = time.perf_counter()
        a.record()
        for l in range(args.prefill_layers): prefill_layer(caches[l % 2], check)
        b.record(); torch.cuda.synchronize()
        return R.max_over_ranks(a.elapsed_time(b)), time.perf_counter() - tb
    prefill_checked_ms, _ = time_prefill(True)
    prefill_ms, prefill_wall = time_prefill(False)
    stats = caches[0].stats()
    in_bytes = B * S * n_kv * 128 * 2 * 2                                        # K and V, one layer, this rank
    out_bytes = stats["bytes_used"]
    tiles_layer = B * n_kv * (S // 16) * 2
    # ---- the encoder alone on a whole layer of this rank: [64 * n_kv, 32768, 128] per kind in one call
    enc = {}
    for kind, codec in (("k", ck), ("v", cv)):
        x = torch.stack([seqs[i % 4][0 if kind == "k" else 1] for i in range(B)], 0).permute(0, 2, 1, 3).reshape(B * n_kv, S, 128).contiguous()
        te = TileEncoder(kind, dev)
        for _ in range(2): pg = te.encode(codec, x)
        torch.cuda.synchronize(); ts = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); pg = te.encode(codec, x); e1.record(); torch.cuda.synchronize(); ts.append(e0.elapsed_time(e1))
        ms = sorted(ts)[len(ts) // 2]
        enc[kind] = {"ms": ms, "gbs_in_plus_out": (x.numel() * 2 + pg.nbytes) / (ms * 1e-3) / 1e9, "blocks_per_s": B * n_kv * (S // 16) / (ms * 1e-3), "ratio": pg.ratio}
        del x, pg
    # ---- decode step
    slots = torch.arange(B, dtype=torch.int32, device=dev)
    q = torch.randn(B, n_q, 128, device=dev).to(torch.bfloat16)
    k1 = seqs[1][0][:B].contiguous(); v1 = seqs[1][1][:B].contiguous()            # [B, n_kv, 128]: one new token per sequence
    def step(i):
        c = caches[i % 2]
        c.append(slots, k1, v1)
        return c.attention(q, slots, 128 ** -0.5, max_len=S + 64)
    for i in range(warm): step(i)
    R.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(R.local) as clk:
        R.barrier(); c_from = time.perf_counter()
        flip = [0]
        def attend_only():
            flip[0] ^= 1
            caches[flip[0]].attention(q, slots, 128 ** -0.5, max_len=S + 64)
        preload = keep_busy(attend_only, R)
        t0.record()
        for i in range(args.steps): step(i)
        t1.record()
        R.barrier(); c_to = time.perf_counter()
    ms_per_step = R.max_over_ranks(t0.elapsed_time(t1) / args.steps)
    ka = []
    for i in range(20):
        c = caches[i % 2]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); c.attention(q, slots, 128 ** -0.5, max_len=S + 64); e1.record(); torch.cuda.synchronize(); ka.append(e0.elapsed_time(e1) * 1e3)
    attn_us = R.max_over_ranks(sorted(ka)[len(ka) // 2])
    st_now = caches[0].stats()
    nbytes = st_now["bytes_used"] + 2 * B * n_q * 128 * 2
    # end to end: the new token's K/V and the queries from pinned host memory, the outputs back
    hk, hv, hq = k1.cpu().pin_memory(), v1.cpu().pin_memory(), q.cpu().pin_memory()
    ho = torch.empty(B, n_q, 128, dtype=torch.bfloat16).pin_memory()
    dk, dv, dq = torch.empty_like(k1), torch.empty_like(v1), torch.empty_like(q)
    def e2e_step(i):
        dk.copy_(hk, non_blocking=True); dv.copy_(hv, non_blocking=True); dq.copy_(hq, non_blocking=True)
        c = caches[i % 2]
        c.append(slots, dk, dv)
        ho.copy_(c.attention(dq, slots, 128 ** -0.5, max_len=S + 64), non_blocking=True)
        torch.cuda.synchronize()
    n_e2e = min(args.steps, 200)
    R.barrier()
    tb = time.perf_counter()
    for i in range(n_e2e): e2e_step(i)
    R.barrier()
    e2e_us = R.max_over_ranks((time.perf_counter() - tb) / n_e2e * 1e6)
    app_err = int(caches[0].append_errors) + int(caches[1].append_errors)
    if rank == 0:
        peak, which = measured_peak_gbs()
        achieved = nbytes / attn_us / 1e3
        line = {"metric": "decode_step_us_per_layer_batch64_32k_ctx", "value": ms_per_step * 1e3, "unit": "us/layer", "n_gpus": world, "steps": args.steps, "warmup": warm,
                "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"large-batch decode: {B} sequences x {S}-token contexts, {n_kv_all * G} q / {n_kv_all} kv heads (GQA {G}), head_dim 128, slot layout; step = append one token per sequence + attention, one layer",
                           "l2": f"steps alternate between two layer caches of {st_now['bytes_used'] / 1e9:.2f} GB each", "kv_heads_rank0": n_kv,
                           "parallelism": "single GPU" if world == 1 else f"kv heads sharded over {world} GPUs ({n_kv} per GPU), no collective on the attention path", "launch": "eager",
                           "preload": f"{preload} untimed attention launches right before the timed region, inside the clock-sampling window"},
                "attention_us": attn_us, "append_errors": app_err,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None, "peak_source": which,
                             "algorithmic_bytes_per_launch": nbytes, "kernel_us": attn_us, "kernel": "decode_attn_kernel<slot>, events around the launch, max over ranks"},
                "prefill_encode": {"layers_timed": args.prefill_layers, "ms_per_layer": prefill_ms / args.prefill_layers,
                                   "ms_for_64_layers_scaled": prefill_ms / args.prefill_layers * n_layers_model, "scale_factor": n_layers_model / args.prefill_layers,
                                   "gbs_in_plus_out": (in_bytes + out_bytes) * args.prefill_layers / (prefill_ms * 1e-3) / 1e9,
                                   "blocks_per_s": tiles_layer * args.prefill_layers / (prefill_ms * 1e-3), "host_wall_ms_per_layer": prefill_wall * 1e3 / args.prefill_layers,
                                   "how": "CompressedKVCache.prefill(check=False), one library call per sequence and layer (64 per layer), their status words read together by settle_prefills (forced after 1 GiB of kept escape slots, i.e. every 24 prompts); per rank",
                                   "ms_per_layer_host_check_per_prompt": prefill_checked_ms / args.prefill_layers},
                "encode_whole_layer": enc,
                "e2e": {"value": e2e_us, "unit": "us/layer", "h2d_bytes_per_step": int(hk.numel() * 2 * 2 + hq.numel() * 2), "d2h_bytes_per_step": int(ho.numel() * 2)},
                "gpu_launches": 2 * args.steps, "clocks": clk.summary(c_from, c_to)}
        print(json.dumps(line), flush=True)
    R.finish()


def run_encode_only(args):
    import torch
    from gaac_b200 import Codec, TileEncoder
    from gaac_b200.synth import synth_kv
    dev = torch.device("cuda", 0)
    out = {}
    for kind in "kv":
        x = synth_kv(kind, N_KV, 65536, seed=55, device=dev)
        codec = Codec(N_KV, dev).calibrate(x[:, :2048]); te = TileEncoder(kind, dev)
        for _ in range(max(1, args.warmup)): te.encode(codec, x)
        torch.cuda.synchronize(); ts = []
        for _ in range(args.steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); pg = te.encode(codec, x); b.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(b))
        out[kind] = {"encode_ms_median": sorted(ts)[len(ts) // 2], "tiles": N_KV * (65536 // 16), "ratio": pg.ratio}
    print(json.dumps({"profile_encode": out}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40, help="timed steps (ctx64k / ctx128k: one step = 32 attention layers)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="ctx64k", choices=["ctx64k", "ctx128k", "paged16", "batch64"],
                    help="ctx64k = the headline line; the others print one line for their workload")
    ap.add_argument("--nccl-exchange", action="store_true", help="N > 1: exchange the partials with an NCCL all-gather instead of peer-memory stores")
    ap.add_argument("--two-kernel-exchange", action="store_true", help="N > 1: push-only attention launch + separate wait-and-merge kernel instead of the fused launch")
    ap.add_argument("--no-graph", action="store_true", help="launch every layer eagerly instead of replaying CUDA graphs")
    ap.add_argument("--no-side", action="store_true", help="skip the side measurements (CPU baseline, encoder, library decode, reference kernel)")
    ap.add_argument("--profile", action="store_true", help="ctx64k / ctx128k / paged16: only the warm-up and --steps eager steps (no graphs, no preload, no e2e, no side measurements): the command to run under ncu")
    ap.add_argument("--profile-encode", action="store_true", help="only the block encoder on [8, 65536, 128] K and V, --steps times each: the command to run under ncu")
    ap.add_argument("--nsplit", type=int, default=0, help="paged16: split count instead of the heuristic's")
    ap.add_argument("--shard", default="", help="paged16, single process: run the sequences rank r of n ranks would get, as 'r/n'")
    ap.add_argument("--pool-blocks", type=int, default=1 << 20, help="paged16: blocks of the paged pool over all ranks (3008 B x 16 tile slots each)")
    ap.add_argument("--prefill-layers", type=int, default=8, help="batch64: layers of the prefill-encode pass that are timed (scaled to 64)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.profile_encode:
        run_encode_only(args)
    elif args.workload == "paged16":
        run_paged16(args)
    elif args.workload == "batch64":
        run_batch64(args)
    else:
        run_context(args, 131072 if args.workload == "ctx128k" else 65536)


if __name__ == "__main__":
    main()
