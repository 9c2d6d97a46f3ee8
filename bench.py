"""Benchmark of the GAAC hot path on B200: fused decode attention over the compressed KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Workload (synthetic, see gaac_b200/synth.py): one decode-attention layer, batch 1, 32 query heads / 8 KV heads (GQA 4),
head_dim 128, 65536-token context, KV fully encoded into the slot layout with a 0-token tail; softmax scale 1/sqrt(128).
A step = one layer call.  Steps rotate over several independent KV sets whose total size exceeds the L2 cache, so every
step streams its compressed bytes from HBM.  With N > 1 GPUs the context is split into N contiguous token ranges, each rank
attends over its range and the per-rank partials (m, l, acc) are all-gathered over NCCL and merged (strong scaling).

One JSON line on stdout (rank 0).  `value` is microseconds per layer, device-timed, inputs resident in HBM; `e2e` is the same
call fed from pinned host memory with the result read back to the host every step.
"""
from __future__ import annotations
import argparse, json, os, subprocess, sys, threading, time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_Q, N_KV, HEAD_DIM, CTX = 32, 8, 128, 65536
N_SETS = 4                       # independent KV sets rotated over ("layers"): 4 x ~193 MB compressed > 126 MB of L2
SCALE = HEAD_DIM ** -0.5
WORKLOAD = "decode attention, batch 1, 32 q heads / 8 kv heads (GQA 4), head_dim 128, 65536-token context, slot layout, 0-token tail"
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_attn_kernel launch at this workload, from the ncu capture
# summarised in profiles/; None until a capture exists.
NCU_TRAFFIC_BYTES = 196.7e6
LAYERS_PER_GRAPH = 16              # layers captured in one CUDA graph of the timed region (a 32-layer model replays two of them per step)


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True); self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try: self.proc.wait(timeout=5)
            except Exception: pass

    def summary(self) -> dict:
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(mhz)}


def page_bytes(pg) -> int:
    return pg.nbytes


# ------------------------------------------------------------------------------------------------ reference arm (CPU)
class CpuPath:
    """The reference's CPU path for this workload - decode the compressed cache (gaac/codec.py:186-218) and run softmax
    attention on the decoded KV - restated in numpy (oracle/), run on a bounded sample and scaled to the full layer."""

    def __init__(self, sample_heads: int, sample_tokens: int, threads: int):
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
        self.frac = (sample_heads * sample_tokens) / (N_KV * CTX)
        self.sample = f"{sample_heads} of {N_KV} kv heads x {sample_tokens} of {CTX} tokens (codec decode + softmax attention), time scaled by {1 / self.frac:.0f}"

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
    (the comparison of examples/attention.py:27-32 on the host), all host threads, on a bounded sample scaled to the layer."""

    def __init__(self, sample_heads: int, sample_tokens: int, threads: int):
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
        self.frac = (sample_heads * sample_tokens) / (N_KV * CTX)
        self.sample = (f"{sample_heads} of {N_KV} kv heads x {sample_tokens} of {CTX} tokens (reference Codec.decode on CPU + torch SDPA), "
                       f"time scaled by {1 / self.frac:.0f}")

    def step_us_per_layer(self) -> float:
        torch, F = self.torch, self.torch.nn.functional
        t = time.perf_counter()
        k = self.ref.Codec.decode(self.kp); v = self.ref.Codec.decode(self.vp)                   # [H, S, 128] bf16
        F.scaled_dot_product_attention(self.q, k.unsqueeze(0), v.unsqueeze(0), scale=SCALE, enable_gqa=True)
        return (time.perf_counter() - t) / self.frac * 1e6


def make_cpu_path(sample_heads: int, sample_tokens: int, threads: int):
    """(path, kind): the reference's own CPU code when its package travelled with the repository, else the oracle's restatement."""
    try:
        return RefCpuPath(sample_heads, sample_tokens, threads), "reference"
    except Exception as e:
        print(f"reference CPU path unavailable ({type(e).__name__}: {e}); timing the oracle port", file=sys.stderr, flush=True)
        return CpuPath(sample_heads, sample_tokens, threads), "port"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    cpu, kind = make_cpu_path(1, 16384, threads)
    t_first = time.perf_counter(); cpu.step_us_per_layer(); t_first = time.perf_counter() - t_first
    if t_first * (args.steps + args.warmup) > 150.0:          # keep the whole run within a few minutes
        cpu, kind = make_cpu_path(1, 4096, threads)
    for _ in range(args.warmup): cpu.step_us_per_layer()
    vals = [cpu.step_us_per_layer() for _ in range(args.steps)]
    us = sum(vals) / len(vals)
    line = {"impl": "reference", "metric": "decode_attn_us_per_layer_64k_ctx", "value": us, "unit": "us/layer", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if kind == "reference" else "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "path": ("CPU: the unmodified reference package (baseline/_ref): Codec.decode + torch scaled_dot_product_attention" if kind == "reference"
                                                     else "CPU: numpy restatement (oracle/) of the reference codec decode + softmax attention")},
            "cpu_baseline": {"value": us, "unit": "us/layer", "cores": threads, "kind": kind, "sample": cpu.sample},
            "e2e": {"value": us, "unit": "us/layer", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ our arm (GPU)
def run_ours(args):
    import torch
    import torch.distributed as dist
    from gaac_b200 import Codec, TileEncoder, _lib
    from gaac_b200.kernel import _ext, choose_nsplit_sm100, combine_parts, workspace
    from gaac_b200.synth import synth_kv
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0")); local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE {world}: launch with torch.distributed.run"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))     # fail fast instead of hanging
    _lib.lib()

    # ---- this rank's share of the context: contiguous, tile aligned
    tiles = CTX // 16
    t_lo, t_hi = tiles * rank // world, tiles * (rank + 1) // world
    S_loc = (t_hi - t_lo) * 16
    sets = []
    for i in range(N_SETS):
        k = synth_kv("k", N_KV, CTX, seed=100 + i, device=dev); v = synth_kv("v", N_KV, CTX, seed=100 + i, device=dev)
        ck, cv = Codec(N_KV, dev).calibrate(k[:, :2048]), Codec(N_KV, dev).calibrate(v[:, :2048])
        kp = TileEncoder("k", dev).encode(ck, k[:, t_lo * 16:t_hi * 16].contiguous()); vp = TileEncoder("v", dev).encode(cv, v[:, t_lo * 16:t_hi * 16].contiguous())
        sets.append((kp, vp))
        del k, v
    comp_bytes = sum(page_bytes(kp) + page_bytes(vp) for kp, vp in sets) / N_SETS
    algo_bytes = comp_bytes + 2 * N_Q * HEAD_DIM * 2                                   # + q + out (bf16)
    bf16_bytes = 2 * N_KV * S_loc * HEAD_DIM * 2
    nsplit = choose_nsplit_sm100(1, N_KV, S_loc)
    g = torch.Generator(device=dev).manual_seed(7)
    q = torch.randn(1, N_Q, HEAD_DIM, generator=g, device=dev).to(torch.bfloat16)
    slots = torch.zeros(1, dtype=torch.int32, device=dev)
    SL = torch.full((N_KV,), S_loc, dtype=torch.int32, device=dev)
    e32 = torch.empty(0, dtype=torch.int32, device=dev); ebf = torch.empty(0, dtype=torch.bfloat16, device=dev)
    part = torch.empty(N_Q, 130, dtype=torch.float32, device=dev)
    gathered = torch.empty(world * N_Q, 130, dtype=torch.float32, device=dev)
    ext = _ext()
    # N > 1: the partials travel by plain stores from the attention kernel's epilogue into every rank's receive buffer
    # (peer memory); NCCL all-gather + merge kernel is the fallback when the peer mapping cannot be set up on every rank.
    peer, exchange_mode = None, "none"
    if world > 1:
        exchange_mode = "nccl all-gather + merge kernel"
        ok = 0
        if not args.nccl_exchange:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")          # plain peer loads/stores only
            try:
                from gaac_b200.dist import PeerExchange
                peer = PeerExchange(N_Q, dev); ok = 1
            except Exception as e:
                print(f"[rank {rank}] peer exchange unavailable: {type(e).__name__}: {e}", file=sys.stderr, flush=True)
        okt = torch.tensor([ok], dtype=torch.int32, device=dev); dist.all_reduce(okt, op=dist.ReduceOp.MIN)
        if int(okt) == 1:
            exchange_mode = "partials pushed into peer memory by the attention kernel (NVLink stores) + wait-and-merge kernel"
        else:
            peer = None

    def layer(i, qq):
        kp, vp = sets[i % N_SETS]
        common = (kp.sm, kp.codes, kp.flags, kp.tile_off, kp.ovf, kp.ovf_head_start, kp.base3, kp.base4,
                  vp.sm, vp.codes, vp.flags, vp.tile_off, vp.ovf, vp.ovf_head_start, vp.base3, vp.base4,
                  qq.view(N_Q, HEAD_DIM), slots, N_Q, N_KV, SL, S_loc, SCALE, nsplit, ebf, ebf, e32, 0)
        if world == 1:
            return ext.gaac_attn_launch(*common)
        if peer is not None:
            ext.gaac_attn_launch(*common, exchange=peer.x)
            return peer.merge(N_KV)
        ext.gaac_attn_launch(*common, partial=part)
        dist.all_gather_into_tensor(gathered, part)
        return combine_parts(gathered.view(world, N_Q, 130))

    launches_per_step = 1 if world == 1 else 2       # ours: attention (+ the merge of the gathered partials); NCCL's kernel not counted

    def barrier():
        if world > 1: dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(3, args.warmup)):
        layer(i, q)
    barrier()
    # CUDA graphs: the launch path of a decode loop, which the reference's serving engine also captures.  One graph holds
    # LAYERS_PER_GRAPH consecutive layers, as a decode step of a model does (the kernels carry programmatic-dependent-launch edges,
    # so a layer's CTAs become resident while the previous layer's split merge is finishing); single-layer graphs cover the
    # remainder of steps / LAYERS_PER_GRAPH.
    graphs, g_all, g_four, launch_mode = None, None, None, "eager"
    if not (args.profile or args.no_graph):
        try:
            graphs = []
            for i in range(N_SETS):
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_):
                    o_ = layer(i, q)
                graphs.append((g_, o_))
            g_all = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_all):
                o_all = [layer(i, q) for i in range(LAYERS_PER_GRAPH)]
            g_four = torch.cuda.CUDAGraph()                                              # for the remainder of steps / LAYERS_PER_GRAPH
            with torch.cuda.graph(g_four):
                o_four = [layer(i, q) for i in range(4)]
            launch_mode = f"cuda graph replay, {LAYERS_PER_GRAPH} layers per graph"
        except Exception as e:                                                          # capture unsupported: same on every rank
            graphs = g_all = g_four = None; launch_mode = f"eager (graph capture failed: {type(e).__name__})"
        barrier()

    def run_steps(n, events=None):
        """Exactly n layer steps."""
        if graphs is None:
            for i in range(n):
                if events: events[i][0].record()
                layer(i, q)
                if events: events[i][1].record()
            return
        for _ in range(n // LAYERS_PER_GRAPH): g_all.replay()
        n %= LAYERS_PER_GRAPH
        for _ in range(n // 4): g_four.replay()
        for i in range(n % 4): graphs[i % N_SETS][0].replay()
    run_steps(2 * LAYERS_PER_GRAPH + 1)
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)] if graphs is None else None
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        t0.record()
        run_steps(args.steps, ev)
        t1.record()
        barrier()
        # keep the GPU busy a little longer so the 100 ms sampler sees the loaded clocks (the same number of calls on every
        # rank: the calls contain an exchange when N > 1)
        if not args.profile: run_steps(4000)
        torch.cuda.synchronize()
    total_ms = t0.elapsed_time(t1)
    kern_ms = sorted(a.elapsed_time(b) for a, b in ev) if ev else [total_ms / args.steps]   # graph mode: device time per layer of the replayed region
    if world > 1:
        tt = torch.tensor([total_ms], dtype=torch.float64, device=dev); dist.all_reduce(tt, op=dist.ReduceOp.MAX); total_ms = float(tt)
    us_per_layer = total_ms / args.steps * 1e3
    kern_us = sum(kern_ms) / len(kern_ms) * 1e3                                         # mean event-bracketed call duration

    def finish():
        # N > 1: leave without tearing NCCL down.  Destroying the process group while captured graphs still hold its
        # kernels blocked for minutes here; every rank has printed and synchronised, so a plain process exit is clean.
        sys.stdout.flush(); sys.stderr.flush()
        if world > 1:
            barrier()
            os._exit(0)

    if args.profile:
        if rank == 0: print(json.dumps({"profile_run": True, "us_per_layer": us_per_layer, "kernel_us": kern_us, "nsplit": nsplit}), flush=True)
        finish()
        return
    # ---- end to end: q from pinned host memory, result back on the host, every step
    q_host = q.cpu().pin_memory(); out_host = torch.empty(1, N_Q, HEAD_DIM, dtype=torch.bfloat16).pin_memory()
    q_dev = torch.empty_like(q)
    from gaac_b200 import attention as public_attention
    def e2e_step(i):
        q_dev.copy_(q_host, non_blocking=True)
        out = layer(i, q_dev) if world > 1 else public_attention(q_dev, *sets[i % N_SETS], scale=SCALE, nsplit=nsplit)     # the call a user makes
        out_host.copy_(out.view(1, N_Q, HEAD_DIM), non_blocking=True)
        torch.cuda.synchronize()
    for i in range(3): e2e_step(i)
    # the same step as one CUDA graph per KV set (copy in, attention through the public call, copy out), replayed and synchronised
    # every step: how a serving loop issues a decode step; falls back to the eager step when capture is not possible
    if world == 1 and not args.no_graph:
        try:
            torch.cuda.synchronize()
            e2e_graphs = []
            for i in range(N_SETS):
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_):
                    q_dev.copy_(q_host, non_blocking=True)
                    o_ = public_attention(q_dev, *sets[i], scale=SCALE, nsplit=nsplit)
                    out_host.copy_(o_.view(1, N_Q, HEAD_DIM), non_blocking=True)
                e2e_graphs.append((g_, o_))
            def e2e_step(i):
                e2e_graphs[i % N_SETS][0].replay()
                torch.cuda.synchronize()
            for i in range(3): e2e_step(i)
        except Exception as e:
            print(f"e2e graph capture failed ({type(e).__name__}); timing the eager step", file=sys.stderr, flush=True)
    barrier()
    tb = time.perf_counter()
    for i in range(args.steps): e2e_step(i)
    barrier()
    e2e_us = (time.perf_counter() - tb) / args.steps * 1e6
    if world > 1:
        tt = torch.tensor([e2e_us], dtype=torch.float64, device=dev); dist.all_reduce(tt, op=dist.ReduceOp.MAX); e2e_us = float(tt)

    extras = {}
    if rank == 0 and world == 1:
        extras = side_measurements(torch, dev, sets, q, args)
    if rank == 0:
        peak, which = measured_peak_gbs()
        achieved = algo_bytes / (kern_us * 1e-6) / 1e9
        line = {"metric": "decode_attn_us_per_layer_64k_ctx", "value": us_per_layer, "unit": "us/layer", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
                "ms_per_step": us_per_layer / 1e3, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": WORKLOAD, "l2": f"steps rotate over {N_SETS} KV sets ({comp_bytes * N_SETS / 1e6:.0f} MB compressed per rank) larger than L2",
                           "nsplit": nsplit, "tokens_per_rank": S_loc, "launch": launch_mode, "parallelism": "single GPU" if world == 1 else f"context split x{world}; {exchange_mode}"},
                "hbm_gbs_compressed": achieved * (kern_us / us_per_layer) if world == 1 else world * algo_bytes / (us_per_layer * 1e-6) / 1e9,
                "bf16_equiv_gbs": world * bf16_bytes / (us_per_layer * 1e-6) / 1e9,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES * S_loc / CTX,
                             "peak_source": which, "algorithmic_bytes_per_launch": algo_bytes, "kernel_us": kern_us, "frac_of_8TBs_nominal": achieved / 8000.0},
                "e2e": {"value": e2e_us, "unit": "us/layer", "h2d_bytes_per_step": q_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2},
                "gpu_launches": launches_per_step * args.steps, "clocks": clk.summary()}
        if peer is not None: line["config"]["exchange_wait_ran_out"] = peer.error()
        line.update(extras)
        print(json.dumps(line), flush=True)
    finish()


def run_encode_only(args):
    import torch
    from gaac_b200 import Codec, TileEncoder
    from gaac_b200.synth import synth_kv
    dev = torch.device("cuda", 0)
    out = {}
    for kind in "kv":
        x = synth_kv(kind, N_KV, CTX, seed=55, device=dev)
        codec = Codec(N_KV, dev).calibrate(x[:, :2048]); te = TileEncoder(kind, dev)
        for _ in range(max(1, args.warmup)): te.encode(codec, x)
        torch.cuda.synchronize(); ts = []
        for _ in range(args.steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); pg = te.encode(codec, x); b.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(b))
        out[kind] = {"encode_ms_median": sorted(ts)[len(ts) // 2], "tiles": N_KV * (CTX // 16), "ratio": pg.ratio}
    print(json.dumps({"profile_encode": out}), flush=True)


def run_other_workload(args):
    """Secondary workloads on one GPU (not the headline line): `batch64` = one GPU's share of BASELINE config 4 (64 sequences x
    1 kv head, GQA 8, 32768-token contexts, slot layout); `paged16` = BASELINE config 2's attention (16 sequences, contexts
    uniform in [4096, 65536] + a 0-15 token filling block, 32 q / 8 kv heads, paged layout, seeded random block table)."""
    import numpy as np, torch
    from gaac_b200 import Codec, TileEncoder, attention
    from gaac_b200.kernel import choose_nsplit_sm100
    from gaac_b200.synth import synth_kv
    dev = torch.device("cuda", 0)

    def timed(fn):
        for i in range(max(3, args.warmup)): fn(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(args.steps): fn(i)
        b.record(); torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps * 1e3

    if args.workload == "batch64":
        B, S, G = 64, 32768, 8
        sets = []
        for i in range(2):                                                  # two KV sets of 0.8 GB: every step streams from HBM
            k = synth_kv("k", 8, S, 300 + i, dev).repeat(8, 1, 1); v = synth_kv("v", 8, S, 300 + i, dev).repeat(8, 1, 1)
            ck, cv = Codec(1, dev).calibrate(k[:1, :2048]), Codec(1, dev).calibrate(v[:1, :2048])
            sets.append((TileEncoder("k", dev).encode(ck, k), TileEncoder("v", dev).encode(cv, v))); del k, v
        q = torch.randn(B, G, 128, device=dev).to(torch.bfloat16)
        nbytes = sets[0][0].nbytes + sets[0][1].nbytes; ns = choose_nsplit_sm100(B, 1, S)
        us = timed(lambda i: attention(q, *sets[i % 2], nsplit=ns))
        desc = "64 sequences x 1 kv head x 8 q heads, 32768-token contexts, slot layout (one GPU's share of config 4)"
    else:
        from gaac_b200.vllm.store import LayerState, OVF_OFF
        from gaac_b200.vllm.paged_kernel import paged_attention
        n_kv, G, B = 8, 4, 16
        rng = np.random.default_rng(0)
        lens = [int(l) // 16 * 16 + int(t) for l, t in zip(rng.integers(4096, 65537, B), rng.integers(0, 16, B))]
        num_blocks = sum((l + 15) // 16 for l in lens) + 1024
        cal_k, cal_v = synth_kv("k", n_kv, 2048, 7, dev), synth_kv("v", n_kv, 2048, 7, dev)
        ck, cv = Codec(n_kv, dev).calibrate(cal_k), Codec(n_kv, dev).calibrate(cal_v)
        st = LayerState(num_blocks, n_kv, raw_tiles=B * 2 * n_kv + 4096, ovf_slot=128, device=dev,
                        bases={"k3": ck.base3.cpu(), "k4": ck.base4.cpu(), "v3": cv.base3.cpu(), "v4": cv.base4.cpu()})
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
        q = torch.randn(B, n_kv * G, 128, device=dev).to(torch.bfloat16)
        out = torch.empty(B, n_kv * G * 128, dtype=torch.bfloat16, device=dev)
        full, part = sum(l // 16 for l in lens), sum(l % 16 for l in lens)
        nbytes = full * 2 * n_kv * (2880 + 53) + part * 2 * n_kv * 256      # slot payload + mean escape bytes; filling blocks are raw BF16
        ns = choose_nsplit_sm100(B, n_kv, bt.shape[1] * 16, ragged=True)
        us = timed(lambda i: paged_attention(q, out, buf, st.raw, st.mt, btd, sl, st.bases, st.TS, n_kv * G, n_kv, ns))
        desc = f"16 sequences, contexts 4096..65536 (+0..15 filling tokens, {sum(lens)} tokens in all), 32 q / 8 kv heads, paged layout, random block table"
    peak, which = measured_peak_gbs()
    print(json.dumps({"metric": "decode_attn_us_per_layer", "workload": args.workload, "value": us, "unit": "us/layer", "n_gpus": 1, "steps": args.steps,
                      "config": {"workload": desc, "nsplit": ns}, "compressed_mb": nbytes / 1e6,
                      "roofline": {"bound": "hbm", "achieved": nbytes / us / 1e3, "peak": peak, "unit": "GB/s", "frac": nbytes / us / 1e3 / peak, "peak_source": which}}), flush=True)


def side_measurements(torch, dev, sets, q, args) -> dict:
    """Numbers reported beside the headline (outside its timed region): the CPU baseline on a bounded sample, the encoder's
    throughput, and a library BF16-KV decode (flash-attn / SDPA) at the same shape for context."""
    from gaac_b200 import Codec, TileEncoder
    from gaac_b200.synth import synth_kv
    out = {}
    threads = os.cpu_count() or 1
    cpu, kind = make_cpu_path(1, 16384, threads)
    cpu.step_us_per_layer()
    tb, vals = time.perf_counter(), []
    while time.perf_counter() - tb < 10.0: vals.append(cpu.step_us_per_layer())
    out["cpu_baseline"] = {"value": sum(vals) / len(vals), "unit": "us/layer", "cores": threads, "kind": kind, "sample": cpu.sample + f", mean of {len(vals)} runs"}
    # encoder: 8 x 65536 tokens per kind
    try:
        enc = {}
        for kind in "kv":
            x = synth_kv(kind, N_KV, CTX, seed=55, device=dev)
            codec = Codec(N_KV, dev).calibrate(x[:, :2048]); te = TileEncoder(kind, dev)
            xs = [x, x.clone(), x.clone()]
            for i in range(3): te.encode(codec, xs[i % 3])
            torch.cuda.synchronize(); ts = []
            for i in range(9):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); pg = te.encode(codec, xs[i % 3]); b.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(b))
            ms = sorted(ts)[len(ts) // 2]
            enc[kind] = {"ms": ms, "blocks_per_s": N_KV * (CTX // 16) / (ms * 1e-3), "gbs_in_plus_out": (x.numel() * 2 + pg.nbytes) / (ms * 1e-3) / 1e9, "ratio": pg.ratio}
            del x, xs
        out["encode"] = enc
    except Exception as e:                                   # side number only
        out["encode"] = {"error": repr(e)}
    # library BF16-KV decode at the same shape (context, not our kernel)
    try:
        k = torch.randn(N_SETS, 1, CTX, N_KV, HEAD_DIM, device=dev).to(torch.bfloat16); v = torch.randn_like(k)
        qq = q.view(1, 1, N_Q, HEAD_DIM)
        try:
            from flash_attn import flash_attn_with_kvcache
            f = lambda i: flash_attn_with_kvcache(qq, k[i % N_SETS], v[i % N_SETS], softmax_scale=SCALE, causal=True); name = "flash_attn_with_kvcache"
            f(0)
        except Exception:
            import torch.nn.functional as F
            f = lambda i: F.scaled_dot_product_attention(qq.transpose(1, 2), k[i % N_SETS].transpose(1, 2), v[i % N_SETS].transpose(1, 2), scale=SCALE, enable_gqa=True); name = "sdpa"
        for i in range(5): f(i)
        torch.cuda.synchronize(); ts = []
        for i in range(40):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); f(i); b.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(b))
        out["bf16_kv_decode_library"] = {"name": name, "us": sorted(ts)[len(ts) // 2] * 1e3}
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="config1", choices=["config1", "batch64", "paged16"], help="config1 = the headline line; the others print a one-GPU line for a secondary workload")
    ap.add_argument("--nccl-exchange", action="store_true", help="N > 1: exchange the partials with an NCCL all-gather instead of peer-memory stores")
    ap.add_argument("--no-graph", action="store_true", help="launch every layer eagerly instead of replaying CUDA graphs")
    ap.add_argument("--profile", action="store_true", help="only the warm-up and the timed steps (no e2e, no side measurements): the command to run under ncu")
    ap.add_argument("--profile-encode", action="store_true", help="only the block encoder on [8, 65536, 128] K and V, --steps times each: the command to run under ncu")
    args = ap.parse_args()
    if args.workload != "config1":
        run_other_workload(args)
        return
    if args.profile_encode:
        run_encode_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
