"""Benchmark of the packed-KV decode-attention hot path.

Workload (N = 1): V-only TurboQuant decode attention at the Qwen2.5-7B
attention shape - 28 query heads, 4 KV heads (GQA 7), head_dim 128, batch 1,
one query token, context 32768, keys fp16, values PolarQuant 3-bit packed.
One step = one decode token = 28 layers, each layer with its own KV buffers
(1.145 GB of KV per step, far larger than L2, so no flush is needed).

  value  : algorithmic KV bytes read per second with everything resident in HBM
           (the 28-layer step replayed as one CUDA graph);
  e2e    : the same metric through the public cache / attention-hook API with
           HOST inputs: per step the new token's q, k, v for all layers are
           copied from pinned host memory, appended (K copy, V quantize) and
           attended, and the outputs are copied back to the host;
  roofline: flash-decode launch time from CUDA events vs the measured HBM peak;
  cpu_baseline: the numpy oracle of the same composed path on the host cores.

With --gpus N > 1 (torchrun, one rank per GPU) every rank runs the same
per-GPU workload on its own sequences (batch sharding, no data-path
collective): weak scaling.  --impl reference times the CPU oracle only.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

METRIC = "packed-KV decode-attn GB/s"
N_LAYERS, N_Q, N_KV, DIM, CTX, V_BITS = 28, 28, 4, 128, 32768, 3
N_REP = N_Q // N_KV
KV_BYTES_LAYER = N_KV * CTX * (DIM * 2) + N_KV * CTX * (13 * 4 + 4)   # fp16 K + packed V + norms
QO_BYTES_LAYER = N_Q * DIM * 2 * 2
ALGO_BYTES_LAYER = KV_BYTES_LAYER + QO_BYTES_LAYER                       # 40.9 MB
WORKLOAD = ("V-only TurboQuant decode attention, Qwen2.5-7B shape: 28 q / 4 kv heads, d=128, "
            "B=1, ctx 32768, K fp16, V PolarQuant 3-bit; step = 1 token x 28 layers")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------
# clocks (read-only NVML sampling during the timed region)
# ---------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# ---------------------------------------------------------------------------
# CPU oracle timing (reference arm and cpu_baseline leg)
# ---------------------------------------------------------------------------
def cpu_oracle_run(layers: int, ctx: int, threads: int, seed: int = 0):
    """Times the numpy oracle's composed decode attention (scores -> softmax ->
    butterfly-pulled-out packed-V sum) on `layers` independent layer-steps of
    the workload shape at context `ctx`.  Returns (seconds, algorithmic bytes)."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    o = entry.load_oracle()
    rng = np.random.default_rng(seed)
    signs = o.signs_from_seed(DIM, 43)
    cent = o.codebook(V_BITS)
    kd = rng.standard_normal((N_KV, ctx, DIM)).astype(np.float16)
    vp = rng.integers(0, 2 ** 30, (N_KV, ctx, 13), dtype=np.int64).astype(np.uint32)
    vp[..., 12] &= 0x00FFFFFF
    vn = (rng.random((N_KV, ctx)) * 10 + 1).astype(np.float32)
    qs = rng.standard_normal((layers, N_Q, DIM)).astype(np.float16)
    vdesc = dict(packed=vp, norms=vn, centroids=cent, signs=signs, bits=V_BITS)
    scale = 1.0 / math.sqrt(DIM)

    def one(i):
        out, _ = o.decode_attention(qs[i], k_dense=kd, v_polar=vdesc, attn_scale=scale, n_rep=N_REP)
        return float(out[0, 0])

    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(one, range(layers)))
    dt = time.perf_counter() - t0
    per_layer = N_KV * ctx * (DIM * 2 + 56) + QO_BYTES_LAYER
    return dt, layers * per_layer


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    threads = max(1, min(cores, 8))
    ctx = 8192
    layers = threads
    times = []
    for i in range(args.warmup + args.steps):
        dt, nbytes = cpu_oracle_run(layers, ctx, threads, seed=i)
        if i >= args.warmup:
            times.append(dt)
    dt = sum(times) / len(times)
    val = nbytes / dt / 1e9
    sample = f"{layers} layer-steps at ctx {ctx} per step ({nbytes / 1e6:.1f} MB of KV), {threads} threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def gpu_arm(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tq = entry.load_package()
    from turboquant_mlx_b200 import base

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    n_alloc = CTX + 256
    scale = 1.0 / math.sqrt(DIM)

    # ---- caches filled through the public API (prefill insert of CTX tokens) ----
    caches = []
    for layer in range(N_LAYERS):
        c = tq.VOnlyTurboQuantCache(bits=V_BITS, seed=42, fused=True)
        k = torch.randn((1, N_KV, CTX, DIM), generator=gen, device=dev, dtype=torch.float16)
        v = (torch.randn((1, N_KV, CTX, DIM), generator=gen, device=dev) *
             torch.exp(0.5 * torch.randn((1, N_KV, CTX, 1), generator=gen, device=dev))).to(torch.float16)
        c.reserve(1, N_KV, n_alloc, DIM, DIM, torch.float16, dev)
        c.update_and_fetch(k, v)          # prefill insert: K copied, V quantized and packed
        caches.append(c)
        del k, v
    q_dev = torch.randn((N_LAYERS, 1, N_Q, 1, DIM), generator=gen, device=dev).to(torch.float16)
    out_dev = torch.empty((N_LAYERS, 1, N_Q, 1, DIM), dtype=torch.float16, device=dev)
    torch.cuda.synchronize()

    # ---- device-resident step: 28 flash-decode launches, captured as one graph ----
    from turboquant_mlx_b200.v_only_cache import v_only_attention

    if args.kernel_only:
        for _ in range(args.warmup + args.steps):
            for layer in range(N_LAYERS):
                v_only_attention(q_dev[layer], caches[layer], scale, kv_stable=True)
        torch.cuda.synchronize()
        print(json.dumps({"kernel_only": True, "layers": N_LAYERS, "launches": (args.warmup + args.steps) * N_LAYERS}))
        return

    # The caches are static here (nothing appends between launches), so the kernel may
    # prefetch K / V while the previous layer's launch drains (kv_stable).
    def device_step():
        for layer in range(N_LAYERS):
            v_only_attention(q_dev[layer], caches[layer], scale, kv_stable=True, out=out_dev[layer])

    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            device_step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        device_step()

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    sampler = ClockSampler(local)
    with sampler:
        ms_step = timed(graph.replay, args.steps, args.warmup)
    step_bytes = N_LAYERS * ALGO_BYTES_LAYER
    value = world * step_bytes / (ms_step * 1e-3) / 1e9
    toks = world / (ms_step * 1e-3)

    # ---- roofline of the dominant kernel: one flash-decode call, event-timed per launch ----
    def one_layer_calls():
        for layer in range(N_LAYERS):
            v_only_attention(q_dev[layer], caches[layer], scale, kv_stable=True)
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2):
        one_layer_calls()
    ms_calls = timed(g2.replay, max(args.steps, 20), 3)
    launch_ms = ms_calls / N_LAYERS
    peak, peak_kind = measured_peaks()
    achieved = ALGO_BYTES_LAYER / (launch_ms * 1e-3) / 1e9
    # dram__bytes_read.sum + dram__bytes_write.sum per launch of this kernel on this workload, from the
    # ncu capture summarised in profiles/flash_mma_kernel_c2.md (40.97 MB read + 2.3 KB written)
    traffic = 40_966_656 + 2_304 if N_LAYERS == 28 else None

    # ---- end to end through the public API with host buffers -------------------
    tq.apply_patch()
    per_layer_in = (N_Q + 2 * N_KV) * DIM
    h_in = torch.randn((N_LAYERS, per_layer_in), dtype=torch.float16).pin_memory()
    h_out = torch.empty((N_LAYERS, N_Q * DIM), dtype=torch.float16).pin_memory()
    d_in = torch.empty_like(h_in, device=dev)
    d_out = torch.empty((N_LAYERS, N_Q * DIM), dtype=torch.float16, device=dev)

    def e2e_body():
        d_in.copy_(h_in, non_blocking=True)
        outs = []
        for layer in range(N_LAYERS):
            row = d_in[layer]
            q = row[:N_Q * DIM].view(1, N_Q, 1, DIM)
            k = row[N_Q * DIM:(N_Q + N_KV) * DIM].view(1, N_KV, 1, DIM)
            v = row[(N_Q + N_KV) * DIM:].view(1, N_KV, 1, DIM)
            c = caches[layer]
            keys, values = c.update_and_fetch(k, v)
            outs.append(base.scaled_dot_product_attention(q, keys, values, c, scale, None))
            c.trim(1)                     # hold the context at CTX for the next step
        torch.stack(outs, out=d_out.view(N_LAYERS, 1, N_Q, 1, DIM))     # one gather of the 28 layer outputs
        h_out.copy_(d_out, non_blocking=True)

    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        e2e_body()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g3 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g3):
        e2e_body()

    def e2e_step():
        g3.replay()
        torch.cuda.current_stream().synchronize()   # the host reads the result every step

    ms_e2e = timed(e2e_step, args.steps, args.warmup)
    tq.remove_patch()
    e2e_val = world * step_bytes / (ms_e2e * 1e-3) / 1e9
    h2d = h_in.numel() * 2
    d2h = h_out.numel() * 2

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": N_LAYERS, "kv_bytes_per_step": step_bytes,
                   "l2": "inputs (1.15 GB per step) larger than L2, no flush",
                   "sharding": "one independent sequence per GPU, no collective",
                   "tok_per_s": toks, "pct_of_8TBs": value / world / 8000.0 * 100,
                   "e2e_path": "CUDA-graph replay of H2D(q,k,v) -> append -> hooked SDPA -> D2H, ctx held at 32768"},
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e},
        "gpu_launches": args.steps * N_LAYERS,
        "clocks": sampler.summary(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind,
                     "kernel": "flash_mma_kernel (split-K flash decode, merge fused)", "us_per_launch": launch_ms * 1e3,
                     "bytes_per_launch": ALGO_BYTES_LAYER},
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        cores = len(os.sched_getaffinity(0))
        threads = max(1, min(cores, 8))
        dt, nbytes = cpu_oracle_run(threads, 8192, threads)
        line["cpu_baseline"] = {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": f"{threads} layer-steps at ctx 8192 ({nbytes / 1e6:.1f} MB), numpy oracle"}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# other BASELINE configurations (parity-test shapes; secondary measurements)
# ---------------------------------------------------------------------------
def _time_graph(torch, fn, iters, warmup=3):
    """Mean ms of fn() replayed as a CUDA graph (inputs must already be resident)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(warmup):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def workload_c1(args):
    """Config 1: PolarQuant 3-bit encode + decode round trip, [1, 4, 4096, 128] fp16,
    and the same kernels at a saturating 2^21 vectors (buffers rotated, > L2)."""
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    tq = entry.load_package()
    from turboquant_mlx_b200.kernels import dequantize_into, quantize_into
    peak, kind = measured_peaks()
    pq = tq.PolarQuantizer(DIM, 3, seed=43, device=dev)
    res = {}
    for name, n, nbuf in (("c1_16384", 4 * 4096, 64), ("sat_2M", 1 << 21, 3)):
        gen = torch.Generator(device=dev).manual_seed(5)
        xs = [(torch.randn((1, n, DIM), generator=gen, device=dev) *
               torch.exp(0.5 * torch.randn((1, n, 1), generator=gen, device=dev))).half() for _ in range(nbuf)]
        packed = [torch.empty((1, n, 13), dtype=torch.uint32, device=dev) for _ in range(nbuf)]
        norms = [torch.empty((1, n), dtype=torch.float32, device=dev) for _ in range(nbuf)]
        outs = [torch.empty((1, n, DIM), dtype=torch.float16, device=dev) for _ in range(nbuf)]

        def enc():
            for i in range(nbuf):
                quantize_into(xs[i], pq.signs, pq.boundaries, DIM, 3, packed[i], norms[i])

        def dec():
            for i in range(nbuf):
                dequantize_into(packed[i], norms[i], pq.centroids, pq.signs, DIM, 3, outs[i], n)

        ms_e = _time_graph(torch, enc, args.steps) / nbuf
        ms_d = _time_graph(torch, dec, args.steps) / nbuf
        b = n * 312
        res[name] = {"vectors": n, "encode_us": ms_e * 1e3, "encode_GBs": b / ms_e / 1e6,
                     "encode_frac": b / ms_e / 1e6 / peak, "decode_us": ms_d * 1e3,
                     "decode_GBs": b / ms_d / 1e6, "decode_frac": b / ms_d / 1e6 / peak}
    print(json.dumps({"metric": "PolarQuant 3-bit encode / decode GB/s", "unit": "GB/s", "n_gpus": 1,
                      "value": res["sat_2M"]["encode_GBs"], "peak": peak, "peak_kind": kind,
                      "config": {"workload": "C1 round trip, 312 algorithmic bytes per vector per direction"},
                      "results": res}))


def workload_c3(args):
    """Config 3: full TurboQuantKVCache (K 4-bit, V 3-bit), 32 q / 8 kv heads, batch 32,
    context 8192, one decode token per sequence; 260.0 MB of packed KV per layer-step."""
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    tq = entry.load_package()
    B, nq, nkv, ctx, layers = 32, 32, 8, 8192, 2
    gen = torch.Generator(device=dev).manual_seed(9)
    caches = []
    for _ in range(layers):
        c = tq.TurboQuantKVCache(bits=3, k_bits=4, v_bits=3, fused=True)
        c.reserve(B, nkv, ctx + 256, DIM, DIM, dev)
        for s0 in range(0, ctx, 2048):
            k = (torch.randn((B, nkv, 2048, DIM), generator=gen, device=dev) *
                 torch.exp(0.5 * torch.randn((B, nkv, 2048, 1), generator=gen, device=dev))).half()
            c.update_and_fetch(k, k.flip(-1))
        caches.append(c)
    q = torch.randn((layers, B, nq, 1, DIM), generator=gen, device=dev).half()
    scale = 1.0 / math.sqrt(DIM)

    def step():
        for l in range(layers):
            tq.turboquant_attention(q[l], caches[l], scale)

    ms = _time_graph(torch, step, args.steps) / layers
    nbytes = B * nkv * ctx * (68 + 56)
    peak, kind = measured_peaks()
    print(json.dumps({"metric": METRIC, "unit": "GB/s", "n_gpus": 1, "value": nbytes / ms / 1e6,
                      "us_per_layer_step": ms * 1e3, "frac_of_peak": nbytes / ms / 1e6 / peak, "peak": peak,
                      "peak_kind": kind, "tensor_core_path": tq._lib.lib().tq_flash_decode_last_kernel() == 1,
                      "config": {"workload": "C3 full TurboQuant cache decode: B=32, 32q/8kv, ctx 8192, K 4-bit + V 3-bit",
                                 "bytes_per_layer_step": nbytes}}))


def workload_c4_prefill(args):
    """Config 4's prompt step, attention only: Qwen2.5-7B attention shape (28 q / 4 kv heads, d 128),
    one 32768-token causal prefill of one layer through tq_prefill_sdpa (tcgen05 tiles); FLOPs counted
    as 4 * S^2 * d * n_q / 2.  The library attention of the installed torch is timed beside it."""
    import torch
    import torch.nn.functional as F
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    tq = entry.load_package()
    nq, nkv, S = 28, 4, args.ctx or 32768
    gen = torch.Generator(device=dev).manual_seed(13)
    dtype = torch.bfloat16
    q = torch.randn((1, nq, S, DIM), generator=gen, device=dev).to(dtype)
    k = torch.randn((1, nkv, S, DIM), generator=gen, device=dev).to(dtype)
    v = torch.randn((1, nkv, S, DIM), generator=gen, device=dev).to(dtype)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(DIM)

    def timed(fn, iters, warmup=3):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    with ClockSampler(0) as clk:
        ms = timed(lambda: tq.prefill_attention(q, k, v, scale, causal=True, out=out), args.steps)
    status = tq.kernels.prefill_status(dev)
    ms_lib = timed(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=True),
                   max(2, args.steps // 2))
    flops = 4.0 * S * S * DIM * nq / 2
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
        os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    peak = peaks.get("bf16_tflops_sustained", 1400.0) if ms * args.steps > 1000 else peaks.get("bf16_tflops", 1590.0)
    print(json.dumps({"metric": "prefill-attn TFLOP/s", "unit": "TFLOP/s", "n_gpus": 1, "value": flops / ms / 1e9,
                      "ms_per_layer": ms, "kernel_status": status, "dtype": "bf16",
                      "roofline": {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": peak, "unit": "TFLOP/s",
                                   "frac": flops / ms / 1e9 / peak, "traffic": None,
                                   "peak_kind": "measured" if peaks else "fallback"},
                      "library_sdpa": {"ms_per_layer": ms_lib, "tflops": flops / ms_lib / 1e9},
                      "clocks": clk.summary(),
                      "config": {"workload": f"C4 prompt step, attention of one layer: 28q/4kv, d 128, S={S} causal, bf16",
                                 "flops_per_layer": flops}}))


def workload_c4(args):
    """Config 4 end to end: random-init Qwen2.5-7B architecture (28 layers, hidden 3584, 28 q / 4 kv heads,
    d 128, vocab 152064, bf16 weights ~N(0, 0.02)), a prompt of uniform-random token ids prefilled into plain
    bf16 caches (prompt attention through tq_prefill_sdpa), conversion to the K8 / V4 group-64 cache, then greedy
    decode steps through the hooked attention.  MLP width, RoPE base and norm eps are assumed (printed)."""
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    tq = entry.load_package()
    from turboquant_mlx_b200.qwen2 import Qwen2Config, Qwen2Model
    cfg = Qwen2Config()
    if args.layers != 28:
        cfg.n_layers = args.layers
    S, n_new = args.ctx or 32768, max(2, args.steps if args.steps != 50 else 256)
    model = Qwen2Model(cfg, dev, torch.bfloat16, seed=0)
    prompt = torch.randint(0, cfg.vocab, (1, S), generator=torch.Generator().manual_seed(1)).to(dev)
    tq.apply_patch()
    try:
        caches = [tq.KVCache() for _ in range(cfg.n_layers)]
        torch.cuda.synchronize()
        e0, e1, e2, e3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
        e0.record()
        logits = model.forward(prompt, caches)
        e1.record()
        caches = [tq.MixedQuantKVCache.from_kvcache(c, k_bits=8, v_bits=4, group_size=64) for c in caches]
        tok = logits[:, -1].argmax(-1, keepdim=True)
        e2.record()
        toks = [tok]
        with ClockSampler(0) as clk:
            for _ in range(n_new - 1):
                tok = model.forward(tok, caches)[:, -1].argmax(-1, keepdim=True)
                toks.append(tok)
            e3.record()
            torch.cuda.synchronize()
        prefill_status = tq.kernels.prefill_status(dev)
    finally:
        tq.remove_patch()
    t_prefill, t_convert, t_decode = e0.elapsed_time(e1), e1.elapsed_time(e2), e2.elapsed_time(e3)
    kv_bytes_per_token = cfg.n_layers * cfg.n_kv_heads * (S + n_new // 2) * (136 + 72)
    print(json.dumps({"metric": "K8/V4 end-to-end decode tok/s", "unit": "tok/s", "n_gpus": 1,
                      "value": (n_new - 1) / (t_decode / 1e3), "decode_ms_per_token": t_decode / (n_new - 1),
                      "prefill_ms": t_prefill, "prefill_tok_per_s": S / (t_prefill / 1e3), "convert_ms": t_convert,
                      "prefill_kernel_status": prefill_status, "tokens": [int(t) for t in torch.cat(toks, 1)[0, :8]],
                      "kv_GBs_during_decode": kv_bytes_per_token / (t_decode / (n_new - 1)) / 1e6,
                      "cache_bytes": sum(c.nbytes for c in caches), "params": model.n_params(), "dtype": "bf16",
                      "data": "synthetic", "clocks": clk.summary(),
                      "config": {"workload": f"C4: prompt {S}, {n_new} greedy tokens, K8/V4 group 64", **cfg.describe()}}))


def workload_c5(args):
    """Config 5: long-context decode, Llama-3-70B attention shape (64 q / 8 kv heads, d 128), K 8-bit
    group-affine + V PolarQuant 3-bit, the sequence split across the ranks: 131072 positions per GPU
    (1M tokens at 8 GPUs).  Every rank attends over its chunk, the (m, l, acc) partial states (33 KB per rank)
    reach every rank by peer-to-peer stores over NVLink (--exchange p2p, default; the NCCL all-gather is timed
    beside it) and are merged locally.  201.3 MB of KV per GPU per layer-step."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tq = entry.load_package()
    from turboquant_mlx_b200.distributed import partial_buffer
    nq, nkv, S, layers = 64, 8, 131072, 6
    gen = torch.Generator(device=dev).manual_seed(77 + rank)
    pq = tq.PolarQuantizer(DIM, 3, seed=43, device=dev)
    ks, vs = [], []
    for _ in range(layers):
        codes = torch.randint(0, 256, (1, nkv, S, DIM), generator=gen, device=dev, dtype=torch.uint8)
        scales = (torch.rand((1, nkv, S, 2), generator=gen, device=dev) * 0.02 + 0.01).half()
        biases = (torch.rand((1, nkv, S, 2), generator=gen, device=dev) * -2.0 - 1.0).half()
        vp = torch.randint(0, 2 ** 30, (1, nkv, S, 13), generator=gen, device=dev, dtype=torch.int64)
        vp[..., 12] &= 0x00FFFFFF
        vn = torch.exp(0.5 * torch.randn((1, nkv, S), generator=gen, device=dev)) * 11.3
        ks.append(dict(format="affine", codes=codes, scales=scales, biases=biases, bits=8, group=64))
        vs.append(dict(format="polar", packed=vp.to(torch.uint32), norms=vn.float(), centroids=pq.centroids,
                       signs=pq.signs, bits=3))
        del vp
    q = torch.randn((layers, 1, nq, DIM), generator=torch.Generator(device=dev).manual_seed(5), device=dev).half()
    scale = 1.0 / math.sqrt(DIM)
    # per layer: one prepared flash-decode call writing (m, l, acc) straight into the send buffer, one
    # NCCL all-gather (eager), one prepared merge call
    from turboquant_mlx_b200.distributed import partial_views
    rows = nq
    sends = [partial_buffer(rows, DIM, dev)[0] for _ in range(layers)]
    recvs = [partial_buffer(rows, DIM, dev, world) for _ in range(layers)]
    outs = [torch.empty((rows, DIM), dtype=torch.float16, device=dev) for _ in range(layers)]
    plans, merges = [], []
    for l in range(layers):
        m, lsum, acc = partial_views(sends[l], rows, DIM)
        plans.append(tq.FlashDecodePlan(q[l], k=ks[l], v=vs[l], attn_scale=scale, partials=True,
                                        partial_out=(m.view(1, nq), lsum.view(1, nq), acc.view(1, nq, DIM))))
        gm, gl, gacc = partial_views(recvs[l], rows, DIM)
        merges.append(tq.MergePlan(gm, gl, gacc, pq.signs, outs[l]))
    p2p = world > 1 and args.exchange in ("p2p", "fused")
    if p2p:
        # one exchange object for all layers (two alternating slots), one merge call per slot
        from turboquant_mlx_b200.distributed import PeerExchange
        ex, note = None, ""
        try:
            ex = PeerExchange(rows * (DIM + 2), dev)
        except Exception as exc:      # symmetric memory not available here: every rank falls back together
            note = f"peer exchange unavailable ({type(exc).__name__}), NCCL all-gather used"
        agreed = torch.tensor([1 if ex is not None else 0], device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        p2p = bool(agreed.item())
    fused = p2p and args.exchange == "fused" and world <= 8
    if p2p:
        ex_status = tq._lib.ptr(ex.status)
        slot_merges = []
        for slot in range(2):
            gm, gl, gacc = partial_views(ex.data[slot], rows, DIM)
            slot_merges.append([tq.MergePlan(gm, gl, gacc, pq.signs, outs[l]) for l in range(layers)])
    if fused:
        # the decode kernel's final step stores the merged state into every rank's slot itself
        slot_plans = []
        for slot in range(2):
            tg = ex.targets(slot, rows, DIM)
            slot_plans.append([])
            for l in range(layers):
                m, lsum, acc = partial_views(sends[l], rows, DIM)
                slot_plans[slot].append(tq.FlashDecodePlan(
                    q[l], k=ks[l], v=vs[l], attn_scale=scale, partials=True, peers=tg,
                    partial_out=(m.view(1, nq), lsum.view(1, nq), acc.view(1, nq, DIM))))

    def step():
        for l in range(layers):
            if fused:
                slot, _, flags_ptr, want = ex.next_fused(nkv)
                slot_plans[slot][l].run()
                slot_merges[slot][l].run_after_peers(flags_ptr, world, want, ex_status)
                continue
            plans[l].run()
            if p2p:
                _, flags_ptr, epoch = ex.push(sends[l])
                slot_merges[epoch & 1][l].run_after_peers(flags_ptr, world, epoch, ex_status)
                continue
            if world > 1:
                dist.all_gather_into_tensor(recvs[l].view(-1), sends[l])
            else:
                recvs[l].copy_(sends[l].unsqueeze(0), non_blocking=True)
            merges[l].run()

    def kernels_only():
        for l in range(layers):
            plans[l].run()

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    ms = timed(step, args.steps, max(args.warmup, 3)) / layers
    if p2p:
        ex.check()
        # the same step through the NCCL all-gather, for the record and as a cross-check of the result
        ref = [o.clone() for o in outs]
        was_fused, p2p, fused = fused, False, False
        ms_nccl = timed(step, args.steps, 3) / layers
        p2p, fused = True, was_fused
        err = max(float((a.float() - b.float()).abs().max()) for a, b in zip(outs, ref))
    ms_k = timed(kernels_only, args.steps, 3) / layers
    mode = ("peer stores from the decode kernel's final step + gated merge" if fused else
            "peer-to-peer stores + flags (tq_peer_push, gated merge)" if p2p else "NCCL all_gather") + \
        ", eager launches through prepared calls"
    nbytes = nkv * S * (136 + 56)
    peak, kind = measured_peaks()
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "unit": "GB/s", "n_gpus": world, "value": world * nbytes / ms / 1e6,
            "scaling": "weak", "us_per_layer_step": ms * 1e3, "us_kernel_only": ms_k * 1e3,
            "per_gpu_frac_of_peak": nbytes / ms / 1e6 / peak, "peak": peak, "peak_kind": kind,
            "tensor_core_path": tq._lib.lib().tq_flash_decode_last_kernel() == 1,
            **({"us_per_layer_step_nccl": ms_nccl * 1e3, "max_abs_diff_vs_nccl_path": err} if p2p else {}),
            "config": {"workload": "C5 sequence-sharded long-context decode: 64q/8kv, K8 affine + V3 polar, "
                                   "131072 positions per GPU, partial states all-gathered and merged per layer",
                       "context_total": world * S, "bytes_per_gpu_per_layer_step": nbytes,
                       "exchange_bytes_per_rank": nq * (DIM + 2) * 4, "timing": mode + ", CUDA events, max over ranks"}}))
    if world > 1:
        dist.destroy_process_group()


def main():
    global N_LAYERS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--layers", type=int, default=28,
                    help="layers (independent KV buffers) per step; fewer for a profiler capture")
    ap.add_argument("--kernel-only", action="store_true",
                    help="plain launches of the flash-decode kernel only (no graph, no e2e): profiler case")
    ap.add_argument("--ctx", type=int, default=0, help="c4p: prompt length (default 32768)")
    ap.add_argument("--exchange", default="fused", choices=["nccl", "p2p", "fused"],
                    help="c5: how the partial states travel between the ranks")
    ap.add_argument("--workload", default="c2", choices=["c2", "c1", "c3", "c5", "c4p", "c4"],
                    help="c2 = the headline benchmark; c1 / c3 = secondary measurements of other configurations")
    args = ap.parse_args()
    if args.workload == "c1":
        return workload_c1(args)
    if args.workload == "c3":
        return workload_c3(args)
    if args.workload == "c5":
        return workload_c5(args)
    if args.workload == "c4p":
        return workload_c4_prefill(args)
    if args.workload == "c4":
        return workload_c4(args)
    N_LAYERS = args.layers
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
