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
           copied from pinned host memory, appended (K copy, V quantize: done by
           the decode launch itself) and attended, and the outputs are copied
           back to the host;
  roofline: flash-decode launch time from CUDA events vs the measured HBM peak;
  cpu_baseline: the numpy oracle of the same composed path on the host cores.

With --gpus N > 1 (torchrun, one rank per GPU) ONE sequence of N x 32768 tokens is
sharded along the sequence: every rank holds 32768 positions of every KV head, runs
the decode kernel in partial mode on its chunk, the (m, l, acc) partial states cross
NVLink (peer stores issued by the decode kernel's final step) and the same launch waits
(bounded) for the other ranks' states and merges them, per layer, inside the timed
region: weak scaling, N = 1 is the plain workload.
--impl reference times the CPU oracle only.
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
DTYPE = "f16"   # operands of both contractions are fp16 (fp32 accumulation, fp32 softmax state)
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
    the workload shape at context `ctx`; the (layer, kv head) groups are independent
    and are spread over `threads` host threads.  Returns (seconds, algorithmic bytes)."""
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
    scale = 1.0 / math.sqrt(DIM)

    def one(task):
        i, h = divmod(task, N_KV)
        vdesc = dict(packed=vp[h:h + 1], norms=vn[h:h + 1], centroids=cent, signs=signs, bits=V_BITS)
        out, _ = o.decode_attention(qs[i, h * N_REP:(h + 1) * N_REP], k_dense=kd[h:h + 1], v_polar=vdesc,
                                    attn_scale=scale, n_rep=N_REP)
        return float(out[0, 0])

    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(one, range(layers * N_KV)))
    dt = time.perf_counter() - t0
    per_layer = N_KV * ctx * (DIM * 2 + 56) + QO_BYTES_LAYER
    return dt, layers * per_layer


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    threads = max(1, min(cores, 8))
    ctx = CTX                      # the workload's own context; a step is bounded by the layer count
    layers = max(1, threads // N_KV)
    times = []
    for i in range(args.warmup + args.steps):
        dt, nbytes = cpu_oracle_run(layers, ctx, threads, seed=i)
        if i >= args.warmup:
            times.append(dt)
    dt = sum(times) / len(times)
    val = nbytes / dt / 1e9
    sample = f"{layers} layer-steps at ctx {ctx} per step ({nbytes / 1e6:.1f} MB of KV), {threads} threads"
    # the reference's own arithmetic needs the mlx array library; probe for it so that a box that has it shows up
    import importlib.util
    mlx_note = ("mlx importable: the numpy restatement is still what is timed here" if importlib.util.find_spec("mlx")
                else "mlx unavailable: numpy restatement of the reference's pure path (oracle/tq_oracle.py)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": DTYPE,
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample, "reference_runtime": mlx_note},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def _sync_all(torch, dist, world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def _timed(torch, dist, world, dev, fn, steps, warmup):
    """Mean ms of fn() over `steps` calls after `warmup` calls: CUDA events on the current stream,
    barrier + synchronize on both sides, max over ranks."""
    for _ in range(warmup):
        fn()
    _sync_all(torch, dist, world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    _sync_all(torch, dist, world)
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def _capture(torch, fn, dev):
    """fn() captured as one CUDA graph (after two eager runs on a side stream)."""
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


class ShardedLayers:
    """One decode step of `layers` attention layers with the sequence sharded across the ranks, one
    launch per layer: the decode kernel attends over this rank's chunk in partial mode; the CTA that
    completes a (batch, kv head) group stores its merged (m, l, acc) rows into every rank's receive
    slot (plain peer stores over NVLink + one system-scope counter add per peer), then waits (bounded)
    for the other ranks' rows in its own slot, merges them and writes the layer's output.  Every layer
    has a receive slot and a workspace of its own (reused one step later), so no launch waits for
    another and the whole step replays from one CUDA graph."""

    def __init__(self, tq, qs, ks, vs, scale, v_signs, dev, world, n_q, n_kv, out_dtype, new_rows=None):
        import torch
        from turboquant_mlx_b200.distributed import PeerExchange, partial_buffer, partial_views
        self.layers = len(ks)
        rows = n_q
        self.ex = PeerExchange(rows * (DIM + 2), dev, slots=self.layers)
        self.world, self.n_kv = world, n_kv
        self.outs = [torch.empty((rows, DIM), dtype=out_dtype, device=dev) for _ in range(self.layers)]
        self.sends = [partial_buffer(rows, DIM, dev)[0] for _ in range(self.layers)]
        self.plans, self.local_plans = [], []
        for l in range(self.layers):
            m, lsum, acc = partial_views(self.sends[l], rows, DIM)
            po = (m.view(1, n_q), lsum.view(1, n_q), acc.view(1, n_q, DIM))
            kw = {} if new_rows is None else dict(new_k=new_rows[l][0], new_v=new_rows[l][1])
            self.plans.append(tq.FlashDecodePlan(qs[l], k=ks[l], v=vs[l], attn_scale=scale, partials=True,
                                                 peers=self.ex.targets(l, rows, DIM, exclusive=True),
                                                 gather=self.ex.gather_spec(l, rows, DIM),
                                                 out=self.outs[l].view(1, n_q, DIM), partial_out=po,
                                                 kv_stable=True, q_stable=True,
                                                 workspace=tq.kernels.decode_workspace(dev), **kw))
            self.local_plans.append(tq.FlashDecodePlan(qs[l], k=ks[l], v=vs[l], attn_scale=scale, partials=True,
                                                       partial_out=po, kv_stable=True, q_stable=True,
                                                       workspace=tq.kernels.decode_workspace(dev)))

    def step(self):
        for l in range(self.layers):
            self.plans[l].run()

    def kernels_only(self):
        for l in range(self.layers):
            self.local_plans[l].run()

    def status(self):
        """Largest status word of the decode workspaces (synchronises): non-zero when a bounded wait
        (a tile that never arrived, a rank that never pushed) gave up."""
        import torch
        return max(int(p._keep_ws[:4].view(torch.int32).item()) for p in self.plans + self.local_plans)


def gpu_arm(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")    # plain peer stores / loads only: no multicast objects
        if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "WARN"):
            del os.environ["NCCL_DEBUG"]                  # keeps NCCL's version banner off stdout (one JSON line)
        dist.init_process_group("nccl", device_id=dev)
    tq = entry.load_package()
    from turboquant_mlx_b200 import base
    from turboquant_mlx_b200.kernels import flash_status

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    n_alloc = CTX + 256
    scale = 1.0 / math.sqrt(DIM)
    peak, peak_kind = measured_peaks()

    # ---- caches filled through the public API (prefill insert of this rank's CTX tokens) ----
    caches = []
    for layer in range(N_LAYERS):
        c = tq.VOnlyTurboQuantCache(bits=V_BITS, seed=42, fused=True, defer_append=True, inputs_stable=True)
        k = torch.randn((1, N_KV, CTX, DIM), generator=gen, device=dev, dtype=torch.float16)
        v = (torch.randn((1, N_KV, CTX, DIM), generator=gen, device=dev) *
             torch.exp(0.5 * torch.randn((1, N_KV, CTX, 1), generator=gen, device=dev))).to(torch.float16)
        c.reserve(1, N_KV, n_alloc, DIM, DIM, torch.float16, dev)
        c.update_and_fetch(k, v)          # prefill insert: K copied, V quantized and packed
        caches.append(c)
        del k, v
    qgen = torch.Generator(device=dev).manual_seed(99)        # the query is replicated across the ranks
    q_dev = torch.randn((N_LAYERS, 1, N_Q, 1, DIM), generator=qgen, device=dev).to(torch.float16)
    out_dev = torch.empty((N_LAYERS, 1, N_Q, 1, DIM), dtype=torch.float16, device=dev)
    torch.cuda.synchronize()

    from turboquant_mlx_b200.v_only_cache import v_only_attention

    if args.kernel_only:
        for _ in range(args.warmup + args.steps):
            for layer in range(N_LAYERS):
                v_only_attention(q_dev[layer], caches[layer], scale, kv_stable=True, q_stable=True)
        torch.cuda.synchronize()
        print(json.dumps({"kernel_only": True, "layers": N_LAYERS, "launches": (args.warmup + args.steps) * N_LAYERS,
                          "status": flash_status(dev, N_KV)}))
        return

    step_bytes = N_LAYERS * ALGO_BYTES_LAYER
    sampler = ClockSampler(local)
    extra_cfg = {}

    if world == 1:
        # ---- device-resident step: 28 flash-decode launches, one graph.  The caches and queries are
        # static here, so each launch may read its inputs while the launches in front of it drain
        # (kv_stable, q_stable): consecutive layers overlap, the CTAs of three to four launches sharing every SM.
        def device_step():
            for layer in range(N_LAYERS):
                v_only_attention(q_dev[layer], caches[layer], scale, kv_stable=True, q_stable=True, out=out_dev[layer])

        graph = _capture(torch, device_step, dev)
        with sampler:
            ms_step = _timed(torch, dist, world, dev, graph.replay, args.steps, args.warmup)
            # roofline of the dominant kernel: the same launches, event-timed over a longer region
            # 200 replays = 40 ms: long enough for ~20 clock samples, short enough that the SM clock holds its
            # boost (over 120 ms of this load it settled at 1830 MHz with no throttle reason reported)
            ms_calls = _timed(torch, dist, world, dev, graph.replay, max(args.steps, 200), 3)
        launch_ms = ms_calls / N_LAYERS
        launches_per_step = N_LAYERS
        sharding = "one GPU, no collective"
        status = max(tq.kernels.workspace_status(c._decode_ws) for c in caches)
    else:
        # ---- one sequence of world x CTX tokens, sharded along the sequence ----
        ks = [dict(format="dense", data=c._k_cache.keys[:, :, :CTX, :]) for c in caches]
        vs = [dict(format="polar", packed=c._v_tq.v_packed[:, :, :CTX, :], norms=c._v_tq.v_norms[:, :, :CTX],
                   centroids=c._v_tq._v_q.centroids, signs=c._v_tq._v_q.signs, bits=V_BITS,
                   boundaries=c._v_tq._v_q.boundaries) for c in caches]
        qs = [q_dev[l, :, :, 0, :] for l in range(N_LAYERS)]
        signs = caches[0]._v_tq._v_q.signs
        sh = ShardedLayers(tq, qs, ks, vs, scale, signs, dev, world, N_Q, N_KV, torch.float16)
        # cross-check once before timing: peer-store exchange == NCCL all-gather + merge, equal on all ranks
        from turboquant_mlx_b200.distributed import sequence_parallel_decode
        sh.step()
        torch.cuda.synchronize()
        ref0 = sequence_parallel_decode(qs[0], k=ks[0], v=vs[0], attn_scale=scale, out_dtype=torch.float16)
        diff = float((ref0[0].float() - sh.outs[0].float()).abs().max())
        gathered = [torch.empty_like(sh.outs[0]) for _ in range(world)]
        dist.all_gather(gathered, sh.outs[0])
        rank_diff = max(float((g_.float() - gathered[0].float()).abs().max()) for g_ in gathered)
        graph = _capture(torch, sh.step, dev)
        gk = _capture(torch, sh.kernels_only, dev)
        with sampler:
            ms_step = _timed(torch, dist, world, dev, graph.replay, args.steps, args.warmup)
            ms_calls = _timed(torch, dist, world, dev, gk.replay, max(args.steps, 100), 3)
            ms_total = _timed(torch, dist, world, dev, graph.replay, max(args.steps, 100), 3)
        launch_ms = ms_calls / N_LAYERS
        launches_per_step = N_LAYERS
        sharding = (f"one sequence of {world * CTX} tokens split along the sequence, {CTX} positions per GPU; per "
                    "layer ONE launch: partial-mode decode -> (m, l, acc) rows stored to every rank over NVLink -> "
                    "bounded wait for the other ranks' rows -> merge; one CUDA graph per step")
        status = sh.status()
        extra_cfg = {"us_per_layer_kernel_only": launch_ms * 1e3, "us_per_layer_total": ms_total / N_LAYERS * 1e3,
                     "us_per_layer_exchange_and_merge": (ms_total - ms_calls) / N_LAYERS * 1e3,
                     "exchange_bytes_per_rank_per_layer": N_Q * (DIM + 2) * 4,
                     "max_abs_diff_vs_nccl_allgather_path": diff, "max_abs_diff_across_ranks": rank_diff,
                     "what_limits_the_rest": "not NVLink bytes (14.6 KB per rank and layer): every layer is an all-to-all "
                                             "dependency, so the CTA that completes a kv head waits one NVLink trip after "
                                             "the slowest rank, and each graph replay drains that wait once"}

    value = world * step_bytes / (ms_step * 1e-3) / 1e9
    toks = 1.0 / (ms_step * 1e-3)
    achieved = ALGO_BYTES_LAYER / (launch_ms * 1e-3) / 1e9
    # dram__bytes_read.sum + dram__bytes_write.sum per launch of this kernel on this workload, from an
    # ncu capture (its read traffic equals the algorithmic bytes to 0.2 %)
    traffic = 40_966_656 + 2_304 if N_LAYERS == 28 else None

    # ---- end to end through the public API with host buffers -------------------
    per_layer_in = (N_Q + 2 * N_KV) * DIM
    h_in = torch.randn((N_LAYERS, per_layer_in), dtype=torch.float16).pin_memory()
    h_out = torch.empty((N_LAYERS, N_Q * DIM), dtype=torch.float16).pin_memory()
    d_in = torch.empty_like(h_in, device=dev)
    d_out = torch.empty((N_LAYERS, N_Q * DIM), dtype=torch.float16, device=dev)

    def rows_of(layer):
        row = d_in[layer]
        return (row[:N_Q * DIM].view(1, N_Q, 1, DIM), row[N_Q * DIM:(N_Q + N_KV) * DIM].view(1, N_KV, 1, DIM),
                row[(N_Q + N_KV) * DIM:].view(1, N_KV, 1, DIM))

    if world == 1:
        tq.apply_patch()

        def e2e_body():
            d_in.copy_(h_in, non_blocking=True)
            outs = []
            for layer in range(N_LAYERS):
                q, k, v = rows_of(layer)
                c = caches[layer]
                keys, values = c.update_and_fetch(k, v)      # recorded; the attention launch appends
                outs.append(base.scaled_dot_product_attention(q, keys, values, c, scale, None))
                c.trim(1)                     # hold the context at CTX for the next step
            torch.stack(outs, out=d_out.view(N_LAYERS, 1, N_Q, 1, DIM))     # one gather of the 28 layer outputs
            h_out.copy_(d_out, non_blocking=True)
        e2e_launches = N_LAYERS + 1
        e2e_path = ("CUDA-graph replay of H2D(q,k,v) -> per layer: cache.update_and_fetch (deferred) + hooked SDPA "
                    "= one decode launch that appends the token and attends -> D2H, ctx held at 32768")
    else:
        # the step's token belongs to the last chunk: the last rank's decode launch appends it
        last = rank == world - 1
        ks2, vs2, new_rows = [], [], None
        S2 = CTX + 1 if last else CTX
        for c in caches:
            ks2.append(dict(format="dense", data=c._k_cache.keys[:, :, :S2, :]))
            vs2.append(dict(format="polar", packed=c._v_tq.v_packed[:, :, :S2, :], norms=c._v_tq.v_norms[:, :, :S2],
                            centroids=c._v_tq._v_q.centroids, signs=c._v_tq._v_q.signs, bits=V_BITS,
                            boundaries=c._v_tq._v_q.boundaries))
        if last:
            new_rows = [(rows_of(l)[1][:, :, 0, :], rows_of(l)[2][:, :, 0, :]) for l in range(N_LAYERS)]
        qs2 = [rows_of(l)[0][:, :, 0, :] for l in range(N_LAYERS)]
        sh2 = ShardedLayers(tq, qs2, ks2, vs2, scale, caches[0]._v_tq._v_q.signs, dev, world, N_Q, N_KV,
                            torch.float16, new_rows=new_rows)

        def e2e_body():
            d_in.copy_(h_in, non_blocking=True)
            sh2.step()
            torch.stack(sh2.outs, out=d_out.view(N_LAYERS, N_Q, DIM))
            h_out.copy_(d_out, non_blocking=True)
        e2e_launches = N_LAYERS + 1
        e2e_path = ("CUDA-graph replay of H2D(q,k,v) -> per layer one decode launch (the last rank's appends the "
                    "token) with peer push, gather and merge -> D2H, ctx held")

    g3 = _capture(torch, e2e_body, dev)

    def e2e_step():
        g3.replay()
        torch.cuda.current_stream().synchronize()   # the host reads the result every step

    ms_e2e = _timed(torch, dist, world, dev, e2e_step, args.steps, args.warmup)
    if world == 1:
        tq.remove_patch()
        status = status or max(tq.kernels.workspace_status(c._decode_ws) for c in caches)
    else:
        status = status or sh2.status()
    e2e_val = world * step_bytes / (ms_e2e * 1e-3) / 1e9
    h2d = h_in.numel() * 2
    d2h = h_out.numel() * 2

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": N_LAYERS, "kv_bytes_per_step_per_gpu": step_bytes,
                   "l2": "inputs (1.15 GB per step per GPU) larger than L2, no flush",
                   "sharding": sharding, "context_total": world * CTX,
                   "tok_per_s": toks, "pct_of_8TBs_per_gpu": value / world / 8000.0 * 100,
                   "decode_kernel_status": status, "e2e_path": e2e_path, **extra_cfg},
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e, "gpu_launches_per_step": e2e_launches},
        "gpu_launches": args.steps * launches_per_step,
        "clocks": sampler.summary(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind,
                     "kernel": "flash_mma_kernel (split-K flash decode, merge fused)", "us_per_launch": launch_ms * 1e3,
                     "bytes_per_launch": ALGO_BYTES_LAYER},
    }
    if world > 1 and not args.no_c5:
        del caches, q_dev
        torch.cuda.empty_cache()
        line["config"]["c5"] = c5_measure(args, tq, torch, dist, dev, world, rank)
    if rank == 0 and world == 1 and not args.no_cpu:
        cores = len(os.sched_getaffinity(0))
        threads = max(1, min(cores, 8))
        n_l = max(1, threads // N_KV)
        reps = 8
        t_cpu, nbytes = 0.0, 0
        for i in range(reps):
            dt, nb = cpu_oracle_run(n_l, CTX, threads, seed=100 + i)
            t_cpu, nbytes = t_cpu + dt, nbytes + nb
        line["cpu_baseline"] = {"value": nbytes / t_cpu / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": f"{reps} x {n_l} layer-steps at ctx {CTX} ({nbytes / 1e6:.1f} MB), "
                                          f"numpy oracle, (layer, kv head) groups over {threads} threads"}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
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
    sizes = (("c1_16384", 4 * 4096, 64), ("sat_2M", 1 << 21, 3))
    if args.vectors > 0:        # one size only (profiling aid): few launches in front of the captured one
        sizes = (("sat_2M", args.vectors, 3),)
    for name, n, nbuf in sizes:
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
    context 8192, one decode token per sequence; 260.0 MB of packed KV per layer-step.
    Under torchrun the KV heads are sharded across the ranks (8 heads -> N ranks, each rank keeps
    its GQA groups whole, no exchange on the data path): strong scaling of one workload."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    tq = entry.load_package()
    from turboquant_mlx_b200.distributed import shard_range
    # layers per CUDA graph: enough launches in flight to fill a GPU that holds only 1 / world of the kv heads
    B, nq_all, nkv_all, ctx, layers = 32, 32, 8, 8192, 2 * world
    h0, h1 = shard_range(nkv_all, world, rank)
    nkv = h1 - h0
    nq = nkv * (nq_all // nkv_all)
    gen = torch.Generator(device=dev).manual_seed(9 + rank)
    caches = []
    for _ in range(layers):
        c = tq.TurboQuantKVCache(bits=3, k_bits=4, v_bits=3, fused=True, inputs_stable=True)
        c.reserve(B, nkv, ctx + 256, DIM, DIM, dev)
        for s0 in range(0, ctx, 2048):
            k = (torch.randn((B, nkv, 2048, DIM), generator=gen, device=dev) *
                 torch.exp(0.5 * torch.randn((B, nkv, 2048, 1), generator=gen, device=dev))).half()
            c.update_and_fetch(k, k.flip(-1))
        caches.append(c)
    q = torch.randn((layers, B, nq, 1, DIM), generator=gen, device=dev).half()
    scale = 1.0 / math.sqrt(DIM)
    from turboquant_mlx_b200.fused_attention import cache_kv_descriptors
    outs = [torch.empty((B, nq, DIM), dtype=torch.float16, device=dev) for _ in range(layers)]

    def step():
        for l in range(layers):
            if args.splits > 0:      # tuning aid: a fixed split count instead of the planner's
                k, v = cache_kv_descriptors(caches[l])
                tq.flash_decode(q[l, :, :, 0, :], k=k, v=v, attn_scale=scale, num_splits=args.splits, out=outs[l],
                                kv_stable=True, q_stable=True, workspace_owner=caches[l])
            else:
                tq.turboquant_attention(q[l], caches[l], scale)

    g = _capture(torch, step, dev)
    ms = _timed(torch, dist, world, dev, g.replay, max(args.steps, 20), 3) / layers
    nbytes = B * nkv_all * ctx * (68 + 56)
    peak, kind = measured_peaks()
    status = max([tq.kernels.flash_status(dev, B * nkv)] +
                 [tq.kernels.workspace_status(c._decode_ws) for c in caches if c._decode_ws is not None])
    if rank == 0:
        print(json.dumps({"metric": METRIC, "unit": "GB/s", "n_gpus": world, "value": nbytes / ms / 1e6,
                          "scaling": "strong" if world > 1 else "weak",
                          "us_per_layer_step": ms * 1e3, "frac_of_peak_per_gpu": nbytes / world / ms / 1e6 / peak,
                          "peak": peak, "peak_kind": kind,
                          "tensor_core_path": tq._lib.lib().tq_flash_decode_last_kernel() == 1,
                          "decode_kernel_status": status, "splits_forced": args.splits,
                          "config": {"workload": "C3 full TurboQuant cache decode: B=32, 32q/8kv, ctx 8192, K 4-bit + V 3-bit",
                                     "bytes_per_layer_step": nbytes,
                                     "sharding": f"kv heads {nkv_all} -> {world} ranks, no exchange" if world > 1 else "one GPU"}}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    from turboquant_mlx_b200.qwen2 import Qwen2Config, Qwen2Model, StaticDecoder
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
        ec = torch.cuda.Event(enable_timing=True)
        ec.record()
        # decode: one CUDA-graph replay per token (position and length live on the device); the first
        # two tokens (one eager step that warms the host-side caches, the capture, one replay) are not timed
        dec = StaticDecoder(model, caches, S + n_new + 8)
        warm = dec.generate(tok, 2) if not args.eager else None
        toks = [tok] + ([warm] if warm is not None else [])
        n_timed = n_new - 1 - (2 if warm is not None else 0)
        torch.cuda.synchronize()
        with ClockSampler(0) as clk:
            e2.record()
            rest = dec.generate(toks[-1][:, -1:], n_timed, use_graph=not args.eager)
            e3.record()
            torch.cuda.synchronize()
        toks.append(rest)
        decode_status = tq.kernels.flash_status(dev, cfg.n_kv_heads)
        prefill_status = tq.kernels.prefill_status(dev)
    finally:
        tq.remove_patch()
    t_prefill, t_convert, t_decode = e0.elapsed_time(e1), e1.elapsed_time(ec), e2.elapsed_time(e3)
    kv_bytes_per_token = cfg.n_layers * cfg.n_kv_heads * (S + n_new // 2) * (136 + 72)
    weight_bytes = 2 * (model.n_params() - model.emb.numel())      # read once per token (bf16)
    peak, _ = measured_peaks()
    print(json.dumps({"metric": "K8/V4 end-to-end decode tok/s", "unit": "tok/s", "n_gpus": 1,
                      "value": n_timed / (t_decode / 1e3), "decode_ms_per_token": t_decode / n_timed,
                      "decode_mode": "eager" if args.eager else "one CUDA-graph replay per token",
                      "decode_kernel_status": decode_status,
                      "hbm_floor_ms_per_token": (weight_bytes + kv_bytes_per_token) / peak / 1e6,
                      "prefill_ms": t_prefill, "prefill_tok_per_s": S / (t_prefill / 1e3), "convert_ms": t_convert,
                      "prefill_kernel_status": prefill_status, "tokens": [int(t) for t in torch.cat(toks, 1)[0, :8]],
                      "kv_GBs_during_decode": kv_bytes_per_token / (t_decode / n_timed) / 1e6,
                      "cache_bytes": sum(c.nbytes for c in caches), "params": model.n_params(), "dtype": "bf16",
                      "data": "synthetic", "clocks": clk.summary(),
                      "config": {"workload": f"C4: prompt {S}, {n_new} greedy tokens, K8/V4 group 64", **cfg.describe()}}))


def c5_measure(args, tq, torch, dist, dev, world, rank):
    """Config 5: long-context decode, Llama-3-70B attention shape (64 q / 8 kv heads, d 128), K 8-bit
    group-affine + V PolarQuant 3-bit, the sequence split across the ranks: 131072 positions per GPU
    (1M tokens at 8 GPUs).  Every rank attends over its chunk, the (m, l, acc) partial states (33 KB per
    rank) reach every rank by peer stores issued by the decode kernel and are merged locally; the step is
    one CUDA graph.  201.3 MB of KV per GPU per layer-step.  Returns the record."""
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
    nbytes = nkv * S * (136 + 56)
    peak, kind = measured_peaks()
    rec = {"workload": "C5 sequence-sharded long-context decode: 64q/8kv, K8 affine + V3 polar, "
                       "131072 positions per GPU", "n_gpus": world, "context_total": world * S,
           "bytes_per_gpu_per_layer_step": nbytes, "exchange_bytes_per_rank": nq * (DIM + 2) * 4}
    if world > 1:
        sh = ShardedLayers(tq, [q[l] for l in range(layers)], ks, vs, scale, pq.signs, dev, world, nq, nkv,
                           torch.float16)
        sh.step()
        torch.cuda.synchronize()
        from turboquant_mlx_b200.distributed import sequence_parallel_decode
        ref0 = sequence_parallel_decode(q[0], k=ks[0], v=vs[0], attn_scale=scale, out_dtype=torch.float16)
        rec["max_abs_diff_vs_nccl_allgather_path"] = float((ref0[0].float() - sh.outs[0].float()).abs().max())
        g = _capture(torch, sh.step, dev)
        gk = _capture(torch, sh.kernels_only, dev)
        ms = _timed(torch, dist, world, dev, g.replay, max(args.steps, 50), 3) / layers
        ms_k = _timed(torch, dist, world, dev, gk.replay, max(args.steps, 50), 3) / layers
    else:
        outs = [torch.empty((1, nq, DIM), dtype=torch.float16, device=dev) for _ in range(layers)]
        wss = [tq.kernels.decode_workspace(dev) for _ in range(layers)]

        def step():
            for l in range(layers):
                tq.flash_decode(q[l], k=ks[l], v=vs[l], attn_scale=scale, kv_stable=True, q_stable=True, out=outs[l],
                                workspace=wss[l])
        g = _capture(torch, step, dev)
        ms = ms_k = _timed(torch, dist, world, dev, g.replay, max(args.steps, 50), 3) / layers
    rec.update({"GBs_aggregate": world * nbytes / ms / 1e6, "us_per_layer_step": ms * 1e3,
                "us_kernel_only": ms_k * 1e3, "per_gpu_frac_of_peak": nbytes / ms / 1e6 / peak, "peak": peak,
                "peak_kind": kind, "tensor_core_path": tq._lib.lib().tq_flash_decode_last_kernel() == 1,
                "decode_kernel_status": sh.status() if world > 1 else max(tq.kernels.workspace_status(w) for w in wss)})
    return rec


def workload_c5(args):
    """Config 5 alone (see c5_measure); under torchrun the sequence is sharded across the ranks."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")    # plain peer stores / loads only: no multicast objects
        dist.init_process_group("nccl", device_id=dev)
    tq = entry.load_package()
    rec = c5_measure(args, tq, torch, dist, dev, world, rank)
    if rank == 0:
        print(json.dumps({"metric": METRIC, "unit": "GB/s", "n_gpus": world, "value": rec["GBs_aggregate"],
                          "scaling": "weak", "config": rec}))
    if world > 1:
        dist.barrier()
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
    ap.add_argument("--no-c5", action="store_true", help="N > 1: skip the secondary config-5 record")
    ap.add_argument("--eager", action="store_true", help="c4: decode steps launched eagerly instead of graph replay")
    ap.add_argument("--vectors", type=int, default=0, help="c1: run this many vectors only (default: 16384 and 2^21)")
    ap.add_argument("--splits", type=int, default=0, help="c3: force the split count of the decode kernel (0 = planner)")
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
