#!/usr/bin/env python
"""Benchmark of the attention path on B200.

Headline workload (the fields of the JSON line): Llama-3-8B-shaped causal prefill attention
(BASELINE.json configs[1]): 32 layers, 32 query / 8 KV heads, head_dim 128, one sequence of 4096
tokens, bf16 q/k/v, RoPE + append + causal GQA attention per layer, f32 output. A step is one pass
over all 32 layers. With N GPUs every rank processes its own sequence (independent sequences, no
data-path collective): weak scaling.

The same line carries one object per remaining BASELINE.json config, each with its own roofline:
  decode_small_f32       configs[0]  Qwen3-0.6B-shaped decode, f32 cache (+ CPU baseline, + host-buffer e2e)
  decode / decode_sweep  configs[2]  Qwen3-30B-A3B-shaped decode at B = 8 / B = 1, 32, 64
  prefill_chunked_gemma  configs[3]  Gemma-3-4B-shaped chunked prefill, head_dim 256
  decode_seq_split       configs[4]  Qwen2.5-14B-shaped long-context decode, KV sequence split over the
                                     ranks (also at N = 1), with `decode_scaling`
  decode_head_shard      configs[2]  at B = 32 / 64 with the KV heads split over the ranks (N > 1)
  decode_turboquant      configs[2]  shape over the reference's default 3-bit cache
  projections            the matmuls either side of the path (weight-streaming and tensor-core kernels) and the
                         configs[0] attention half-layer from host hidden states

`--impl reference` times the CPU restatement of the reference's attention (oracle/) on the host
cores for the headline workload, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

S_PREFILL = 4096
N_LAYERS_PREFILL = 32


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only queries) from a thread while a
    region runs; falls back to one nvidia-smi query when NVML is unavailable."""

    def __init__(self, gpu_index: int, period_s: float = 0.005):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.samples = []
        self.reasons = set()
        self.sm_max = None
        self._stop = None
        self._thread = None
        self._err = None

    def _run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.gpu_index
            if visible:
                try:
                    idx = int(visible.split(",")[self.gpu_index])
                except ValueError:
                    idx = self.gpu_index
            h = nv.nvmlDeviceGetHandleByIndex(idx)
            self.sm_max = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {
                getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            }
            get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self._stop.is_set():
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                mask = int(get_reasons(h))
                for bit, name in names.items():
                    if bit and (mask & bit):
                        self.reasons.add(name)
                time.sleep(self.period_s)
            nv.nvmlShutdown()
        except Exception as e:  # pragma: no cover - depends on the box
            self._err = repr(e)

    def start(self):
        import threading
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["sampler not started"]}
        self._stop.set()
        self._thread.join(timeout=5)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["no samples: " + str(self._err)]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def visible_pairs_causal(S: int) -> int:
    return S * (S + 1) // 2


# ---- CPU legs (the oracle: a restatement of the reference's scalar CPU attention) ------------------------

def cpu_prefill_sample(stride: int = 16, threads: int = 0, native: bool = True):
    """Times the oracle (the reference's per-token CPU attention) on every `stride`-th query
    position of one Llama-3-8B-shaped layer over a fully populated Q8 cache, and scales by the
    visible (query, key) pairs to a whole layer. Returns (one_pass, scale, info, oracle)."""
    from gguf_runner_b200 import presets
    from gguf_runner_b200.binding import KV_Q8_ROW
    from tests.oracle_binding import Oracle, lib as oracle_lib

    cores = threads or oracle_lib().ora_threads_available()
    cfg = presets.llama3_8b_prefill(n_layers=1, seq_len=S_PREFILL, kv_format=KV_Q8_ROW)
    ora = Oracle(cfg, threads=cores, native=native)
    rng = np.random.default_rng(1002)
    k = rng.standard_normal((S_PREFILL, cfg.kv_dim)).astype(np.float32)
    v = rng.standard_normal((S_PREFILL, cfg.kv_dim)).astype(np.float32)
    qd = np.zeros(cfg.q_dim, np.float32)
    for pos in range(S_PREFILL):  # populate the cache (untimed): rope + append only
        kr = k[pos].copy()
        ora.apply_rope_qk(0, pos, qd.copy(), kr)
        ora.kv_write_token(0, pos, kr, v[pos])
    positions = list(range(stride - 1, S_PREFILL, stride))
    qs = rng.standard_normal((len(positions), cfg.q_dim)).astype(np.float32)

    def one_pass():
        t0 = time.perf_counter()
        for i, pos in enumerate(positions):
            q = qs[i].copy()
            kr = k[pos].copy()
            ora.apply_rope_qk(0, pos, q, kr)
            ora.kv_write_token(0, pos, kr, v[pos])
            ora.attention_token(0, pos, q)
        return time.perf_counter() - t0

    pairs_sample = sum(p + 1 for p in positions)
    scale = visible_pairs_causal(S_PREFILL) / pairs_sample
    build = "-O3 -march=native (built on this host)" if native else "-O2, strict IEEE (the parity build)"
    info = {"cores": cores, "kind": "port", "build": build,
            "sample": f"one layer, every {stride}th query position of S={S_PREFILL} ({len(positions)} tokens) over a "
                      f"populated q8_row cache; layer time = sample time x {scale:.2f} (visible-pair ratio), "
                      f"x {N_LAYERS_PREFILL} layers"}
    return one_pass, scale, info, ora


def cpu_prefill_baseline(stride: int, reps: int = 1):
    """tokens/s of the 32-layer prefill pass on the host cores, native and strict builds."""
    out = {}
    for native in (True, False):
        one_pass, scale, info, ora = cpu_prefill_sample(stride=stride, native=native)
        one_pass()
        t = min(one_pass() for _ in range(max(1, reps)))
        out["native" if native else "strict"] = (S_PREFILL / (t * scale * N_LAYERS_PREFILL), info)
        ora.close()
    value, info = out["native"]
    return dict(info, value=value, unit="tokens/s", value_parity_build=out["strict"][0])


def cpu_decode_cfg1():
    """configs[0] on the host cores, full size: 28 layers, T = 2048, one new token per step, q8_row cache (the
    reference's closest-to-lossless format); all cores and one thread, native and strict builds."""
    from gguf_runner_b200 import presets
    from gguf_runner_b200.binding import KV_Q8_ROW
    from tests.oracle_binding import Oracle, lib as oracle_lib
    T, L = 2048, 28
    cores = oracle_lib().ora_threads_available()
    cfg = presets.qwen3_0p6b_decode(n_layers=L, seq_len=T, kv_format=KV_Q8_ROW)
    rng = np.random.default_rng(1001)
    q = rng.standard_normal((L, 1, cfg.q_dim)).astype(np.float32)
    k = rng.standard_normal((L, 1, cfg.kv_dim)).astype(np.float32)
    v = rng.standard_normal((L, 1, cfg.kv_dim)).astype(np.float32)
    res = {}
    for native in (True, False):
        ora = Oracle(cfg, threads=cores, native=native)
        qd = np.zeros(cfg.q_dim, np.float32)
        for l in range(L):
            rows = rng.standard_normal((T - 1, 2, cfg.kv_dim)).astype(np.float32)
            for pos in range(T - 1):
                kr = rows[pos, 0].copy()
                ora.apply_rope_qk(l, pos, qd.copy(), kr)
                ora.kv_write_token(l, pos, kr, rows[pos, 1])

        def step():
            t0 = time.perf_counter()
            for l in range(L):
                ora.decode(l, [T - 1], q[l], k[l], v[l])
            return time.perf_counter() - t0

        for threads in (cores, 1):
            ora.set_threads(threads)
            step()
            t = min(step() for _ in range(5))
            res[("native" if native else "strict", threads)] = 1.0 / t
        ora.close()
    return {"value": res[("native", cores)], "unit": "tokens/s", "cores": cores, "kind": "port",
            "build": "-O3 -march=native (built on this host)",
            "value_one_thread": res[("native", 1)],
            "value_parity_build": res[("strict", cores)], "value_parity_build_one_thread": res[("strict", 1)],
            "sample": "full size: all 28 layers, 2048 cached positions, q8_row cache, best of 5 steps"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    results = {}
    for native in (True, False):
        one_pass, scale, info, ora = cpu_prefill_sample(stride=args.cpu_stride, native=native)
        for _ in range(args.warmup if native else 1):
            one_pass()
        times = [one_pass() for _ in range(args.steps if native else 1)]
        results[native] = (float(np.mean(times)), scale, info)
        ora.close()
    t, scale, info = results[True]
    step_s = t * scale * N_LAYERS_PREFILL
    value = S_PREFILL / step_s
    strict_value = S_PREFILL / (results[False][0] * scale * N_LAYERS_PREFILL)
    line = {
        "impl": "reference", "metric": "prefill attention tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": dict(info, value=value, unit="tokens/s", value_parity_build=strict_value,
                             note="ms_per_step is extrapolated from the sample: each timed step runs the sample only"),
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int):
    return {"workload": "Llama-3-8B-shaped causal prefill attention (BASELINE.json configs[1]): 32 layers, 32 q / 8 kv "
                        "heads, head_dim 128, batch 1, S=4096, bf16 q/k/v, adjacent-pair RoPE theta 5e5, f32 out",
            "sequences": n_gpus, "seq_len": S_PREFILL, "layers": N_LAYERS_PREFILL,
            "parallelism": f"{n_gpus} independent sequences, one per GPU" if n_gpus > 1 else "single GPU",
            "l2": "each step streams 1.6 GB of q/k/v, 0.5 GB of cache and 2.1 GB of output per GPU, far above the 126 MB L2",
            "timing": "value: K steps between CUDA events with no per-launch instrumentation; roofline: the same K steps "
                      "repeated with an event pair around every launch"}


# ---- GPU arm ---------------------------------------------------------------------------------------------

def fill_cache_random(torch, ctx, seed):
    """Fills a bf16 / f32 cache with N(0,1) values (synthetic stand-in for appended rows)."""
    from gguf_runner_b200.binding import RawCuda
    k, v, _, _, nbytes = ctx.kv_device_ptrs()
    dt = torch.bfloat16 if ctx.config.kv_format == 1 else torch.float32
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    for ptr in (k, v):
        flat = torch.as_tensor(RawCuda(ptr, nbytes), device="cuda").view(dt)
        step = 1 << 28
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = torch.randn(n, generator=gen, device="cuda", dtype=torch.float32).to(dt)


def timed_steps(torch, fn, steps, warmup=3, sync=None):
    """Milliseconds per call of fn over `steps` calls (CUDA events on the current stream, after warm-up)."""
    for _ in range(warmup):
        fn()
    (sync or torch.cuda.synchronize)()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    (sync or torch.cuda.synchronize)()
    return e0.elapsed_time(e1) / steps


def instrumented(torch, ctx, fn, steps):
    """Runs fn `steps` times with an event pair around every launch; returns {kind: (ms per launch, launches per step)}."""
    ctx.set_kernel_timing(True)
    for _ in range(steps):
        fn()
    torch.cuda.synchronize()
    out = {}
    for kind in (0, 1, 2, 3):
        ms, n = ctx.kernel_time(kind)
        out[kind] = (ms / n if n else 0.0, n / steps)
    ctx.set_kernel_timing(False)
    return out


def tensor_roofline(peaks, flops, ms, **extra):
    achieved = flops / (ms * 1e-3) / 1e12
    r = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
         "frac": achieved / peaks["bf16_tflops"], "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"],
         "peak_sustained": peaks["bf16_tflops_sustained"],
         "peak_source": peaks["source"] + " (cuBLAS bf16: burst figure in `peak`, seconds-long loop in `peak_sustained`; "
                        "the timed regions here last well under a second, so `frac` uses the burst figure)"}
    r.update(extra)
    return r


def hbm_roofline(peaks, nbytes, ms, **extra):
    achieved = nbytes / (ms * 1e-3) / 1e9
    r = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
         "peak_source": peaks["source"] + " (copy bandwidth)"}
    r.update(extra)
    return r


def bench_prefill(torch, dist, args, rank, world, local_rank, peaks):
    import gguf_runner_b200 as g
    from gguf_runner_b200 import presets

    cfg = presets.llama3_8b_prefill(n_layers=N_LAYERS_PREFILL, seq_len=S_PREFILL, device=local_rank)
    ctx = g.AttnContext(cfg)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1002 + rank)
    S, L = S_PREFILL, N_LAYERS_PREFILL

    def rnd(*shape):
        return torch.randn(*shape, generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)

    q = [rnd(S, cfg.q_dim) for _ in range(L)]
    k = [rnd(S, cfg.kv_dim) for _ in range(L)]
    v = [rnd(S, cfg.kv_dim) for _ in range(L)]
    out = [torch.empty(S, cfg.q_dim, device="cuda", dtype=torch.float32) for _ in range(L)]

    def step():
        for l in range(L):
            ctx.prefill(l, 0, q[l], k[l], v[l], out=out[l])

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = ctx.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    sync_all()
    elapsed_ms = e0.elapsed_time(e1)
    launches = ctx.launch_count - launches0
    # the same K steps again with an event pair around every launch: kernel durations for the roofline
    t0 = time.perf_counter()
    per_kind = instrumented(torch, ctx, step, args.steps)
    instrumented_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([elapsed_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = world * S / (ms_per_step * 1e-3)

    flops_per_launch = 4.0 * cfg.n_heads * cfg.head_dim * visible_pairs_causal(S)
    attn_ms, attn_per_step = per_kind[0]
    rope_ms, rope_per_step = per_kind[1]
    roofline = tensor_roofline(
        peaks, flops_per_launch, attn_ms, kernel="prefill attention (one launch per layer)",
        # DRAM bytes of one launch of this shape, read + write, taken from an ncu capture of the same kernel and shape
        # (not measured by this run): the kernel is bound by the tensor cores and the MUFU unit, its traffic is the
        # q / K / V minimum plus the part of the output that left L2
        traffic=67.6e6, traffic_unit="bytes per launch",
        traffic_source="constant: dram__bytes_read.sum + dram__bytes_write.sum of an ncu capture of this kernel at this shape",
        flops_per_launch=flops_per_launch, avg_launch_ms=attn_ms, launches_per_step=attn_per_step,
        rope_append_avg_ms=rope_ms, rope_append_launches_per_step=rope_per_step,
        step_frac=(flops_per_launch * L) / (ms_per_step * 1e-3) / 1e12 / peaks["bf16_tflops"],
        ms_per_step_instrumented=instrumented_ms)

    # end to end through the C ABI with host buffers (pinned): H2D of q/k/v and D2H of out inside the timed region
    hq = [torch.empty(S, cfg.q_dim, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    hk = [torch.empty(S, cfg.kv_dim, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    hv = [torch.empty(S, cfg.kv_dim, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    hout = torch.empty(S, cfg.q_dim, dtype=torch.float32).pin_memory()
    for i in range(2):
        hq[i].copy_(q[i])
        hk[i].copy_(k[i])
        hv[i].copy_(v[i])
    torch.cuda.synchronize()

    def e2e_step():
        for l in range(L):
            ctx.prefill(l, 0, hq[l & 1], hk[l & 1], hv[l & 1], out=hout)

    e2e_step()
    sync_all()
    e2e_steps = max(1, min(args.steps, 3))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    h2d = L * (S * cfg.q_dim + 2 * S * cfg.kv_dim) * 2
    d2h = L * S * cfg.q_dim * 4
    e2e = {"value": world * S / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": e2e_s * 1e3,
           "call": "ggr_attn_prefill(GGR_PTR_HOST) per layer from pinned host buffers; bound by the f32 output crossing PCIe"}
    ctx.close()
    del q, k, v, out
    torch.cuda.empty_cache()
    return value, ms_per_step, roofline, e2e, clocks, launches


def bench_prefill_gemma(torch, args, local_rank, peaks):
    """Gemma-3-4B-shaped chunked prefill (configs[3]): 34 layers (window 1024 on 5 of every 6), 8 q / 4 kv heads,
    head_dim 256, context 32768 processed in 2048-token chunks against the accumulated bf16 cache."""
    import gguf_runner_b200 as g
    from gguf_runner_b200 import presets
    S, chunk, L = 32768, 2048, 34
    cfg = presets.gemma3_4b_prefill(n_layers=L, seq_len=S, device=local_rank)
    ctx = g.AttnContext(cfg)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1004)
    # one chunk of inputs per layer kind is reused for every chunk and layer: the cache rows differ per layer
    q = torch.randn(chunk, cfg.q_dim, generator=gen, device="cuda").to(torch.bfloat16)
    k = torch.randn(chunk, cfg.kv_dim, generator=gen, device="cuda").to(torch.bfloat16)
    v = torch.randn(chunk, cfg.kv_dim, generator=gen, device="cuda").to(torch.bfloat16)
    out = torch.empty(chunk, cfg.q_dim, device="cuda")

    def step():
        for c0 in range(0, S, chunk):
            for l in range(L):
                ctx.prefill(l, c0, q, k, v, out=out)

    ms = timed_steps(torch, step, 1, warmup=1)
    per_kind = instrumented(torch, ctx, step, 1)
    attn_ms_total = per_kind[0][0] * per_kind[0][1]
    pairs_global = S * (S + 1) // 2
    w = 1024
    pairs_local = sum(min(p + 1, w) for p in range(S))
    flops = 4.0 * cfg.n_heads * cfg.head_dim * (5 * pairs_global + 29 * pairs_local)
    res = {"workload": "Gemma-3-4B-shaped chunked prefill (configs[3]): 34 layers (29 with window 1024, 5 global), 8 q / "
                       "4 kv heads, head_dim 256, context 32768 in 2048-token chunks, bf16",
           "tokens_per_s": S / (ms * 1e-3), "ms_per_pass": ms,
           "roofline": tensor_roofline(peaks, flops, attn_ms_total,
                                       kernel="prefill attention, head_dim 256 (all launches of the pass)",
                                       flops_per_pass=flops, attention_ms_per_pass=attn_ms_total,
                                       launches=per_kind[0][1], rope_append_ms_per_pass=per_kind[1][0] * per_kind[1][1],
                                       pass_frac=flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"], traffic=None)}
    ctx.close()
    torch.cuda.empty_cache()
    return res


def bench_decode_cfg1(torch, args, local_rank, peaks, with_cpu):
    """Qwen3-0.6B-shaped decode (configs[0]): 28 layers, 16 q / 8 kv heads, T=2048, batch 1, f32 cache.
    16.8 MB per layer is ~2.6 us of HBM time, below a kernel launch: the step is launch-bound, so the
    28-layer step is timed both as plain launches and replayed from a CUDA graph."""
    import gguf_runner_b200 as g
    from gguf_runner_b200 import presets
    from gguf_runner_b200.binding import KV_F32
    T, L = 2048, 28
    cfg = presets.qwen3_0p6b_decode(n_layers=L, seq_len=T, kv_format=KV_F32, device=local_rank)
    ctx = g.AttnContext(cfg)
    fill_cache_random(torch, ctx, 1001)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2001)
    q = torch.randn(L, 1, cfg.q_dim, generator=gen, device="cuda")
    k = torch.randn(L, 1, cfg.kv_dim, generator=gen, device="cuda")
    v = torch.randn(L, 1, cfg.kv_dim, generator=gen, device="cuda")
    out = torch.empty(L, 1, cfg.q_dim, device="cuda")
    pos = [T - 1]

    def step():
        for l in range(L):
            ctx.decode(l, pos, q[l], k[l], v[l], out=out[l])

    plain_ms = timed_steps(torch, step, 20)
    per_kind = instrumented(torch, ctx, step, 5)
    graph_ms, graph_err = None, None
    try:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            step()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                step()
        torch.cuda.synchronize()
        graph_ms = timed_steps(torch, graph.replay, 50)
    except Exception as e:  # capture is an optimisation of the host loop, not part of the path
        graph_err = repr(e)[:200]
    bytes_per_layer = T * cfg.kv_dim * 4 * 2
    best = min(x for x in (plain_ms, graph_ms) if x)
    # drop-in call: what the unmodified engine would issue per layer and token (host f32 buffers, pageable)
    hq, hk, hv = (x.cpu().numpy() for x in (q, k, v))
    hout = np.empty((1, cfg.q_dim), np.float32)

    def host_step():
        for l in range(L):
            ctx.decode(l, pos, hq[l], hk[l], hv[l], out=hout)

    for _ in range(3):
        host_step()
    t0 = time.perf_counter()
    for _ in range(20):
        host_step()
    host_s = (time.perf_counter() - t0) / 20
    res = {"workload": "Qwen3-0.6B-shaped decode (configs[0]): 28 layers, 16 q / 8 kv heads, T=2048, batch 1, f32 cache",
           "ms_per_step_plain_launches": plain_ms, "ms_per_step_cuda_graph": graph_ms,
           "tokens_per_s": 1.0 / (best * 1e-3), "split_count": ctx.last_split_count,
           "roofline": hbm_roofline(peaks, bytes_per_layer, per_kind[0][0], kernel="split-KV decode attention (one launch per layer)",
                                    bytes_per_launch=bytes_per_layer, avg_launch_ms=per_kind[0][0],
                                    step_frac=L * bytes_per_layer / (best * 1e-3) / 1e9 / peaks["hbm_gbs"], traffic=16.9e6,
                                    traffic_unit="bytes per launch",
                                    traffic_source="constant: ncu capture of this kernel at this shape (16.8 MB of cache)",
                                    note="`frac` is the kernel alone; `step_frac` the whole 28-layer step, which is "
                                         "bound by launch latency (2.6 us of HBM time per layer)"),
           "e2e": {"value": 1.0 / host_s, "unit": "tokens/s", "ms_per_step": host_s * 1e3,
                   "h2d_bytes_per_step": L * (cfg.q_dim + 2 * cfg.kv_dim) * 4, "d2h_bytes_per_step": L * cfg.q_dim * 4,
                   "call": "ggr_attn_decode(GGR_PTR_HOST) per layer from pageable host f32 buffers (one pinned staging "
                           "copy in, one out, one stream synchronisation per call)"}}
    if graph_ms is None:
        res["cuda_graph_error"] = graph_err
    ctx.close()
    torch.cuda.empty_cache()
    if with_cpu:
        res["cpu_baseline"] = cpu_decode_cfg1()
    return res


def bench_decode_cfg3(torch, args, local_rank, peaks, B=8, n_res=None):
    """Qwen3-30B-A3B-shaped decode: 48 layers, 32 q / 4 kv heads, T=32768, bf16 cache, one new token per step.
    With n_res < 48 only n_res layers are resident and the 48 launches of a step cycle through them (each
    layer holds gigabytes, so the L2 cannot help)."""
    import gguf_runner_b200 as g
    from gguf_runner_b200 import presets
    T, L = 32768, 48
    n_res = n_res or L
    cfg = presets.qwen3_30b_a3b_decode(n_layers=n_res, seq_len=T, max_batch=B, device=local_rank)
    ctx = g.AttnContext(cfg)
    fill_cache_random(torch, ctx, 1003)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2003)
    q = torch.randn(n_res, B, cfg.q_dim, generator=gen, device="cuda")
    k = torch.randn(n_res, B, cfg.kv_dim, generator=gen, device="cuda")
    v = torch.randn(n_res, B, cfg.kv_dim, generator=gen, device="cuda")
    out = torch.empty(n_res, B, cfg.q_dim, device="cuda")
    pos = [T - 1] * B

    def step():
        for l in range(L):
            r = l % n_res
            ctx.decode(r, pos, q[r], k[r], v[r], out=out[r])

    steps = max(3, args.steps)
    ms_per_step = timed_steps(torch, step, steps, warmup=max(3, args.warmup))
    per_kind = instrumented(torch, ctx, step, steps)
    bytes_per_launch = B * T * cfg.n_kv_heads * cfg.head_dim * 2 * 2  # K and V, bf16
    resident = "all 48 layers resident" if n_res == L else f"{n_res} layers resident, cycled by the 48 launches of a step"
    res = {"workload": f"Qwen3-30B-A3B-shaped decode (configs[2]): 48 layers, 32 q / 4 kv heads, T=32768, B={B}, bf16 cache, {resident}",
           "tokens_per_s": B / (ms_per_step * 1e-3), "ms_per_step": ms_per_step, "split_count": ctx.last_split_count,
           "roofline": hbm_roofline(peaks, bytes_per_launch, per_kind[0][0], kernel="split-KV decode attention",
                                    bytes_per_launch=bytes_per_launch, avg_launch_ms=per_kind[0][0],
                                    step_frac=L * bytes_per_launch / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                    # every cache byte is read exactly once, so the traffic of another batch size is
                                    # the B = 8 capture scaled by B
                                    traffic=540.6e6 * B / 8, traffic_unit="bytes per launch",
                                    traffic_source="constant: ncu capture of this kernel at B=8 (540.6 MB of DRAM traffic for "
                                                   "536.9 MB of cache), scaled by B")}
    ctx.close()
    torch.cuda.empty_cache()
    return res


def bench_decode_turbo(torch, args, local_rank, peaks, B=8):
    """The config-3 decode shape over a TurboQuant cache (the reference's default format, 3 bits per element)."""
    import gguf_runner_b200 as g
    from gguf_runner_b200 import presets
    from gguf_runner_b200.binding import KV_TURBO, RawCuda
    T, L = 32768, 8
    cfg = presets.qwen3_30b_a3b_decode(n_layers=L, seq_len=T, max_batch=B, device=local_rank, kv_format=KV_TURBO)
    ctx = g.AttnContext(cfg)
    # synthetic cache content: random codes, sigma in (0.5, 1.5); sign bits and residual norms stay zero
    kp, vp, ksp, vsp, nbytes = ctx.kv_device_ptrs()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1006)
    for ptr in (kp, vp):
        flat = torch.as_tensor(RawCuda(ptr, nbytes), device="cuda").view(torch.uint8)
        flat.copy_(torch.randint(0, 256, (flat.numel(),), generator=gen, device="cuda", dtype=torch.uint8))
    n_aux = B * L * T * cfg.n_kv_heads
    for ptr in (ksp, vsp):
        flat = torch.as_tensor(RawCuda(ptr, n_aux * 4), device="cuda").view(torch.float32)
        flat.copy_(torch.rand(n_aux, generator=gen, device="cuda") + 0.5)
    q = torch.randn(L, B, cfg.q_dim, generator=gen, device="cuda")
    k = torch.randn(L, B, cfg.kv_dim, generator=gen, device="cuda")
    v = torch.randn(L, B, cfg.kv_dim, generator=gen, device="cuda")
    out = torch.empty(L, B, cfg.q_dim, device="cuda")
    pos = [T - 1] * B

    def step():
        for l in range(L):
            ctx.decode(l, pos, q[l], k[l], v[l], out=out[l])

    ms_per_step = timed_steps(torch, step, max(3, args.steps))
    per_kind = instrumented(torch, ctx, step, max(3, args.steps))
    # per key and kv head: codes D/4 + sign bits D/8 bytes and two floats, for K and for V
    bytes_per_launch = B * T * cfg.n_kv_heads * (cfg.head_dim * 3 // 8 + 8) * 2
    res = {"workload": f"config-3 decode shape over a TurboQuant cache: 32 q / 4 kv heads, T=32768, B={B}, {L} layers resident",
           "ms_per_layer": ms_per_step / L, "attention_ms_per_layer": per_kind[0][0],
           "rope_and_append_ms_per_layer": per_kind[1][0] * per_kind[1][1] / L,
           "cache_bytes_per_layer": bytes_per_launch, "bf16_cache_bytes_per_layer": B * T * cfg.n_kv_heads * cfg.head_dim * 4,
           "roofline": hbm_roofline(peaks, bytes_per_launch, per_kind[0][0], kernel="attn_turbo_mma_kernel", traffic=None,
                                    note="bound by expanding the 3-bit codes (ALU and shared memory), not by HBM")}
    ctx.close()
    torch.cuda.empty_cache()
    return res


def bench_projections(torch, args, local_rank, peaks):
    """The matmuls either side of the path with device-resident weights: the weight-streaming kernel on a
    Llama-3-8B-shaped 14336 x 4096 matrix (Q4_K, Q8_0 and BF16), the tcgen05 GEMM on the same matrix for a 4096-token chunk, and the Qwen3-0.6B-shaped attention half-layer of configs[0] end to end from host hidden states."""
    import gguf_runner_b200 as g
    from gguf_runner_b200 import presets
    from gguf_runner_b200.binding import KV_Q8_ROW, W_BF16, W_Q4_K, W_Q8_0, Weights
    from tests.oracle_binding import bf16_bits, quantize_q4_k, quantize_q8_0
    rng = np.random.default_rng(77)
    res = {}
    ctx = g.AttnContext(presets.qwen3_0p6b_decode(n_layers=1, seq_len=64, device=local_rank))
    rows, cols = 14336, 4096  # an FFN-sized matrix: at 4096 x 4096 a launch is bound by its fixed ~10 us, not by HBM
    wf = (rng.standard_normal((rows, cols)) / 64.0).astype(np.float32)
    # several matrices are cycled so that the weights come from HBM, not from the 126 MB L2
    n_mats = 6
    for name, wtype, raw, nbytes in (("q4_k", W_Q4_K, quantize_q4_k(wf), rows * cols * 144 // 256),
                                     ("q8_0", W_Q8_0, quantize_q8_0(wf), rows * cols * 34 // 32),
                                     ("bf16", W_BF16, bf16_bits(wf), rows * cols * 2)):
        mats = [Weights(wtype, rows, cols, raw, device=local_rank) for _ in range(n_mats)]
        for n in (1, 4):
            x = torch.randn(n, cols, device="cuda")
            out = torch.empty(n, rows, device="cuda")
            state = {"i": 0}

            def step():
                ctx.proj_matmul(mats[state["i"] % n_mats], x, out=out)
                state["i"] += 1

            for _ in range(6):
                step()
            pair_ms = instrumented(torch, ctx, step, 24)[3][0]

            def burst():
                for _ in range(24):
                    step()

            kern_ms = timed_steps(torch, burst, 5) / 24.0
            res[f"gemv_{name}_n{n}"] = hbm_roofline(peaks, nbytes, kern_ms, kernel="proj_gemv_kernel", shape=f"{rows}x{cols}, {n} row(s)",
                                                    bytes_per_launch=nbytes, avg_launch_ms=kern_ms, avg_launch_ms_event_pair=pair_ms,
                                                    traffic=None,
                                                    note="24 back-to-back launches between one pair of events, 6 matrices cycled so the "
                                                         "weights come from HBM; an event pair around every launch adds ~5 us to each")
        if name == "bf16":
            m = 4096
            x = torch.randn(m, cols, device="cuda")
            out = torch.empty(m, rows, device="cuda")  # [4096 x 4096] x [14336 x 4096]^T
            gemm_step = lambda: ctx.proj_matmul(mats[0], x, out=out)
            for _ in range(3):
                gemm_step()
            ms = instrumented(torch, ctx, gemm_step, 10)[3][0]
            flops = 2.0 * m * rows * cols
            res["gemm_bf16_m4096"] = tensor_roofline(peaks, flops, ms, kernel="proj_gemm_kernel",
                                                     shape=f"[{m} x {cols}] x [{rows} x {cols}]^T", avg_call_ms=ms, traffic=None)
        for w in mats:
            w.close()
    ctx.close()
    # configs[0] from hidden states: 28 layers, hidden 1024, Q8_0 weights, q8_row cache (the reference's formats)
    T, L, dim = 2048, 28, 1024
    cfg = presets.qwen3_0p6b_decode(n_layers=L, seq_len=T, kv_format=KV_Q8_ROW, device=local_rank)
    ctx = g.AttnContext(cfg)
    shapes = [(cfg.q_dim, dim), (cfg.kv_dim, dim), (cfg.kv_dim, dim), (dim, cfg.q_dim)]
    layers = []
    for l in range(L):
        layers.append([Weights(W_Q8_0, r, c, quantize_q8_0((rng.standard_normal((r, c)) / np.sqrt(c)).astype(np.float32)),
                               device=local_rank) for r, c in shapes])
    xb = rng.standard_normal((1, dim)).astype(np.float32)
    out = np.empty((1, dim), np.float32)
    # fill the cache through the path itself (a prompt of T - 1 tokens per layer)
    prompt = torch.randn(T - 1, dim, device="cuda")
    for l in range(L):
        ctx.layer_prefill(l, 0, prompt, *layers[l])
    torch.cuda.synchronize()

    def host_step():
        for l in range(L):
            ctx.layer_decode(l, [T - 1], xb, *layers[l], out=out)

    for _ in range(3):
        host_step()
    t0 = time.perf_counter()
    for _ in range(20):
        host_step()
    host_s = (time.perf_counter() - t0) / 20
    dxb = torch.from_numpy(xb).cuda()
    dout = torch.empty(1, dim, device="cuda")

    def dev_step():
        for l in range(L):
            ctx.layer_decode(l, [T - 1], dxb, *layers[l], out=dout)

    dev_ms = timed_steps(torch, dev_step, 20)
    # the same step replayed from a CUDA graph: without the host's launch cost (the ctypes loop above issues 84 launches)
    graph_ms = None
    try:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            dev_step()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                dev_step()
        torch.cuda.synchronize()
        graph_ms = timed_steps(torch, graph.replay, 50)
    except Exception:  # capture is an optimisation of the host loop, not part of the path
        graph_ms = None
    res["layer_decode_configs0"] = {
        "workload": "configs[0] attention half-layer from the hidden state: 28 layers, hidden 1024, Q8_0 projection weights, "
                    "q8_row cache, T=2048, batch 1 (q / k / v projections, rope + append + attention, output projection)",
        "ms_per_step_device_resident": dev_ms, "tokens_per_s_device_resident": 1.0 / (dev_ms * 1e-3),
        "ms_per_step_cuda_graph": graph_ms, "launches_per_step": 3 * L,
        "e2e": {"value": 1.0 / host_s, "unit": "tokens/s", "ms_per_step": host_s * 1e3,
                "h2d_bytes_per_step": L * dim * 4, "d2h_bytes_per_step": L * dim * 4,
                "call": "ggr_attn_layer_decode(GGR_PTR_HOST): one hidden row in and one out per layer"}}
    ctx.close()
    for ws in layers:
        for w in ws:
            w.close()
    torch.cuda.empty_cache()
    return res


def seq_split_run(torch, dist, args, world, rank, local_rank, peaks, use_nccl):
    """One measurement of configs[4] with the KV sequence split over `world` ranks (world = 1: the whole
    sequence on this GPU, same kernels and exchange)."""
    import gguf_runner_b200 as g
    from gguf_runner_b200 import presets
    from gguf_runner_b200.binding import SHARD_KV_SEQUENCE
    T, L, B = 131072, 48, 16
    per = T // world
    per_layer_bytes = B * per * 8 * 128 * 2 * 2
    n_res = int(max(1, min(L, (100 << 30) // per_layer_bytes)))
    cfg = presets.qwen25_14b_decode(n_layers=n_res, seq_len=T, max_batch=B, device=local_rank,
                                    shard_mode=SHARD_KV_SEQUENCE, shard_pos_begin=rank * per, shard_pos_count=per,
                                    n_ranks=world, rank=rank)
    ctx = g.AttnContext(cfg)
    fill_cache_random(torch, ctx, 1005 + rank)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2005)  # q/k/v are replicated: same seed on every rank
    q = torch.randn(n_res, B, cfg.q_dim, generator=gen, device="cuda")
    k = torch.randn(n_res, B, cfg.kv_dim, generator=gen, device="cuda")
    v = torch.randn(n_res, B, cfg.kv_dim, generator=gen, device="cuda")
    part = torch.empty(B, cfg.n_heads, cfg.head_dim + 2, device="cuda")
    gathered = torch.empty(world, B, cfg.n_heads, cfg.head_dim + 2, device="cuda")
    out = torch.empty(B, cfg.q_dim, device="cuda")
    pos = [T - 1] * B
    multi = world > 1

    def step_nccl():
        for l in range(L):
            r = l % n_res
            if multi:
                ctx.decode_partial(r, pos, q[r], k[r], v[r], partial=part)
                dist.all_gather_into_tensor(gathered, part)
            else:
                ctx.decode_partial(r, pos, q[r], k[r], v[r], partial=gathered[0])
            ctx.combine_partials(gathered, out=out)

    # fused exchange: the decode kernel stores its states into the peers' receive buffers itself
    _base, handle = ctx.exchange_create(B)
    if multi:
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        ctx.exchange_connect(ipc_handles=handles)
        dist.barrier()
    else:
        ctx.exchange_connect(same_process_ptrs=[_base])

    def step_fused():
        for l in range(L):
            r = l % n_res
            ctx.decode_exchange(r, pos, q[r], k[r], v[r], out=out)

    def sync():
        torch.cuda.synchronize()
        if multi:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(step):
        ms = timed_steps(torch, step, max(3, args.steps), warmup=max(3, args.warmup), sync=sync)
        if multi:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # both variants must agree before either is timed
    step_nccl()
    ref = out.clone()
    step_fused()
    torch.cuda.synchronize()
    agree = float((out - ref).abs().max().item())
    nccl_ms = timed(step_nccl) if use_nccl else None
    ms_per_step = timed(step_fused)
    sync()
    per_kind = instrumented(torch, ctx, step_fused, max(3, args.steps))
    ctx.synchronize()
    sync()
    res = {"world": world, "per": per, "n_res": n_res, "ms_per_step": ms_per_step, "nccl_ms": nccl_ms, "agree": agree,
           "launch_ms": per_kind[0][0], "merge_ms_per_step": per_kind[2][0] * per_kind[2][1],
           "bytes_per_launch": per_layer_bytes, "exchange_bytes": B * cfg.n_heads * (cfg.head_dim + 2) * 4,
           "split_count": ctx.last_split_count}
    ctx.close()
    del q, k, v
    torch.cuda.empty_cache()
    return res


def bench_decode_seq_split(torch, dist, args, rank, world, local_rank, peaks):
    """Qwen2.5-14B-shaped long-context decode (configs[4]): T=131072, B=16, the KV sequence split into one
    contiguous slab per rank; partial (o, m, l) exchanged by the decode kernel itself (peer stores + flags) or
    all-gathered with NCCL, merged on every rank. Strong scaling: the work is fixed, so the N = 1 point (the whole
    sequence on one GPU) is measured in the same run on rank 0 as the anchor of the efficiency figure."""
    B, L = 16, 48
    n1 = None
    if world > 1:
        if rank == 0:
            n1 = seq_split_run(torch, None, args, 1, 0, local_rank, peaks, use_nccl=False)
        dist.barrier()
        torch.cuda.synchronize()
    r = seq_split_run(torch, dist, args, world, rank, local_rank, peaks, use_nccl=True)
    if world == 1:
        n1 = r
    tok = B / (r["ms_per_step"] * 1e-3)
    per_gpu = hbm_roofline(peaks, r["bytes_per_launch"], r["launch_ms"], bytes_per_launch=r["bytes_per_launch"],
                           avg_launch_ms=r["launch_ms"],
                           step_frac=L * r["bytes_per_launch"] / (r["ms_per_step"] * 1e-3) / 1e9 / peaks["hbm_gbs"])
    res = {"workload": f"Qwen2.5-14B-shaped decode (configs[4]): 48 layers, 40 q / 8 kv heads, T=131072, B=16, bf16 cache, "
                       f"KV sequence split over {world} GPU(s) ({r['per']} positions each), {r['n_res']} resident layers cycled",
           "tokens_per_s": tok, "ms_per_step": r["ms_per_step"], "split_count": r["split_count"],
           "exchange": "fused: the decode kernel stores (o/l, m, l) into every rank's receive buffer over NVLink and "
                       "raises a flag; a bounded-wait kernel merges",
           "tokens_per_s_nccl_all_gather": B / (r["nccl_ms"] * 1e-3), "ms_per_step_nccl_all_gather": r["nccl_ms"],
           "max_abs_diff_fused_vs_nccl": r["agree"], "per_gpu_roofline": per_gpu,
           "exchange_bytes_per_layer_per_gpu": r["exchange_bytes"]}
    scaling = None
    if rank == 0 and n1 is not None:
        tok1 = B / (n1["ms_per_step"] * 1e-3)
        scaling = {"n": world, "tokens_per_s": tok, "tokens_per_s_n1": tok1, "efficiency_vs_n1": tok / (world * tok1),
                   "per_gpu_frac": per_gpu["frac"], "per_gpu_step_frac": per_gpu["step_frac"],
                   "merge_ms_per_step": r["merge_ms_per_step"], "scaling": "strong (fixed T=131072, B=16)",
                   "n1_anchor": "measured in this run on rank 0 with the whole sequence on one GPU"}
    return res, scaling


def bench_decode_head_shard(torch, dist, args, rank, world, local_rank, peaks, B):
    """configs[2] at a large batch with the KV heads split over the ranks (no collective: every rank's output is
    its own slice of q_dim). With more ranks than KV heads (8 > 4) the batch is split as well."""
    import gguf_runner_b200 as g
    from gguf_runner_b200 import presets, sharding
    T, L = 32768, 48
    base = presets.qwen3_30b_a3b_decode(n_layers=1, seq_len=T, max_batch=B, device=local_rank)
    head_groups = min(world, base.n_kv_heads)
    batch_groups = world // head_groups
    hr, br = rank % head_groups, rank // head_groups
    Bl = B // batch_groups
    per_layer_bytes = Bl * T * (base.n_kv_heads // head_groups) * 128 * 2 * 2
    n_res = int(max(1, min(L, (60 << 30) // per_layer_bytes)))
    import dataclasses
    cfg, _qs, _ks = sharding.head_shard_config(dataclasses.replace(base, n_layers=n_res, max_batch=Bl), hr, head_groups)
    ctx = g.AttnContext(cfg)
    fill_cache_random(torch, ctx, 1103 + rank)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2103 + rank)
    q = torch.randn(n_res, Bl, cfg.q_dim, generator=gen, device="cuda")
    k = torch.randn(n_res, Bl, cfg.kv_dim, generator=gen, device="cuda")
    v = torch.randn(n_res, Bl, cfg.kv_dim, generator=gen, device="cuda")
    out = torch.empty(n_res, Bl, cfg.q_dim, device="cuda")
    pos = [T - 1] * Bl

    def step():
        for l in range(L):
            r = l % n_res
            ctx.decode(r, pos, q[r], k[r], v[r], out=out[r])

    def sync():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    ms = timed_steps(torch, step, max(3, args.steps), warmup=max(3, args.warmup), sync=sync)
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    per_kind = instrumented(torch, ctx, step, max(3, args.steps))
    sync()
    res = {"workload": f"Qwen3-30B-A3B-shaped decode (configs[2]) at B={B}, T=32768: KV heads split over {head_groups} rank(s)"
                       f"{', batch over ' + str(batch_groups) if batch_groups > 1 else ''}; {cfg.n_kv_heads} kv head(s) and "
                       f"{Bl} sequences per GPU, {n_res} resident layers cycled, no collective",
           "tokens_per_s": B / (ms * 1e-3), "ms_per_step": ms,
           "per_gpu_roofline": hbm_roofline(peaks, per_layer_bytes, per_kind[0][0], bytes_per_launch=per_layer_bytes,
                                            avg_launch_ms=per_kind[0][0],
                                            step_frac=L * per_layer_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"])}
    ctx.close()
    torch.cuda.empty_cache()
    return res


def run_prefill_trace():
    """Cycle counters and wall-clock stamps of the tensor-core prefill kernels (diagnostic build of the library,
    -DGGR_TC_TRACE): CTA 0 accumulates, per role, the cycles it spends in each wait and each phase of a key tile and of
    an item; the head_dim-256 kernel also stamps %globaltimer at its set-up, Q placement, loop end and epilogue in
    its first and last CTA. Run as
    `GGR_ATTN_LIBRARY=gguf_runner_b200/libggr_attn_trace.so python bench.py --case prefill_trace`
    after `python -m gguf_runner_b200.build --trace`."""
    import ctypes as C
    import torch
    import gguf_runner_b200 as g
    from gguf_runner_b200 import presets
    L_ = g.lib()
    if not hasattr(L_, "ggr_attn_debug_set_trace"):
        raise SystemExit("this library has no trace hooks: build with `python -m gguf_runner_b200.build --trace` and set "
                         "GGR_ATTN_LIBRARY to gguf_runner_b200/libggr_attn_trace.so")
    L_.ggr_attn_debug_set_trace.argtypes = [C.c_void_p]
    L_.ggr_attn_debug_set_trace.restype = None
    torch.cuda.set_device(0)
    tr = torch.zeros(160, dtype=torch.int64, device="cuda")
    L_.ggr_attn_debug_set_trace(C.c_void_p(tr.data_ptr()))
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)

    def rows(m, cfg):
        return (torch.randn(m, cfg.q_dim, generator=gen, device="cuda").to(torch.bfloat16),
                torch.randn(m, cfg.kv_dim, generator=gen, device="cuda").to(torch.bfloat16),
                torch.randn(m, cfg.kv_dim, generator=gen, device="cuda").to(torch.bfloat16))

    # head_dim 128: one Llama-3-8B-shaped layer, S = 4096
    cfg = presets.llama3_8b_prefill(n_layers=1, seq_len=S_PREFILL)
    ctx = g.AttnContext(cfg)
    q, k, v = rows(S_PREFILL, cfg)
    for _ in range(3):
        ctx.prefill(0, 0, q, k, v)
    torch.cuda.synchronize()
    t = tr.cpu().tolist()
    n = max(1, t[6])
    print(f"prefill_tc_kernel<128>, S={S_PREFILL}, CTA 0: MMA issuer {t[0]} cycles over {n} key tiles; per tile: wait V {t[1] / n:.0f}, "
          f"wait P (tile 0 / 1) {t[2] / n:.0f} / {t[3] / n:.0f}, wait K {t[4] / n:.0f}, issue P V {t[5] / n:.0f}, issue Q K^T {t[7] / n:.0f}")
    for w in (0, 1):
        o = t[8 + 8 * w:16 + 8 * w]
        nt = max(1, o[6])
        print(f"  softmax warpgroup {w}: {o[0]} cycles over {nt} tiles; per tile: wait S {o[1] / nt:.0f}, load {o[2] / nt:.0f}, "
              f"max and mask {o[3] / nt:.0f}, rescale {o[4] / nt:.0f}, exponentials and store {o[5] / nt:.0f}")
        o2 = t[128 + 4 * w:132 + 4 * w]
        ni = max(1, o2[3])
        print(f"    {o2[3]} items; per item: wait for the item {o2[0] / ni:.0f}, wait for the last P V {o2[1] / ni:.0f}, "
              f"epilogue {o2[2] / ni:.0f} cycles")
    ctx.close()

    # head_dim 256: a window layer and a global layer of the Gemma-3-4B shape, one 2048-row chunk at context 4096
    cfg = presets.gemma3_4b_prefill(n_layers=6, seq_len=8192)
    ctx = g.AttnContext(cfg)
    m = 2048
    q, k, v = rows(m, cfg)
    for layer, what in ((4, "window layer"), (5, "global layer")):
        for _ in range(3):
            ctx.prefill(layer, 4096, q, k, v)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            ctx.prefill(layer, 4096, q, k, v)
        e1.record()
        torch.cuda.synchronize()
        t = tr.cpu().tolist()
        ns = max(1, t[6])
        print(f"prefill_tc_wide_kernel<256>, {what}, rows 4096-6143: {e0.elapsed_time(e1) / 20 * 1e3:.1f} us per call (rope + attention)")
        print(f"  CTA 0 MMA issuer: {t[0]} cycles over {ns} key tiles; per tile: wait K {t[4] / ns:.0f}, issue Q K^T {t[7] / ns:.0f}, "
              f"wait V {t[1] / ns:.0f}, wait P {t[2] / ns:.0f}, issue P V {t[5] / ns:.0f}")
        o = t[8:16]
        nt = max(1, o[6])
        print(f"  CTA 0 softmax: {o[0]} cycles; per tile: wait S {o[1] / nt:.0f}, load {o[2] / nt:.0f}, max and mask {o[3] / nt:.0f}, "
              f"rescale {o[4] / nt:.0f}, exponentials and store {o[5] / nt:.0f}")
        for name, base in (("first CTA", 32), ("last CTA", 40)):
            b = t[base]
            print(f"  {name} (ns after its start): set-up {t[base + 1] - b}, dependency wait over {t[base + 2] - b}, Q in tensor memory "
                  f"{t[base + 3] - b}, key loop done {t[base + 4] - b}, last P V landed {t[base + 5] - b}, rows sent {t[base + 6] - b}, "
                  f"exit {t[base + 7] - b}")
    ctx.close()


def run_decode_stamps():
    """Phase time stamps of the decode kernels (diagnostic build of the library, -DGGR_TC_TRACE): every CTA writes
    %globaltimer at the start, after the fused prologue, after streaming its keys, after the CTA merge and at the
    end; the last CTA of a (sequence, kv head) also stamps its ticket and the (m, l) loads of the split merge.
    Run as `GGR_ATTN_LIBRARY=gguf_runner_b200/libggr_attn_trace.so python bench.py --case decode_stamps`
    after `python -m gguf_runner_b200.build --trace`."""
    import ctypes as C
    import torch
    import gguf_runner_b200 as g
    from gguf_runner_b200 import presets
    from gguf_runner_b200.binding import KV_F32
    L_ = g.lib()
    if not hasattr(L_, "ggr_attn_debug_set_trace"):
        raise SystemExit("this library has no trace hooks: build with `python -m gguf_runner_b200.build --trace` and set "
                         "GGR_ATTN_LIBRARY to gguf_runner_b200/libggr_attn_trace.so")
    L_.ggr_attn_debug_set_trace.argtypes = [C.c_void_p]
    L_.ggr_attn_debug_set_trace.restype = None
    torch.cuda.set_device(0)
    cases = [("configs[0] f32 T=2048 B=1", presets.qwen3_0p6b_decode(n_layers=2, seq_len=2048, kv_format=KV_F32), 1, 2048),
             ("configs[2] bf16 T=32768 B=1", presets.qwen3_30b_a3b_decode(n_layers=2, seq_len=32768, max_batch=1), 1, 32768),
             ("configs[2] bf16 T=32768 B=8", presets.qwen3_30b_a3b_decode(n_layers=2, seq_len=32768, max_batch=8), 8, 32768)]
    for name, cfg, B, T in cases:
        tr = torch.zeros(8 * 8192, dtype=torch.int64, device="cuda")
        L_.ggr_attn_debug_set_trace(C.c_void_p(tr.data_ptr()))
        ctx = g.AttnContext(cfg)
        fill_cache_random(torch, ctx, 3)
        gen = torch.Generator(device="cuda")
        gen.manual_seed(1)
        q = torch.randn(B, cfg.q_dim, generator=gen, device="cuda")
        k = torch.randn(B, cfg.kv_dim, generator=gen, device="cuda")
        v = torch.randn(B, cfg.kv_dim, generator=gen, device="cuda")
        out = torch.empty(B, cfg.q_dim, device="cuda")
        for _ in range(5):
            for l in range(2):
                ctx.decode(l, [T - 1] * B, q, k, v, out=out)
        torch.cuda.synchronize()
        tr.zero_()
        ctx.decode(0, [T - 1] * B, q, k, v, out=out)
        torch.cuda.synchronize()
        n = ctx.last_split_count * cfg.n_kv_heads * B
        t = tr.cpu().numpy()[:n * 8].reshape(n, 8).astype(np.float64)
        t0 = t[:, 0].min()
        print(f"{name}: splits={ctx.last_split_count} CTAs={n}: first start to last end {(t[:, 4].max() - t0) / 1e3:.1f} us")
        print("  CTA start offsets (us): min %.1f median %.1f max %.1f" % tuple(np.percentile(t[:, 0] - t0, [0, 50, 100]) / 1e3))
        for a_, b_, nm in ((0, 1, "prologue (rope, append)"), (1, 2, "stream"), (2, 3, "cta merge"), (3, 4, "ticket / split merge")):
            d = (t[:, b_] - t[:, a_]) / 1e3
            print("  %-26s median %.1f us  max %.1f us" % (nm, np.median(d), d.max()))
        last = t[t[:, 5] > 0]
        if len(last):
            print("  last CTAs: ticket %.1f us, (m, l) loads and weights %.1f us, output loads and stores %.1f us" % (
                np.median(last[:, 5] - last[:, 3]) / 1e3, np.median(last[:, 6] - last[:, 5]) / 1e3,
                np.median(last[:, 4] - last[:, 6]) / 1e3))
        ctx.close()


def run_small_case(args):
    """Small single-GPU cases for profiler captures (`ncu ... python bench.py --case NAME`): a few launches of
    one kernel on inputs above the L2 size but at most ~1 GB on the device. Prints no benchmark line."""
    import torch
    import gguf_runner_b200 as g
    from gguf_runner_b200 import presets
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    if args.case == "prefill_small":
        # one Llama-3-8B-shaped layer pair: S=4096, 32 q / 8 kv heads, bf16 (0.5 GB on the device)
        cfg = presets.llama3_8b_prefill(n_layers=2, seq_len=S_PREFILL)
        ctx = g.AttnContext(cfg)
        q = torch.randn(S_PREFILL, cfg.q_dim, generator=gen, device="cuda").to(torch.bfloat16)
        k = torch.randn(S_PREFILL, cfg.kv_dim, generator=gen, device="cuda").to(torch.bfloat16)
        v = torch.randn(S_PREFILL, cfg.kv_dim, generator=gen, device="cuda").to(torch.bfloat16)
        for _ in range(3):
            for l in range(2):
                out = ctx.prefill(l, 0, q, k, v)
    elif args.case == "prefill_gemma_small":
        # two Gemma-3-4B-shaped layers (one window, one global): 8192 positions in 2048-token chunks (0.1 GB)
        cfg = presets.gemma3_4b_prefill(n_layers=6, seq_len=8192)
        ctx = g.AttnContext(cfg)
        q = torch.randn(2048, cfg.q_dim, generator=gen, device="cuda").to(torch.bfloat16)
        k = torch.randn(2048, cfg.kv_dim, generator=gen, device="cuda").to(torch.bfloat16)
        v = torch.randn(2048, cfg.kv_dim, generator=gen, device="cuda").to(torch.bfloat16)
        for c0 in range(0, 8192, 2048):
            for l in (4, 5):
                out = ctx.prefill(l, c0, q, k, v)
    elif args.case in ("decode_small", "decode_b1_small"):
        # two Qwen3-30B-A3B-shaped layers: T=32768, B=8 (1 GB on the device) or B=1 (0.13 GB)
        B, T = (8 if args.case == "decode_small" else 1), 32768
        cfg = presets.qwen3_30b_a3b_decode(n_layers=2, seq_len=T, max_batch=B)
        ctx = g.AttnContext(cfg)
        fill_cache_random(torch, ctx, 3)
        q = torch.randn(B, cfg.q_dim, generator=gen, device="cuda")
        k = torch.randn(B, cfg.kv_dim, generator=gen, device="cuda")
        v = torch.randn(B, cfg.kv_dim, generator=gen, device="cuda")
        for _ in range(3):
            for l in range(2):
                out = ctx.decode(l, [T - 1] * B, q, k, v)
    elif args.case == "decode_cfg1_small":
        # the Qwen3-0.6B-shaped decode (f32 cache, T=2048), all 28 layers (0.47 GB on the device)
        from gguf_runner_b200.binding import KV_F32
        cfg = presets.qwen3_0p6b_decode(n_layers=28, seq_len=2048, kv_format=KV_F32)
        ctx = g.AttnContext(cfg)
        fill_cache_random(torch, ctx, 3)
        q = torch.randn(1, cfg.q_dim, generator=gen, device="cuda")
        k = torch.randn(1, cfg.kv_dim, generator=gen, device="cuda")
        v = torch.randn(1, cfg.kv_dim, generator=gen, device="cuda")
        for _ in range(2):
            for l in range(28):
                out = ctx.decode(l, [2047], q, k, v)
    elif args.case == "proj_small":
        # the projection kernels on a 4096 x 4096 matrix: tensor-core GEMM for 2048 rows, weight-streaming kernel for
        # one row over six Q8_0 matrices (0.2 GB on the device)
        from gguf_runner_b200.binding import W_BF16, W_Q8_0, Weights
        from tests.oracle_binding import bf16_bits, quantize_q8_0
        rng = np.random.default_rng(5)
        wf = (rng.standard_normal((4096, 4096)) / 64.0).astype(np.float32)
        wb = Weights(W_BF16, 4096, 4096, bf16_bits(wf))
        wq = [Weights(W_Q8_0, 4096, 4096, quantize_q8_0(wf)) for _ in range(6)]
        ctx = g.AttnContext(presets.qwen3_0p6b_decode(n_layers=1, seq_len=64))
        xm = torch.randn(2048, 4096, generator=gen, device="cuda")
        x1 = torch.randn(1, 4096, generator=gen, device="cuda")
        for _ in range(3):
            out = ctx.proj_matmul(wb, xm)
        for i in range(12):
            out1 = ctx.proj_matmul(wq[i % 6], x1)
    elif args.case == "proj_gemv_big":
        # the weight-streaming kernel on an FFN-sized 14336 x 4096 Q8_0 matrix, one row, six matrices cycled (0.4 GB)
        from gguf_runner_b200.binding import W_Q8_0, Weights
        from tests.oracle_binding import quantize_q8_0
        rng = np.random.default_rng(6)
        raw = quantize_q8_0((rng.standard_normal((14336, 4096)) / 64.0).astype(np.float32))
        wq = [Weights(W_Q8_0, 14336, 4096, raw) for _ in range(6)]
        ctx = g.AttnContext(presets.qwen3_0p6b_decode(n_layers=1, seq_len=64))
        x1 = torch.randn(1, 4096, generator=gen, device="cuda")
        for i in range(12):
            out = ctx.proj_matmul(wq[i % 6], x1)
    elif args.case == "decode_turbo_small":
        # two layers of the config-3 decode shape over a TurboQuant cache: T=32768, B=8 (0.25 GB on the device);
        # the cache keeps its zero rows (timing of the tensor-core kernel does not depend on the code values)
        from gguf_runner_b200.binding import KV_TURBO
        B, T = 8, 32768
        cfg = presets.qwen3_30b_a3b_decode(n_layers=2, seq_len=T, max_batch=B, kv_format=KV_TURBO)
        ctx = g.AttnContext(cfg)
        q = torch.randn(B, cfg.q_dim, generator=gen, device="cuda")
        k = torch.randn(B, cfg.kv_dim, generator=gen, device="cuda")
        v = torch.randn(B, cfg.kv_dim, generator=gen, device="cuda")
        for _ in range(3):
            for l in range(2):
                out = ctx.decode(l, [T - 1] * B, q, k, v)
    else:
        raise SystemExit(f"unknown case {args.case}")
    torch.cuda.synchronize()
    print("case", args.case, "done, mean |out| =", float(out.abs().mean()))


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the attention path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = measured_peaks()
    with_cpu = rank == 0 and world == 1 and not args.no_cpu

    value, ms_per_step, roofline, e2e, clocks, launches = bench_prefill(torch, dist, args, rank, world, local_rank, peaks)
    extras = {}
    if not args.no_extras:
        if world == 1:
            extras["decode"] = bench_decode_cfg3(torch, args, local_rank, peaks, B=args.decode_batch)
            extras["decode_sweep"] = [bench_decode_cfg3(torch, args, local_rank, peaks, B=1),
                                      bench_decode_cfg3(torch, args, local_rank, peaks, B=32, n_res=12),
                                      bench_decode_cfg3(torch, args, local_rank, peaks, B=64, n_res=8)]
            extras["prefill_chunked_gemma"] = bench_prefill_gemma(torch, args, local_rank, peaks)
            extras["decode_small_f32"] = bench_decode_cfg1(torch, args, local_rank, peaks, with_cpu)
            extras["decode_turboquant"] = bench_decode_turbo(torch, args, local_rank, peaks, B=args.decode_batch)
            extras["projections"] = bench_projections(torch, args, local_rank, peaks)
        seq, scaling = bench_decode_seq_split(torch, dist, args, rank, world, local_rank, peaks)
        extras["decode_seq_split"] = seq
        extras["decode_scaling"] = scaling
        if world > 1:
            extras["decode_head_shard"] = [bench_decode_head_shard(torch, dist, args, rank, world, local_rank, peaks, B=b)
                                           for b in (32, 64)]

    cpu = cpu_prefill_baseline(args.cpu_stride) if with_cpu else None

    if rank == 0:
        line = {
            "metric": "prefill attention tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world), "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches, "clocks": clocks,
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--decode-batch", type=int, default=8)
    ap.add_argument("--cpu-stride", type=int, default=16)
    ap.add_argument("--case", default=None, help="run a small profiling case (prefill_small, prefill_gemma_small, decode_small, "
                                                 "decode_b1_small, decode_cfg1_small, decode_turbo_small, proj_small, proj_gemv_big) or print the "
                                                 "decode kernels' phase stamps or the prefill kernels' cycle counters (decode_stamps, prefill_trace: diagnostic "
                                                 "library build) and exit")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.case == "decode_stamps":
        run_decode_stamps()
        return
    if args.case == "prefill_trace":
        run_prefill_trace()
        return
    if args.case:
        run_small_case(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
