#!/usr/bin/env python
"""Benchmark of the NVFP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extra]

Headline (the JSON line's `value`): HBM throughput of `nvfp4_quantize` on a 16384 x 7168 bf16
activation matrix with 0.1 % outliers, 128x4-swizzled scale factors - algorithmic bytes (input +
packed output + scale buffer + the global scale = 300 941 316 B per launch) divided by device time.
One step = one launch over one such batch.  With N GPUs every rank quantizes its own batch (the
op shards by rows with no exchange: weak scaling) and `value` is the sum over ranks.

The same line carries, under "extra", the other kernels of the path at their stated shapes
(quantize 4096x7168, RMSNorm+quantize 8192x7168, GEMM 8192^3 and 16x8192x8192, and the
N-sharded Llama-3-70B gate/up projection with its NCCL all-gather), each with its own roofline.

`--impl reference` times the CPU restatement of the reference's arithmetic (oracle/, built with
OpenMP) on the host cores on the same workload; the reference's own kernels need the TIRx
compiler and cannot run.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path[:0] = [str(REPO / "tirx-kernels_b200"), str(REPO)]

HEADLINE = {"dtype": "bfloat16", "m": 16384, "k": 7168, "sf_layout": "128x4"}
METRIC = "nvfp4_quantize HBM throughput (16384x7168 bf16, 128x4 SF, 0.1% outliers); nvfp4_gemm TFLOPS under extra"
WORKLOAD = "nvfp4_quantize bf16_128x4_m16384_k7168 (0.1% outliers x50), one batch per GPU"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel (mean of the two
# launches of the ncu summary kept under profiles/ for this kernel and shape: 234.95 MB read + ~13.3 MB written
# inside the kernel window; the rest of the 66 MB of output is still dirty in L2 when it ends).
HEADLINE_DRAM_TRAFFIC_BYTES = 248_232_000


def rank_env() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


# ---- clocks -------------------------------------------------------------------------------------
class ClockSampler:
    """Samples the SM clock and throttle reasons of one GPU (NVML, every 10 ms) while a region runs."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None

    def __enter__(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() \
                else self.index
            self._nvml, self._handle = pynvml, pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._pump, daemon=True)
            self._thread.start()
        except Exception:
            self._thread = None
        return self

    def _pump(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                for name, bit in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                break
            time.sleep(0.01)

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        busy = [c for c in self.samples if c > 0.5 * max(self.samples)] or self.samples
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def keep_busy(fn, seconds: float) -> None:
    """Runs `fn` back to back for about `seconds` so that clock samples are taken under load."""
    import torch

    end = time.perf_counter() + seconds
    while time.perf_counter() < end:
        for _ in range(20):
            fn()
        torch.cuda.synchronize()


# ---- data -----------------------------------------------------------------------------------------
def headline_input(m: int, k: int, seed: int = 42):
    """N(0,1) with 0.1 % seeded positions multiplied by 50, as bf16, plus the 448*6/amax scale (host)."""
    import torch

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g, dtype=torch.float32)
    pos = torch.randperm(m * k, generator=g)[: -(-m * k // 1000)]
    x.view(-1)[pos] *= 50.0
    x = x.to(torch.bfloat16)
    gs = torch.tensor([2688.0], dtype=torch.float32) / x.float().abs().max()
    return x, gs


def timed_region(fn, steps: int, warmup: int, distributed: bool):
    """Device milliseconds for `steps` calls of fn (max over ranks), after `warmup` untimed calls."""
    import torch

    for _ in range(warmup):
        fn()
    if distributed:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    elapsed = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device="cuda")
    if distributed:
        torch.distributed.barrier()
        torch.distributed.all_reduce(elapsed, op=torch.distributed.ReduceOp.MAX)
    return float(elapsed.item())


# ---- our arm ----------------------------------------------------------------------------------------
def run_ours(args) -> dict:
    import torch

    from tirx_kernels import _checks, _native
    from tirx_kernels.flashinfer.quantization import nvfp4_quantize as quant

    rank, local_rank, world = rank_env()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    _native.lib()  # fail loudly if the CUDA extension is missing

    m, k, layout = HEADLINE["m"], HEADLINE["k"], HEADLINE["sf_layout"]
    x_host, gs_host = headline_input(m, k, seed=42 + rank)
    ex = quant.get_kernel(**HEADLINE).config["launcher"]
    x, gs = x_host.cuda(), gs_host.cuda()
    out, sf = quant._alloc_outputs(m, k, layout)
    step_bytes = quant.algorithmic_bytes(m, k, layout)

    def step():
        quant._run_launch(ex, x, gs, out, sf, m, k, layout)

    # the clock sampler runs from a short busy period before the timed region to one after it, so
    # that its samples describe the GPU under this very load even when the region lasts milliseconds
    with ClockSampler(local_rank) as sampler:
        keep_busy(step, 0.3)
        elapsed_ms = timed_region(step, args.steps, args.warmup, distributed)
        keep_busy(step, 0.15)
    clocks = sampler.summary()
    ms_per_step = elapsed_ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    roofline = _checks.roofline_hbm(step_bytes, ms_per_step * 1e3)
    roofline["traffic"] = HEADLINE_DRAM_TRAFFIC_BYTES

    # end to end through the module's executable with host buffers: H2D of the batch, launch, D2H of
    # the packed bytes and scale factors, every step
    x_pin, out_pin, sf_pin = x_host.pin_memory(), torch.empty_like(out, device="cpu").pin_memory(), \
        torch.empty_like(sf, device="cpu").pin_memory()

    def e2e_step():
        x.copy_(x_pin, non_blocking=True)
        quant._run_launch(ex, x, gs, out, sf, m, k, layout)
        out_pin.copy_(out, non_blocking=True)
        sf_pin.copy_(sf, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    copy_rates = host_copy_rates(x, x_pin, out, out_pin, sf, sf_pin, distributed)
    serial_ms = timed_region(e2e_step, e2e_steps, 2, distributed) / e2e_steps
    # the same through the host-buffer pipeline of the package: row chunks on three streams, upload, kernel
    # and download overlapped (every byte still crosses PCIe inside the timed region)
    from tirx_kernels.flashinfer.quantization.host_pipeline import HostQuantizePipeline

    pipeline = HostQuantizePipeline(HEADLINE["dtype"], m, k, layout, chunks=8)
    e2e_ms = timed_region(lambda: pipeline(x_pin, gs, out_pin, sf_pin), e2e_steps, 2, distributed) / e2e_steps
    torch.cuda.synchronize()
    pipelined_ok = bool(torch.equal(out_pin, out.cpu()) and torch.equal(sf_pin, sf.cpu()))
    e2e = {"value": world * step_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": x_pin.numel() * 2, "d2h_bytes_per_step": out_pin.numel() + sf_pin.numel(),
           "path": "HostQuantizePipeline: 8 row chunks, upload / kernel / download on three streams",
           "launches_per_step": pipeline.launches_per_call, "matches_device_path": pipelined_ok,
           "host_copy_gbs_per_rank": copy_rates,
           "serial_copy_launch_copy": {"value": world * step_bytes / (serial_ms * 1e-3) / 1e9, "ms_per_step": serial_ms}}

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 scale math on bf16 input, e2m1/e4m3 output", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "l2": "inputs larger than L2: 301 MB touched per step, no flush needed",
                   "algorithmic_bytes_per_step": step_bytes},
        "roofline": roofline, "e2e": e2e, "gpu_launches": args.steps, "clocks": clocks,
    }
    if rank == 0:
        line["cpu_baseline"] = cpu_baseline(x_host, float(gs_host.item()), layout, budget_s=8.0)
    if not args.no_extra:
        line["extra"] = extras(args, rank, world, distributed)
        summary = line["extra"].get("ffn_gate_up_tp", {}).get("scaling_summary")
        if summary:  # last key of the line: the sharded projection against one GPU of the same box
            line["ffn_gate_up_tp"] = summary
    if distributed:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    return line if rank == 0 else {}


def host_copy_rates(x, x_pin, out, out_pin, sf, sf_pin, distributed: bool) -> dict:
    """Pinned-memory copy rates of every rank, all ranks copying at the same time (GB/s): what the end-to-end
    leg can reach when N ranks share the host's PCIe and memory fabric."""
    import torch

    def one_way(fn, nbytes):
        if distributed:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(3):
            fn()
        end.record()
        torch.cuda.synchronize()
        return 3 * nbytes / (start.elapsed_time(end) * 1e-3) / 1e9

    def download():
        out_pin.copy_(out, non_blocking=True)
        sf_pin.copy_(sf, non_blocking=True)

    h2d = one_way(lambda: x.copy_(x_pin, non_blocking=True), x_pin.numel() * 2)
    d2h = one_way(download, out_pin.numel() + sf_pin.numel())
    rates = torch.tensor([h2d, d2h], dtype=torch.float64, device="cuda")
    if distributed:
        gathered = [torch.zeros_like(rates) for _ in range(torch.distributed.get_world_size())]
        torch.distributed.all_gather(gathered, rates)
    else:
        gathered = [rates]
    return {"h2d": [round(float(g[0]), 1) for g in gathered], "d2h": [round(float(g[1]), 1) for g in gathered]}


def cpu_baseline(x_host, gs: float, layout: str, budget_s: float, steps: int | None = None) -> dict:
    """The C restatement of the reference arithmetic (OpenMP, all host cores) on the same batch."""
    import numpy as np

    from oracle import c_oracle, nvfp4_oracle

    import torch

    c_oracle.use_all_host_threads()  # torchrun pins OMP_NUM_THREADS=1 for its ranks
    bits = x_host.contiguous().view(torch.int16).numpy().view(np.uint16)
    m, k = bits.shape
    step_bytes = m * k * 2 + m * k // 2 + nvfp4_oracle.sf_buffer_size(m, k // 16, layout) + 4
    c_oracle.nvfp4_quantize(bits, "bfloat16", gs, layout)  # warm-up, loads the library
    times = []
    began = time.perf_counter()
    while (steps is None and time.perf_counter() - began < budget_s) or (steps is not None and len(times) < steps):
        t0 = time.perf_counter()
        c_oracle.nvfp4_quantize(bits, "bfloat16", gs, layout)
        times.append(time.perf_counter() - t0)
        if len(times) >= 200:
            break
    mean = statistics.fmean(times)
    return {"value": step_bytes / mean / 1e9, "unit": "GB/s", "cores": c_oracle.threads(), "kind": "port",
            "sample": f"{len(times)} passes over the full {m}x{k} batch, {mean * 1e3:.1f} ms each",
            "ms_per_step": mean * 1e3}


# ---- the other kernels of the path -----------------------------------------------------------------------
def _bench_us(fn, reps: int = 30, warm: int = 5) -> float:
    import torch

    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / reps * 1e3


def _graph_us(launches, replays: int = 20) -> float:
    """Device microseconds per launch of a CUDA graph holding `launches` (callables issued in order
    on the capturing stream): removes the host's per-launch cost from small-kernel timings."""
    import torch

    for fn in launches:  # warm up outside capture: first calls configure kernels and allocate scratch
        fn()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        for fn in launches:
            fn()
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for fn in launches:
                fn()
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / (replays * len(launches)) * 1e3


def extras(args, rank: int, world: int, distributed: bool) -> dict:
    """Per-kernel numbers at the stated shapes.  Working sets exceed L2 or rotate over several buffer
    sets so that launches do not hit a warm cache."""
    import torch

    from tirx_kernels import _checks, _native
    from tirx_kernels.basic import nvfp4_gemm as gemm
    from tirx_kernels.flashinfer.norm import rmsnorm_fp4quant as rms
    from tirx_kernels.flashinfer.quantization import nvfp4_quantize as quant

    out: dict = {}
    if rank == 0:
        # quantize 4096 x 7168, linear scales: 75 MB per launch < L2, so rotate over eight buffer sets (600 MB)
        m, k = 4096, 7168
        sets = []
        for i in range(8):
            xi = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
            oi, si = quant._alloc_outputs(m, k, "linear")
            sets.append((xi, oi, si))
        gs1 = torch.tensor([2688.0 / 5.5], device="cuda")
        ex1 = quant.get_kernel("bfloat16", m, k, "linear").config["launcher"]
        state = {"i": 0}

        def q1():
            xi, oi, si = sets[state["i"] % 8]
            state["i"] += 1
            quant._run_launch(ex1, xi, gs1, oi, si, m, k, "linear")

        us = _bench_us(q1, reps=40)
        state["i"] = 0
        us_graph = _graph_us([q1] * 8)  # 8 launches over the 8 rotating sets, replayed 20 times
        out["quantize_bf16_linear_m4096_k7168"] = {"us": us_graph, "us_with_host_launch_cost": us,
                                                   "timing": "CUDA graph of 8 launches rotating over 8 buffer sets",
                                                   "roofline": _checks.roofline_hbm(
                                                       quant.algorithmic_bytes(m, k, "linear"), us_graph)}
        del sets

        # RMSNorm + quantize 8192 x 7168: 150 MB per launch, of which the 117 MB input alone would fit in L2, and
        # streaming loads marked evict-first let part of an alternate set survive a launch (two sets in turn
        # measured 12 % faster than four).  Four sets in turn (600 MB) give the cold figure.
        cfg = next(c for c in rms.BENCH_CONFIGS if c["case"] == "bench_nv_swizzled_large")
        exr = rms.get_kernel(**{kk: v for kk, v in cfg.items() if kk != "label"}).config["launcher"]
        rsets = [(rms._prepare_tensors(cfg), rms._prepare_output(cfg, initialize=False)) for _ in range(4)]
        rlaunches = [(lambda d=d, o=o: rms._launch(exr, d, o, cfg)) for d, o in rsets] * 3
        us_graph = _graph_us(rlaunches)
        us_same = _graph_us(rlaunches[:1] * 10)
        out["rmsnorm_fp4quant_bf16_m8192_h7168_swizzled"] = {
            "us": us_graph, "us_same_buffers_back_to_back": us_same,
            "timing": "CUDA graph of 12 launches rotating over 4 buffer sets (cold inputs)",
            "roofline": _checks.roofline_hbm(rms.algorithmic_bytes(8192, 7168, 16, True), us_graph)}
        del rsets, rlaunches
        # the same kernel on 32768 rows (470 MB input, cold by size): the launch-size-independent rate
        big = dict(cfg)
        big["M"] = 32768
        dbig, obig = rms._prepare_tensors(big), rms._prepare_output(big, initialize=False)
        exr_big = rms.get_kernel(**{kk: v for kk, v in big.items() if kk != "label"}).config["launcher"]
        us_big = _graph_us([lambda: rms._launch(exr_big, dbig, obig, big)] * 4)
        out["rmsnorm_fp4quant_bf16_m32768_h7168_swizzled"] = {
            "us": us_big, "timing": "CUDA graph of 4 launches",
            "roofline": _checks.roofline_hbm(rms.algorithmic_bytes(32768, 7168, 16, True), us_big)}
        del dbig, obig

        # residual add + RMSNorm + quantize 8192 x 7168 (385 MB per launch > L2)
        from tirx_kernels.flashinfer.norm import add_rmsnorm_fp4quant as addrms

        cfg = next(c for c in addrms.BENCH_CONFIGS if c["case"] == "bench_nv_swizzled_large")
        data, output = addrms._prepare_tensors(cfg), addrms._prepare_output(cfg)
        exa = addrms.get_kernel(**{kk: v for kk, v in cfg.items() if kk != "label"}).config["launcher"]
        add_launch = lambda: addrms._launch(exa, data, output, cfg)
        us_graph = _graph_us([add_launch] * 10)
        us = _bench_us(add_launch, reps=30)
        out["add_rmsnorm_fp4quant_bf16_m8192_h7168_swizzled"] = {
            "us": us_graph, "us_with_host_launch_cost": us, "timing": "CUDA graph of 10 launches",
            "roofline": _checks.roofline_hbm(addrms.algorithmic_bytes(8192, 7168, 16, False, False), us_graph)}
        del data, output

        # GEMM 8192^3 (205 MB touched per launch > L2) and the decode shape
        for (M, N, K) in ((8192, 8192, 8192), (16, 8192, 8192)):
            A_fp4, B_fp4, A_sf, B_sf, alpha, C_ref = gemm.prepare_data(M, N, K)
            alpha_t = torch.tensor([float(alpha)], device="cuda")
            D = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            del C_ref
            exg = gemm._compile_executable(M, N, K)
            if M > 16:
                us = _bench_us(lambda: exg(A_fp4, B_fp4, A_sf, B_sf, alpha_t, D), reps=20)
                entry = {"us": us, "tflops": gemm.flops(M, N, K) / us / 1e6}
                entry.update(gemm_role_timers(lambda: exg(A_fp4, B_fp4, A_sf, B_sf, alpha_t, D), K, us))
            else:
                # decode: weights (36 MB) fit in L2, so rotate over sixteen copies (570 MB) inside a CUDA graph
                copies = [(B_fp4.clone(), B_sf.clone()) for _ in range(16)]
                launches = [(lambda b=b, sfb=sfb: exg(A_fp4, b, A_sf, sfb, alpha_t, D)) for b, sfb in copies]
                us = _graph_us(launches)
                us_warm = _bench_us(lambda: exg(A_fp4, B_fp4, A_sf, B_sf, alpha_t, D), reps=100)
                entry = {"us": us, "us_l2_warm_with_host_launch_cost": us_warm,
                         "timing": "CUDA graph of 16 launches rotating over 16 weight copies (cold weights)",
                         "tflops": gemm.flops(M, N, K) / us / 1e6}
                del copies, launches
            _native.nvfp4_gemm_status()
            entry["roofline"] = (_checks.roofline_nvfp4(gemm.flops(M, N, K), us) if M > 16
                                 else _checks.roofline_hbm(gemm.algorithmic_bytes(M, N, K), us))
            if M > 16 and not args.no_cublaslt:
                try:
                    D2 = torch.empty_like(D)
                    lt = lambda: _native.nvfp4_gemm_cublaslt(A_fp4, B_fp4, A_sf, B_sf, float(alpha), D2, M, N, K)
                    us_lt = _bench_us(lt, reps=20)
                    entry["cublaslt_us"] = us_lt
                    entry["cublaslt_rel_fro"] = gemm.relative_frobenius_error(D, D2)
                except Exception as error:  # the library peer is optional
                    entry["cublaslt_error"] = str(error)[:200]
            out[f"nvfp4_gemm_{M}x{N}x{K}"] = entry
            del A_fp4, B_fp4, A_sf, B_sf, D
    out["ffn_gate_up_tp"] = ffn_sharded(rank, world, distributed)
    return out


def gemm_role_timers(launch, K: int, us: float) -> dict:
    """In-kernel role timers of one more launch (CTA 0): where the MMA role's time goes per 256-wide K slab
    and per tile, the SM clock the kernel saw, and the launch time normalised by that clock (the GEMM runs
    under the power cap: a slower clock and a slower kernel are told apart by `us_x_sm_ghz`)."""
    import ctypes

    import torch

    from tirx_kernels import _native

    lib = _native.lib()
    _native.check(lib.b2_nvfp4_gemm_role_timers(1, None, None), "b2_nvfp4_gemm_role_timers")
    launch()
    torch.cuda.synchronize()
    out = (ctypes.c_ulonglong * 12)()
    _native.check(lib.b2_nvfp4_gemm_role_timers(0, out, None), "b2_nvfp4_gemm_role_timers")
    t = [int(v) for v in out]
    tiles, slabs = max(t[8], 1), max(t[8], 1) * (K // 256)
    ghz = t[4] / max(t[11], 1)
    return {"role_timers_cta0": {
        "tiles": t[8], "cycles_per_k_slab": round(t[4] / slabs, 1),
        "mma_issue_cycles_per_k_slab": round(t[5] / slabs, 1),
        "mma_wait_for_operands_and_scales_per_k_slab": round(t[2] / slabs, 1),
        "mma_wait_for_drained_accumulator_per_tile": round(t[3] / tiles, 1),
        "epilogue_body_cycles_per_tile": round(t[7] / tiles, 1),
        "tensor_cycles_needed_per_k_slab": 512, "sm_ghz_in_kernel": round(ghz, 3)},
        "us_x_sm_ghz": round(us * ghz, 1)}


def ffn_sharded(rank: int, world: int, distributed: bool, M: int = 8192, N: int = 28672, K: int = 8192) -> dict:
    """Llama-3-70B gate/up projection sharded by weight columns: every rank quantizes the full
    activation, multiplies by its N/world shard, then an NCCL all-gather assembles the bf16 output
    as [world, M, N/world] (strong scaling; times are the max over ranks)."""
    import torch

    from tirx_kernels import _checks, _native
    from tirx_kernels.basic import nvfp4_gemm as gemm

    from tirx_kernels.basic import ffn_tp

    start, stop = ffn_tp.shard_rows(N, world, rank)
    shard = stop - start
    g = torch.Generator(device="cuda").manual_seed(1000 + rank)
    act = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, generator=torch.Generator(device="cuda").manual_seed(0))
    w = (0.02 * torch.randn(shard, K, device="cuda", dtype=torch.float32, generator=g)).to(torch.bfloat16)
    w_amax = w.float().abs().max().reshape(1)
    if distributed:
        torch.distributed.all_reduce(w_amax, op=torch.distributed.ReduceOp.MAX)
    w_gs = 2688.0 / w_amax
    B_fp4, B_sf = gemm.quantize_operand(w, w_gs)  # offline weight quantization, untimed
    del w
    a_gs = (2688.0 / act.float().abs().max()).reshape(1)
    alpha_t = (1.0 / (a_gs * w_gs)).reshape(1).float()
    A_fp4 = torch.empty(M, K // 2, dtype=torch.uint8, device="cuda")
    A_sf = torch.empty(M * K // 16, dtype=torch.uint8, device="cuda")
    D = torch.empty(M, shard, dtype=torch.bfloat16, device="cuda")
    gathered = torch.empty(world, M, shard, dtype=torch.bfloat16, device="cuda") if distributed else None
    exg = gemm._compile_executable(M, shard, K)

    def quantize(x=act):
        _native.nvfp4_quantize(x, A_fp4, A_sf, a_gs, M, K, "bfloat16", "128x4")
        return A_fp4, A_sf

    def matmul(a=A_fp4, a_sf=A_sf, b=B_fp4, b_sf=B_sf, al=alpha_t, out=D):
        exg(a, b, a_sf, b_sf, al, out)

    def gather():
        if distributed:
            torch.distributed.all_gather_into_tensor(gathered.view(-1), D.view(-1))

    projection = ffn_tp.ShardedProjection(world, rank, M, N, K, B_fp4, B_sf, alpha_t, quantize,
                                          lambda a, a_sf, b, b_sf, al, out: exg(a, b, a_sf, b_sf, al, out))

    def whole():
        projection.forward(act, D, gathered)

    def phase_us(fn, reps=10):
        ms = timed_region(fn, reps, 3, distributed)
        return ms / reps * 1e3

    t_q, t_g = phase_us(quantize), phase_us(matmul)
    t_ag = phase_us(gather) if distributed else 0.0
    t_all = phase_us(whole)
    _native.nvfp4_gemm_status()

    # fused path: the GEMM epilogue stores every tile into all GPUs' [M, N] buffers over NVLink; two buffer
    # sets alternate so that one barrier per step is enough
    fused = {}
    if distributed:
        sets = [ffn_tp.PeerOutputBuffers(M, N, world, rank) for _ in range(2)]
        turn = [0]

        def fused_gemm():
            buf = sets[turn[0] & 1]
            turn[0] += 1
            _native.nvfp4_gemm_allgather(A_fp4, B_fp4, A_sf, B_sf, alpha_t, buf.addresses, rank, M, shard, K)
            torch.distributed.all_reduce(token)

        def fused_whole():
            buf = sets[turn[0] & 1]
            turn[0] += 1
            ffn_tp.fused_forward(projection, act, buf)

        token = torch.zeros(1, device="cuda")
        whole()
        turn[0] = 0
        fused_whole()
        torch.cuda.synchronize()
        torch.distributed.barrier()
        identical = bool(torch.equal(sets[0].local, ffn_tp.assemble(gathered)))
        t_fg, t_fall = phase_us(fused_gemm), phase_us(fused_whole)
        _native.nvfp4_gemm_status()
        fused = {
            "fused_gemm_allgather_us": t_fg, "fused_step_us": t_fall,
            "fused_equals_nccl_path": identical,
            "fused_total_tflops": gemm.flops(M, N, K) / t_fall / 1e6,
            "fused_send_gbs": (world - 1) * M * shard * 2 / t_fg / 1e3,
        }
        torch.cuda.synchronize()
        torch.distributed.barrier()
        for buf in sets:
            buf.close()
    result = {
        "M": M, "N": N, "K": K, "world": world, "shard_n": shard,
        "quantize_us": t_q, "gemm_us": t_g, "allgather_us": t_ag, "step_us": t_all,
        "gemm_tflops_per_gpu": gemm.flops(M, shard, K) / t_g / 1e6,
        "gemm_roofline": _checks.roofline_nvfp4(gemm.flops(M, shard, K), t_g),
        "quantize_roofline": _checks.roofline_hbm(M * K * 2 + M * K // 2 + M * K // 16 + 4, t_q),
        "total_tflops": gemm.flops(M, N, K) / t_all / 1e6, "scaling": "strong",
    }
    result.update(fused)
    if distributed:
        received = (world - 1) * M * shard * 2
        result["allgather_recv_gbs"] = received / t_ag / 1e3
        result["allgather_frac_of_770gbs_peer_copy"] = result["allgather_recv_gbs"] / 770.0
        # the unsharded projection on one GPU of this very box (rank 0; the others wait): the denominator
        # of every strong-scaling figure below
        single = torch.zeros(3, dtype=torch.float64, device="cuda")
        if rank == 0:
            gw = torch.Generator(device="cuda").manual_seed(1000)
            w_full = (0.02 * torch.randn(N, K, device="cuda", dtype=torch.float32, generator=gw)).to(torch.bfloat16)
            Bf, Bs = gemm.quantize_operand(w_full, 2688.0 / w_full.float().abs().max().reshape(1))
            del w_full
            Df = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            exf = gemm._compile_executable(M, N, K)

            def full_step():
                quantize()
                exf(A_fp4, Bf, A_sf, Bs, alpha_t, Df)

            single[0] = timed_region(lambda: exf(A_fp4, Bf, A_sf, Bs, alpha_t, Df), 10, 3, False) / 10 * 1e3
            single[1] = timed_region(full_step, 10, 3, False) / 10 * 1e3
            single[2] = timed_region(quantize, 10, 3, False) / 10 * 1e3
            _native.nvfp4_gemm_status()
            del Bf, Bs, Df
        torch.distributed.barrier()
        torch.distributed.broadcast(single, src=0)
        g1, s1, q1 = (float(v) for v in single)
        # what the exchange allows: every GPU must receive (world-1)/world of the bf16 output over NVLink, at
        # best at the peer-copy rate measured on this pool (770 GB/s per direction), hidden behind the GEMM
        exchange_us = received / 770.0 / 1e3
        bound_step = q1 + max(g1 / world, exchange_us)
        result["single_gpu"] = {"gemm_us": g1, "step_us": s1, "quantize_us": q1}
        result["scaling_summary"] = {
            "gpus": world,
            "nccl_path": {"step_us": t_all, "speedup_vs_1gpu": s1 / t_all, "of_linear": s1 / t_all / world},
            "fused_path": {"step_us": t_fall, "speedup_vs_1gpu": s1 / t_fall, "of_linear": s1 / t_fall / world},
            "gemm_phase_of_linear": g1 / t_g / world,
            "bound_at_measured_peer_copy": {"exchange_us": exchange_us, "step_us": bound_step,
                                            "speedup_vs_1gpu": s1 / bound_step},
            "fused_step_over_bound": t_fall / bound_step,
        }
    return result


# ---- reference arm ------------------------------------------------------------------------------------------
def run_reference(args) -> dict:
    """The reference's arithmetic on the host cores (C restatement with OpenMP): one step = one full batch."""
    rank, _, world = rank_env()
    if rank != 0:
        return {}
    x_host, gs_host = headline_input(HEADLINE["m"], HEADLINE["k"])
    base = cpu_baseline(x_host, float(gs_host.item()), HEADLINE["sf_layout"], budget_s=0.0,
                        steps=args.steps + args.warmup)
    return {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 scale math on bf16 input, e2m1/e4m3 output",
        "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "note": "the reference's GPU kernels need the TIRx compiler (tvm.tirx), absent here; this is "
                           "the CPU restatement of its arithmetic on the host cores, rank 0 only"},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--no-extra", action="store_true", help="headline only")
    parser.add_argument("--no-cublaslt", action="store_true", help="do not time the cuBLASLt NVFP4 peer")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    line = run_reference(args) if args.impl == "reference" else run_ours(args)
    if line:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
