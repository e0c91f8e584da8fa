"""Test and benchmark runner for the kernel modules.

Keeps the public surface of the reference's tirx_kernels/runner.py that the hot path
uses - ``run_kernel_test`` (:744-761), ``run_kernel_bench`` (:764-798), the two-stage
``prepare_kernel_bench`` / ``run_prepared_kernel_bench`` split (:801-867),
``prepared_gpu_benchmark`` (:98-114), ``bench`` (:492-519), ``compile_kernel`` (:735-741),
``hardware_num_sms`` (:320-334) - and drops everything that only exists to drive TVM.

Timing.  The reference delegates to ``tvm.tirx.bench.bench`` (Proton by default).  Here
``bench`` times with CUDA events on the current stream after a warm-up budget.  Timer
``event`` (default) brackets every launch with its own pair of events and reads a 256 MiB
buffer before it, so each launch starts with a cold, clean L2 - the conditions of the
reference's protocol (25 ms warm-up, 100 ms repeat, 5 rounds, mean); launches of a few
microseconds also carry the host's launch latency in this mode.  Timer ``event_warm`` times
back-to-back launches between one pair of events.  Timers ``proton`` (cold L2, as ``event``) and
``cudagraph_proton`` (launches replayed from a CUDA graph, warm L2) report pure kernel time from
``triton.profiler``, the reference's default protocol.

Late GPU assignment (``bind_cuda_assignment`` and friends, reference :347-449, :522-558)
serves the bench suite's prepared-child protocol, see ``bench/_prepared_child.py``.
"""

from __future__ import annotations

import os
import statistics
import time
from collections.abc import Callable, Mapping
from dataclasses import dataclass, field
from types import ModuleType
from typing import Sequence, Any, Protocol, runtime_checkable

DEFAULT_BENCH_ROUNDS = 5
DEFAULT_BENCH_COOLDOWN_S = 0.0
DEFAULT_WARMUP_MS = 25
DEFAULT_REPEAT_MS = 100
PREPARE_NUM_SMS_ENV = "TIRX_PREPARE_NUM_SMS"
PREPARE_CUDA_ARCH_ENV = "TIRX_PREPARE_CUDA_ARCH"
_EXTERNAL_REFERENCES_ENV = "TIRX_INTERNAL_BENCH_REFERENCES"
L2_FLUSH_BYTES = 256 * 1024 * 1024
SUPPORTED_TIMERS = ("event", "event_warm", "proton", "cudagraph_proton")


# ---- external references (library peers timed beside our kernels) -------------------------
def set_external_references_enabled(enabled: bool) -> None:
    if not isinstance(enabled, bool):
        raise TypeError("external reference mode must be a bool")
    os.environ[_EXTERNAL_REFERENCES_ENV] = "1" if enabled else "0"


def external_references_enabled() -> bool:
    return os.environ.get(_EXTERNAL_REFERENCES_ENV) == "1"


# ---- expected-value provider ----------------------------------------------------------------
# The reference's run_test compares with a third-party GPU kernel at test time.  This package
# ships no expected-value generator of its own: a test harness installs one here (the
# repository's tests install the CPU oracle); without one, run_test applies the reference's
# self-contained checks only.
_REFERENCE_PROVIDER: Callable[..., Any] | None = None


def set_reference_provider(provider: Callable[..., Any] | None) -> None:
    global _REFERENCE_PROVIDER
    _REFERENCE_PROVIDER = provider


def reference_provider() -> Callable[..., Any] | None:
    return _REFERENCE_PROVIDER


# ---- prepared benchmarks ------------------------------------------------------------------------
@runtime_checkable
class PreparedBenchmark(Protocol):
    def run_gpu(self, **kwargs: Any) -> dict[str, Any]: ...


@dataclass(frozen=True)
class ExplicitPreparedBenchmark:
    """Kernel-owned state prepared on the CPU and consumed by the GPU stage of the same process."""

    run_gpu_fn: Callable[..., dict[str, Any]]
    state: Any
    required_num_gpus: int = 1
    close_fn: Callable[[], None] | None = None
    owner_pid: int = field(default_factory=os.getpid, init=False, repr=False)

    def _check_owner(self) -> None:
        if os.getpid() != self.owner_pid:
            raise RuntimeError(
                f"prepared benchmark is process-local: created in PID {self.owner_pid}, "
                f"used in PID {os.getpid()}"
            )

    def __reduce_ex__(self, protocol: int):
        raise TypeError("prepared benchmarks cannot be serialized across processes")

    def run_gpu(self, **kwargs: Any) -> dict[str, Any]:
        self._check_owner()
        return self.run_gpu_fn(self.state, **kwargs)

    def close(self) -> None:
        self._check_owner()
        if self.close_fn is not None:
            self.close_fn()


def prepared_gpu_benchmark(run_gpu: Callable[..., dict[str, Any]], state: Any, *,
                           required_num_gpus: int = 1,
                           close: Callable[[], None] | None = None) -> ExplicitPreparedBenchmark:
    if not callable(run_gpu):
        raise TypeError("run_gpu must be callable")
    if isinstance(required_num_gpus, bool) or not isinstance(required_num_gpus, int):
        raise TypeError("required_num_gpus must be an integer")
    if required_num_gpus < 1:
        raise ValueError("required_num_gpus must be positive")
    if close is not None and not callable(close):
        raise TypeError("close must be callable")
    return ExplicitPreparedBenchmark(run_gpu, state, required_num_gpus, close)


@dataclass(frozen=True)
class PreparedKernelBenchmark:
    kernel: str
    label: str
    benchmark: Any
    owner_pid: int = field(default_factory=os.getpid, init=False, repr=False)

    def assert_process_local(self) -> None:
        if os.getpid() != self.owner_pid:
            raise RuntimeError("prepared kernel benchmark used outside its preparing process")

    @property
    def required_num_gpus(self) -> int:
        return int(getattr(self.benchmark, "required_num_gpus", 1))


# ---- late GPU assignment (the bench suite hands a prepared child its GPU after CPU prepare) ---------
_ASSIGNMENT: tuple[tuple[int, ...], tuple[str, ...]] | None = None


def cuda_is_initialized() -> bool:
    """True once this process has created a CUDA context through torch (reference runner.py:313-317)."""
    import sys

    torch = sys.modules.get("torch")
    return bool(torch is not None and torch.cuda.is_initialized())


def canonical_cuda_uuid(value: Any) -> str:
    text = value.decode() if isinstance(value, bytes) else str(value)
    text = text.strip().lower()
    return text[4:] if text.startswith("gpu-") else text


def physical_cuda_uuids(device_indices: Sequence[int]) -> tuple[str, ...]:
    """UUIDs of the given visible device indices, as the driver reports them (reference :347-381)."""
    import torch

    return tuple(canonical_cuda_uuid(torch.cuda.get_device_properties(int(i)).uuid) for i in device_indices)


def bind_cuda_assignment(device_indices: Sequence[int], expected_uuids: Sequence[str]) -> tuple[str, ...]:
    """Select the late-bound device and prove it is the card the scheduler meant (reference :384-409)."""
    global _ASSIGNMENT
    indices = tuple(int(i) for i in device_indices)
    expected = tuple(canonical_cuda_uuid(u) for u in expected_uuids)
    if not indices or len(indices) != len(expected) or len(set(indices)) != len(indices):
        raise ValueError(f"invalid CUDA assignment indices={device_indices!r}, uuids={expected_uuids!r}")
    import torch

    torch.cuda.set_device(indices[0])
    actual = physical_cuda_uuids(indices)
    if actual != expected:
        raise RuntimeError(f"late GPU assignment identity mismatch: requested {list(expected)}, "
                           f"physical {list(actual)}")
    _ASSIGNMENT = (indices, actual)
    return actual


def current_cuda_assignment() -> tuple[tuple[int, ...], tuple[str, ...]]:
    if _ASSIGNMENT is None:
        raise RuntimeError("no CUDA assignment is active in this process")
    return _ASSIGNMENT


def current_process_cuda_memory_bytes(device_indices: Sequence[int]) -> dict[int, int | None]:
    """Device memory this process still holds on each card, from NVML; None where it cannot be read
    (reference :522-558).  The scheduler uses it to decide whether a card can be handed on."""
    result: dict[int, int | None] = {int(i): None for i in device_indices}
    try:
        import pynvml
        import torch

        pynvml.nvmlInit()
        for index in result:
            uuid = torch.cuda.get_device_properties(index).uuid
            handle = pynvml.nvmlDeviceGetHandleByUUID(f"GPU-{canonical_cuda_uuid(uuid)}".encode())
            used = 0
            for proc in pynvml.nvmlDeviceGetComputeRunningProcesses(handle):
                if proc.pid == os.getpid():
                    used = int(proc.usedGpuMemory or 0)
            result[index] = used
    except Exception:
        pass
    return result


# ---- device facts -------------------------------------------------------------------------------
def hardware_num_sms(default: int = 148) -> int:
    """SM count for launch math: env override, then the live device, then the B200 value."""
    configured = os.environ.get(PREPARE_NUM_SMS_ENV)
    if configured is not None:
        value = int(configured)
        if value < 1:
            raise ValueError(f"{PREPARE_NUM_SMS_ENV} must be positive, got {value}")
        return value
    import sys

    torch = sys.modules.get("torch")
    if torch is not None and torch.cuda.is_available() and torch.cuda.is_initialized():
        return int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    return default


def compile_kernel(handle, *, arch: str | None = None, cuda_compile_mode: str | None = None):
    """Resolve a module's `get_kernel` handle into its launchable executable.

    The kernels are compiled ahead of time into the C-ABI library, so "compiling" binds the
    handle's launcher and proves the library loads; `arch` other than sm_100a is rejected.
    """
    if arch not in (None, "sm_100a"):
        raise ValueError(f"this build targets sm_100a only, got arch={arch!r}")
    from tirx_kernels import _native

    _native.lib()
    launcher = handle.config.get("launcher")
    if launcher is None:
        raise TypeError(f"kernel handle {handle.symbol!r} carries no launcher")
    return launcher


# ---- timing -----------------------------------------------------------------------------------------
def _chain_ms(fn, n: int) -> float:
    """Device time per iteration of `n` back-to-back launches inside one pair of CUDA events."""
    import torch

    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(n):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / n


def _cold_ms(fn, n: int, flush) -> float:
    """Mean device time of `n` launches, each preceded by an L2 flush and bracketed by its own pair
    of events.  The flush READS a buffer larger than L2: a write would leave dirty lines whose
    write-back the timed kernel then pays for.  (Timing [flush, fn] chains and subtracting the flush
    alone is biased: back-to-back flushes partly hit in L2 and run faster than interleaved ones.)"""
    import torch

    pairs = []
    for _ in range(n):
        flush.sum()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        pairs.append((start, end))
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in pairs) / n


def _time_one(fn: Callable[[], Any], warmup_ms: float, repeat_ms: float, flush) -> float:
    """Mean device time of one launch of `fn` in microseconds (warm: back-to-back launches between
    one pair of events; cold: see `_cold_ms`)."""
    import torch

    fn()
    torch.cuda.synchronize()
    estimate_ms = max(_chain_ms(fn, 5), 1e-3)
    n_warmup = max(3, int(warmup_ms / estimate_ms))
    n_repeat = max(10, min(2000, int(repeat_ms / estimate_ms)))
    _chain_ms(fn, n_warmup)
    if flush is None:
        return _chain_ms(fn, n_repeat) * 1e3
    return _cold_ms(fn, min(n_repeat, 500), flush) * 1e3


def _hatchet_kernel_ns(node, inside: bool, scope_name: str) -> float:
    """Sum of the kernel times (ns) recorded below the scope `scope_name` in a Proton profile tree."""
    frame = node.get("frame", {})
    inside = inside or frame.get("name") == scope_name
    total = 0.0
    children = node.get("children", [])
    if inside and not children:
        total += float(node.get("metrics", {}).get("time (ns)", 0.0))
    for child in children:
        total += _hatchet_kernel_ns(child, inside, scope_name)
    return total


def _proton_us(fn: Callable[[], Any], n: int, flush, graph: bool) -> float:
    """Mean kernel time of one launch of `fn` in microseconds as Proton (triton.profiler, CUPTI activity
    records) sees it: pure device time of the kernels `fn` launches, no launch gaps and no host cost -
    the protocol of the reference's `tvm.tirx.bench` (`proton`, and `cudagraph_proton`, which replays the
    launches from a CUDA graph).  The L2 flush runs in a scope of its own and is not counted."""
    import json
    import tempfile

    import torch

    try:
        import triton.profiler as proton
    except Exception as error:
        raise RuntimeError(f"timer 'proton' needs triton.profiler: {type(error).__name__}: {error}") from error
    replay = None
    if graph:
        stream = torch.cuda.Stream()
        cuda_graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            with torch.cuda.graph(cuda_graph, stream=stream):
                fn()
        replay = cuda_graph.replay
    launch = replay or fn
    with tempfile.TemporaryDirectory() as folder:
        base = os.path.join(folder, "b2_proton")
        proton.start(base, context="shadow", data="tree", backend="cupti")
        try:
            for _ in range(n):
                if flush is not None:
                    with proton.scope("b2_flush"):  # recorded, but only the kernels below "b2_timed" are summed
                        flush.sum()
                with proton.scope("b2_timed"):
                    launch()
            torch.cuda.synchronize()
        finally:
            proton.finalize()
        with open(base + ".hatchet") as handle:
            tree = json.load(handle)
    roots = tree if isinstance(tree, list) else [tree]
    total_ns = sum(_hatchet_kernel_ns(root, False, "b2_timed") for root in roots)
    if total_ns <= 0.0:
        raise RuntimeError("Proton recorded no kernel time (CUPTI activity records unavailable on this machine?)")
    return total_ns / n / 1e3


def bench(funcs: Mapping[str, Callable[[], Any]], *, references: Mapping[str, Callable[[], Any]] | None = None,
          warmup: int | None = None, repeat: int | None = None, timer: str | None = None,
          rounds: int | None = None, cooldown_s: float | None = None, **_ignored: Any) -> dict[str, Any]:
    """Time each launch closure; reference builders run only when references are enabled.

    Returns the reference's record shape: ``impls`` (name -> mean microseconds over rounds),
    ``round_samples``, ``errors``, ``timer`` and ``benchmark_protocol``.
    """
    import torch

    timer = timer or "event"
    if timer not in SUPPORTED_TIMERS:
        raise ValueError(f"timer {timer!r} is not provided by this build; choose one of {SUPPORTED_TIMERS}")
    warmup_ms = DEFAULT_WARMUP_MS if warmup is None else warmup
    repeat_ms = DEFAULT_REPEAT_MS if repeat is None else repeat
    rounds = DEFAULT_BENCH_ROUNDS if rounds is None else rounds
    cooldown_s = DEFAULT_BENCH_COOLDOWN_S if cooldown_s is None else cooldown_s

    launches: dict[str, Callable[[], Any]] = dict(funcs)
    errors: dict[str, str] = {}
    if references and external_references_enabled():
        for name, builder in references.items():
            try:
                launches[name] = builder()
            except Exception as error:  # a broken peer must not hide our own number
                errors[name] = f"{type(error).__name__}: {error}"
    flush = None
    if timer in ("event", "proton"):
        flush = torch.zeros(L2_FLUSH_BYTES // 8, dtype=torch.int64, device="cuda")
    samples: dict[str, list[float]] = {name: [] for name in launches}
    for _ in range(rounds):
        for name, fn in launches.items():
            if cooldown_s:
                time.sleep(cooldown_s)
            if timer in ("proton", "cudagraph_proton"):
                fn()
                torch.cuda.synchronize()
                estimate_ms = max(_chain_ms(fn, 5), 1e-3)
                _chain_ms(fn, max(3, int(warmup_ms / estimate_ms)))
                n_repeat = max(10, min(200, int(repeat_ms / estimate_ms)))
                samples[name].append(_proton_us(fn, n_repeat, flush, graph=timer == "cudagraph_proton"))
            else:
                samples[name].append(_time_one(fn, warmup_ms, repeat_ms, flush))
    return {
        "impls": {name: statistics.fmean(values) for name, values in samples.items()},
        "round_samples": samples,
        "errors": errors,
        "timer": timer,
        "benchmark_protocol": {
            "warmup": warmup_ms,
            "repeat": repeat_ms,
            "cooldown_s": cooldown_s,
            "rounds": rounds,
            "round_aggregate": "mean",
            "order": list(launches),
            "l2": "flushed before every timed launch" if flush is not None else "warm",
        },
    }


# ---- test / bench drivers -----------------------------------------------------------------------------
def _params(config: dict[str, Any]) -> dict[str, Any]:
    return {key: value for key, value in config.items() if key != "label"}


def run_kernel_test(kernel_name: str, config: dict[str, Any], *, registry=None) -> None:
    """Run one correctness config through the module's ``run_test``."""
    if registry is None:
        from tirx_kernels.registry import discover_kernels

        registry = discover_kernels()
    module = registry[kernel_name]
    params = _params(config)
    module.get_kernel(**params)  # the reference validates the kernel object first; ours validates the config
    module.run_test(**params)


def prepare_kernel_bench(kernel_name: str, config: dict[str, Any], *, module: ModuleType | None = None,
                         require_cuda_uninitialized: bool = True) -> PreparedKernelBenchmark:
    if module is None:
        from tirx_kernels.registry import load_kernel

        module = load_kernel(kernel_name, strict=True)
    if require_cuda_uninitialized:
        import sys

        torch = sys.modules.get("torch")
        if torch is not None and torch.cuda.is_initialized():
            raise RuntimeError("CPU prepare requires a process with CUDA still uninitialized")
    prepare = getattr(module, "prepare_bench", None)
    if prepare is None:
        raise TypeError(f"kernel {kernel_name!r} module {module.__name__!r} has no prepare_bench()")
    benchmark = prepare(**_params(config))
    if not isinstance(benchmark, PreparedBenchmark):
        raise TypeError(f"kernel {kernel_name!r} prepare_bench() must return an object with run_gpu()")
    return PreparedKernelBenchmark(kernel_name, config.get("label", "default"), benchmark)


def run_prepared_kernel_bench(prepared: PreparedKernelBenchmark, *, warmup: int | None = None,
                              repeat: int | None = None, timer: str | None = None,
                              rounds: int | None = None, cooldown: float | None = None) -> dict[str, Any]:
    prepared.assert_process_local()
    given = {"warmup": warmup, "repeat": repeat, "timer": timer, "rounds": rounds, "cooldown_s": cooldown}
    result = prepared.benchmark.run_gpu(**{k: v for k, v in given.items() if v is not None})
    if not isinstance(result, dict):
        result = {}
    result.setdefault("kernel", prepared.kernel)
    result.setdefault("label", prepared.label)
    return result


def close_prepared_kernel_bench(prepared: PreparedKernelBenchmark) -> None:
    prepared.assert_process_local()
    close = getattr(prepared.benchmark, "close", None)
    if close is not None:
        close()


def run_kernel_bench(kernel_name: str, config: dict[str, Any], *, registry=None, warmup: int | None = None,
                     repeat: int | None = None, timer: str | None = None, rounds: int | None = None,
                     cooldown: float | None = None) -> dict[str, Any]:
    module = None if registry is None else registry[kernel_name]
    prepared = prepare_kernel_bench(kernel_name, config, module=module, require_cuda_uninitialized=False)
    try:
        return run_prepared_kernel_bench(prepared, warmup=warmup, repeat=repeat, timer=timer,
                                         rounds=rounds, cooldown=cooldown)
    finally:
        close_prepared_kernel_bench(prepared)
