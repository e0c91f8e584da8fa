"""Prepared-child side of the bench suite's control protocol.

The reference's bench suite starts one child per workload with ``python -m tirx_kernels.bench
--prepared-control-fd FD --prepared-num-gpus N --kernel K --config C``, lets it do all CPU work
first and assigns a GPU late (tirx_kernels/bench/__main__.py:101-354).  Messages are JSON
objects, one per line, over the inherited socket:

    child -> parent   READY {timestamps, required_num_gpus}        CPU prepare finished, no CUDA yet
                      FAIL {phase: prepare|gpu|protocol, error, traceback}
                      RUNNING_GPU {gpu_attempt, gpu_started, physical_gpu_uuids, ...}
                      RESULT_READY {gpu_attempt, gpu_finished, resident_context_bytes_after_cleanup, result}
                      INTERFERED {gpu_attempt, ...}                 SIGUSR1 arrived during the GPU stage
    parent -> child   ASSIGN {gpu_indices, gpu_uuids} | CANCEL      after READY / INTERFERED
                      ACCEPT_RESULT | RETRY_GPU | CANCEL            after RESULT_READY

The kernels here are compiled ahead of time, so "CPU prepare" loads the module, resolves the
config, binds the launcher and proves the C-ABI library loads - all without creating a CUDA context.
"""

from __future__ import annotations

import gc
import json
import signal
import socket
import sys
import time
import traceback
from unittest import SkipTest


class GpuAttemptInterrupted(BaseException):
    """Raised out of the GPU stage when the scheduler signals interference (SIGUSR1)."""


def send(control: socket.socket, message: dict) -> None:
    control.sendall(json.dumps(message, separators=(",", ":")).encode() + b"\n")


def validated_assignment(gpu_indices, gpu_uuids, required: int) -> list[int]:
    if not isinstance(gpu_indices, list) or len(gpu_indices) != required:
        raise ValueError(f"invalid GPU assignment: {gpu_indices!r}")
    names = [str(index) for index in gpu_indices]
    if len(set(names)) != len(names):
        raise ValueError(f"GPU assignment contains duplicates: {gpu_indices!r}")
    if any(not name.isdigit() for name in names):
        raise ValueError(f"GPU assignment contains an invalid physical index: {gpu_indices!r}")
    if not isinstance(gpu_uuids, list) or len(gpu_uuids) != required:
        raise ValueError(f"invalid physical GPU UUID assignment: {gpu_uuids!r}")
    return [int(name) for name in names]


def _release_device_memory() -> None:
    torch = sys.modules.get("torch")
    if torch is not None and torch.cuda.is_initialized():
        try:
            torch.cuda.synchronize()
        except Exception:
            pass
        gc.collect()
        torch.cuda.empty_cache()


def run(args, find_config, *, child_started: float) -> int:
    """Serve one prepared child until its result is accepted, it is cancelled, or it fails."""
    control = socket.socket(fileno=args.prepared_control_fd)
    reader = control.makefile("r", encoding="utf-8")
    prepared = None
    runner = None
    try:
        # ---- CPU prepare -----------------------------------------------------------------------------
        try:
            import_started = time.time()
            from tirx_kernels import runner
            from tirx_kernels.registry import load_kernel

            framework_loaded = time.time()
            rounds = runner.DEFAULT_BENCH_ROUNDS if args.rounds is None else args.rounds
            cooldown = runner.DEFAULT_BENCH_COOLDOWN_S if args.cooldown is None else args.cooldown
            if rounds < 1:
                raise ValueError("--rounds must be >= 1")
            if cooldown < 0:
                raise ValueError("--cooldown must be >= 0")
            if not args.kernel or not args.config:
                raise ValueError("prepared child requires --kernel and --config")
            if runner.cuda_is_initialized():
                raise RuntimeError("CUDA was initialized before CPU prepare")
            module = load_kernel(args.kernel, strict=True)
            module_loaded = time.time()
            config = find_config(module, args.config)
            config_resolved = time.time()
            prepared = runner.prepare_kernel_bench(args.kernel, config, module=module,
                                                   require_cuda_uninitialized=True)
            if prepared.required_num_gpus != args.prepared_num_gpus:
                raise ValueError(f"workload declares num_gpus={args.prepared_num_gpus}, but prepared "
                                 f"benchmark requires {prepared.required_num_gpus}")
            if runner.cuda_is_initialized():
                raise RuntimeError("CPU prepare created a CUDA context")
            send(control, {"type": "READY", "child_started": child_started, "prepare_started": child_started,
                           "framework_import_started": import_started, "framework_loaded": framework_loaded,
                           "module_loaded": module_loaded, "config_resolved": config_resolved,
                           "ready": time.time(), "required_num_gpus": prepared.required_num_gpus})
        except BaseException as error:
            send(control, {"type": "FAIL", "phase": "prepare", "error": f"{type(error).__name__}: {error}",
                           "traceback": traceback.format_exc()})
            return 1

        def on_interference(_signum, _frame):
            raise GpuAttemptInterrupted()

        # ---- GPU stage, possibly several attempts -----------------------------------------------------
        attempt, abandoned = 1, []
        while True:
            line = reader.readline()
            if not line:
                return 1
            command = json.loads(line)
            if command.get("type") == "CANCEL":
                return 0
            if command.get("type") != "ASSIGN":
                raise ValueError(f"expected ASSIGN or CANCEL, got {command!r}")
            indices = validated_assignment(command.get("gpu_indices"), command.get("gpu_uuids"),
                                           args.prepared_num_gpus)
            if attempt == 1 and runner.cuda_is_initialized():
                raise RuntimeError("CUDA was initialized before late GPU assignment")
            previous = signal.signal(signal.SIGUSR1, on_interference)
            started = None
            try:
                uuids = list(runner.bind_cuda_assignment(indices, command["gpu_uuids"]))
                leftover = runner.current_process_cuda_memory_bytes(abandoned)
                started = time.time()
                send(control, {"type": "RUNNING_GPU", "gpu_attempt": attempt, "gpu_started": started,
                               "physical_gpu_uuids": uuids,
                               "abandoned_gpu_resident_bytes_after_reassignment": {str(k): v for k, v in leftover.items()}})
                try:
                    result = runner.run_prepared_kernel_bench(prepared, warmup=args.warmup, repeat=args.repeat,
                                                              timer=args.timer, rounds=rounds, cooldown=cooldown)
                except SkipTest as skipped:
                    result = {"kernel": args.kernel, "label": args.config, "status": "SKIP", "reason": str(skipped)}
                # a result is proposed only after all device work is done and cached memory is returned
                signal.signal(signal.SIGUSR1, signal.SIG_IGN)
                _release_device_memory()
                resident = runner.current_process_cuda_memory_bytes(indices)
                result["retry_in_place"] = attempt > 1
                send(control, {"type": "RESULT_READY", "gpu_attempt": attempt, "gpu_finished": time.time(),
                               "resident_context_bytes_after_cleanup": {str(k): v for k, v in resident.items()},
                               "result": result})
                decision = reader.readline()
                if not decision:
                    return 1
                verdict = json.loads(decision).get("type")
                if verdict in ("ACCEPT_RESULT", "CANCEL"):
                    return 0
                if verdict != "RETRY_GPU":
                    raise ValueError(f"expected ACCEPT_RESULT, RETRY_GPU, or CANCEL, got {verdict!r}")
            except GpuAttemptInterrupted:
                signal.signal(signal.SIGUSR1, signal.SIG_IGN)
                _release_device_memory()
                resident = runner.current_process_cuda_memory_bytes(indices)
                send(control, {"type": "INTERFERED", "gpu_attempt": attempt, "gpu_started": started,
                               "gpu_finished": time.time(), "physical_gpu_uuids": list(command["gpu_uuids"]),
                               "resident_context_bytes_after_cleanup": {str(k): v for k, v in resident.items()},
                               "descendant_cleanup": {"descendant_pids": [], "forced_kill_pids": []}})
            except BaseException as error:
                send(control, {"type": "FAIL", "phase": "gpu", "gpu_attempt": attempt, "gpu_started": started,
                               "gpu_finished": time.time(), "error": f"{type(error).__name__}: {error}",
                               "traceback": traceback.format_exc()})
                return 1
            finally:
                signal.signal(signal.SIGUSR1, previous)
            abandoned.extend(i for i in indices if i not in abandoned)
            attempt += 1
    except BaseException as error:
        try:
            send(control, {"type": "FAIL", "phase": "protocol", "error": f"{type(error).__name__}: {error}",
                           "traceback": traceback.format_exc()})
        except OSError:
            pass
        return 1
    finally:
        if prepared is not None and runner is not None:
            try:
                runner.close_prepared_kernel_bench(prepared)
            except Exception:
                pass
        reader.close()
        control.close()
