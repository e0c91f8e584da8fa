"""``python -m tirx_kernels.bench``: time registry-owned benchmark configs.

Plain (one-process) mode of the reference CLI (tirx_kernels/bench/__main__.py:357-511):
same flags, ``BENCH_CONFIGS`` preferred over ``CONFIGS`` (:18-19), result file
``{"results": [...]}`` and the human line ``OK kernel [label]: impl=...µs``.  With the hidden flags
``--prepared-control-fd`` / ``--prepared-num-gpus`` the process instead serves the bench suite's
prepared-child protocol (:101-354), implemented in ``_prepared_child.py``.
"""

import argparse
import json
import os
import sys
import traceback
from unittest import SkipTest

TIMER_CHOICES = ("event", "event_warm", "proton", "cudagraph_proton", "kineto", "megamoe", "e2e")


def bench_configs(module) -> list:
    return getattr(module, "BENCH_CONFIGS", getattr(module, "CONFIGS", []))


def find_bench_config(module, label: str) -> dict:
    matches = [c for c in bench_configs(module) if c.get("label") == label]
    if len(matches) != 1:
        raise KeyError(f"kernel {module.KERNEL_META['name']!r} config {label!r}: "
                       f"expected exactly one match, found {len(matches)}")
    return matches[0]


def main() -> None:
    import time

    child_started = time.time()
    parser = argparse.ArgumentParser(description="Run kernel benchmarks")
    parser.add_argument("--kernel", type=str, default=None, help="Run only this kernel")
    parser.add_argument("--config", type=str, default=None, help="Run only this config label")
    parser.add_argument("--json", action="store_true", help="Output JSON results")
    parser.add_argument("--json-file", type=str, default=None, help="Write JSON results to this file")
    parser.add_argument("--cc", type=int, default=None, help="Compute capability filter")
    parser.add_argument("--warmup", type=int, default=None, help="Warm-up budget in ms")
    parser.add_argument("--repeat", type=int, default=None, help="Timed budget in ms")
    parser.add_argument("--timer", type=str, choices=TIMER_CHOICES, default=None,
                        help="'event' (CUDA events, cold L2 per launch; default), 'event_warm', 'proton' (kernel "
                             "time from triton.profiler, cold L2) or 'cudagraph_proton' (the same over CUDA-graph "
                             "replays); the remaining names belong to the reference's TVM timer and are rejected")
    parser.add_argument("--with-references", action="store_true",
                        help="Also time external library peers (cuBLASLt NVFP4)")
    parser.add_argument("--rounds", type=int, default=None, help="Independent timing rounds")
    parser.add_argument("--cooldown", type=float, default=None, help="Seconds slept before every timing")
    parser.add_argument("--prepared-control-fd", type=int, default=None, help=argparse.SUPPRESS)
    parser.add_argument("--prepared-num-gpus", type=int, default=1, help=argparse.SUPPRESS)
    args = parser.parse_args()
    if args.prepared_num_gpus < 1:
        print("ERROR: --prepared-num-gpus must be >= 1", file=sys.stderr)
        sys.exit(2)

    if args.prepared_control_fd is not None:
        from tirx_kernels.bench import _prepared_child
        from tirx_kernels.runner import set_external_references_enabled

        set_external_references_enabled(args.with_references)
        sys.exit(_prepared_child.run(args, find_bench_config, child_started=child_started))

    if args.json or args.json_file:
        os.environ["TIRX_BENCH_JSON"] = "1"

    from tirx_kernels.registry import discover_kernels, load_kernel
    from tirx_kernels.runner import (DEFAULT_BENCH_COOLDOWN_S, DEFAULT_BENCH_ROUNDS, run_kernel_bench,
                                     set_external_references_enabled)

    set_external_references_enabled(args.with_references)
    rounds = DEFAULT_BENCH_ROUNDS if args.rounds is None else args.rounds
    cooldown = DEFAULT_BENCH_COOLDOWN_S if args.cooldown is None else args.cooldown
    if rounds < 1:
        print("ERROR: --rounds must be >= 1", file=sys.stderr)
        sys.exit(2)
    if cooldown < 0:
        print("ERROR: --cooldown must be >= 0", file=sys.stderr)
        sys.exit(2)

    if args.kernel:
        try:
            module = load_kernel(args.kernel)
        except KeyError:
            print(f"ERROR: kernel '{args.kernel}' not found.", file=sys.stderr)
            sys.exit(1)
        if args.cc is not None and module.KERNEL_META.get("compute_capability") != args.cc:
            print(f"ERROR: kernel '{args.kernel}' compute_capability="
                  f"{module.KERNEL_META.get('compute_capability')} != filter {args.cc}", file=sys.stderr)
            sys.exit(1)
        kernels = {args.kernel: module}
    else:
        kernels = discover_kernels(min_compute_capability=args.cc)

    quiet = bool(args.json or args.json_file)
    results = []
    for name in sorted(kernels):
        for config in bench_configs(kernels[name]):
            label = config.get("label", "default")
            if args.config and label != args.config:
                continue
            try:
                results.append(run_kernel_bench(name, config, registry=kernels, warmup=args.warmup,
                                                repeat=args.repeat, timer=args.timer, rounds=rounds,
                                                cooldown=cooldown))
            except SkipTest as skip:
                results.append({"kernel": name, "label": label, "status": "SKIP", "reason": str(skip)})
                if not quiet:
                    print(f"SKIP  {name} [{label}]: {skip}", file=sys.stderr)
            except Exception as error:
                results.append({"kernel": name, "label": label, "status": "FAIL", "error": str(error)})
                if not quiet:
                    print(f"FAIL  {name} [{label}]: {error}", file=sys.stderr)
                    traceback.print_exc(file=sys.stderr)

    if args.json_file:
        with open(args.json_file, "w") as handle:
            json.dump({"results": results}, handle, indent=2)
    elif args.json:
        print(json.dumps({"results": results}, indent=2))
    else:
        for record in results:
            kernel, label = record.get("kernel", "?"), record.get("label", "?")
            status = record.get("status", "ok")
            if status == "FAIL":
                print(f"FAIL  {kernel} [{label}]: {record.get('error', '?')}")
            elif status == "SKIP":
                print(f"SKIP  {kernel} [{label}]: {record.get('reason', '?')}")
            else:
                timings = ", ".join(f"{k}={v:.3f}µs" for k, v in record.get("impls", {}).items())
                extra = record.get("roofline")
                suffix = f"  [{extra['achieved']:.1f} {extra['unit']}, {100 * extra['frac']:.1f}% of peak]" if extra else ""
                print(f"OK    {kernel} [{label}]: {timings}{suffix}")


if __name__ == "__main__":
    main()
