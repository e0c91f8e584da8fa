"""``python -m tirx_kernels.test``: run registry-owned correctness configs.

Same flags, output lines, JSON summary and exit codes as the reference CLI
(tirx_kernels/test/__main__.py:39-116): 0 all passed, 1 a config failed or the kernel is
unknown, 2 no config matched the filters.
"""

import argparse
import json
import sys
import traceback
from unittest import SkipTest

from tirx_kernels.registry import discover_kernels
from tirx_kernels.runner import run_kernel_test


def config_gpu_count(config: dict) -> int:
    """GPUs a config needs: ``world_size`` / ``num_processes`` (must agree), default 1."""
    declared = [config[key] for key in ("world_size", "num_processes") if key in config]
    if len(declared) == 2 and declared[0] != declared[1]:
        raise ValueError(
            f"conflicting config GPU counts: world_size={declared[0]!r}, num_processes={declared[1]!r}"
        )
    count = declared[0] if declared else 1
    if isinstance(count, bool) or not isinstance(count, int) or count < 1:
        raise ValueError(f"invalid config GPU count: {count!r}")
    return count


def select_configs(kernels: dict, *, label=None, num_gpus=None):
    for name in sorted(kernels):
        for config in getattr(kernels[name], "CONFIGS", []):
            if label is not None and config.get("label", "default") != label:
                continue
            if num_gpus is not None and config_gpu_count(config) != num_gpus:
                continue
            yield name, config


def main() -> None:
    parser = argparse.ArgumentParser(description="Run kernel correctness tests")
    parser.add_argument("--kernel", type=str, default=None, help="Run only this kernel")
    parser.add_argument("--config", type=str, default=None, help="Run only this config label")
    parser.add_argument("--json", action="store_true", help="Output JSON results")
    parser.add_argument("--cc", type=int, default=None, help="Compute capability filter")
    parser.add_argument("--num-gpus", type=int, default=None,
                        help="Run only configs requiring this many GPUs (world_size/num_processes, default 1)")
    args = parser.parse_args()
    if args.num_gpus is not None and args.num_gpus < 1:
        parser.error("--num-gpus must be positive")

    kernels = discover_kernels(min_compute_capability=args.cc)
    if args.kernel:
        if args.kernel not in kernels:
            print(f"ERROR: kernel '{args.kernel}' not found. Available: {sorted(kernels)}")
            sys.exit(1)
        kernels = {args.kernel: kernels[args.kernel]}

    results = []
    tally = {"PASS": 0, "FAIL": 0, "SKIP": 0}
    for name, config in select_configs(kernels, label=args.config, num_gpus=args.num_gpus):
        label = config.get("label", "default")
        entry = {"kernel": name, "config": label}
        try:
            run_kernel_test(name, config, registry=kernels)
            entry["status"] = "PASS"
            line = f"PASS  {name} [{label}]"
        except SkipTest as skip:
            entry.update(status="SKIP", reason=str(skip))
            line = f"SKIP  {name} [{label}]: {skip}"
        except Exception as error:
            entry.update(status="FAIL", error=str(error))
            line = f"FAIL  {name} [{label}]: {error}"
            if not args.json:
                traceback.print_exc()
        tally[entry["status"]] += 1
        results.append(entry)
        if not args.json:
            print(line)

    if not results:
        message = "no kernel configs matched the requested filters"
        if args.json:
            print(json.dumps({"passed": 0, "failed": 0, "skipped": 0, "results": [], "error": message}))
        else:
            print(f"ERROR: {message}", file=sys.stderr)
        sys.exit(2)

    if args.json:
        print(json.dumps({"passed": tally["PASS"], "failed": tally["FAIL"], "skipped": tally["SKIP"],
                          "results": results}, indent=2))
    else:
        print(f"\n{'=' * 60}")
        print(f"Total: {len(results)}  Passed: {tally['PASS']}  Failed: {tally['FAIL']}  Skipped: {tally['SKIP']}")
    sys.exit(1 if tally["FAIL"] else 0)


if __name__ == "__main__":
    main()
