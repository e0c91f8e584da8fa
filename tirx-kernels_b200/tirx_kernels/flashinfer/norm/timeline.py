"""Per-CTA timeline of ``flashinfer_rmsnorm_fp4quant`` on one GPU.

    python -m tirx_kernels.flashinfer.norm.timeline [--M 8192] [--H 7168] [--sets 4] [--step-us 2]

Launches the kernel over rotating buffer sets (cold inputs) with the library's timeline recorder on
(``b2_rmsnorm_fp4quant_timeline``) and prints, for the last launch: how long a CTA lives, how that splits
into waiting for its rows (including the reduction) and quantizing, and, per time window, how many CTAs
are in either phase and at what rate rows finish arriving.  The kernel reads every row from HBM exactly
once, so "rows reduced per window" is the input rate HBM sustains.  Observability only; the reference has
no counterpart.
"""

from __future__ import annotations

import argparse


def record(M: int, H: int, sets: int = 4):
    """Returns (start, reduced, end) in microseconds from the first CTA's start, and the SM ids."""
    import torch

    from tirx_kernels import _native
    from tirx_kernels.flashinfer.norm import rmsnorm_fp4quant as rms

    cfg = dict(next(c for c in rms.BENCH_CONFIGS if c["case"] == "bench_nv_swizzled_large"))
    cfg["M"], cfg["H"] = M, H
    launcher = rms.get_kernel(**{k: v for k, v in cfg.items() if k != "label"}).config["launcher"]
    buffers = [(rms._prepare_tensors(cfg), rms._prepare_output(cfg, initialize=False)) for _ in range(sets)]
    words = torch.zeros(4 * M, dtype=torch.int64, device="cuda")
    lib = _native.lib()
    for turn in range(2 * sets):
        data, out = buffers[turn % sets]
        words.zero_()
        torch.cuda.synchronize()
        _native.check(lib.b2_rmsnorm_fp4quant_timeline(words.data_ptr()), "b2_rmsnorm_fp4quant_timeline")
        rms._launch(launcher, data, out, cfg)
        torch.cuda.synchronize()
        _native.check(lib.b2_rmsnorm_fp4quant_timeline(None), "b2_rmsnorm_fp4quant_timeline")
    t = words.cpu().numpy().reshape(-1, 4)
    t = t[t[:, 0] > 0]
    if len(t) == 0:
        raise RuntimeError("this shape does not take the register-resident kernel: nothing was recorded")
    origin = t[:, 0].min()
    return (t[:, 0] - origin) / 1e3, (t[:, 1] - origin) / 1e3, (t[:, 2] - origin) / 1e3, t[:, 3]


def report(M: int, H: int, sets: int, step: float) -> None:
    import numpy as np

    start, reduced, end, sm = record(M, H, sets)
    cta_bytes = (M // len(start)) * H * 2
    print(f"rmsnorm_fp4quant {M} x {H}: {len(start)} CTAs on {len(set(sm.tolist()))} SMs, first start to last end "
          f"{end.max():.2f} us")
    print(f"CTA lifetime {np.mean(end - start):.2f} us = {np.mean(reduced - start):.2f} waiting for its rows (reduction "
          f"included) + {np.mean(end - reduced):.2f} quantizing and storing")
    print(f"first rows reduced at {reduced.min():.2f} us, last CTA starts at {start.max():.2f} us")
    for lo in np.arange(0.0, end.max(), step):
        waiting = int(((start <= lo) & (reduced > lo)).sum())
        quantizing = int(((reduced <= lo) & (end > lo)).sum())
        arrived = int(((reduced >= lo) & (reduced < lo + step)).sum()) * cta_bytes
        print(f"  {lo:5.1f}-{lo + step:5.1f} us: {waiting:4d} CTAs waiting, {quantizing:4d} quantizing at {lo:.0f} us; "
              f"{arrived / 1e6:5.1f} MB of rows reduced in the window = {arrived / step / 1e6:4.2f} TB/s")


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--M", type=int, default=8192)
    parser.add_argument("--H", type=int, default=7168)
    parser.add_argument("--sets", type=int, default=4)
    parser.add_argument("--step-us", type=float, default=2.0)
    args = parser.parse_args()
    report(args.M, args.H, args.sets, args.step_us)


if __name__ == "__main__":
    main()
