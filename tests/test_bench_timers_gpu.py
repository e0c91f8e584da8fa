"""The bench runner's timers on a real launch: CUDA events (cold and warm) and the reference's protocol,
Proton kernel time (`--timer proton`, `--timer cudagraph_proton`; tirx_kernels/bench/__main__.py:382-392 and
runner.py:492-519 of the reference delegate to `tvm.tirx.bench`, whose default timer is Proton).

The Proton timers run in a child process with a time limit: Proton attaches a profiler (CUPTI) to the process,
which a machine may refuse or another attached profiler may block, and neither may take the suite with it."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

REPO = Path(__file__).resolve().parent.parent

CHILD = """
import json, sys
sys.path[:0] = [{package!r}]
import torch
from tirx_kernels import _native, runner
m, k = 1024, 2048
x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
out = torch.empty(m, k // 2, dtype=torch.uint8, device="cuda")
sf = torch.empty(m * k // 16, dtype=torch.uint8, device="cuda")
gs = torch.ones(1, device="cuda")
launch = lambda: _native.nvfp4_quantize(x, out, sf, gs, m, k, "bfloat16", "128x4")
result = runner.bench({{"tirx": launch}}, warmup=5, repeat=10, timer={timer!r}, rounds=1, cooldown_s=0.0)
print("RESULT " + json.dumps({{"timer": result["timer"], "us": result["impls"]["tirx"]}}))
"""


def _launch():
    from tirx_kernels import _native

    m, k = 1024, 2048
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(m, k // 2, dtype=torch.uint8, device="cuda")
    sf = torch.empty(m * k // 16, dtype=torch.uint8, device="cuda")
    gs = torch.ones(1, device="cuda")
    return lambda: _native.nvfp4_quantize(x, out, sf, gs, m, k, "bfloat16", "128x4")


@pytest.mark.parametrize("timer", ["event", "event_warm"])
def test_event_timers_return_a_plausible_kernel_time(timer, native):
    from tirx_kernels import runner

    result = runner.bench({"tirx": _launch()}, warmup=5, repeat=10, timer=timer, rounds=1, cooldown_s=0.0)
    assert result["timer"] == timer
    microseconds = result["impls"]["tirx"]
    print(f"{timer}: {microseconds:.2f} us")
    assert 0.5 < microseconds < 200.0  # 1024 x 2048: a few microseconds of kernel, tens with host launch cost


@pytest.mark.parametrize("timer", ["proton", "cudagraph_proton"])
def test_proton_timers_return_a_plausible_kernel_time(timer, native):
    try:
        import triton.profiler  # noqa: F401
    except Exception as error:
        pytest.skip(f"triton.profiler is not importable here: {type(error).__name__}: {error}")
    code = CHILD.format(package=str(REPO / "tirx-kernels_b200"), timer=timer)
    try:
        child = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=180)
    except subprocess.TimeoutExpired:
        pytest.skip("the Proton timer did not finish within 180 s on this machine (profiler unavailable or busy)")
    lines = [line for line in child.stdout.splitlines() if line.startswith("RESULT ")]
    if child.returncode != 0 or not lines:
        pytest.skip(f"the Proton timer could not run here (exit {child.returncode}): {child.stderr.strip()[-300:]}")
    record = json.loads(lines[-1][len("RESULT "):])
    print(f"{timer}: {record['us']:.2f} us")
    assert record["timer"] == timer
    assert 0.5 < record["us"] < 200.0
