"""The bench runner's timers on a real launch: CUDA events (cold and warm) and the reference's protocol,
Proton kernel time (`--timer proton`, `--timer cudagraph_proton`; tirx_kernels/bench/__main__.py:382-392 and
runner.py:492-519 of the reference delegate to `tvm.tirx.bench`, whose default timer is Proton)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _launch():
    from tirx_kernels import _native

    m, k = 1024, 2048
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(m, k // 2, dtype=torch.uint8, device="cuda")
    sf = torch.empty(m * k // 16, dtype=torch.uint8, device="cuda")
    gs = torch.ones(1, device="cuda")
    return lambda: _native.nvfp4_quantize(x, out, sf, gs, m, k, "bfloat16", "128x4")


@pytest.mark.parametrize("timer", ["event", "event_warm", "proton", "cudagraph_proton"])
def test_every_timer_returns_a_plausible_kernel_time(timer, native):
    from tirx_kernels import runner

    if timer.endswith("proton"):
        try:
            import triton.profiler  # noqa: F401
        except Exception as error:
            pytest.skip(f"triton.profiler is not importable here: {type(error).__name__}: {error}")
    result = runner.bench({"tirx": _launch()}, warmup=5, repeat=10, timer=timer, rounds=1, cooldown_s=0.0)
    assert result["timer"] == timer
    microseconds = result["impls"]["tirx"]
    print(f"{timer}: {microseconds:.2f} us")
    assert 0.5 < microseconds < 200.0  # 1024 x 2048: a few microseconds of kernel, tens with host launch cost
