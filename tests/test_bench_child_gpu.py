"""GPU leg of the bench suite's prepared-child protocol: late assignment by physical UUID, the
benchmark result, a retry in place, and an identity mismatch."""

import json
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

REPO = Path(__file__).resolve().parent.parent


def _child(*extra):
    import os

    parent, child = socket.socketpair()
    env = {**os.environ, "PYTHONPATH": f"{REPO / 'tirx-kernels_b200'}:{REPO}"}
    proc = subprocess.Popen([sys.executable, "-m", "tirx_kernels.bench", "--prepared-control-fd", str(child.fileno()),
                             "--warmup", "5", "--repeat", "10", "--rounds", "1", *extra],
                            pass_fds=[child.fileno()], env=env)
    child.close()
    return proc, parent, parent.makefile("r", encoding="utf-8")


def _uuid() -> str:
    return str(torch.cuda.get_device_properties(0).uuid)


def test_assign_run_retry_accept():
    proc, parent, reader = _child("--kernel", "nvfp4_quantize", "--config", "fp16_128x4_m128_k1024")
    assert json.loads(reader.readline())["type"] == "READY"
    assign = json.dumps({"type": "ASSIGN", "gpu_indices": [0], "gpu_uuids": [_uuid()]}).encode() + b"\n"
    for attempt in (1, 2):
        parent.sendall(assign)
        running = json.loads(reader.readline())
        assert running["type"] == "RUNNING_GPU" and running["gpu_attempt"] == attempt
        ready = json.loads(reader.readline())
        assert ready["type"] == "RESULT_READY" and ready["gpu_attempt"] == attempt
        result = ready["result"]
        assert result["kernel"] == "nvfp4_quantize" and result["impls"]["tirx"] > 0
        assert result["retry_in_place"] == (attempt > 1)
        parent.sendall(b'{"type":"RETRY_GPU"}\n' if attempt == 1 else b'{"type":"ACCEPT_RESULT"}\n')
    assert proc.wait(timeout=120) == 0


def test_identity_mismatch_fails_the_gpu_phase():
    proc, parent, reader = _child("--kernel", "nvfp4_gemm", "--config", "1024x1024x1024")
    assert json.loads(reader.readline())["type"] == "READY"
    parent.sendall(json.dumps({"type": "ASSIGN", "gpu_indices": [0],
                               "gpu_uuids": ["GPU-00000000-0000-0000-0000-000000000000"]}).encode() + b"\n")
    message = json.loads(reader.readline())
    assert message["type"] == "FAIL" and message["phase"] == "gpu" and "identity mismatch" in message["error"]
    assert proc.wait(timeout=120) == 1
