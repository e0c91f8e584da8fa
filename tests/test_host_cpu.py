"""CPU checks of the host side: the C-ABI library exports what the header declares, the registry,
runner and CLIs behave like the reference's, and the sharding helpers partition correctly."""

import ctypes
import json
import re
import subprocess
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
ENV = {"PYTHONPATH": f"{REPO / 'tirx-kernels_b200'}:{REPO}"}


def _declared_symbols():
    header = (REPO / "include" / "b200_nvfp4.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", header)))


def test_libraries_export_every_declared_symbol():
    from tirx_kernels import _native

    declared = _declared_symbols()
    assert len(declared) >= 10
    main = ctypes.CDLL(str(_native.library_path("libb200nvfp4.so")))
    baseline = ctypes.CDLL(str(_native.library_path("libb200nvfp4_cublaslt.so")))
    for symbol in declared:
        owner = baseline if symbol == "b2_nvfp4_gemm_cublaslt" else main
        assert hasattr(owner, symbol), f"{symbol} is declared but not exported"
    assert set(_native.MAIN_SIGNATURES) | set(_native.CUBLASLT_SIGNATURES) == set(declared)
    assert main.b2_abi_version() == 1


def test_size_helper_and_argument_validation_need_no_gpu():
    from tirx_kernels import _native

    lib = _native.lib()
    assert lib.b2_nvfp4_sf_bytes(4096, 7168, 0) == 4096 * 448
    assert lib.b2_nvfp4_sf_bytes(120, 1040, 1) == 128 * 68
    assert lib.b2_nvfp4_sf_bytes(13, 1024, 2) == 16 * 64
    assert lib.b2_nvfp4_sf_bytes(4, 24, 0) == -1
    # rejected before any CUDA call is made
    assert lib.b2_nvfp4_quantize(None, None, None, None, 4, 24, 0, 0, 0, 0, None) == _native.ERR_INVALID_ARGUMENT
    assert "k=24" in _native.last_error()
    assert lib.b2_nvfp4_gemm(None, None, None, None, None, None, 128, 128, 256, None) == _native.ERR_INVALID_ARGUMENT
    assert lib.b2_rmsnorm_fp4quant(None, None, None, None, None, 4, 32, 1e-6, 0, 16, 0, 0, 0, None) \
        == _native.ERR_INVALID_ARGUMENT


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from tirx_kernels import _native

    monkeypatch.setenv("B200_NVFP4_LIB_DIR", str(tmp_path))
    monkeypatch.setattr(_native, "_MAIN", None)
    with pytest.raises(_native.NativeLibraryError, match="no CPU or PyTorch fallback"):
        _native.lib()


def test_registry_indexes_the_kernels_without_importing_them():
    from tirx_kernels import registry

    index = registry.kernel_index(strict=True)
    assert sorted(index) == ["flashinfer_add_rmsnorm_fp4quant", "flashinfer_rmsnorm_fp4quant", "nvfp4_gemm",
                             "nvfp4_quantize", "nvfp4_quantize_per_token"]
    assert index["nvfp4_gemm"].category == "basic" and index["nvfp4_quantize"].category == "flashinfer"
    assert index["nvfp4_quantize"].module_name == "tirx_kernels.flashinfer.quantization.nvfp4_quantize"
    with pytest.raises(KeyError):
        registry.load_kernel("rmsnorm")
    module = registry.load_kernel("nvfp4_gemm", strict=True)
    assert module.KERNEL_META == {"name": "nvfp4_gemm", "category": "basic", "compute_capability": 10}


def test_registry_rejects_bad_metadata(tmp_path, monkeypatch):
    from tirx_kernels import registry

    good = tmp_path / "a.py"
    good.write_text('KERNEL_META = {"name": "k", "category": "basic", "compute_capability": 10}\n')
    assert registry._read_literal_meta(good)["name"] == "k"
    twice = tmp_path / "b.py"
    twice.write_text(good.read_text() * 2)
    with pytest.raises(ValueError, match="more than once"):
        registry._read_literal_meta(twice)
    computed = tmp_path / "c.py"
    computed.write_text("KERNEL_META = dict(name='k')\n")
    with pytest.raises(ValueError):
        registry._read_literal_meta(computed)
    assert registry._meta_problems({"name": "k", "category": "other", "compute_capability": 10}, "basic")
    assert registry._meta_problems({"name": "", "category": "basic", "compute_capability": True}, "basic")


def test_config_labels_are_unique_and_keep_the_reference_vocabulary():
    from tirx_kernels import registry

    for name in ("nvfp4_gemm", "nvfp4_quantize", "nvfp4_quantize_per_token", "flashinfer_rmsnorm_fp4quant",
                 "flashinfer_add_rmsnorm_fp4quant"):
        module = registry.load_kernel(name)
        for configs in (module.CONFIGS, getattr(module, "BENCH_CONFIGS", [])):
            labels = [c["label"] for c in configs]
            assert len(labels) == len(set(labels))
    quant = registry.load_kernel("nvfp4_quantize")
    assert "bf16_128x4_m16384_k7168" in [c["label"] for c in quant.BENCH_CONFIGS]
    assert "fp16_linear_m13_k1040" in [c["label"] for c in quant.CONFIGS]
    gemm = registry.load_kernel("nvfp4_gemm")
    assert [c["label"] for c in gemm.CONFIGS][:5] == [f"{s}x{s}x{s}" for s in (1024, 2048, 4096, 8192, 16384)]
    rms = registry.load_kernel("flashinfer_rmsnorm_fp4quant")
    assert len(rms.CONFIGS) == 1025
    assert len(registry.load_kernel("flashinfer_add_rmsnorm_fp4quant").CONFIGS) == 1245
    assert len(registry.load_kernel("nvfp4_quantize_per_token").CONFIGS) == 17


def test_runner_prepared_benchmark_contract():
    from tirx_kernels import runner

    calls = []
    prepared = runner.prepared_gpu_benchmark(lambda state, **kw: calls.append((state, kw)) or {"impls": {}}, {"s": 1})
    assert prepared.run_gpu(rounds=2) == {"impls": {}} and calls == [({"s": 1}, {"rounds": 2})]
    with pytest.raises(TypeError):
        runner.prepared_gpu_benchmark(None, {})
    with pytest.raises(ValueError):
        runner.prepared_gpu_benchmark(lambda s: {}, {}, required_num_gpus=0)
    with pytest.raises(TypeError):
        import pickle

        pickle.dumps(prepared)
    assert {"event", "event_warm", "proton", "cudagraph_proton"} <= set(runner.SUPPORTED_TIMERS)
    with pytest.raises(ValueError, match="not provided by this build"):
        runner.bench({}, timer="kineto")
    runner.set_external_references_enabled(True)
    assert runner.external_references_enabled()
    runner.set_external_references_enabled(False)
    assert not runner.external_references_enabled()


def test_hardware_num_sms_honours_the_environment(monkeypatch):
    from tirx_kernels import runner

    monkeypatch.setenv(runner.PREPARE_NUM_SMS_ENV, "132")
    assert runner.hardware_num_sms() == 132
    monkeypatch.setenv(runner.PREPARE_NUM_SMS_ENV, "0")
    with pytest.raises(ValueError):
        runner.hardware_num_sms()


def _cli(*args):
    return subprocess.run([sys.executable, "-m", *args], capture_output=True, text=True, env={**ENV, "PATH": "/usr/bin:/bin"})


def test_test_cli_exit_codes_match_the_reference():
    unknown = _cli("tirx_kernels.test", "--kernel", "no_such_kernel")
    assert unknown.returncode == 1 and "not found" in unknown.stdout
    nothing = _cli("tirx_kernels.test", "--kernel", "nvfp4_gemm", "--config", "no_such_label", "--json")
    assert nothing.returncode == 2
    assert json.loads(nothing.stdout)["error"] == "no kernel configs matched the requested filters"


def test_registry_cli_lists_kernels():
    listing = _cli("tirx_kernels.registry", "--format", "json")
    assert listing.returncode == 0
    names = [entry["name"] for entry in json.loads(listing.stdout)]
    assert names == ["flashinfer_add_rmsnorm_fp4quant", "flashinfer_rmsnorm_fp4quant", "nvfp4_gemm", "nvfp4_quantize",
                     "nvfp4_quantize_per_token"]
    runs = _cli("tirx_kernels.registry", "--format", "benchrun", "--category", "basic")
    assert "nvfp4_gemm|8192x8192x8192|python -m tirx_kernels.bench --kernel nvfp4_gemm" in runs.stdout


def test_config_gpu_count_filter():
    import importlib

    cli = importlib.import_module("tirx_kernels.test.__main__")
    assert cli.config_gpu_count({"label": "x"}) == 1
    assert cli.config_gpu_count({"world_size": 4, "num_processes": 4}) == 4
    with pytest.raises(ValueError):
        cli.config_gpu_count({"world_size": 4, "num_processes": 2})
    with pytest.raises(ValueError):
        cli.config_gpu_count({"world_size": 0})


def test_shard_bounds_and_assembly():
    import torch

    from tirx_kernels.basic import ffn_tp

    assert ffn_tp.shard_rows(28672, 8, 3) == (3 * 3584, 4 * 3584)
    with pytest.raises(ValueError):
        ffn_tp.shard_rows(28672, 3, 0)
    with pytest.raises(ValueError):
        ffn_tp.shard_rows(1024, 16, 0)  # 64-row slabs would split a 128-row scale tile
    full = torch.arange(6 * 8).reshape(6, 8)
    gathered = torch.stack([full[:, 0:4], full[:, 4:8]])
    assert torch.equal(ffn_tp.assemble(gathered), full)


def test_bench_suite_workload_files_name_real_configs():
    """Every label a workload file lists resolves to exactly one benchmark config of its kernel."""
    import yaml

    from tirx_kernels import registry
    from tirx_kernels.bench.__main__ import find_bench_config

    files = sorted((REPO / "tirx-kernels_b200" / "tirx_kernels" / "bench_suite" / "config").rglob("*.yaml"))
    assert len(files) == 5
    for path in files:
        workload = yaml.safe_load(path.read_text())
        module = registry.load_kernel(workload["kernel"])
        assert path.stem == workload["kernel"] and workload["selection_rationale"]
        defaults = [c for c in workload["configs"] if c["default"]]
        assert {c["selection_role"] for c in defaults} >= {"small", "large"}
        for entry in workload["configs"]:
            assert find_bench_config(module, entry["config"])["label"] == entry["config"]


def _prepared_child(*extra):
    import socket

    parent, child = socket.socketpair()
    proc = subprocess.Popen([sys.executable, "-m", "tirx_kernels.bench", "--prepared-control-fd", str(child.fileno()),
                             *extra], pass_fds=[child.fileno()], env={**ENV, "PATH": "/usr/bin:/bin"})
    child.close()
    return proc, parent, parent.makefile("r", encoding="utf-8")


def test_prepared_child_reports_ready_without_touching_cuda_and_obeys_cancel():
    proc, parent, reader = _prepared_child("--kernel", "nvfp4_gemm", "--config", "1024x1024x1024")
    ready = json.loads(reader.readline())
    assert ready["type"] == "READY" and ready["required_num_gpus"] == 1
    assert ready["child_started"] <= ready["framework_loaded"] <= ready["module_loaded"] <= ready["ready"]
    parent.sendall(b'{"type":"CANCEL"}\n')
    assert proc.wait(timeout=60) == 0


def test_prepared_child_fails_in_the_prepare_phase_for_an_unknown_config():
    proc, parent, reader = _prepared_child("--kernel", "nvfp4_gemm", "--config", "no_such_label")
    message = json.loads(reader.readline())
    assert message["type"] == "FAIL" and message["phase"] == "prepare" and "no_such_label" in message["error"]
    assert proc.wait(timeout=60) == 1


def test_prepared_child_rejects_a_malformed_assignment():
    proc, parent, reader = _prepared_child("--kernel", "nvfp4_quantize", "--config", "fp16_128x4_m128_k1024")
    assert json.loads(reader.readline())["type"] == "READY"
    parent.sendall(b'{"type":"ASSIGN","gpu_indices":[0,0],"gpu_uuids":["x"]}\n')
    message = json.loads(reader.readline())
    assert message["type"] == "FAIL" and message["phase"] == "protocol" and "invalid GPU assignment" in message["error"]
    assert proc.wait(timeout=60) == 1
