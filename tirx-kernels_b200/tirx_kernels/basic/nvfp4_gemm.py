"""``nvfp4_gemm``: dense block-scaled NVFP4 GEMM, hand-written tcgen05 kernel for sm_100a.

Drop-in for tirx_kernels/basic/nvfp4_gemm.py of the reference: same ``KERNEL_META`` (:1000),
square ``CONFIGS`` labels ``"{s}x{s}x{s}"`` (:1001-1003), the executable signature
``ex(A_fp4, B_fp4, A_sf, B_sf, alpha_tensor, out)`` (:992-997, :1019-1023) and the data
contract of ``prepare_data`` (:47-66): operands quantized with the encode scale
``448*6/amax`` into packed E2M1 with 128x4-swizzled E4M3 block scales, ``alpha`` the
reciprocal of the product of the two encode scales.

``D[M,N] (bf16) = alpha * A[M,K] . B[N,K]^T`` with fp32 accumulation in tensor memory.
The kernel is ``b2_nvfp4_gemm`` in the C-ABI library; operands are produced by this
package's own ``nvfp4_quantize`` kernel (the reference calls flashinfer's).  Shapes the
reference rejects but this build accepts: any ``M >= 1`` (rows beyond M are zero-filled on
load and masked on store), ``N % 128 == 0``.
"""

from __future__ import annotations

from tirx_kernels import _checks, _native
from tirx_kernels._protocol import KernelHandle
from tirx_kernels.runner import bench

KERNEL_META = {"name": "nvfp4_gemm", "category": "basic", "compute_capability": 10}

# Above this many multiply-accumulates an installed CPU oracle computes a seeded sample of
# ORACLE_SAMPLE_ROWS full output rows instead of the whole product (256 x 8192 x 8192 is the limit).
ORACLE_MAC_LIMIT = 2048 * 2048 * 4096
ORACLE_SAMPLE_ROWS = 256
TOLERANCE = 2e-3         # relative Frobenius error of the kernel against dequantize-then-fp32-matmul
CHECKER_TOLERANCE = 2e-4  # the device-side fp32 checker against the CPU oracle on the sampled rows
# Filled by every run_test: the errors it measured, for harnesses that want to print them.
LAST_CHECK: dict = {}


def _validate(M: int, N: int, K: int) -> None:
    if M < 1 or N < 1 or K < 1:
        raise ValueError(f"M, N, K must be positive, got {M}, {N}, {K}")
    if N % 128 != 0 or K % 256 != 0:
        raise ValueError("N, K must be divisible by 128, 256 respectively")


def flops(M: int, N: int, K: int) -> int:
    return 2 * M * N * K


def algorithmic_bytes(M: int, N: int, K: int) -> int:
    """Operands, both scale buffers (rows padded to 128) and the bf16 output."""
    pad = lambda rows: _checks.ceil_div(rows, 128) * 128
    return (M + N) * K // 2 + (pad(M) + pad(N)) * K // 16 + M * N * 2


class _Runner:
    """Executable for one (M, N, K); tensor maps are cached by pointer inside the library."""

    def __init__(self, M: int, N: int, K: int):
        _validate(M, N, K)
        self.shape = M, N, K

    def __call__(self, A, B, SFA, SFB, alpha, D) -> None:
        M, N, K = self.shape
        if A.numel() != M * K // 2 or B.numel() != N * K // 2 or D.numel() != M * N:
            raise ValueError("operand sizes do not match (M, N, K)")
        _native.nvfp4_gemm(A, B, SFA.view(-1), SFB.view(-1), alpha.view(-1), D, M, N, K)


def get_kernel(M: int, N: int, K: int, **kwargs) -> KernelHandle:
    _validate(M, N, K)
    return KernelHandle("b2_nvfp4_gemm", {"launcher": _Runner(M, N, K), "M": M, "N": N, "K": K})


def _compile_executable(M: int, N: int, K: int):
    return _Runner(M, N, K)


def quantize_operand(x, global_sf):
    """bf16/fp16 [rows, K] -> (packed E2M1 uint8 [rows, K/2], 128x4-swizzled E4M3 scales)."""
    import torch

    rows, k = x.shape
    dtype = {torch.float16: "float16", torch.bfloat16: "bfloat16"}[x.dtype]
    packed = torch.empty(rows, k // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(_checks.sf_numel(rows, k // 16, "128x4"), dtype=torch.uint8, device=x.device)
    gs = global_sf.reshape(1).to(device=x.device, dtype=torch.float32)
    _native.nvfp4_quantize(x.contiguous(), packed, sf, gs, rows, k, dtype, "128x4")
    return packed, sf


def prepare_data(M: int, N: int, K: int, *, return_origin: bool = False, b_std: float = 1.0, **kwargs):
    """Seeded operands, quantized on the GPU; returns (A_fp4, B_fp4, A_sf, B_sf, alpha, C_ref).

    A ~ N(0,1) [M,K] and B ~ N(0,b_std) [N,K] are drawn on the CPU (seed 0) in bf16;
    ``C_ref`` is the bf16 product of the unquantized operands, as in the reference.
    """
    import torch

    _validate(M, N, K)
    generator = torch.Generator().manual_seed(0)
    A_origin = torch.randn(M, K, generator=generator, dtype=torch.float32).to(torch.bfloat16).cuda()
    B_origin = (b_std * torch.randn(N, K, generator=generator, dtype=torch.float32)).to(torch.bfloat16).cuda()
    A_global_sf = 448 * 6 / A_origin.float().abs().nan_to_num().max()
    B_global_sf = 448 * 6 / B_origin.float().abs().nan_to_num().max()
    A_fp4, A_sf = quantize_operand(A_origin, A_global_sf)
    B_fp4, B_sf = quantize_operand(B_origin, B_global_sf)
    alpha = 1.0 / (A_global_sf * B_global_sf)
    C_ref = torch.mm(A_origin, B_origin.T)
    if return_origin:
        return A_fp4, B_fp4, A_sf, B_sf, alpha, C_ref, A_origin, B_origin
    return A_fp4, B_fp4, A_sf, B_sf, alpha, C_ref


def relative_frobenius_error(got, want) -> float:
    got, want = got.float(), want.float()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


def check_output(out, A_fp4, B_fp4, A_sf, B_sf, alpha: float, *, label: str = "") -> dict:
    """Holds a GEMM output to the tolerance at any size and returns the errors it measured.

    Always: relative Frobenius error <= 2e-3 of the WHOLE output against dequantize-then-fp32-matmul
    (TF32 off) of the very bytes the kernel consumed, computed on the device (`_checks`).  With an
    expected-value provider installed, that provider (the CPU oracle in the tests) pins it: in full
    for products up to ORACLE_MAC_LIMIT multiply-accumulates; beyond that on a seeded sample of
    ORACLE_SAMPLE_ROWS full output rows, on which the device-side checker must agree with the
    provider as well (fp32 summation order and the rare bf16 rounding flip are all that separate
    the two).  The reference's check is :1019-1027.
    """
    import torch

    from tirx_kernels.runner import reference_provider

    M, N = out.shape
    K = A_fp4.shape[1] * 2
    errors = {"label": label or f"{M}x{N}x{K}", "M": M, "N": N, "K": K}
    checker = _checks.dequantized_matmul_fp32(A_fp4, B_fp4, A_sf, B_sf, alpha)
    errors["rel_fro_vs_device_fp32_checker"] = relative_frobenius_error(out, checker)
    provider = reference_provider()
    if provider is not None:
        operands = dict(A_fp4=A_fp4, B_fp4=B_fp4, A_sf=A_sf, B_sf=B_sf, alpha=alpha)
        if M * N * K <= ORACLE_MAC_LIMIT:
            want = provider("nvfp4_gemm", **operands)
            errors["rel_fro_vs_oracle"] = relative_frobenius_error(out.cpu(), want)
            errors["checker_vs_oracle"] = relative_frobenius_error(checker.cpu(), want)
            errors["oracle_rows"] = M
        else:
            generator = torch.Generator().manual_seed(M * 31 + N * 17 + K)
            rows = torch.randperm(M, generator=generator)[: min(M, ORACLE_SAMPLE_ROWS)].sort().values
            want = provider("nvfp4_gemm", rows=rows, **operands)
            errors["rel_fro_vs_oracle"] = relative_frobenius_error(out[rows.to(out.device)].cpu(), want)
            errors["checker_vs_oracle"] = relative_frobenius_error(checker[rows.to(out.device)].cpu(), want)
            errors["oracle_rows"] = int(rows.numel())
    LAST_CHECK.clear()
    LAST_CHECK.update(errors)
    print("nvfp4_gemm check " + " ".join(f"{k}={v:.3e}" if isinstance(v, float) else f"{k}={v}" for k, v in errors.items()))
    assert errors["rel_fro_vs_device_fp32_checker"] <= TOLERANCE, \
        f"nvfp4_gemm relative Frobenius error {errors['rel_fro_vs_device_fp32_checker']:.3e} > {TOLERANCE} (device fp32 checker)"
    if "rel_fro_vs_oracle" in errors:
        assert errors["checker_vs_oracle"] <= CHECKER_TOLERANCE, \
            f"device fp32 checker is {errors['checker_vs_oracle']:.3e} from the oracle on its rows"
        assert errors["rel_fro_vs_oracle"] <= TOLERANCE, \
            f"nvfp4_gemm relative Frobenius error {errors['rel_fro_vs_oracle']:.3e} > {TOLERANCE} (oracle)"
    return errors


def run_test(M: int = 1024, N: int = 1024, K: int = 1024, **kwargs) -> None:
    """Launch one shape and verify it.

    The device status word is clean, the output correlates with the bf16 product of the unquantized
    operands (cosine > 0.97, the reference's check, :1024-1027), and `check_output` holds it to the
    2e-3 bar at every size.
    """
    import torch
    import torch.nn.functional as F

    label = kwargs.pop("label", "")
    A_fp4, B_fp4, A_sf, B_sf, alpha, C_ref = prepare_data(M, N, K, **kwargs)
    alpha_tensor = torch.tensor([float(alpha)], device="cuda", dtype=torch.float32)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ex = _compile_executable(M, N, K)
    if ex(A_fp4, B_fp4, A_sf, B_sf, alpha_tensor, out) is not None:
        raise AssertionError("nvfp4_gemm executable must return None")
    torch.cuda.synchronize()
    _native.nvfp4_gemm_status()
    if not torch.isfinite(out.float()).all():
        raise AssertionError("nvfp4_gemm left non-finite (unwritten) outputs")
    cosine_sim = F.cosine_similarity(out.reshape(-1).float(), C_ref.reshape(-1).float(), dim=0)
    assert cosine_sim > 0.97, f"nvfp4_gemm cosine_sim {cosine_sim:.6f} <= 0.97"
    del C_ref
    check_output(out, A_fp4, B_fp4, A_sf, B_sf, float(alpha_tensor.item()), label=label)


def prepare_bench(M: int = 1024, N: int = 1024, K: int = 1024, **kwargs):
    from tirx_kernels.runner import external_references_enabled, prepared_gpu_benchmark

    if external_references_enabled():
        _native.cublaslt_lib()
    state = {"config": {"M": M, "N": N, "K": K, **kwargs}, "executable": _compile_executable(M, N, K)}
    return prepared_gpu_benchmark(run_gpu, state)


def run_gpu(prepared, *, warmup=None, repeat=None, timer=None, **kwargs):
    """Kernel-only timing; with ``--with-references`` the cuBLASLt NVFP4 matmul is timed beside it."""
    import torch

    config = {**prepared["config"], **kwargs}
    M, N, K = config.pop("M"), config.pop("N"), config.pop("K")
    data_kwargs = {k: config.pop(k) for k in ("b_std",) if k in config}
    ex = prepared["executable"]
    A_fp4, B_fp4, A_sf, B_sf, alpha, C_ref = prepare_data(M, N, K, **data_kwargs)
    alpha_value = float(alpha)
    alpha_tensor = torch.tensor([alpha_value], device="cuda", dtype=torch.float32)
    out_tir = torch.empty_like(C_ref)
    funcs = {"tir": lambda: ex(A_fp4, B_fp4, A_sf, B_sf, alpha_tensor, out_tir)}
    metadata = {}

    def _cublaslt():
        out_lt = torch.empty_like(out_tir)
        launch = lambda: _native.nvfp4_gemm_cublaslt(A_fp4, B_fp4, A_sf, B_sf, alpha_value, out_lt, M, N, K)
        launch()
        funcs["tir"]()
        torch.cuda.synchronize()
        metadata["cublaslt_vs_tir_rel_fro"] = relative_frobenius_error(out_tir, out_lt)
        return launch

    def _flashinfer():
        """flashinfer's `mm_fp4`, the reference's second timing peer (tirx_kernels/basic/nvfp4_gemm.py:1153-1222):
        the same packed operands and swizzled scales, tuned once for this shape before it is timed.  The
        back-end is the one the reference reports (cuDNN) unless B2_FLASHINFER_MM_FP4_BACKEND names another."""
        import os

        import flashinfer

        backend = os.environ.get("B2_FLASHINFER_MM_FP4_BACKEND", "cudnn")
        out_fi = torch.empty_like(out_tir)
        pad = lambda rows: _checks.ceil_div(rows, 128) * 128
        a_sf = A_sf.view(pad(M), K // 16)
        b_sf = B_sf.view(pad(N), K // 16)

        def launch():
            flashinfer.mm_fp4(A_fp4, B_fp4.T, a_sf, b_sf.T, alpha_tensor, out=out_fi, block_size=16, backend=backend,
                              use_nvfp4=True)

        with flashinfer.autotune(True):
            launch()
        torch.cuda.synchronize()
        funcs["tir"]()
        torch.cuda.synchronize()
        metadata["flashinfer_mm_fp4_backend"] = backend
        metadata["flashinfer_mm_fp4_vs_tir_rel_fro"] = relative_frobenius_error(out_tir, out_fi)
        return launch

    protocol = {k: config.pop(k) for k in ("rounds", "cooldown_s") if k in config}
    result = bench(funcs, warmup=warmup, repeat=repeat, timer=timer,
                   references={"cublaslt_nvfp4": _cublaslt, "flashinfer_mm_fp4": _flashinfer}, **protocol)
    _native.nvfp4_gemm_status()
    microseconds = result["impls"]["tir"]
    if M >= 1024:
        result["roofline"] = _checks.roofline_nvfp4(flops(M, N, K), microseconds)
    else:  # decode-shaped: weights are streamed once, the tensor cores idle
        result["roofline"] = _checks.roofline_hbm(algorithmic_bytes(M, N, K), microseconds)
        result["roofline"]["tflops"] = flops(M, N, K) / (microseconds * 1e-6) / 1e12
    result["metadata"] = {**result.get("metadata", {}), **metadata}
    return result


def run_bench(M: int = 1024, N: int = 1024, K: int = 1024, *, warmup=None, repeat=None, timer=None, **kwargs):
    protocol = {name: kwargs.pop(name) for name in ("rounds", "cooldown_s") if name in kwargs}
    return prepare_bench(M=M, N=N, K=K, **kwargs).run_gpu(warmup=warmup, repeat=repeat, timer=timer, **protocol)


# The reference's five squares, then the shapes it rejects that this build is measured on:
# the decode-shaped M=16 problem and one Llama-3-70B gate/up projection shard per GPU count.
CONFIGS = [{"M": s, "N": s, "K": s, "label": f"{s}x{s}x{s}"} for s in [1024, 2048, 4096, 8192, 16384]]
CONFIGS += [
    {"M": 16, "N": 8192, "K": 8192, "label": "16x8192x8192"},
    {"M": 384, "N": 640, "K": 768, "label": "384x640x768"},
]
CONFIGS += [
    {"M": 8192, "N": 28672 // g, "K": 8192, "b_std": 0.02, "label": f"ffn_shard_tp{g}_m8192_n{28672 // g}_k8192"}
    for g in (1, 2, 4, 8)
]
