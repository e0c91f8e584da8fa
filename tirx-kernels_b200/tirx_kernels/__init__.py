"""B200-native drop-in for the NVFP4 hot path of mlc-ai/TIRx-kernels.

Keeps the reference's package layout for the three registry entries it replaces
(`nvfp4_gemm`, `nvfp4_quantize`, `flashinfer_rmsnorm_fp4quant`), its registry, runner
and `python -m tirx_kernels.{registry,test,bench}` CLIs.  The kernels are hand-written
CUDA for sm_100a in a C-ABI shared library (see `tirx_kernels._native`); there is no
TVM/TIRx, no Triton and no CPU fallback.
"""

__version__ = "0.1.0"
