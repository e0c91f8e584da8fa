"""Quantizing an activation that lives in pinned HOST memory.

Not a registry kernel: a helper above ``nvfp4_quantize`` for callers whose tensors start and end on
the host (the reference has no such entry; its executables take device tensors).  The rows are cut
into chunks that flow host -> device, through the quantizer, and device -> host on three CUDA
streams, so the upload of chunk i+1, the kernel of chunk i and the download of chunk i-1 overlap and
the PCIe link runs in both directions at once.  Chunks are multiples of 128 rows, which keeps every
chunk's slice of a swizzled scale buffer contiguous.
"""

from __future__ import annotations

from tirx_kernels import _checks, _native


class HostQuantizePipeline:
    def __init__(self, dtype: str, m: int, k: int, sf_layout: str = "128x4", chunks: int = 8):
        import torch

        from tirx_kernels.flashinfer.quantization import nvfp4_quantize as quant

        quant._validate(dtype, m, k, sf_layout, False)
        self.dtype, self.m, self.k, self.sf_layout = dtype, m, k, sf_layout
        rows = max(128, _checks.ceil_div(_checks.ceil_div(m, max(chunks, 1)), 128) * 128)
        self.bounds = [(r, min(r + rows, m)) for r in range(0, m, rows)]
        self.x = torch.empty(m, k, dtype=quant._torch_dtype(dtype), device="cuda")
        self.out, self.sf = quant._alloc_outputs(m, k, sf_layout)
        self.sf_cols = k // 16 if sf_layout == "linear" else _checks.ceil_div(k // 16, 4) * 4
        self.upload, self.compute, self.download = (torch.cuda.Stream() for _ in range(3))
        self.launches_per_call = len(self.bounds)

    def _sf_slice(self, r0: int, r1: int):
        """The contiguous part of the scale buffer that rows [r0, r1) own (r0 is a multiple of 128)."""
        tile = {"linear": 1, "128x4": 128, "8x4": 8}[self.sf_layout]
        end = _checks.ceil_div(r1, tile) * tile
        return self.sf[r0 * self.sf_cols:end * self.sf_cols]

    def __call__(self, x_pinned, global_scale, out_pinned, sf_pinned) -> None:
        """Enqueue one pass; the current stream is ordered after the last download."""
        import torch

        current = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(current)
        for stream in (self.upload, self.compute, self.download):
            stream.wait_event(start)
        for r0, r1 in self.bounds:
            with torch.cuda.stream(self.upload):
                self.x[r0:r1].copy_(x_pinned[r0:r1], non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(self.upload)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(uploaded)
                sf_part = self._sf_slice(r0, r1)
                _native.nvfp4_quantize(self.x[r0:r1], self.out[r0:r1], sf_part, global_scale, r1 - r0, self.k,
                                       self.dtype, self.sf_layout)
                computed = torch.cuda.Event()
                computed.record(self.compute)
            with torch.cuda.stream(self.download):
                self.download.wait_event(computed)
                out_pinned[r0:r1].copy_(self.out[r0:r1], non_blocking=True)
                lo = r0 * self.sf_cols
                sf_pinned[lo:lo + sf_part.numel()].copy_(sf_part, non_blocking=True)
        done = torch.cuda.Event()
        done.record(self.download)
        current.wait_event(done)
