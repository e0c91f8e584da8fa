"""N-sharded NVFP4 projection: the gate/up GEMM of a Llama-style FFN split over the GPUs of one box.

Not a registry kernel (no ``KERNEL_META``): this is the host-side harness of the sharded
workload.  The reference has no multi-GPU form of ``nvfp4_gemm``; the pattern - one process per
GPU, an NCCL group, rank-max timing - is the one its TP kernels use
(tirx_kernels/basic/utils/_runtime.py:38-60, 365-404).

Partitioning.  The weight ``B[N, K]`` is split by rows (output columns) into ``world`` contiguous
slabs of ``N / world`` rows; slabs are multiples of 128 rows so the 128x4-swizzled scale buffer
splits on tile boundaries.  Every rank quantizes the full activation (re-computing it is cheaper
than exchanging packed bytes), multiplies by its slab and contributes ``D_r[M, N/world]``.  The
only exchange is one all-gather of the bf16 outputs; it yields ``[world, M, N/world]``, which
``assemble`` views as the row-major ``[M, N]`` result.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable


def shard_rows(n: int, world: int, rank: int) -> tuple[int, int]:
    """[start, stop) of the weight rows owned by `rank`."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of world {world}")
    if n % world != 0 or (n // world) % 128 != 0:
        raise ValueError(f"N={n} must split into {world} slabs that are multiples of 128 rows")
    size = n // world
    return rank * size, (rank + 1) * size


def slice_weight_shard(B_fp4, B_sf, n: int, k: int, world: int, rank: int):
    """Views of one rank's packed rows and of its scale tiles inside the full-weight buffers."""
    start, stop = shard_rows(n, world, rank)
    sf_per_row = k // 16
    return B_fp4[start:stop], B_sf.reshape(-1)[start * sf_per_row:stop * sf_per_row]


def assemble(gathered):
    """``[world, M, N/world]`` (all-gather order) -> row-major ``[M, N]``."""
    world, m, shard = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, world * shard)


@dataclass
class ShardedProjection:
    """One rank's state: its weight slab (packed + scales), the two scale products and buffers.

    `quantize(act) -> (A_fp4, A_sf)` and `gemm(A_fp4, A_sf, B_fp4, B_sf, alpha, out)` are injected so
    that the same control flow runs on the GPU (the C-ABI kernels) and, in CPU tests, on a
    stand-in; `all_gather(out_flat, in_flat)` defaults to ``torch.distributed``.
    """

    world: int
    rank: int
    m: int
    n: int
    k: int
    B_fp4: object
    B_sf: object
    alpha: object
    quantize: Callable
    gemm: Callable
    all_gather: Callable | None = None

    def __post_init__(self):
        self.start, self.stop = shard_rows(self.n, self.world, self.rank)
        self.shard = self.stop - self.start

    def forward(self, act, out, gathered=None):
        """Quantize the activation, multiply by this rank's slab, gather; returns what was gathered."""
        A_fp4, A_sf = self.quantize(act)
        self.gemm(A_fp4, A_sf, self.B_fp4, self.B_sf, self.alpha, out)
        if self.world == 1:
            return out.reshape(1, self.m, self.shard)
        gather = self.all_gather
        if gather is None:
            import torch.distributed as dist

            gather = lambda dst, src: dist.all_gather_into_tensor(dst, src)
        gather(gathered.reshape(-1), out.reshape(-1))
        return gathered


class _RawDeviceMemory:
    """Exposes a raw device address to torch through the CUDA array interface (as int16 words)."""

    def __init__(self, ptr: int, words: int):
        self.__cuda_array_interface__ = {
            "shape": (words,),
            "typestr": "<i2",
            "data": (int(ptr), False),
            "version": 3,
            "strides": None,
        }


class PeerOutputBuffers:
    """One ``[M, world * shard]`` bf16 buffer per GPU, each mapped into every process of the box.

    The fused path (``b2_nvfp4_gemm_allgather``) stores its tiles into all of them, so after a
    cross-rank barrier every GPU holds the row-major ``[M, N]`` result with no separate gather and
    no re-layout.  Handles travel through ``torch.distributed`` (any backend); the memory itself is
    allocated and mapped by the C-ABI library.  ``local`` is a torch view of this rank's buffer.
    """

    def __init__(self, m: int, n: int, world: int, rank: int, group=None):
        import torch
        import torch.distributed as dist

        from .. import _native

        shard_rows(n, world, rank)
        self.m, self.n, self.world, self.rank = m, n, world, rank
        self.nbytes = m * n * 2
        self._native = _native
        self._own = _native.peer_alloc(self.nbytes)
        self._opened: list[int] = []
        self.addresses = [0] * world
        self.addresses[rank] = self._own
        if world > 1:
            handle = _native.peer_export(self._own)
            handles: list = [None] * world
            dist.all_gather_object(handles, handle, group=group)
            for g, h in enumerate(handles):
                if g == rank:
                    continue
                ptr = _native.peer_open(h)
                self._opened.append(ptr)
                self.addresses[g] = ptr
        self.local = torch.as_tensor(_RawDeviceMemory(self._own, m * n), device="cuda").view(torch.bfloat16).view(m, n)

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's; every rank calls it after a barrier."""
        for ptr in self._opened:
            self._native.peer_close(ptr)
        self._opened = []
        if self._own:
            self.local = None
            self._native.peer_free(self._own)
            self._own = 0


def fused_forward(proj: ShardedProjection, act, buffers: PeerOutputBuffers, barrier: Callable | None = None,
                  launch: Callable | None = None):
    """Quantize, then GEMM with the all-gather done by the GEMM's own epilogue over peer stores.

    Returns the row-major ``[M, N]`` tensor on this GPU.  `launch` defaults to the fused kernel
    (``b2_nvfp4_gemm_allgather``).  `barrier()` must order every rank's GEMM
    before any rank's read (default: a one-element NCCL all-reduce on the current stream).  A caller
    that runs steps back to back alternates between two `PeerOutputBuffers`, so that a fast rank's
    next step cannot overwrite rows a slow rank is still reading.
    """
    from .. import _native

    A_fp4, A_sf = proj.quantize(act)
    if launch is None:  # `launch` lets a CPU test stand in for the kernel, as `quantize` / `gemm` do above
        launch = _native.nvfp4_gemm_allgather
    launch(A_fp4, proj.B_fp4, A_sf, proj.B_sf, proj.alpha, buffers.addresses, proj.rank, proj.m, proj.shard, proj.k)
    if proj.world > 1:
        if barrier is None:
            import torch
            import torch.distributed as dist

            token = getattr(buffers, "_token", None)
            if token is None:
                token = buffers._token = torch.zeros(1, device="cuda")
            dist.all_reduce(token)
        else:
            barrier()
    return buffers.local
