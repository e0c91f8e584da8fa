"""GPU tests of the GEMM whose epilogue performs the output all-gather (b2_nvfp4_gemm_allgather).

One GPU: the ranks of a 2- and a 4-way sharding run one after another in one process, every
"peer" buffer living on the same device, which exercises the column offset, the leading dimension
and the replicated stores bit for bit against the plain GEMM.  Two GPUs (skipped on a one-GPU
machine): two processes exchange CUDA IPC handles and each must end up holding the full result,
identical to the NCCL all-gather path.
"""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _module():
    from tirx_kernels.basic import nvfp4_gemm

    return nvfp4_gemm


@pytest.mark.parametrize("world,M,N,K", [(2, 256, 512, 512), (4, 384, 1024, 768), (2, 200, 256, 256),
                                         (1, 256, 256, 256)])
def test_ranks_in_sequence_fill_every_buffer(world, M, N, K, native, oracle_expected):
    from tirx_kernels.basic import ffn_tp

    mod = _module()
    A_fp4, B_fp4, A_sf, B_sf, alpha, _ = mod.prepare_data(M, N, K)
    alpha_t = torch.tensor([float(alpha)], device="cuda")
    full = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    native.nvfp4_gemm(A_fp4, B_fp4, A_sf, B_sf, alpha_t, full, M, N, K)
    buffers = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    addresses = [b.data_ptr() for b in buffers]
    for rank in range(world):
        b_rows, b_sf = ffn_tp.slice_weight_shard(B_fp4, B_sf, N, K, world, rank)
        native.nvfp4_gemm_allgather(A_fp4, b_rows.contiguous(), A_sf, b_sf.contiguous(), alpha_t, addresses,
                                    rank, M, N // world, K)
    torch.cuda.synchronize()
    native.nvfp4_gemm_status()
    for b in buffers:
        assert torch.equal(b, full)
    # and the gathered rows themselves against the oracle, not only against the plain GEMM
    mod.check_output(buffers[-1], A_fp4, B_fp4, A_sf, B_sf, float(alpha_t.item()))


def test_rejects_what_it_cannot_run(native):
    mod = _module()
    M, N, K = 256, 256, 256
    A_fp4, B_fp4, A_sf, B_sf, alpha, _ = mod.prepare_data(M, N, K)
    alpha_t = torch.tensor([float(alpha)], device="cuda")
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="M > 128"):
        native.nvfp4_gemm_allgather(A_fp4[:64], B_fp4, A_sf, B_sf, alpha_t, [out.data_ptr()], 0, 64, N, K)
    with pytest.raises(ValueError, match="rank"):
        native.nvfp4_gemm_allgather(A_fp4, B_fp4, A_sf, B_sf, alpha_t, [out.data_ptr()], 1, M, N, K)
    with pytest.raises(ValueError, match="null or not 32-byte aligned"):
        native.nvfp4_gemm_allgather(A_fp4, B_fp4, A_sf, B_sf, alpha_t, [out.data_ptr() + 2], 0, M, N, K)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_gpu_worker(rank: int, world: int, port: int, M: int, N: int, K: int, results):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from tirx_kernels import _native
        from tirx_kernels.basic import ffn_tp, nvfp4_gemm as mod

        A_fp4, B_fp4, A_sf, B_sf, alpha, _ = mod.prepare_data(M, N, K)  # same seed on every rank
        alpha_t = torch.tensor([float(alpha)], device="cuda")
        full = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        _native.nvfp4_gemm(A_fp4, B_fp4, A_sf, B_sf, alpha_t, full, M, N, K)
        b_rows, b_sf = ffn_tp.slice_weight_shard(B_fp4, B_sf, N, K, world, rank)
        b_rows, b_sf = b_rows.contiguous(), b_sf.contiguous()
        buffers = ffn_tp.PeerOutputBuffers(M, N, world, rank)
        buffers.local.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        proj = ffn_tp.ShardedProjection(world, rank, M, N, K, b_rows, b_sf, alpha_t,
                                        quantize=lambda act: (A_fp4, A_sf), gemm=None)
        out = ffn_tp.fused_forward(proj, None, buffers)
        torch.cuda.synchronize()
        _native.nvfp4_gemm_status()
        # the gathered result against the oracle (sampled rows beyond its size limit) and the device-side
        # fp32 checker, then against the plain GEMM bit for bit
        import sys
        from pathlib import Path

        sys.path.insert(0, str(Path(__file__).resolve().parent))
        sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
        import oracle_provider
        from tirx_kernels import runner

        runner.set_reference_provider(oracle_provider.make_provider(_native))
        errors = mod.check_output(out, A_fp4, B_fp4, A_sf, B_sf, float(alpha_t.item()))
        results[rank] = bool(torch.equal(out, full)) and errors["rel_fro_vs_oracle"] <= 2e-3
        dist.barrier()
        buffers.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("M,N,K", [(512, 1024, 512), (8192, 7168, 2048)])
def test_two_processes_two_gpus(M, N, K):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_two_gpu_worker, args=(r, 2, port, M, N, K, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(results) == {0: True, 1: True}
