"""world_size-2 run of the sharded projection's host logic on CPU (gloo): every rank works on its
weight slab with the oracle standing in for the kernels, the outputs are all-gathered, and the
assembled matrix must equal the unsharded product bit for bit."""

import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parent.parent
M, N, K = 128, 512, 256


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _problem():
    from oracle import nvfp4_oracle as o

    g = torch.Generator().manual_seed(0)
    act = torch.randn(M, K, generator=g).to(torch.bfloat16)
    weight = (0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16)
    w_gs = np.float32(2688.0 / weight.float().abs().max().item())
    B_fp4, B_sf = o.nvfp4_quantize(_bits(weight), o.BF16, w_gs, "128x4")
    return act, torch.from_numpy(B_fp4), torch.from_numpy(B_sf), w_gs


def _cpu_quantize(act):
    from oracle import nvfp4_oracle as o

    gs = np.float32(2688.0 / act.float().abs().max().item())
    packed, sf = o.nvfp4_quantize(_bits(act), o.BF16, gs, "128x4")
    return (torch.from_numpy(packed), gs), torch.from_numpy(sf)


def _cpu_gemm(A, A_sf, B_fp4, B_sf, alpha, out):
    from oracle import nvfp4_oracle as o

    packed, a_gs = A
    bits = o.nvfp4_gemm(packed.numpy(), B_fp4.numpy(), A_sf.numpy(), B_sf.numpy(), 1.0 / (a_gs * alpha))
    out.copy_(torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16))


def _rank_main(rank, world, store_path, result_path):
    for entry in (REPO, REPO / "tirx-kernels_b200"):
        sys.path.insert(0, str(entry))
    from tirx_kernels.basic import ffn_tp

    dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world)
    act, B_fp4, B_sf, w_gs = _problem()
    mine_fp4, mine_sf = ffn_tp.slice_weight_shard(B_fp4, B_sf, N, K, world, rank)
    proj = ffn_tp.ShardedProjection(world, rank, M, N, K, mine_fp4.contiguous(), mine_sf.contiguous(), w_gs,
                                    _cpu_quantize, _cpu_gemm)
    out = torch.empty(M, N // world, dtype=torch.bfloat16)
    gathered = torch.empty(world, M, N // world, dtype=torch.bfloat16)
    result = ffn_tp.assemble(proj.forward(act, out, gathered))
    # rank-max reduction of a per-rank scalar, the pattern the benchmark uses for timing
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == world
    if rank == 0:
        torch.save(result.contiguous(), result_path)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_product():
    with tempfile.TemporaryDirectory() as tmp:
        store, result_path = os.path.join(tmp, "store"), os.path.join(tmp, "result.pt")
        mp.spawn(_rank_main, args=(2, store, result_path), nprocs=2, join=True)
        sharded = torch.load(result_path)
    act, B_fp4, B_sf, w_gs = _problem()
    A, A_sf = _cpu_quantize(act)
    full = torch.empty(M, N, dtype=torch.bfloat16)
    _cpu_gemm(A, A_sf, B_fp4, B_sf, w_gs, full)
    assert torch.equal(sharded, full)


def test_a_rank_that_never_joins_ends_in_a_timeout_not_a_hang():
    """Failure detection on the host: the group's timeout turns a missing rank into an error."""
    with tempfile.TemporaryDirectory() as tmp:
        store = os.path.join(tmp, "store")
        with pytest.raises(Exception):
            dist.init_process_group("gloo", init_method=f"file://{store}", rank=0, world_size=2,
                                    timeout=__import__("datetime").timedelta(seconds=2))
        if dist.is_initialized():
            dist.destroy_process_group()


def _fused_rank_main(rank, world, store_path, result_path):
    for entry in (REPO, REPO / "tirx-kernels_b200"):
        sys.path.insert(0, str(entry))
    from types import SimpleNamespace

    from tirx_kernels.basic import ffn_tp

    dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world)
    act, B_fp4, B_sf, w_gs = _problem()
    mine_fp4, mine_sf = ffn_tp.slice_weight_shard(B_fp4, B_sf, N, K, world, rank)
    proj = ffn_tp.ShardedProjection(world, rank, M, N, K, mine_fp4.contiguous(), mine_sf.contiguous(), w_gs,
                                    _cpu_quantize, _cpu_gemm)
    sets = [SimpleNamespace(addresses=[0] * world, local=torch.zeros(M, N, dtype=torch.bfloat16)) for _ in range(2)]
    barriers = []

    def stand_in(A, B, A_sf, B_sf_, alpha, addresses, rank_, m, shard, k):
        """Computes this rank's columns and 'stores' them into every rank's buffer (an all-gather stands in
        for the peer stores, which have no CPU form)."""
        assert (rank_, m, shard, k) == (rank, M, N // world, K) and len(addresses) == world
        mine = torch.empty(m, shard, dtype=torch.bfloat16)
        _cpu_gemm(A, A_sf, B, B_sf_, alpha, mine)
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        current["buffers"].local.copy_(torch.cat(parts, dim=1))

    current = {}
    outputs = []
    for step in range(3):  # back-to-back steps alternate between the two buffer sets
        current["buffers"] = sets[step & 1]
        out = ffn_tp.fused_forward(proj, act, sets[step & 1], barrier=lambda: (barriers.append(step), dist.barrier()),
                                   launch=stand_in)
        outputs.append(out.clone())
    assert barriers == [0, 1, 2]
    assert torch.equal(outputs[0], outputs[1]) and torch.equal(outputs[1], outputs[2])
    if rank == 0:
        torch.save(outputs[-1].contiguous(), result_path)
    dist.barrier()
    dist.destroy_process_group()


def test_fused_forward_host_logic_on_two_ranks():
    """The fused path's control flow (quantize, one launch, one barrier per step, alternating buffer sets)
    yields the row-major unsharded product on every rank."""
    with tempfile.TemporaryDirectory() as tmp:
        store, result_path = os.path.join(tmp, "store"), os.path.join(tmp, "result.pt")
        mp.spawn(_fused_rank_main, args=(2, store, result_path), nprocs=2, join=True)
        fused = torch.load(result_path)
    act, B_fp4, B_sf, w_gs = _problem()
    A, A_sf = _cpu_quantize(act)
    full = torch.empty(M, N, dtype=torch.bfloat16)
    _cpu_gemm(A, A_sf, B_fp4, B_sf, w_gs, full)
    assert torch.equal(fused, full)
