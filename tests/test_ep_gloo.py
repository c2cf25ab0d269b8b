"""Expert-parallel fused_moe: the exchange plan on two CPU ranks (gloo), numeric steps by torch.

The product path runs the numeric steps with CUDA kernels; here they are replaced by torch
restatements so that the part that is new with N > 1 ranks (counts, split sizes, arrival order,
inverse permutation, combine) is exercised without a GPU.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from dlcompiler_b200.distributed import ep_moe
from oracle import dlblas_oracle as oracle


class TorchOps:
    """CPU stand-ins for the CUDA kernels, with the same contracts and rounding points."""

    @staticmethod
    def sort_slots(topk_ids, num_experts):
        flat = topk_ids.reshape(-1).long()
        order = torch.sort(flat, stable=True)[1].to(torch.int32)
        counts = torch.bincount(flat, minlength=num_experts)
        prefix = torch.cat([counts.new_zeros(1), counts.cumsum(0)]).to(torch.int32)
        return order, prefix

    @staticmethod
    def gather_rows(src, row_map, rows, div):
        return src[(row_map[:rows].long() // div)]

    @staticmethod
    def expert_mlp(rows, weights, expert_of_row, w1, w2):
        out = torch.zeros(rows.size(0), w2.size(1), dtype=rows.dtype)
        for e in range(w1.size(0)):
            idx = torch.nonzero(expert_of_row == e).flatten()
            if idx.numel() == 0:
                continue
            gu = (rows[idx].float() @ w1[e].float().t()).to(rows.dtype)
            gate, up = gu.chunk(2, dim=-1)
            act = F.silu(gate) * up
            y = act.float() @ w2[e].float().t()
            out[idx] = (y * weights[idx, None]).to(rows.dtype)
        return out

    @staticmethod
    def combine(partial, tokens, top_k, topk_ids, num_experts):
        return partial.view(tokens, top_k, -1).float().sum(1).to(partial.dtype)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T, H, I, E, k, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        hs = torch.randn(T, H, generator=g).to(torch.bfloat16)
        w1 = (torch.randn(E, 2 * I, H, generator=g) * H ** -0.5).to(torch.bfloat16)
        w2 = (torch.randn(E, H, I, generator=g) * I ** -0.5).to(torch.bfloat16)
        tw, ti = oracle.softmax_topk(torch.randn(T, E, generator=g), k)
        if rank == 0:
            ti[: T // 2] = ti[: T // 2] % (E // world)        # skew: rank 0's tokens only use rank 0's experts
        ctx = ep_moe.EpMoeContext(dist.group.WORLD, E, torch.device("cpu"), ops=TorchOps)
        tl = T // world
        sl = slice(rank * tl, (rank + 1) * tl)
        el = E // world
        # every rank must derive the same routing for the comparison below
        if world > 1:
            dist.broadcast(ti, src=0)
        out = ep_moe.ep_fused_moe(ctx, hs[sl], w1[rank * el:(rank + 1) * el], w2[rank * el:(rank + 1) * el],
                                  tw[sl], ti[sl], k)
        ref = oracle.fused_moe_rounding_faithful(hs, w1, w2, tw, ti.long())[sl]
        ret[rank] = bool(torch.equal(out, ref))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ep_plan_matches_single_process_result(world):
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    mp.spawn(_worker, args=(world, port, 64, 32, 48, 8, 2, ret), nprocs=world, join=True)
    assert dict(ret) == {r: True for r in range(world)}


def test_exchange_plan_sizes_and_validation():
    # 2 ranks x 4 experts (2 per rank); counts[src, e]
    cm = torch.tensor([[3, 0, 2, 1], [1, 1, 0, 4]])
    send, recv, rec = ep_moe.exchange_plan(cm, rank=0, experts_per_rank=2)
    assert send == [3, 3] and recv == [3, 2]
    assert rec.tolist() == [[3, 0], [1, 1]]
    send, recv, rec = ep_moe.exchange_plan(cm, rank=1, experts_per_rank=2)
    assert send == [2, 4] and recv == [3, 4]
    assert rec.tolist() == [[2, 1], [0, 4]]
    # a corrupted plan is rejected on the host, before any collective is issued
    with pytest.raises(AssertionError):
        ep_moe.exchange_plan(torch.tensor([[1, -1, 0, 0], [0, 0, 0, 0]]), 0, 2)
    with pytest.raises(AssertionError):
        ep_moe.exchange_plan(torch.tensor([[1, 1, 0], [0, 0, 0]]), 0, 2)


def test_result_return_form_follows_the_down_gemm_tile_count():
    """The peer-memory exchange pulls results when the down GEMM fits one wave of tiles, pushes otherwise:
    the benchmark shape (4096 tokens, top-2, 8 experts, hidden 4096) on 148 SMs pulls only at 8 ranks."""
    for world, expect in ((1, False), (2, False), (4, False), (8, True)):
        slots = 4096 // world * 2
        assert ep_moe.prefers_pull(slots, 8 // world, 4096, 148) is expect
    assert ep_moe.prefers_pull(512, 4, 512, 148)          # small problems: one wave
    assert not ep_moe.prefers_pull(1024, 1, 4096, 132)    # the same 144 tiles on a smaller device: two waves
