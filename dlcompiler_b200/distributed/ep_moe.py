"""Expert-parallel fused_moe: tokens and experts sharded over the ranks of one node.

Each of the G ranks holds T/G tokens and E/G experts.  One step:

  1. sort the local (token, k) slots by global expert id (moe_align kernel, block 1): rows bound
     for rank r are then contiguous, and the per-expert counts fall out of the block prefix;
  2. all-gather the [E] count vectors (every rank learns the full G x E count matrix; the host
     reads it once to size the exchanges);
  3. pack rows in destination order (permute kernel) and all-to-all them, together with each
     row's fp32 routing weight;
  4. on the expert side: label received rows with their local expert, moe_align (block 128),
     gather, grouped GEMM gate/up + silu, grouped GEMM down x weight, rows back in arrival order;
  5. all-to-all the results back, undo the sort, sum each token's top-k rows (combine kernel).

The reference has no collective code; its expert-parallel hook keeps tokens replicated and
masks non-local experts (python/dlBLAS/dlblas/kernels/fused_moe.py:113-114, 329-332; available
here as fused_moe(expert_offset=..., num_experts=...)).  Rounding points are the same as in the
single-GPU fused_moe, so the sharded result is bit-identical to the unsharded one.

The exchange plan is plain index arithmetic on torch tensors and is independent of the device;
the numeric steps go through an `ops` object (CUDA kernels by default) so the plan can be
exercised on CPU ranks with gloo.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

KERNELS_PER_STEP = 8  # align, pack, align, gather, gemm, gemm, unpack, combine


class CudaOps:
    """Numeric steps on the GPU (libdlblas_b200 kernels).  No fallback: needs CUDA tensors."""

    @staticmethod
    def sort_slots(topk_ids, num_experts):
        from ..kernels.fused_moe import _moe_align

        sorted_ids, _, _, block_start = _moe_align(topk_ids, 1, num_experts)
        return sorted_ids[:topk_ids.numel()], block_start          # block 1: blocks == rows

    @staticmethod
    def gather_rows(src, row_map, rows, div):
        from ..kernels.fused_moe import _permute_rows

        n = torch.tensor([rows], dtype=torch.int32, device=src.device)
        return _permute_rows(src, row_map, n, src.size(0) * div, div, rows)

    @staticmethod
    def expert_mlp(rows, weights, expert_of_row, w1, w2, events=None):
        """Rows [R, H] with their local expert id and routing weight -> down(silu(gate)*up) * weight, [R, H_out]."""
        from .. import _lib
        from ..kernels.fused_moe import BLOCK_M, _EventPair, _grouped_gemm, _moe_align, _permute_rows

        R = rows.size(0)
        E, N, _ = w1.shape
        sorted_ids, _, num_post, block_start = _moe_align(expert_of_row, BLOCK_M, E)
        cap = sorted_ids.numel()
        a_sorted = _permute_rows(rows, sorted_ids, num_post, R, 1, cap)
        act = torch.empty((cap, N // 2), dtype=rows.dtype, device=rows.device)
        ev = _EventPair(events, "grouped_gemm_gate_up_silu")
        _grouped_gemm(a_sorted, w1, act, N // 2, sorted_ids, block_start, None, R, _lib.GEMM_FUSE_SILU)
        ev.stop()
        out = torch.empty((R, w2.size(1)), dtype=rows.dtype, device=rows.device)
        ev = _EventPair(events, "grouped_gemm_down_scatter")
        _grouped_gemm(act, w2, out, w2.size(1), sorted_ids, block_start, weights, R,
                      _lib.GEMM_WEIGHT | _lib.GEMM_SCATTER)
        ev.stop()
        return out

    @staticmethod
    def combine(partial, tokens, top_k):
        from .. import _lib

        out = torch.empty((tokens, partial.size(1)), dtype=partial.dtype, device=partial.device)
        lib = _lib.load()
        with torch.cuda.device(partial.device):
            rc = lib.dlb_moe_combine(partial.data_ptr(), out.data_ptr(), tokens, top_k, partial.size(1),
                                     out.stride(0), _lib.dtype_code(out), _lib.stream_ptr(partial.device))
        _lib.check(rc, "moe_combine")
        return out


@dataclass
class EpMoeContext:
    group: object
    num_experts: int
    device: torch.device
    ops: object = CudaOps

    def __post_init__(self):
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.num_experts % self.world != 0:
            raise AssertionError(f"{self.num_experts} experts do not divide over {self.world} ranks")
        self.experts_per_rank = self.num_experts // self.world


def exchange_plan(count_matrix: torch.Tensor, rank: int, experts_per_rank: int):
    """Sizes of one dispatch from the G x E count matrix (a host tensor).

    Returns (send_splits, recv_splits, recv_expert_counts) where send_splits[r] is the number of
    rows this rank sends to rank r, recv_splits[s] the number it receives from rank s, and
    recv_expert_counts[s, e] the rows from rank s for local expert e (arrival order is
    source-major, expert-minor).  Validates that the matrix is consistent before any exchange.
    """
    G = count_matrix.size(0)
    if count_matrix.dim() != 2 or count_matrix.size(1) != G * experts_per_rank:
        raise AssertionError(f"count matrix shape {tuple(count_matrix.shape)} does not match {G} ranks x "
                             f"{G * experts_per_rank} experts")
    if bool((count_matrix < 0).any()):
        raise AssertionError("negative expert count in the exchange plan")
    per_rank = count_matrix.view(G, G, experts_per_rank)            # [src, dst, e_local]
    send_splits = per_rank[rank].sum(-1).tolist()
    recv_expert_counts = per_rank[:, rank, :].contiguous()          # [src, e_local]
    recv_splits = recv_expert_counts.sum(-1).tolist()
    return send_splits, recv_splits, recv_expert_counts


def ep_fused_moe(ctx: EpMoeContext, hidden_states, w1_local, w2_local, topk_weights, topk_ids, topk: int,
                 _events: list = None):
    """fused_moe over an expert-parallel group.  `topk_ids` are GLOBAL expert ids; `w1_local` /
    `w2_local` hold experts [rank*E/G, (rank+1)*E/G).  Returns this rank's tokens' outputs."""
    ops = ctx.ops
    T, H = hidden_states.shape
    numel = T * topk
    dev = hidden_states.device
    epr = ctx.experts_per_rank

    # 1. local sort by global expert
    sorted_slots, expert_prefix = ops.sort_slots(topk_ids, ctx.num_experts)     # int32 [numel], [E+1]
    counts = (expert_prefix[1:] - expert_prefix[:-1]).to(torch.int64)

    # 2. count matrix on every rank
    all_counts = torch.empty((ctx.world, ctx.num_experts), dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(all_counts, counts.unsqueeze(0).contiguous(), group=ctx.group)
    count_matrix = all_counts.cpu()
    send_splits, recv_splits, recv_expert_counts = exchange_plan(count_matrix, ctx.rank, epr)
    if sum(send_splits) != numel:
        raise AssertionError(f"rank {ctx.rank}: plan sends {sum(send_splits)} rows but {numel} slots exist")
    R = sum(recv_splits)

    # 3. pack + dispatch
    send_rows = ops.gather_rows(hidden_states, sorted_slots, numel, topk)        # [numel, H], expert-major
    send_w = topk_weights.to(torch.float32).reshape(-1)[sorted_slots.long()].contiguous()
    recv_rows = torch.empty((R, H), dtype=hidden_states.dtype, device=dev)
    recv_w = torch.empty((R,), dtype=torch.float32, device=dev)
    dist.all_to_all_single(recv_rows, send_rows, recv_splits, send_splits, group=ctx.group)
    dist.all_to_all_single(recv_w, send_w, recv_splits, send_splits, group=ctx.group)

    # 4. expert side
    local_expert = torch.arange(epr, dtype=torch.int32, device=dev).repeat(ctx.world)
    expert_of_row = torch.repeat_interleave(local_expert, recv_expert_counts.reshape(-1).to(dev), output_size=R)
    if R > 0:
        y = ops.expert_mlp(recv_rows, recv_w, expert_of_row, w1_local, w2_local, _events)
    else:
        y = torch.empty((0, w2_local.size(1)), dtype=hidden_states.dtype, device=dev)

    # 5. combine
    back = torch.empty((numel, y.size(1)), dtype=y.dtype, device=dev)
    dist.all_to_all_single(back, y, send_splits, recv_splits, group=ctx.group)
    inverse = torch.empty(numel, dtype=torch.int32, device=dev)
    inverse[sorted_slots.long()] = torch.arange(numel, dtype=torch.int32, device=dev)
    partial = ops.gather_rows(back, inverse, numel, 1)                            # slot order [T*topk, H]
    return ops.combine(partial, T, topk)
