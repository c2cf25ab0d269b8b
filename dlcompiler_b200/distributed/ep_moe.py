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
    def expert_mlp(rows, weights, expert_of_row, w1, w2):
        """Rows [R, H] with their local expert id and routing weight -> down(silu(gate)*up) * weight, [R, H_out]."""
        from .. import _lib
        from ..kernels import fused_moe as fm
        from ..kernels.fused_moe import BLOCK_M, _moe_align, _permute_rows

        R = rows.size(0)
        E, N, _ = w1.shape
        sorted_ids, _, num_post, block_start = _moe_align(expert_of_row, BLOCK_M, E)
        cap = sorted_ids.numel()
        a_sorted = _permute_rows(rows, sorted_ids, num_post, R, 1, cap)
        act = torch.empty((cap, N // 2), dtype=rows.dtype, device=rows.device)
        fm._grouped_gemm(a_sorted, w1, act, N // 2, sorted_ids, block_start, None, R, _lib.GEMM_FUSE_SILU)
        out = torch.empty((R, w2.size(1)), dtype=rows.dtype, device=rows.device)
        fm._grouped_gemm(act, w2, out, w2.size(1), sorted_ids, block_start, weights, R,
                         _lib.GEMM_WEIGHT | _lib.GEMM_SCATTER)
        return out

    @staticmethod
    def combine(partial, tokens, top_k, topk_ids, num_experts):
        """Sum of each token's top-k rows; slots whose expert id is outside [0, num_experts) add nothing."""
        from .. import _lib

        out = torch.empty((tokens, partial.size(1)), dtype=partial.dtype, device=partial.device)
        ids = topk_ids.reshape(-1)
        if ids.dtype not in (torch.int32, torch.int64):
            ids = ids.to(torch.int64)
        ids = ids.contiguous()
        lib = _lib.load()
        with torch.cuda.device(partial.device):
            rc = lib.dlb_moe_combine(partial.data_ptr(), out.data_ptr(), tokens, top_k, partial.size(1),
                                     out.stride(0), _lib.dtype_code(out), ids.data_ptr(),
                                     int(ids.dtype == torch.int64), 0, num_experts,
                                     _lib.stream_ptr(partial.device))
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


def ep_fused_moe(ctx: EpMoeContext, hidden_states, w1_local, w2_local, topk_weights, topk_ids, topk: int):
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
        y = ops.expert_mlp(recv_rows, recv_w, expert_of_row, w1_local, w2_local)
    else:
        y = torch.empty((0, w2_local.size(1)), dtype=hidden_states.dtype, device=dev)

    # 5. combine
    back = torch.empty((numel, y.size(1)), dtype=y.dtype, device=dev)
    dist.all_to_all_single(back, y, send_splits, recv_splits, group=ctx.group)
    inverse = torch.empty(numel, dtype=torch.int32, device=dev)
    inverse[sorted_slots.long()] = torch.arange(numel, dtype=torch.int32, device=dev)
    partial = ops.gather_rows(back, inverse, numel, 1)                            # slot order [T*topk, H]
    return ops.combine(partial, T, topk, topk_ids, ctx.num_experts)


# ----------------------------------------------------------------------------------------------
# Peer-memory variant: dispatch and combine are plain NVLink stores issued by our own kernels
# ----------------------------------------------------------------------------------------------
def prefers_pull(slots_per_rank: int, experts_per_rank: int, out_hidden: int, sm_count: int) -> bool:
    """True when the down GEMM of one rank is expected to fit in one wave of 128 x 256 tiles (one persistent
    CTA per SM), the case in which pulled results beat pushed ones.  Balanced routing is assumed: a rank
    receives as many rows as it sends, plus at most one padding block per local expert."""
    m_blocks = (slots_per_rank + 127) // 128 + experts_per_rank
    return m_blocks * ((out_hidden + 255) // 256) <= sm_count


class EpPeerContext:
    """Symmetric buffers and pointer tables for the peer-memory exchange (see csrc/ep_moe.cu).

    Every rank allocates the same buffers through torch's symmetric-memory allocator (plumbing
    only: it hands out device memory that every rank of the node can address) and keeps, for
    each buffer, the device pointers of all ranks' copies.  Capacity covers the worst case of
    every slot of every rank landing on one rank.
    """

    def __init__(self, group, num_experts: int, device, max_tokens_per_rank: int, top_k: int, hidden: int,
                 out_hidden: int, inter: int, dtype=torch.bfloat16, pull: bool = None):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from .. import _lib

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device
        self.num_experts = num_experts
        if num_experts % self.world != 0:
            raise AssertionError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.experts_per_rank = num_experts // self.world
        self.top_k, self.hidden, self.out_hidden, self.inter, self.dtype = top_k, hidden, out_hidden, inter, dtype
        self.max_slots = max_tokens_per_rank * top_k
        cap = self.world * self.max_slots + self.experts_per_rank * 128
        self.cap = (cap + 127) // 128 * 128
        if self.cap >= 1 << 24:
            raise AssertionError("receive capacity exceeds the 24-bit slot field of the row metadata")

        def sym(shape, dt):
            t = symm_mem.empty(shape, dtype=dt, device=device)
            hdl = symm_mem.rendezvous(t, group)
            ptrs = []
            for r in range(self.world):
                remote = hdl.get_buffer(r, t.shape, t.dtype)
                ptrs.append(remote.data_ptr())
            if ptrs[self.rank] != t.data_ptr():
                raise AssertionError("symmetric buffer pointer table does not contain the local buffer")
            table = (ctypes.c_void_p * self.world)(*ptrs)
            return t, hdl, table

        self.counts, self._h_counts, self.counts_tbl = sym((self.world * num_experts,), torch.int32)
        self.flags, self._h_flags, self.flags_tbl = sym((8 * 16,), torch.int32)
        self.rows, self._h_rows, self.rows_tbl = sym((self.cap, hidden), dtype)
        self.w, self._h_w, self.w_tbl = sym((self.cap,), torch.float32)
        self.meta, self._h_meta, self.meta_tbl = sym((self.cap,), torch.int32)
        # results travel back in one of two ways: pulled by the combine out of the owners' output buffer
        # `y`, or pushed by the down GEMM's epilogue into the senders' `back` buffers.  The push rides under
        # the main loop of the GEMM's later tiles, the pull is a separate pass; so the push wins whenever the
        # down GEMM has more than one wave of tiles (measured at 4 GPUs: 0.78 ms pushed, 0.90 ms pulled), and
        # the pull wins when all tiles finish together and nothing is left to hide the pushes behind
        # (8 GPUs: 0.478 ms pushed, 0.455 ms pulled).  Default: decide from the expected tile count.
        if pull is None:
            sms = torch.cuda.get_device_properties(device).multi_processor_count
            pull = prefers_pull(self.max_slots, self.experts_per_rank, out_hidden, sms)
        self.pull = bool(pull)
        if pull:
            self.y, self._h_y, self.y_tbl = sym((self.cap, out_hidden), dtype)
            result_buf = self.y
        else:
            self.back, self._h_back, self.back_tbl = sym((self.max_slots, out_hidden), dtype)
            result_buf = self.back
        for t in (self.counts, self.flags, self.rows, self.w, self.meta, result_buf):
            t.zero_()
        # plan outputs and the activation buffer are ordinary local memory
        self.dest_pos = torch.empty(max(self.max_slots, 1), dtype=torch.int32, device=device)
        self.counters = torch.zeros(2, dtype=torch.int32, device=device)     # last-CTA counters (send, down GEMM)
        # flag slot 2, entry `rank`, of every rank: raised by this rank's down GEMM
        self.signal2_tbl = (ctypes.c_void_p * self.world)(
            *[int(self.flags_tbl[r]) + 4 * (2 * 16 + self.rank) for r in range(self.world)])
        self.block_start = torch.empty(self.experts_per_rank + 1, dtype=torch.int32, device=device)
        self.num_post = torch.empty(1, dtype=torch.int32, device=device)
        self.row_map = torch.empty(self.cap, dtype=torch.int32, device=device)
        self.act = torch.empty((self.cap, inter), dtype=dtype, device=device)
        self.epoch = 0
        self.status = _lib.status_word(device)
        torch.cuda.synchronize(device)
        dist.barrier(group)


PEER_KERNELS_PER_STEP = 5  # route, send, gemm (gate/up), gemm (down + peer scatter), combine


def ep_fused_moe_peer(ctx: EpPeerContext, hidden_states, w1_local, w2_local, topk_weights, topk_ids, topk: int):
    """Expert-parallel fused_moe whose token exchange runs inside our own kernels over peer memory.

    Same contract as `ep_fused_moe`.  Five launches per step, nothing returns to the host in between:
      route    count slots per expert, exchange counts (peer stores + cross-GPU barrier), receive
               layout, destination row of every slot
      send     rows, weights and (rank, slot) tags stored into the owners' buffers; last CTA raises a flag
      GEMM     gate/up + silu on the received rows (its producer waits for every rank's flag first)
      GEMM     down x weight into this rank's output buffer; last CTA raises a flag on every rank
      combine  waits for every rank's flag, then reads each token's top-k rows out of the owners' output
               buffers (peer loads) and sums them
    With `ctx.pull` off the down GEMM's epilogue instead stores each row into the SENDER's result buffer
    and the combine reads locally.  `EpPeerContext` picks the form from the number of tiles the down GEMM
    is expected to have (one wave or less: pull).

    Every rank of the group must call this once per step, in the same order.  The kernels wait for each
    other on flags in peer memory; a wait gives up after the wait budget (2 s unless changed with
    `_lib.set_wait_budget_ms` or DLBLAS_B200_WAIT_BUDGET_MS), which is therefore the largest skew between
    ranks a step tolerates.  A wait that gave up does not stop the step: the kernels go on with whatever had
    arrived and record the fact in the device status word, so a caller has to call `check_device_status()`
    (it synchronises) before it trusts the output; it raises `DlblasError` if any wait of the step timed out.
    Ids outside [0, num_experts) are sent nowhere and add nothing to their token's output.
    """
    from .. import _lib

    lib = _lib.load()
    dev = hidden_states.device
    T, H = hidden_states.shape
    numel = T * topk
    assert numel <= ctx.max_slots and H == ctx.hidden and topk == ctx.top_k
    assert hidden_states.dtype == ctx.dtype and hidden_states.stride(1) == 1
    assert w1_local.is_contiguous() and w2_local.is_contiguous()
    ids = topk_ids.reshape(-1)
    if ids.dtype not in (torch.int32, torch.int64):
        ids = ids.to(torch.int64)
    ids = ids.contiguous()
    tw = topk_weights.to(torch.float32).reshape(-1).contiguous()
    ctx.epoch += 1
    epoch, world, rank = ctx.epoch, ctx.world, ctx.rank
    stream = _lib.stream_ptr(dev)
    is64 = int(ids.dtype == torch.int64)
    dt = _lib.dtype_code(ctx.act)
    E_local, N1, _ = w1_local.shape
    _, H_out, inter = w2_local.shape
    out = torch.empty((T, H_out), dtype=ctx.dtype, device=dev)
    flags_local = ctx.flags.data_ptr()
    with torch.cuda.device(dev):
        rc = lib.dlb_ep_route(ids.data_ptr(), is64, numel, ctx.counts_tbl, ctx.flags_tbl, ctx.dest_pos.data_ptr(),
                              ctx.block_start.data_ptr(), ctx.num_post.data_ptr(), ctx.row_map.data_ptr(), rank, world,
                              ctx.num_experts, ctx.cap, epoch, ctx.status.data_ptr(), stream)
        _lib.check(rc, "ep_route")
        rc = lib.dlb_ep_send(hidden_states.data_ptr(), hidden_states.stride(0), H, hidden_states.element_size(),
                             ids.data_ptr(), is64, tw.data_ptr(), ctx.dest_pos.data_ptr(), ctx.rows_tbl, ctx.w_tbl,
                             ctx.meta_tbl, ctx.flags_tbl, ctx.counters[0:1].data_ptr(), numel, topk, rank, world,
                             ctx.num_experts, ctx.cap, epoch, stream)
        _lib.check(rc, "ep_send")
        rc = lib.dlb_moe_grouped_gemm_sync(
            ctx.rows.data_ptr(), ctx.cap, ctx.rows.stride(0), w1_local.data_ptr(), E_local, N1, H, w1_local.stride(1),
            ctx.act.data_ptr(), None, 0, ctx.act.stride(0), ctx.inter, ctx.row_map.data_ptr(),
            ctx.block_start.data_ptr(), None, None, ctx.cap, _lib.GEMM_FUSE_SILU, dt,
            flags_local + 4 * (1 * 16), None, None, world, epoch, ctx.status.data_ptr(), stream)
        _lib.check(rc, "moe_grouped_gemm_sync(gate/up)")
        if ctx.pull:
            rc = lib.dlb_moe_grouped_gemm_sync(
                ctx.act.data_ptr(), ctx.cap, ctx.act.stride(0), w2_local.data_ptr(), E_local, H_out, inter,
                w2_local.stride(1), ctx.y.data_ptr(), None, 0, ctx.y.stride(0), H_out, ctx.row_map.data_ptr(),
                ctx.block_start.data_ptr(), ctx.w.data_ptr(), None, ctx.cap, _lib.GEMM_WEIGHT, dt, None,
                ctx.signal2_tbl, ctx.counters[1:2].data_ptr(), world, epoch, ctx.status.data_ptr(), stream)
        else:
            rc = lib.dlb_moe_grouped_gemm_sync(
                ctx.act.data_ptr(), ctx.cap, ctx.act.stride(0), w2_local.data_ptr(), E_local, H_out, inter,
                w2_local.stride(1), None, ctx.back_tbl, world, ctx.back.stride(0), H_out, ctx.row_map.data_ptr(),
                ctx.block_start.data_ptr(), ctx.w.data_ptr(), ctx.meta.data_ptr(), ctx.cap,
                _lib.GEMM_WEIGHT | _lib.GEMM_PEER, dt, None, ctx.signal2_tbl, ctx.counters[1:2].data_ptr(), world,
                epoch, ctx.status.data_ptr(), stream)
        _lib.check(rc, "moe_grouped_gemm_sync(down)")
        if ctx.pull:
            rc = lib.dlb_ep_combine_pull(ctx.y_tbl, ctx.y.stride(0), ids.data_ptr(), is64, ctx.dest_pos.data_ptr(),
                                         out.data_ptr(), T, topk, H_out, out.stride(0), dt,
                                         flags_local + 4 * (2 * 16), world, ctx.num_experts, ctx.cap, epoch,
                                         ctx.status.data_ptr(), stream)
        else:
            rc = lib.dlb_ep_combine(ctx.back.data_ptr(), out.data_ptr(), T, topk, H_out, out.stride(0), dt,
                                    flags_local + 4 * (2 * 16), world, epoch, ctx.dest_pos.data_ptr(),
                                    ctx.status.data_ptr(), stream)
        _lib.check(rc, "ep_combine")
    return out
