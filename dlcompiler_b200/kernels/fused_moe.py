"""fused_moe and helpers with the signatures of python/dlBLAS/dlblas/kernels/fused_moe.py.

Pipeline of `fused_moe` (all five steps are CUDA kernels of libdlblas_b200.so):
  moe_align_block_size -> row permute -> grouped GEMM (gate/up, fused silu*mul)
  -> grouped GEMM (down, x routing weight, scatter by slot) -> top-k combine.
"""
from __future__ import annotations

import torch

from .. import _lib

BLOCK_M = 128  # rows per expert block of the grouped GEMM


def _align_capacity(numel: int, num_experts: int, block: int) -> int:
    cap = numel + num_experts * (block - 1)
    return (cap + block - 1) // block * block


def _moe_align(topk_ids: torch.Tensor, block: int, num_experts: int):
    """Run the align kernel; returns (sorted_token_ids, expert_ids, num_post_padded, block_start)."""
    ids = topk_ids.reshape(-1)
    if ids.dtype not in (torch.int32, torch.int64):
        ids = ids.to(torch.int64)
    ids = ids.contiguous()
    numel = ids.numel()
    dev = ids.device
    cap = _align_capacity(numel, num_experts, block)
    sorted_ids = torch.empty(cap, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(max(cap // block, 1), dtype=torch.int32, device=dev)
    meta = torch.empty(num_experts + 2, dtype=torch.int32, device=dev)
    num_post = meta[:1]
    block_start = meta[1:]
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.dlb_moe_align_block_size(ids.data_ptr(), int(ids.dtype == torch.int64), numel, num_experts, block,
                                          sorted_ids.data_ptr(), cap, expert_ids.data_ptr(), expert_ids.numel(),
                                          num_post.data_ptr(), block_start.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "moe_align_block_size")
    return sorted_ids, expert_ids, num_post, block_start


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """Sort the (token, k) slots by expert and pad each expert to a multiple of `block_size`.

    Returns (sorted_token_ids int32 [cap], expert_ids int32 [cap / block_size],
    num_tokens_post_padded int32 [1]); padding entries hold `topk_ids.numel()`, unused
    `expert_ids` entries hold -1, order inside an expert is ascending slot index.
    This is the block-padded form of the reference's argsort + start/end ranges
    (fused_moe.py:314-320, 267-293).
    """
    _lib.require_cuda(topk_ids)
    s, e, n, _ = _moe_align(topk_ids, block_size, num_experts)
    return s, e, n


def _permute_rows(src, row_map, num_post, numel, div, cap):
    hidden = src.size(-1)
    dst = torch.empty((cap, hidden), dtype=src.dtype, device=src.device)
    lib = _lib.load()
    with torch.cuda.device(src.device):
        rc = lib.dlb_moe_permute_rows(src.data_ptr(), dst.data_ptr(), row_map.data_ptr(), num_post.data_ptr(), numel,
                                      div, hidden, src.stride(0), cap, src.element_size(),
                                      _lib.stream_ptr(src.device))
    _lib.check(rc, "moe_permute_rows")
    return dst


def _grouped_gemm(a, b, out, n_out, row_map, block_start, weights, numel, flags):
    E, rows_per_expert, K = b.shape
    assert b.stride(2) == 1 and b.stride(0) == rows_per_expert * b.stride(1), "B must be [E, N, K] with dense experts"
    assert a.stride(1) == 1 and out.stride(-1) == 1
    lib = _lib.load()
    status = _lib.status_word(a.device)
    with torch.cuda.device(a.device):
        rc = lib.dlb_moe_grouped_gemm(a.data_ptr(), a.size(0), a.stride(0), b.data_ptr(), E, rows_per_expert, K,
                                      b.stride(1), out.data_ptr(), out.stride(0), n_out, row_map.data_ptr(),
                                      block_start.data_ptr(), _lib.ptr(weights), numel, flags,
                                      _lib.dtype_code(a), status.data_ptr(), _lib.stream_ptr(a.device))
    _lib.check(rc, "moe_grouped_gemm")


def fused_moe(hidden_states: torch.Tensor,
              w1: torch.Tensor,
              w2: torch.Tensor,
              topk_weights: torch.Tensor,
              topk_ids: torch.Tensor,
              topk: int,
              expert_offset: int = 0,
              num_experts: int = None,
              renormalize: bool = False) -> torch.Tensor:
    """Mixture-of-experts MLP: out[t] = sum_k w[t,k] * down_e(silu(gate_e(x_t)) * up_e(x_t)), e = ids[t,k].

    Arguments as in the reference (fused_moe.py:296-304): `w1` is [E, 2*I, H] with the gate
    projection in the first I rows of each expert, `w2` is [E, H_out, I]; `expert_offset` /
    `num_experts` select the slice [expert_offset, expert_offset + E) of a larger global expert
    set (ids outside the slice contribute zero, as in the reference's expert-parallel mode).
    Rounding points match the reference: GEMM outputs are rounded to the activation dtype,
    silu and the product are rounded separately, routing weights are applied in fp32 before the
    cast, and the top-k sum accumulates in fp32.  A slot whose id lies outside the slice adds
    nothing to its token (the reference zero-fills its intermediates for that, fused_moe.py:329-332;
    here the combine skips the slot, so no buffer needs clearing).
    """
    dev = _lib.require_cuda(hidden_states, w1, w2, topk_weights, topk_ids)
    assert hidden_states.dim() == 2 and w1.dim() == 3 and w2.dim() == 3
    assert hidden_states.dtype in (torch.float16, torch.bfloat16)
    assert w1.dtype == hidden_states.dtype and w2.dtype == hidden_states.dtype
    M, H = hidden_states.shape
    E, N, K1 = w1.shape
    assert K1 == H and N % 2 == 0
    inter = N // 2
    E2, H_out, K2 = w2.shape
    assert E2 == E and K2 == inter
    assert topk_ids.shape == (M, topk) and topk_weights.shape == (M, topk)
    if num_experts is None:
        num_experts = E

    if renormalize:
        topk_weights = topk_weights / topk_weights.sum(dim=-1, keepdim=True)
    topk_weights = topk_weights.to(torch.float32).contiguous()
    if hidden_states.stride(1) != 1:
        hidden_states = hidden_states.contiguous()
    w1 = w1 if w1.is_contiguous() else w1.contiguous()
    w2 = w2 if w2.is_contiguous() else w2.contiguous()

    local_ids = topk_ids if expert_offset == 0 else topk_ids - expert_offset
    numel = M * topk
    out = hidden_states.new_empty((M, H_out))
    if M == 0:
        return out
    sorted_ids, _, num_post, block_start = _moe_align(local_ids, BLOCK_M, E)
    cap = sorted_ids.numel()

    a_sorted = _permute_rows(hidden_states, sorted_ids, num_post, numel, topk, cap)
    act = torch.empty((cap, inter), dtype=hidden_states.dtype, device=dev)
    _grouped_gemm(a_sorted, w1, act, inter, sorted_ids, block_start, None, numel, _lib.GEMM_FUSE_SILU)
    partial = torch.empty((numel, H_out), dtype=hidden_states.dtype, device=dev)
    _grouped_gemm(act, w2, partial, H_out, sorted_ids, block_start, topk_weights, numel,
                  _lib.GEMM_WEIGHT | _lib.GEMM_SCATTER)
    ids = topk_ids if topk_ids.dtype in (torch.int32, torch.int64) else topk_ids.to(torch.int64)
    ids = ids.contiguous()
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.dlb_moe_combine(partial.data_ptr(), out.data_ptr(), M, topk, H_out, out.stride(0),
                                 _lib.dtype_code(out), ids.data_ptr(), int(ids.dtype == torch.int64),
                                 expert_offset, expert_offset + E, _lib.stream_ptr(dev))
    _lib.check(rc, "moe_combine")
    return out


def get_start_end(topk_idx: torch.Tensor, sorted_idx: torch.Tensor, num_experts: int):
    """Per-expert [start, end) ranges inside `sorted_idx` (fused_moe.py:267-293).

    One kernel launch, no host synchronisation.  `sorted_idx` (the argsort of the flattened ids) only
    gives the dtype of the result, as in the reference (`sorted_idx.new_empty`): the ranges follow from
    the ids alone, start = number of smaller ids (negative ones included), and an expert without slots
    gets start = end = 0 as the reference's kernel leaves it.
    """
    _lib.require_cuda(topk_idx, sorted_idx)
    flat = topk_idx.flatten()
    if flat.dtype not in (torch.int32, torch.int64):
        flat = flat.to(torch.int64)
    flat = flat.contiguous()
    out_dtype = torch.int64 if sorted_idx.dtype == torch.int64 else torch.int32
    start_end = torch.empty((2, num_experts), dtype=out_dtype, device=flat.device)
    lib = _lib.load()
    with torch.cuda.device(flat.device):
        rc = lib.dlb_moe_start_end(flat.data_ptr(), int(flat.dtype == torch.int64), flat.numel(), num_experts,
                                   start_end[0].data_ptr(), start_end[1].data_ptr(), int(out_dtype == torch.int64),
                                   _lib.stream_ptr(flat.device))
    _lib.check(rc, "get_start_end")
    if out_dtype != sorted_idx.dtype:
        start_end = start_end.to(sorted_idx.dtype)
    return start_end[0], start_end[1]


def fused_moe_kernel_launcher(
    A: torch.Tensor,
    B: torch.Tensor,
    C: torch.Tensor,
    sorted_idx: torch.Tensor,
    exp_start: torch.Tensor,
    exp_end: torch.Tensor,
    weights: torch.Tensor,
    enable_weights: bool = False,
    top_k: int = 1,
    num_tokens: int = None,
    expert_offset: int = 0,
    reindex_a: bool = True,
    reindex_c: bool = True,
):
    """One grouped GEMM with the reference launcher's contract (fused_moe.py:178-235).

    `sorted_idx` lists slot ids grouped by expert, `exp_start/exp_end` give each expert's range
    in it.  Row i of that list reads A[sorted_idx[i] // top_k] (reindex_a) or A[i], and writes
    C[sorted_idx[i]] (reindex_c) or C[i]; with `enable_weights` the fp32 accumulator is scaled
    by weights.flatten()[sorted_idx[i]] before the cast.  The ranges are re-laid-out into
    128-row blocks on the device (index arithmetic only) and fed to the tensor-core kernel.
    """
    dev = _lib.require_cuda(A, B, C, sorted_idx, exp_start, exp_end)
    E, N, K = B.shape
    A = A.flatten(0, -2)
    C2 = C.flatten(0, -2)
    assert C2.data_ptr() == C.data_ptr(), "C must be viewable as 2-D without a copy"
    n_sorted = sorted_idx.numel()
    # ranges of the local experts, padded to 128-row blocks
    starts = exp_start[expert_offset:expert_offset + E].to(torch.int64)
    ends = exp_end[expert_offset:expert_offset + E].to(torch.int64)
    counts = (ends - starts).clamp_(min=0)
    nblk = (counts + BLOCK_M - 1) // BLOCK_M
    blk_end = nblk.cumsum(0)
    block_start = torch.cat([blk_end.new_zeros(1), blk_end]).to(torch.int32)
    seg_off = (blk_end - nblk) * BLOCK_M
    cap = _align_capacity(n_sorted, E, BLOCK_M)
    pos = torch.arange(n_sorted, device=dev, dtype=torch.int64)
    owner = torch.searchsorted(ends, pos, right=True).clamp_(max=E - 1)
    in_range = (pos >= starts[owner]) & (pos < ends[owner])
    padded_pos = seg_off[owner] + (pos - starts[owner])
    padded_pos = torch.where(in_range, padded_pos, torch.full_like(padded_pos, cap))  # dropped below
    sentinel = n_sorted
    slot_map = torch.full((cap + 1,), sentinel, dtype=torch.int32, device=dev)
    pos_map = torch.full((cap + 1,), sentinel, dtype=torch.int32, device=dev)
    slot_map[padded_pos] = sorted_idx.to(torch.int32)
    pos_map[padded_pos] = pos.to(torch.int32)
    slot_map, pos_map = slot_map[:cap].contiguous(), pos_map[:cap].contiguous()
    num_post = (block_start[-1:] * BLOCK_M).to(torch.int32)

    if A.stride(1) != 1:
        A = A.contiguous()
    a_sorted = _permute_rows(A, slot_map if reindex_a else pos_map, num_post, sentinel,
                             top_k if reindex_a else 1, cap)
    flags = _lib.GEMM_SCATTER
    w = None
    if enable_weights:
        flags |= _lib.GEMM_WEIGHT
        w = weights.to(torch.float32).contiguous().flatten()
        if not reindex_c:
            # weights are indexed by slot id; gather them into sorted order for position-indexed output
            w = w[sorted_idx.to(torch.int64)].contiguous()
    if enable_weights and reindex_c:
        row_map = slot_map
    else:
        row_map = slot_map if reindex_c else pos_map
    Bc = B if B.is_contiguous() else B.contiguous()
    _grouped_gemm(a_sorted, Bc, C2, N, row_map, block_start, w, sentinel, flags)
