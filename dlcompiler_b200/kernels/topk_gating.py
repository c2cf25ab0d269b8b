"""GShard-style top-k gating with capacity: the reference's `dlblas.topk_gating`
(python/dlBLAS/dlblas/__init__.py:13-23, python/dlBLAS/dlblas/kernels/topk_gating.py:259-294)."""
from __future__ import annotations

import torch

from .. import _lib
from .fused_moe import _moe_align


def _capacity(num_tokens: int, num_experts: int, capacity_factor: float, min_capacity: int) -> int:
    """ceil(tokens / experts * capacity_factor), at least min_capacity (topk_gating.py:13-22; the product is
    formed with an fp32 tensor there, reproduced here so the integer agrees)."""
    cap = torch.ceil((num_tokens / num_experts) * torch.tensor(capacity_factor)).to(torch.int64)
    return max(int(cap), int(min_capacity))


class TopKGatingFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: torch.Tensor, k: int, capacity_factor: float = 1.0, min_capacity: int = 2,
                higher_precision: bool = False):
        dev = _lib.require_cuda(logits)
        assert logits.dim() == 2
        S, E = logits.shape
        capacity = _capacity(S, E, capacity_factor * k, min_capacity)
        x = logits.float().contiguous()
        lib = _lib.load()
        stream = _lib.stream_ptr(dev)
        gates = torch.empty((S, E), dtype=torch.float32, device=dev)
        ids = torch.empty((S, k), dtype=torch.int32, device=dev)
        scratch_w = torch.empty((S, k), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.dlb_gshard_gate(x.data_ptr(), S, E, k, gates.data_ptr(), ids.data_ptr(),
                                           scratch_w.data_ptr(), stream), "topk_gating(gate)")
        ids_km = ids.t().contiguous().view(-1)                        # choice-major: all first choices, then second, ...
        sorted_ids, _, _, prefix = _moe_align(ids_km, 1, E)
        nblk = max(1, min(256, S // 64))
        colsum = torch.empty((nblk, E), dtype=torch.float32, device=dev)
        loc = torch.empty(k * S, dtype=torch.int32, device=dev)
        me = torch.empty(E, dtype=torch.float32, device=dev)
        ce = torch.empty(E, dtype=torch.float32, device=dev)
        l_aux = torch.empty((), dtype=torch.float32, device=dev)
        ec_idx = torch.empty(k * S, dtype=torch.int32, device=dev)
        weights = torch.empty(k * S, dtype=torch.float32, device=dev)
        select = torch.empty(E * capacity, dtype=torch.int64, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.dlb_gshard_assign(gates.data_ptr(), ids_km.data_ptr(), sorted_ids.data_ptr(),
                                             prefix.data_ptr(), S, E, k, capacity, colsum.data_ptr(), nblk,
                                             loc.data_ptr(), me.data_ptr(), ce.data_ptr(), l_aux.data_ptr(),
                                             ec_idx.data_ptr(), weights.data_ptr(), select.data_ptr(), stream),
                       "topk_gating(assign)")
        ctx.out_dtype = logits.dtype
        ctx.higher_precision = bool(higher_precision)
        ctx.mark_non_differentiable(ec_idx, select)
        if higher_precision:
            ctx.save_for_backward(gates, ce, ids_km, loc)
            ctx.top_k, ctx.capacity = k, capacity
        else:
            ctx.save_for_backward(gates, ce)
        return l_aux.to(logits.dtype), ec_idx, weights.to(logits.dtype), select

    @staticmethod
    def backward(ctx, grad_l_aux, grad_ec_idx=None, grad_weights=None, grad_select=None):
        gates = ctx.saved_tensors[0]
        ce = ctx.saved_tensors[1]
        dev = gates.device
        S, E = gates.shape
        g = (torch.zeros(1, device=dev) if grad_l_aux is None else grad_l_aux.float().reshape(1)).contiguous()
        grad_logits = torch.empty_like(gates)
        lib = _lib.load()
        with torch.cuda.device(dev):
            if ctx.higher_precision:
                # the routing weights back-propagate too (topk_gating.py:286-294).  The gradient is the exact
                # derivative of weights = kept gate / max(sum of kept gates, eps); the reference's kernel divides
                # the saved, already normalised gates by the denominator twice more (topk_gating.py:164-166 with
                # gate_ks stored after the division at :75-77), which is not the derivative of its own forward.
                ids_km, loc = ctx.saved_tensors[2], ctx.saved_tensors[3]
                gw = (torch.zeros(ctx.top_k * S, device=dev) if grad_weights is None
                      else grad_weights.float().reshape(-1)).contiguous()
                _lib.check(lib.dlb_gshard_gate_bwd_weights(gates.data_ptr(), ce.data_ptr(), g.data_ptr(),
                                                           ids_km.data_ptr(), loc.data_ptr(), gw.data_ptr(),
                                                           grad_logits.data_ptr(), S, E, ctx.top_k, ctx.capacity,
                                                           _lib.stream_ptr(dev)), "topk_gating(backward, weights)")
            else:
                # as in the reference's default path, only the auxiliary loss back-propagates (topk_gating.py:279-284)
                _lib.check(lib.dlb_gshard_gate_bwd(gates.data_ptr(), ce.data_ptr(), g.data_ptr(),
                                                   grad_logits.data_ptr(), S, E, _lib.stream_ptr(dev)),
                           "topk_gating(backward)")
        return grad_logits.to(ctx.out_dtype), None, None, None, None


def topk_gating(logits: torch.Tensor, k: int, capacity_factor: float = 1.0, min_capacity: int = 2,
                higher_precision: bool = False):
    """Returns (l_aux, token_rearranged_ec_idx int32 [k*s], token_exp_weights [k*s],
    expert_select_token_idx int64 [e*c]) like the reference op.  Ties between equal gate values go to
    the lower expert index; `expert_select_token_idx` lists each expert's kept tokens in arrival order
    (the reference's `torch.topk` leaves the order among equal priorities unspecified)."""
    return TopKGatingFunc.apply(logits, k, capacity_factor, min_capacity, higher_precision)
