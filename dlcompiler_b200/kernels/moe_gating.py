"""MoE routers: group-limited sigmoid top-k (DeepSeek-V3 style) and softmax top-k.

The reference builds its fused_moe routing weights in torch
(python/dlBLAS/tests/kernels/test_fused_moe.py:207-218: softmax in fp32, then
`torch.topk`); `softmax_topk` is that as one kernel.  The group-limited sigmoid
router has no counterpart in the reference; its definition is the one in the
docstring of `grouped_topk_gating`.
"""
from __future__ import annotations

import torch

from .. import _lib


def grouped_topk_gating(logits: torch.Tensor, bias: torch.Tensor | None, top_k: int, n_group: int = 1,
                        topk_group: int = 1, routed_scaling_factor: float = 1.0, renormalize: bool = True,
                        scoring_func: str = "sigmoid"):
    """Group-limited top-k routing.

    scores = sigmoid(logits) (or softmax); selection score = scores + bias; each of the
    `n_group` equal groups is scored by the sum of its two largest selection scores and
    the best `topk_group` groups are kept; the `top_k` experts with the largest selection
    score inside the kept groups are chosen (ties go to the lower index; output is in
    descending order of selection score).  Weights are the un-biased scores of the chosen
    experts, divided by their sum when `renormalize`, times `routed_scaling_factor`.

    Returns (topk_ids int32 [T, top_k], topk_weights fp32 [T, top_k]).
    """
    assert logits.dim() == 2 and logits.dtype == torch.float32
    _lib.require_cuda(logits, bias)
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    T, E = logits.shape
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == E
        bias = bias.contiguous()
    ids = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    scoring = {"sigmoid": _lib.SCORE_SIGMOID, "softmax": _lib.SCORE_SOFTMAX}[scoring_func]
    lib = _lib.load()
    with torch.cuda.device(logits.device):
        rc = lib.dlb_grouped_topk_gating(logits.data_ptr(), _lib.ptr(bias), ids.data_ptr(), weights.data_ptr(), T, E,
                                         logits.stride(0) if T > 1 else E, n_group, topk_group, top_k, scoring,
                                         int(renormalize), float(routed_scaling_factor),
                                         _lib.stream_ptr(logits.device))
    _lib.check(rc, "grouped_topk_gating")
    return ids, weights


def softmax_topk(router_logits: torch.Tensor, top_k: int, renormalize: bool = False):
    """softmax over experts in fp32, then top-k: (topk_weights fp32, topk_ids int32)."""
    ids, w = grouped_topk_gating(router_logits.float(), None, top_k, 1, 1, 1.0, renormalize, "softmax")
    return w, ids
