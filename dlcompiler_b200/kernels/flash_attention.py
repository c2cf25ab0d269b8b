"""Dense flash attention with the call conventions of python/dlBLAS/dlblas/kernels/flash_attention.py
([B, H, M, D], returns o; LSE in natural log with the scale included) and
python/dlBLAS/dlblas/kernels/flash_attention_v2.py ([b, s, h, d], non-causal through `call`).

Both run on the varlen tcgen05 prefill kernel: a dense batch is a set of equal-length sequences, and
the kernel takes arbitrary token / head strides through its tensor maps, so no data is copied.
"""
from __future__ import annotations

import math

import torch

from .prefill_attention import context_attention_fwd


def flash_attention_fwd(q, k, v, causal=False, sm_scale=None):
    """q [B, H, M, D], k/v [B, Hk, N, D] -> (o [B, H, M, D], L fp32 [B, H, M]).

    Shape rules of the reference wrapper (flash_attention.py:170-180): equal feature sizes, H a
    multiple of Hk.  This implementation needs M == N (no bottom-right aligned causal offset) and D in
    {64, 128}.  L = m * sm_scale + log(sum) (flash_attention.py:152-155).
    """
    Dq, Dk, Dv = q.shape[-1], k.shape[-1], v.shape[-1]
    assert Dq == Dk == Dv, "feature size of q, k, v should be equal"
    B, H, M, D = q.shape
    N = k.shape[2]
    Hk, Hv = k.shape[1], v.shape[1]
    assert Hk == Hv, "num of heads in k and v should be equal"
    assert H % Hk == 0, "number of heads in q must be a multiple of that in k & v"
    assert M == N, "this implementation needs equal query and key lengths"
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    o = torch.empty_like(q)
    L = torch.empty((B, H, M), device=q.device, dtype=torch.float32)
    start = torch.zeros(1, dtype=torch.int32, device=q.device)
    length = torch.full((1,), M, dtype=torch.int32, device=q.device)
    for b in range(B):
        # [H, M, D] viewed as [M, H, D]: token stride D, head stride M * D
        context_attention_fwd(q[b].transpose(0, 1), k[b].transpose(0, 1), v[b].transpose(0, 1),
                              o[b].transpose(0, 1), start, length, M, lse=L[b], causal=causal, sm_scale=sm_scale)
    return o, L


def call(q, k, v, causal, sm_scale, dropout_p):
    """Reference entry point (flash_attention.py:170): returns o.  Dropout is not implemented."""
    assert not dropout_p, "dropout is not supported"
    return flash_attention_fwd(q, k, v, causal, sm_scale)[0]


def flash_attention_v2(q, k, v, causal=False, softmax_scale=None, return_lse=False, q_cos=None, q_sin=None):
    """q, k, v [b, s, h, d] (flash_attention_v2.py:215-224); the reference's public `call(q, k, v)` is
    the non-causal case.  Accumulation is fp32 (the reference kernel accumulates in fp16).  `q_cos` /
    `q_sin` ([b, s, d]): rotate q inside the kernel (see `context_attention_fwd`)."""
    batch, seqlen_q, nheads, d = q.shape
    assert k.shape == (batch, seqlen_q, nheads, d) and v.shape == k.shape
    assert q.dtype == k.dtype == v.dtype and q.dtype in (torch.float16, torch.bfloat16)
    softmax_scale = softmax_scale or 1.0 / math.sqrt(d)
    q2, k2, v2 = (t.reshape(batch * seqlen_q, nheads, d) for t in (q, k, v))
    o = torch.empty_like(q2)
    start = torch.arange(batch, dtype=torch.int32, device=q.device) * seqlen_q
    length = torch.full((batch,), seqlen_q, dtype=torch.int32, device=q.device)
    lse = torch.empty((nheads, batch * seqlen_q), dtype=torch.float32, device=q.device) if return_lse else None
    context_attention_fwd(q2, k2, v2, o, start, length, seqlen_q, lse=lse, causal=causal, sm_scale=softmax_scale,
                          q_cos=q_cos, q_sin=q_sin)
    o = o.view(batch, seqlen_q, nheads, d)
    if return_lse:
        return o, lse.view(nheads, batch, seqlen_q).permute(1, 0, 2)
    return o
