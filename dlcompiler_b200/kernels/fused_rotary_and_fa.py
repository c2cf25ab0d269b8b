"""`fused_rotary_and_fa` with the call convention of
python/dlBLAS/dlblas/kernels/fused_rotary_and_fa.py:391 (`call(q, k, v, cos, sin)`).

Reference semantics (fused_rotary_and_fa.py:120-182): rotate-half rotary embedding of q once and
of every k tile, `x0' = x0*cos0 - x1*sin0`, `x1' = x0*sin1 + x1*cos1`, evaluated in the tensors'
16-bit type, then dense non-causal softmax attention over the rotated q and k.

Here the two steps are two launches on the caller's stream: the rotary kernel writes rotated copies
of q and k, the tcgen05 attention kernel reads them.  The rotation is not folded into the attention
kernel: its Q and K tiles go from global memory to swizzled shared memory by TMA and from there
straight into the tensor cores, so a rotation in between would be an extra shared-memory read-modify-
write pass with a proxy fence per tile, repeated for every query tile and query head that re-reads a
K tile, whereas the stand-alone pass touches every element once at HBM speed (7 % of the attention
time at 4 x 8192 tokens).
"""
from __future__ import annotations

import torch

from .apply_rotary_pos_emb import apply_rotary_pos_emb
from .flash_attention import flash_attention_v2


def fused_rotary_and_fa(q, k, v, cos, sin, causal=False, softmax_scale=None):
    """q, k, v [b, s, h, d]; cos, sin [b, s, d] (fused_rotary_and_fa.py:404-412) -> o [b, s, h, d]."""
    batch, seqlen, nheads, d = q.shape
    assert k.shape == (batch, seqlen, nheads, d) and v.shape == k.shape
    assert q.dtype in (torch.float16, torch.bfloat16), "Only support fp16 and bf16"
    assert cos.shape == (batch, seqlen, d) and sin.shape == cos.shape
    q3 = q.reshape(batch * seqlen, nheads, d)
    k3 = k.reshape(batch * seqlen, nheads, d)
    q_rot, k_rot = apply_rotary_pos_emb(q3, k3, cos.reshape(batch * seqlen, d), sin.reshape(batch * seqlen, d))
    return flash_attention_v2(q_rot.view(batch, seqlen, nheads, d), k_rot.view(batch, seqlen, nheads, d), v,
                              causal=causal, softmax_scale=softmax_scale)


def call(q, k, v, cos, sin):
    """Reference entry point (fused_rotary_and_fa.py:391)."""
    return fused_rotary_and_fa(q, k, v, cos, sin)
