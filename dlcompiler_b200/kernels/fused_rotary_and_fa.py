"""`fused_rotary_and_fa` with the call convention of
python/dlBLAS/dlblas/kernels/fused_rotary_and_fa.py:391 (`call(q, k, v, cos, sin)`).

Reference semantics (fused_rotary_and_fa.py:120-182): rotate-half rotary embedding of q once and
of every k tile, `x0' = x0*cos0 - x1*sin0`, `x1' = x0*sin1 + x1*cos1`, evaluated in the tensors'
16-bit type, then dense non-causal softmax attention over the rotated q and k.

Here q is rotated inside the attention kernel: its tile is loaded once per CTA, and the softmax warps
rotate it in place in shared memory before the first MMA.  k is rotated once per token by the rotary
kernel (keys only) instead of once per tile inside the loop: every k tile is re-read by all the query
tiles and heads that attend to it, so a rotation inside the loop would repeat the same arithmetic up to
seqlen / 128 times; in a serving stack `fill_kv_cache(..., cos=, sin=)` does that one pass while it writes
the cache, and no stand-alone pass is left.
"""
from __future__ import annotations

import torch

from .. import _lib
from .flash_attention import flash_attention_v2


def fused_rotary_and_fa(q, k, v, cos, sin, causal=False, softmax_scale=None):
    """q, k, v [b, s, h, d]; cos, sin [b, s, d] (fused_rotary_and_fa.py:404-412) -> o [b, s, h, d]."""
    batch, seqlen, nheads, d = q.shape
    assert k.shape == (batch, seqlen, nheads, d) and v.shape == k.shape
    assert q.dtype in (torch.float16, torch.bfloat16), "Only support fp16 and bf16"
    assert cos.shape == (batch, seqlen, d) and sin.shape == cos.shape
    dev = _lib.require_cuda(q, k, v, cos, sin)
    tokens = batch * seqlen
    k3 = k.reshape(tokens, nheads, d)
    cos2 = cos.to(q.dtype).reshape(tokens, d).contiguous()
    sin2 = sin.to(q.dtype).reshape(tokens, d).contiguous()
    k_rot = torch.empty_like(k3)
    lib = _lib.load()
    with torch.cuda.device(dev):
        # keys only: no query heads in this launch
        rc = lib.dlb_apply_rotary(None, k3.data_ptr(), cos2.data_ptr(), sin2.data_ptr(), None, k_rot.data_ptr(),
                                  tokens, 0, nheads, d, 0, 0, k3.stride(0), k3.stride(1), 0, 0, k_rot.stride(0),
                                  k_rot.stride(1), _lib.dtype_code(q), _lib.stream_ptr(dev))
    _lib.check(rc, "fused_rotary_and_fa(keys)")
    if d % 16 == 0:
        return flash_attention_v2(q, k_rot.view(batch, seqlen, nheads, d), v, causal=causal,
                                  softmax_scale=softmax_scale, q_cos=cos2, q_sin=sin2)
    # head sizes the in-kernel rotation does not cover: rotate q with the stand-alone kernel as well
    from .apply_rotary_pos_emb import apply_rotary_pos_emb

    q3 = q.reshape(tokens, nheads, d)
    q_rot, _ = apply_rotary_pos_emb(q3, k3, cos2, sin2)
    return flash_attention_v2(q_rot.view(batch, seqlen, nheads, d), k_rot.view(batch, seqlen, nheads, d), v,
                              causal=causal, softmax_scale=softmax_scale)


def call(q, k, v, cos, sin):
    """Reference entry point (fused_rotary_and_fa.py:391)."""
    return fused_rotary_and_fa(q, k, v, cos, sin)
