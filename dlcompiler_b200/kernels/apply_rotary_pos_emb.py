"""apply_rotary_pos_emb with the signature of python/dlBLAS/dlblas/kernels/apply_rotary_pos_emb.py:98."""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _lib


def apply_rotary_pos_emb(
    q: Tensor,
    k: Tensor,
    cos: Tensor,
    sin: Tensor,
    q_embed: Tensor = None,
    k_embed: Tensor = None,
):
    """Rotate-half rotary embedding of query and key ([tokens, heads, dim]); `cos`/`sin` hold `dim`
    values per token (any leading shape with tokens * dim elements) and are used in q's dtype;
    outputs may be the inputs.  Returns (q_embed, k_embed)."""
    dev = _lib.require_cuda(q, k, q_embed, k_embed)
    if cos.device != q.device:
        cos = cos.to(device=q.device)
    if sin.device != q.device:
        sin = sin.to(device=q.device)
    if q_embed is None:
        q_embed = torch.empty_like(q)
    if k_embed is None:
        k_embed = torch.empty_like(k)
    dim = q.size(-1)
    tokens = cos.numel() // cos.size(-1)
    assert cos.size(-1) == dim and sin.numel() == cos.numel() and k.size(-1) == dim
    assert q.dim() == 3 and k.dim() == 3 and q.size(0) == tokens and k.size(0) == tokens
    assert q.stride(-1) == 1 and k.stride(-1) == 1 and q_embed.stride(-1) == 1 and k_embed.stride(-1) == 1
    cos = cos.to(q.dtype).contiguous()
    sin = sin.to(q.dtype).contiguous()
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.dlb_apply_rotary(q.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(), q_embed.data_ptr(),
                                  k_embed.data_ptr(), tokens, q.size(-2), k.size(-2), dim, q.stride(0), q.stride(1),
                                  k.stride(0), k.stride(1), q_embed.stride(0), q_embed.stride(1), k_embed.stride(0),
                                  k_embed.stride(1), _lib.dtype_code(q), _lib.stream_ptr(dev))
    _lib.check(rc, "apply_rotary_pos_emb")
    return q_embed, k_embed
