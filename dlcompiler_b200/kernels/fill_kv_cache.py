"""fill_kv_cache with the signature of python/dlBLAS/dlblas/kernels/fill_kv_cache.py:131."""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _lib


def _is64(t):
    assert t.dtype in (torch.int32, torch.int64), f"index tensor must be int32 or int64, got {t.dtype}"
    return int(t.dtype == torch.int64)


def fill_kv_cache(
    k_states: Tensor,
    v_states: Tensor,
    k_caches: Tensor,
    v_caches: Tensor,
    q_start_loc: Tensor,
    q_seq_length: Tensor,
    kv_seq_length: Tensor,
    max_q_seq_length: int,
    block_offsets: Tensor,
    cos: Tensor = None,
    sin: Tensor = None,
):
    """Copy the new tokens' key/value states ([tokens, heads, d]) into the paged caches
    ([pages, page_size, heads, d]) at the positions that follow each sequence's history.

    Extension: with `cos` / `sin` ([tokens, d], fp16/bf16 states, d a multiple of 16) the keys are rotated
    (rotate-half rotary embedding, bit-identical to `apply_rotary_pos_emb`) while they are written, so the
    cache holds rotated keys and the attention kernels read it as it is; the reference rotates every K tile
    inside its attention loop instead (fused_rotary_and_fa.py:177-178)."""
    dev = _lib.require_cuda(k_states, v_states, k_caches, v_caches, q_start_loc, q_seq_length, kv_seq_length,
                            block_offsets)
    block_offsets = block_offsets.contiguous()
    batch_size = block_offsets.size(0)
    block_size, num_heads, head_dim = k_caches.size()[1:]
    head_dim_v = v_states.size(-1)
    assert k_states.dtype == k_caches.dtype and v_states.dtype == v_caches.dtype
    assert k_states.element_size() == v_states.element_size()
    assert k_states.stride(-1) == 1 and v_states.stride(-1) == 1 and k_caches.stride(-1) == 1 and v_caches.stride(-1) == 1
    q_start_loc, q_seq_length, kv_seq_length = (t.contiguous() for t in (q_start_loc, q_seq_length, kv_seq_length))
    kc = ks = None
    dt = 0
    if cos is not None or sin is not None:
        assert cos is not None and sin is not None, "cos and sin go together"
        assert k_states.dtype in (torch.float16, torch.bfloat16) and head_dim % 16 == 0
        kc = cos.to(device=dev, dtype=k_states.dtype).reshape(-1, head_dim).contiguous()
        ks = sin.to(device=dev, dtype=k_states.dtype).reshape(-1, head_dim).contiguous()
        assert kc.shape[0] == k_states.shape[0] and ks.shape == kc.shape, "cos / sin need one row per new token"
        dt = _lib.dtype_code(k_states)
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.dlb_fill_kv_cache(
            k_states.data_ptr(), v_states.data_ptr(), k_caches.data_ptr(), v_caches.data_ptr(), q_start_loc.data_ptr(),
            q_seq_length.data_ptr(), kv_seq_length.data_ptr(), block_offsets.data_ptr(), batch_size,
            int(max_q_seq_length), block_size, num_heads, head_dim, head_dim_v, k_caches.size(0), block_offsets.size(1),
            k_states.stride(-3), k_states.stride(-2), v_states.stride(-3), v_states.stride(-2),
            k_caches.stride(0), k_caches.stride(1), k_caches.stride(2), v_caches.stride(0), v_caches.stride(1),
            v_caches.stride(2), block_offsets.stride(0), _is64(q_start_loc), _is64(q_seq_length),
            _is64(kv_seq_length), _is64(block_offsets), k_states.element_size(), _lib.ptr(kc), _lib.ptr(ks), dt,
            _lib.stream_ptr(dev))
    _lib.check(rc, "fill_kv_cache")
