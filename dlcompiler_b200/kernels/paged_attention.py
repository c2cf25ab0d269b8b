"""paged_attention_fwd with the signature of python/dlBLAS/dlblas/kernels/paged_attention.py:492."""
from __future__ import annotations

import logging
import os

import torch
from torch import Tensor

from .. import _lib

logger = logging.getLogger("dlblas")

# Split work items aimed at per launch: 4 waves of 2 CTAs per SM.  A split pays a fixed price (barrier set-up,
# Q fragments, the cross-warp merge and the partial's round trip through the merge kernel), so splits should be
# as long as load balance allows: at 16 sequences of 1k-32k tokens, 512-token splits (16 waves) reach 4.95 TB/s,
# 2048-token splits (4 waves) 5.92 TB/s and 4096-token splits 6.04 TB/s.
_TARGET_CTAS = 148 * 2 * 4


def _pick_chunk(batch: int, kv_heads: int, max_ctx: int, page_size: int) -> int:
    """Tokens per KV split: a power of two, at least one 64-key tile and one page.
    DLBLAS_B200_DECODE_CHUNK in the environment forces the value (rounded up to a legal one)."""
    forced = os.environ.get("DLBLAS_B200_DECODE_CHUNK")
    if forced:
        chunk = 1 << max(int(forced) - 1, 1).bit_length()
        return max(64, page_size, chunk)
    want = max(1, batch * kv_heads * max_ctx // _TARGET_CTAS)
    chunk = 1 << (want.bit_length() - 1)
    lo = max(256, page_size)
    return max(lo, min(chunk, 4096))


def paged_attention_fwd(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    o: Tensor,
    block_offsets: Tensor,
    q_start_loc: Tensor,
    q_seqlens: Tensor,
    kv_seqlens: Tensor,
    max_seqlen: int,
    window_size: int = None,
    sm_scale: float = None,
    logit_softcapping: float = None,
    q_cos: Tensor = None,
    q_sin: Tensor = None,
):
    """Paged attention forward.

    Args follow the reference (paged_attention.py:492-519): caches `k`/`v` [num_pages, page_size, Hkv, D],
    `o` written in place, `block_offsets` [batch, max_pages] page ids (int32 or int64), `kv_seqlens`
    [batch].  Decode (`q` [batch, Hq, D], one query token per sequence, paged_attention.py:559): the KV
    length is split in fixed-size chunks (count adapts to each sequence) and merged by log-sum-exp.
    Prefill (`q` [total_q, Hq, D] packed by `q_start_loc` / `q_seqlens`): query i of a sequence sits at
    position `kv_seqlens - q_seqlens + i` and attends causally to the cache, which must already hold the
    new tokens' K/V (fill_kv_cache runs first, as in the reference's callers).
    Sliding window and tanh soft-cap as in the reference, in both branches.
    The q/k head size and the v/out head size may differ (paged_attention.py:526-539); both must be
    multiples of 8 up to 128 (the kernels run at tile widths 64 and 128 and let the copy engine zero-fill
    the missing columns in shared memory; the cache is never copied or padded).  fp16/bf16, page size a
    power of two >= 16.
    Extension (prefill branch): `q_cos` / `q_sin` ([total_q, D]) rotate q inside the kernel, see
    `context_attention_fwd`; the cache must hold rotated keys (`fill_kv_cache(..., cos=, sin=)`).
    """
    dev = _lib.require_cuda(q, k, v, o, block_offsets, kv_seqlens)
    if window_size is None:
        window_size = -1
    if logit_softcapping is None:
        logit_softcapping = -1.0
    Lq, Lk, Lv = q.shape[-1], k.shape[-1], v.shape[-1]
    assert Lq == Lk, f"q and k head sizes differ: {Lq} vs {Lk}"
    assert Lv == o.shape[-1], f"v head size {Lv} does not match the output's {o.shape[-1]}"
    if sm_scale is None:
        sm_scale = 1.0 / (Lq**0.5)
    batch, head = q_seqlens.shape[0], q.shape[-2]
    BLOCK = k.size(1)
    assert BLOCK >= 16
    is_decoding = q.shape[-3] == q_seqlens.size(0)
    assert Lk % 8 == 0 and Lv % 8 == 0 and Lk <= 128 and Lv <= 128, "head sizes: multiples of 8 up to 128"
    if not is_decoding:
        return _paged_prefill(q, k, v, o, block_offsets, q_start_loc, q_seqlens, kv_seqlens, max_seqlen,
                              window_size, sm_scale, logit_softcapping, dev, q_cos, q_sin)
    assert q_cos is None and q_sin is None, "the decode branch takes q already rotated"
    assert k.dim() == 4 and v.dim() == 4 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert q.stride(-1) == 1 and o.stride(-1) == 1
    assert block_offsets.dim() == 2 and block_offsets.stride(1) == 1
    assert block_offsets.dtype in (torch.int32, torch.int64) and kv_seqlens.dtype in (torch.int32, torch.int64)
    kv_seqlens = kv_seqlens.contiguous()
    hkv = k.shape[-2]
    max_pages = block_offsets.size(1)
    max_ctx = max_pages * BLOCK
    chunk = _pick_chunk(batch, hkv, max_ctx, BLOCK)
    max_splits = (max_ctx + chunk - 1) // chunk
    if window_size > 0:
        # a window touches at most window + one tile of alignment slack
        max_splits = min(max_splits, (window_size + 1 + 64 + chunk - 1) // chunk + 1)
    lib = _lib.load()
    nfloats = lib.dlb_paged_decode_workspace_floats(batch, head, max(Lq, Lv), max_splits)
    partial = torch.empty(max(nfloats, 1), dtype=torch.float32, device=dev)
    status = _lib.status_word(dev)
    with torch.cuda.device(dev):
        rc = lib.dlb_paged_decode(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), block_offsets.data_ptr(), kv_seqlens.data_ptr(),
            partial.data_ptr(), batch, head, hkv, Lq, Lv, BLOCK, k.size(0), max_pages,
            q.stride(-3), q.stride(-2), o.stride(-3), o.stride(-2),
            k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1), v.stride(2),
            block_offsets.stride(0), int(block_offsets.dtype == torch.int64), int(kv_seqlens.dtype == torch.int64),
            chunk, max_splits, window_size, float(sm_scale), float(logit_softcapping), _lib.dtype_code(q),
            status.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "paged_attention_fwd(decode)")
    return o


def _paged_prefill(q, k, v, o, block_offsets, q_start_loc, q_seqlens, kv_seqlens, max_seqlen, window_size, sm_scale,
                   logit_softcapping, dev, q_cos=None, q_sin=None):
    """Prefill branch of paged_attention_fwd (paged_attention.py:617-671): the tcgen05 prefill kernel with
    its K/V tiles fetched page by page."""
    assert q.dim() == 3 and o.shape[:-1] == q.shape[:-1] and q.stride(-1) == 1 and o.stride(-1) == 1
    assert k.dim() == 4 and v.dim() == 4 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert block_offsets.dim() == 2 and block_offsets.stride(1) == 1
    assert block_offsets.dtype in (torch.int32, torch.int64)
    batch = q_seqlens.shape[0]
    q_start = q_start_loc.to(device=dev, dtype=torch.int32).contiguous()
    q_len = q_seqlens.to(device=dev, dtype=torch.int32).contiguous()
    kv_len = kv_seqlens.to(device=dev, dtype=torch.int32).contiguous()
    from .prefill_attention import _rotary_tables

    cos, sin = _rotary_tables(q, q_cos, q_sin)
    lib = _lib.load()
    status = _lib.status_word(dev)
    with torch.cuda.device(dev):
        rc = lib.dlb_flash_prefill_paged(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), None, block_offsets.data_ptr(),
            q_start.data_ptr(), q_len.data_ptr(), kv_len.data_ptr(), batch, q.shape[0], int(max_seqlen),
            q.shape[1], k.shape[2], q.shape[2], v.shape[3], k.size(1), k.size(0), block_offsets.size(1),
            q.stride(0), q.stride(1), k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1), v.stride(2),
            o.stride(0), o.stride(1), block_offsets.stride(0), int(block_offsets.dtype == torch.int64),
            int(window_size), float(sm_scale), float(logit_softcapping), 1, _lib.ptr(cos), _lib.ptr(sin),
            _lib.dtype_code(q), status.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "paged_attention_fwd(prefill)")
    return o
