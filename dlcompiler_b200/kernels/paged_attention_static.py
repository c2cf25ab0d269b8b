"""Paged flash-decode through the allocation-free entry point of libdlblas_b200."""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _lib
from .paged_attention import _pick_chunk


def paged_decode_no_alloc(q: Tensor, k: Tensor, v: Tensor, o: Tensor, block_offsets: Tensor, kv_seqlens: Tensor,
                          sm_scale: float = None, window_size: int = None, logit_softcapping: float = None):
    """Decode attention for callers that must not allocate device memory around the call.

    Same math and arguments as the decode case of `paged_attention_fwd` (q [batch, Hq, D],
    paged caches, output written into `o`), but neither this function nor the library call
    behind it creates a tensor or calls the CUDA allocator: the split-KV workspace is a fixed
    32 MiB device array inside the library.  Intended for engines that gave all their device
    memory to the KV cache at start-up, and for token loops that must stay out of the
    allocator.  Consequences: the problem must fit the array (batch * Hq * splits * (D + 2)
    floats; an AssertionError says so otherwise), `kv_seqlens` and `block_offsets` must already
    be contiguous int32/int64 tensors, concurrent calls on one device must be serialised, and
    the first call on a device should happen before any CUDA-graph capture.
    """
    dev = _lib.require_cuda(q, k, v, o, block_offsets, kv_seqlens)
    assert q.dim() == 3 and k.dim() == 4 and v.dim() == 4 and block_offsets.dim() == 2
    assert q.stride(-1) == 1 and o.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert block_offsets.stride(1) == 1 and kv_seqlens.is_contiguous()
    batch, head, D = q.shape
    page = k.size(1)
    hkv = k.size(2)
    max_pages = block_offsets.size(1)
    if sm_scale is None:
        sm_scale = 1.0 / (D**0.5)
    window = -1 if window_size is None else window_size
    softcap = -1.0 if logit_softcapping is None else logit_softcapping
    max_ctx = max_pages * page
    chunk = _pick_chunk(batch, hkv, max_ctx, page)
    max_splits = (max_ctx + chunk - 1) // chunk
    # grow the chunk until the partials fit the fixed array
    while max_splits > 1 and batch * head * max_splits * (D + 2) > _lib.DECODE_STATIC_FLOATS:
        chunk *= 2
        max_splits = (max_ctx + chunk - 1) // chunk
    lib = _lib.load()
    # the status word is a torch tensor: use it only if an earlier call already made it (NULL is allowed)
    status = _lib.existing_status_word(dev)
    with torch.cuda.device(dev):
        rc = lib.dlb_paged_decode_static(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), block_offsets.data_ptr(), kv_seqlens.data_ptr(),
            batch, head, hkv, D, page, k.size(0), max_pages, q.stride(0), q.stride(1), o.stride(0), o.stride(1),
            k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1), v.stride(2), block_offsets.stride(0),
            int(block_offsets.dtype == torch.int64), int(kv_seqlens.dtype == torch.int64), chunk, max_splits, window,
            float(sm_scale), float(softcap), _lib.dtype_code(q), _lib.ptr(status), _lib.stream_ptr(dev))
    _lib.check(rc, "paged_decode_no_alloc")
    return o
