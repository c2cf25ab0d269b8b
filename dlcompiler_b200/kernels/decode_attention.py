"""decode_attention_fwd with the signature of python/dlBLAS/dlblas/kernels/decode_attention.py:559."""
from __future__ import annotations

import torch

from .. import _lib
from .paged_attention import _pick_chunk


def decode_attention_fwd(
    q,
    k_buffer,
    v_buffer,
    o,
    req_to_token,
    b_req_idx,
    b_start_loc,
    b_seq_len,
    attn_logits,
    max_len_in_batch,
    sm_scale,
    logit_cap=0.0,
):
    """Token-granular decode attention: request `b_req_idx[i]` reads its keys and values from rows
    `req_to_token[b_req_idx[i], :b_seq_len[i]]` of `k_buffer` / `v_buffer` ([tokens, Hkv, D]).

    The reference runs two stages through a materialised `attn_logits` buffer
    (decode_attention.py:559-620); here the same math is one split-KV pass of the paged decode
    kernel with a page size of one token, so `attn_logits` and `b_start_loc` are accepted for
    signature compatibility and not touched.  `logit_cap > 0` applies cap * tanh(qk / cap).
    """
    dev = _lib.require_cuda(q, k_buffer, v_buffer, o, req_to_token, b_req_idx, b_seq_len)
    assert q.dim() == 3 and k_buffer.dim() == 3 and v_buffer.dim() == 3
    batch, head, D = q.shape
    Dv = v_buffer.shape[-1]
    assert k_buffer.shape[-1] == D and o.shape[-1] == Dv, "k must have the query's head size, o the value's"
    assert D % 8 == 0 and Dv % 8 == 0 and D <= 128 and Dv <= 128, "head sizes: multiples of 8 up to 128"
    assert q.stride(-1) == 1 and o.stride(-1) == 1 and k_buffer.stride(-1) == 1 and v_buffer.stride(-1) == 1
    hkv = k_buffer.shape[1]
    table = req_to_token.index_select(0, b_req_idx.to(torch.int64))
    if table.dtype not in (torch.int32, torch.int64):
        table = table.to(torch.int64)
    max_ctx = min(int(max_len_in_batch), table.size(1)) if max_len_in_batch else table.size(1)
    table = table[:, :max(max_ctx, 1)].contiguous()
    lens = b_seq_len if b_seq_len.dtype in (torch.int32, torch.int64) else b_seq_len.to(torch.int64)
    lens = lens.contiguous()
    chunk = _pick_chunk(batch, hkv, table.size(1), 1)
    max_splits = (table.size(1) + chunk - 1) // chunk
    lib = _lib.load()
    nfloats = lib.dlb_paged_decode_workspace_floats(batch, head, max(D, Dv), max_splits)
    partial = torch.empty(max(nfloats, 1), dtype=torch.float32, device=dev)
    status = _lib.status_word(dev)
    with torch.cuda.device(dev):
        rc = lib.dlb_paged_decode(
            q.data_ptr(), k_buffer.data_ptr(), v_buffer.data_ptr(), o.data_ptr(), table.data_ptr(), lens.data_ptr(),
            partial.data_ptr(), batch, head, hkv, D, Dv, 1, k_buffer.size(0), table.size(1),
            q.stride(0), q.stride(1), o.stride(0), o.stride(1),
            k_buffer.stride(0), k_buffer.stride(0), k_buffer.stride(1),
            v_buffer.stride(0), v_buffer.stride(0), v_buffer.stride(1),
            table.stride(0), int(table.dtype == torch.int64), int(lens.dtype == torch.int64),
            chunk, max_splits, -1, float(sm_scale), float(logit_cap) if logit_cap and logit_cap > 0 else -1.0,
            _lib.dtype_code(q), status.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "decode_attention_fwd")
    return o
