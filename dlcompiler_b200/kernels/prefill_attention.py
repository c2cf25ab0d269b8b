"""context_attention_fwd with the signature of python/dlBLAS/dlblas/kernels/prefill_attention.py:155."""
from __future__ import annotations

import torch

from .. import _lib


def _rotary_tables(q, q_cos, q_sin):
    """cos / sin rows for an in-kernel rotation of q: [tokens, D] in q's dtype, contiguous, or (None, None)."""
    if q_cos is None and q_sin is None:
        return None, None
    assert q_cos is not None and q_sin is not None, "cos and sin go together"
    D = q.shape[-1]
    assert D % 16 == 0, "in-kernel rotary needs a head size that is a multiple of 16"
    cos = q_cos.to(device=q.device, dtype=q.dtype).reshape(-1, D).contiguous()
    sin = q_sin.to(device=q.device, dtype=q.dtype).reshape(-1, D).contiguous()
    assert cos.shape == (q.shape[0], D) and sin.shape == cos.shape, "cos / sin need one row of D values per q token"
    return cos, sin


def context_attention_fwd(q, k, v, o, b_start_loc, b_seq_len, max_input_len, lse=None, causal=True,
                          sm_scale=None, q_cos=None, q_sin=None):
    """Variable-length causal GQA attention over packed sequences, written to `o` in place.

    q [total, Hq, D], k/v [total, Hkv, D]; sequence i occupies rows
    [b_start_loc[i], b_start_loc[i] + b_seq_len[i]).  sm_scale defaults to D**-0.5 as in the
    reference (prefill_attention.py:157).  Extension over the reference: if `lse` (fp32
    [Hq, total]) is given it receives m * sm_scale + log(sum), the natural-log convention of
    python/dlBLAS/dlblas/kernels/flash_attention.py:152-155.

    The tensor-core kernel is built for tile widths 64 and 128.  Any other head size up to 128 (the
    reference rounds up to a power of two and masks, prefill_attention.py:179-180; its test runs 96, 80 and
    13, tests/kernels/test_attention_kernels.py:157) runs on the next width.  For multiples of 8 nothing is
    copied: the tensor maps carry the true size and the copy engine zero-fills the missing columns of every
    tile in shared memory.  Sizes that are not multiples of 8 (rows that are not 16-byte aligned cannot be
    addressed by the copy engine) are zero-padded to the next multiple of 8 on the device first, one extra
    pass over q, k, v and o.  Zero feature columns add exact zeros to every score; the softmax scale comes
    from the true head size.

    Extension: with `q_cos` / `q_sin` ([total, D], D a multiple of 16) the rotary embedding of q
    (rotate-half, arithmetic in q's dtype, bit-identical to `apply_rotary_pos_emb`) is applied to each Q
    tile inside the attention kernel; k must arrive rotated (`fill_kv_cache(..., cos=, sin=)` or
    `apply_rotary_pos_emb`).  This is the query side of the reference's fused rotary + attention kernel
    (fused_rotary_and_fa.py:132-133).
    """
    dev = _lib.require_cuda(q, k, v, o, b_start_loc, b_seq_len, lse)
    assert q.dim() == 3 and k.dim() == 3 and v.dim() == 3 and o.shape == q.shape
    Lq, Lk, Lv = q.shape[-1], k.shape[-1], v.shape[-1]
    assert Lq == Lk == Lv
    assert q.dtype in (torch.float16, torch.bfloat16) and k.dtype == q.dtype and v.dtype == q.dtype
    assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1 and o.stride(-1) == 1
    if sm_scale is None:
        sm_scale = 1.0 / (Lq**0.5)
    assert 1 <= Lq <= 128, "head sizes above 128 are not built"
    if Lq % 8 != 0 or any(t.stride(0) % 8 or t.stride(1) % 8 for t in (q, k, v, o)):
        assert q_cos is None, "in-kernel rotary needs 16-byte aligned rows"
        pad = (Lq + 7) // 8 * 8 - Lq
        qp, kp, vp = (torch.nn.functional.pad(t, (0, pad)) for t in (q, k, v))
        op = torch.empty_like(qp)
        context_attention_fwd(qp, kp, vp, op, b_start_loc, b_seq_len, max_input_len, lse=lse, causal=causal,
                              sm_scale=sm_scale)
        o.copy_(op[..., :Lq])
        return o
    batch, head = b_seq_len.shape[0], q.shape[1]
    assert head % k.shape[1] == 0
    b_start_loc = b_start_loc.to(torch.int32).contiguous()
    b_seq_len = b_seq_len.to(torch.int32).contiguous()
    if lse is not None:
        assert lse.dtype == torch.float32 and lse.shape == (head, q.shape[0]) and lse.is_contiguous()
    assert o.stride(0) % 8 == 0 and o.stride(1) % 8 == 0, "output strides must be multiples of 8 elements"
    cos, sin = _rotary_tables(q, q_cos, q_sin)
    lib = _lib.load()
    status = _lib.status_word(dev)
    with torch.cuda.device(dev):
        rc = lib.dlb_flash_prefill_varlen(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), _lib.ptr(lse), b_start_loc.data_ptr(),
            b_seq_len.data_ptr(), batch, q.shape[0], int(max_input_len), head, k.shape[1], Lq, Lv,
            q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1), o.stride(0), o.stride(1),
            float(sm_scale), int(causal), _lib.ptr(cos), _lib.ptr(sin), _lib.dtype_code(q), status.data_ptr(),
            _lib.stream_ptr(dev))
    _lib.check(rc, "context_attention_fwd")
    return o
