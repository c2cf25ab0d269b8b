"""silu_and_mul with the signature of python/dlBLAS/dlblas/kernels/activation.py:88."""
from __future__ import annotations

import torch

from .. import _lib


def silu_and_mul(gate_up: torch.Tensor, out: torch.Tensor = None):
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, N + i]  (gate = first half of the last dim).

    Same contract as the reference wrapper (activation.py:88-130): 2-D input, optional
    caller-provided `out`, row strides honoured.  Math in fp32, one rounding on store.
    """
    assert gate_up.dim() == 2
    _lib.require_cuda(gate_up, out)
    M = gate_up.size(0)
    N = gate_up.size(-1) // 2
    assert gate_up.size(-1) == 2 * N, "last dimension must be even"
    if out is None:
        out = gate_up.new_empty((M, N))
    assert out.shape == (M, N) and out.dtype == gate_up.dtype
    if gate_up.stride(1) != 1:
        gate_up = gate_up.contiguous()
    assert out.stride(1) == 1 or N <= 1, "out must be contiguous along its last dimension"
    lib = _lib.load()
    with torch.cuda.device(gate_up.device):
        rc = lib.dlb_silu_and_mul(gate_up.data_ptr(), out.data_ptr(), M, N, gate_up.stride(0) if M > 1 else 2 * N,
                                  out.stride(0) if M > 1 else N, _lib.dtype_code(gate_up),
                                  _lib.stream_ptr(gate_up.device))
    _lib.check(rc, "silu_and_mul")
    return out
