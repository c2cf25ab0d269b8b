"""rms_norm (python/dlBLAS/dlblas/kernels/rms_norm.py:78) and add_rms_norm
(python/dlBLAS/dlblas/kernels/add_rms_norm.py:43) with the reference signatures."""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _lib


def _launch(x, weight, residual, out, out_residual, eps, weight_after_cast):
    dev = _lib.require_cuda(x, weight, residual, out, out_residual)
    n = weight.shape[0]
    assert x.size(-1) == n and x.stride(-1) == 1 and out.stride(-1) == 1 and weight.is_contiguous()
    rows = x.numel() // n
    x2, o2 = x.reshape(rows, n), out.view(rows, n)
    r2 = residual.reshape(rows, n) if residual is not None else None
    or2 = out_residual.view(rows, n) if out_residual is not None else None
    if r2 is not None and or2 is not None:
        assert r2.stride(0) == or2.stride(0), "residual and out_residual must share their row stride"
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.dlb_rms_norm(x2.data_ptr(), weight.data_ptr(), _lib.ptr(r2), o2.data_ptr(), _lib.ptr(or2), rows, n,
                              x2.stride(0) if rows > 1 else n, (r2.stride(0) if rows > 1 else n) if r2 is not None else n,
                              o2.stride(0) if rows > 1 else n, float(eps), int(weight_after_cast), _lib.dtype_code(x),
                              _lib.stream_ptr(dev))
    _lib.check(rc, "rms_norm")


def rms_norm(
    hidden_states: Tensor,
    weight: Tensor,
    eps: float = 1e-6,
    residual: Tensor = None,
    out: Tensor = None,
    out_residual: Tensor = None,
):
    """out = (weight * x_f32 * rsqrt(mean(x^2) + eps)).to(dtype); with `residual`, x = hidden_states +
    residual (added in the storage dtype) and (out, out_residual) is returned (rms_norm.py:78-132)."""
    if not hidden_states.is_contiguous():
        hidden_states = hidden_states.contiguous()
    if out is None:
        out = torch.empty_like(hidden_states)
    if residual is None:
        _launch(hidden_states, weight, None, out, None, eps, 0)
        return out
    if out_residual is None:
        out_residual = torch.empty_like(hidden_states)
    _launch(hidden_states, weight, residual, out, out_residual, eps, 0)
    return out, out_residual


def add_rms_norm(hidden_states: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                 residual: torch.Tensor = None):
    """The registry op `add_rms_norm` (add_rms_norm.py:43-80): the normalised value is rounded to the
    storage dtype before it is multiplied by the weight.  Returns out, or (out, residual_out)."""
    assert hidden_states.dim() == 2 and hidden_states.shape[1] == weight.shape[0]
    out = torch.empty_like(hidden_states)
    if residual is None:
        _launch(hidden_states, weight, None, out, None, eps, 1)
        return out
    residual_out = torch.empty_like(residual)
    _launch(hidden_states, weight, residual, out, residual_out, eps, 1)
    return out, residual_out
