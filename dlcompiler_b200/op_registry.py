"""Name -> operator look-up with the calling convention of the reference's registry.

The reference resolves `dlblas.topk_gating`, `flash_attention_v2`, `add_rms_norm` and `rms_norm`
through `get_op(op_name, args)` (python/dlBLAS/dlblas/op_registry.py:70-109), which filters the
registered implementations by argument types, auto-tunes the candidates and returns an `OpImpl`
whose `__call__` runs the kernel (op_struct.py:29-43).  Here every name has exactly one
implementation, so there is nothing to tune or cache: `get_op` checks the name and the number of
arguments and returns the operator object directly.  Unknown names raise `NameError`, as in the
reference (op_registry.py:71-72); a name with no implementation for the given arguments raises
`LookupError` (op_registry.py:97-98).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable


@dataclass(frozen=True)
class OpImpl:
    """One registered operator: `call` runs it, `n_args` is the arity it was registered with."""
    name: str
    n_args: int
    call: Callable[..., Any]

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        return self.call(*args, **kwargs)


class OpRegistry:
    def __init__(self) -> None:
        self.ops: dict[str, list[OpImpl]] = {}

    def register(self, name: str, n_args: int, call: Callable[..., Any]) -> None:
        self.ops.setdefault(name, []).append(OpImpl(name, n_args, call))

    def get_list_op_names(self) -> list[str]:
        return list(self.ops.keys())

    def get_op(self, op_name: str, args: tuple, configs=None) -> OpImpl:
        if op_name not in self.ops:
            raise NameError(f"op {op_name} not found")
        for impl in self.ops[op_name]:
            if impl.n_args == len(args):
                return impl
        raise LookupError(f"no candidates for op {op_name} with args")


op_registry = OpRegistry()


def register_dlblas_op(name: str, n_args: int, call: Callable[..., Any]) -> None:
    op_registry.register(name, n_args, call)


def get_op(op_name: str, args: tuple, configs=None) -> OpImpl:
    """`get_op(name, args)(*args)` runs operator `name` (the reference's look-up convention)."""
    return op_registry.get_op(op_name, args, configs)


def _register_builtin_ops() -> None:
    from .kernels.flash_attention import flash_attention_v2
    from .kernels.rms_norm import add_rms_norm
    from .kernels.topk_gating import topk_gating

    # (logits, k, capacity_factor, min_capacity, higher_precision): topk_gating.py:314
    register_dlblas_op("topk_gating", 5, topk_gating)
    # (q, k, v): flash_attention_v2.py:330
    register_dlblas_op("flash_attention_v2", 3, lambda q, k, v: flash_attention_v2(q, k, v))

    # add_rms_norm.py:103-118 registers one `call(hidden_states, weight, eps, residual)` under both names:
    # with a residual it returns (out, residual_out), without one only out (add_rms_norm.py:77-80)
    def _norm_call(hidden_states, weight, eps=1e-6, residual=None):
        return add_rms_norm(hidden_states, weight, eps, residual)

    from .kernels.fused_rotary_and_fa import call as _rotary_fa_call
    # (q, k, v, cos, sin): fused_rotary_and_fa.py:413
    register_dlblas_op("fused_rotary_and_fa", 5, _rotary_fa_call)
    register_dlblas_op("add_rms_norm", 4, _norm_call)
    register_dlblas_op("rms_norm", 3, _norm_call)


_register_builtin_ops()
