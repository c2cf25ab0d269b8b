"""dlcompiler_b200: B200-native (sm_100a) implementation of the dlBLAS hot-path operators.

The operator functions keep the names, argument order and defaults of the
reference's `dlblas.kernels.*` modules (torch tensors in, torch tensors out) and
call hand-written CUDA kernels in libdlblas_b200.so through a C ABI.  There is
no Triton, no backend dispatch and no CPU fallback on this path.
"""
from . import _lib
from ._lib import DlblasError, check_device_status, is_built
from .kernels.activation import silu_and_mul
from .kernels.apply_rotary_pos_emb import apply_rotary_pos_emb
from .kernels.fill_kv_cache import fill_kv_cache
from .kernels.rms_norm import add_rms_norm, rms_norm
from .kernels.decode_attention import decode_attention_fwd
from .kernels.flash_attention import flash_attention_fwd, flash_attention_v2
from .kernels.fused_rotary_and_fa import fused_rotary_and_fa
from .kernels.fused_moe import fused_moe, fused_moe_kernel_launcher, get_start_end, moe_align_block_size
from .kernels.moe_gating import grouped_topk_gating, softmax_topk
from .kernels.paged_attention import paged_attention_fwd
from .kernels.prefill_attention import context_attention_fwd
from .kernels.topk_gating import topk_gating
from .op_registry import get_op, op_registry, register_dlblas_op

__all__ = [
    "DlblasError", "check_device_status", "is_built", "silu_and_mul", "fused_moe", "fused_moe_kernel_launcher",
    "get_start_end", "moe_align_block_size", "grouped_topk_gating", "softmax_topk", "paged_attention_fwd",
    "context_attention_fwd", "decode_attention_fwd", "flash_attention_fwd", "flash_attention_v2", "apply_rotary_pos_emb", "fill_kv_cache", "rms_norm", "add_rms_norm", "topk_gating", "fused_rotary_and_fa", "get_op", "op_registry", "register_dlblas_op",
]
