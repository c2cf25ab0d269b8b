"""The C-ABI library: it loads, exports every symbol the header declares, and rejects bad
arguments before touching the device (no GPU needed)."""
import os
import re

import pytest

from dlcompiler_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "dlblas_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dlb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/dlblas_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes prototypes and header declarations differ"
    assert lib.dlb_version() >= 100


def test_ctypes_prototypes_match_the_header_argument_by_argument():
    """Every prototype in include/dlblas_b200.h against the ctypes table: same number of arguments and, per
    argument, the same kind (pointer, int, int64_t, float).  The .cu files include the same header, so a
    definition that drifts from it does not compile; this closes the third side of the triangle."""
    from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

    text = open(os.path.join(ROOT, "include", "dlblas_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = re.findall(r"^([\w \*]+?)\b(dlb_\w+)\s*\(([^)]*)\)\s*;", text, flags=re.M)
    assert len(protos) == len(_lib.SIGNATURES)

    def kind(decl):
        decl = decl.strip()
        if "*" in decl:
            return "ptr"
        base = decl.split()[:-1] if len(decl.split()) > 1 else [decl]
        base = " ".join(t for t in base if t != "const")
        return {"int": "int", "int64_t": "i64", "float": "f32"}[base]

    ctype_kind = {c_void_p: "ptr", c_char_p: "ptr", c_int: "int", c_int64: "i64", c_float: "f32"}
    for ret, name, args in protos:
        res, argtypes = _lib.SIGNATURES[name]
        want = [] if args.strip() in ("", "void") else [kind(a) for a in args.split(",")]
        got = [ctype_kind[t] for t in argtypes]
        assert got == want, f"{name}: ctypes {got} != header {want}"
        assert ctype_kind[res] == kind(ret + " x"), f"{name}: return type"


def test_argument_errors_are_reported_without_a_device():
    lib = _lib.load()
    rc = lib.dlb_silu_and_mul(None, None, -1, 8, 16, 8, _lib.DTYPE_BF16, None)
    assert rc < 0 and b"negative" in lib.dlb_last_error()
    rc = lib.dlb_grouped_topk_gating(None, None, None, None, 4, 1000, 1000, 1, 1, 2, 0, 1, 1.0, None)
    assert rc < 0 and b"experts" in lib.dlb_last_error()
    with pytest.raises(AssertionError):
        _lib.check(rc, "gating")
    rc = lib.dlb_paged_decode(None, None, None, None, None, None, None, 1, 32, 8, 100, 64, 64, 1, 1, 0, 0, 0, 0, 0, 0,
                              0, 0, 0, 0, 0, 0, 0, 256, 1, -1, 1.0, -1.0, _lib.DTYPE_BF16, None, None)
    assert rc < 0 and b"head_dim" in lib.dlb_last_error()
    rc = lib.dlb_moe_grouped_gemm(1, 100, 64, 1, 4, 128, 64, 64, 1, 128, 128, 1, 1, None, 10, 0, _lib.DTYPE_BF16,
                                  None, None)
    assert rc < 0 and b"128-row" in lib.dlb_last_error()
    assert lib.dlb_paged_decode_workspace_floats(64, 32, 128, 8) == 64 * 32 * 8 * 130
    assert lib.dlb_set_wait_budget_ms(0) < 0 and lib.dlb_set_wait_budget_ms(2000) == 0
    rc = lib.dlb_moe_start_end(None, 1, 16, 4000, None, None, 1, None)
    assert rc < 0 and b"experts" in lib.dlb_last_error()


def test_wrappers_refuse_cpu_tensors():
    import torch

    from dlcompiler_b200 import silu_and_mul

    with pytest.raises(AssertionError):
        silu_and_mul(torch.zeros(4, 8, dtype=torch.bfloat16))


def test_op_registry_shell_resolves_the_reference_names():
    """`get_op(name, args)` as the reference's consumers call it (dlblas/__init__.py:13-23): known names give a
    callable operator object, unknown names raise NameError, a wrong arity raises LookupError."""
    import pytest
    import dlcompiler_b200 as dl
    assert set(dl.op_registry.get_list_op_names()) >= {"topk_gating", "flash_attention_v2", "add_rms_norm", "rms_norm",
                                                        "fused_rotary_and_fa"}
    op = dl.get_op("topk_gating", (None, 2, 1.0, 2, False))
    assert callable(op) and op.name == "topk_gating"
    assert dl.get_op("rms_norm", (None, None, 1e-6)).n_args == 3
    with pytest.raises(NameError):
        dl.get_op("no_such_op", ())
    with pytest.raises(LookupError):
        dl.get_op("flash_attention_v2", (None,))
