"""Generate golden fixtures by EXECUTING the reference tests' own ground-truth functions on the CPU.

Run once where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/DLCompiler

Nothing is copied from the reference: the ground-truth functions are located in the
reference's test files with `ast`, compiled in memory (decorators dropped, `.cuda()` calls
removed so they run on the CPU) and called on seeded inputs.  Inputs and outputs are stored
as small `.pt` files next to this script; the test-suite loads them without needing the
reference checkout.
"""
from __future__ import annotations

import argparse
import ast
import math
import os

import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


class _StripCuda(ast.NodeTransformer):
    """x.cuda() -> x ; device="cuda" keyword -> device="cpu"."""

    def visit_Call(self, node):
        self.generic_visit(node)
        if isinstance(node.func, ast.Attribute) and node.func.attr == "cuda" and not node.args:
            return node.func.value
        for kw in node.keywords:
            if kw.arg == "device" and isinstance(kw.value, ast.Constant) and kw.value.value == "cuda":
                kw.value = ast.Constant("cpu")
        return node


def load_functions(path: str, names: list[str], extra_ns: dict | None = None) -> dict:
    """Compile the named functions (`func` or `Class.method`) of a reference file in memory."""
    tree = ast.parse(open(path).read())
    found = {}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            found[node.name] = node
        elif isinstance(node, ast.ClassDef):
            for sub in node.body:
                key = f"{node.name}.{sub.name}" if isinstance(sub, ast.FunctionDef) else None
                if key in names:
                    found[key] = sub
    missing = [n for n in names if n not in found]
    if missing:
        raise RuntimeError(f"{path}: cannot find {missing}")
    ns = {"torch": torch, "math": math, "F": F}
    ns.update(extra_ns or {})
    out = {}
    for key, node in found.items():
        node.decorator_list = []
        node = _StripCuda().visit(node)
        mod = ast.Module(body=[node], type_ignores=[])
        ast.fix_missing_locations(mod)
        exec(compile(mod, path, "exec"), ns)
        out[key] = ns[node.name]
    return out


def _fixture_value(gen_fn, *args):
    """The reference ground truths are pytest fixtures (generators): take the yielded value."""
    return next(gen_fn(None, *args))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (DLCompiler)")
    args = ap.parse_args()
    tests = os.path.join(args.reference, "python/dlBLAS/tests/kernels")
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---------------------------------------------------------------- silu_and_mul
    fns = load_functions(os.path.join(tests, "test_activation.py"), ["TestSiluAndMul.gt"])
    cases = []
    for i, (rows, feat, dtype) in enumerate([(16, 4096, torch.float16), (16, 768, torch.float16),
                                             (16, 2 * 1376, torch.bfloat16)]):
        g = torch.Generator().manual_seed(1000 + i)
        x = torch.rand(rows, feat, generator=g).to(dtype)
        cases.append({"x": x, "gt": _fixture_value(fns["TestSiluAndMul.gt"], x)})
    torch.save(cases, os.path.join(HERE, "silu_and_mul.pt"))

    # ---------------------------------------------------------------- fused_moe (launcher + end to end)
    fns = load_functions(os.path.join(tests, "test_fused_moe.py"),
                         ["TestFusedMoEKernelLauncher.gt", "_mlp_forward", "TestFusedMoe.gt"])
    g = torch.Generator().manual_seed(2000)
    M, K, N, E, top_k = 256, 64, 128, 4, 2
    A = ((torch.rand(M, K, generator=g) - 0.5) / 2).to(torch.float16)
    B = ((torch.rand(E, N, K, generator=g) - 0.5) / 2).to(torch.float16)
    router = torch.rand(M, E, generator=g).to(torch.float16)
    weights, topk_idx = router.topk(top_k, dim=-1)
    launcher = {"A": A, "B": B, "weights": weights, "topk_idx": topk_idx, "top_k": top_k,
                "gt": _fixture_value(fns["TestFusedMoEKernelLauncher.gt"], A, B, top_k, topk_idx, True, weights)}
    e2e = []
    for i, dtype in enumerate([torch.float16, torch.bfloat16]):
        g = torch.Generator().manual_seed(2100 + i)
        seq, in_size, hidden, out_size = 128, 128, 256, 128
        hs = ((torch.rand(seq, in_size, generator=g) - 0.5) / 2).to(dtype)
        w1 = ((torch.rand(E, hidden, in_size, generator=g) - 0.5) / 2).to(dtype)
        w2 = ((torch.rand(E, out_size, hidden // 2, generator=g) - 0.5) / 2).to(dtype)
        logits = torch.rand(seq, E, generator=g).to(dtype)
        tw, ti = torch.topk(torch.softmax(logits, dim=-1, dtype=torch.float32), top_k, dim=-1)
        e2e.append({"hidden_states": hs, "w1": w1, "w2": w2, "topk_weights": tw, "topk_idx": ti,
                    "renormalize": True,
                    "gt": _fixture_value(fns["TestFusedMoe.gt"], hs, w1, w2, tw, ti, True)})
    torch.save({"launcher": launcher, "e2e": e2e}, os.path.join(HERE, "fused_moe.pt"))

    # ---------------------------------------------------------------- varlen prefill attention
    fns = load_functions(os.path.join(tests, "test_prefill_attention.py"), ["TestPrefillAttention._torch_att"])
    att = fns["TestPrefillAttention._torch_att"]
    cases = []
    for i, (lens, hq, hkv, dtype) in enumerate([([96, 200, 128, 70], 2, 2, torch.float16),
                                                ([130, 64, 257], 4, 1, torch.bfloat16)]):
        g = torch.Generator().manual_seed(3000 + i)
        total, d = sum(lens), 128
        q = (torch.randn(total, hq, d, generator=g) * 0.2 + 0.1).to(dtype)
        k = (torch.randn(total, hkv, d, generator=g) * 0.2 + 0.4).to(dtype)
        v = (torch.randn(total, hkv, d, generator=g) * 0.2 + 0.3).to(dtype)
        outs, st = [], 0
        for n in lens:
            # the reference function is multi-head only: grouped queries = kv heads repeated
            kk = k[st:st + n].repeat_interleave(hq // hkv, 1)
            vv = v[st:st + n].repeat_interleave(hq // hkv, 1)
            outs.append(att(None, q[st:st + n], kk, vv, 1, n, hq, d))
            st += n
        cases.append({"q": q, "k": k, "v": v, "lens": lens, "gt": torch.cat(outs, 0)})
    torch.save(cases, os.path.join(HERE, "prefill_attention.pt"))

    # fp32 flash-attention CPU reference used by the reference's compiler tests
    fa = load_functions(os.path.join(args.reference, "test/ascend/cpu_verify/test_fa.py"), ["flash_attention_cpu"])
    g = torch.Generator().manual_seed(20)
    q = (torch.randn(1, 2, 192, 128, generator=g) * 0.5).to(torch.float16)
    k = (torch.randn(1, 2, 192, 128, generator=g) * 0.5).to(torch.float16)
    v = (torch.randn(1, 2, 192, 128, generator=g) * 0.5).to(torch.float16)
    torch.save({"q": q, "k": k, "v": v, "sm_scale": 0.5,
                "gt": fa["flash_attention_cpu"](q, k, v, 0.5, causal=True)}, os.path.join(HERE, "fa_cpu.pt"))

    # ---------------------------------------------------------------- paged decode attention
    fns = load_functions(os.path.join(tests, "test_paged_attention.py"),
                         ["_conti_input", "_make_bias", "_make_blocked_cache", "_naive_attention"])
    cases = []
    # first the reference test's own geometry (test_paged_attention.py:247-262: head sizes 48 and 32 with a
    # v head size of 32, 8 / 2 and 2 / 2 heads, 16-token pages, fp16), then the sizes of the benchmark
    ref_geometry = [(dk, 32, hq, hkv, 16, [50, 40, 30, 20], torch.float16)
                    for dk in (48, 32) for hq, hkv in ((8, 2), (2, 2))]
    for i, (d, dv, hq, hkv, page, hist, dtype) in enumerate(ref_geometry + [
            (64, 64, 8, 2, 16, [50, 40, 30, 20], torch.float16),
            (128, 128, 8, 2, 16, [150, 77, 200, 16], torch.bfloat16),
            (128, 128, 4, 4, 64, [64, 65, 1, 200], torch.float16),
            (96, 64, 4, 2, 32, [70, 3, 129, 64], torch.bfloat16)]):
        torch.manual_seed(123 + i)
        seq_lens = torch.tensor([1, 1, 1, 1])
        history = torch.tensor(hist)
        full = seq_lens + history
        bq = torch.rand(4, 1, hq, d).to(dtype)
        bk = torch.rand(4, int(full.max()), hkv, d).to(dtype)
        bv = torch.rand(4, int(full.max()), hkv, dv).to(dtype)
        nblk = (full + page - 1) // page
        offs = [torch.arange(int(n)) * 4 + idx for idx, n in enumerate(nblk)]
        table = torch.zeros(4, max(len(o) for o in offs), dtype=torch.int64)
        for o, row in zip(offs, table):
            row[:len(o)] = o
        mask = fns["_make_bias"](seq_lens, history, -1e30)
        gt = fns["_naive_attention"](bq, (bk, bv), mask)
        blocked_k, blocked_v = fns["_make_blocked_cache"](bk, bv, seq_lens, history, table, page, hkv, d, dv)
        cases.append({"q": fns["_conti_input"](bq, seq_lens), "k_cache": blocked_k, "v_cache": blocked_v,
                      "block_offsets": table, "kv_seqlens": full, "gt": fns["_conti_input"](gt, seq_lens)})
    torch.save(cases, os.path.join(HERE, "paged_decode.pt"))
    # ---------------------------------------------------------------- paged prefill with history (same test file:
    # the reference's test of the prefill branch, test_paged_attention.py:150-290, with its own mask builder)
    cases = []
    ref_geometry = [(dk, 32, hq, hkv, 16, [30, 50, 70, 90], [50, 40, 30, 20], torch.float16)
                    for dk in (48, 32) for hq, hkv in ((8, 2), (2, 2))]     # test_paged_attention.py:247-262
    for i, (d, dv, hq, hkv, page, seqs, hist, dtype) in enumerate(ref_geometry + [
            (64, 64, 8, 2, 16, [30, 50, 70, 90], [50, 40, 30, 20], torch.float16),
            (128, 128, 8, 2, 64, [5, 130, 1, 64], [100, 37, 200, 0], torch.bfloat16),
            (128, 128, 4, 4, 16, [17, 33, 2, 80], [0, 15, 64, 1], torch.float16),
            (80, 128, 4, 2, 32, [40, 150, 3, 64], [9, 0, 70, 64], torch.bfloat16)]):
        torch.manual_seed(223 + i)
        seq_lens = torch.tensor(seqs)
        history = torch.tensor(hist)
        full = seq_lens + history
        bq = torch.rand(4, int(seq_lens.max()), hq, d).to(dtype)
        bk = torch.rand(4, int(full.max()), hkv, d).to(dtype)
        bv = torch.rand(4, int(full.max()), hkv, dv).to(dtype)
        nblk = (full + page - 1) // page
        offs = [torch.arange(int(n)) * 4 + idx for idx, n in enumerate(nblk)]
        table = torch.zeros(4, max(len(o) for o in offs), dtype=torch.int64)
        for o, row in zip(offs, table):
            row[:len(o)] = o
        mask = fns["_make_bias"](seq_lens, history, -1e30)
        gt = fns["_naive_attention"](bq, (bk, bv), mask)
        blocked_k, blocked_v = fns["_make_blocked_cache"](bk, bv, seq_lens, history, table, page, hkv, d, dv)
        cases.append({"q": fns["_conti_input"](bq, seq_lens), "k_cache": blocked_k, "v_cache": blocked_v,
                      "block_offsets": table, "q_seqlens": seq_lens, "kv_seqlens": full,
                      "gt": fns["_conti_input"](gt, seq_lens)})
    torch.save(cases, os.path.join(HERE, "paged_prefill.pt"))
    # ---------------------------------------------------------------- rms_norm / add_rms_norm
    fns = load_functions(os.path.join(tests, "test_rms_norm.py"), ["TestRMSNorm.gt"])
    rms_gt = fns["TestRMSNorm.gt"]           # a fixture that `return`s its value
    fuse = load_functions(os.path.join(tests, "test_add_rms_norm.py"), ["FuseRMSNorm.forward"])["FuseRMSNorm.forward"]

    class _Holder:                           # the attributes FuseRMSNorm.forward reads from `self`
        def __init__(self, w, eps):
            self.weight, self.variance_epsilon = w, eps

    cases = []
    for i, (rows, n, dtype) in enumerate([(4, 8, torch.float16), (4, 8, torch.float32), (16, 4096, torch.bfloat16),
                                          (8, 1000, torch.float16)]):
        g = torch.Generator().manual_seed(4000 + i)
        x = torch.rand(rows, n, generator=g).to(dtype)
        w = torch.rand(n, generator=g).to(dtype)
        res = torch.randn(rows, n, generator=g).to(dtype)
        fused_out, fused_res = fuse(_Holder(w, 1e-6), x.clone(), res.clone())
        cases.append({"x": x, "w": w, "res": res, "eps": 1e-6, "gt_rms": rms_gt(None, x, w, 1e-6),
                      "gt_add_out": fused_out, "gt_add_res": fused_res})
    torch.save(cases, os.path.join(HERE, "rms_norm.pt"))

    # ---------------------------------------------------------------- rotary
    fns = load_functions(os.path.join(tests, "test_apply_rotary.py"), ["_rotate_half", "TestApplyRotary.gt"])
    cases = []
    for i, (hq, hk, dim, dtype) in enumerate([(8, 8, 16, torch.bfloat16), (8, 4, 16, torch.float16),
                                              (8, 4, 16, torch.float32), (4, 2, 128, torch.bfloat16)]):
        g = torch.Generator().manual_seed(5000 + i)
        tokens, max_len = 45, 16
        q = torch.rand(tokens, hq, dim, generator=g).to(dtype)
        k = torch.rand(tokens, hk, dim, generator=g).to(dtype)
        pos = torch.randint(0, max_len, (tokens,), generator=g)
        cos = torch.rand(max_len, dim, generator=g).to(dtype)[pos, None, :]
        sin = torch.rand(max_len, dim, generator=g).to(dtype)[pos, None, :]
        gq, gk = _fixture_value(fns["TestApplyRotary.gt"], q, k, cos, sin, pos)
        cases.append({"q": q, "k": k, "cos": cos, "sin": sin, "gt_q": gq, "gt_k": gk})
    torch.save(cases, os.path.join(HERE, "rotary.pt"))

    # ---------------------------------------------------------------- fill_kv_cache
    fns = load_functions(os.path.join(tests, "test_fill_kv_cache.py"), ["_div_up", "TestFillKVCache.gt"])
    cases = []
    for i, (seq_lens, hist) in enumerate([((1, 1, 1, 1), (1, 16, 31, 24)), ((1, 8, 16, 24), (1, 16, 31, 24)),
                                          ((70, 3), (60, 200))]):
        g = torch.Generator().manual_seed(6000 + i)
        heads, d, page = (8, 128, 64) if i == 0 else (2, 64, 64)
        kv_lens = [s + h for s, h in zip(seq_lens, hist)]
        nblk = [(n + page - 1) // page for n in kv_lens]
        B, mx = len(seq_lens), max(nblk)
        ks = torch.rand(sum(seq_lens), heads, d, generator=g).to(torch.bfloat16)
        vs = torch.rand(sum(seq_lens), heads, d, generator=g).to(torch.bfloat16)
        kc = torch.zeros(B * mx, page, heads, d, dtype=torch.bfloat16)
        vc = torch.rand(B * mx, page, heads, d, generator=g).to(torch.bfloat16)
        table = torch.zeros(B, mx, dtype=torch.int64)
        perm = torch.randperm(B * mx, generator=g)
        off = 0
        for b in range(B):
            table[b, :nblk[b]] = perm[off:off + nblk[b]]
            off += nblk[b]
        gk, gv = _fixture_value(fns["TestFillKVCache.gt"], ks, vs, kc, vc, list(seq_lens), list(hist), table, page)
        cases.append({"k_states": ks, "v_states": vs, "k_caches": kc, "v_caches": vc, "seq_lens": list(seq_lens),
                      "history_lens": list(hist), "block_offsets": table, "gt_k": gk, "gt_v": gv})
    torch.save(cases, os.path.join(HERE, "fill_kv_cache.pt"))

    # ---------------------------------------------------------------- GShard top-k gating with capacity
    from collections import namedtuple
    from typing import Tuple

    info = namedtuple("GatingTokenRearrangeInfo",
                      ["token_rearranged_ec_idx", "token_exp_weights", "expert_select_token_idx"])
    bench_file = os.path.join(args.reference, "python/dlBLAS/benchmarks/topk_gating.py")
    fns = load_functions(bench_file, ["_capacity", "fused_topkgating_opt"],
                         {"Tensor": torch.Tensor, "Tuple": Tuple, "TUTEL_INSTALLED": False,
                          "GatingTokenRearrangeInfo": info})
    cases = []
    for i, (S, E, k, cf, mc) in enumerate([(256, 8, 2, 1.0, 2), (512, 64, 8, 1.0, 2), (128, 16, 4, 0.5, 4),
                                           (64, 32, 2, 2.0, 2)]):
        g = torch.Generator().manual_seed(7000 + i)
        logits = torch.randn(S, E, generator=g)
        l_aux, rearr = fns["fused_topkgating_opt"](logits, k, cf, mc)
        cases.append({"logits": logits, "k": k, "capacity_factor": cf, "min_capacity": mc, "l_aux": l_aux,
                      "ec_idx": rearr.token_rearranged_ec_idx, "weights": rearr.token_exp_weights,
                      "select": rearr.expert_select_token_idx})
    torch.save(cases, os.path.join(HERE, "topk_gating.pt"))

    for f in sorted(os.listdir(HERE)):
        if f.endswith(".pt"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
