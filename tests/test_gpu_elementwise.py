"""GPU parity: silu_and_mul, routers, moe_align_block_size (through the C ABI via the wrappers)."""
import os

import pytest
import torch

from dlcompiler_b200 import grouped_topk_gating, moe_align_block_size, silu_and_mul, softmax_topk
from dlcompiler_b200 import workloads as W
from dlcompiler_b200.kernels.fused_moe import _moe_align
from oracle import dlblas_oracle as oracle

pytestmark = pytest.mark.gpu


def _ulp_close(out, ref, max_ulp=1):
    """bf16/fp16 results may differ by one rounding step where fp32 intermediates differ in the last bit."""
    eps = torch.finfo(out.dtype).eps
    torch.testing.assert_close(out.float(), ref.float(), rtol=max_ulp * eps, atol=1e-6)


def test_silu_golden(cuda_device, golden_dir):
    for case in torch.load(os.path.join(golden_dir, "silu_and_mul.pt"), weights_only=True):
        out = silu_and_mul(case["x"].to(cuda_device)).cpu()
        _ulp_close(out, case["gt"], max_ulp=2)   # reference ground truth rounds silu separately


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,n", [(1, 8), (3, 11008), (256, 2048), (256, 384), (7, 13), (0, 64), (5, 1)])
def test_silu_shapes(cuda_device, dtype, rows, n):
    g = torch.Generator().manual_seed(rows * 1000 + n)
    x = torch.randn(rows, 2 * n, generator=g).to(dtype)
    out = silu_and_mul(x.to(cuda_device)).cpu()
    ref = oracle.silu_and_mul_fp32(x)
    assert out.shape == ref.shape
    if dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-6)
    else:
        _ulp_close(out, ref)


def test_silu_strided_and_out(cuda_device):
    g = torch.Generator().manual_seed(5)
    big = torch.randn(64, 4096 + 64, generator=g).to(torch.bfloat16).to(cuda_device)
    x = big[:, :4096]                       # row stride larger than the row
    outbuf = torch.zeros(64, 2048 + 8, dtype=torch.bfloat16, device=cuda_device)
    out = silu_and_mul(x, out=outbuf[:, :2048])
    assert out.data_ptr() == outbuf.data_ptr()
    _ulp_close(out.cpu(), oracle.silu_and_mul_fp32(x.cpu()))
    assert torch.all(outbuf[:, 2048:] == 0)


def test_silu_full_size_property(cuda_device):
    wl = W.SiluWorkload()
    x = wl.make()["gate_up"].to(cuda_device)
    out = silu_and_mul(x)
    # sampled rows against the oracle, plus the identity silu(g)*u == -silu(g)*(-u) on the full tensor
    rows = torch.tensor([0, 1, 777, 4095])
    _ulp_close(out[rows].cpu(), oracle.silu_and_mul_fp32(x[rows].cpu()))
    x2 = x.clone()
    x2[:, wl.hidden:] = -x2[:, wl.hidden:]
    assert torch.equal(silu_and_mul(x2), -out)


def test_grouped_gating_config(cuda_device):
    wl = W.GatingWorkload()
    d = wl.make()
    ids, w = grouped_topk_gating(d["logits"].to(cuda_device), d["bias"].to(cuda_device), wl.top_k, wl.n_group,
                                 wl.topk_group, wl.scale_factor, True, "sigmoid")
    rid, rw = oracle.grouped_topk_gating(d["logits"], d["bias"], wl.top_k, wl.n_group, wl.topk_group,
                                         wl.scale_factor, True, "sigmoid")
    ids, w = ids.cpu(), w.cpu()
    if not torch.equal(ids, rid):
        bad = (ids != rid).any(-1).nonzero().flatten()
        m = oracle.gating_margins(d["logits"][bad], d["bias"], wl.top_k, wl.n_group, wl.topk_group)
        raise AssertionError(f"{bad.numel()} tokens differ; smallest fp64 margin among them {m.min().item():.3e}")
    torch.testing.assert_close(w, rw, rtol=1e-3, atol=1e-3)   # stated bound: <= 1e-3 on fp32 weights
    torch.testing.assert_close(w, rw, rtol=2e-6, atol=1e-6)   # achieved


@pytest.mark.parametrize("T,E,ng,tg,k,scoring", [
    (1, 256, 8, 4, 8, "sigmoid"), (33, 64, 1, 1, 6, "softmax"), (100, 8, 1, 1, 2, "softmax"),
    (257, 128, 4, 2, 8, "sigmoid"), (64, 32, 8, 3, 4, "sigmoid"), (19, 512, 16, 4, 8, "sigmoid"),
    (50, 160, 1, 1, 6, "softmax"), (0, 64, 1, 1, 2, "softmax"),
])
def test_gating_shapes(cuda_device, T, E, ng, tg, k, scoring):
    g = torch.Generator().manual_seed(T + E)
    logits = torch.randn(T, E, generator=g)
    bias = torch.randn(E, generator=g) * 0.01 if scoring == "sigmoid" else None
    ids, w = grouped_topk_gating(logits.to(cuda_device), None if bias is None else bias.to(cuda_device), k, ng, tg,
                                 1.0, True, scoring)
    rid, rw = oracle.grouped_topk_gating(logits, bias, k, ng, tg, 1.0, True, scoring)
    assert torch.equal(ids.cpu(), rid)
    torch.testing.assert_close(w.cpu(), rw, rtol=1e-5, atol=1e-6)


def test_gating_ties_go_to_lower_index(cuda_device):
    logits = torch.zeros(4, 64, device=cuda_device)
    ids, w = grouped_topk_gating(logits, None, 4, 4, 2, 1.0, True, "sigmoid")
    assert ids.cpu().tolist() == [[0, 1, 2, 3]] * 4
    w2, ids2 = softmax_topk(torch.zeros(2, 8, device=cuda_device), 2)
    assert ids2.cpu().tolist() == [[0, 1]] * 2
    torch.testing.assert_close(w2.cpu(), torch.full((2, 2), 0.125))


@pytest.mark.parametrize("E,ng,tg,k", [(256, 8, 4, 8), (128, 1, 1, 6), (512, 16, 4, 8)])
def test_gating_many_equal_scores(cuda_device, E, ng, tg, k):
    """Logits from five distinct values: equal scores inside lanes, across lanes and across groups."""
    g = torch.Generator().manual_seed(E)
    logits = torch.randint(-2, 3, (96, E), generator=g).float()
    bias = torch.randint(0, 2, (E,), generator=g).float() * 0.25
    ids, w = grouped_topk_gating(logits.to(cuda_device), bias.to(cuda_device), k, ng, tg, 1.0, True, "sigmoid")
    rid, rw = oracle.grouped_topk_gating(logits, bias, k, ng, tg, 1.0, True, "sigmoid")
    assert torch.equal(ids.cpu(), rid)
    torch.testing.assert_close(w.cpu(), rw, rtol=1e-5, atol=1e-6)


def test_gating_is_deterministic(cuda_device):
    wl = W.GatingWorkload(tokens=4096)
    d = wl.make()
    lg, b = d["logits"].to(cuda_device), d["bias"].to(cuda_device)
    a = grouped_topk_gating(lg, b, 8, 8, 4, 2.5)
    for _ in range(3):
        c = grouped_topk_gating(lg, b, 8, 8, 4, 2.5)
        assert torch.equal(a[0], c[0]) and torch.equal(a[1], c[1])


@pytest.mark.parametrize("numel,E,block,dtype", [
    (0, 4, 16, torch.int64), (1, 4, 16, torch.int32), (37, 5, 8, torch.int64), (8192, 8, 128, torch.int64),
    (1000, 256, 128, torch.int32), (131072, 256, 128, torch.int32), (5000, 1024, 64, torch.int64),
    (4096, 1, 128, torch.int64),
])
def test_moe_align_bit_exact(cuda_device, numel, E, block, dtype):
    g = torch.Generator().manual_seed(numel + E)
    ids = torch.randint(0, E, (numel,), generator=g).to(dtype)
    s, e, n, bs = _moe_align(ids.to(cuda_device), block, E)
    rs, re_, rn, rbs = oracle.moe_align_block_size(ids, block, E)
    assert torch.equal(n.cpu(), rn)
    assert torch.equal(s.cpu(), rs)
    assert torch.equal(e.cpu(), re_)
    assert torch.equal(bs.cpu(), rbs)


def test_moe_align_config_and_foreign_ids(cuda_device):
    wl = W.MoeWorkload()
    logits = wl.make(weights=False)["router_logits"]
    _, ids = oracle.softmax_topk(logits, wl.top_k)
    s, e, n = moe_align_block_size(ids.to(cuda_device), 128, wl.experts)
    rs, re_, rn, _ = oracle.moe_align_block_size(ids, 128, wl.experts)
    assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re_) and torch.equal(n.cpu(), rn)
    # ids outside [0, E) are dropped (expert-parallel slices)
    local = ids - 4
    s, e, n = moe_align_block_size(local.to(cuda_device), 128, 4)
    rs, re_, rn, _ = oracle.moe_align_block_size(local, 128, 4)
    assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re_) and torch.equal(n.cpu(), rn)


def test_grouped_gating_matches_transformers_fixture(cuda_device, golden_dir):
    """The CUDA router against the output of transformers' DeepseekV3MoE.route_tokens_to_experts (fixture made by
    tests/golden/make_golden_third_party.py): same expert set per token, weights within fp32 rounding."""
    for case in torch.load(os.path.join(golden_dir, "grouped_gating_hf.pt"), weights_only=True):
        ids, w = grouped_topk_gating(case["logits"].to(cuda_device), case["bias"].to(cuda_device), case["top_k"],
                                     case["n_group"], case["topk_group"], case["scale"], case["renormalize"], "sigmoid")
        keep = oracle.gating_margins(case["logits"], case["bias"], case["top_k"], case["n_group"],
                                     case["topk_group"]) > 1e-6
        a, ai = torch.sort(ids.cpu().long()[keep], dim=-1)
        b, bi = torch.sort(case["ids"].long()[keep], dim=-1)
        assert torch.equal(a, b)
        torch.testing.assert_close(w.cpu()[keep].gather(1, ai), case["weights"][keep].gather(1, bi), rtol=2e-6, atol=2e-6)


def test_moe_align_matches_vllm_documented_example(cuda_device, golden_dir):
    d = torch.load(os.path.join(golden_dir, "moe_align_vllm_doc.pt"), weights_only=True)
    ids, block, want = d["topk_ids"], d["block_size"], d["token_ids"]
    s, e, n = moe_align_block_size(ids.to(cuda_device), block, int(ids.max()) + 1)
    assert int(n.item()) == want.numel()
    assert torch.equal(s.cpu()[:want.numel()], want)
    assert e.cpu()[:want.numel() // block].tolist() == [1, 2, 3, 4]
