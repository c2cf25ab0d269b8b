"""GPU parity: fused_moe (tcgen05 grouped GEMM) against the CPU oracle and the golden fixtures."""
import os

import pytest
import torch

from dlcompiler_b200 import fused_moe, fused_moe_kernel_launcher, get_start_end
from dlcompiler_b200 import workloads as W
from oracle import dlblas_oracle as oracle

pytestmark = pytest.mark.gpu

# stated bound for bf16 GEMM results
RTOL = ATOL = 2e-2


def _to(dev, *ts):
    return [t.to(dev) for t in ts]


def test_launcher_golden(cuda_device, golden_dir):
    c = torch.load(os.path.join(golden_dir, "fused_moe.pt"), weights_only=True)["launcher"]
    A, B, weights, topk_idx = _to(cuda_device, c["A"], c["B"], c["weights"], c["topk_idx"])
    top_k, E = c["top_k"], B.size(0)
    flat = topk_idx.flatten()
    sorted_idx = flat.argsort()
    exp_start, exp_end = get_start_end(flat, sorted_idx, E)
    C = torch.zeros(A.size(0), top_k, B.size(1), dtype=A.dtype, device=cuda_device)
    fused_moe_kernel_launcher(A, B, C, sorted_idx, exp_start, exp_end, weights, enable_weights=True, top_k=top_k,
                              num_tokens=A.size(0), expert_offset=0, reindex_a=True, reindex_c=True)
    # reference test: assert_close defaults for fp16 (test_fused_moe.py:145)
    torch.testing.assert_close(C.flatten(0, 1).cpu(), c["gt"], rtol=1e-3, atol=1e-3)


def test_launcher_sorted_output_order(cuda_device, golden_dir):
    """reindex_c=False writes rows in expert-sorted order (GEMM1 of fused_moe.py:334-348)."""
    c = torch.load(os.path.join(golden_dir, "fused_moe.pt"), weights_only=True)["launcher"]
    A, B, topk_idx = _to(cuda_device, c["A"], c["B"], c["topk_idx"])
    top_k, E = c["top_k"], B.size(0)
    flat = topk_idx.flatten()
    sorted_idx = flat.argsort(stable=True)
    exp_start, exp_end = get_start_end(flat, sorted_idx, E)
    C = torch.zeros(A.size(0) * top_k, B.size(1), dtype=A.dtype, device=cuda_device)
    fused_moe_kernel_launcher(A, B, C, sorted_idx, exp_start, exp_end, None, enable_weights=False, top_k=top_k,
                              num_tokens=A.size(0), reindex_a=True, reindex_c=False)
    ref = oracle.fused_moe_launcher_gt(c["A"], c["B"], top_k, c["topk_idx"])[sorted_idx.cpu()]
    torch.testing.assert_close(C.cpu(), ref, rtol=1e-3, atol=1e-3)


def test_fused_moe_golden(cuda_device, golden_dir):
    for c in torch.load(os.path.join(golden_dir, "fused_moe.pt"), weights_only=True)["e2e"]:
        hs, w1, w2, tw, ti = _to(cuda_device, c["hidden_states"], c["w1"], c["w2"], c["topk_weights"], c["topk_idx"])
        out = fused_moe(hs, w1, w2, tw, ti, topk=ti.size(1), renormalize=c["renormalize"]).cpu()
        tol = 1e-3 if out.dtype == torch.float16 else 8e-3     # reference test: 1e-3 for fp16
        torch.testing.assert_close(out, c["gt"], rtol=tol, atol=tol)
        rf = oracle.fused_moe_rounding_faithful(c["hidden_states"], c["w1"], c["w2"], c["topk_weights"],
                                                c["topk_idx"], renormalize=True)
        eps = torch.finfo(out.dtype).eps
        torch.testing.assert_close(out.float(), rf.float(), rtol=2 * eps, atol=2 * eps * rf.abs().max().item())


@pytest.mark.parametrize("T,H,I,E,k,dtype", [
    (1, 128, 128, 4, 2, torch.bfloat16),
    (77, 256, 384, 8, 2, torch.bfloat16),       # ragged: N not a multiple of the tile, K not a multiple of 64*?
    (300, 1024, 512, 8, 3, torch.float16),
    (512, 512, 1024, 16, 4, torch.bfloat16),
    (64, 64, 64, 2, 1, torch.bfloat16),
    (129, 200, 72, 3, 2, torch.bfloat16),       # K and N multiples of 8 only
])
def test_fused_moe_shapes(cuda_device, T, H, I, E, k, dtype):
    g = torch.Generator().manual_seed(T * 7 + H)
    hs = (torch.randn(T, H, generator=g)).to(dtype)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * (H ** -0.5)).to(dtype)
    w2 = (torch.randn(E, H, I, generator=g) * (I ** -0.5)).to(dtype)
    tw, ti = oracle.softmax_topk(torch.randn(T, E, generator=g), k)
    out = fused_moe(*_to(cuda_device, hs, w1, w2, tw, ti), topk=k).cpu()
    ref = oracle.fused_moe_rounding_faithful(hs, w1, w2, tw, ti.long())
    torch.testing.assert_close(out.float(), ref.float(), rtol=RTOL, atol=ATOL)
    eps = torch.finfo(dtype).eps
    torch.testing.assert_close(out.float(), ref.float(), rtol=4 * eps, atol=4 * eps * ref.abs().max().item())


def test_fused_moe_empty_and_unused_experts(cuda_device):
    dev = cuda_device
    hs = torch.randn(0, 128, dtype=torch.bfloat16, device=dev)
    w1 = torch.randn(4, 256, 128, dtype=torch.bfloat16, device=dev)
    w2 = torch.randn(4, 128, 128, dtype=torch.bfloat16, device=dev)
    out = fused_moe(hs, w1, w2, torch.zeros(0, 2, device=dev), torch.zeros(0, 2, dtype=torch.int64, device=dev), 2)
    assert out.shape == (0, 128)
    # every token routed to expert 3 only
    g = torch.Generator().manual_seed(3)
    hs = torch.randn(200, 128, generator=g).to(torch.bfloat16)
    w1c = (torch.randn(4, 256, 128, generator=g) * 0.1).to(torch.bfloat16)
    w2c = (torch.randn(4, 128, 128, generator=g) * 0.1).to(torch.bfloat16)
    ti = torch.full((200, 1), 3, dtype=torch.int64)
    tw = torch.ones(200, 1)
    out = fused_moe(*_to(dev, hs, w1c, w2c, tw, ti), topk=1).cpu()
    ref = oracle.fused_moe_rounding_faithful(hs, w1c, w2c, tw, ti)
    torch.testing.assert_close(out.float(), ref.float(), rtol=RTOL, atol=ATOL)


def test_fused_moe_expert_slices_sum_to_full(cuda_device):
    """The reference's expert-parallel mode: each slice computes its local experts, zeros elsewhere
    (fused_moe.py:113-114, 329-332); the slices add up to the full result."""
    g = torch.Generator().manual_seed(9)
    T, H, I, E, k = 256, 256, 256, 8, 2
    hs = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16)
    tw, ti = oracle.softmax_topk(torch.randn(T, E, generator=g), k)
    hs_d, w1_d, w2_d, tw_d, ti_d = _to(cuda_device, hs, w1, w2, tw, ti)
    full = fused_moe(hs_d, w1_d, w2_d, tw_d, ti_d, k).float()
    acc = torch.zeros_like(full)
    for off in range(0, E, 2):
        acc += fused_moe(hs_d, w1_d[off:off + 2], w2_d[off:off + 2], tw_d, ti_d, k, expert_offset=off,
                         num_experts=E).float()
    torch.testing.assert_close(acc, full, rtol=RTOL, atol=ATOL)


def test_fused_moe_config_sample_and_linearity(cuda_device):
    """Full benchmark shape: a token sample against the oracle, plus size-independent properties."""
    wl = W.MoeWorkload()
    d = wl.make()
    tw, ti = oracle.softmax_topk(d["router_logits"], wl.top_k)
    hs, w1, w2, tw_d, ti_d = _to(cuda_device, d["hidden_states"], d["w1"], d["w2"], tw, ti)
    out = fused_moe(hs, w1, w2, tw_d, ti_d, wl.top_k)
    again = fused_moe(hs, w1, w2, tw_d, ti_d, wl.top_k)
    assert torch.equal(out, again)                                   # deterministic
    sample = torch.arange(0, wl.tokens, 173)[:24]
    ref = oracle.fused_moe_rounding_faithful(d["hidden_states"][sample], d["w1"], d["w2"], tw[sample],
                                             ti[sample].long())
    torch.testing.assert_close(out[sample].cpu().float(), ref.float(), rtol=RTOL, atol=ATOL)
    # scaling the routing weights by 2 scales the output by 2 (exact in binary floating point)
    twice = fused_moe(hs, w1, w2, tw_d * 2, ti_d, wl.top_k)
    assert torch.equal(twice, out * 2)
    # a token's result does not depend on the other tokens in the batch
    sub = fused_moe(hs[sample.to(cuda_device)], w1, w2, tw_d[sample.to(cuda_device)], ti_d[sample.to(cuda_device)],
                    wl.top_k)
    assert torch.equal(sub, out[sample.to(cuda_device)])
