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


@pytest.mark.parametrize("T,H,I,E,k,dtype,skew", [
    (1200, 256, 384, 2, 2, torch.bfloat16, 0.0),     # both experts get 1200 rows: 9 + 1 blocks -> 4-5 pairs + a tail
    (1500, 512, 256, 3, 1, torch.bfloat16, 2.0),     # skewed: one long expert, one short, odd and even counts
    (2048, 200, 72, 4, 2, torch.float16, 1.0),       # K, N multiples of 8 only, on the pair path
    (1024, 128, 128, 2, 1, torch.bfloat16, 50.0),    # everything on expert 0, expert 1 empty
])
def test_fused_moe_many_blocks_per_expert(cuda_device, T, H, I, E, k, dtype, skew):
    """Few experts with many 128-row blocks each: odd and even block counts, a long and a short expert, an
    empty expert; bit-reproducible from call to call."""
    g = torch.Generator().manual_seed(T + 13 * E)
    hs = (torch.randn(T, H, generator=g)).to(dtype)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * (H ** -0.5)).to(dtype)
    w2 = (torch.randn(E, H, I, generator=g) * (I ** -0.5)).to(dtype)
    logits = torch.randn(T, E, generator=g) - skew * torch.arange(E)
    tw, ti = oracle.softmax_topk(logits, k)
    args = _to(cuda_device, hs, w1, w2, tw, ti)
    out = fused_moe(*args, topk=k)
    assert torch.equal(out, fused_moe(*args, topk=k))
    ref = oracle.fused_moe_rounding_faithful(hs, w1, w2, tw, ti.long())
    eps = torch.finfo(dtype).eps
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=4 * eps, atol=4 * eps * ref.abs().max().item())


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


def test_fused_moe_config_all_tokens_and_linearity(cuda_device):
    """Full benchmark shape: every token against the oracle, plus size-independent properties."""
    wl = W.MoeWorkload()
    d = wl.make()
    tw, ti = oracle.softmax_topk(d["router_logits"], wl.top_k)
    hs, w1, w2, tw_d, ti_d = _to(cuda_device, d["hidden_states"], d["w1"], d["w2"], tw, ti)
    out = fused_moe(hs, w1, w2, tw_d, ti_d, wl.top_k)
    again = fused_moe(hs, w1, w2, tw_d, ti_d, wl.top_k)
    assert torch.equal(out, again)                                   # deterministic
    torch.set_num_threads(os.cpu_count() or 1)
    ref = oracle.fused_moe_rounding_faithful(d["hidden_states"], d["w1"], d["w2"], tw, ti.long())
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=RTOL, atol=ATOL)
    sample = torch.arange(0, wl.tokens, 173)[:24]
    # scaling the routing weights by 2 scales the output by 2 (exact in binary floating point)
    twice = fused_moe(hs, w1, w2, tw_d * 2, ti_d, wl.top_k)
    assert torch.equal(twice, out * 2)
    # a token's result does not depend on the other tokens in the batch
    sub = fused_moe(hs[sample.to(cuda_device)], w1, w2, tw_d[sample.to(cuda_device)], ti_d[sample.to(cuda_device)],
                    wl.top_k)
    assert torch.equal(sub, out[sample.to(cuda_device)])


def test_fused_moe_ids_outside_the_expert_range_add_nothing(cuda_device):
    """Padding ids (-1) and ids of experts this call does not hold contribute zero, with the default
    arguments as well as with an explicit num_experts (the reference zero-fills its intermediate buffers
    for this, fused_moe.py:308-312, 329-332); no stale memory may leak into the sum."""
    g = torch.Generator().manual_seed(21)
    T, H, I, E, k = 200, 256, 256, 4, 2
    hs = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16)
    tw, ti = oracle.softmax_topk(torch.randn(T, E, generator=g), k)
    ti = ti.long().clone()
    ti[::3, 1] = -1
    ti[1::7, 0] = E + 2
    keep = ((ti >= 0) & (ti < E))
    ref = oracle.fused_moe_rounding_faithful(hs, w1, w2, tw * keep, ti.clamp(0, E - 1))
    hs_d, w1_d, w2_d, tw_d, ti_d = _to(cuda_device, hs, w1, w2, tw, ti)
    # poison the allocator's free blocks so that an unwritten row would show
    junk = torch.full((T * k, H), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    del junk
    for kwargs in ({}, {"num_experts": E}):
        out = fused_moe(hs_d, w1_d, w2_d, tw_d, ti_d, k, **kwargs)
        assert torch.isfinite(out.float()).all()
        torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=RTOL, atol=ATOL)


def test_get_start_end_matches_the_reference_kernel_semantics(cuda_device):
    """[start, end) per expert inside the argsort of the ids (fused_moe.py:238-293): negative ids sort first and
    shift every start, ids >= num_experts sort last, an absent expert gets (0, 0); dtype follows sorted_idx."""
    from dlcompiler_b200 import get_start_end

    g = torch.Generator().manual_seed(5)
    E = 8
    ids = torch.randint(0, E, (300, 2), generator=g)
    ids[ids == 5] = 6                       # expert 5 has no slot
    ids[::11, 0] = -1
    ids[3::13, 1] = E + 1
    flat = ids.flatten()
    order = flat.argsort()
    sv = flat[order]
    exp_s, exp_e = [], []
    for e in range(E):
        pos = torch.nonzero(sv == e).flatten()
        exp_s.append(int(pos[0]) if pos.numel() else 0)
        exp_e.append(int(pos[0]) + pos.numel() if pos.numel() else 0)
    for dt in (torch.int64, torch.int32):
        s, e = get_start_end(ids.to(cuda_device), order.to(dt).to(cuda_device), E)
        assert s.dtype == dt and e.dtype == dt
        assert s.cpu().tolist() == exp_s and e.cpu().tolist() == exp_e
    s0, e0 = oracle.start_end_from_counts(torch.randint(0, E, (64, 2), generator=g), E)
    assert (e0 - s0).sum() == 128
