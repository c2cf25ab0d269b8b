"""The CPU oracle against fixtures produced by the reference tests' own ground-truth code."""
import os

import torch

from oracle import dlblas_oracle as oracle


def _load(golden_dir, name):
    return torch.load(os.path.join(golden_dir, name), weights_only=True)


def test_silu_matches_reference_ground_truth(golden_dir):
    for case in _load(golden_dir, "silu_and_mul.pt"):
        x, gt = case["x"], case["gt"]
        # same formula, same dtype: bit-exact
        assert torch.equal(oracle.silu_and_mul(x), gt)
        # fp32 form differs from the half-precision ground truth by at most one rounding
        eps = torch.finfo(x.dtype).eps
        torch.testing.assert_close(oracle.silu_and_mul_fp32(x), gt, rtol=2 * eps, atol=1e-5)


def test_fused_moe_launcher_ground_truth(golden_dir):
    c = _load(golden_dir, "fused_moe.pt")["launcher"]
    out = oracle.fused_moe_launcher_gt(c["A"], c["B"], c["top_k"], c["topk_idx"], c["weights"])
    assert torch.equal(out, c["gt"])


def test_fused_moe_end_to_end_ground_truth(golden_dir):
    for c in _load(golden_dir, "fused_moe.pt")["e2e"]:
        out = oracle.fused_moe(c["hidden_states"], c["w1"], c["w2"], c["topk_weights"], c["topk_idx"],
                               renormalize=c["renormalize"])
        assert torch.equal(out, c["gt"])
        # the kernel-faithful rounding variant stays within the reference test's tolerance band
        # (its own test uses atol=rtol=1e-3 for fp16; bf16 has 8x coarser steps)
        tol = 1e-3 if out.dtype == torch.float16 else 8e-3
        rf = oracle.fused_moe_rounding_faithful(c["hidden_states"], c["w1"], c["w2"], c["topk_weights"],
                                                c["topk_idx"], renormalize=c["renormalize"])
        torch.testing.assert_close(rf, c["gt"], atol=tol, rtol=tol)


def test_prefill_attention_ground_truth(golden_dir):
    for c in _load(golden_dir, "prefill_attention.pt"):
        lens = c["lens"]
        start = [0]
        for n in lens[:-1]:
            start.append(start[-1] + n)
        out = oracle.context_attention(c["q"], c["k"], c["v"], torch.tensor(start), torch.tensor(lens))
        # reference test tolerance: atol=1e-2, rtol=0 (test_prefill_attention.py:83)
        torch.testing.assert_close(out, c["gt"], atol=1e-2 if out.dtype == torch.float16 else 2e-2, rtol=0)


def test_flash_attention_cpu_reference(golden_dir):
    c = _load(golden_dir, "fa_cpu.pt")
    q, k, v = c["q"][0], c["k"][0], c["v"][0]          # [H, S, D]
    S = q.shape[1]
    qq, kk, vv = (t.transpose(0, 1).contiguous() for t in (q, k, v))
    out, lse = oracle.context_attention(qq, kk, vv, torch.tensor([0]), torch.tensor([S]), sm_scale=c["sm_scale"],
                                        return_lse=True)
    torch.testing.assert_close(out.transpose(0, 1), c["gt"][0], atol=2e-3, rtol=0)
    # LSE against a direct evaluation of max*scale + log(sum) (flash_attention.py:152-155)
    sc = torch.matmul(q.float(), k.float().transpose(1, 2)) * c["sm_scale"]
    sc = sc.masked_fill(torch.triu(torch.ones(S, S), diagonal=1).bool(), float("-inf"))
    torch.testing.assert_close(lse, torch.logsumexp(sc, dim=-1), atol=1e-4, rtol=1e-5)


def test_paged_decode_ground_truth(golden_dir):
    for c in _load(golden_dir, "paged_decode.pt"):
        out = oracle.paged_decode_attention(c["q"], c["k_cache"], c["v_cache"], c["block_offsets"], c["kv_seqlens"])
        # reference test tolerance for fp16: atol=1e-3, rtol=1e-5 (test_paged_attention.py:286)
        tol = 1e-3 if out.dtype == torch.float16 else 8e-3
        torch.testing.assert_close(out, c["gt"], atol=tol, rtol=1e-5)


def test_paged_prefill_ground_truth(golden_dir):
    """Prefill over a paged cache with history against the reference test's own mask builder and naive
    attention (test_paged_attention.py:14-25,61-84)."""
    for c in _load(golden_dir, "paged_prefill.pt"):
        q_lens = c["q_seqlens"]
        start = torch.cumsum(q_lens, 0) - q_lens
        out = oracle.paged_prefill_attention(c["q"], c["k_cache"], c["v_cache"], c["block_offsets"], start, q_lens,
                                             c["kv_seqlens"])
        tol = 1e-3 if out.dtype == torch.float16 else 8e-3
        torch.testing.assert_close(out, c["gt"], atol=tol, rtol=1e-5)


def test_rms_norm_ground_truths(golden_dir):
    for c in _load(golden_dir, "rms_norm.pt"):
        x, w, res, eps = c["x"], c["w"], c["res"], c["eps"]
        assert torch.equal(oracle.rms_norm_test_gt(x, w, eps), c["gt_rms"])
        # the registry op's convention (cast, then weight) is exactly the fused module of test_add_rms_norm.py
        out, new_x = oracle.rms_norm(x, w, eps, residual=res, weight_after_cast=True)
        assert torch.equal(new_x, c["gt_add_res"])
        torch.testing.assert_close(out, c["gt_add_out"], rtol=2 * torch.finfo(x.dtype).eps, atol=1e-6)
        # the rms_norm.py kernel convention (weight in fp32, one rounding) differs by at most one rounding
        out2, _ = oracle.rms_norm(x, w, eps)
        torch.testing.assert_close(out2, c["gt_rms"], rtol=2 * torch.finfo(x.dtype).eps, atol=1e-6)


def test_rotary_ground_truth(golden_dir):
    for c in _load(golden_dir, "rotary.pt"):
        q, k = oracle.apply_rotary_pos_emb(c["q"], c["k"], c["cos"], c["sin"])
        assert torch.equal(q, c["gt_q"]) and torch.equal(k, c["gt_k"])


def test_fill_kv_cache_ground_truth(golden_dir):
    for c in _load(golden_dir, "fill_kv_cache.pt"):
        kc, vc = oracle.fill_kv_cache(c["k_states"], c["v_states"], c["k_caches"], c["v_caches"], c["seq_lens"],
                                      c["history_lens"], c["block_offsets"])
        assert torch.equal(kc, c["gt_k"]) and torch.equal(vc, c["gt_v"])


def _selection_priorities(select, priority, E):
    """Priority of every selected (expert, token) pair, sorted per expert: equal for any valid tie order."""
    cap = select.numel() // E
    sel = select.view(E, cap)
    return torch.stack([priority[sel[e], e].sort(descending=True)[0] for e in range(E)])


def test_gshard_topk_gating_ground_truth(golden_dir):
    for c in _load(golden_dir, "topk_gating.pt"):
        E = c["logits"].size(1)
        l_aux, ec, w, sel, prio = oracle.topk_gating(c["logits"], c["k"], c["capacity_factor"], c["min_capacity"])
        torch.testing.assert_close(l_aux, c["l_aux"], rtol=1e-6, atol=1e-7)
        assert torch.equal(ec, c["ec_idx"])
        torch.testing.assert_close(w, c["weights"], rtol=1e-6, atol=1e-8)
        assert sel.shape == c["select"].shape
        # torch.topk leaves the order among equal priorities open: compare what was selected, not where
        assert torch.equal(_selection_priorities(sel, prio, E), _selection_priorities(c["select"], prio, E))


# ---- third-party pins for the two operators that the reference project does not contain ------------------
def _same_routing(ids, w, case, tol=2e-6):
    """ids as sets per token (the third-party router returns them unsorted), weights matched by id."""
    ref_ids, ref_w = case["ids"].long(), case["weights"]
    a, ai = torch.sort(ids.long(), dim=-1)
    b, bi = torch.sort(ref_ids, dim=-1)
    assert torch.equal(a, b)
    torch.testing.assert_close(w.gather(1, ai), ref_w.gather(1, bi), rtol=tol, atol=tol)


def test_grouped_gating_matches_transformers_deepseek_v3_router(golden_dir):
    """Group-limited sigmoid routing against the output of transformers' DeepseekV3MoE.route_tokens_to_experts
    (executed by tests/golden/make_golden_third_party.py).  That router fills masked groups with 0 instead of
    -inf, which selects differently only when a biased score is <= 0; the fixtures' biases keep them positive.
    Tokens whose float64 decision margin is below fp32 noise are excluded (two sigmoid implementations may
    order them differently); the fixtures have none or a handful."""
    for case in _load(golden_dir, "grouped_gating_hf.pt"):
        ids, w = oracle.grouped_topk_gating(case["logits"], case["bias"], case["top_k"], case["n_group"],
                                            case["topk_group"], case["scale"], case["renormalize"], "sigmoid")
        keep = oracle.gating_margins(case["logits"], case["bias"], case["top_k"], case["n_group"],
                                     case["topk_group"]) > 1e-6
        assert keep.float().mean() > 0.98
        sub = {"ids": case["ids"][keep], "weights": case["weights"][keep]}
        _same_routing(ids[keep], w[keep], sub)


def test_moe_align_matches_vllm_documented_example(golden_dir):
    """The worked example in the docstring of vLLM's moe_align_block_size (experts numbered 1..4): same slot
    order inside an expert, same sentinel (numel), same per-expert padding to a block."""
    d = _load(golden_dir, "moe_align_vllm_doc.pt")
    ids, block, want = d["topk_ids"], d["block_size"], d["token_ids"]
    s, e, n, _ = oracle.moe_align_block_size(ids, block, int(ids.max()) + 1)
    assert int(n) == want.numel()
    assert torch.equal(s[:want.numel()], want)
    assert e[:want.numel() // block].tolist() == [1, 2, 3, 4]
