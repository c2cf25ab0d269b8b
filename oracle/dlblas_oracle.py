"""CPU oracle for the dlBLAS hot-path operators.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch on the CPU, the ground-truth code that the
reference's own tests use for each operator (citations below are paths inside
the reference project, DeepLink-org/DLCompiler).  It is the checker for the
CUDA kernels and the timed CPU baseline of the benchmark; nothing in the
shipped package imports it and it must never be used as a compute path.

Parity status
  pinned   silu_and_mul, fused_moe (launcher and end-to-end), varlen prefill
           attention, paged decode attention, paged prefill with history,
           rms_norm / add_rms_norm, rotary embedding, fill_kv_cache, GShard
           topk_gating: checked against fixtures produced by executing the
           reference tests' (for topk_gating: the reference benchmark's) own
           ground-truth functions (tests/golden/make_golden.py, tests/golden/*.pt).
           The sliding-window and soft-cap forms of the paged prefill and the
           topk_gating gradients have no reference fixture; they are tied to the
           pinned functions by tests/test_oracle_props.py and by autograd.
  THIRD-PARTY PINNED  grouped_topk_gating (group-limited sigmoid routing) and
           moe_align_block_size: the reference project contains neither.  They restate
           the published algorithms and are checked against other implementations of
           them: the routing against the output of transformers 5.5.0
           DeepseekV3MoE.route_tokens_to_experts executed on seeded inputs
           (tests/golden/grouped_gating_hf.pt), the block-padded sort against the worked
           example in the docstring of vLLM 0.22's moe_align_block_size
           (tests/golden/moe_align_vllm_doc.pt); both fixtures are produced by
           tests/golden/make_golden_third_party.py.  Against the REFERENCE these two
           stay "parity unpinned": it has nothing to compare with.
           The LSE output of prefill is pinned only through its formula
           (python/dlBLAS/dlblas/kernels/flash_attention.py:152-155).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# silu_and_mul
# --------------------------------------------------------------------------------------
def silu_and_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """Test ground truth, python/dlBLAS/tests/kernels/test_activation.py:22-25:
    silu on the first half times the second half, evaluated in the input dtype."""
    n = gate_up.size(-1) // 2
    gate, up = gate_up[..., :n], gate_up[..., n:]
    return F.silu(gate) * up


def silu_and_mul_fp32(gate_up: torch.Tensor) -> torch.Tensor:
    """Kernel-faithful form: fp32 math, one rounding on store
    (python/dlBLAS/dlblas/kernels/activation.py:73-85; same as the swiglu ground truth of
    test/ascend/passed_tests/test_swiglu.py:31-35)."""
    n = gate_up.size(-1) // 2
    g = gate_up[..., :n].float()
    u = gate_up[..., n:].float()
    return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)


# --------------------------------------------------------------------------------------
# routers
# --------------------------------------------------------------------------------------
def _stable_topk(scores: torch.Tensor, k: int):
    """Largest k along the last dim, ties to the LOWER index, descending order.
    (torch.topk on CPU does not guarantee the tie order, a stable descending sort does.)"""
    vals, idx = torch.sort(scores, dim=-1, descending=True, stable=True)
    return vals[..., :k], idx[..., :k]


def fma32(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """Correctly rounded fp32 fused multiply-add a*b+c (one rounding), as `fmaf` / the GPU's FFMA
    compute it.  The product of two fp32 numbers is exact in fp64; the fp64 sum is then rounded
    TO ODD (Knuth's two-sum gives the exact error of the addition, which supplies the sticky bit),
    so that the final rounding to fp32 cannot double-round.  Finite, non-overflowing operands only.
    """
    f64 = torch.float64
    p = a.to(f64) * b.to(f64)
    c64 = c.to(f64).expand_as(p)
    s = p + c64
    bb = s - p
    err = (p - (s - bb)) + (c64 - bb)                 # exact: p + c64 == s + err
    bits = s.contiguous().view(torch.int64)
    inexact_even = (err != 0) & ((bits & 1) == 0)
    grows = (err > 0) == (s > 0)                      # the exact sum lies beyond s, away from zero
    odd = torch.where(grows, bits | 1, bits - 1)      # truncate toward zero, then set the sticky bit
    bits = torch.where(inexact_even, odd, bits)
    return bits.view(f64).to(torch.float32)


# 2^r on [-0.5, 0.5], degree 5 with the constant term fixed at 1 (relative error 1e-7); highest first
_EXP2_COEF = (1.3287431793287396e-03, 9.671507403254509e-03, 5.550655722618103e-02,
              2.4022242426872253e-01, 6.931470632553101e-01, 1.0)
_NEG_LOG2E_HI = -1.4426950216293335          # fp32 nearest to -log2(e)
_NEG_LOG2E_LO = -1.925963033500011e-08           # -log2(e) - _NEG_LOG2E_HI, to fp32
_RINT_MAGIC = 12582912.0                     # 1.5 * 2^23: adding it rounds to an integer
_RCP_MAGIC = 0x7EF311C7                      # bits(1/d) ~ _RCP_MAGIC - bits(d)


def sigmoid_spec(x: torch.Tensor) -> torch.Tensor:
    """sigmoid as a fixed sequence of correctly-rounded fp32 operations (fused multiply-add, add,
    sub, integer add/sub on the bit patterns; no division).  The CUDA router evaluates exactly this
    sequence, so both sides produce bit-identical scores and near-ties cannot flip an expert id.
    Accurate to about 3e-7 relative:
        xc = clamp(x, -87, 86);  z = fma(xc, -log2e, M);  n = z - M           (M = 1.5 * 2^23)
        r = fma(xc, -log2e_lo, fma(xc, -log2e_hi, -n))                          (|r| <= 0.5)
        p = Horner_fma(r);  e = p * 2^n  (n added to the exponent bits);  d = 1 + e
        y = bits^-1(0x7EF311C7 - bits(d));  three times  y = fma(y, fma(-d, y, 1), y);  sigmoid = y
    """
    f = torch.float32
    c = lambda v: torch.tensor(v, dtype=torch.float64).to(f)          # nearest fp32 constant
    xc = torch.clamp(x.to(f), -87.0, 86.0)
    z = fma32(xc, c(_NEG_LOG2E_HI), c(_RINT_MAGIC))
    n = z - c(_RINT_MAGIC)
    r = fma32(xc, c(_NEG_LOG2E_HI), -n)
    r = fma32(xc, c(_NEG_LOG2E_LO), r)
    p = c(_EXP2_COEF[0]).expand_as(r)
    for coef in _EXP2_COEF[1:]:
        p = fma32(p, r, c(coef))
    e = (p.contiguous().view(torch.int32) + (z.contiguous().view(torch.int32) << 23)).view(f)
    d = 1.0 + e
    y = (_RCP_MAGIC - d.contiguous().view(torch.int32)).view(f)       # 5 % first guess of 1/d from the bits
    for _ in range(3):                                                # Newton: error 5e-2 -> 2.5e-3 -> 6e-6 -> rounding
        y = fma32(y, fma32(-d, y, c(1.0)), y)
    return y


def grouped_topk_gating(logits: torch.Tensor, bias: torch.Tensor | None, top_k: int, n_group: int = 1,
                        topk_group: int = 1, routed_scaling_factor: float = 1.0, renormalize: bool = True,
                        scoring_func: str = "sigmoid"):
    """Group-limited top-k routing (absent from the reference; pinned to the transformers DeepSeek-V3 router).

    Definition: scores = sigmoid_spec(logits) or softmax(logits) in fp32; choice = scores + bias
    (for softmax without bias the selection runs on the logits, which order identically);
    group score = sum of the 2 largest `choice` in each of the n_group equal groups; keep the
    topk_group best groups (ties: lower group index); experts of other groups get -inf;
    select top_k experts by `choice` (ties: lower expert index, output sorted by descending
    `choice`); weights = scores[ids], / (sum + 1e-20) if renormalize, * routed_scaling_factor.
    Returns (ids int32 [T, k], weights fp32 [T, k]).
    """
    logits = logits.float()
    T, E = logits.shape
    scores = sigmoid_spec(logits) if scoring_func == "sigmoid" else torch.softmax(logits, dim=-1)
    if bias is not None:
        choice = scores + bias.float().unsqueeze(0)
    elif scoring_func == "softmax":
        choice = logits.clone()      # softmax is monotone: select on the logits, free of exp() rounding
    else:
        choice = scores.clone()
    if n_group > 1:
        grp = choice.view(T, n_group, E // n_group)
        g_scores = _stable_topk(grp, 2)[0].sum(dim=-1)                      # [T, n_group]
        _, g_idx = _stable_topk(g_scores, topk_group)
        g_mask = torch.zeros_like(g_scores, dtype=torch.bool)
        g_mask.scatter_(1, g_idx, True)
        e_mask = g_mask.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E)
        choice = choice.masked_fill(~e_mask, float("-inf"))
    _, ids = _stable_topk(choice, top_k)
    w = scores.gather(1, ids)
    if renormalize:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    w = w * routed_scaling_factor
    return ids.to(torch.int32), w


def gating_margins(logits: torch.Tensor, bias: torch.Tensor | None, top_k: int, n_group: int, topk_group: int):
    """float64 decision margins of grouped sigmoid routing, per token.

    Returns the smallest gap, over the three decision layers (which groups are kept, which
    experts are selected, and the order of the selected experts), between two quantities
    whose comparison decides an output id.  If the minimum over all tokens is far above
    fp32 rounding noise (~1e-7), every correct implementation must return the same ids.
    """
    x = logits.double()
    T, E = x.shape
    s = torch.sigmoid(x)
    c = s + (bias.double().unsqueeze(0) if bias is not None else 0.0)
    margins = []
    if n_group > 1:
        grp = c.view(T, n_group, E // n_group)
        gs = torch.sort(grp, dim=-1, descending=True)[0][..., :2].sum(-1)
        gsort = torch.sort(gs, dim=-1, descending=True)[0]
        if topk_group < n_group:
            margins.append(gsort[:, topk_group - 1] - gsort[:, topk_group])
        gidx = torch.sort(gs, dim=-1, descending=True, stable=True)[1][:, :topk_group]
        gm = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, gidx, True)
        em = gm.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E)
        c = c.masked_fill(~em, float("-inf"))
    cs = torch.sort(c, dim=-1, descending=True)[0]
    gaps = cs[:, :top_k] - cs[:, 1:top_k + 1]
    gaps = torch.where(torch.isfinite(gaps), gaps, torch.full_like(gaps, float("inf")))
    margins.append(gaps.min(dim=-1)[0])
    return torch.stack(margins, 0).min(dim=0)[0]


def softmax_topk(router_logits: torch.Tensor, top_k: int, renormalize: bool = False):
    """Router of python/dlBLAS/tests/kernels/test_fused_moe.py:207-218: softmax in fp32, then top-k."""
    ids, w = grouped_topk_gating(router_logits, None, top_k, 1, 1, 1.0, renormalize, "softmax")
    return w, ids


# --------------------------------------------------------------------------------------
# moe_align_block_size
# --------------------------------------------------------------------------------------
def moe_align_block_size(topk_ids: torch.Tensor, block: int, num_experts: int):
    """Block-padded counting sort of the slots by expert (absent from the reference; pinned to vLLM's documented example).

    Conventions fixed here: sorted_token_ids has numel + num_experts*(block-1) entries rounded
    up to a multiple of `block`, filled with the sentinel `numel`; within an expert the slots
    are in ascending index order; expert_ids has capacity/block entries, -1 when unused; ids
    outside [0, num_experts) are dropped.  The reference's equivalent is argsort plus
    per-expert [start, end) ranges (python/dlBLAS/dlblas/kernels/fused_moe.py:314-320,
    267-293); `start_end_from_align` converts to that form.
    Returns (sorted_token_ids, expert_ids, num_tokens_post_padded, block_start) as int32.
    """
    flat = topk_ids.reshape(-1).to(torch.int64)
    numel = flat.numel()
    cap = numel + num_experts * (block - 1)
    cap = (cap + block - 1) // block * block
    sorted_ids = torch.full((cap,), numel, dtype=torch.int32)
    expert_ids = torch.full((max(cap // block, 1),), -1, dtype=torch.int32)
    block_start = torch.zeros(num_experts + 1, dtype=torch.int32)
    pos = 0
    blk = 0
    for e in range(num_experts):
        block_start[e] = blk
        slots = torch.nonzero(flat == e).flatten()
        n = slots.numel()
        sorted_ids[pos:pos + n] = slots.to(torch.int32)
        nb = (n + block - 1) // block
        expert_ids[blk:blk + nb] = e
        blk += nb
        pos += nb * block
    block_start[num_experts] = blk
    return sorted_ids, expert_ids, torch.tensor([pos], dtype=torch.int32), block_start


def start_end_from_counts(topk_ids: torch.Tensor, num_experts: int):
    """exp_start / exp_end of python/dlBLAS/dlblas/kernels/fused_moe.py:267-293 (docstring formula)."""
    cnt = F.one_hot(topk_ids.flatten().to(torch.int64), num_classes=num_experts).sum(0)
    end = cnt.cumsum(0)
    return end - cnt, end


# --------------------------------------------------------------------------------------
# fused_moe
# --------------------------------------------------------------------------------------
def fused_moe_launcher_gt(A, B, top_k, topk_idx, weights=None):
    """Launcher ground truth, python/dlBLAS/tests/kernels/test_fused_moe.py:98-112."""
    M, N, E = A.size(0), B.size(1), B.size(0)
    C = B.new_zeros(M, top_k, N)
    for eid in range(E):
        token_idx, k_idx = torch.where(topk_idx == eid)
        if len(token_idx) == 0:
            continue
        C[token_idx, k_idx] = A[token_idx] @ B[eid].t()
    if weights is not None:
        C = C * weights[..., None]
    return C.flatten(0, 1)


def fused_moe(hidden_states, w1, w2, topk_weights, topk_ids, renormalize=False):
    """End-to-end ground truth, python/dlBLAS/tests/kernels/test_fused_moe.py:148-151, 227-244:
    per expert, down(silu(gate(x)) * up(x)) * weight, index_add into the output."""
    if renormalize:
        topk_weights = topk_weights / topk_weights.sum(dim=-1, keepdim=True)
    output = hidden_states.new_zeros(hidden_states.size(0), w2.size(1))
    for eid in range(w1.size(0)):
        token_idx, k_idx = torch.where(topk_ids == eid)
        if token_idx.numel() == 0:
            continue
        gate_proj, up_proj = w1[eid].chunk(2, dim=0)
        x = hidden_states[token_idx]
        tmp = F.linear(F.silu(F.linear(x, gate_proj)) * F.linear(x, up_proj), w2[eid])
        tmp = tmp * topk_weights[token_idx, k_idx, None]
        output.index_add_(0, token_idx, tmp.to(output.dtype))
    return output


def fused_moe_rounding_faithful(hidden_states, w1, w2, topk_weights, topk_ids, renormalize=False):
    """Same result as the reference *kernel path* including its rounding points
    (python/dlBLAS/dlblas/kernels/fused_moe.py:351-352, 162-166, 375): GEMM outputs rounded to
    the activation dtype, silu and product rounded separately, weight applied to the fp32
    accumulator before the cast, top-k sum accumulated in fp32 and rounded once."""
    dt = hidden_states.dtype
    if renormalize:
        topk_weights = topk_weights / topk_weights.sum(dim=-1, keepdim=True)
    M, topk = topk_ids.shape
    partial = torch.zeros(M, topk, w2.size(1), dtype=dt)
    for eid in range(w1.size(0)):
        token_idx, k_idx = torch.where(topk_ids == eid)
        if token_idx.numel() == 0:
            continue
        x = hidden_states[token_idx].float()
        gu = (x @ w1[eid].float().t()).to(dt)
        gate, up = gu.chunk(2, dim=-1)
        act = F.silu(gate) * up
        y = act.float() @ w2[eid].float().t()
        y = (y * topk_weights[token_idx, k_idx, None].float()).to(dt)
        partial[token_idx, k_idx] = y
    return partial.float().sum(dim=1).to(dt)


# --------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------
def _torch_att(xq, xk, xv, seqlen, num_head, head_dim):
    """Single-sequence causal attention, python/dlBLAS/tests/kernels/test_prefill_attention.py:11-36
    (same-count heads; additive -1e8 mask, softmax in fp32, P cast back before P.V)."""
    xq = xq.view(1, seqlen, num_head, head_dim).transpose(1, 2)
    keys = xk.view(1, seqlen, num_head, head_dim).transpose(1, 2)
    values = xv.view(1, seqlen, num_head, head_dim).transpose(1, 2)
    mask = torch.tril(torch.ones(seqlen, seqlen), diagonal=0).unsqueeze(0).unsqueeze(0)
    mask[mask == 0.0] = -100000000.0
    scores = torch.matmul(xq, keys.transpose(2, 3)) / math.sqrt(head_dim)
    scores = F.softmax(scores.float() + mask, dim=-1).type_as(xq)
    return torch.matmul(scores, values).transpose(1, 2).contiguous().reshape(-1, num_head, head_dim)


def context_attention(q, k, v, b_start_loc, b_seq_len, causal=True, sm_scale=None, return_lse=False,
                      block_rows=1024):
    """Varlen causal GQA prefill: the per-sequence loop of test_prefill_attention.py:68-77 with the
    kv heads repeated for grouped queries (prefill_attention.py:159), evaluated in query-row
    blocks to bound memory.  Scores are formed in fp32 from the 16-bit inputs (as the kernels
    do); P is cast to the value dtype before P.V.  LSE = max*scale + log(sum) in natural log
    (flash_attention.py:152-155), shape [Hq, total]."""
    total, hq, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    out = torch.zeros_like(q)
    lse = torch.full((hq, total), float("-inf"), dtype=torch.float32)
    for s0, n in zip(b_start_loc.tolist(), b_seq_len.tolist()):
        if n == 0:
            continue
        qs = q[s0:s0 + n].transpose(0, 1).float()                    # [hq, n, d]
        ks = k[s0:s0 + n].transpose(0, 1).repeat_interleave(group, 0).float()
        vs = v[s0:s0 + n].transpose(0, 1).repeat_interleave(group, 0)
        for r0 in range(0, n, block_rows):
            r1 = min(n, r0 + block_rows)
            kend = r1 if causal else n
            sc = torch.matmul(qs[:, r0:r1], ks[:, :kend].transpose(1, 2)) * sm_scale
            if causal:
                qi = torch.arange(r0, r1).unsqueeze(1)
                kj = torch.arange(0, kend).unsqueeze(0)
                sc = sc.masked_fill((kj > qi).unsqueeze(0), float("-inf"))
            m = sc.max(dim=-1, keepdim=True)[0]
            p = torch.exp(sc - m)
            l = p.sum(dim=-1, keepdim=True)
            pn = (p / l).to(v.dtype)
            o = torch.matmul(pn.float(), vs[:, :kend].float())
            out[s0 + r0:s0 + r1] = o.transpose(0, 1).to(q.dtype)
            lse[:, s0 + r0:s0 + r1] = (m + torch.log(l)).squeeze(-1)
    return (out, lse) if return_lse else out


def make_blocked_cache(batched_k, batched_v, kv_lens, block_offsets, block_size):
    """Scatter dense [B, L, H, D] keys/values into a paged cache [pages, block, H, D]
    (python/dlBLAS/tests/kernels/test_paged_attention.py:28-58)."""
    num_pages = int(block_offsets.max().item()) + 1
    hk, d, dv = batched_k.shape[2], batched_k.shape[3], batched_v.shape[3]
    blocked_k = batched_k.new_zeros(num_pages, block_size, hk, d)
    blocked_v = batched_v.new_zeros(num_pages, block_size, hk, dv)
    for b, offs in enumerate(block_offsets):
        n = int(kv_lens[b])
        for i, st in enumerate(range(0, n, block_size)):
            size = min(block_size, n - st)
            blocked_k[offs[i], :size] = batched_k[b, st:st + size]
            blocked_v[offs[i], :size] = batched_v[b, st:st + size]
    return blocked_k, blocked_v


def paged_decode_attention(q, k_cache, v_cache, block_offsets, kv_seqlens, sm_scale=None, window_size=None,
                           logit_softcapping=None):
    """Decode ground truth: `_naive_attention` of test_paged_attention.py:61-84 specialised to one
    query token per sequence, reading K/V through the block table.  q [B, Hq, D]; scores in
    fp32, softmax in fp32, P cast to the value dtype before P.V; optional sliding window
    (the query at position ctx - 1 sees keys ctx - 1 - window .. ctx - 1, paged_attention.py:163-165,192-194
    with history_len = ctx - 1) and tanh soft-cap as in paged_attention.py:175-200."""
    B, hq, d = q.shape
    page = k_cache.shape[1]
    hkv = k_cache.shape[2]
    group = hq // hkv
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    out = torch.zeros(B, hq, v_cache.shape[-1], dtype=q.dtype)
    for b in range(B):
        n = int(kv_seqlens[b])
        if n == 0:
            continue
        npg = (n + page - 1) // page
        pages = block_offsets[b, :npg].to(torch.int64)
        ks = k_cache[pages].reshape(npg * page, hkv, -1)[:n]
        vs = v_cache[pages].reshape(npg * page, hkv, -1)[:n]
        lo = max(0, n - 1 - window_size) if (window_size is not None and window_size > 0) else 0
        ks, vs = ks[lo:], vs[lo:]
        kf = ks.transpose(0, 1).repeat_interleave(group, 0).float()      # [hq, n, d]
        vf = vs.transpose(0, 1).repeat_interleave(group, 0)
        sc = torch.matmul(q[b].float().unsqueeze(1), kf.transpose(1, 2)) * sm_scale   # [hq, 1, n]
        if logit_softcapping is not None and logit_softcapping > 0:
            sc = logit_softcapping * torch.tanh(sc / logit_softcapping)
        p = torch.softmax(sc, dim=-1, dtype=torch.float32).to(vf.dtype)
        out[b] = torch.matmul(p.float(), vf.float()).squeeze(1).to(q.dtype)
    return out


def paged_prefill_attention(q, k_cache, v_cache, block_offsets, q_start_loc, q_seqlens, kv_seqlens, sm_scale=None,
                            window_size=None, logit_softcapping=None):
    """Prefill over a paged cache that already holds `kv_seqlens - q_seqlens` earlier tokens per sequence
    (ground truth of test_paged_attention.py:61-84 with the causal mask of :14-25 shifted by the history
    length, as the kernel does at paged_attention.py:362).  q [total_q, Hq, D] packed by sequence; query i
    of a sequence sits at position history + i and sees keys 0 .. history + i; with a window only keys
    >= max(history + i - window, 0) (paged_attention.py:421-424,447); optional tanh soft-cap of the scaled
    scores (paged_attention.py:441-444).  Scores and softmax in fp32, P cast to the value dtype before P.V."""
    total, hq, d = q.shape
    page = k_cache.shape[1]
    hkv = k_cache.shape[2]
    group = hq // hkv
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    out = torch.zeros(total, hq, v_cache.shape[-1], dtype=q.dtype)
    for b in range(len(q_seqlens)):
        nq, n = int(q_seqlens[b]), int(kv_seqlens[b])
        if nq == 0:
            continue
        s0 = int(q_start_loc[b])
        hist = n - nq
        npg = (n + page - 1) // page
        pages = block_offsets[b, :npg].to(torch.int64)
        ks = k_cache[pages].reshape(npg * page, hkv, -1)[:n]
        vs = v_cache[pages].reshape(npg * page, hkv, -1)[:n]
        kf = ks.transpose(0, 1).repeat_interleave(group, 0).float()      # [hq, n, d]
        vf = vs.transpose(0, 1).repeat_interleave(group, 0)
        qf = q[s0:s0 + nq].transpose(0, 1).float()                        # [hq, nq, d]
        sc = torch.matmul(qf, kf.transpose(1, 2)) * sm_scale              # [hq, nq, n]
        if logit_softcapping is not None and logit_softcapping > 0:
            sc = logit_softcapping * torch.tanh(sc / logit_softcapping)
        pos = torch.arange(nq)[:, None] + hist
        keys = torch.arange(n)[None, :]
        hidden = keys > pos
        if window_size is not None and window_size > 0:
            hidden = hidden | (keys < (pos - window_size).clamp(min=0))
        sc = sc.masked_fill(hidden, float("-inf"))
        p = torch.softmax(sc, dim=-1, dtype=torch.float32).to(vf.dtype)
        out[s0:s0 + nq] = torch.matmul(p.float(), vf.float()).transpose(0, 1).to(q.dtype)
    return out


# --------------------------------------------------------------------------------------
# rms_norm, rotary embedding, fill_kv_cache (the steps next to the hot path)
# --------------------------------------------------------------------------------------
def rms_norm_test_gt(x, weight, eps):
    """Test ground truth, python/dlBLAS/tests/kernels/test_rms_norm.py:26-31: normalise in fp32, cast,
    then multiply by the weight in the storage dtype."""
    xf = x.to(torch.float32)
    variance = xf.pow(2).mean(-1, keepdim=True)
    xf = xf * torch.rsqrt(variance + eps)
    return weight * xf.to(x.dtype)


def rms_norm(x, weight, eps=1e-6, residual=None, weight_after_cast=False):
    """Kernel-faithful form.  new_x = x + residual in the storage dtype
    (python/dlBLAS/dlblas/kernels/rms_norm.py:68-70); weight_after_cast=False multiplies by the weight in
    fp32 and rounds once (rms_norm.py:8-16), True rounds first and multiplies in the storage dtype
    (python/dlBLAS/dlblas/kernels/add_rms_norm.py:33-38).  Returns (out, new_x)."""
    new_x = x + residual if residual is not None else x
    xf = new_x.to(torch.float32)
    var = (xf * xf).sum(-1, keepdim=True) * (1.0 / x.size(-1))
    normed = xf * torch.rsqrt(var + eps)
    if weight_after_cast:
        out = normed.to(x.dtype) * weight
    else:
        out = (weight.to(torch.float32) * normed).to(x.dtype)
    return out, new_x


def _rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin):
    """Test ground truth, python/dlBLAS/tests/kernels/test_apply_rotary.py:80-86:
    x * cos + rotate_half(x) * sin in the tensors' dtype (cos/sin broadcast over heads)."""
    cos = cos.reshape(q.size(0), 1, -1).to(q.dtype)
    sin = sin.reshape(q.size(0), 1, -1).to(q.dtype)
    return q * cos + _rotate_half(q) * sin, k * cos + _rotate_half(k) * sin


def fill_kv_cache(k_states, v_states, k_caches, v_caches, seq_lens, history_lens, block_offsets):
    """Test ground truth, python/dlBLAS/tests/kernels/test_fill_kv_cache.py:97-137: new token i of
    sequence b goes to slot (history + i) % page of page block_offsets[b, (history + i) // page]."""
    page = k_caches.size(1)
    kc, vc = k_caches.clone(), v_caches.clone()
    start = 0
    for b, (n, h) in enumerate(zip(seq_lens, history_lens)):
        for i in range(n):
            pos = h + i
            pg = int(block_offsets[b, pos // page])
            kc[pg, pos % page] = k_states[start + i]
            vc[pg, pos % page] = v_states[start + i]
        start += n
    return kc, vc


# --------------------------------------------------------------------------------------
# GShard-style top-k gating with capacity (the reference's `topk_gating` op)
# --------------------------------------------------------------------------------------
def topk_gating(logits, k, capacity_factor=1.0, min_capacity=2):
    """Restatement of python/dlBLAS/benchmarks/topk_gating.py:132-206 (`fused_topkgating_opt`, the torch
    reference the dlBLAS benchmark checks its kernels against), with the two points that code leaves to
    `torch.topk`'s unspecified tie order made explicit: equal gate values go to the lower expert index,
    and `expert_select_token_idx` lists each expert's kept tokens in queue order (choice-major, then
    token), padding unfilled capacity with the lowest-numbered tokens that were not kept.
    Returns (l_aux, token_rearranged_ec_idx int32 [k*s], token_exp_weights [k*s],
    expert_select_token_idx int64 [e*c], priority [s, e]) -- `priority` (k - choice for kept choices, else 0)
    is what the reference feeds to torch.topk and lets tests compare selections up to ties."""
    x = logits.float()
    S, E = x.shape
    gates = F.softmax(x, dim=1)
    capacity = int(torch.ceil((S / E) * torch.tensor(capacity_factor * k)).to(torch.int64))
    capacity = max(capacity, int(min_capacity))
    _, idx = _stable_topk(x, k)                                   # softmax is monotone: rank on the logits
    idx_km = idx.t().reshape(-1)                                  # [k*s], choice-major
    masks = F.one_hot(idx_km, num_classes=E)
    locations = torch.cumsum(masks, dim=0) - 1
    masks = masks.reshape(k, S, E)
    locations = locations.reshape(k, S, E)
    me = gates.mean(dim=0)
    ce = masks[0].float().mean(dim=0)
    l_aux = torch.mean(me * ce) * E * E
    masks = masks * torch.lt(locations, capacity)
    locations_s = torch.sum(locations * masks, dim=2)
    gate_s, indices_s = torch.max(gates * masks.float(), dim=2)
    indices_s = torch.where(gate_s > 0, indices_s, torch.zeros_like(indices_s))
    denom = torch.clamp(gate_s.sum(dim=0), min=torch.finfo(torch.float32).eps)
    gate_s = gate_s / denom
    ec_idx = (indices_s.int() * capacity + locations_s.int()).reshape(-1)
    priority = (masks * torch.arange(k, 0, -1).reshape(k, 1, 1)).sum(dim=0)          # [s, e]
    select = torch.zeros(E, capacity, dtype=torch.int64)
    for e in range(E):
        order = torch.nonzero(idx_km == e).flatten()[:capacity] % S                  # queue order
        kept = order.tolist()
        fill = [t for t in range(S) if t not in set(kept)][:capacity - len(kept)]
        select[e] = torch.tensor(kept + fill, dtype=torch.int64)
    return l_aux, ec_idx, gate_s.reshape(-1), select.reshape(-1), priority


def topk_gating_backward(logits, k, grad_l_aux=1.0):
    """d l_aux / d logits by autograd through the same expression (me depends on the logits, ce does not)."""
    x = logits.float().clone().requires_grad_(True)
    S, E = x.shape
    gates = F.softmax(x, dim=1)
    _, idx = _stable_topk(x.detach(), k)
    ce = F.one_hot(idx[:, 0], num_classes=E).float().mean(dim=0)
    l_aux = torch.mean(gates.mean(dim=0) * ce) * E * E
    l_aux.backward(torch.tensor(grad_l_aux))
    return x.grad


def topk_gating_backward_weights(logits, k, capacity_factor=1.0, min_capacity=2, grad_l_aux=1.0, grad_weights=None):
    """d (grad_l_aux * l_aux + sum(grad_weights * token_exp_weights)) / d logits by autograd through the
    forward expression of `topk_gating` above, in fp64 (the routing decisions -- ids, queue positions,
    capacity drops -- do not depend on the logits differentiably).  This is the gradient the reference's
    `higher_precision` backward (python/dlBLAS/dlblas/kernels/topk_gating.py:145-256) sets out to compute."""
    x = logits.double().clone().requires_grad_(True)
    S, E = x.shape
    gates = F.softmax(x, dim=1)
    capacity = int(torch.ceil((S / E) * torch.tensor(capacity_factor * k)).to(torch.int64))
    capacity = max(capacity, int(min_capacity))
    _, idx = _stable_topk(logits.float(), k)
    idx_km = idx.t().reshape(-1)
    masks = F.one_hot(idx_km, num_classes=E)
    locations = (torch.cumsum(masks, dim=0) - 1).reshape(k, S, E)
    masks = masks.reshape(k, S, E)
    ce = masks[0].double().mean(dim=0)
    l_aux = torch.mean(gates.mean(dim=0) * ce) * E * E
    masks = masks * torch.lt(locations, capacity)
    gate_s = (gates * masks.double()).sum(dim=2)                  # one non-zero term per (choice, token)
    denom = torch.clamp(gate_s.sum(dim=0), min=torch.finfo(torch.float32).eps)
    w = (gate_s / denom).reshape(-1)
    loss = grad_l_aux * l_aux
    if grad_weights is not None:
        loss = loss + (grad_weights.double() * w).sum()
    loss.backward()
    return x.grad.float()

