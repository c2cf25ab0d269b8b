"""GPU parity: varlen prefill attention (tcgen05) and paged flash-decode against the CPU oracle."""
import os

import pytest
import torch

from dlcompiler_b200 import context_attention_fwd, paged_attention_fwd
from dlcompiler_b200 import workloads as W
from oracle import dlblas_oracle as oracle

pytestmark = pytest.mark.gpu

# stated bound for bf16 attention outputs
RTOL = ATOL = 2e-2


def _run_prefill(dev, d, lse=False, causal=True):
    q, k, v = d["q"].to(dev), d["k"].to(dev), d["v"].to(dev)
    o = torch.full_like(q, float("nan"))
    l = torch.full((q.shape[1], q.shape[0]), float("nan"), device=dev) if lse else None
    context_attention_fwd(q, k, v, o, d["b_start_loc"].to(dev), d["b_seq_len"].to(dev), d["max_input_len"], lse=l,
                          causal=causal)
    return o.cpu(), (l.cpu() if lse else None)


def test_prefill_golden(cuda_device, golden_dir):
    for c in torch.load(os.path.join(golden_dir, "prefill_attention.pt"), weights_only=True):
        lens = c["lens"]
        start = [0]
        for n in lens[:-1]:
            start.append(start[-1] + n)
        d = {"q": c["q"], "k": c["k"], "v": c["v"], "b_start_loc": torch.tensor(start, dtype=torch.int32),
             "b_seq_len": torch.tensor(lens, dtype=torch.int32), "max_input_len": max(lens)}
        out, _ = _run_prefill(cuda_device, d)
        # reference test: atol=1e-2, rtol=0 for fp16 (test_prefill_attention.py:83)
        torch.testing.assert_close(out, c["gt"], atol=1e-2 if out.dtype == torch.float16 else 2e-2, rtol=0)


@pytest.mark.parametrize("lens,hq,hkv,dtype", [
    ([1], 4, 4, torch.bfloat16),
    ([63, 64, 65], 4, 2, torch.bfloat16),
    ([127, 128, 129, 1], 8, 2, torch.float16),
    ([512, 1024, 512, 1024], 6, 6, torch.float16),      # the reference test's lengths
    ([300, 0, 700], 8, 1, torch.bfloat16),               # an empty sequence in the batch
    ([2048], 32, 8, torch.bfloat16),
])
def test_prefill_shapes_with_lse(cuda_device, lens, hq, hkv, dtype):
    wl = W.PrefillWorkload(seq_lens=lens, hq=hq, hkv=hkv, dtype=dtype)
    d = wl.make()
    out, lse = _run_prefill(cuda_device, d, lse=True)
    ref, rlse = oracle.context_attention(d["q"], d["k"], d["v"], d["b_start_loc"], d["b_seq_len"], return_lse=True)
    torch.testing.assert_close(out.float(), ref.float(), rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(lse, rlse, rtol=1e-3, atol=1e-3)


def test_prefill_non_causal(cuda_device):
    wl = W.PrefillWorkload(seq_lens=[200, 77], hq=4, hkv=2)
    d = wl.make()
    out, _ = _run_prefill(cuda_device, d, causal=False)
    ref = oracle.context_attention(d["q"], d["k"], d["v"], d["b_start_loc"], d["b_seq_len"], causal=False)
    torch.testing.assert_close(out.float(), ref.float(), rtol=RTOL, atol=ATOL)


def test_prefill_config_full_groups_and_properties(cuda_device):
    """Full benchmark shape: for every sequence one whole (sequence, kv head) group, all 8192 rows of its four
    query heads, against the oracle; plus properties that hold at any size (causality, determinism)."""
    wl = W.PrefillWorkload()
    d = wl.make()
    out, lse = _run_prefill(cuda_device, d, lse=True)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    torch.set_num_threads(os.cpu_count() or 1)
    for b in range(wl.batch):
        s0, n = int(d["b_start_loc"][b]), int(d["b_seq_len"][b])
        kvh = (3 * b + 1) % wl.hkv
        heads = slice(4 * kvh, 4 * kvh + 4)
        ref, rlse = oracle.context_attention(d["q"][s0:s0 + n, heads], d["k"][s0:s0 + n, kvh:kvh + 1],
                                             d["v"][s0:s0 + n, kvh:kvh + 1], torch.tensor([0]), torch.tensor([n]),
                                             return_lse=True)
        torch.testing.assert_close(out[s0:s0 + n, heads].float(), ref.float(), rtol=RTOL, atol=ATOL)
        torch.testing.assert_close(lse[heads, s0:s0 + n], rlse, rtol=1e-3, atol=1e-3)
    # determinism: the same inputs give the same bits (catches a softmax warp racing ahead of the MMAs)
    for _ in range(2):
        again, _ = _run_prefill(cuda_device, d)
        assert torch.equal(again, out)
    # causality: changing the last 100 keys/values of a sequence leaves earlier rows bit-identical
    d2 = dict(d)
    d2["k"] = d["k"].clone()
    d2["v"] = d["v"].clone()
    d2["k"][8192 - 100:8192] = 0
    d2["v"][8192 - 100:8192] = 1
    out2, _ = _run_prefill(cuda_device, d2)
    assert torch.equal(out2[:8192 - 100], out[:8192 - 100])
    assert torch.equal(out2[8192:], out[8192:])


def _run_decode(dev, d, **kw):
    q = d["q"].to(dev)
    o = torch.full(q.shape[:-1] + (d["v_cache"].shape[-1],), float("nan"), dtype=q.dtype, device=dev)
    B = q.shape[0]
    paged_attention_fwd(q, d["k_cache"].to(dev), d["v_cache"].to(dev), o, d["block_table"].to(dev),
                        torch.arange(B, device=dev), torch.ones(B, dtype=torch.int64, device=dev),
                        d["kv_seqlens"].to(dev), 1, **kw)
    return o.cpu()


def test_decode_golden(cuda_device, golden_dir):
    for c in torch.load(os.path.join(golden_dir, "paged_decode.pt"), weights_only=True):
        d = {"q": c["q"], "k_cache": c["k_cache"], "v_cache": c["v_cache"], "block_table": c["block_offsets"],
             "kv_seqlens": c["kv_seqlens"]}
        out = _run_decode(cuda_device, d)
        # reference test: atol=1e-3, rtol=1e-5 for fp16 (test_paged_attention.py:286)
        tol = 1e-3 if out.dtype == torch.float16 else 8e-3
        torch.testing.assert_close(out, c["gt"], atol=tol, rtol=1e-5)


@pytest.mark.parametrize("batch,lo,hi,page,hq,hkv,D,dtype", [
    (1, 1, 1, 16, 4, 4, 64, torch.float16),
    (5, 1, 300, 16, 8, 2, 128, torch.bfloat16),
    (7, 50, 1500, 32, 32, 8, 128, torch.bfloat16),
    (4, 1000, 5000, 64, 32, 8, 128, torch.bfloat16),
    (3, 100, 900, 128, 16, 1, 64, torch.float16),        # 16 q heads on one kv head
    (2, 64, 640, 64, 40, 2, 128, torch.bfloat16),        # group of 20 > 16 rows: two head blocks
    (6, 0, 100, 16, 8, 8, 128, torch.bfloat16),          # may contain empty contexts
])
def test_decode_shapes(cuda_device, batch, lo, hi, page, hq, hkv, D, dtype):
    wl = W.DecodeWorkload(batch=batch, ctx_lo=lo, ctx_hi=hi, page=page, hq=hq, hkv=hkv, head_dim=D, dtype=dtype)
    d = wl.make()
    out = _run_decode(cuda_device, d)
    ref = oracle.paged_decode_attention(d["q"], d["k_cache"], d["v_cache"], d["block_table"], d["kv_seqlens"])
    torch.testing.assert_close(out.float(), ref.float(), rtol=RTOL, atol=ATOL)


def test_decode_window_softcap_int64_and_stale_cache(cuda_device):
    wl = W.DecodeWorkload(batch=6, ctx_lo=10, ctx_hi=3000, page=64, hq=8, hkv=2, head_dim=128)
    d = wl.make()
    d["block_table"] = d["block_table"].to(torch.int64)
    d["kv_seqlens"] = d["kv_seqlens"].to(torch.int64)
    for kw in ({"window_size": 333}, {"logit_softcapping": 5.0}, {"sm_scale": 0.03},
               {"window_size": 100, "logit_softcapping": 30.0}):
        out = _run_decode(cuda_device, d, **kw)
        ref = oracle.paged_decode_attention(d["q"], d["k_cache"], d["v_cache"], d["block_table"], d["kv_seqlens"],
                                            **kw)
        torch.testing.assert_close(out.float(), ref.float(), rtol=RTOL, atol=ATOL)
    # slots past the context length may hold anything, including NaN bit patterns
    base = _run_decode(cuda_device, d)
    dirty = dict(d)
    kc, vc = d["k_cache"].clone(), d["v_cache"].clone()
    for b in range(6):
        n = int(d["kv_seqlens"][b])
        pg = int(d["block_table"][b, (n - 1) // 64]) if n > 0 else None
        if pg is not None and n % 64:
            kc[pg, n % 64:] = float("nan")
            vc[pg, n % 64:] = float("nan")
    dirty["k_cache"], dirty["v_cache"] = kc, vc
    assert torch.equal(_run_decode(cuda_device, dirty), base)


def test_decode_config_all_sequences_and_properties(cuda_device):
    """Full benchmark shape (caches generated on the device): every sequence against the oracle."""
    wl = W.DecodeWorkload()
    d = wl.make(device=cuda_device)
    out = _run_decode(cuda_device, d)
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out, _run_decode(cuda_device, d))             # deterministic
    ctx = d["kv_seqlens"]
    for b in range(wl.batch):
        n = int(ctx[b])
        npg = (n + wl.page - 1) // wl.page
        pages = d["block_table"][b, :npg].long()
        kc = d["k_cache"][pages.to(cuda_device)].cpu()
        vc = d["v_cache"][pages.to(cuda_device)].cpu()
        table = torch.arange(npg, dtype=torch.int32).unsqueeze(0)
        ref = oracle.paged_decode_attention(d["q"][b:b + 1], kc, vc, table, ctx[b:b + 1])
        torch.testing.assert_close(out[b:b + 1].float(), ref.float(), rtol=RTOL, atol=ATOL)


# ------------------------------------------------------------------ head size 64 and the dense entry points
@pytest.mark.parametrize("lens,hq,hkv,dtype", [
    ([100, 257], 4, 2, torch.bfloat16),
    ([1024], 8, 8, torch.float16),
])
def test_prefill_head_size_64(cuda_device, lens, hq, hkv, dtype):
    wl = W.PrefillWorkload(seq_lens=lens, hq=hq, hkv=hkv, head_dim=64, dtype=dtype)
    d = wl.make()
    out, lse = _run_prefill(cuda_device, d, lse=True)
    ref, rlse = oracle.context_attention(d["q"], d["k"], d["v"], d["b_start_loc"], d["b_seq_len"], return_lse=True)
    torch.testing.assert_close(out.float(), ref.float(), rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(lse, rlse, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("head_dim", [96, 80, 13, 32, 48])
def test_prefill_other_head_sizes(cuda_device, head_dim):
    """The head sizes of the reference's own context-attention test (test_attention_kernels.py:136-160: 4 heads,
    lengths 8 and 12, sizes 128, 96, 80, 13; it only checks that the call runs) and of its paged test (48, 32),
    here checked against the oracle, with a longer ragged sequence added."""
    wl = W.PrefillWorkload(seq_lens=[8, 12, 150], hq=4, hkv=4, head_dim=head_dim, dtype=torch.float16)
    d = wl.make()
    out, lse = _run_prefill(cuda_device, d, lse=True)
    ref, rlse = oracle.context_attention(d["q"], d["k"], d["v"], d["b_start_loc"], d["b_seq_len"], return_lse=True)
    torch.testing.assert_close(out.float(), ref.float(), rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(lse, rlse, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("causal", [False, True])
def test_dense_flash_attention_bhmd(cuda_device, causal):
    """[B, H, M, D] layout of flash_attention.py:170-211 with grouped heads, LSE of :152-155."""
    from dlcompiler_b200 import flash_attention_fwd

    g = torch.Generator().manual_seed(21)
    B, H, Hk, M, D = 2, 4, 2, 300, 128
    q = torch.randn(B, H, M, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, Hk, M, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Hk, M, D, generator=g).to(torch.bfloat16)
    o, L = flash_attention_fwd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=causal, sm_scale=0.11)
    for b in range(B):
        ref, rl = oracle.context_attention(q[b].transpose(0, 1).contiguous(), k[b].transpose(0, 1).contiguous(),
                                           v[b].transpose(0, 1).contiguous(), torch.tensor([0]), torch.tensor([M]),
                                           causal=causal, sm_scale=0.11, return_lse=True)
        torch.testing.assert_close(o[b].cpu().transpose(0, 1).float(), ref.float(), rtol=RTOL, atol=ATOL)
        torch.testing.assert_close(L[b].cpu(), rl, rtol=1e-3, atol=1e-3)


def test_dense_flash_attention_v2_bshd(cuda_device):
    """[b, s, h, d] layout, d = 64, non-causal: the reference benchmark's configuration
    (benchmarks/flash_attention_v2.py:13-30 checks against scaled_dot_product_attention, atol 1e-2)."""
    import torch.nn.functional as F

    from dlcompiler_b200 import flash_attention_v2

    g = torch.Generator().manual_seed(22)
    b, s, h, d = 2, 777, 4, 64
    q, k, v = (torch.rand(b, s, h, d, generator=g).to(torch.float16) for _ in range(3))
    o = flash_attention_v2(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)).cpu()
    ref = F.scaled_dot_product_attention(q.transpose(1, 2).float(), k.transpose(1, 2).float(),
                                         v.transpose(1, 2).float()).transpose(1, 2)
    torch.testing.assert_close(o.float(), ref, atol=1e-2, rtol=0)


# ------------------------------------------------------------------ small pages and token-granular decode
@pytest.mark.parametrize("page", [1, 2, 4, 8])
def test_decode_small_pages(cuda_device, page):
    from dlcompiler_b200 import _lib

    wl = W.DecodeWorkload(batch=3, ctx_lo=5, ctx_hi=400, page=page, hq=8, hkv=2, head_dim=128)
    d = wl.make()
    dev = cuda_device
    q = d["q"].to(dev)
    o = torch.full_like(q, float("nan"))
    kc, vc, tb, ln = d["k_cache"].to(dev), d["v_cache"].to(dev), d["block_table"].to(dev), d["kv_seqlens"].to(dev)
    lib = _lib.load()
    chunk, splits = 256, (tb.size(1) * page + 255) // 256
    part = torch.empty(max(lib.dlb_paged_decode_workspace_floats(3, 8, 128, splits), 1), device=dev)
    rc = lib.dlb_paged_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), tb.data_ptr(), ln.data_ptr(),
                              part.data_ptr(), 3, 8, 2, 128, 128, page, kc.size(0), tb.size(1), q.stride(0), q.stride(1),
                              o.stride(0), o.stride(1), kc.stride(0), kc.stride(1), kc.stride(2), vc.stride(0),
                              vc.stride(1), vc.stride(2), tb.stride(0), 0, 0, chunk, splits, -1, 128 ** -0.5, -1.0,
                              _lib.DTYPE_BF16, _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "paged_decode")
    ref = oracle.paged_decode_attention(d["q"], d["k_cache"], d["v_cache"], d["block_table"], d["kv_seqlens"])
    torch.testing.assert_close(o.cpu().float(), ref.float(), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("hq,hkv,cap", [(8, 8, 0.0), (32, 8, 0.0), (16, 2, 20.0)])
def test_decode_attention_fwd_token_granular(cuda_device, hq, hkv, cap):
    """decode_attention_fwd (decode_attention.py:559): request -> token table, page size one."""
    from dlcompiler_b200 import decode_attention_fwd

    g = torch.Generator().manual_seed(hq + hkv)
    B, D, max_ctx, pool = 5, 128, 700, 4000
    lens = torch.randint(1, max_ctx + 1, (B,), generator=g)
    req_to_token = torch.zeros(9, max_ctx, dtype=torch.int32)
    b_req_idx = torch.tensor([7, 2, 5, 0, 3])
    perm = torch.randperm(pool, generator=g)
    off = 0
    for i in range(B):
        n = int(lens[i])
        req_to_token[b_req_idx[i], :n] = perm[off:off + n].to(torch.int32)
        off += n
    kb = torch.randn(pool, hkv, D, generator=g).to(torch.bfloat16)
    vb = torch.randn(pool, hkv, D, generator=g).to(torch.bfloat16)
    q = torch.randn(B, hq, D, generator=g).to(torch.bfloat16)
    dev = cuda_device
    o = torch.full_like(q, float("nan")).to(dev)
    start = torch.cat([lens.new_zeros(1), lens.cumsum(0)[:-1]])
    decode_attention_fwd(q.to(dev), kb.to(dev), vb.to(dev), o, req_to_token.to(dev), b_req_idx.to(dev),
                         start.to(dev), lens.to(dev), None, max_ctx, D ** -0.5, logit_cap=cap)
    ref = oracle.paged_decode_attention(q, kb.unsqueeze(1), vb.unsqueeze(1), req_to_token[b_req_idx], lens,
                                        sm_scale=D ** -0.5, logit_softcapping=cap if cap > 0 else None)
    torch.testing.assert_close(o.cpu().float(), ref.float(), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("dk,dv,dtype", [(64, 64, torch.bfloat16), (48, 32, torch.float16), (96, 64, torch.bfloat16),
                                         (128, 80, torch.float16)])
def test_decode_attention_fwd_token_granular_head_sizes(cuda_device, dk, dv, dtype):
    """The one-token-page gather at the 64-wide tile, at head sizes below the tile width (chunks past the head
    size are zero-length copies) and with a v head size that differs from the q / k one."""
    from dlcompiler_b200 import decode_attention_fwd

    g = torch.Generator().manual_seed(dk * 1000 + dv)
    B, hq, hkv, max_ctx, pool = 4, 8, 2, 300, 1500
    lens = torch.randint(1, max_ctx + 1, (B,), generator=g)
    req_to_token = torch.zeros(B, max_ctx, dtype=torch.int32)
    perm = torch.randperm(pool, generator=g)
    off = 0
    for i in range(B):
        n = int(lens[i])
        req_to_token[i, :n] = perm[off:off + n].to(torch.int32)
        off += n
    kb = torch.randn(pool, hkv, dk, generator=g).to(dtype)
    vb = torch.randn(pool, hkv, dv, generator=g).to(dtype)
    q = torch.randn(B, hq, dk, generator=g).to(dtype)
    dev = cuda_device
    o = torch.full((B, hq, dv), float("nan"), dtype=dtype, device=dev)
    start = torch.cat([lens.new_zeros(1), lens.cumsum(0)[:-1]])
    decode_attention_fwd(q.to(dev), kb.to(dev), vb.to(dev), o, req_to_token.to(dev), torch.arange(B, device=dev),
                         start.to(dev), lens.to(dev), None, max_ctx, dk ** -0.5)
    ref = oracle.paged_decode_attention(q, kb.unsqueeze(1), vb.unsqueeze(1), req_to_token, lens, sm_scale=dk ** -0.5)
    torch.testing.assert_close(o.cpu().float(), ref.float(), rtol=RTOL, atol=ATOL)


# ------------------------------------------------------------------ prefill over a paged cache with history
def _paged_prefill_case(seed, q_lens, hist_lens, page, hq, hkv, D, dtype, table_dtype=torch.int32):
    g = torch.Generator().manual_seed(seed)
    q_lens, hist_lens = torch.tensor(q_lens), torch.tensor(hist_lens)
    kv_lens = q_lens + hist_lens
    pages_per_seq = (kv_lens + page - 1) // page
    total_pages = int(pages_per_seq.sum())
    perm = torch.randperm(total_pages + 3, generator=g)          # a few pages stay unused
    table = torch.zeros(len(q_lens), int(pages_per_seq.max()) + 1, dtype=table_dtype)
    k_cache = torch.randn(total_pages + 3, page, hkv, D, generator=g).to(dtype)
    v_cache = torch.randn(total_pages + 3, page, hkv, D, generator=g).to(dtype)
    at = 0
    for b, n in enumerate(pages_per_seq.tolist()):
        table[b, :n] = perm[at:at + n].to(table_dtype)
        at += n
    q = torch.randn(int(q_lens.sum()), hq, D, generator=g).to(dtype)
    q_start = torch.cumsum(q_lens, 0) - q_lens
    return dict(q=q, k_cache=k_cache, v_cache=v_cache, table=table, q_start=q_start, q_lens=q_lens, kv_lens=kv_lens)


@pytest.mark.parametrize("q_lens,hist_lens,page,hq,hkv,D,dtype,tdt", [
    ([5, 130, 64], [0, 0, 0], 64, 8, 2, 128, torch.bfloat16, torch.int32),          # no history: plain prefill
    ([3, 200, 1, 77], [100, 37, 500, 64], 64, 8, 2, 128, torch.bfloat16, torch.int64),
    ([129, 16], [63, 1000], 16, 4, 4, 64, torch.float16, torch.int32),              # four pages per key block
    ([300, 2], [129, 31], 128, 8, 1, 128, torch.float16, torch.int32),              # two key blocks per page
    ([40], [24], 32, 2, 2, 64, torch.bfloat16, torch.int64),
])
def test_paged_prefill_with_history(cuda_device, q_lens, hist_lens, page, hq, hkv, D, dtype, tdt):
    """The prefill branch of paged_attention_fwd: new tokens attend causally to a cache that already holds
    their own K/V and `hist` earlier tokens, against the oracle's masked naive attention."""
    d = _paged_prefill_case(sum(q_lens) + page, q_lens, hist_lens, page, hq, hkv, D, dtype, tdt)
    dev = cuda_device
    q = d["q"].to(dev)
    o = torch.full_like(q, float("nan"))
    paged_attention_fwd(q, d["k_cache"].to(dev), d["v_cache"].to(dev), o, d["table"].to(dev), d["q_start"].to(dev),
                        d["q_lens"].to(dev), d["kv_lens"].to(dev), int(max(q_lens)))
    ref = oracle.paged_prefill_attention(d["q"], d["k_cache"], d["v_cache"], d["table"], d["q_start"], d["q_lens"],
                                         d["kv_lens"])
    out = o.cpu()
    assert torch.isfinite(out.float()).all()
    torch.testing.assert_close(out.float(), ref.float(), rtol=RTOL, atol=ATOL)


def test_paged_prefill_equals_contiguous_prefill(cuda_device):
    """Without history the paged branch and context_attention_fwd see the same keys in the same 64-key
    blocks, so their outputs are bit-identical."""
    d = _paged_prefill_case(3, [257, 64, 90], [0, 0, 0], 64, 8, 2, 128, torch.bfloat16)
    dev = cuda_device
    q = d["q"].to(dev)
    o = torch.empty_like(q)
    paged_attention_fwd(q, d["k_cache"].to(dev), d["v_cache"].to(dev), o, d["table"].to(dev), d["q_start"].to(dev),
                        d["q_lens"].to(dev), d["kv_lens"].to(dev), 257)
    # the same K/V, token-contiguous
    ks, vs = [], []
    for b, n in enumerate(d["kv_lens"].tolist()):
        npg = (n + 63) // 64
        pages = d["table"][b, :npg].long()
        ks.append(d["k_cache"][pages].reshape(npg * 64, 2, 128)[:n])
        vs.append(d["v_cache"][pages].reshape(npg * 64, 2, 128)[:n])
    o2 = torch.empty_like(q)
    context_attention_fwd(q, torch.cat(ks).to(dev), torch.cat(vs).to(dev), o2, d["q_start"].int().to(dev),
                          d["q_lens"].int().to(dev), 257)
    assert torch.equal(o, o2)


@pytest.mark.parametrize("window,softcap", [(100, None), (17, None), (None, 30.0), (64, 20.0), (5000, None)])
def test_paged_prefill_window_and_softcap(cuda_device, window, softcap):
    """Sliding window (a query sees its last window + 1 keys) and tanh soft-cap in the prefill branch."""
    d = _paged_prefill_case(17, [3, 200, 130, 64], [100, 37, 500, 0], 64, 8, 2, 128, torch.bfloat16)
    dev = cuda_device
    q = d["q"].to(dev)
    o = torch.full_like(q, float("nan"))
    paged_attention_fwd(q, d["k_cache"].to(dev), d["v_cache"].to(dev), o, d["table"].to(dev), d["q_start"].to(dev),
                        d["q_lens"].to(dev), d["kv_lens"].to(dev), 200, window_size=window, logit_softcapping=softcap)
    ref = oracle.paged_prefill_attention(d["q"], d["k_cache"], d["v_cache"], d["table"], d["q_start"], d["q_lens"],
                                         d["kv_lens"], window_size=window, logit_softcapping=softcap)
    out = o.cpu()
    assert torch.isfinite(out.float()).all()
    torch.testing.assert_close(out.float(), ref.float(), rtol=RTOL, atol=ATOL)


def test_paged_prefill_golden(cuda_device, golden_dir):
    """The prefill branch against the reference test's own ground truth (fixtures made by executing
    test_paged_attention.py's mask builder and naive attention on the CPU)."""
    for c in torch.load(os.path.join(golden_dir, "paged_prefill.pt"), weights_only=True):
        dev = cuda_device
        q = c["q"].to(dev)
        o = torch.full(q.shape[:-1] + (c["v_cache"].shape[-1],), float("nan"), dtype=q.dtype, device=dev)
        q_lens = c["q_seqlens"]
        start = torch.cumsum(q_lens, 0) - q_lens
        paged_attention_fwd(q, c["k_cache"].to(dev), c["v_cache"].to(dev), o, c["block_offsets"].to(dev),
                            start.to(dev), q_lens.to(dev), c["kv_seqlens"].to(dev), int(q_lens.max()))
        # reference test: atol=1e-3, rtol=1e-5 for fp16 (test_paged_attention.py:286)
        tol = 1e-3 if q.dtype == torch.float16 else 8e-3
        torch.testing.assert_close(o.cpu(), c["gt"], atol=tol, rtol=1e-5)


def test_paged_prefill_ignores_stale_cache_slots(cuda_device, golden_dir):
    """Cache slots past a sequence's last key (the tail of its last page, and every page that no sequence
    uses) may hold anything, NaN bit patterns included: the output must not change by a bit."""
    for c in torch.load(os.path.join(golden_dir, "paged_prefill.pt"), weights_only=True)[:6]:
        dev = cuda_device
        q = c["q"].to(dev)
        q_lens = c["q_seqlens"]
        start = torch.cumsum(q_lens, 0) - q_lens
        page = c["k_cache"].shape[1]

        def run(kc, vc):
            o = torch.full(q.shape[:-1] + (vc.shape[-1],), float("nan"), dtype=q.dtype, device=dev)
            paged_attention_fwd(q, kc.to(dev), vc.to(dev), o, c["block_offsets"].to(dev), start.to(dev),
                                q_lens.to(dev), c["kv_seqlens"].to(dev), int(q_lens.max()))
            return o.cpu()

        base = run(c["k_cache"], c["v_cache"])
        kc, vc = c["k_cache"].clone(), c["v_cache"].clone()
        live = torch.zeros(kc.shape[0], page, dtype=torch.bool)
        for b, n in enumerate(c["kv_seqlens"].tolist()):
            for t in range(n):
                live[int(c["block_offsets"][b, t // page]), t % page] = True
        kc[~live] = float("nan")
        vc[~live] = float("nan")
        out = run(kc, vc)
        assert torch.isfinite(out.float()).all()
        assert torch.equal(out, base)


@pytest.mark.parametrize("q_lens,hist", [([30, 50, 70, 90], [50, 40, 30, 20]), ([1, 1, 1, 1], [50, 40, 30, 20])])
def test_paged_window_at_the_reference_test_sizes(cuda_device, q_lens, hist):
    """The reference's sliding-window test geometry (test_paged_attention.py:303-316): head size 16 for q, k
    and v, 4 / 2 heads, window 32, 16-token pages, fp16; prefill with history and decode."""
    d = _paged_prefill_case(31, q_lens, hist, 16, 4, 2, 16, torch.float16)
    dev = cuda_device
    q = d["q"].to(dev)
    o = torch.full_like(q, float("nan"))
    paged_attention_fwd(q, d["k_cache"].to(dev), d["v_cache"].to(dev), o, d["table"].to(dev), d["q_start"].to(dev),
                        d["q_lens"].to(dev), d["kv_lens"].to(dev), max(q_lens), window_size=32)
    ref = oracle.paged_prefill_attention(d["q"], d["k_cache"], d["v_cache"], d["table"], d["q_start"], d["q_lens"],
                                         d["kv_lens"], window_size=32)
    torch.testing.assert_close(o.cpu().float(), ref.float(), rtol=1e-3, atol=1e-3)
