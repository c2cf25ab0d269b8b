"""GPU parity for the steps next to the hot path: rms_norm / add_rms_norm, rotary embedding, fill_kv_cache."""
import os

import pytest
import torch

from dlcompiler_b200 import add_rms_norm, apply_rotary_pos_emb, fill_kv_cache, paged_attention_fwd, rms_norm
from oracle import dlblas_oracle as oracle

pytestmark = pytest.mark.gpu


def _ulp(out, ref, n=2):
    if out.numel() == 0:
        assert out.shape == ref.shape
        return
    eps = torch.finfo(out.dtype).eps
    torch.testing.assert_close(out.float(), ref.float(), rtol=n * eps, atol=n * eps * max(1.0, ref.abs().max().item()))


def test_rms_norm_golden(cuda_device, golden_dir):
    dev = cuda_device
    for c in torch.load(os.path.join(golden_dir, "rms_norm.pt"), weights_only=True):
        x, w, res = c["x"].to(dev), c["w"].to(dev), c["res"].to(dev)
        _ulp(rms_norm(x, w, c["eps"]).cpu(), c["gt_rms"])                      # reference test: default assert_close
        out, new_res = add_rms_norm(x, w, c["eps"], res)
        assert torch.equal(new_res.cpu(), c["gt_add_res"])
        _ulp(out.cpu(), c["gt_add_out"])
        ref, _ = oracle.rms_norm(c["x"], c["w"], c["eps"])
        _ulp(rms_norm(x, w, c["eps"]).cpu(), ref, n=1)


@pytest.mark.parametrize("rows,n,dtype", [(1, 8, torch.float16), (7, 4096, torch.bfloat16), (3, 11008, torch.bfloat16),
                                          (5, 100, torch.float32), (2, 20000, torch.bfloat16), (4, 130, torch.float16),
                                          (0, 64, torch.bfloat16)])
def test_rms_norm_shapes_residual_and_out(cuda_device, rows, n, dtype):
    g = torch.Generator().manual_seed(rows * 31 + n)
    x = torch.randn(rows, n, generator=g).to(dtype)
    w = torch.rand(n, generator=g).to(dtype)
    res = torch.randn(rows, n, generator=g).to(dtype)
    dev = cuda_device
    out, out_res = rms_norm(x.to(dev), w.to(dev), 1e-5, residual=res.to(dev))
    ref, ref_res = oracle.rms_norm(x, w, 1e-5, residual=res)
    assert torch.equal(out_res.cpu(), ref_res)
    _ulp(out.cpu(), ref)
    buf = torch.zeros(rows, n, dtype=dtype, device=dev)
    assert rms_norm(x.to(dev), w.to(dev), 1e-5, out=buf).data_ptr() == buf.data_ptr()
    _ulp(buf.cpu(), oracle.rms_norm(x, w, 1e-5)[0])
    o3 = add_rms_norm(x.to(dev), w.to(dev), 1e-5)
    _ulp(o3.cpu(), oracle.rms_norm(x, w, 1e-5, weight_after_cast=True)[0])


def test_rms_norm_relative_l2_of_reference_test(cuda_device):
    """4096 x 4096 fp16 with residual, relative L2 <= 0.003 (tests/kernels/test_add_rms_norm.py:44-75)."""
    g = torch.Generator().manual_seed(1)
    x = torch.randn(4096, 4096, generator=g).half()
    r = torch.randn(4096, 4096, generator=g).half()
    w = torch.randn(4096, generator=g).half()
    out, res = add_rms_norm(x.to(cuda_device), w.to(cuda_device), 1e-6, r.to(cuda_device))
    ref, ref_res = oracle.rms_norm(x, w, 1e-6, residual=r, weight_after_cast=True)
    assert torch.equal(res.cpu(), ref_res)
    rel = ((out.cpu().float() - ref.float()).pow(2).sum() / ref.float().pow(2).sum()).sqrt().item()
    assert rel <= 0.003


def test_rotary_golden_and_inplace(cuda_device, golden_dir):
    dev = cuda_device
    for c in torch.load(os.path.join(golden_dir, "rotary.pt"), weights_only=True):
        q, k = c["q"].to(dev), c["k"].to(dev)
        qe, ke = apply_rotary_pos_emb(q, k, c["cos"].to(dev), c["sin"].to(dev))
        tol = dict(rtol=1e-5, atol=1e-3) if q.dtype == torch.float16 else {}     # reference test's tolerances
        torch.testing.assert_close(qe.cpu(), c["gt_q"], **tol)
        torch.testing.assert_close(ke.cpu(), c["gt_k"], **tol)
        if q.dtype != torch.float32:
            assert torch.equal(qe.cpu(), c["gt_q"]) and torch.equal(ke.cpu(), c["gt_k"])   # same rounding points
        q2, k2 = q.clone(), k.clone()
        apply_rotary_pos_emb(q2, k2, c["cos"].to(dev), c["sin"].to(dev), q2, k2)          # outputs alias inputs
        assert torch.equal(q2, qe) and torch.equal(k2, ke)


def test_rotary_strided_views(cuda_device):
    g = torch.Generator().manual_seed(3)
    T, hq, hk, d = 300, 32, 8, 128
    qkv = torch.randn(T, (hq + 2 * hk) * d, generator=g).to(torch.bfloat16).to(cuda_device)
    q = qkv[:, :hq * d].view(T, hq, d)
    k = qkv[:, hq * d:(hq + hk) * d].view(T, hk, d)
    cos = torch.rand(T, d, generator=g).to(torch.bfloat16)
    sin = torch.rand(T, d, generator=g).to(torch.bfloat16)
    qe, ke = apply_rotary_pos_emb(q, k, cos.to(cuda_device), sin.to(cuda_device))
    rq, rk = oracle.apply_rotary_pos_emb(q.cpu(), k.cpu(), cos, sin)
    assert torch.equal(qe.cpu(), rq) and torch.equal(ke.cpu(), rk)


def test_fill_kv_cache_golden(cuda_device, golden_dir):
    dev = cuda_device
    for c in torch.load(os.path.join(golden_dir, "fill_kv_cache.pt"), weights_only=True):
        kc, vc = c["k_caches"].to(dev), c["v_caches"].to(dev)
        q_len = torch.tensor(c["seq_lens"])
        kv_len = q_len + torch.tensor(c["history_lens"])
        start = q_len.cumsum(0) - q_len
        fill_kv_cache(c["k_states"].to(dev), c["v_states"].to(dev), kc, vc, start.to(dev), q_len.to(dev),
                      kv_len.to(dev), int(q_len.max()), c["block_offsets"].to(dev))
        assert torch.equal(kc.cpu(), c["gt_k"]) and torch.equal(vc.cpu(), c["gt_v"])


@pytest.mark.parametrize("dtype,heads,dk,dv,page,idx", [
    (torch.float32, 3, 20, 12, 16, torch.int32),     # odd sizes: 4-byte copy path, different K and V widths
    (torch.float16, 2, 48, 32, 16, torch.int64),     # the paged-attention test's head sizes
    (torch.bfloat16, 8, 128, 128, 64, torch.int32),
])
def test_fill_kv_cache_shapes(cuda_device, dtype, heads, dk, dv, page, idx):
    g = torch.Generator().manual_seed(dk)
    seq_lens, hist = [5, 40, 1, 17], [0, 30, 63, 100]
    kv = [a + b for a, b in zip(seq_lens, hist)]
    nblk = [(n + page - 1) // page for n in kv]
    B, mx = 4, max(nblk)
    ks = torch.randn(sum(seq_lens), heads, dk, generator=g).to(dtype)
    vs = torch.randn(sum(seq_lens), heads, dv, generator=g).to(dtype)
    kc = torch.randn(B * mx, page, heads, dk, generator=g).to(dtype)
    vc = torch.randn(B * mx, page, heads, dv, generator=g).to(dtype)
    table = torch.zeros(B, mx, dtype=idx)
    perm = torch.randperm(B * mx, generator=g)
    off = 0
    for b in range(B):
        table[b, :nblk[b]] = perm[off:off + nblk[b]].to(idx)
        off += nblk[b]
    dev = cuda_device
    kcd, vcd = kc.to(dev), vc.to(dev)
    q_len = torch.tensor(seq_lens, dtype=idx)
    fill_kv_cache(ks.to(dev), vs.to(dev), kcd, vcd, (q_len.cumsum(0) - q_len).to(dev), q_len.to(dev),
                  torch.tensor(kv, dtype=idx).to(dev), max(seq_lens), table.to(dev))
    rk, rv = oracle.fill_kv_cache(ks, vs, kc, vc, seq_lens, hist, table)
    assert torch.equal(kcd.cpu(), rk) and torch.equal(vcd.cpu(), rv)


def test_fill_then_decode_round_trip(cuda_device):
    """fill_kv_cache produces the layout paged decode reads: decode over a cache built token by token
    equals decode over the oracle-built cache."""
    from dlcompiler_b200 import workloads as W

    wl = W.DecodeWorkload(batch=3, ctx_lo=70, ctx_hi=300, page=64, hq=8, hkv=2, head_dim=128)
    d = wl.make()
    dev = cuda_device
    ctx = d["kv_seqlens"]
    kc = torch.zeros_like(d["k_cache"]).to(dev)
    vc = torch.zeros_like(d["v_cache"]).to(dev)
    # dense K/V per sequence, read back from the oracle-side cache
    ks, vs = [], []
    for b in range(3):
        n = int(ctx[b])
        pages = d["block_table"][b, :(n + 63) // 64].long()
        ks.append(d["k_cache"][pages].reshape(-1, 2, 128)[:n])
        vs.append(d["v_cache"][pages].reshape(-1, 2, 128)[:n])
    q_len = ctx.clone()
    fill_kv_cache(torch.cat(ks).to(dev), torch.cat(vs).to(dev), kc, vc, (q_len.cumsum(0) - q_len).int().to(dev),
                  q_len.to(dev), ctx.to(dev), int(q_len.max()), d["block_table"].to(dev))
    q = d["q"].to(dev)
    o1, o2 = torch.empty_like(q), torch.empty_like(q)
    args = (d["block_table"].to(dev), torch.arange(3, device=dev), torch.ones(3, dtype=torch.int64, device=dev),
            ctx.to(dev), 1)
    paged_attention_fwd(q, kc, vc, o1, *args)
    paged_attention_fwd(q, d["k_cache"].to(dev), d["v_cache"].to(dev), o2, *args)
    assert torch.equal(o1, o2)


def test_registry_lookup_runs_the_same_kernels(cuda_device):
    """`get_op(name, args)(*args)`, the reference's calling convention for its registered ops
    (dlblas/__init__.py:13-23, add_rms_norm.py:103-118), gives the direct call's result."""
    import dlcompiler_b200 as dl
    g = torch.Generator().manual_seed(5)
    x = torch.randn(33, 512, generator=g).to(torch.bfloat16).to(cuda_device)
    w = torch.randn(512, generator=g).to(torch.bfloat16).to(cuda_device)
    res = torch.randn(33, 512, generator=g).to(torch.bfloat16).to(cuda_device)
    args = (x, w, 1e-6)
    assert torch.equal(dl.get_op("rms_norm", args)(*args), add_rms_norm(x, w, 1e-6))
    args = (x, w, 1e-6, res)
    out, res_out = dl.get_op("add_rms_norm", args)(*args)
    ref_out, ref_res = add_rms_norm(x, w, 1e-6, res)
    assert torch.equal(out, ref_out) and torch.equal(res_out, ref_res)
    q = torch.randn(2, 64, 4, 64, generator=g).to(torch.bfloat16).to(cuda_device)
    args = (q, q, q)
    assert torch.equal(dl.get_op("flash_attention_v2", args)(*args), dl.flash_attention_v2(q, q, q))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_rotary_and_fa(cuda_device, dtype):
    """Rotary on q and k, then dense non-causal attention (fused_rotary_and_fa.py:120-182), against the
    oracle's rotary followed by the oracle's attention."""
    import dlcompiler_b200 as dl
    g = torch.Generator().manual_seed(11)
    b, s, h, d = 2, 200, 4, 128
    q, k, v = (torch.randn(b, s, h, d, generator=g).to(dtype) for _ in range(3))
    ang = torch.rand(b, s, d // 2, generator=g) * 6.283
    cos = torch.cat([ang.cos(), ang.cos()], dim=-1).to(dtype)
    sin = torch.cat([ang.sin(), ang.sin()], dim=-1).to(dtype)
    out = dl.get_op("fused_rotary_and_fa", (q, k, v, cos, sin))(
        q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device)).cpu()
    qr, kr = oracle.apply_rotary_pos_emb(q.reshape(b * s, h, d), k.reshape(b * s, h, d), cos.reshape(b * s, d),
                                         sin.reshape(b * s, d))
    ref = oracle.context_attention(qr, kr, v.reshape(b * s, h, d), torch.arange(b) * s, torch.full((b,), s),
                                   causal=False)
    torch.testing.assert_close(out.reshape(b * s, h, d).float(), ref.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("D,dtype", [(128, torch.bfloat16), (64, torch.float16), (96, torch.bfloat16), (32, torch.float16)])
def test_rotary_inside_prefill_and_fill_equal_the_separate_kernels(cuda_device, D, dtype):
    """Rotary folded into the neighbouring kernels: q rotated on its tile inside the attention kernel, k rotated
    while fill_kv_cache writes it.  Both must give the bits of the stand-alone rotary kernel followed by the plain
    kernels: the rotated cache is compared directly, the attention output through both routes."""
    from dlcompiler_b200 import context_attention_fwd

    dev = cuda_device
    g = torch.Generator().manual_seed(D)
    q_lens, hist = torch.tensor([70, 1, 200, 129]), torch.tensor([0, 35, 16, 100])
    kv_lens = q_lens + hist
    hq, hkv, page = 8, 2, 16
    total = int(q_lens.sum())
    q = torch.randn(total, hq, D, generator=g).to(dtype).to(dev)
    k_new = torch.randn(total, hkv, D, generator=g).to(dtype).to(dev)
    v_new = torch.randn(total, hkv, D, generator=g).to(dtype).to(dev)
    cos = torch.rand(total, D, generator=g).to(dtype).to(dev)
    sin = torch.rand(total, D, generator=g).to(dtype).to(dev)
    pages_per_seq = (kv_lens + page - 1) // page
    n_pages = int(pages_per_seq.sum())
    table = torch.zeros(4, int(pages_per_seq.max()), dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g)
    at = 0
    for b, n in enumerate(pages_per_seq.tolist()):
        table[b, :n] = perm[at:at + n].to(torch.int32)
        at += n
    base_k = torch.randn(n_pages, page, hkv, D, generator=g).to(dtype).to(dev)     # history keys (already rotated)
    base_v = torch.randn(n_pages, page, hkv, D, generator=g).to(dtype).to(dev)
    start = (torch.cumsum(q_lens, 0) - q_lens).to(dev)
    ql, kl, tb = q_lens.to(dev), kv_lens.to(dev), table.to(dev)

    # route A: stand-alone rotary, plain fill, plain paged prefill
    q_rot, k_rot = apply_rotary_pos_emb(q, k_new, cos, sin)
    kc_a, vc_a = base_k.clone(), base_v.clone()
    fill_kv_cache(k_rot, v_new, kc_a, vc_a, start, ql, kl, int(q_lens.max()), tb)
    o_a = torch.full_like(q, float("nan"))
    paged_attention_fwd(q_rot, kc_a, vc_a, o_a, tb, start, ql, kl, int(q_lens.max()))
    # route B: k rotated by the fill, q rotated inside the attention kernel
    kc_b, vc_b = base_k.clone(), base_v.clone()
    fill_kv_cache(k_new, v_new, kc_b, vc_b, start, ql, kl, int(q_lens.max()), tb, cos=cos, sin=sin)
    assert torch.equal(kc_a, kc_b) and torch.equal(vc_a, vc_b)
    o_b = torch.full_like(q, float("nan"))
    paged_attention_fwd(q, kc_b, vc_b, o_b, tb, start, ql, kl, int(q_lens.max()), q_cos=cos, q_sin=sin)
    assert torch.isfinite(o_a.float()).all()
    assert torch.equal(o_a, o_b)
    # the contiguous entry point, same comparison (no history)
    o_c = torch.empty_like(q)
    context_attention_fwd(q_rot, k_rot, v_new, o_c, start.int(), ql.int(), int(q_lens.max()))
    o_d = torch.empty_like(q)
    context_attention_fwd(q, k_rot, v_new, o_d, start.int(), ql.int(), int(q_lens.max()), q_cos=cos, q_sin=sin)
    assert torch.equal(o_c, o_d)
    # and against the oracle, end to end
    rq, rk = oracle.apply_rotary_pos_emb(q.cpu(), k_new.cpu(), cos.cpu(), sin.cpu())
    ref = oracle.context_attention(rq, rk, v_new.cpu(), start.cpu(), q_lens)
    torch.testing.assert_close(o_d.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
