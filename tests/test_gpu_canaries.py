"""Out-of-bounds writes: every output (and the decode workspace) sits between two canary bands that must come
back untouched.  The memory checker of the toolkit is not available on the GPU pool, so the bands stand in for
it; odd and tiny shapes are used on purpose (tails are where an index slips)."""
import pytest
import torch

import dlcompiler_b200 as dl
from dlcompiler_b200 import _lib
from dlcompiler_b200 import workloads as W

pytestmark = pytest.mark.gpu

BAND = 4096     # elements on either side


class Guarded:
    """A tensor of the requested shape carved out of a larger buffer filled with a canary pattern."""

    def __init__(self, shape, dtype, device):
        n = 1
        for s in shape:
            n *= s
        self.buf = torch.empty(n + 2 * BAND, dtype=dtype, device=device)
        self.pattern = 3 if not dtype.is_floating_point else -1234.5
        self.buf.fill_(self.pattern)
        self.t = self.buf[BAND:BAND + n].view(shape)
        self.n = n

    def check(self, what):
        lo, hi = self.buf[:BAND], self.buf[BAND + self.n:]
        assert bool((lo == self.pattern).all()) and bool((hi == self.pattern).all()), f"{what}: canary band overwritten"


def test_canaries_elementwise_and_routing(cuda_device):
    dev = cuda_device
    x = torch.randn(37, 2 * 1384, device=dev).bfloat16()
    out = Guarded((37, 1384), torch.bfloat16, dev)
    dl.silu_and_mul(x, out.t)
    out.check("silu_and_mul")
    h = torch.randn(33, 520, device=dev).bfloat16()
    w = torch.rand(520, device=dev).bfloat16()
    r = torch.randn(33, 520, device=dev).bfloat16()
    o, o_r = Guarded((33, 520), torch.bfloat16, dev), Guarded((33, 520), torch.bfloat16, dev)
    dl.rms_norm(h, w, 1e-6, residual=r, out=o.t, out_residual=o_r.t)
    o.check("rms_norm out")
    o_r.check("rms_norm out_residual")
    q, k = torch.randn(19, 5, 64, device=dev).half(), torch.randn(19, 3, 64, device=dev).half()
    cos, sin = torch.rand(19, 64, device=dev).half(), torch.rand(19, 64, device=dev).half()
    qo, ko = Guarded((19, 5, 64), torch.float16, dev), Guarded((19, 3, 64), torch.float16, dev)
    dl.apply_rotary_pos_emb(q, k, cos, sin, qo.t, ko.t)
    qo.check("rotary q")
    ko.check("rotary k")


def test_canaries_fused_moe_pieces(cuda_device):
    dev = cuda_device
    lib = _lib.load()
    T, E, k, block = 301, 7, 3, 128
    ids = torch.randint(-1, E + 1, (T * k,), device=dev, dtype=torch.int64)
    numel = T * k
    cap = (numel + E * (block - 1) + block - 1) // block * block
    sorted_ids = Guarded((cap,), torch.int32, dev)
    expert_ids = Guarded((cap // block,), torch.int32, dev)
    meta = Guarded((E + 2,), torch.int32, dev)
    with torch.cuda.device(dev):
        rc = lib.dlb_moe_align_block_size(ids.data_ptr(), 1, numel, E, block, sorted_ids.t.data_ptr(), cap,
                                          expert_ids.t.data_ptr(), cap // block, meta.t[:1].data_ptr(),
                                          meta.t[1:].data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "align")
    torch.cuda.synchronize()
    for g, name in ((sorted_ids, "sorted_token_ids"), (expert_ids, "expert_ids"), (meta, "num_post / block_start")):
        g.check("moe_align " + name)
    se = Guarded((2, E), torch.int64, dev)
    with torch.cuda.device(dev):
        rc = lib.dlb_moe_start_end(ids.data_ptr(), 1, numel, E, se.t[0].data_ptr(), se.t[1].data_ptr(), 1,
                                   _lib.stream_ptr(dev))
    _lib.check(rc, "start_end")
    se.check("moe_start_end")
    # the grouped GEMM's scatter epilogue and the combine, through fused_moe's own allocations: guard the inputs
    # instead (a stray store into hidden states or weights would show as a changed checksum)
    H, I = 136, 200
    hs = Guarded((T, H), torch.bfloat16, dev)
    hs.t.copy_(torch.randn(T, H, device=dev))
    w1 = Guarded((E, 2 * I, H), torch.bfloat16, dev)
    w1.t.copy_(torch.randn(E, 2 * I, H, device=dev) * 0.1)
    w2 = Guarded((E, H, I), torch.bfloat16, dev)
    w2.t.copy_(torch.randn(E, H, I, device=dev) * 0.1)
    before = [t.t.float().sum().item() for t in (hs, w1, w2)]
    tw = torch.rand(T, k, device=dev)
    out = dl.fused_moe(hs.t, w1.t, w2.t, tw, ids.view(T, k), k)
    assert torch.isfinite(out.float()).all()
    for g, name, b in zip((hs, w1, w2), ("hidden", "w1", "w2"), before):
        g.check("fused_moe " + name)
        assert g.t.float().sum().item() == b


def test_canaries_attention(cuda_device):
    dev = cuda_device
    wl = W.PrefillWorkload(seq_lens=[130, 1, 77], hq=6, hkv=2, head_dim=96)
    d = wl.make()
    q, k, v = d["q"].to(dev), d["k"].to(dev), d["v"].to(dev)
    o = Guarded(tuple(q.shape), q.dtype, dev)
    lse = Guarded((6, q.shape[0]), torch.float32, dev)
    dl.context_attention_fwd(q, k, v, o.t, d["b_start_loc"].to(dev), d["b_seq_len"].to(dev), 130, lse=lse.t)
    o.check("prefill o")
    lse.check("prefill lse")
    dw = W.DecodeWorkload(batch=3, ctx_lo=1, ctx_hi=700, page=16, hq=8, hkv=2, head_dim=128)
    dd = dw.make()
    qd = dd["q"].to(dev)
    kc, vc, tb, ln = (dd[n].to(dev) for n in ("k_cache", "v_cache", "block_table", "kv_seqlens"))
    lib = _lib.load()
    chunk, splits = 256, (tb.size(1) * 16 + 255) // 256
    od = Guarded((3, 8, 128), qd.dtype, dev)
    part = Guarded((lib.dlb_paged_decode_workspace_floats(3, 8, 128, splits),), torch.float32, dev)
    with torch.cuda.device(dev):
        rc = lib.dlb_paged_decode(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), od.t.data_ptr(), tb.data_ptr(),
                                  ln.data_ptr(), part.t.data_ptr(), 3, 8, 2, 128, 128, 16, kc.size(0), tb.size(1),
                                  qd.stride(0), qd.stride(1), od.t.stride(0), od.t.stride(1), kc.stride(0), kc.stride(1),
                                  kc.stride(2), vc.stride(0), vc.stride(1), vc.stride(2), tb.stride(0), 0, 0, chunk,
                                  splits, -1, 128 ** -0.5, -1.0, _lib.DTYPE_BF16, _lib.status_word(dev).data_ptr(),
                                  _lib.stream_ptr(dev))
    _lib.check(rc, "paged_decode")
    torch.cuda.synchronize()
    od.check("decode o")
    part.check("decode split workspace")
    # fill_kv_cache: pages that no sequence owns stay as they were
    pages, page = 12, 16
    kcache = Guarded((pages, page, 2, 64), torch.float16, dev)
    vcache = Guarded((pages, page, 2, 64), torch.float16, dev)
    kcache.t.fill_(7.0)
    vcache.t.fill_(7.0)
    ks, vs = torch.randn(40, 2, 64, device=dev).half(), torch.randn(40, 2, 64, device=dev).half()
    table = torch.tensor([[3, 9, 0], [5, 1, 0]], dtype=torch.int32, device=dev)
    qlen = torch.tensor([25, 15], dtype=torch.int32, device=dev)
    kvlen = torch.tensor([30, 15], dtype=torch.int32, device=dev)
    start = torch.tensor([0, 25], dtype=torch.int32, device=dev)
    dl.fill_kv_cache(ks, vs, kcache.t, vcache.t, start, qlen, kvlen, 25, table)
    kcache.check("fill_kv_cache k")
    vcache.check("fill_kv_cache v")
    untouched = [p for p in range(pages) if p not in (3, 9, 5)]
    assert bool((kcache.t[untouched] == 7.0).all()) and bool((vcache.t[untouched] == 7.0).all())
    assert bool((kcache.t[3, :5] == 7.0).all())          # history slots of sequence 0
