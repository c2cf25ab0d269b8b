"""Properties of the CPU oracle and of the workload definitions (no GPU)."""
import torch

from dlcompiler_b200 import workloads as W
from oracle import dlblas_oracle as oracle


def test_algorithmic_work_matches_the_stated_figures():
    assert W.SiluWorkload().bytes() == 270_532_608
    assert W.GatingWorkload().bytes() == 17_826_816
    assert W.MoeWorkload().flops() == 2_886_218_022_912
    assert W.MoeWorkload().flops(tokens=1) == 704_643_072
    assert W.PrefillWorkload().flops() == 2_199_023_255_552
    lens = torch.tensor([1000, 24])
    assert W.DecodeWorkload.bytes(lens) == 1024 * 4096 + 2 * 2 * 32 * 128 * 2


def test_moe_align_oracle_properties():
    g = torch.Generator().manual_seed(7)
    for numel, E, block in [(0, 4, 16), (1, 4, 16), (37, 5, 8), (8192, 8, 128), (1000, 256, 128)]:
        ids = torch.randint(0, E, (numel,), generator=g)
        s, e, n, bs = oracle.moe_align_block_size(ids, block, E)
        n = int(n)
        assert n % block == 0 and n <= s.numel()
        valid = s[:n][s[:n] < numel].long()
        assert torch.equal(valid.sort()[0], torch.arange(numel))            # a permutation of the slots
        assert torch.all(s[n:] == numel)
        for b in range(n // block):
            blk = s[b * block:(b + 1) * block]
            real = blk[blk < numel].long()
            assert torch.all(ids[real] == e[b])                             # one expert per block
            assert torch.all(real[1:] > real[:-1])                          # stable inside the block
        assert int(bs[-1]) == n // block
        start, end = oracle.start_end_from_counts(ids, E)
        assert torch.equal((end - start + block - 1) // block, (bs[1:] - bs[:-1]).long())


def test_moe_align_oracle_drops_foreign_experts():
    ids = torch.tensor([0, 5, 1, -1, 1, 7])
    s, e, n, _ = oracle.moe_align_block_size(ids, 4, 2)
    assert int(n) == 8
    assert s[:8].tolist() == [0, 6, 6, 6, 2, 4, 6, 6]
    assert e[:2].tolist() == [0, 1]


def test_grouped_gating_oracle_structure_and_margins():
    wl = W.GatingWorkload(tokens=2048)
    d = wl.make()
    ids, w = oracle.grouped_topk_gating(d["logits"], d["bias"], wl.top_k, wl.n_group, wl.topk_group,
                                        wl.scale_factor, True, "sigmoid")
    assert ids.shape == (2048, 8) and ids.dtype == torch.int32
    groups = (ids // (wl.experts // wl.n_group))
    assert all(len(set(r.tolist())) <= wl.topk_group for r in groups)       # at most 4 groups used
    assert all(len(set(r.tolist())) == wl.top_k for r in ids)               # distinct experts
    torch.testing.assert_close(w.sum(-1), torch.full((2048,), wl.scale_factor), rtol=1e-5, atol=1e-5)
    choice = oracle.sigmoid_spec(d["logits"]) + d["bias"]
    picked = choice.gather(1, ids.long())
    assert torch.all(picked[:, 1:] <= picked[:, :-1])                       # descending order
    # fp64 decision margins: ids are well-defined if every margin is far above fp32 noise
    m = oracle.gating_margins(d["logits"], d["bias"], wl.top_k, wl.n_group, wl.topk_group)
    assert m.min() > 0


def test_sigmoid_spec_accuracy_and_range():
    x = torch.randn(1 << 16, generator=torch.Generator().manual_seed(3)) * 4
    ref = torch.sigmoid(x.double())
    rel = ((oracle.sigmoid_spec(x).double() - ref) / ref).abs().max()
    assert rel < 5e-7
    edge = oracle.sigmoid_spec(torch.tensor([-1e4, -88.0, 0.0, 88.0, 1e4]))
    assert torch.isfinite(edge).all() and edge[2] == 0.5 and edge[-1] == 1.0 and edge[0] >= 0


def test_fma32_is_the_correctly_rounded_fused_multiply_add():
    """The oracle's fp32 FMA against C's fmaf (compiled here with gcc), including sums that sit a
    hair beside an fp32 rounding midpoint, where rounding to fp64 first would round twice."""
    import ctypes, shutil, subprocess, tempfile, os
    import numpy as np
    import pytest
    if shutil.which("gcc") is None:
        pytest.skip("gcc not available")
    d = tempfile.mkdtemp()
    with open(os.path.join(d, "f.c"), "w") as fh:
        fh.write("#include <math.h>\nvoid f(const float*a,const float*b,const float*c,float*o,long n)"
                 "{for(long i=0;i<n;i++)o[i]=fmaf(a[i],b[i],c[i]);}\n")
    subprocess.check_call(["gcc", "-O2", "-shared", "-fPIC", "-o", os.path.join(d, "f.so"), os.path.join(d, "f.c"), "-lm"])
    lib = ctypes.CDLL(os.path.join(d, "f.so"))

    def same(a, b, c):
        out = np.empty_like(a)
        vp = lambda x: x.ctypes.data_as(ctypes.c_void_p)
        lib.f(vp(a), vp(b), vp(c), vp(out), ctypes.c_long(a.size))
        mine = oracle.fma32(torch.from_numpy(a), torch.from_numpy(b), torch.from_numpy(c)).numpy()
        return np.array_equal(mine.view(np.int32), out.view(np.int32))

    g = np.random.default_rng(0)
    n = 1 << 20
    a, b, c = (g.standard_normal(n).astype(np.float32) for _ in range(3))
    assert same(a, b, c)
    wide = lambda: (g.standard_normal(n) * 10.0 ** g.uniform(-8, 8, n)).astype(np.float32)
    assert same(wide(), wide(), wide())
    a = wide()
    assert same(a, b, (-(a.astype(np.float64) * b.astype(np.float64))).astype(np.float32))      # cancellation
    # a*b = 2^-24 * (1 -/+ 2^-40): c + a*b lies 2^-64 below / above the midpoint of c's ulp
    k = np.arange(1, 4097, dtype=np.float64)
    cc = (1.0 + k * 2.0 ** -23).astype(np.float32)
    a1 = np.full(cc.shape, 2.0 ** -12 * (1 + 2.0 ** -20), np.float32)
    b_lo = np.full(cc.shape, 2.0 ** -12 * (1 - 2.0 ** -20), np.float32)
    assert same(a1, b_lo, cc) and same(a1, -b_lo, -cc)
    b_hi = np.full(cc.shape, 2.0 ** -12 * (1 + 2.0 ** -20), np.float32)
    assert same(a1, b_hi, cc) and same(-a1, b_hi, -cc)


def test_gating_tie_break_is_lowest_index():
    logits = torch.zeros(1, 64)
    ids, w = oracle.grouped_topk_gating(logits, None, 4, 4, 2, 1.0, True, "sigmoid")
    assert ids.tolist() == [[0, 1, 2, 3]]
    torch.testing.assert_close(w, torch.full((1, 4), 0.25))


def test_softmax_topk_matches_torch_when_no_ties():
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(512, 8, generator=g)
    w, ids = oracle.softmax_topk(logits, 2)
    tw, ti = torch.topk(torch.softmax(logits, -1, dtype=torch.float32), 2, dim=-1)
    assert torch.equal(ids.long(), ti)
    torch.testing.assert_close(w, tw)


def test_prefill_oracle_blocking_is_invisible():
    wl = W.PrefillWorkload(seq_lens=[70, 33], hq=4, hkv=2)
    d = wl.make()
    a = oracle.context_attention(d["q"], d["k"], d["v"], d["b_start_loc"], d["b_seq_len"], block_rows=1024)
    b = oracle.context_attention(d["q"], d["k"], d["v"], d["b_start_loc"], d["b_seq_len"], block_rows=16)
    torch.testing.assert_close(a, b, atol=1e-2, rtol=0)


def test_decode_oracle_window_and_softcap():
    wl = W.DecodeWorkload(batch=3, ctx_lo=10, ctx_hi=200, page=16, hq=4, hkv=2, head_dim=64)
    d = wl.make()
    full = oracle.paged_decode_attention(d["q"], d["k_cache"], d["v_cache"], d["block_table"], d["kv_seqlens"])
    big_window = oracle.paged_decode_attention(d["q"], d["k_cache"], d["v_cache"], d["block_table"],
                                               d["kv_seqlens"], window_size=10_000)
    assert torch.equal(full, big_window)
    capped = oracle.paged_decode_attention(d["q"], d["k_cache"], d["v_cache"], d["block_table"], d["kv_seqlens"],
                                           logit_softcapping=1e6)
    torch.testing.assert_close(full, capped, atol=1e-2, rtol=0)


def test_paged_prefill_oracle_is_the_tail_of_a_full_prefill():
    """The history form of the prefill oracle against the plain causal one: the last n - hist rows of a
    full prefill over n tokens are exactly a prefill of those rows over a cache holding all n keys; a
    window at least as long as the context changes nothing, a short one equals attention over the
    truncated key range."""
    g = torch.Generator().manual_seed(0)
    n, hist, page, hkv, hq, D = 50, 20, 16, 2, 4, 64
    k = torch.randn(n, hkv, D, generator=g).bfloat16()
    v = torch.randn(n, hkv, D, generator=g).bfloat16()
    q = torch.randn(n, hq, D, generator=g).bfloat16()
    full = oracle.context_attention(q, k, v, torch.tensor([0]), torch.tensor([n]))
    npg = (n + page - 1) // page
    kc = torch.zeros(npg, page, hkv, D).bfloat16()
    vc = torch.zeros_like(kc)
    kc.view(-1, hkv, D)[:n] = k
    vc.view(-1, hkv, D)[:n] = v
    table = torch.arange(npg)[None]
    args = (q[hist:], kc, vc, table, torch.tensor([0]), torch.tensor([n - hist]), torch.tensor([n]))
    assert torch.equal(oracle.paged_prefill_attention(*args), full[hist:])
    assert torch.equal(oracle.paged_prefill_attention(*args, window_size=n), full[hist:])
    w = 7
    out = oracle.paged_prefill_attention(*args, window_size=w)
    row = n - 1                                   # last query: keys row - w .. row
    # the last query alone over its window, computed directly
    kf = k[row - w:row + 1].transpose(0, 1).repeat_interleave(hq // hkv, 0).float()
    vf = v[row - w:row + 1].transpose(0, 1).repeat_interleave(hq // hkv, 0)
    sc = torch.matmul(q[row].float().unsqueeze(1), kf.transpose(1, 2)) / D ** 0.5
    p = torch.softmax(sc, dim=-1, dtype=torch.float32).to(vf.dtype)
    direct = torch.matmul(p.float(), vf.float()).squeeze(1).to(q.dtype)
    assert torch.equal(out[-1], direct)
