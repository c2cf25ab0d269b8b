"""The allocation-free decode entry point (collected last on purpose: a failure here cannot
hide the result of any other test in a run that stops at the first failure).

Some users of the library cannot allocate device memory around a decode step: their memory
pool was given to the KV cache at start-up, or the token loop must not enter the allocator.
`dlb_paged_decode_static` serves them with a fixed workspace inside the library; this test
checks, through the C ABI, that it returns exactly what the regular entry point returns, on two
consecutive calls (the second call reuses the workspace the first one left dirty), and that an
oversized request is refused instead of overrunning the workspace.
"""
import pytest
import torch

from dlcompiler_b200 import _lib, paged_attention_fwd
from dlcompiler_b200 import workloads as W
from dlcompiler_b200.kernels.paged_attention_static import paged_decode_no_alloc

pytestmark = pytest.mark.gpu


def _inputs(dev, seed, batch, lo, hi):
    wl = W.DecodeWorkload(batch=batch, ctx_lo=lo, ctx_hi=hi, page=64, hq=32, hkv=8, head_dim=128, seed=seed)
    d = wl.make()
    return {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in d.items()}


def _regular(d):
    q = d["q"]
    o = torch.full_like(q, float("nan"))
    B = q.shape[0]
    paged_attention_fwd(q, d["k_cache"], d["v_cache"], o, d["block_table"], torch.arange(B, device=q.device),
                        torch.ones(B, dtype=torch.int64, device=q.device), d["kv_seqlens"], 1)
    return o


def test_static_scratch_decode_matches_regular_entry_point_twice(cuda_device):
    first = _inputs(cuda_device, seed=40, batch=6, lo=500, hi=9000)     # several splits per sequence
    second = _inputs(cuda_device, seed=41, batch=3, lo=1, hi=3000)      # fewer, shorter: stale partials remain
    for d in (first, second):
        expect = _regular(d)
        before = torch.cuda.memory_allocated(cuda_device)
        out = torch.full_like(d["q"], float("nan"))
        torch.cuda.synchronize()
        paged_decode_no_alloc(d["q"], d["k_cache"], d["v_cache"], out, d["block_table"], d["kv_seqlens"])
        torch.cuda.synchronize()
        # same kernels, same split plan: the tolerance the decode tests use is met with zero slack
        torch.testing.assert_close(out.float(), expect.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(out, expect)
        assert torch.cuda.memory_allocated(cuda_device) <= before + out.numel() * out.element_size()


def test_static_scratch_decode_as_the_first_call_of_a_process(cuda_device):
    """In a fresh process, with no other library call before it, the entry point must still allocate
    nothing (not even the status word the other wrappers create on first use)."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = """
import torch
from dlcompiler_b200 import workloads as W
from dlcompiler_b200.kernels.paged_attention_static import paged_decode_no_alloc
dev = torch.device("cuda:0")
d = W.DecodeWorkload(batch=3, ctx_lo=200, ctx_hi=5000, page=64, seed=42).make()
d = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in d.items()}
out = torch.full_like(d["q"], float("nan"))
torch.cuda.synchronize()
before = torch.cuda.memory_allocated(dev)
paged_decode_no_alloc(d["q"], d["k_cache"], d["v_cache"], out, d["block_table"], d["kv_seqlens"])
torch.cuda.synchronize()
assert torch.cuda.memory_allocated(dev) == before, "the call allocated device memory"
assert torch.isfinite(out.float()).all()
from dlcompiler_b200 import paged_attention_fwd
exp = torch.full_like(out, float("nan"))
B = out.shape[0]
paged_attention_fwd(d["q"], d["k_cache"], d["v_cache"], exp, d["block_table"], torch.arange(B, device=dev),
                    torch.ones(B, dtype=torch.int64, device=dev), d["kv_seqlens"], 1)
assert torch.equal(out, exp)
print("first-call ok")
"""
    res = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "first-call ok" in res.stdout, res.stdout + res.stderr


def test_static_scratch_rejects_oversized_requests(cuda_device):
    lib = _lib.load()
    too_many_splits = 4096
    assert lib.dlb_paged_decode_workspace_floats(64, 32, 128, too_many_splits) > _lib.DECODE_STATIC_FLOATS
    rc = lib.dlb_paged_decode_static(1, 1, 1, 1, 1, 1, 64, 32, 8, 128, 64, 16, 16, 4096, 128, 4096, 128, 1, 1, 1, 1, 1,
                                     1, 16, 0, 0, 64, too_many_splits, -1, 1.0, -1.0, _lib.DTYPE_BF16, None, None)
    assert rc == -5
    assert b"static" in lib.dlb_last_error()
