"""Expert-parallel fused_moe on GPUs through NCCL, against the single-GPU fused_moe (bit-exact)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import dlcompiler_b200 as dl
    from dlcompiler_b200 import workloads as W
    from dlcompiler_b200.distributed import ep_moe

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        wl = W.MoeWorkload(tokens=512, hidden=512, inter=768, experts=8, top_k=2)
        d = wl.make()
        hs, w1, w2 = d["hidden_states"].to(dev), d["w1"].to(dev), d["w2"].to(dev)
        tw, ti = dl.softmax_topk(d["router_logits"].to(dev), wl.top_k)
        full = dl.fused_moe(hs, w1, w2, tw, ti, wl.top_k)
        ctx = ep_moe.EpMoeContext(dist.group.WORLD, wl.experts, dev)
        tl, el = wl.tokens // world, wl.experts // world
        sl = slice(rank * tl, (rank + 1) * tl)
        out = ep_moe.ep_fused_moe(ctx, hs[sl], w1[rank * el:(rank + 1) * el].contiguous(),
                                  w2[rank * el:(rank + 1) * el].contiguous(), tw[sl], ti[sl], wl.top_k)
        torch.cuda.synchronize()
        dl.check_device_status()
        ok = bool(torch.equal(out, full[sl]))
        # the peer-memory exchange (our own kernels over NVLink) must give the same bits, step after step,
        # whether the results are pulled by the combine or pushed by the down GEMM's epilogue (None: context decides)
        for pull in (True, False, None):
            pctx = ep_moe.EpPeerContext(dist.group.WORLD, wl.experts, dev, tl, wl.top_k, wl.hidden, wl.hidden,
                                        wl.inter, pull=pull)
            for _ in range(3):
                out2 = ep_moe.ep_fused_moe_peer(pctx, hs[sl], w1[rank * el:(rank + 1) * el].contiguous(),
                                                w2[rank * el:(rank + 1) * el].contiguous(), tw[sl], ti[sl], wl.top_k)
                torch.cuda.synchronize()
                dl.check_device_status()
                ok = ok and bool(torch.equal(out2, full[sl]))
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def _run(world):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {r: True for r in range(world)}


def test_ep_single_rank_group(cuda_device):
    _run(1)


def test_ep_two_ranks(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(2)
