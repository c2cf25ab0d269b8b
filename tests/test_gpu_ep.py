"""Expert-parallel fused_moe on 1, 2, 4 and 8 GPUs against the single-GPU fused_moe (bit-exact), the
failure path of a cross-GPU wait (one GPU, a peer that never signals), and ids outside the expert range."""
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
            # ids outside [0, E) (padding) are sent nowhere and add nothing, step after step (the buffers keep
            # the rows of the steps before)
            ti_pad = ti.clone()
            ti_pad[1::5, 1] = -1
            ti_pad[2::9, 0] = wl.experts + 3
            full_pad = dl.fused_moe(hs, w1, w2, tw, ti_pad, wl.top_k)
            for _ in range(2):
                out3 = ep_moe.ep_fused_moe_peer(pctx, hs[sl], w1[rank * el:(rank + 1) * el].contiguous(),
                                                w2[rank * el:(rank + 1) * el].contiguous(), tw[sl], ti_pad[sl],
                                                wl.top_k)
                torch.cuda.synchronize()
                dl.check_device_status()
                ok = ok and bool(torch.equal(out3, full_pad[sl]))
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


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_many_ranks(cuda_device, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world)


def test_cross_gpu_wait_gives_up_and_reports(cuda_device):
    """A rank whose peer never raises its flag: the barrier kernel runs out of its wait budget, returns,
    and the status word says where.  One GPU stands in for two ranks (both table entries point at the
    same zeroed flag buffer, so the flag of "rank 1" is never written); nothing faults and nothing hangs."""
    import ctypes

    import dlcompiler_b200 as dl
    from dlcompiler_b200 import _lib

    lib = _lib.load()
    dev = cuda_device
    flags = torch.zeros(8 * 16, dtype=torch.int32, device=dev)
    table = (ctypes.c_void_p * 2)(flags.data_ptr(), flags.data_ptr())
    status = _lib.status_word(dev)
    dl.check_device_status()
    _lib.set_wait_budget_ms(50)
    try:
        slot = 3
        with torch.cuda.device(dev):
            rc = lib.dlb_ep_barrier(table, slot, 0, 2, 1, status.data_ptr(), _lib.stream_ptr(dev))
        _lib.check(rc, "ep_barrier")
        torch.cuda.synchronize()
        vals = status.cpu().tolist()
        assert vals[0] == 1 and vals[1] == 42 + slot and vals[2] == 0 and vals[3] == 1
        assert flags[slot * 16 + 0].item() == 1 and flags[slot * 16 + 1].item() == 0
        with pytest.raises(dl.DlblasError):
            dl.check_device_status()
        dl.check_device_status()                     # raised once, then clean
        # the context is still usable
        assert torch.equal(dl.silu_and_mul(torch.ones(4, 16, dtype=torch.bfloat16, device=dev)).cpu(),
                           torch.full((4, 8), 0.73046875, dtype=torch.bfloat16))
    finally:
        _lib.set_wait_budget_ms(2000)
