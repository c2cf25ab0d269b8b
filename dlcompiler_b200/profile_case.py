"""Run one hot-path op a few times on a profiler-sized case (inputs larger than L2, a few GB at most).

    python -m dlcompiler_b200.profile_case {silu,gating,moe,prefill,decode} [--iters N]

Meant to be wrapped by `ncu -k regex:<kernel> -c <n>`; it prints nothing but a one-line summary.
"""
from __future__ import annotations

import argparse

import torch

import dlcompiler_b200 as dl
from dlcompiler_b200 import workloads as W


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["silu", "gating", "moe", "prefill", "decode"])
    ap.add_argument("--iters", type=int, default=2)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    if a.op == "silu":
        x = W.SiluWorkload().make()["gate_up"].to(dev)                 # the benchmark shape: 270 MB
        fn = lambda: dl.silu_and_mul(x)
        what = "silu_and_mul bf16 [4096, 2x11008]"
    elif a.op == "gating":
        wl = W.GatingWorkload(tokens=16384 * 8)                        # 134 MB of logits > L2
        d = wl.make()
        lg, b = d["logits"].to(dev), d["bias"].to(dev)
        fn = lambda: dl.grouped_topk_gating(lg, b, wl.top_k, wl.n_group, wl.topk_group, wl.scale_factor)
        what = "grouped gating fp32 [131072, 256]"
    elif a.op == "moe":
        wl = W.MoeWorkload(tokens=2048, hidden=4096, inter=7168, experts=4, top_k=2)   # 0.7 GB of weights
        d = wl.make()
        tw, ti = dl.softmax_topk(d["router_logits"].to(dev), wl.top_k)
        hs, w1, w2 = d["hidden_states"].to(dev), d["w1"].to(dev), d["w2"].to(dev)
        fn = lambda: dl.fused_moe(hs, w1, w2, tw, ti, wl.top_k)
        what = "fused_moe T=2048 H=4096 I=7168 E=4 top_k=2 bf16"
    elif a.op == "prefill":
        wl = W.PrefillWorkload(batch=2, seq_len=4096)                  # q/k/v/o 168 MB > L2
        d = wl.make()
        q, k, v = d["q"].to(dev), d["k"].to(dev), d["v"].to(dev)
        o = torch.empty_like(q)
        st, ln = d["b_start_loc"].to(dev), d["b_seq_len"].to(dev)
        fn = lambda: dl.context_attention_fwd(q, k, v, o, st, ln, d["max_input_len"])
        what = "prefill B=2 S=4096 Hq=32 Hkv=8 D=128 bf16"
    else:
        wl = W.DecodeWorkload(batch=16)                                # ~1.1 GB of KV cache
        d = wl.make(device=dev)
        q = d["q"].to(dev)
        o = torch.empty_like(q)
        tb, ln = d["block_table"].to(dev), d["kv_seqlens"].to(dev)
        qs, ql = torch.arange(wl.batch, device=dev), torch.ones(wl.batch, dtype=torch.int64, device=dev)
        fn = lambda: dl.paged_attention_fwd(q, d["k_cache"], d["v_cache"], o, tb, qs, ql, ln, 1)
        what = f"paged decode B=16 ctx_sum={int(d['kv_seqlens'].sum())} page 64 bf16"
    for _ in range(a.iters):
        fn()
    torch.cuda.synchronize()
    dl.check_device_status()
    print(f"profile_case {a.op}: {what}, {a.iters} iterations")


if __name__ == "__main__":
    main()
