"""Benchmark of the dlBLAS hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--ops all|none]
    python bench.py --profile-case {silu,gating,moe,moe_c3,moe_c3_unit,prefill,prefill_c4,decode,decode_p1,rotary,rotary_c4} [--steps N]

Headline (one JSON line on stdout): fused_moe on the Mixtral-like configuration
(T=4096, H=4096, I=14336, E=8, top_k=2, bf16) in TFLOP/s, whole job.  N > 1 runs the
same total workload expert-parallel (tokens and experts sharded over the ranks, all-to-all
dispatch/combine), so scaling is strong.  The line also carries, under "ops", the other
four configurations (silu_and_mul, grouped gating, varlen prefill, paged decode) with
their own roofline fractions, measured at N=1.

`--impl reference` times the CPU checker (the torch restatement of the reference's own
test ground truth, oracle/dlblas_oracle.py) on the host cores, every step one pass over all 4096
tokens of the same configuration.

`--profile-case` runs one op a few times on a profiler-sized case (inputs larger than L2, a few GB at
most) and prints one line on stderr; it is the command an `ncu -k regex:<kernel> -c <n>` capture wraps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch at the benchmark shapes, from ncu captures of the
# kernels as they are in this tree (a capture on a smaller case is scaled by the units one launch
# processes); None where the kernel changed after its last capture.
NCU_TRAFFIC = {
    "grouped_gemm": {"gate_up_silu": 2968.7e6, "down_scatter": 1468.0e6, "per_step": 4436.7e6},
    "silu_and_mul": 229.0e6,
    "flash_prefill": 635.1e6,
    "paged_decode": 4430.5e6,
    "rms_norm": 480.8e6,
    "apply_rotary_pos_emb": 630.4e6,
    "fill_kv_cache": 221.9e6,
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["basis"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["basis"] = "fallback"
    return d


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.rows = []
        self.proc = None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            ident = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            ident = str(device_index)
        self.cmd = ["nvidia-smi", "-i", ident, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                    "-lms", "20"]

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def wait_first(self, limit_s=15.0):
        """Blocks until the first sample has arrived (nvidia-smi takes a second or more to start on a box
        with many GPUs), so that a short timed region is not over before sampling begins."""
        t0 = time.perf_counter()
        while self.proc is not None and not self.rows and time.perf_counter() - t0 < limit_s:
            time.sleep(0.02)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------- helpers
def time_steps(fn, steps, warmup, barrier=None, min_warm_s=0.0):
    """W untimed steps (repeated until at least `min_warm_s` seconds of load have passed, so that the
    clock sampler sees the device under load), then K steps between CUDA events on the current stream;
    returns (ms per step, warm-up steps actually run)."""
    t0 = time.perf_counter()
    done = 0
    while done < warmup or time.perf_counter() - t0 < min_warm_s:
        fn()
        done += 1
        if done % 8 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    return start.elapsed_time(end) / steps, done


def time_op(fn, steps, warmup, min_warm_s=0.0):
    return time_steps(fn, steps, warmup, min_warm_s=min_warm_s)[0]


# tensor-bound ops are timed in the same regime as the headline and as the sustained cuBLAS peak they are
# compared with: the device is loaded with the op itself for this long before the timed launches
TENSOR_OP_WARM_S = 0.5


class GemmLaunchTimer:
    """Brackets every grouped-GEMM launch of the library with a pair of CUDA events while installed, so
    that the dominant kernel is timed inside the steps, on the stream it is launched on.  The library's
    public functions stay free of timing arguments: the two launch sites are wrapped from here."""

    def __init__(self):
        self.pairs = []

    def _wrap(self, fn):
        def timed(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **kw)
            e1.record()
            self.pairs.append((e0, e1))
            return r
        return timed

    def __enter__(self):
        from dlcompiler_b200 import _lib
        from dlcompiler_b200.kernels import fused_moe as fm

        self._fm, self._lib = fm, _lib.load()
        self._orig_gemm = fm._grouped_gemm
        self._orig_sync = self._lib.dlb_moe_grouped_gemm_sync
        fm._grouped_gemm = self._wrap(self._orig_gemm)
        self._lib.dlb_moe_grouped_gemm_sync = self._wrap(self._orig_sync)
        return self

    def __exit__(self, *exc):
        self._fm._grouped_gemm = self._orig_gemm
        self._lib.dlb_moe_grouped_gemm_sync = self._orig_sync

    def ms_per_step(self, steps, launches_per_step=2):
        timed = self.pairs[-launches_per_step * steps:]
        return sum(a.elapsed_time(b) for a, b in timed) / steps


class PipelinedE2E:
    """End-to-end step with host buffers, double-buffered the way a serving loop would run it:
    the pinned-host -> device copy of a step's inputs and the device -> pinned-host copy of its result run
    on their own streams, so they overlap the compute of the neighbouring steps.  Every step still copies
    all of its inputs in and its result out inside the timed region."""

    def __init__(self, host_inputs, compute, out_shape, out_dtype, dev):
        self.host_inputs = [t.pin_memory() for t in host_inputs]
        self.dev_inputs = [[torch.empty(t.shape, dtype=t.dtype, device=dev) for t in host_inputs] for _ in range(2)]
        self.out_h = [torch.empty(out_shape, dtype=out_dtype).pin_memory() for _ in range(2)]
        self.compute = compute
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_comp = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]
        self.i = 0
        self.h2d = sum(t.numel() * t.element_size() for t in host_inputs)
        self.d2h = self.out_h[0].numel() * self.out_h[0].element_size()

    def step(self):
        b = self.i & 1
        main = torch.cuda.current_stream()
        with torch.cuda.stream(self.s_in):
            if self.i >= 2:
                self.s_in.wait_event(self.ev_comp[b])        # the compute that last read these device inputs
            for d, h in zip(self.dev_inputs[b], self.host_inputs):
                d.copy_(h, non_blocking=True)
            self.ev_in[b].record(self.s_in)
        main.wait_event(self.ev_in[b])
        out = self.compute(*self.dev_inputs[b])
        self.ev_comp[b].record(main)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_comp[b])
            self.out_h[b].copy_(out, non_blocking=True)
            out.record_stream(self.s_out)
            self.ev_out[b].record(self.s_out)
        self.i += 1

    def drain(self):
        torch.cuda.current_stream().wait_stream(self.s_out)
        torch.cuda.current_stream().wait_stream(self.s_in)


def time_pipelined(pipe, steps, warmup, barrier=None, min_warm_s=0.0):
    """Same regime as `time_steps`: W warm-up steps, repeated until `min_warm_s` seconds of load."""
    t0 = time.perf_counter()
    done = 0
    while done < warmup or time.perf_counter() - t0 < min_warm_s:
        pipe.step()
        done += 1
        if done % 8 == 0:
            torch.cuda.synchronize()
    pipe.drain()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    pipe.s_in.wait_event(start)
    for _ in range(steps):
        pipe.step()
    pipe.drain()                       # the last result has reached host memory before the end event
    end.record()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    return start.elapsed_time(end) / steps, done


# --------------------------------------------------------------------------- per-op benches (N = 1)
def bench_silu(dev, peaks, steps, warmup):
    import dlcompiler_b200 as dl
    from dlcompiler_b200 import workloads as W

    wl = W.SiluWorkload()
    x = wl.make()["gate_up"].to(dev)
    out = torch.empty(wl.tokens, wl.hidden, dtype=x.dtype, device=dev)
    ms = time_op(lambda: dl.silu_and_mul(x, out), steps, warmup)   # 270 MB per pass > 126 MB L2
    gbs = wl.bytes() / ms / 1e6
    return {"workload": "C1 silu_and_mul bf16 [4096, 2x11008]", "ms": ms, "value": gbs, "unit": "GB/s",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC["silu_and_mul"],
                         "basis": peaks["basis"]},
            "l2": "working set 270 MB > L2", "gpu_launches": steps}


def bench_gating(dev, peaks, steps, warmup):
    import dlcompiler_b200 as dl
    from dlcompiler_b200 import workloads as W

    wl = W.GatingWorkload()
    d = wl.make()
    nbuf = 16                                    # 16 x 17.8 MB rotating sets > 126 MB L2
    logits = [d["logits"].to(dev).clone() for _ in range(nbuf)]
    bias = d["bias"].to(dev)

    def sweep():
        for i in range(nbuf):
            dl.grouped_topk_gating(logits[i], bias, wl.top_k, wl.n_group, wl.topk_group, wl.scale_factor)

    # A 2-3 us kernel is launch-bound from Python: replay the 16-launch sweep from a CUDA graph so the
    # number is the kernel's, with cold (HBM-resident) inputs for every launch.
    sweep()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sweep()
    reps = max(steps, 20)
    ms = time_op(graph.replay, reps, max(warmup, 3)) / nbuf
    gbs = wl.bytes() / ms / 1e6
    return {"workload": "C2 grouped sigmoid gating fp32 [16384, 256] top-8", "ms": ms, "value": gbs, "unit": "GB/s",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": None, "basis": peaks["basis"]},
            "l2": "16 rotating input sets (285 MB) > L2, launches replayed from a CUDA graph",
            "gpu_launches": reps * nbuf}


def bench_prefill(dev, peaks, steps, warmup):
    import dlcompiler_b200 as dl
    from dlcompiler_b200 import workloads as W

    wl = W.PrefillWorkload()
    d = wl.make()
    q, k, v = d["q"].to(dev), d["k"].to(dev), d["v"].to(dev)
    o = torch.empty_like(q)
    lse = torch.empty(wl.hq, q.shape[0], dtype=torch.float32, device=dev)
    st, ln = d["b_start_loc"].to(dev), d["b_seq_len"].to(dev)
    run = lambda: dl.context_attention_fwd(q, k, v, o, st, ln, d["max_input_len"], lse=lse)
    ms_short = time_op(run, steps, warmup)                     # a short run from an idle device: burst clocks
    ms = time_op(run, steps, warmup, TENSOR_OP_WARM_S)
    tf = wl.flops() / ms / 1e9
    tf_short = wl.flops() / ms_short / 1e9
    return {"workload": "C4 varlen causal GQA prefill bf16 B=4 S=8192 Hq=32 Hkv=8 D=128", "ms": ms, "value": tf,
            "unit": "TFLOP/s", "regime": f"after {TENSOR_OP_WARM_S} s of the same launches (sustained clocks)",
            "short_run": {"ms": ms_short, "value": tf_short, "frac_of_burst_peak": tf_short / peaks["bf16_tflops"],
                          "regime": "first launches on an idle device, against the burst cuBLAS figure"},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16_tflops_sustained"], "traffic": NCU_TRAFFIC["flash_prefill"],
                         "basis": peaks["basis"]},
            "l2": "q/k/v/o 670 MB > L2", "gpu_launches": steps}


def bench_decode(dev, peaks, steps, warmup):
    import dlcompiler_b200 as dl
    from dlcompiler_b200 import workloads as W

    wl = W.DecodeWorkload()
    d = wl.make(device=dev)
    q = d["q"].to(dev)
    o = torch.empty_like(q)
    table, lens = d["block_table"].to(dev), d["kv_seqlens"].to(dev)
    qs = torch.arange(wl.batch, device=dev)
    ql = torch.ones(wl.batch, dtype=torch.int64, device=dev)
    ms = time_op(lambda: dl.paged_attention_fwd(q, d["k_cache"], d["v_cache"], o, table, qs, ql, lens, 1), steps,
                    warmup)
    nbytes = wl.bytes(d["kv_seqlens"])
    gbs = nbytes / ms / 1e6
    return {"workload": f"C5 paged decode bf16 B=64 ctx U[1024,32768] page 64 (ctx_sum={int(d['kv_seqlens'].sum())})",
            "ms": ms, "value": gbs, "unit": "GB/s", "tflops": wl.flops(d["kv_seqlens"]) / ms / 1e9,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC["paged_decode"],
                         "basis": peaks["basis"]},
            "l2": "KV cache 4.4 GB > L2", "gpu_launches": 2 * steps}


def _hbm_entry(workload, nbytes, ms, peaks, launches, note):
    gbs = nbytes / ms / 1e6
    return {"workload": workload, "ms": ms, "value": gbs, "unit": "GB/s",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": None, "basis": peaks["basis"]},
            "l2": note, "gpu_launches": launches}


def bench_neighbours(dev, peaks, steps, warmup):
    """The steps either side of the hot path (rms_norm, rotary, fill_kv_cache, token-granular decode)."""
    import dlcompiler_b200 as dl
    from dlcompiler_b200 import workloads as W

    out = {}
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    # rms_norm with residual: 4 tensors of [16384, 4096] bf16 move per pass
    T, H = 16384, 4096
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    r = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    w = torch.rand(H, generator=g, device=dev).to(torch.bfloat16)
    o, o_r = torch.empty_like(x), torch.empty_like(x)
    ms = time_op(lambda: dl.rms_norm(x, w, 1e-6, residual=r, out=o, out_residual=o_r), steps, warmup)
    out["rms_norm"] = _hbm_entry("rms_norm + residual bf16 [16384, 4096]", 4 * T * H * 2 + H * 2, ms, peaks, steps,
                                 "537 MB per pass > L2")
    out["rms_norm"]["roofline"]["traffic"] = NCU_TRAFFIC["rms_norm"]
    del x, r, o, o_r
    # rotary embedding of the prefill configuration's q and k
    tok, hq, hk, d = 32768, 32, 8, 128
    q = torch.randn(tok, hq, d, generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn(tok, hk, d, generator=g, device=dev).to(torch.bfloat16)
    cos = torch.rand(tok, d, generator=g, device=dev).to(torch.bfloat16)
    sin = torch.rand(tok, d, generator=g, device=dev).to(torch.bfloat16)
    # (into separate outputs: q and k keep their N(0, 1) values for the paged prefill below)
    q_rot, k_rot = torch.empty_like(q), torch.empty_like(k)
    ms = time_op(lambda: dl.apply_rotary_pos_emb(q, k, cos, sin, q_rot, k_rot), steps, warmup)
    del q_rot, k_rot
    out["apply_rotary_pos_emb"] = _hbm_entry("rotary, q [32768, 32, 128] k [32768, 8, 128] bf16 -> rotated copies",
                                             2 * (q.numel() + k.numel()) * 2 + 2 * cos.numel() * 2, ms, peaks, steps,
                                             "688 MB per pass > L2")
    out["apply_rotary_pos_emb"]["roofline"]["traffic"] = NCU_TRAFFIC["apply_rotary_pos_emb"]
    # fill_kv_cache: the prefill configuration's 4 x 8192 new tokens into 64-token pages
    B, S, page = 4, 8192, 64
    pages = B * S // page
    kc = torch.empty(pages, page, hk, d, dtype=torch.bfloat16, device=dev)
    vc = torch.empty_like(kc)
    table = torch.randperm(pages, generator=g, device=dev).to(torch.int32).view(B, S // page)
    qlen = torch.full((B,), S, dtype=torch.int32, device=dev)
    start = torch.arange(B, dtype=torch.int32, device=dev) * S
    v_states = torch.randn(tok, hk, d, generator=g, device=dev).to(torch.bfloat16)
    ms = time_op(lambda: dl.fill_kv_cache(k, v_states, kc, vc, start, qlen, qlen, S, table), steps, warmup)
    out["fill_kv_cache"] = _hbm_entry("fill_kv_cache 4 x 8192 tokens, 8 heads x 128, page 64, bf16",
                                      4 * k.numel() * 2, ms, peaks, steps, "268 MB per pass > L2")
    out["fill_kv_cache"]["roofline"]["traffic"] = NCU_TRAFFIC["fill_kv_cache"]
    # paged prefill: the same 4 x 8192 queries against the cache just filled (no history), page 64
    o_pp = torch.empty_like(q)
    qlen64 = qlen.to(torch.int64)
    start64 = start.to(torch.int64)
    ms = time_op(lambda: dl.paged_attention_fwd(q, kc, vc, o_pp, table, start64, qlen64, qlen64, S), steps, warmup,
                 TENSOR_OP_WARM_S)
    pp_flops = sum(4 * S * S * d * hq // 2 for _ in range(B))
    tf = pp_flops / ms / 1e9
    out["paged_prefill"] = {"workload": "paged_attention_fwd prefill, C4 shape (B=4 S=8192 Hq=32 Hkv=8 D=128) over "
                                        "64-token pages, bf16", "ms": ms, "value": tf, "unit": "TFLOP/s",
                            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops_sustained"],
                                         "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops_sustained"],
                                         "traffic": None, "basis": peaks["basis"]},
                            "l2": "q/cache/o 670 MB > L2", "gpu_launches": steps}
    # the same two steps with the rotary embedding folded in: k rotated while the cache is filled, q rotated on
    # its tile inside the attention kernel (no stand-alone rotary pass is left in this path)
    ms = time_op(lambda: dl.fill_kv_cache(k, v_states, kc, vc, start, qlen, qlen, S, table, cos=cos, sin=sin), steps,
                 warmup)
    out["fill_kv_cache_rotary"] = _hbm_entry("fill_kv_cache rotating k on the way (4 x 8192 tokens, page 64, bf16)",
                                             4 * k.numel() * 2 + 2 * cos.numel() * 2, ms, peaks, steps,
                                             "285 MB per pass > L2")
    ms = time_op(lambda: dl.paged_attention_fwd(q, kc, vc, o_pp, table, start64, qlen64, qlen64, S, q_cos=cos,
                                                q_sin=sin), steps, warmup, TENSOR_OP_WARM_S)
    tf = pp_flops / ms / 1e9
    out["paged_prefill_rotary"] = {"workload": "paged_attention_fwd prefill rotating q inside the kernel, C4 shape over "
                                               "64-token pages, bf16", "ms": ms, "value": tf, "unit": "TFLOP/s",
                                   "roofline": {"bound": "tensor", "achieved": tf,
                                                "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                                                "frac": tf / peaks["bf16_tflops_sustained"], "traffic": None,
                                                "basis": peaks["basis"]},
                                   "l2": "q/cache/o 670 MB > L2", "gpu_launches": steps}
    del q, k, v_states, kc, vc, cos, sin, o_pp
    # token-granular decode (page size 1): 16 requests of the decode configuration
    wl = W.DecodeWorkload(batch=16, page=1)
    dd = wl.make(device=dev)
    qd = dd["q"].to(dev)
    od = torch.empty_like(qd)
    tb, ln = dd["block_table"].to(dev), dd["kv_seqlens"].to(dev)
    kb, vb = dd["k_cache"].squeeze(1), dd["v_cache"].squeeze(1)
    req = torch.arange(wl.batch, device=dev)
    ms = time_op(lambda: dl.decode_attention_fwd(qd, kb, vb, od, tb, req, None, ln, None, tb.size(1), d ** -0.5),
                    steps, warmup)
    out["decode_attention_fwd"] = _hbm_entry(f"decode_attention_fwd (page size 1) B=16 ctx_sum={int(ln.sum())} bf16",
                                             wl.bytes(dd["kv_seqlens"]), ms, peaks, 2 * steps, "KV 1.1 GB > L2")
    return out


# --------------------------------------------------------------------------- CPU baseline
def cpu_fused_moe(sample_tokens, threads=None, budget_s=12.0, max_passes=6):
    """Times the CPU checker's fused_moe (reference test ground truth) on a token sample of C3:
    repeated passes until about `budget_s` seconds of CPU work, best pass reported."""
    from dlcompiler_b200 import workloads as W
    from oracle import dlblas_oracle as oracle

    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    wl = W.MoeWorkload()
    d = wl.make()
    hs = d["hidden_states"][:sample_tokens]
    tw, ti = oracle.softmax_topk(d["router_logits"][:sample_tokens], wl.top_k)
    ti = ti.long()
    oracle.fused_moe(hs[:64], d["w1"], d["w2"], tw[:64], ti[:64])          # warm-up
    best, total, passes = float("inf"), 0.0, 0
    while passes < max_passes and total < budget_s:
        t0 = time.perf_counter()
        oracle.fused_moe(hs, d["w1"], d["w2"], tw, ti)
        dt = time.perf_counter() - t0
        best = min(best, dt)
        total += dt
        passes += 1
    tf = wl.flops(sample_tokens) / best / 1e12
    return tf, best, threads, passes


def run_reference(args):
    """The reference arm: the CPU implementation on the host cores, every step one pass over the same
    configuration as our arm (all 4096 tokens of C3)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        args._stdout_guard.restore()
        return
    from dlcompiler_b200 import workloads as W
    from oracle import dlblas_oracle as oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    wl = W.MoeWorkload()
    d = wl.make()
    hs = d["hidden_states"]
    tw, ti = oracle.softmax_topk(d["router_logits"], wl.top_k)
    ti = ti.long()
    for _ in range(min(args.warmup, 2)):
        oracle.fused_moe(hs, d["w1"], d["w2"], tw, ti)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.fused_moe(hs, d["w1"], d["w2"], tw, ti)
    dt = (time.perf_counter() - t0) / args.steps
    tf = wl.flops() / dt / 1e12
    what = ("all 4096 tokens per step; torch CPU restatement of the reference test ground truth (the "
            "reference's Triton kernels cannot run on CPU)")
    line = {
        "impl": "reference", "metric": "fused_moe_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 2), "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": MOE_WORKLOAD, "sample": "whole workload every step"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": what},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    args._stdout_guard.restore()
    print(json.dumps(line), flush=True)


MOE_WORKLOAD = ("C3 fused_moe T=4096 H=4096 I=14336 E=8 top_k=2 bf16 (moe_align block 128 -> gate/up GEMM+silu -> "
                "down GEMM x weight -> combine)")


_ORIGINAL_AFFINITY = None


def restore_cpu_affinity():
    """Gives the process back every core it started with (the CPU baseline leg uses all of them)."""
    if _ORIGINAL_AFFINITY is not None:
        try:
            os.sched_setaffinity(0, _ORIGINAL_AFFINITY)
        except Exception as exc:  # noqa: BLE001
            print(f"[bench] CPU affinity not restored ({exc!r})", file=sys.stderr)


def bind_to_gpu_cpus(device_index):
    """Runs this rank on the CPU cores next to its GPU (the affinity NVML reports for the device), so that the
    pinned host buffers of the end-to-end leg are first touched, and therefore placed, on the GPU's own NUMA
    node.  Host-side placement only; nothing on the GPU is changed.  Silently skipped where NVML or the
    affinity call is unavailable."""
    try:
        import pynvml

        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(device_index).uuid)
        uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        try:
            handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
        except Exception:  # noqa: BLE001 - older bindings want bytes
            handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1}
        global _ORIGINAL_AFFINITY
        start = os.sched_getaffinity(0)
        cpus &= start
        if cpus:
            _ORIGINAL_AFFINITY = start
            os.sched_setaffinity(0, cpus)
    except Exception as exc:  # noqa: BLE001 - placement is an optimisation, never a requirement
        print(f"[bench] CPU affinity not set ({exc!r})", file=sys.stderr)


# --------------------------------------------------------------------------- headline: fused_moe
def run_ours(args):
    import dlcompiler_b200 as dl
    from dlcompiler_b200 import _lib
    from dlcompiler_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _lib.load()
    peaks = load_peaks()
    wl = W.MoeWorkload()

    # at every N: the pinned buffers of the end-to-end leg belong on the GPU's own NUMA node
    bind_to_gpu_cpus(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        os.environ.setdefault("NCCL_DEBUG", "WARN")     # stdout is redirected anyway; a caller's setting stands
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()

    d = wl.make(weights=False)
    # routing inputs of the step: softmax -> top-2 of the seeded router logits (our router kernel)
    tw_dev, ti_dev = dl.softmax_topk(d["router_logits"].to(dev), wl.top_k)
    tw_cpu, ti_cpu = tw_dev.cpu(), ti_dev.cpu()
    ep_check = None
    timer = GemmLaunchTimer()

    if world == 1:
        wts = wl.make()
        w1, w2 = wts["w1"].to(dev), wts["w2"].to(dev)
        del wts
        hs, tw, ti = d["hidden_states"].to(dev), tw_cpu.to(dev), ti_cpu.to(dev)

        def step():
            return dl.fused_moe(hs, w1, w2, tw, ti, wl.top_k)

        def e2e_compute(h, w, i):
            return dl.fused_moe(h, w1, w2, w, i, wl.top_k)

        host_inputs = [d["hidden_states"], tw_cpu, ti_cpu]
        out_rows = wl.tokens
        launches_per_step = 5
        warm_steps, warm_s = args.warmup, args.warm_seconds
        parallelism = "single GPU"
    else:
        from dlcompiler_b200.distributed import ep_moe

        t_local = wl.tokens // world
        e_local = wl.experts // world
        sl = slice(rank * t_local, (rank + 1) * t_local)
        hs, tw, ti = d["hidden_states"][sl].to(dev), tw_cpu[sl].to(dev), ti_cpu[sl].to(dev)
        wts = wl.make()
        # correctness of the sharded step, outside any timed region: this rank's token slice through the
        # single-GPU fused_moe with ALL experts' weights must give the same bits as the exchange
        w1_all, w2_all = wts["w1"].to(dev), wts["w2"].to(dev)
        expect = dl.fused_moe(hs, w1_all, w2_all, tw, ti, wl.top_k)
        torch.cuda.synchronize()
        del w1_all, w2_all
        torch.cuda.empty_cache()
        w1 = wts["w1"][rank * e_local:(rank + 1) * e_local].to(dev)
        w2 = wts["w2"][rank * e_local:(rank + 1) * e_local].to(dev)
        del wts
        exchange = args.exchange
        if exchange == "peer":
            try:
                ctx = ep_moe.EpPeerContext(dist.group.WORLD, wl.experts, dev, t_local, wl.top_k, wl.hidden, wl.hidden,
                                           wl.inter)
                ep_step = ep_moe.ep_fused_moe_peer
                launches = ep_moe.PEER_KERNELS_PER_STEP
            except Exception as exc:  # symmetric memory unavailable on this box: NCCL exchange instead
                print(f"[bench] peer-memory exchange unavailable ({exc!r}); using the NCCL all-to-all path",
                      file=sys.stderr)
                exchange = "nccl"
        if exchange == "nccl":
            ctx = ep_moe.EpMoeContext(dist.group.WORLD, wl.experts, dev)
            ep_step = ep_moe.ep_fused_moe
            launches = ep_moe.KERNELS_PER_STEP

        def step():
            return ep_step(ctx, hs, w1, w2, tw, ti, wl.top_k)

        def e2e_compute(h, w, i):
            return ep_step(ctx, h, w1, w2, w, i, wl.top_k)

        # three steps in a row (the symmetric buffers are reused from step to step), each compared bit for bit
        same = True
        for _ in range(3):
            got = step()
            torch.cuda.synchronize()
            same = same and bool(torch.equal(got, expect))
        dl.check_device_status()
        flag = torch.tensor([int(same)], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ep_check = {"ranks": world, "bit_identical": bool(flag.item()), "steps_checked": 3,
                    "against": "single-GPU fused_moe on each rank's token slice with all experts' weights"}
        del expect, got
        host_inputs = [d["hidden_states"][sl].contiguous(), tw_cpu[sl].contiguous(), ti_cpu[sl].contiguous()]
        out_rows = t_local
        launches_per_step = launches
        # every rank must run the same number of steps (the ranks meet in cross-GPU waits): a fixed count,
        # long enough for the clocks to settle under load
        warm_steps, warm_s = max(args.warmup, 1000), 0.0
        how = ("dispatch/combine by our own kernels over NVLink peer memory" if exchange == "peer"
               else "NCCL all-to-all dispatch/combine")
        parallelism = f"ep{world}: tokens and experts sharded over {world} ranks, {how}"

    bar = barrier if dist is not None else None
    with ClockSampler(local_rank) as clk:
        # no step may start while a rank still waits for its sampler
        clk.wait_first()
        barrier()
        with timer:
            ms, warm_ran = time_steps(step, args.steps, warm_steps, bar, min_warm_s=warm_s)
        torch.cuda.synchronize()
    gemm_ms = timer.ms_per_step(args.steps)
    clocks = clk.summary()

    # end to end: pinned host inputs -> device -> fused_moe -> host result, every step; same warm-up regime as
    # the device-only loop, with its own clock record
    pipe = PipelinedE2E(host_inputs, e2e_compute, (out_rows, wl.hidden), torch.bfloat16, dev)
    with ClockSampler(local_rank) as clk_e2e:
        clk_e2e.wait_first()
        barrier()
        ms_e2e, warm_ran_e2e = time_pipelined(pipe, args.steps, warm_steps, bar, min_warm_s=warm_s)
    h2d, d2h = pipe.h2d * world, pipe.d2h * world
    dl.check_device_status()
    if dist is not None:
        # max over ranks of the device-timed step
        t = torch.tensor([ms, ms_e2e, gemm_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e, gemm_ms = t.tolist()
    flops = wl.flops()

    tflops = flops / ms / 1e9
    e2e_tflops = flops / ms_e2e / 1e9
    # dominant kernel: the grouped GEMM (two launches per step, both timed with events inside the steps)
    gemm_flops_per_rank = flops / world
    gemm_tf = gemm_flops_per_rank / gemm_ms / 1e9
    peak = peaks["bf16_tflops_sustained"]
    line = {
        "metric": "fused_moe_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm_ran, "warmup_requested": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": MOE_WORKLOAD, "parallelism": parallelism,
                   "l2": "expert weights 2.8 GB per pass > 126 MB L2"},
        "roofline": {"bound": "tensor", "kernel": "grouped_gemm_kernel (2 launches per step)", "achieved": gemm_tf,
                     "peak": peak, "unit": "TFLOP/s", "frac": gemm_tf / peak,
                     "frac_of_burst": gemm_tf / peaks["bf16_tflops"], "frac_of_nominal_2250": gemm_tf / 2250.0,
                     "traffic": NCU_TRAFFIC["grouped_gemm"]["per_step"] / 2 if world == 1 else None,
                     "traffic_by_launch": NCU_TRAFFIC["grouped_gemm"] if world == 1 else None,
                     "basis": f"{peaks['basis']} sustained cuBLAS bf16", "ms_per_step_in_kernel": gemm_ms},
        "e2e": {"value": e2e_tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e, "warmup": warm_ran_e2e, "clocks": clk_e2e.summary(),
                "how": "public API on pinned host buffers; copies double-buffered on side streams so they "
                       "overlap the neighbouring steps' compute"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    if ep_check is not None:
        line["ep_check"] = ep_check
    if rank == 0 and world == 1:
        if args.ops != "none":
            ops = {}
            for name, fn in (("silu_and_mul", bench_silu), ("grouped_gating", bench_gating),
                             ("flash_prefill", bench_prefill), ("paged_decode", bench_decode)):
                torch.cuda.empty_cache()
                ops[name] = fn(dev, peaks, max(args.steps, 10), max(args.warmup, 3))
            dl.check_device_status()
            line["ops"] = ops
            torch.cuda.empty_cache()
            line["ops_next"] = bench_neighbours(dev, peaks, max(args.steps, 10), max(args.warmup, 3))
            dl.check_device_status()
        if args.cpu_baseline:
            del w1, w2
            torch.cuda.empty_cache()
            restore_cpu_affinity()
            tf, secs, cores, passes = cpu_fused_moe(args.cpu_sample)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": f"first {args.cpu_sample} of 4096 tokens, best of {passes} passes "
                                              f"({secs:.2f} s each); torch CPU restatement of the reference test "
                                              "ground truth"}
    args._stdout_guard.restore()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------- profiler-sized cases
def run_profile_case(args):
    """One op, a few launches, on a case sized for an `ncu` capture: inputs larger than L2, a few GB on the
    device at most."""
    import dlcompiler_b200 as dl
    from dlcompiler_b200 import workloads as W

    dev = torch.device("cuda:0")
    op = args.profile_case
    if op == "silu":
        x = W.SiluWorkload().make()["gate_up"].to(dev)                 # the benchmark shape: 270 MB
        fn = lambda: dl.silu_and_mul(x)
        what = "silu_and_mul bf16 [4096, 2x11008]"
    elif op == "gating":
        wl = W.GatingWorkload(tokens=16384 * 8)                        # 134 MB of logits > L2
        d = wl.make()
        lg, b = d["logits"].to(dev), d["bias"].to(dev)
        fn = lambda: dl.grouped_topk_gating(lg, b, wl.top_k, wl.n_group, wl.topk_group, wl.scale_factor)
        what = "grouped gating fp32 [131072, 256]"
    elif op == "moe":
        wl = W.MoeWorkload(tokens=2048, hidden=4096, inter=7168, experts=4, top_k=2)   # 0.7 GB of weights
        d = wl.make()
        tw, ti = dl.softmax_topk(d["router_logits"].to(dev), wl.top_k)
        hs, w1, w2 = d["hidden_states"].to(dev), d["w1"].to(dev), d["w2"].to(dev)
        fn = lambda: dl.fused_moe(hs, w1, w2, tw, ti, wl.top_k)
        what = "fused_moe T=2048 H=4096 I=7168 E=4 top_k=2 bf16"
    elif op in ("moe_c3", "moe_c3_unit"):
        # the benchmark shape itself, for one-pass DRAM counters: weights drawn on the device with the benchmark's
        # standard deviation (0.02) or with unit variance (the grouped GEMM's clock under the power cap, and
        # with it its DRAM re-reads, depend on the operand values)
        wl = W.MoeWorkload()
        d = wl.make(weights=False)
        std = 0.02 if op == "moe_c3" else 1.0
        g = torch.Generator(device=dev)
        g.manual_seed(11)
        w1 = (torch.randn(wl.experts, 2 * wl.inter, wl.hidden, generator=g, device=dev) * std).to(torch.bfloat16)
        w2 = (torch.randn(wl.experts, wl.hidden, wl.inter, generator=g, device=dev) * std).to(torch.bfloat16)
        tw, ti = dl.softmax_topk(d["router_logits"].to(dev), wl.top_k)
        hs = d["hidden_states"].to(dev)
        fn = lambda: dl.fused_moe(hs, w1, w2, tw, ti, wl.top_k)
        what = f"fused_moe C3 shape, weights N(0, {std}^2) bf16"
    elif op in ("prefill", "prefill_c4"):
        # q/k/v/o 168 MB > L2; prefill_c4 is the benchmark shape itself (670 MB), for one-pass DRAM counters
        wl = W.PrefillWorkload(batch=2, seq_len=4096) if op == "prefill" else W.PrefillWorkload()
        d = wl.make()
        q, k, v = d["q"].to(dev), d["k"].to(dev), d["v"].to(dev)
        o = torch.empty_like(q)
        st, ln = d["b_start_loc"].to(dev), d["b_seq_len"].to(dev)
        fn = lambda: dl.context_attention_fwd(q, k, v, o, st, ln, d["max_input_len"])
        what = f"prefill B={wl.batch} S={wl.seq_len} Hq=32 Hkv=8 D=128 bf16"
    elif op in ("rotary", "rotary_c4"):
        # q + k 84 MB in, 84 MB out, cos/sin 4 MB; rotary_c4: the benchmark's 32768 tokens (688 MB per pass)
        tok, hq, hk, dd = (8192 if op == "rotary" else 32768), 32, 8, 128
        g = torch.Generator(device=dev)
        g.manual_seed(7)
        q = torch.randn(tok, hq, dd, generator=g, device=dev).to(torch.bfloat16)
        k = torch.randn(tok, hk, dd, generator=g, device=dev).to(torch.bfloat16)
        cos = torch.rand(tok, dd, generator=g, device=dev).to(torch.bfloat16)
        sin = torch.rand(tok, dd, generator=g, device=dev).to(torch.bfloat16)
        fn = lambda: dl.apply_rotary_pos_emb(q, k, cos, sin, q, k)
        what = f"rotary in place q [{tok}, 32, 128] k [{tok}, 8, 128] bf16"
    elif op == "decode_p1":
        wl = W.DecodeWorkload(batch=16, page=1)                        # token-granular cache, ~1.1 GB
        d = wl.make(device=dev)
        q = d["q"].to(dev)
        o = torch.empty_like(q)
        tb, ln = d["block_table"].to(dev), d["kv_seqlens"].to(dev)
        kb, vb = d["k_cache"].squeeze(1), d["v_cache"].squeeze(1)
        req = torch.arange(wl.batch, device=dev)
        fn = lambda: dl.decode_attention_fwd(q, kb, vb, o, tb, req, None, ln, None, tb.size(1), q.size(-1) ** -0.5)
        what = f"decode_attention_fwd B=16 ctx_sum={int(d['kv_seqlens'].sum())} page 1 bf16"
    else:
        wl = W.DecodeWorkload(batch=16)                                # ~1.1 GB of KV cache
        d = wl.make(device=dev)
        q = d["q"].to(dev)
        o = torch.empty_like(q)
        tb, ln = d["block_table"].to(dev), d["kv_seqlens"].to(dev)
        qs, ql = torch.arange(wl.batch, device=dev), torch.ones(wl.batch, dtype=torch.int64, device=dev)
        fn = lambda: dl.paged_attention_fwd(q, d["k_cache"], d["v_cache"], o, tb, qs, ql, ln, 1)
        what = f"paged decode B=16 ctx_sum={int(d['kv_seqlens'].sum())} page 64 bf16"
    iters = max(1, min(args.steps, 8))
    for _ in range(iters):
        fn()
    torch.cuda.synchronize()
    dl.check_device_status()
    args._stdout_guard.restore()
    print(f"profile case {op}: {what}, {iters} iterations", file=sys.stderr)


class _StdoutToStderr:
    """Libraries (NCCL) print banners on stdout; the contract is ONE JSON line there.  Everything
    written to file descriptor 1 goes to stderr until `restore()`."""

    def __init__(self):
        sys.stdout.flush()
        self._saved = os.dup(1)
        os.dup2(2, 1)

    def restore(self):
        sys.stdout.flush()
        os.dup2(self._saved, 1)
        os.close(self._saved)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ops", default="all", choices=["all", "none"])
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: token exchange by our peer-memory kernels (default) or by NCCL all-to-all")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    ap.add_argument("--cpu-sample", type=int, default=4096)
    ap.add_argument("--warm-seconds", type=float, default=1.0,
                    help="N = 1: keep warming up until this much wall time has passed (device under load)")
    ap.add_argument("--profile-case", default=None, choices=["silu", "gating", "moe", "moe_c3", "moe_c3_unit", "prefill", "prefill_c4", "decode", "decode_p1", "rotary", "rotary_c4"],
                    help="run one op --steps times (at most 8) on a profiler-sized case and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    guard = _StdoutToStderr()
    args._stdout_guard = guard
    if args.profile_case is not None:
        if "--steps" not in sys.argv:
            args.steps = 2
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
