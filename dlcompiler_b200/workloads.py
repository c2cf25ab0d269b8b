"""Seeded synthetic workloads for the five hot-path configurations and their algorithmic work.

Inputs are generated on the CPU with per-tensor `torch.Generator` seeds so the CUDA kernels
and the CPU checker see identical bits on every machine.  `scale` (0 < scale <= 1) shrinks
the token / batch dimension for parity tests; scale = 1 is the full benchmark size.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def _randn(shape, seed, dtype=torch.float32, std=1.0):
    x = torch.randn(shape, generator=_gen(seed), dtype=torch.float32)
    if std != 1.0:
        x = x * std
    return x.to(dtype)


# ------------------------------------------------------------------ C1: silu_and_mul
@dataclass
class SiluWorkload:
    tokens: int = 4096
    hidden: int = 11008
    dtype: torch.dtype = torch.bfloat16
    seed: int = 0

    def make(self):
        return {"gate_up": _randn((self.tokens, 2 * self.hidden), self.seed * 100, self.dtype)}

    def bytes(self) -> int:
        es = torch.empty(0, dtype=self.dtype).element_size()
        return self.tokens * 3 * self.hidden * es


# ------------------------------------------------------------------ C2: grouped gating
@dataclass
class GatingWorkload:
    tokens: int = 16384
    experts: int = 256
    n_group: int = 8
    topk_group: int = 4
    top_k: int = 8
    scale_factor: float = 2.5
    seed: int = 1

    def make(self):
        return {
            "logits": _randn((self.tokens, self.experts), self.seed * 100),
            "bias": _randn((self.experts,), self.seed * 100 + 1, std=0.01),
        }

    def bytes(self) -> int:
        return self.tokens * self.experts * 4 + self.experts * 4 + 2 * self.tokens * self.top_k * 4


# ------------------------------------------------------------------ C3: fused_moe
@dataclass
class MoeWorkload:
    tokens: int = 4096
    hidden: int = 4096
    inter: int = 14336
    experts: int = 8
    top_k: int = 2
    dtype: torch.dtype = torch.bfloat16
    seed: int = 2

    def make(self, weights: bool = True):
        d = {
            "hidden_states": _randn((self.tokens, self.hidden), self.seed * 100, self.dtype),
            "router_logits": _randn((self.tokens, self.experts), self.seed * 100 + 1),
        }
        if weights:
            d["w1"] = _randn((self.experts, 2 * self.inter, self.hidden), self.seed * 100 + 2, self.dtype, std=0.02)
            d["w2"] = _randn((self.experts, self.hidden, self.inter), self.seed * 100 + 3, self.dtype, std=0.02)
        return d

    def flops(self, tokens: int | None = None) -> int:
        t = self.tokens if tokens is None else tokens
        return 2 * t * self.top_k * 3 * self.inter * self.hidden


# ------------------------------------------------------------------ C4: varlen prefill
@dataclass
class PrefillWorkload:
    batch: int = 4
    seq_len: int = 8192
    hq: int = 32
    hkv: int = 8
    head_dim: int = 128
    dtype: torch.dtype = torch.bfloat16
    seed: int = 3
    seq_lens: list = field(default_factory=list)    # overrides batch x seq_len when given

    def lens(self):
        return list(self.seq_lens) if self.seq_lens else [self.seq_len] * self.batch

    def make(self):
        lens = self.lens()
        total = sum(lens)
        start = [0]
        for n in lens[:-1]:
            start.append(start[-1] + n)
        return {
            "q": _randn((total, self.hq, self.head_dim), self.seed * 100, self.dtype),
            "k": _randn((total, self.hkv, self.head_dim), self.seed * 100 + 1, self.dtype),
            "v": _randn((total, self.hkv, self.head_dim), self.seed * 100 + 2, self.dtype),
            "b_start_loc": torch.tensor(start, dtype=torch.int32),
            "b_seq_len": torch.tensor(lens, dtype=torch.int32),
            "max_input_len": max(lens),
        }

    def flops(self) -> int:
        # causal half of 4 * S^2 * D per (sequence, q head)
        return sum(4 * n * n * self.head_dim * self.hq // 2 for n in self.lens())


# ------------------------------------------------------------------ C5: paged decode
@dataclass
class DecodeWorkload:
    batch: int = 64
    ctx_lo: int = 1024
    ctx_hi: int = 32768
    page: int = 64
    hq: int = 32
    hkv: int = 8
    head_dim: int = 128
    dtype: torch.dtype = torch.bfloat16
    seed: int = 4

    def make(self, device="cpu"):
        """Caches are filled on `device` directly when it is a CUDA device (they are GBs at full size);
        the small tensors are made on the CPU from fixed seeds."""
        g = _gen(self.seed * 100)
        ctx = torch.randint(self.ctx_lo, self.ctx_hi + 1, (self.batch,), generator=g, dtype=torch.int64)
        pages_per_seq = (ctx + self.page - 1) // self.page
        total_pages = int(pages_per_seq.sum())
        perm = torch.randperm(total_pages, generator=_gen(self.seed * 100 + 1))
        max_pages = (self.ctx_hi + self.page - 1) // self.page
        table = torch.zeros((self.batch, max_pages), dtype=torch.int32)
        off = 0
        for b in range(self.batch):
            n = int(pages_per_seq[b])
            table[b, :n] = perm[off:off + n].to(torch.int32)
            off += n
        shape = (total_pages, self.page, self.hkv, self.head_dim)
        if str(device).startswith("cuda"):
            gk = torch.Generator(device=device)
            gk.manual_seed(self.seed * 100 + 2)
            k_cache = torch.randn(shape, generator=gk, device=device, dtype=torch.float32).to(self.dtype)
            gv = torch.Generator(device=device)
            gv.manual_seed(self.seed * 100 + 3)
            v_cache = torch.randn(shape, generator=gv, device=device, dtype=torch.float32).to(self.dtype)
        else:
            k_cache = _randn(shape, self.seed * 100 + 2, self.dtype)
            v_cache = _randn(shape, self.seed * 100 + 3, self.dtype)
        return {
            "q": _randn((self.batch, self.hq, self.head_dim), self.seed * 100 + 4, self.dtype),
            "k_cache": k_cache,
            "v_cache": v_cache,
            "block_table": table,
            "kv_seqlens": ctx.to(torch.int32),
        }

    @staticmethod
    def bytes(kv_seqlens, hkv=8, head_dim=128, hq=32, elem=2) -> int:
        ctx_sum = int(kv_seqlens.sum())
        b = kv_seqlens.numel()
        return ctx_sum * hkv * head_dim * elem * 2 + 2 * b * hq * head_dim * elem

    @staticmethod
    def flops(kv_seqlens, hq=32, head_dim=128) -> int:
        return 4 * int(kv_seqlens.sum()) * head_dim * hq
