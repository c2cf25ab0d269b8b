"""Golden fixtures for the two operators that the reference project does not implement, made from the
implementations of the same published algorithms in third-party packages installed next to torch.

    python tests/golden/make_golden_third_party.py

* Group-limited sigmoid routing (DeepSeek-V3): `DeepseekV3MoE.route_tokens_to_experts` of the `transformers`
  package is EXECUTED on seeded logits (CPU); inputs and its outputs go to grouped_gating_hf.pt.
* moe_align_block_size: the worked example in the docstring of vLLM's `moe_align_block_size` (the operator
  itself is a CUDA op and cannot run here) is PARSED from the installed file and stored in
  moe_align_vllm_doc.pt as a known-answer vector.

Nothing is copied from either package: one is called, the other's documented example is read at run time.
The package versions are recorded in the fixtures.
"""
from __future__ import annotations

import ast
import importlib.util
import os
import re
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def hf_router_cases():
    import transformers
    from transformers.models.deepseek_v3.modeling_deepseek_v3 import DeepseekV3MoE

    cases = []
    for i, (tokens, experts, n_group, topk_group, top_k, scale, norm) in enumerate([
            (192, 256, 8, 4, 8, 2.5, True),          # the benchmark's routing configuration
            (160, 64, 4, 2, 6, 1.0, True),
            (129, 128, 8, 3, 4, 16.0, False)]):
        g = torch.Generator().manual_seed(500 + i)
        logits = torch.randn(tokens, experts, generator=g)
        bias = torch.randn(experts, generator=g) * 0.01
        stub = types.SimpleNamespace(
            gate=types.SimpleNamespace(e_score_correction_bias=bias), n_group=n_group,
            n_routed_experts=experts, topk_group=topk_group, top_k=top_k, norm_topk_prob=norm,
            routed_scaling_factor=scale)
        ids, weights = DeepseekV3MoE.route_tokens_to_experts(stub, logits.clone())
        cases.append({"logits": logits, "bias": bias, "n_group": n_group, "topk_group": topk_group, "top_k": top_k,
                      "scale": scale, "renormalize": norm, "ids": ids.to(torch.int32), "weights": weights,
                      "source": f"transformers {transformers.__version__} DeepseekV3MoE.route_tokens_to_experts"})
    return cases


def vllm_align_example():
    spec = importlib.util.find_spec("vllm")
    root = os.path.dirname(spec.origin)
    path = os.path.join(root, "model_executor", "layers", "fused_moe", "moe_align_block_size.py")
    text = open(path).read()
    doc = text[text.index("def moe_align_block_size"):]
    doc = doc[doc.index('"""'):doc.index('"""', doc.index('"""') + 3)]
    doc = re.sub(r"\s+", " ", doc)
    m = re.search(r"Given topk_ids = (\[\[.*?\]\]), block_size = (\d+), and num_experts = (\d+)", doc)
    ids = ast.literal_eval(m.group(1))
    out = re.search(r"we obtain token_ids (\[[\d, ]+\])", doc)
    version = "unknown"
    try:
        from importlib.metadata import version as _v
        version = _v("vllm")
    except Exception:  # noqa: BLE001
        pass
    return {"topk_ids": torch.tensor(ids, dtype=torch.int64), "block_size": int(m.group(2)),
            "num_experts_in_doc": int(m.group(3)), "token_ids": torch.tensor(ast.literal_eval(out.group(1)), dtype=torch.int32),
            "source": f"vllm {version}, docstring example of moe_align_block_size"}


if __name__ == "__main__":
    torch.save(hf_router_cases(), os.path.join(HERE, "grouped_gating_hf.pt"))
    torch.save(vllm_align_example(), os.path.join(HERE, "moe_align_vllm_doc.pt"))
    for f in ("grouped_gating_hf.pt", "moe_align_vllm_doc.pt"):
        print(f, os.path.getsize(os.path.join(HERE, f)))
