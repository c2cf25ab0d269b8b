"""GPU parity: GShard-style top-k gating with capacity (forward and the auxiliary-loss backward)."""
import os

import pytest
import torch

from dlcompiler_b200 import topk_gating
from oracle import dlblas_oracle as oracle

pytestmark = pytest.mark.gpu


def _prio_of_selection(select, priority, E):
    cap = select.numel() // E
    sel = select.view(E, cap)
    return torch.stack([priority[sel[e], e].sort(descending=True)[0] for e in range(E)])


def _check(dev, logits, k, cf, mc, ref=None):
    E = logits.size(1)
    l_aux, ec, w, sel = topk_gating(logits.to(dev), k, cf, mc)
    rl, rec, rw, rsel, prio = oracle.topk_gating(logits, k, cf, mc)
    torch.testing.assert_close(l_aux.cpu(), rl, rtol=1e-5, atol=1e-6)
    assert torch.equal(ec.cpu(), rec)                                   # integer output: bit-exact
    torch.testing.assert_close(w.cpu(), rw, rtol=1e-5, atol=1e-7)
    assert torch.equal(sel.cpu(), rsel)                                 # our order is fully specified
    if ref is not None:                                                 # the reference's own outputs
        torch.testing.assert_close(l_aux.cpu(), ref["l_aux"], rtol=1e-5, atol=1e-6)
        assert torch.equal(ec.cpu(), ref["ec_idx"])
        torch.testing.assert_close(w.cpu(), ref["weights"], rtol=1e-5, atol=1e-7)
        assert torch.equal(_prio_of_selection(sel.cpu(), prio, E), _prio_of_selection(ref["select"], prio, E))


def test_topk_gating_golden(cuda_device, golden_dir):
    for c in torch.load(os.path.join(golden_dir, "topk_gating.pt"), weights_only=True):
        _check(cuda_device, c["logits"], c["k"], c["capacity_factor"], c["min_capacity"], ref=c)


@pytest.mark.parametrize("S,E,k,cf,mc", [(4096, 64, 8, 1.0, 2),      # the reference benchmark's shape
                                         (1000, 8, 2, 1.25, 4), (16, 4, 1, 1.0, 2), (2048, 256, 6, 0.25, 2)])
def test_topk_gating_shapes(cuda_device, S, E, k, cf, mc):
    g = torch.Generator().manual_seed(S + E)
    _check(cuda_device, torch.randn(S, E, generator=g), k, cf, mc)


def test_topk_gating_backward(cuda_device):
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(512, 64, generator=g)
    x = logits.to(cuda_device).requires_grad_(True)
    l_aux, _, _, _ = topk_gating(x, 8)
    (l_aux * 3.0).backward()
    ref = oracle.topk_gating_backward(logits, 8, grad_l_aux=3.0)
    torch.testing.assert_close(x.grad.cpu(), ref, rtol=1e-4, atol=1e-8)


@pytest.mark.parametrize("S,E,k,cf", [(512, 64, 8, 1.0), (300, 8, 2, 0.5), (64, 16, 4, 2.0)])
def test_topk_gating_backward_through_weights(cuda_device, S, E, k, cf):
    """`higher_precision=True`: the routing weights back-propagate as well; against autograd through the
    oracle's forward expression (capacity drops included: cf = 0.5 drops about half of the choices)."""
    g = torch.Generator().manual_seed(S + k)
    logits = torch.randn(S, E, generator=g)
    gw = torch.randn(k * S, generator=g)
    x = logits.to(cuda_device).requires_grad_(True)
    l_aux, _, w, _ = topk_gating(x, k, cf, 2, True)
    (l_aux * 1.5 + (w * gw.to(cuda_device)).sum()).backward()
    ref = oracle.topk_gating_backward_weights(logits, k, cf, 2, grad_l_aux=1.5, grad_weights=gw)
    torch.testing.assert_close(x.grad.cpu(), ref, rtol=2e-4, atol=2e-6)
    # the default mode still ignores the weights' gradient, as the reference does
    y = logits.to(cuda_device).requires_grad_(True)
    l2, _, w2, _ = topk_gating(y, k, cf, 2, False)
    (l2 * 1.5 + (w2 * gw.to(cuda_device)).sum()).backward()
    torch.testing.assert_close(y.grad.cpu(), oracle.topk_gating_backward(logits, k, grad_l_aux=1.5), rtol=1e-4,
                               atol=1e-8)
