"""Fused optimizers against torch.optim (CPU arithmetic path here, kernels on GPU)."""
import pytest
import torch

from gcow_b200.ops.optim import FusedAdamW, FusedSGD


def _pair(device, seed=0):
    torch.manual_seed(seed)
    shapes = [(7,), (33, 5), (1 << 17,), (3, 3, 3, 3)]
    a = [torch.randn(s, device=device, requires_grad=True) for s in shapes]
    b = [t.detach().clone().requires_grad_(True) for t in a]
    return a, b


def _run(opt_a, opt_b, a, b, steps=4):
    for s in range(steps):
        torch.manual_seed(100 + s)
        for x, y in zip(a, b):
            g = torch.randn_like(x)
            x.grad = g.clone()
            y.grad = g.clone()
        opt_a.step()
        opt_b.step()


@pytest.mark.parametrize("nesterov", [False, True])
def test_sgd_cpu_matches_torch(nesterov):
    a, b = _pair("cpu")
    _run(FusedSGD(a, lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=nesterov),
         torch.optim.SGD(b, lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=nesterov), a, b)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)


def test_adamw_cpu_matches_torch():
    a, b = _pair("cpu")
    _run(FusedAdamW(a, lr=1e-3, weight_decay=0.01, eps=1e-6),
         torch.optim.AdamW(b, lr=1e-3, weight_decay=0.01, eps=1e-6), a, b)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("nesterov", [False, True])
def test_sgd_gpu_matches_torch(nesterov):
    a, b = _pair("cuda")
    fa = FusedSGD(a, lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=nesterov)
    _run(fa, torch.optim.SGD(b, lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=nesterov), a, b)
    assert fa.launches == 4
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
def test_adamw_gpu_matches_torch_and_resumes():
    a, b = _pair("cuda")
    fa = FusedAdamW(a, lr=1e-3, weight_decay=0.01, eps=1e-6)
    tb = torch.optim.AdamW(b, lr=1e-3, weight_decay=0.01, eps=1e-6)
    _run(fa, tb, a, b)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-4, atol=1e-6)
    # state dict round trip keeps stepping identically
    import copy
    sd = copy.deepcopy(fa.state_dict())   # torch.save/load would give separate tensors too
    a2 = [t.detach().clone().requires_grad_(True) for t in a]
    fa2 = FusedAdamW(a2, lr=1e-3, weight_decay=0.01, eps=1e-6)
    fa2.load_state_dict(sd)
    _run(fa, fa2, a, a2, steps=2)
    for x, y in zip(a, a2):
        assert torch.equal(x, y)
