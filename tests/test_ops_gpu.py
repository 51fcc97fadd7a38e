"""Own training kernels against fp32 PyTorch references of the same op."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def test_layernorm_fwd_bwd():
    from gcow_b200.ops import kernels as K
    torch.manual_seed(0)
    for rows, H in ((64, 1024), (1000, 768), (37, 128)):
        x = torch.randn(rows, H, device="cuda", requires_grad=True)
        g = (torch.rand(H, device="cuda") + 0.5).requires_grad_(True)
        b = torch.randn(H, device="cuda", requires_grad=True)
        y = K.layernorm(x, g, b, 1e-12)
        w = torch.randn(rows, H, device="cuda")
        (y.float() * w).sum().backward()
        gx, gg, gb = x.grad.clone(), g.grad.clone(), b.grad.clone()
        x.grad = g.grad = b.grad = None
        xr = x.detach().bfloat16().float().requires_grad_(True)
        yr = F.layer_norm(xr, (H,), g, b, 1e-12)
        (yr * w.bfloat16().float()).sum().backward()
        assert (y.float() - yr).abs().max().item() < 0.05
        assert (gx.float() - xr.grad).abs().max().item() < 0.05 * xr.grad.abs().max().item() + 1e-3
        assert (gg - g.grad).abs().max().item() < 0.02 * g.grad.abs().max().item() + 1e-2
        assert (gb - b.grad).abs().max().item() < 0.02 * b.grad.abs().max().item() + 1e-2


def test_gelu_fwd_bwd():
    from gcow_b200.ops import kernels as K
    x = (torch.randn(4096, 1024, device="cuda") * 2).requires_grad_(True)
    y = K.gelu(x)
    y.float().sum().backward()
    xr = x.detach().bfloat16().float().requires_grad_(True)
    yr = F.gelu(xr)
    yr.sum().backward()
    assert (y.float() - yr).abs().max().item() < 0.02
    assert (x.grad - xr.grad).abs().max().item() < 0.02


def test_softmax_xent_loss_and_grad():
    from gcow_b200.ops import kernels as K
    torch.manual_seed(1)
    rows, V, ld = 300, 30522, 30528
    base = (torch.randn(rows, ld, device="cuda") * 3).bfloat16()
    src = base.clone().requires_grad_(True)
    logits = (src * 1.0)[:, :V]                      # non-leaf strided view, as the vocabulary GEMM returns
    target = torch.randint(0, V, (rows,), device="cuda")
    target[::7] = -100
    ref_in = base[:, :V].float().requires_grad_(True)
    ref = F.cross_entropy(ref_in, target, ignore_index=-100)
    ref.backward()
    loss = K.softmax_xent(logits, target, -100)
    loss.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item())
    g = src.grad[:, :V].float()
    assert (g - ref_in.grad).abs().max().item() < 2e-2 * ref_in.grad.abs().max().item()
    assert float(src.grad[:, V:].abs().sum()) == 0.0


def test_colsum_and_preprocess():
    from gcow_b200.ops import kernels as K
    g = torch.randn(5000, 1024, device="cuda").bfloat16()
    assert (K.colsum(g) - g.float().sum(0)).abs().max().item() < 1e-2
    x = torch.randint(0, 256, (4, 32, 32, 3), dtype=torch.uint8, device="cuda")
    mean = [0.485 * 255, 0.456 * 255, 0.406 * 255]
    std = [0.229 * 255, 0.224 * 255, 0.225 * 255]
    y = K.u8_to_bf16_norm(x, mean, std)
    assert y.shape == (4, 3, 32, 32) and y.is_contiguous(memory_format=torch.channels_last)
    ref = (x.permute(0, 3, 1, 2).float() - torch.tensor(mean, device="cuda").view(1, 3, 1, 1)) / \
        torch.tensor(std, device="cuda").view(1, 3, 1, 1)
    assert (y.float() - ref).abs().max().item() < 0.02


def test_conv1x1_matches_torch():
    from gcow_b200.ops import kernels as K
    torch.manual_seed(2)
    x = torch.randn(8, 64, 28, 28, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    w = (torch.randn(256, 64, 1, 1, device="cuda") * 0.1).requires_grad_(True)
    assert K.conv1x1_usable(x, w)
    y = K.conv1x1(x, w, None)
    y.float().square().mean().backward()
    gx, gw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    yr = F.conv2d(x.float(), w)
    yr.square().mean().backward()
    assert y.shape == yr.shape and (y.float() - yr).abs().max().item() < 0.05 * yr.abs().max().item()
    assert (gx.float() - x.grad.float()).abs().max().item() < 0.05 * x.grad.float().abs().max().item() + 1e-6
    assert (gw - w.grad).abs().max().item() < 0.05 * w.grad.abs().max().item() + 1e-6


def test_linear_with_odd_vocabulary_width():
    from gcow_b200.ops import kernels as K
    torch.manual_seed(3)
    x = torch.randn(2, 64, 128, device="cuda", requires_grad=True)
    w = (torch.randn(1002, 128, device="cuda") * 0.05).requires_grad_(True)
    b = torch.zeros(1002, device="cuda", requires_grad=True)
    t = torch.randint(0, 1002, (128,), device="cuda")
    y = K.linear(x, w, b)
    assert y.shape == (2, 64, 1002)
    loss = K.softmax_xent(y.flatten(0, 1), t)
    loss.backward()
    gx, gw, gb = x.grad.clone(), w.grad.clone(), b.grad.clone()
    x.grad = w.grad = b.grad = None
    ref = F.cross_entropy(F.linear(x, w, b).flatten(0, 1), t)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 0.02
    for a, r in ((gx, x.grad), (gw, w.grad), (gb, b.grad)):
        assert (a.float() - r).abs().max().item() < 0.08 * r.abs().max().item() + 1e-5


def test_bert_tiny_own_vs_torch_ops():
    from gcow_b200.models import bert_tiny
    from gcow_b200 import ops
    torch.manual_seed(4)
    m = bert_tiny().cuda()
    ids = torch.randint(0, 1024, (4, 64), device="cuda")
    lab = torch.where(torch.rand(4, 64, device="cuda") < 0.15, ids, torch.full_like(ids, -100))
    nsp = torch.randint(0, 2, (4,), device="cuda")
    losses = {}
    grads = {}
    for be in ("torch", "own"):
        ops.set_backend(be)
        m.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = m(ids, None, lab, nsp)
        loss.backward()
        losses[be] = loss.item()
        grads[be] = m.layers[0].fc1.weight.grad.clone()
    ops.set_backend("own")
    assert abs(losses["own"] - losses["torch"]) < 0.05
    d = (grads["own"] - grads["torch"]).abs().max().item()
    assert d < 0.1 * grads["torch"].abs().max().item() + 1e-4


@pytest.mark.parametrize("C,hw,res,relu", [(64, 56, False, True), (256, 14, True, True), (2048, 7, True, True), (128, 28, False, False)])
def test_batchnorm_act_fused_matches_torch(C, hw, res, relu):
    from gcow_b200.ops import nn as gnn, set_backend
    torch.manual_seed(C)
    N = 16
    mk = lambda: (torch.randn(N, C, hw, hw, device="cuda") * 2 + 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    x0, r0, w = mk(), mk(), mk()
    outs = {}
    for be in ("torch", "own"):
        set_backend(be)
        bn = gnn.BatchNorm2d(C).cuda()
        with torch.no_grad():
            bn.weight.uniform_(0.5, 1.5); bn.bias.uniform_(-0.5, 0.5)
            torch.manual_seed(1); bn.weight.copy_(torch.rand(C) + 0.5); bn.bias.copy_(torch.rand(C) - 0.5)
        x = x0.clone().requires_grad_(True)
        r = r0.clone().requires_grad_(True) if res else None
        y = bn(x, residual=r, relu=relu)
        (y.float() * w.float()).sum().backward()
        outs[be] = (y.detach().float(), x.grad.float(), r.grad.float() if res else None, bn.weight.grad.clone(),
                    bn.bias.grad.clone(), bn.running_mean.clone(), bn.running_var.clone())
    set_backend("own")
    a, b = outs["own"], outs["torch"]
    # torch rounds to bf16 after bn, after the add and after the relu; the fused kernel once
    assert (a[0] - b[0]).abs().max().item() < 0.02 * b[0].abs().max().item() + 0.07
    assert (a[1] - b[1]).abs().max().item() < 0.03 * b[1].abs().max().item() + 0.02
    if res:
        assert (a[2] - b[2]).abs().max().item() < 0.02 * b[2].abs().max().item() + 0.05
    assert (a[3] - b[3]).abs().max().item() < 0.02 * b[3].abs().max().item() + 0.5
    assert (a[4] - b[4]).abs().max().item() < 0.02 * b[4].abs().max().item() + 0.5
    assert (a[5] - b[5]).abs().max().item() < 1e-2 and (a[6] - b[6]).abs().max().item() < 2e-2


def test_pools_match_torch():
    from gcow_b200.ops import kernels as K
    torch.manual_seed(5)
    x = torch.relu(torch.randn(8, 64, 57, 57, device="cuda")).bfloat16().contiguous(memory_format=torch.channels_last)
    xa = x.clone().requires_grad_(True)
    xb = x.clone().float().requires_grad_(True)
    ya, yb = K.maxpool3x3s2(xa), F.max_pool2d(xb, 3, 2, 1)
    assert ya.shape == yb.shape and torch.equal(ya.float(), yb)
    w = torch.randn_like(yb)
    (ya.float() * w).sum().backward(); (yb * w).sum().backward()
    assert (xa.grad.float() - xb.grad).abs().max().item() < 0.02 * xb.grad.abs().max().item() + 1e-3
    xa2 = x.clone().requires_grad_(True); xb2 = x.clone().float().requires_grad_(True)
    pa, pb = K.global_avgpool(xa2), F.adaptive_avg_pool2d(xb2, 1)
    assert (pa.float() - pb).abs().max().item() < 0.01
    pa.float().sum().backward(); pb.sum().backward()
    assert (xa2.grad.float() - xb2.grad).abs().max().item() < 1e-5


def test_resnet_own_vs_torch_backends_agree():
    from gcow_b200.models import resnet18
    from gcow_b200 import ops
    torch.manual_seed(6)
    m = resnet18(num_classes=10).cuda().to(memory_format=torch.channels_last)
    x = torch.randn(8, 3, 64, 64, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (8,), device="cuda")
    res = {}
    for be in ("torch", "own"):
        ops.set_backend(be)
        m.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = F.cross_entropy(m(x).float(), y)
        loss.backward()
        res[be] = (loss.item(), m.conv1.weight.grad.clone())
    ops.set_backend("own")
    assert abs(res["own"][0] - res["torch"][0]) < 0.05
    d = (res["own"][1] - res["torch"][1]).abs().max().item()
    assert d < 0.15 * res["torch"][1].abs().max().item() + 1e-3
