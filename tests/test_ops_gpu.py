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
    for rows, cols in ((5000, 1024), (16384, 1000), (777, 30), (129, 4096)):     # wide (16-byte) and narrow paths
        g = torch.randn(rows, cols, device="cuda").bfloat16()
        ref = g.float().sum(0)
        assert (K.colsum(g) - ref).abs().max().item() < 2e-3 * ref.abs().max().item() + 1e-2, (rows, cols)
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
def test_batchnorm_act_fused_matches_fp32_reference(C, hw, res, relu):
    """Fused BN(+add)(+ReLU) against the same computation done by PyTorch in fp32."""
    from gcow_b200.ops import nn as gnn, set_backend
    torch.manual_seed(C)
    N = 16
    mk = lambda: (torch.randn(N, C, hw, hw, device="cuda") * 2 + 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    x0, r0, w = mk(), mk(), mk()
    gamma, beta = torch.rand(C, device="cuda") + 0.5, torch.rand(C, device="cuda") - 0.5
    # reference: fp32 all the way
    ref_bn = torch.nn.BatchNorm2d(C).cuda()
    with torch.no_grad():
        ref_bn.weight.copy_(gamma); ref_bn.bias.copy_(beta)
    xr = x0.float().requires_grad_(True)
    rr = r0.float().requires_grad_(True) if res else None
    yr = ref_bn(xr)
    if res:
        yr = yr + rr
    if relu:
        yr = torch.relu(yr)
    (yr * w.float()).sum().backward()
    # own kernels
    set_backend("own")
    bn = gnn.BatchNorm2d(C).cuda()
    with torch.no_grad():
        bn.weight.copy_(gamma); bn.bias.copy_(beta)
    x = x0.clone().requires_grad_(True)
    r = r0.clone().requires_grad_(True) if res else None
    y = bn(x, residual=r, relu=relu)
    assert y.dtype == torch.bfloat16 and y.is_contiguous(memory_format=torch.channels_last)
    (y.float() * w.float()).sum().backward()
    tol = lambda ref: 0.012 * ref.abs().max().item() + 1e-2          # bf16 has 8 bits of mantissa
    assert (y.float() - yr).abs().max().item() < tol(yr)
    assert (x.grad.float() - xr.grad).abs().max().item() < tol(xr.grad)
    if res:
        assert (r.grad.float() - rr.grad).abs().max().item() < tol(rr.grad)
    assert (bn.weight.grad - ref_bn.weight.grad).abs().max().item() < 0.01 * ref_bn.weight.grad.abs().max().item() + 0.5
    assert (bn.bias.grad - ref_bn.bias.grad).abs().max().item() < 0.01 * ref_bn.bias.grad.abs().max().item() + 0.5
    assert (bn.running_mean - ref_bn.running_mean).abs().max().item() < 1e-3
    assert (bn.running_var - ref_bn.running_var).abs().max().item() < 1e-2
    # inference statistics
    bn.eval(); ref_bn.eval()
    ye = bn(x0, residual=r0 if res else None, relu=relu)
    yer = ref_bn(x0.float()) + (r0.float() if res else 0)
    yer = torch.relu(yer) if relu else yer
    assert (ye.float() - yer).abs().max().item() < tol(yer)


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


@pytest.mark.parametrize("k,stride,pad", [(3, 1, 1), (3, 2, 1), (1, 2, 0), (7, 2, 3)])
def test_conv_as_im2col_gemm_matches_torch(k, stride, pad):
    from gcow_b200.ops import kernels as K
    torch.manual_seed(k * 10 + stride)
    x = torch.randn(4, 16, 30, 30, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    w = (torch.randn(24, 16, k, k, device="cuda") * 0.1).requires_grad_(True)
    b = torch.randn(24, device="cuda", requires_grad=True)
    y = K.conv_gemm(x, w, b, stride, pad)
    wgt = torch.randn_like(y.float())
    (y.float() * wgt).sum().backward()
    gx, gw, gb = x.grad.float().clone(), w.grad.clone(), b.grad.clone()
    x.grad = w.grad = b.grad = None
    xr = x.detach().float().requires_grad_(True)
    yr = F.conv2d(xr, w, b, stride=stride, padding=pad)
    (yr * wgt).sum().backward()
    tol = lambda r: 0.02 * r.abs().max().item() + 1e-2
    assert y.shape == yr.shape and (y.float() - yr).abs().max().item() < tol(yr)
    assert (gx - xr.grad).abs().max().item() < tol(xr.grad)
    assert (gw - w.grad).abs().max().item() < tol(w.grad)
    assert (gb - b.grad).abs().max().item() < tol(b.grad)


def test_batched_gemm_and_own_attention():
    from gcow_b200.ops import kernels as K
    torch.manual_seed(8)
    a = (torch.randn(6, 200, 72, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(6, 136, 72, device="cuda") * 0.5).bfloat16()
    ref = torch.einsum("bmk,bnk->bmn", a.float(), b.float())
    y = K.bmm_bf16(a, b, out_dtype=torch.float32)
    y2 = K.bmm_bf16(a.transpose(1, 2).contiguous(), b.transpose(1, 2).contiguous(), a_t=True, b_t=True, out_dtype=torch.float32)
    K.check_errors()
    assert (y - ref).abs().max().item() < 2e-2 and (y2 - ref).abs().max().item() < 2e-2
    # attention against scaled_dot_product_attention in fp32
    B, S, H, D = 2, 128, 4, 64
    qkv = (torch.randn(B, S, 3, H, D, device="cuda") * 0.7).bfloat16().requires_grad_(True)
    w = torch.randn(B, S, H * D, device="cuda")
    o = K.attention(qkv)
    (o.float() * w).sum().backward()
    K.check_errors()
    g = qkv.grad.float().clone()
    x = qkv.detach().float().requires_grad_(True)
    q, k, v = (x[:, :, i].transpose(1, 2) for i in range(3))
    oref = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, S, H * D)
    (oref * w).sum().backward()
    assert (o.float() - oref).abs().max().item() < 0.03
    assert (g - x.grad).abs().max().item() < 0.05 * x.grad.abs().max().item() + 0.02


@pytest.mark.parametrize("shape", [(2, 128, 2, 64), (1, 256, 3, 64), (2, 384, 2, 64), (1, 512, 4, 64)])
def test_fused_attention_matches_fp32_reference(shape):
    """Forward and the three gradients of the fused tcgen05 attention against softmax(QK^T / sqrt d) V in fp32 on
    the same bf16-rounded inputs."""
    from gcow_b200.ops import kernels as K
    B, S, H, D = shape
    torch.manual_seed(sum(shape))
    qkv = (torch.randn(B, S, 3, H, D, device="cuda") * 0.8).bfloat16().requires_grad_(True)
    assert K.fused_attention_usable(qkv)
    w = torch.randn(B, S, H * D, device="cuda").bfloat16()
    o = K.fused_attention(qkv)
    (o.float() * w.float()).sum().backward()
    K.check_errors()
    g = qkv.grad.float().clone()
    x = qkv.detach().float().requires_grad_(True)
    q, k, v = (x[:, :, i].transpose(1, 2) for i in range(3))
    p = torch.softmax(q @ k.transpose(-1, -2) / D ** 0.5, dim=-1)
    oref = (p @ v).transpose(1, 2).reshape(B, S, H * D)
    (oref * w.float()).sum().backward()
    assert (o.float() - oref).abs().max().item() < 0.02
    for i, name in enumerate(("dq", "dk", "dv")):
        err = (g[:, :, i] - x.grad[:, :, i]).abs().max().item()
        assert err < 0.03 * x.grad[:, :, i].abs().max().item() + 0.01, (name, err)


def test_attention_module_routes_to_the_fused_kernel():
    from gcow_b200.ops import kernels as K, nn as gnn, set_backend
    set_backend("own")
    qkv = (torch.randn(1, 128, 3, 2, 64, device="cuda") * 0.5).bfloat16()
    before = K.launch_count()
    o = gnn.attention(qkv)
    assert K.launch_count() == before + 1 and o.shape == (1, 128, 128)      # one launch: the fused forward
    small = (torch.randn(1, 64, 3, 2, 64, device="cuda") * 0.5).bfloat16()  # 64 positions: the batched-GEMM path
    before = K.launch_count()
    gnn.attention(small)
    assert K.launch_count() == before + 3


def test_packed_sdpa_matches_plain_autograd(monkeypatch):
    from gcow_b200.ops import nn as gnn, set_backend
    torch.manual_seed(10)
    B, S, H, D = 2, 64, 4, 64
    base = (torch.randn(B, S, 3, H, D, device="cuda") * 0.5).bfloat16()
    w = torch.randn(B, S, H * D, device="cuda").bfloat16()
    outs = {}
    monkeypatch.setenv("GCOW_ATTENTION", "lib")          # the library arm of the own backend
    for be in ("torch", "own"):
        set_backend(be)
        qkv = base.clone().requires_grad_(True)
        o = gnn.attention(qkv * 1.0)
        (o * w).sum().backward()
        outs[be] = (o.detach().float(), qkv.grad.float())
    set_backend("own")
    assert (outs["own"][0] - outs["torch"][0]).abs().max().item() < 1e-2
    assert (outs["own"][1] - outs["torch"][1]).abs().max().item() < 2e-2 * outs["torch"][1].abs().max().item() + 1e-3


def test_fused_ffn_and_linear_residual_match_unfused():
    """x + fc2(gelu(fc1 x)) and r + lin(x) with every elementwise step inside GEMM epilogues, against fp32 PyTorch."""
    import torch.nn as nn
    import torch.nn.functional as F
    from gcow_b200.ops import nn as gnn, set_backend
    set_backend("own")
    torch.manual_seed(11)
    M, H, Fd = 512, 256, 1024
    fc1, fc2, proj = gnn.Linear(H, Fd).cuda(), gnn.Linear(Fd, H).cuda(), gnn.Linear(H, H).cuda()
    x0 = (torch.randn(4, M // 4, H, device="cuda") * 0.7).bfloat16()
    c0 = (torch.randn(4, M // 4, H, device="cuda") * 0.7).bfloat16()
    gy = (torch.randn(4, M // 4, H, device="cuda") * 0.5).bfloat16()

    def run(fused):
        for m in (fc1, fc2, proj):
            m.zero_grad(set_to_none=True)
        x, c = x0.clone().requires_grad_(True), c0.clone().requires_grad_(True)
        if fused:
            h = gnn.linear_residual(c, proj, x)
            y = gnn.ffn_residual(h, fc1, fc2)
        else:
            xf, cf = x.float(), c.float()
            h = xf + F.linear(cf, proj.weight, proj.bias)
            y = h + F.linear(F.gelu(F.linear(h, fc1.weight, fc1.bias)), fc2.weight, fc2.bias)
        y.backward(gy.to(y.dtype))
        return [y.detach().float(), x.grad.float(), c.grad.float()] + [p.grad.float().clone() for m in (fc1, fc2, proj) for p in m.parameters()]

    from gcow_b200.ops import kernels as K
    before = K.launch_count()
    got = run(True)
    assert K.launch_count() > before           # the fused functions ran, not the fallback
    K.check_errors()
    ref = run(False)
    for i, (a, b) in enumerate(zip(got, ref)):
        err = (a - b).abs().max().item() / (b.abs().max().item() + 1e-6)
        assert err < 3e-2, (i, err)


def test_fused_embeddings_match_pytorch():
    import torch.nn as nn
    from gcow_b200.ops import nn as gnn, set_backend
    torch.manual_seed(12)
    B, S, H, V = 4, 48, 256, 500
    tok, pos, typ = gnn.Embedding(V, H).cuda(), gnn.Embedding(64, H).cuda(), gnn.Embedding(2, H).cuda()
    ids = torch.randint(0, V, (B, S), device="cuda")
    ids[0, :10] = 7                                      # a long run of one id
    ty = torch.randint(0, 2, (B, S), device="cuda")
    gy = torch.randn(B, S, H, device="cuda").bfloat16()
    res = {}
    for be in ("torch", "own"):
        set_backend(be)
        for m in (tok, pos, typ):
            m.zero_grad(set_to_none=True)
        y = gnn.embed_sum3(ids, ty, tok, pos, typ)
        y.backward(gy.to(y.dtype))
        res[be] = [y.detach().float()] + [m.weight.grad.clone() for m in (tok, pos, typ)]
    set_backend("own")
    assert res["own"][0].dtype == torch.float32 and (res["own"][0] - res["torch"][0]).abs().max().item() < 2e-2
    for a, b in zip(res["own"][1:], res["torch"][1:]):
        assert (a - b).abs().max().item() < 1e-3 * max(1.0, b.abs().max().item())


def test_batchnorm_fork_adds_the_two_gradients_in_the_kernel():
    """bn(x, residual, relu, fork=True) returns two tensors on one memory; their gradients arrive separately and are
    added inside the backward kernel. Compared with fp32 PyTorch ops on the same values."""
    import torch.nn.functional as F
    from gcow_b200.ops import nn as gnn, set_backend
    set_backend("own")
    torch.manual_seed(13)
    N, C, H, W = 8, 64, 12, 12
    bn = gnn.BatchNorm2d(C).cuda()
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5); bn.bias.uniform_(-0.3, 0.3)
    x0 = torch.randn(N, C, H, W, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    r0 = torch.randn(N, C, H, W, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    w1 = torch.randn(N, C, H, W, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    w2 = torch.randn(N, C, H, W, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    x, r = x0.clone().requires_grad_(True), r0.clone().requires_grad_(True)
    y1, y2 = bn(x, residual=r, relu=True, fork=True)
    assert y1.data_ptr() == y2.data_ptr() and y1 is not y2
    ((y1 * w1).sum() + (y2 * w2).sum()).backward()
    got = [y1.detach().float(), x.grad.float(), r.grad.float(), bn.weight.grad.clone(), bn.bias.grad.clone()]

    xf, rf = x0.float().requires_grad_(True), r0.float().requires_grad_(True)
    g, b = bn.weight.detach().clone().requires_grad_(True), bn.bias.detach().clone().requires_grad_(True)
    yr = F.relu(F.batch_norm(xf, None, None, g, b, True, 0.1, bn.eps) + rf)
    (yr * (w1.float() + w2.float())).sum().backward()
    ref = [yr.detach(), xf.grad, rf.grad, g.grad, b.grad]
    for i, (a, e) in enumerate(zip(got, ref)):
        err = (a - e).abs().max().item() / (e.abs().max().item() + 1e-6)
        assert err < 3e-2, (i, err)
    # only one of the two outputs used: the other gradient is absent
    bn.zero_grad(set_to_none=True)
    x = x0.clone().requires_grad_(True)
    y1, y2 = bn(x, relu=True, fork=True)
    (y2 * w2).sum().backward()
    xf = x0.float().requires_grad_(True)
    (F.relu(F.batch_norm(xf, None, None, bn.weight.detach(), bn.bias.detach(), True, 0.1, bn.eps)) * w2.float()).sum().backward()
    assert (x.grad.float() - xf.grad).abs().max().item() / xf.grad.abs().max().item() < 3e-2


def test_batchnorm_counts_training_steps_lazily():
    """num_batches_tracked is counted on the host by the own path and lands in the tensor when the state is saved,
    when PyTorch's own path runs, and not twice."""
    from gcow_b200.ops import nn as gnn, set_backend
    set_backend("own")
    bn = gnn.BatchNorm2d(64).cuda()
    x = torch.randn(4, 64, 8, 8, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    for _ in range(5):
        bn(x, relu=True)
    assert int(bn.state_dict()["num_batches_tracked"]) == 5
    assert int(bn.state_dict()["num_batches_tracked"]) == 5
    set_backend("torch")
    bn(x.float())
    set_backend("own")
    assert int(bn.num_batches_tracked) == 6
