"""Implicit-GEMM convolution (forward, data gradient, weight gradient) against an fp32
PyTorch convolution of the same bf16-rounded operands."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

# (N, Ci, H, W, Co, kh, kw, pad_h, pad_w): whole boxes, ragged edges, narrow and wide channel counts,
# a filter without padding, an even filter and an asymmetric one
CASES = [
    (4, 64, 16, 16, 64, 3, 3, 1, 1),
    (3, 64, 9, 7, 128, 3, 3, 1, 1),
    (2, 128, 14, 14, 256, 3, 3, 1, 1),
    (5, 64, 7, 7, 320, 3, 3, 1, 1),
    (2, 64, 12, 10, 64, 3, 3, 0, 0),
    (2, 64, 11, 13, 64, 5, 5, 2, 2),
    (2, 64, 10, 10, 64, 2, 2, 1, 1),
    (2, 192, 8, 9, 64, 1, 3, 0, 1),
    # 64 -> 64 channels, 3x3, padding 1: the weight-stationary kernel (several tiles per image, ragged last tile,
    # an image smaller than one tile)
    (2, 64, 56, 56, 64, 3, 3, 1, 1),
    (3, 64, 30, 20, 64, 3, 3, 1, 1),
    (1, 64, 7, 9, 64, 3, 3, 1, 1),
    # the widest rows the halo-tile weight gradient takes, and one column more (general weight gradient)
    (5, 64, 13, 62, 64, 3, 3, 1, 1),
    (2, 64, 5, 63, 64, 3, 3, 1, 1),
    # enough tiles for the two-accumulator forward tile with 128 output channels: the operand-swapped MMA
    # (channels as M, 256 pixels as N); ragged 245-pixel boxes and whole ones
    (40, 128, 28, 28, 128, 3, 3, 1, 1),
    (48, 64, 20, 20, 128, 3, 3, 1, 1),
]


def _mk(N, Ci, H, W, Co, kh, kw):
    x = (torch.randn(N, Ci, H, W, device="cuda") * 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    w = (torch.randn(Co, Ci, kh, kw, device="cuda") * 0.1).bfloat16().float().contiguous(memory_format=torch.channels_last)
    b = torch.randn(Co, device="cuda") * 0.1
    return x, w, b


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


@pytest.mark.parametrize("case", CASES)
def test_conv_igemm_forward_and_gradients(case):
    from gcow_b200.ops import kernels as K
    N, Ci, H, W, Co, kh, kw, ph, pw = case
    torch.manual_seed(sum(case))
    x, w, b = _mk(N, Ci, H, W, Co, kh, kw)
    xr = x.float().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    br = b.clone().requires_grad_(True)
    ref = F.conv2d(xr, wr, br, stride=1, padding=(ph, pw))
    gy = (torch.randn_like(ref) * 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    ref.backward(gy.float())

    xo = x.clone().requires_grad_(True)
    wo = w.clone().requires_grad_(True)
    bo = b.clone().requires_grad_(True)
    assert K.conv_igemm_usable(xo, wo, (1, 1), (ph, pw), 1, (1, 1))
    y = K.conv_igemm(xo, wo, bo, (ph, pw))
    K.check_errors()
    assert y.shape == ref.shape and y.dtype == torch.bfloat16
    assert _rel(y, ref) < 2e-2
    y.backward(gy)
    K.check_errors()
    assert _rel(xo.grad, xr.grad) < 2e-2
    assert wo.grad.dtype == torch.float32 and wo.grad.shape == wr.grad.shape
    assert _rel(wo.grad, wr.grad) < 5e-3
    assert _rel(bo.grad, br.grad) < 5e-3


# (N, Ci, H, W, Co): whole boxes, ragged pixel boxes, more output than input channels and the reverse
def test_weight_stationary_kernel_serves_the_64_channel_layers_and_agrees_with_the_general_one(monkeypatch):
    from gcow_b200.ops import kernels as K
    N, H, W = 3, 56, 56
    assert K.conv_ws_usable(N, H, W, 64, 64, 3, 3, 1, 1)
    assert not K.conv_ws_usable(N, H, W, 64, 128, 3, 3, 1, 1) and not K.conv_ws_usable(N, H, W, 64, 64, 3, 3, 0, 0)
    torch.manual_seed(5)
    x, w, b = _mk(N, 64, H, W, 64, 3, 3)
    gy = (torch.randn(N, 64, H, W, device="cuda") * 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    outs = []
    for ws in ("1", "0"):
        monkeypatch.setenv("GCOW_CONV_WS", ws)
        monkeypatch.setenv("GCOW_CONV_WS_WGRAD", ws)
        xo = x.clone().requires_grad_(True)
        wo = w.clone().requires_grad_(True)
        y = K.conv_igemm(xo, wo, None, (1, 1))
        y.backward(gy)
        K.check_errors()
        outs.append((y.detach().float(), xo.grad.float(), wo.grad.float()))
    # the same bf16 operands, fp32 accumulation in another order: equal up to the output rounding
    assert _rel(outs[0][0], outs[1][0]) < 1e-2 and _rel(outs[0][1], outs[1][1]) < 1e-2
    assert _rel(outs[0][2], outs[1][2]) < 1e-4
    lib = K._native.cuda()
    assert lib.gcow_conv_wgrad_ws_split(N, H, W) > 1 and lib.gcow_conv_wgrad_ws_split(N, H, 63) == 0


def test_operand_swapped_forward_agrees_with_the_plain_one(monkeypatch):
    import ctypes
    from gcow_b200.ops import kernels as K
    N, C, H, W, Co = 40, 128, 28, 28, 128
    plan = (ctypes.c_int * 6)()
    K._native.cuda().gcow_conv_fwd_plan(N, H, W, C, Co, 3, 3, 1, 1, 148, plan)
    assert plan[0] == 2 and plan[1] == 128                        # the tile shape that swaps
    torch.manual_seed(6)
    x, w, b = _mk(N, C, H, W, Co, 3, 3)
    monkeypatch.setenv("GCOW_CONV_HALO", "0")                     # this shape would otherwise take the halo-tile kernel
    outs = []
    lib = K._native.cuda()
    try:
        for swap in (1, 0):
            lib.gcow_conv_set_swap(swap)
            y = K.conv_igemm(x, w, b, (1, 1))
            K.check_errors()
            outs.append(y.float())
    finally:
        lib.gcow_conv_set_swap(1)
    assert _rel(outs[0], outs[1]) < 1e-2


@pytest.mark.parametrize("shape", [(40, 128, 28, 28), (3, 64, 30, 20), (2, 128, 9, 11), (1, 192, 5, 6)])
def test_halo_tile_forward_agrees_with_the_general_kernel(shape, monkeypatch):
    from gcow_b200.ops import kernels as K
    N, C, H, W = shape
    assert K.conv_halo_usable(N, H, W, C, 128, 3, 3, 1, 1)
    # other output widths, and tiles too large for two pixel stages, stay on the general kernel
    assert not K.conv_halo_usable(N, H, W, C, 256, 3, 3, 1, 1) and not K.conv_halo_usable(2, 28, 28, 512, 128, 3, 3, 1, 1)
    torch.manual_seed(7)
    x, w, b = _mk(N, C, H, W, 128, 3, 3)
    outs = []
    for halo in ("1", "0"):
        monkeypatch.setenv("GCOW_CONV_HALO", halo)
        y = K.conv_igemm(x, w, b, (1, 1))
        K.check_errors()
        outs.append(y.float())
    assert _rel(outs[0], outs[1]) < 1e-2


@pytest.mark.parametrize("shape", [(40, 28, 28, 128, 128), (3, 10, 20, 128, 128), (2, 9, 40, 128, 128), (1, 3, 62, 128, 128),
                                   (2, 5, 1, 128, 128), (9, 14, 14, 256, 256), (3, 13, 11, 128, 384), (2, 7, 12, 256, 128)])
def test_halo_tile_weight_gradient_of_128_channel_layers(shape, monkeypatch):
    from gcow_b200.ops import kernels as K
    N, H, W, Ci, Co = shape
    monkeypatch.setattr(K, "_HALO_WGRAD_MIN_W", 1)
    assert K._native.cuda().gcow_conv_wgrad_halo_split(N, H, W, Ci, Co) >= 1
    assert K._native.cuda().gcow_conv_wgrad_halo_split(N, H, 63, Ci, Co) == 0
    assert K._native.cuda().gcow_conv_wgrad_halo_split(N, H, W, 64, Co) == 0
    torch.manual_seed(8)
    x, w, _ = _mk(N, Ci, H, W, Co, 3, 3)
    gy = (torch.randn(N, Co, H, W, device="cuda") * 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    wr = w.clone().requires_grad_(True)
    F.conv2d(x.float(), wr, None, padding=1).backward(gy.float())
    grads = []
    for halo in ("1", "0"):
        monkeypatch.setenv("GCOW_CONV_HALO_WGRAD", halo)
        wo = w.clone().requires_grad_(True)
        K.conv_igemm(x, wo, None, (1, 1)).backward(gy)
        K.check_errors()
        grads.append(wo.grad.float())
    assert _rel(grads[0], wr.grad) < 5e-3 and _rel(grads[0], grads[1]) < 1e-4


S2_CASES = [(4, 64, 16, 16, 64), (3, 64, 10, 14, 128), (2, 128, 28, 28, 128), (5, 256, 6, 8, 64), (2, 64, 2, 2, 64)]


@pytest.mark.parametrize("case", S2_CASES)
def test_conv_igemm_stride2_forward_and_gradients(case):
    """3x3, stride 2, padding 1 on the implicit-GEMM kernel (strided tensor maps; the input gradient as four parity
    phases) against an fp32 PyTorch convolution of the same bf16-rounded operands."""
    from gcow_b200.ops import kernels as K
    N, Ci, H, W, Co = case
    torch.manual_seed(sum(case))
    x, w, b = _mk(N, Ci, H, W, Co, 3, 3)
    xr = x.float().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    br = b.clone().requires_grad_(True)
    ref = F.conv2d(xr, wr, br, stride=2, padding=1)
    gy = (torch.randn_like(ref) * 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    ref.backward(gy.float())
    xo = x.clone().requires_grad_(True)
    wo = w.clone().requires_grad_(True)
    bo = b.clone().requires_grad_(True)
    assert K.conv_igemm_s2_usable(xo, wo, (2, 2), (1, 1), 1, (1, 1))
    y = K.conv_igemm_s2(xo, wo, bo)
    K.check_errors()
    assert y.shape == ref.shape and y.dtype == torch.bfloat16
    assert _rel(y, ref) < 2e-2
    y.backward(gy)
    K.check_errors()
    assert _rel(xo.grad, xr.grad) < 2e-2
    assert _rel(wo.grad, wr.grad) < 5e-3
    assert _rel(bo.grad, br.grad) < 5e-3


def test_conv_igemm_resnet_layer_shape():
    """One ResNet-50 3x3 layer at a batch that needs several waves of tiles and every split of the weight gradient."""
    from gcow_b200.ops import kernels as K
    torch.manual_seed(5)
    N, C, HW = 32, 128, 28
    x, w, _ = _mk(N, C, HW, HW, C, 3, 3)
    xr, wr = x.float().requires_grad_(True), w.clone().requires_grad_(True)
    ref = F.conv2d(xr, wr, None, padding=1)
    gy = (torch.randn_like(ref) * 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    ref.backward(gy.float())
    xo, wo = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y = K.conv_igemm(xo, wo, None, (1, 1))
    y.backward(gy)
    K.check_errors()
    assert _rel(y, ref) < 2e-2 and _rel(xo.grad, xr.grad) < 2e-2 and _rel(wo.grad, wr.grad) < 5e-3


def test_conv2d_module_uses_igemm_by_default(monkeypatch):
    from gcow_b200.ops import kernels as K, nn as gnn, set_backend
    monkeypatch.delenv("GCOW_CONV", raising=False)
    set_backend("own")
    torch.manual_seed(6)
    conv = gnn.Conv2d(64, 64, 3, padding=1, bias=False).cuda().to(memory_format=torch.channels_last)
    x = torch.randn(4, 64, 14, 14, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    before = K.launch_count()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = conv(x)
    assert K.launch_count() == before + 1 and gnn.last_conv_path() == "igemm"
    ref = F.conv2d(x.float(), conv.weight.bfloat16().float(), padding=1)
    assert _rel(y, ref) < 2e-2
    monkeypatch.setenv("GCOW_CONV", "lib")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        conv(x)
    assert gnn.last_conv_path() == "cudnn"


# (Ci, Co, k, stride, pad, H, input needs a gradient, expected path): the layer kinds of a ResNet that the
# implicit-GEMM kernel does not serve
MODULE_CASES = [
    (64, 256, 1, 1, 0, 14, True, "gemm1x1"),
    (256, 64, 1, 1, 0, 14, True, "gemm1x1"),
    (256, 512, 1, 2, 0, 14, True, "igemm1x1_s2"),
    (64, 128, 1, 2, 0, 15, True, "igemm1x1_s2"),         # odd extent: the last sampled pixel is the last pixel
    (72, 128, 1, 2, 0, 14, True, "gemm1x1_strided"),     # 72 channels: not whole 64-channel rows
    (128, 128, 3, 2, 1, 14, True, "igemm_s2"),
    (64, 128, 3, 2, 1, 15, True, "im2col"),          # odd extent: not covered by the stride-2 implicit GEMM
    (96, 128, 3, 2, 1, 14, True, "im2col"),          # 96 input channels: not whole 64-channel rows
    (3, 64, 7, 2, 3, 32, False, "im2col"),
    (3, 64, 3, 1, 1, 16, False, "im2col"),
]


@pytest.mark.parametrize("case", MODULE_CASES)
def test_conv2d_module_paths_match_fp32_reference(case, monkeypatch):
    from gcow_b200.ops import kernels as K, nn as gnn, set_backend
    monkeypatch.delenv("GCOW_CONV", raising=False)
    set_backend("own")
    Ci, Co, k, s, p, H, xgrad, path = case
    torch.manual_seed(sum(case[:6]))
    conv = gnn.Conv2d(Ci, Co, k, stride=s, padding=p, bias=False).cuda().to(memory_format=torch.channels_last)
    with torch.no_grad():
        conv.weight.copy_(conv.weight.bfloat16().float())
    x = (torch.randn(8, Ci, H, H, device="cuda") * 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    xo = x.clone().requires_grad_(xgrad)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = conv(xo)
    assert gnn.last_conv_path() == path
    xr = x.float().requires_grad_(xgrad)
    wr = conv.weight.detach().clone().requires_grad_(True)
    ref = F.conv2d(xr, wr, None, stride=s, padding=p)
    assert y.shape == ref.shape and _rel(y, ref) < 2e-2
    gy = (torch.randn_like(ref) * 0.5).bfloat16()
    y.backward(gy.to(y.dtype))
    ref.backward(gy.float())
    K.check_errors()
    assert _rel(conv.weight.grad, wr.grad) < 1e-2
    if xgrad:
        assert _rel(xo.grad, xr.grad) < 2e-2


def test_resnet50_step_sends_no_convolution_to_cudnn(monkeypatch):
    """All 53 convolutions of ResNet-50 (hw/models/resenet.py:11-17,79,113 in the reference) run on this library's
    kernels by default, forward and backward."""
    from gcow_b200.models import MODELS
    from gcow_b200.ops import kernels as K, set_backend
    monkeypatch.delenv("GCOW_CONV", raising=False)
    set_backend("own")
    torch.manual_seed(0)
    net = MODELS["resnet50"](num_classes=16).cuda().to(memory_format=torch.channels_last)
    x = torch.randn(8, 3, 224, 224, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    K.conv_path_counts(reset=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = net(x).float().square().mean()
    loss.backward()
    K.check_errors()
    counts = K.conv_path_counts(reset=True)
    assert sum(counts.values()) == 53 and counts.get("cudnn", 0) == 0, counts
    assert (counts["gemm1x1"] == 33 and counts["igemm1x1_s2"] == 3 and counts["igemm"] == 13
            and counts["igemm_s2"] == 3 and counts["im2col"] == 1)
    # at batch 256 the 1x1 layers of the 56 x 56 stage move to the one-tap implicit GEMM (a routing rule on the pixel count)
    big = torch.empty(256, 64, 56, 56, device="meta")
    assert K._onebyone_on_igemm(big) and not K._onebyone_on_igemm(x)
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in net.parameters())
