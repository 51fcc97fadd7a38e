"""tcgen05 bf16 GEMM against an fp32 PyTorch reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, bias=None, residual=None, gelu=False):
    y = a.float() @ b.float().t()
    if bias is not None:
        y = y + bias
    if gelu:
        y = torch.nn.functional.gelu(y)
    if residual is not None:
        y = y + residual.float()
    return y


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 1024), (300, 520, 136),
                                   (4096, 1000, 2048), (77, 40, 72), (1024, 3072, 1024)])
def test_gemm_matches_fp32_reference(M, N, K):
    from gcow_b200.ops import kernels as K_
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    ref = _ref(a, b)
    for dt in (torch.float32, torch.bfloat16):
        for rows in (128, 256):                      # both tile shapes
            y = K_.gemm_bf16(a, b, out_dtype=dt, tile_rows=rows)
            K_.check_errors()
            tol = 2e-2 if dt == torch.bfloat16 else 1e-3
            err = (y.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
            assert err < tol, (dt, rows, err)


def test_gemm_epilogues():
    from gcow_b200.ops import kernels as K_
    torch.manual_seed(0)
    M, N, K = 512, 768, 256
    a = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.3).bfloat16()
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda").bfloat16()
    ref = _ref(a, b, bias, res, True)
    for rows in (128, 256):
        y = K_.gemm_bf16(a, b, bias=bias, gelu=True, residual=res, tile_rows=rows)
        K_.check_errors()
        assert (y.float() - ref).abs().max().item() < 0.06
    acc = torch.ones(M, N, device="cuda")
    K_.gemm_bf16(a, b, out=acc, accumulate=True)
    assert (acc - (_ref(a, b) + 1)).abs().max().item() < 2e-2


def test_strided_operands_and_small_grid():
    from gcow_b200.ops import kernels as K_
    big = (torch.randn(640, 512, device="cuda") * 0.5).bfloat16()
    a = big[:, :256]                      # leading dimension 512, K 256
    b = (torch.randn(1024, 256, device="cuda") * 0.5).bfloat16()
    y = K_.gemm_bf16(a, b, out_dtype=torch.float32, max_ctas=3, tile_rows=256)   # several tiles per CTA
    K_.check_errors()
    assert (y - _ref(a, b)).abs().max().item() < 2e-2
    y = K_.gemm_bf16(a, b, out_dtype=torch.float32, max_ctas=3, tile_rows=128)
    K_.check_errors()
    assert (y - _ref(a, b)).abs().max().item() < 2e-2


def test_linear_autograd_matches_torch():
    from gcow_b200.ops import kernels as K_
    torch.manual_seed(1)
    x = torch.randn(4, 64, 256, device="cuda", requires_grad=True)
    w = (torch.randn(384, 256, device="cuda") * 0.05).requires_grad_(True)
    b = torch.zeros(384, device="cuda", requires_grad=True)
    y = K_.linear(x, w, b)
    y.float().square().mean().backward()
    K_.check_errors()
    gx, gw, gb = x.grad.clone(), w.grad.clone(), b.grad.clone()
    x.grad = w.grad = b.grad = None
    yr = torch.nn.functional.linear(x, w, b)
    yr.square().mean().backward()
    assert (y.float() - yr).abs().max().item() < 0.05
    for g, r in ((gx, x.grad), (gw, w.grad), (gb, b.grad)):
        assert (g.float() - r).abs().max().item() <= 0.03 * r.abs().max().item() + 1e-6


@pytest.mark.parametrize("M,N,K", [(256, 512, 320), (304, 520, 136), (1024, 1024, 4096)])
def test_transposed_operands_without_copies(M, N, K):
    """dgrad (B stored [K,N]) and wgrad (both operands stored [K,rows]) layouts."""
    from gcow_b200.ops import kernels as K_
    torch.manual_seed(7)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    ref = _ref(a, b)
    bt = b.t().contiguous()          # stored [K, N]
    at = a.t().contiguous()          # stored [K, M]
    scale = ref.abs().max().item()
    for rows in (128, 256):
        y1 = K_.gemm_bf16(a, bt, b_t=True, out_dtype=torch.float32, tile_rows=rows)
        y2 = K_.gemm_bf16(at, bt, a_t=True, b_t=True, out_dtype=torch.float32, tile_rows=rows)
        y3 = K_.gemm_bf16(at, b, a_t=True, out_dtype=torch.float32, tile_rows=rows)
        K_.check_errors()
        for y in (y1, y2, y3):
            assert (y - ref).abs().max().item() < 1e-3 * scale + 1e-3


def test_wgrad_split_k_matches_reference():
    from gcow_b200.ops import kernels as K_
    torch.manual_seed(9)
    for M, N, K in ((8192, 256, 512), (16384, 1024, 1024), (4096, 64, 2304), (1000, 256, 256)):
        g = (torch.randn(M, N, device="cuda") * 0.3).bfloat16()
        x = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
        ref = g.float().t() @ x.float()
        y = K_.wgrad_gemm(g, x)
        K_.check_errors()
        assert y.shape == (N, K) and (y - ref).abs().max().item() < 2e-3 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("M,N,K", [(1024, 512, 256), (2048, 1024, 1024), (1100, 288, 192), (4096, 4096, 64)])
def test_pair_gemm_matches_fp32_reference(M, N, K, monkeypatch):
    """The CTA-pair kernel (cta_group::2) incl. ragged edges, a K that is not a whole stage, and every epilogue."""
    from gcow_b200 import _native
    from gcow_b200.ops import kernels as K_
    if not hasattr(_native.cuda(), "gcow_gemm2_bf16") or _native.cuda().gcow_gemm2_max_pairs() <= 0:
        pytest.skip("clusters of two CTAs cannot be scheduled here")
    monkeypatch.setattr(K_, "_pair_gemm", True)
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda").bfloat16()
    before = K_.launch_count()
    y = K_.gemm_bf16(a, b)
    K_.check_errors()
    ref = _ref(a, b)
    assert (y.float() - ref).abs().max().item() / ref.abs().max().item() < 2e-2
    y = K_.gemm_bf16(a, b, bias=bias, residual=res)
    ref2 = _ref(a, b, bias=bias, residual=res)
    assert (y.float() - ref2).abs().max().item() / ref2.abs().max().item() < 2e-2
    pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    act = K_.gemm_bf16(a, b, bias=bias, gelu=True, pre_gelu_out=pre)
    K_.check_errors()
    ref_pre = _ref(a, b, bias=bias)
    assert (pre.float() - ref_pre).abs().max().item() / ref_pre.abs().max().item() < 2e-2
    ref_act = torch.nn.functional.gelu(ref_pre)
    assert (act.float() - ref_act).abs().max().item() / ref_act.abs().max().item() < 2e-2
    g = K_.gemm_bf16(a, b, gelu_grad_of=pre)
    x = pre.float()
    ref_g = ref * (0.5 * (1 + torch.erf(x / 2 ** 0.5)) + x * torch.exp(-0.5 * x * x) / (2 * 3.141592653589793) ** 0.5)
    assert (g.float() - ref_g).abs().max().item() / ref_g.abs().max().item() < 2e-2
    K_.check_errors()
    assert K_.launch_count() == before + 4
    if N % 64 == 0:        # B stored [K][N]: the data-gradient layout
        y = K_.gemm_bf16(a, b.t().contiguous(), b_t=True, residual=res)
        K_.check_errors()
        ref3 = _ref(a, b, residual=res)
        assert (y.float() - ref3).abs().max().item() / ref3.abs().max().item() < 2e-2
