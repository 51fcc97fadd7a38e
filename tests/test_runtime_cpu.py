"""Host-side logic of the two per-step shortcuts of the training path, on CPU tensors: the bf16 weight copies kept by
the optimizer kernels (kernels.bf16_weight) and the gradient targets inside DDP's bucket views
(kernels.take_grad_view / _grad_target)."""
import torch

from gcow_b200.ops import kernels as K


def test_bf16_weight_uses_a_current_copy_and_refreshes_a_stale_one():
    w = torch.nn.Parameter(torch.randn(8, 16))
    assert K.bf16_weight(w).dtype == torch.bfloat16                  # no copy kept: a plain cast
    w._gcow_bf16 = torch.empty_like(w, dtype=torch.bfloat16)
    w._gcow_bf16_version = -1                                        # never written
    got = K.bf16_weight(w)
    assert got is w._gcow_bf16 and torch.equal(got, w.detach().to(torch.bfloat16))
    assert w._gcow_bf16_version == w._version
    w._gcow_bf16.zero_()                                             # stands for "the update kernel wrote it"
    assert K.bf16_weight(w) is w._gcow_bf16 and not K.bf16_weight(w).any()     # current: handed out as it is
    with torch.no_grad():
        w.mul_(2.0)                                                  # somebody else wrote the parameter
    assert torch.equal(K.bf16_weight(w), w.detach().to(torch.bfloat16))


def test_grad_view_is_taken_once_and_only_when_it_fits():
    w = torch.nn.Parameter(torch.randn(8, 4, 3, 3).contiguous(memory_format=torch.channels_last))
    view = torch.zeros_like(w, memory_format=torch.preserve_format)
    w._gcow_grad_view = view
    taken = K.take_grad_view(w)
    assert taken is not None and K.take_grad_view(w) is None         # a second user of the weight gets nothing
    flat, alias = K._grad_target(taken, 8, 36)
    assert flat is not None and flat.shape == (8, 36) and flat.data_ptr() == view.data_ptr()
    assert alias is not view and alias.data_ptr() == view.data_ptr() and alias.stride() == w.stride()
    flat.fill_(3.0)
    assert float(alias.sum()) == 3.0 * w.numel()                     # what the kernel writes is what autograd gets
    # wrong element count, a gradient already present (accumulation), a wrong dtype: no target
    assert K._grad_target(taken, 8, 35) == (None, None)
    w.grad = torch.zeros_like(w)
    assert K._grad_target(taken, 8, 36) == (None, None)
    w.grad = None
    w._gcow_grad_view = view.double()
    assert K.take_grad_view(w) is None


def test_grad_target_respects_the_kernel_alignment():
    base = torch.zeros(64 + 1)
    w = torch.nn.Parameter(torch.randn(64))
    w._gcow_grad_view = base[1:]                                     # 4 bytes past an aligned address
    taken = K.take_grad_view(w)
    assert K._grad_target(taken, 1, 64, align=16) == (None, None)
    flat, alias = K._grad_target(taken, 1, 64, align=4)
    assert flat is not None and alias.shape == w.shape
