"""The hand-written backward passes of the DiT workload agree with autograd (CPU, float64 where possible)."""
import torch
import torch.nn.functional as F

from flame_b200 import dit_workload as W
from flame_b200.checkpoint import dense_permutation


def test_rope_backward_is_the_inverse_rotation():
    torch.manual_seed(0)
    x = torch.randn(2, 16, 3, W.HEAD_DIM, dtype=torch.float64, requires_grad=True)
    ang = torch.rand(16, W.HEAD_DIM // 2, dtype=torch.float64)
    cos, sin = ang.cos(), ang.sin()
    assert torch.autograd.gradcheck(lambda t: W.RoPEFn.apply(t, cos, sin), (x,))
    (g,) = torch.autograd.grad(W._rotate(x, cos, sin).sin().sum(), x)
    (h,) = torch.autograd.grad(W.RoPEFn.apply(x, cos, sin).sin().sum(), x)
    assert torch.allclose(g, h)


def test_rmsnorm_backward_from_its_output():
    torch.manual_seed(0)
    x = torch.randn(3, 5, 32, dtype=torch.float64, requires_grad=True)
    w = (torch.rand(32, dtype=torch.float64) + 0.5).requires_grad_(True)

    def ref(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w

    gx, gw = torch.autograd.grad(ref(x, w).cos().sum(), (x, w))
    hx, hw = torch.autograd.grad(W.RMSNormFn.apply(x, w, 1e-6).double().cos().sum(), (x, w))
    # the function computes in float32 internally
    assert torch.allclose(gx, hx.double(), atol=1e-5) and torch.allclose(gw, hw.double(), atol=1e-4)


def test_swiglu_down_backward_recomputes_the_hidden_state():
    torch.manual_seed(0)
    gu = torch.randn(2, 7, 24, dtype=torch.float32, requires_grad=True)
    wd = torch.randn(6, 12, dtype=torch.float32, requires_grad=True)

    def ref(gu, wd):
        g, u = gu.chunk(2, dim=-1)
        return (F.silu(g) * u) @ wd.t()

    a = torch.autograd.grad(ref(gu, wd).tanh().sum(), (gu, wd))
    b = torch.autograd.grad(W.SwiGLUDownFn.apply(gu, wd).tanh().sum(), (gu, wd))
    assert all(torch.allclose(p, q, atol=1e-5) for p, q in zip(a, b))


def test_dense_permutation():
    t = torch.zeros(2, 6, 4, 8)
    assert dense_permutation(t) == (0, 1, 2, 3)
    v = t.transpose(1, 2)
    p = dense_permutation(v)
    assert p is not None and v.permute(p).is_contiguous() and v.permute(p).data_ptr() == v.data_ptr()
    assert dense_permutation(t[:, :, :2]) is None        # a slice is not dense
    assert dense_permutation(t[..., 0]) is None
