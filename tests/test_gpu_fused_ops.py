"""Single-pass element-wise kernels of the decoder stack against plain PyTorch fp32 references, forward and backward."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from hccl_b200.ops import fused


def _close(a, b, tol):
    scale = b.float().abs().max().item() + 1e-6
    err = (a.float() - b.float()).abs().max().item()
    assert err <= tol * scale, f"max error {err} vs scale {scale}"


@pytest.mark.parametrize("rows,hidden", [(1, 8), (37, 1024), (512, 8192), (300, 4096 + 64)])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_rms_norm_forward_backward(rows, hidden, with_delta):
    g = torch.Generator(device="cuda").manual_seed(rows + hidden)
    x = torch.randn(rows, hidden, device="cuda", generator=g).bfloat16().requires_grad_()
    delta = (torch.randn(rows, hidden, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_() if with_delta else None
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)).bfloat16().requires_grad_()
    x_out, h = fused.add_rms_norm(x, delta, w, 1e-5)
    up_x = torch.randn(rows, hidden, device="cuda", generator=g).bfloat16()
    up_h = torch.randn(rows, hidden, device="cuda", generator=g).bfloat16()
    ((x_out.float() * up_x.float()).sum() + (h.float() * up_h.float()).sum()).backward()

    xr = x.detach().float().requires_grad_()
    dr = delta.detach().float().requires_grad_() if with_delta else None
    wr = w.detach().float().requires_grad_()
    xo_r = xr if dr is None else xr + dr
    hr = xo_r * torch.rsqrt(xo_r.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    ((xo_r * up_x.float()).sum() + (hr * up_h.float()).sum()).backward()
    _close(x_out, xo_r, 1e-2)
    _close(h, hr, 2e-2)
    _close(x.grad, xr.grad, 3e-2)
    if with_delta:
        _close(delta.grad, dr.grad, 3e-2)
    _close(w.grad, wr.grad, 3e-2)


@pytest.mark.parametrize("rows,f", [(3, 8), (129, 3584), (4096, 1024)])
def test_swiglu_forward_backward(rows, f):
    g = torch.Generator(device="cuda").manual_seed(rows * 7 + f)
    gu = (torch.randn(rows, 2 * f, device="cuda", generator=g) * 2).bfloat16().requires_grad_()
    up = torch.randn(rows, f, device="cuda", generator=g).bfloat16()
    out = fused.swiglu(gu)
    (out.float() * up.float()).sum().backward()
    gr = gu.detach().float().requires_grad_()
    ref = fused.swiglu_reference(gr)
    (ref * up.float()).sum().backward()
    _close(out, ref, 1e-2)
    _close(gu.grad, gr.grad, 2e-2)


@pytest.mark.parametrize("s,heads,d,extra", [(5, 1, 16, 0), (257, 8, 128, 2 * 128), (1024, 2, 64, 64)])
def test_rope_forward_backward_on_a_column_slice(s, heads, d, extra):
    """The input is a column slice of a wider projection output (row stride heads * d + extra)."""
    g = torch.Generator(device="cuda").manual_seed(s + heads + d)
    wide = torch.randn(s, heads * d + extra, device="cuda", generator=g).bfloat16().requires_grad_()
    ang = torch.rand(s, d // 2, device="cuda", generator=g) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    up = torch.randn(s, heads, d, device="cuda", generator=g).bfloat16()
    out = fused.rope(wide[:, :heads * d].view(s, heads, d), cos, sin)
    (out.float() * up.float()).sum().backward()
    wr = wide.detach().float().requires_grad_()
    ref = fused.rope_reference(wr[:, :heads * d].view(s, heads, d), cos, sin)
    (ref * up.float()).sum().backward()
    _close(out, ref, 1e-2)
    _close(wide.grad, wr.grad, 2e-2)


def test_fallback_shapes_take_the_reference_path():
    x = torch.randn(4, 12, device="cuda").bfloat16()          # hidden not a multiple of 8
    w = torch.ones(12, device="cuda").bfloat16()
    _, h = fused.add_rms_norm(x, None, w)
    _close(h, fused.add_rms_norm_reference(x.float(), None, w.float(), 1e-5)[1], 2e-2)
