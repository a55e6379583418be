"""The tcgen05 / TMEM matmul against a plain PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from hccl_b200.ops import mc2


def _ref(a, b, ta, tb):
    A = a.float().t() if ta else a.float()
    B = b.float().t() if tb else b.float()
    return A @ B


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (256, 512, 512), (384, 768, 1024), (1000, 520, 328), (16, 128, 1024),
                                   (2048, 3584, 2048)])
def test_matmul_layouts(ta, tb, m, n, k):
    if ta and m % 8:
        pytest.skip("transposed A needs M % 8 == 0")
    torch.manual_seed(m * 7 + n * 3 + k)
    a = (torch.randn((k, m) if ta else (m, k), device="cuda") * 0.5).bfloat16()
    b = (torch.randn((n, k) if tb else (k, n), device="cuda") * 0.5).bfloat16()
    out = mc2.matmul(a, b, trans_a=ta, trans_b=tb)
    torch.cuda.synchronize()
    ref = _ref(a, b, ta, tb)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-2 * scale + 1e-2, f"max err {err} (scale {scale})"


def test_matmul_repeated_launches_and_values():
    a = torch.eye(256, device="cuda").bfloat16()
    b = torch.arange(256 * 256, device="cuda").reshape(256, 256).remainder(97).bfloat16()   # [N, K]
    for _ in range(5):
        out = mc2.matmul(a, b)
        torch.cuda.synchronize()
        assert torch.equal(out, b.t().contiguous())
