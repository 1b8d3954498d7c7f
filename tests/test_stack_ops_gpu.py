"""The small per-token operators of a decoder step (RMSNorm with the residual add folded in, rotary embedding at
device-side positions, position bump) against plain torch formulas; fp32 tolerance of the path, bf16 rel 2e-2."""
import numpy as np
import pytest
import torch

from ojasx_b200 import ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,hidden", [(1, 2560), (5, 2560), (3, 100), (2, 5000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_with_and_without_residual(cuda, rows, hidden, dtype):
    g = torch.Generator(device=cuda).manual_seed(rows + hidden)
    x = torch.randn(rows, hidden, device=cuda, generator=g).to(dtype)
    add = torch.randn(rows, hidden, device=cuda, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, device=cuda, generator=g)).float()

    def ref(v):
        v = v.float()
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * w

    tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    got = ops.rmsnorm(x.clone(), w, 1e-6)
    assert torch.allclose(got.float(), ref(x), **tol)
    xs = x.clone()
    got = ops.rmsnorm(xs, w, 1e-6, add=add)
    summed = (x.float() + add.float()).to(dtype)
    assert torch.equal(xs, summed)                      # the residual stream is updated in place, rounded once
    assert torch.allclose(got.float(), ref(summed), **tol)


def test_rope_and_position_bump(cuda):
    B, Hq, Hkv, hd, theta = 3, 8, 2, 64, 1e6
    g = torch.Generator(device=cuda).manual_seed(1)
    q = torch.randn(B, Hq, hd, device=cuda, generator=g)
    k = torch.randn(B, Hkv, hd, device=cuda, generator=g)
    pos = torch.tensor([0, 7, 1023], dtype=torch.int32, device=cuda)

    def ref(t):
        half = hd // 2
        inv = 1.0 / (theta ** (torch.arange(half, device=cuda, dtype=torch.float64) * 2 / hd))
        ang = pos.double()[:, None, None] * inv
        c, s = torch.cos(ang), torch.sin(ang)
        t = t.double()
        return torch.cat([t[..., :half] * c - t[..., half:] * s, t[..., half:] * c + t[..., :half] * s], -1)

    q2, k2 = q.clone(), k.clone()
    ops.rope_qk_(q2, k2, pos, theta)
    assert torch.allclose(q2.double(), ref(q), rtol=1e-4, atol=1e-4)
    assert torch.allclose(k2.double(), ref(k), rtol=1e-4, atol=1e-4)
    ops.add_int_(pos, 5)
    assert pos.tolist() == [5, 12, 1028]
