"""The allocation-free MoE entry point against the regular one.

Collected last on purpose: if it fails, a run that stops at the first failure has already run
every other test.  It goes through the C ABI directly (ctypes), not through the Python operators.
"""
import numpy as np
import pytest
import torch

import ojasx_b200
from ojasx_b200 import ops, synth

pytestmark = pytest.mark.gpu


def _call(fn, h, x, idx, w, y):
    rc = fn(h, x.data_ptr(), idx.data_ptr(), w.data_ptr(), y.data_ptr(), x.shape[0], idx.shape[1], 0,
            torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc


def test_no_alloc_moe_matches_regular_entry_point_twice(cuda):
    """Two calls in a row (different tokens, different routing) must each equal the regular entry
    point: the static scratch keeps the first call's contents when the second one starts."""
    L = ojasx_b200.lib()
    w = synth.make_vq_moe(41, 32, 2560, 640, block_dim=8, outlier_frac=0.0038, unit_scales=False)
    moe = ops.VQMoE(w)
    rng = np.random.default_rng(6)
    for call, B in enumerate((8, 3)):          # 80 pairs (just under the limit), then 30 pairs
        x = torch.from_numpy(rng.standard_normal((B, 2560)).astype(np.float32)).to(cuda)
        idx = torch.from_numpy(np.stack([rng.choice(32, 10, replace=False) for _ in range(B)]).astype(np.int32)).to(cuda)
        wts = torch.from_numpy(rng.uniform(0.02, 0.3, (B, 10)).astype(np.float32)).to(cuda)
        if call == 1:
            idx[0, 2] = -1                      # a skipped pair: its stale scratch slot must not leak in
        want = torch.full_like(x, float("nan"))
        got = torch.full_like(x, float("nan"))
        assert _call(L.ojasx_b200_moe_forward, moe.handle, x, idx, wts, want) == 0
        assert _call(L.ojasx_b200_moe_forward_noalloc, moe.handle, x, idx, wts, got) == 0
        g, r = got.cpu().numpy(), want.cpu().numpy()
        assert np.all(np.isfinite(g))
        # same kernels, same order: the tolerance of the MoE tests (rel 1e-5 / abs 1e-6) is met with equality
        assert np.all(np.abs(g - r) <= 1e-6 + 1e-5 * np.abs(r))
        assert np.array_equal(g, r)


def test_no_alloc_moe_rejects_sizes_beyond_the_static_scratch(cuda):
    L = ojasx_b200.lib()
    w = synth.make_vq_moe(42, 4, 2560, 640, block_dim=8, outlier_frac=0.0)
    moe = ops.VQMoE(w)
    B = 9                                        # 90 pairs * 3200 floats > 262144
    x = torch.zeros(B, 2560, device=cuda)
    idx = torch.zeros(B, 10, dtype=torch.int32, device=cuda)
    wts = torch.ones(B, 10, device=cuda)
    y = torch.full_like(x, 7.0)
    assert _call(L.ojasx_b200_moe_forward_noalloc, moe.handle, x, idx, wts, y) == -5
    assert b"exceeds" in L.ojasx_b200_last_error()
    assert torch.all(y == 7.0)                   # rejected calls touch nothing
    assert L.ojasx_b200_moe_forward_noalloc(None, None, None, None, None, 1, 1, 0, None) == -1
