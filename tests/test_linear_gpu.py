"""GPU parity of the VQ linear path against the CPU oracle (bit-exact: the kernel keeps the
reference's fp32 evaluation order)."""
import numpy as np
import pytest
import torch

import ojasx_b200
from ojasx_b200 import lut_ctypes, ops, synth

pytestmark = pytest.mark.gpu

# in, out, block_dim, scales, bias, outliers
SHAPES = [
    (2560, 2560, 8, False, False, 0.0038),   # BASELINE config 0
    (2560, 6912, 8, False, False, 0.0038),   # gate / up of config 1
    (6912, 2560, 8, True, True, 0.0038),     # down of config 1 (+ scales and bias)
    (256, 128, 16, True, False, 0.0),        # shape of the reference's own linear test
    (64, 32, 16, False, False, 0.03),        # shape of the reference's CSR test
    (640, 2560, 8, False, False, 0.0038),    # expert down projection
    (200, 77, 8, True, True, 0.01),          # G = 25: unaligned rows, ragged tiles
    (96, 33, 4, False, True, 0.0),           # block_dim 4
    (512, 70, 32, True, False, 0.01),        # block_dim 32
]


@pytest.mark.parametrize("K,M,D,sc,bi,frac", SHAPES)
def test_linear_device_bit_exact(cuda, oracle, K, M, D, sc, bi, frac):
    w = synth.make_vq_linear(11 + K + M, K, M, block_dim=D, outlier_frac=frac, with_scales=sc, with_bias=bi)
    x = np.random.default_rng(5).standard_normal((3, K)).astype(np.float32)
    want = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=D)
    layer = ops.VQLinear.from_weights(w)
    got = layer(torch.from_numpy(x).to(cuda)).cpu().numpy()
    assert np.array_equal(got, want), f"max abs diff {np.abs(got - want).max()}"


@pytest.mark.parametrize("K,M,D,batch", [(2560, 6912, 8, 1), (6912, 2560, 8, 3), (2560, 151936 // 8, 8, 1), (640, 2560, 8, 2),
                                         (256, 128, 16, 1), (2560, 1024, 8, 5)])
def test_linear_cluster_and_persistent_kernels_agree(cuda, oracle, monkeypatch, K, M, D, batch):
    """Single problems normally take the cluster kernel; OJASX_B200_LINEAR_KERNEL=persistent forces the
    streaming kernel.  Both must reproduce the oracle bit for bit."""
    w = synth.make_vq_linear(K + M, K, M, block_dim=D, with_scales=True, with_bias=True)
    x = np.random.default_rng(8).standard_normal((batch, K)).astype(np.float32)
    want = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=D)
    layer = ops.VQLinear.from_weights(w)
    xt = torch.from_numpy(x).to(cuda)
    got_default = layer(xt).cpu().numpy()
    monkeypatch.setenv("OJASX_B200_LINEAR_KERNEL", "persistent")
    got_persistent = layer(xt).cpu().numpy()
    assert np.array_equal(got_persistent, want)
    assert np.array_equal(got_default, want)


def test_linear_host_abi_matches_reference_bindings(cuda, oracle):
    """The reference's ctypes class, bound to this library, on host arrays."""
    w = synth.make_vq_linear(3, 2560, 2560, block_dim=8)
    x = np.random.default_rng(1).standard_normal(2560).astype(np.float32)
    layer = lut_ctypes.NativeSplitManifoldLinear(2560, 2560, 8, 256)
    layer.initialize_weights(w.codebook, w.codes, np.ones(2560, np.float32))
    layer.set_outliers(*w.csr)
    got = layer.forward(x)
    want = oracle.linear_forward(w.codebook, w.codes, None, None, w.csr, x, block_dim=8)
    assert got.shape == (2560,)
    assert np.array_equal(got, want)
    assert layer.compressed_bytes == 2560 * 320 + 8192 + 2560 * 4 + len(w.csr[2]) * 8 + 2561 * 4


def test_linear_row_slices_and_bf16(cuda, oracle):
    w = synth.make_vq_linear(9, 2560, 6912, block_dim=8)
    xb = synth.to_bf16_f32(np.random.default_rng(2).standard_normal((4, 2560)).astype(np.float32))
    want = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, xb, block_dim=8)
    layer = ops.VQLinear.from_weights(w)
    xt = torch.from_numpy(xb).to(cuda)
    # row slices (the row-split contract used for sharding): concatenation equals the whole layer
    parts = [layer(xt, r0, r1).cpu().numpy() for r0, r1 in ((0, 864), (864, 3456), (3456, 6912))]
    assert np.array_equal(np.concatenate(parts, axis=1), want)
    # bf16 activations: exact widening, fp32 compute, round-to-nearest-even on the way out
    got = layer(xt.to(torch.bfloat16)).float().cpu().numpy()
    assert np.array_equal(got, synth.to_bf16_f32(want))


def test_linear_group_launch(cuda, oracle):
    ws = [synth.make_vq_linear(100 + i, 2560, 6912 if i % 2 else 2560, block_dim=8) for i in range(5)]
    layers = [ops.VQLinear.from_weights(w) for w in ws]
    group = ops.VQLinearGroup(layers)
    x = np.random.default_rng(4).standard_normal((5, 2560)).astype(np.float32)
    y = torch.zeros((5, 6912), device=cuda)
    n0 = ojasx_b200.launch_count()
    group.forward(torch.from_numpy(x).to(cuda), y)
    torch.cuda.synchronize()
    assert ojasx_b200.launch_count() == n0 + 1
    y = y.cpu().numpy()
    for i, w in enumerate(ws):
        want = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x[i], block_dim=8)
        assert np.array_equal(y[i, : w.out_features], want)


def test_linear_errors(cuda):
    w = synth.make_vq_linear(1, 64, 32, block_dim=16, outlier_frac=0)
    layer = ops.VQLinear.from_weights(w)
    with pytest.raises(ValueError, match="Input feature mismatch"):
        layer(torch.zeros(3, 63, device=cuda))
    with pytest.raises(ojasx_b200.OjasxB200Error):
        layer(torch.zeros(3, 64))  # CPU tensor: no fallback
    L = ojasx_b200.lib()
    assert L.ojasx_linear_forward(None, None, None, 1, 0) == -1
    assert L.ojasx_b200_linear_forward(layer.handle, None, None, 1, 0, 0, 32, None) == -1
