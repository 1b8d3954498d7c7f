"""OQPack packages loaded straight onto the GPU: outputs against the reference modules' own CPU outputs
(stored beside the package by tests/golden/make_oqpack_fixture.py) and, for the CSR extension, the oracle."""
import os

import numpy as np
import pytest
import torch

from ojasx_b200 import oqpack, synth
from ojasx_b200.module import ResidualVQLinear, encode_uint8_layout

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_reference_package_runs_on_device(cuda):
    layers, skipped = oqpack.load_quantized_layers(os.path.join(HERE, "golden", "oqpack_toy"), device=cuda,
                                                   verify_checksums=True)
    assert not skipped
    want = np.load(os.path.join(HERE, "golden", "oqpack_toy_expected.npz"))
    for name, layer in layers.items():
        assert layer.packed_codes.is_cuda
        got = layer(torch.from_numpy(want[f"{name}_x"]).to(cuda)).cpu().numpy()
        ref = want[f"{name}_y"]
        # the reference multiplies a dequantised weight (torch matmul order); fp32 tolerance of the path
        assert np.allclose(got, ref, rtol=1e-4, atol=1e-5), (name, np.abs(got - ref).max())


def test_outlier_extension_round_trip_on_device(cuda, oracle, tmp_path):
    w = synth.make_vq_linear(12, 2560, 300, block_dim=8, outlier_frac=0.0038, with_scales=True, with_bias=True)
    enc = encode_uint8_layout(w.codes, w.codebook, w.scales, "cpu")
    enc.outliers = tuple(torch.from_numpy(np.ascontiguousarray(a)) for a in w.csr)
    oqpack.save_quantized_layers({"mlp.up": ResidualVQLinear(enc, torch.from_numpy(w.bias))}, str(tmp_path / "p"))
    layers, _ = oqpack.load_quantized_layers(str(tmp_path / "p"), device=cuda)
    x = np.random.default_rng(0).standard_normal((2, 2560)).astype(np.float32)
    got = layers["mlp.up"](torch.from_numpy(x).to(cuda)).cpu().numpy()
    want = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=8)
    assert np.array_equal(got, want)
