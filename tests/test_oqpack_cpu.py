"""OQPack reader on the committed package written by the reference's own writer (tests/golden/oqpack_toy,
made by tests/golden/make_oqpack_fixture.py): manifest, integrity checks, tensor wiring (no CUDA needed)."""
import os
import shutil

import numpy as np
import pytest
import torch

from ojasx_b200 import oqpack

PKG = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oqpack_toy")


def test_manifest_and_integrity():
    m = oqpack.verify_oqpack_integrity(PKG, verify_checksums=True)
    assert set(m["layer_specs"]) == {"a", "b", "c"}
    assert m["tensors"]["a.packed_codes"]["dtype"] == "uint8"
    assert m["tensors"]["c.codebooks"]["shape"] == [2, 16, 8]


def test_tampered_shard_is_rejected(tmp_path):
    dst = tmp_path / "pkg"
    shutil.copytree(PKG, dst)
    shard = next(p for p in os.listdir(dst) if p.endswith(".safetensors"))
    with open(dst / shard, "r+b") as f:
        f.seek(-1, os.SEEK_END)
        last = f.read(1)
        f.seek(-1, os.SEEK_END)
        f.write(bytes([last[0] ^ 1]))
    oqpack.verify_oqpack_integrity(str(dst), verify_checksums=False)      # size still matches
    with pytest.raises(oqpack.OQPackValidationError, match="checksum"):
        oqpack.verify_oqpack_integrity(str(dst), verify_checksums=True)
    os.remove(dst / shard)
    with pytest.raises(oqpack.OQPackValidationError, match="Missing shard"):
        oqpack.verify_oqpack_integrity(str(dst), verify_checksums=False)


def test_layers_wrap_the_stored_tensors_unchanged():
    from safetensors import safe_open
    layers, skipped = oqpack.load_quantized_layers(PKG, device="cpu")
    assert not skipped and set(layers) == {"a", "b", "c"}
    shard = os.path.join(PKG, "shard-00001-of-00001.safetensors")
    with safe_open(shard, framework="pt", device="cpu") as f:
        for name, layer in layers.items():
            enc = layer.encoded()
            assert torch.equal(enc.packed_codes, f.get_tensor(f"{name}.packed_codes"))
            assert torch.equal(enc.codebooks, f.get_tensor(f"{name}.codebooks"))
            assert torch.equal(enc.row_scales, f.get_tensor(f"{name}.row_scales"))
    assert (layers["a"].bits_per_stage, layers["a"].encoded().stages, layers["a"].block_size) == (8, 1, 8)
    assert (layers["c"].bits_per_stage, layers["c"].encoded().stages) == (4, 2)
    assert layers["b"].bias is None and layers["a"].bias.shape == (96,)
    only_a, _ = oqpack.load_quantized_layers(PKG, device="cpu", names=["a"])
    assert list(only_a) == ["a"]


def test_unsupported_codecs_are_reported():
    assert oqpack.supported_layer({"type": "residual_vq_linear", "codec": "leech24_shell2_residual", "bits_per_stage": 8}) \
        == "codec leech24_shell2_residual"
    assert oqpack.supported_layer({"type": "residual_vq_linear", "bits_per_stage": 8, "rotation_reflections": 2}) \
        == "rotated input basis"
    assert oqpack.supported_layer({"type": "residual_vq_fused_experts"}) == "module type residual_vq_fused_experts"
    assert oqpack.supported_layer({"type": "residual_vq_linear", "bits_per_stage": 8}) is None


def test_writer_round_trip_with_outliers(tmp_path):
    from ojasx_b200 import synth
    from ojasx_b200.module import ResidualVQLinear, encode_uint8_layout
    w = synth.make_vq_linear(4, 64, 40, block_dim=8, outlier_frac=0.05, with_scales=True, with_bias=True)
    enc = encode_uint8_layout(w.codes, w.codebook, w.scales, "cpu")
    enc.outliers = tuple(torch.from_numpy(np.ascontiguousarray(a)) for a in w.csr)
    layer = ResidualVQLinear(enc, torch.from_numpy(w.bias))
    oqpack.save_quantized_layers({"blocks.0.proj": layer}, str(tmp_path / "p"), model_id="t")
    back, skipped = oqpack.load_quantized_layers(str(tmp_path / "p"), device="cpu", verify_checksums=True)
    assert not skipped
    got = back["blocks.0.proj"].encoded()
    assert torch.equal(got.packed_codes, enc.packed_codes) and torch.equal(got.codebooks, enc.codebooks)
    for a, b in zip(got.outliers, enc.outliers):
        assert torch.equal(a, b)
    assert torch.equal(back["blocks.0.proj"].bias, layer.bias)
