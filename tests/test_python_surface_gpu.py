"""GPU tests of the package-level operator surface: the pattern of the reference's own tests
(tests/test_m10_compression_aware_math.py:241-383, tests/test_m5_native_fused_kernels.py:123-193,
tests/test_m6_backend_abi_llamacpp.py): every fast path against dequantise + F.linear on small random
layers, across bit widths, stage counts, non-divisible feature counts, input ranks and row slices."""
import ctypes

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from ojasx_b200 import OjasxB200Error, backend_abi, codec, math_engine, module, synth, tilelang_backend

pytestmark = pytest.mark.gpu


def _random_encoded(seed, rows, cols, block, bits, stages, device):
    g = torch.Generator().manual_seed(seed)
    G = (cols + block - 1) // block
    Q = 1 << bits
    codes = [torch.randint(0, Q, (rows * G,), generator=g, dtype=torch.int64) for _ in range(stages)]
    packed = torch.stack([codec.pack_codes(c, bits) for c in codes])
    cbs = torch.randn(stages, Q, block, generator=g) * 0.05
    scales = torch.rand(rows, generator=g) + 0.5
    return codec.QuantizedWeight((rows, cols), block, bits, packed.to(device), cbs.to(device), scales.to(device), {})


CASES = [(64, 48, 8, 4, 2), (33, 50, 8, 4, 3), (40, 64, 4, 2, 4), (17, 24, 4, 1, 5), (128, 256, 8, 8, 1),
         (96, 100, 8, 8, 1), (70, 512, 16, 8, 1), (50, 60, 8, 8, 2), (31, 37, 4, 8, 1),
         # word-aligned rows of narrow codes: the table kernel of rvq_generic.cu (ragged last block included)
         (200, 256, 8, 4, 4), (77, 250, 8, 4, 3), (64, 512, 8, 1, 8), (300, 2560, 8, 4, 4), (45, 128, 4, 2, 2)]


@pytest.mark.parametrize("rows,cols,block,bits,stages", CASES)
def test_subspace_lut_rvq_gemm_matches_dequantised_linear(cuda, rows, cols, block, bits, stages):
    enc = _random_encoded(rows + cols, rows, cols, block, bits, stages, cuda)
    w = codec.dequantize_weight(enc)
    bias = torch.randn(rows, device=cuda) * 0.1
    for shape in ((cols,), (3, cols), (2, 3, cols)):
        x = torch.randn(*shape, device=cuda)
        got = math_engine.subspace_lut_rvq_gemm(x, enc, bias=bias)
        want = F.linear(x, w, bias)
        assert got.shape == want.shape and got.dtype == x.dtype
        assert (got - want).abs().max().item() < 1e-4
    out, sched = tilelang_backend.dispatch_universal_compressed_gemm(torch.randn(5, cols, device=cuda), enc, bias)
    assert out.shape == (5, rows) and sched.backend == "cuda_sm_100a"


def test_narrow_width_table_kernel_agrees_with_the_compatibility_kernel(cuda, monkeypatch):
    """4 bits x 4 stages (the reference's default artefacts): table kernel against the dequantise-and-dot kernel
    (OJASX_B200_RVQ_COMPAT=1) on the same layer, batch and row slice."""
    enc = _random_encoded(9, 700, 2560, 8, 4, 4, cuda)
    x = torch.randn(3, 2560, device=cuda)
    fast = math_engine.fused_rvq_gemm_native(enc, x, 100, 650)
    monkeypatch.setenv("OJASX_B200_RVQ_COMPAT", "1")
    slow = math_engine.fused_rvq_gemm_native(enc, x, 100, 650)
    assert fast.shape == slow.shape == (3, 550)
    assert torch.allclose(fast, slow, rtol=1e-4, atol=1e-4)


def test_pack_unpack_roundtrip():
    for bits in (1, 2, 4, 8):
        c = torch.randint(0, 1 << bits, (1001,))
        p = codec.pack_codes(c, bits)
        assert p.numel() == (1001 * bits + 7) // 8
        assert torch.equal(codec.unpack_codes(p, bits, 1001).long(), c)
    with pytest.raises(ValueError):
        codec.pack_codes(torch.tensor([4]), 2)




def test_uint8_layout_is_bit_exact_with_the_native_oracle_and_bf16_rounds_once(cuda, oracle):
    w = synth.make_vq_linear(5, 2560, 2560, block_dim=8, outlier_frac=0.0, with_scales=True)
    enc = module.encode_uint8_layout(w.codes, w.codebook, w.scales, cuda)
    x = np.random.default_rng(0).standard_normal((4, 2560)).astype(np.float32)
    want = oracle.linear_forward(w.codebook, w.codes, w.scales, None, None, x, block_dim=8)
    got = math_engine.subspace_lut_rvq_gemm(torch.from_numpy(x).to(cuda), enc)
    assert np.array_equal(got.cpu().numpy(), want)
    xb = synth.to_bf16_f32(x)
    want_b = synth.to_bf16_f32(oracle.linear_forward(w.codebook, w.codes, w.scales, None, None, xb, block_dim=8))
    got_b = math_engine.subspace_lut_rvq_gemm(torch.from_numpy(xb).to(cuda).bfloat16(), enc)
    assert got_b.dtype == torch.bfloat16 and np.array_equal(got_b.float().cpu().numpy(), want_b)
    got_h = math_engine.subspace_lut_rvq_gemm(torch.from_numpy(x).to(cuda).half(), enc)   # fp16: widened, computed, cast back
    assert got_h.dtype == torch.float16


def test_fused_rvq_gemm_native_row_slices_and_errors(cuda):
    enc = _random_encoded(3, 90, 64, 8, 4, 2, cuda)
    w = codec.dequantize_weight(enc)
    x = torch.randn(3, 64, device=cuda)
    full = F.linear(x, w)
    for a, b in ((0, 90), (10, 33), (89, 90)):
        got = math_engine.fused_rvq_gemm_native(enc, x, a, b)
        assert got.shape == (3, b - a)
        assert torch.allclose(got, full[:, a:b], atol=1e-5, rtol=1e-4)
    with pytest.raises(IndexError):
        math_engine.fused_rvq_gemm_native(enc, x, 5, 5)
    with pytest.raises(ValueError, match="Expected inputs with 64 features"):
        math_engine.fused_rvq_gemm_native(enc, torch.randn(3, 63, device=cuda), 0, 90)
    with pytest.raises(ValueError, match="Input feature mismatch"):
        math_engine.subspace_lut_rvq_gemm(torch.randn(2, 65, device=cuda), enc)
    with pytest.raises(OjasxB200Error):
        math_engine.subspace_lut_rvq_gemm(torch.randn(2, 64), enc)   # CPU tensor: no fallback


def test_module_toggles_descriptor_and_ggml_dispatch(cuda):
    enc = _random_encoded(9, 48, 72, 8, 8, 1, cuda)
    bias = torch.randn(48, device=cuda)
    layer = module.ResidualVQLinear(enc, bias).to(cuda)
    x = torch.randn(2, 5, 72, device=cuda)
    want = F.linear(x, codec.dequantize_weight(enc), bias)
    layer.set_subspace_lut_mode(True)
    y1 = layer(x)
    layer.set_subspace_lut_mode(False)
    layer.set_fused_native_gemm(True)
    y2 = layer(x)
    assert (y1 - want).abs().max() < 1e-4 and (y2 - want).abs().max() < 1e-4
    assert set(dict(layer.named_buffers())) == {"packed_codes", "codebooks", "row_scales", "bias"}
    assert ctypes.sizeof(backend_abi.CRVQLayerDesc) == 56
    desc, meta = backend_abi.build_c_layer_descriptor(layer)
    assert desc.packed_codes == layer.packed_codes.data_ptr() and desc.rows == 48 and desc.columns == 72
    assert meta["workspace_bytes"] == 0 and meta["has_bias"]
    y3 = backend_abi.LlamaCppGGMLAdapter.dispatch_ggml_custom_matmul(layer, x.bfloat16())
    assert y3.dtype == torch.bfloat16 and y3.shape == (2, 5, 48)
    with pytest.raises(ValueError, match="Expected inputs with 72 features"):
        backend_abi.LlamaCppGGMLAdapter.dispatch_ggml_custom_matmul(layer, torch.randn(2, 71, device=cuda))
    assert backend_abi.OjasxStatus.NULL_POINTER == -2


def test_fused_experts_module_signature(cuda, oracle):
    w = synth.make_vq_moe(4, 8, 256, 64, block_dim=8, outlier_frac=0.0)
    experts = module.ResidualVQFusedExperts.from_weights(w)
    x = np.random.default_rng(1).standard_normal((3, 256)).astype(np.float32)
    idx = np.array([[0, 3], [7, 1], [2, 2]], np.int64)
    wts = np.array([[0.6, 0.4], [0.5, 0.5], [0.9, 0.1]], np.float32)
    got = experts(torch.from_numpy(x).to(cuda), torch.from_numpy(idx).to(cuda), torch.from_numpy(wts).to(cuda)).cpu().numpy()
    for t in range(3):
        want = oracle.moe_forward(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes,
                                  w.down_scales, x[t], idx[t].astype(np.int32), wts[t], block_dim=8)
        assert np.all(np.abs(got[t] - want) <= 1e-6 + 1e-5 * np.abs(want))
