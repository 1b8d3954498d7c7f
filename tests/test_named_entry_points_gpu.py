"""Entry points of the reference's operator surface that sit around the kernels: the cache manager
(ojasx_24x96/kv_cache.py:85-266), the fused-experts adapter over flattened projections with its gate clamp
(ojasx_24x96/module.py:577-708), the engine's from_oqpack / audit_forward_graph
(ojasx_24x96/inference_engine.py:190-232, 268-357) and the SplitManifoldLUTLinear module
(split_manifold_lut_experiment/engine/split_manifold_engine.py:22-250)."""
import os

import numpy as np
import pytest
import torch
from torch import nn

from ojasx_b200 import inference_engine as ie
from ojasx_b200 import kv_cache, module, ops, synth
from ojasx_b200.split_manifold_engine import SplitManifoldLUTLinear

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_kv_cache_manager_counts_crops_and_resets(cuda, oracle):
    kv = synth.make_vq_kv(5, 2, 40, kv_heads=4, q_heads=8, head_dim=96)
    caches = [ops.VQKVCache(2, 4, 8, 96, 8, 64, kv.k_codebook, kv.v_codebook) for _ in range(3)]
    for c in caches:
        c.load(kv.k_codes, kv.v_codes)
    mgr = kv_cache.OjasXKVCacheManager(max_context_length=64)
    mgr.update(caches)
    st = mgr.stats()
    assert (st.sequence_length, st.num_cached_layers, st.max_context_length, st.dtype) == (40, 3, 64, "uint8_codebook_vq")
    assert st.allocated_bytes == 3 * (2 * 2 * 4 * 64 * 12 + 2 * 4 * 4 * 256 * 8) and st.to_dict()["sequence_length"] == 40
    with pytest.raises(ValueError, match="exceeds admission bound"):
        kv_cache.OjasXKVCacheManager(max_context_length=39).update(caches)
    mgr.crop(25)
    assert mgr.sequence_length == 25 and all(c.seq_len == 25 for c in caches)
    q = torch.from_numpy(kv.q).to(cuda)
    got = caches[1].decode(q).cpu().numpy()
    for b in range(2):
        for h in range(4):
            want = oracle.kvq_decode(kv.q[b, 2 * h:2 * h + 2], kv.k_codes[b, h, :25], kv.v_codes[b, h, :25], kv.k_codebook[h],
                                     kv.v_codebook[h], block_dim=8)
            assert np.allclose(got[b, 2 * h:2 * h + 2], want, rtol=1e-4, atol=2e-6)
    with pytest.raises(ValueError):
        mgr.crop(-1)
    mgr.reset()
    assert mgr.past_key_values is None and mgr.sequence_length == 0 and all(c.seq_len == 0 for c in caches)
    # a plain tensor structure is still counted and trimmed along its sequence axis
    pkv = tuple((torch.zeros(1, 2, 10, 4), torch.zeros(1, 2, 10, 4)) for _ in range(2))
    mgr.update(pkv)
    assert mgr.sequence_length == 10 and mgr.allocated_bytes == 4 * 80 * 4 and mgr.dtype == "float32"
    mgr.crop(6)
    assert mgr.past_key_values[1][0].shape[-2] == 6 and mgr.sequence_length == 6


@pytest.mark.parametrize("limit", [None, 0.05])
def test_fused_experts_over_flattened_projections_with_gate_clamp(cuda, oracle, limit):
    """Reference constructor: two ResidualVQLinear projections over [E*2I, H] and [E*H, I]; with a limit the gate is
    clamped from above and up to [-limit, limit] before silu(gate)*up (module.py:646-651)."""
    E, H, I, D, k = 6, 256, 128, 8, 3
    w = synth.make_vq_moe(31, E, H, I, block_dim=D, outlier_frac=0.01, unit_scales=False, with_router=False)

    def proj(codes, cb, scales, csr):
        enc = module.encode_uint8_layout(codes.reshape(-1, codes.shape[-1]), cb, scales.reshape(-1), "cpu")
        enc.outliers = tuple(torch.from_numpy(np.ascontiguousarray(a)) for a in csr)
        return module.ResidualVQLinear(enc)

    experts = module.ResidualVQFusedExperts(E, H, I, gate_up_proj=proj(w.gate_up_codes, w.codebook, w.gate_up_scales, w.gate_up_csr),
                                            down_proj=proj(w.down_codes, w.down_codebook, w.down_scales, w.down_csr),
                                            act_fn=nn.SiLU(), gate_limit=limit)
    rng = np.random.default_rng(2)
    x = rng.standard_normal((5, H)).astype(np.float32)
    idx = np.stack([rng.choice(E, k, replace=False) for _ in range(5)]).astype(np.int64)
    wts = rng.uniform(0.1, 0.6, (5, k)).astype(np.float32)
    got = experts(torch.from_numpy(x).to(cuda), torch.from_numpy(idx).to(cuda), torch.from_numpy(wts).to(cuda)).cpu().numpy()

    def rows_csr(csr, r0, r1):     # CSR of the rows [r0, r1) of a flattened matrix
        rp, ci, va = csr
        return (rp[r0:r1 + 1] - rp[r0]).astype(np.int32), ci[rp[r0]:rp[r1]], va[rp[r0]:rp[r1]]

    for t in range(5):
        y = np.zeros(H, np.float32)
        for j in range(k):
            e = int(idx[t, j])
            gu = oracle.linear_forward(w.codebook, w.gate_up_codes[e], w.gate_up_scales[e], None,
                                       rows_csr(w.gate_up_csr, e * 2 * I, (e + 1) * 2 * I), x[t], block_dim=D)
            gate, up = gu[:I].copy(), gu[I:].copy()
            if limit is not None:
                gate, up = np.minimum(gate, np.float32(limit)), np.clip(up, -np.float32(limit), np.float32(limit))
            inter = ((gate / (np.float32(1) + np.exp(-gate.astype(np.float64)).astype(np.float32))) * up).astype(np.float32)
            out = oracle.linear_forward(w.down_codebook, w.down_codes[e], w.down_scales[e], None,
                                        rows_csr(w.down_csr, e * H, (e + 1) * H), inter, block_dim=D)
            y = (y + out * wts[t, j]).astype(np.float32)
        assert np.all(np.abs(got[t] - y) <= 1e-6 + 1e-5 * np.abs(y)), np.abs(got[t] - y).max()
    if limit is None:       # without a clamp this is the reference library's MoE
        want = oracle.moe_forward(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes, w.down_scales,
                                  x[0], idx[0].astype(np.int32), wts[0], block_dim=D, gu_csr=w.gate_up_csr, dn_csr=w.down_csr)
        assert np.all(np.abs(got[0] - want) <= 1e-6 + 1e-5 * np.abs(want))
    with pytest.raises(ValueError):
        module.ResidualVQFusedExperts(E, H, I, gate_up_proj=experts.gate_up_proj, down_proj=experts.down_proj, act_fn=nn.GELU())


class _ToySkeleton(nn.Module):
    """Same sub-module names as the model the reference wrote into tests/golden/oqpack_toy."""

    def __init__(self):
        super().__init__()
        self.a, self.b, self.c = nn.Linear(64, 96), nn.Linear(96, 32, bias=False), nn.Linear(64, 48)
        self.norm = nn.LayerNorm(32)

    def forward(self, x):
        return self.norm(self.b(torch.relu(self.a(x)))), self.c(x)


def test_engine_from_oqpack_and_audit_on_a_module(cuda):
    engine, manifest = ie.UniversalInferenceEngine.from_oqpack(_ToySkeleton, os.path.join(HERE, "golden", "oqpack_toy"), device=cuda)
    assert manifest["model_id"] == "toy" and not manifest["skipped_layers"]
    assert all(isinstance(getattr(engine.model, n), module.ResidualVQLinear) for n in "abc")
    assert engine.model.norm.weight.is_cuda
    want = np.load(os.path.join(HERE, "golden", "oqpack_toy_expected.npz"))
    x = torch.from_numpy(want["a_x"]).to(cuda)
    (y, z), report = engine.audit_forward_graph(x)
    assert y.shape == (3, 32) and z.shape == (3, 48)
    for n in "abc":     # every loaded layer against the reference module's own CPU output for the stored input
        got = getattr(engine.model, n)(torch.from_numpy(want[f"{n}_x"]).to(cuda)).cpu().numpy()
        assert np.allclose(got, want[f"{n}_y"], rtol=1e-4, atol=1e-5), n
    assert report.total_quantized_modules == 3 and report.executed_quantized_modules == 3
    assert report.execution_coverage_ratio == 1.0 and report.all_outputs_finite and report.total_forward_calls == 3
    assert report.traces["a"].input_shape == (3, 64) and report.traces["b"].output_shape == (3, 32)
    assert report.traces["a"].output_l2_norm > 0 and report.to_dict()["traces"]["c"]["call_count"] == 1
    assert engine.forward_any(x)[0].shape == (3, 32)


def test_audit_on_the_decoder_stack(cuda):
    cfg = ie.StackConfig(layers=2, hidden=128, q_heads=4, kv_heads=2, head_dim=32, experts=8, top_k=2, inter=64, vocab=300,
                         max_seq_len=16, distinct_layers=2, outlier_frac=0.01)
    engine = ie.UniversalInferenceEngine(ie.VQDecoderStack(ie.make_stack_weights(3, cfg), cfg, batch=2))
    logits, report = engine.audit_forward_graph(torch.tensor([5, 17], device=cuda))
    assert logits.shape == (2, 300) and report.total_quantized_modules == 2 * 5 + 1
    assert report.execution_coverage_ratio == 1.0 and report.all_outputs_finite
    assert report.traces["layers.1.moe"].module_type == "VQMoE" and 1 <= len(report.active_moe_experts_union) <= 8
    assert report.traces["lm_head"].output_shape == (2, 300)
    # the wrappers are gone again: a second, unaudited step runs as usual
    assert engine.model.decode_step(torch.tensor([1, 2], device=cuda)).shape == (2, 300)


def test_split_manifold_lut_linear_module(cuda, oracle):
    """Buffers and methods of the reference's Python module; table and output bit-identical to the CPU library."""
    K, M, D = 512, 200, 16
    w = synth.make_vq_linear(8, K, M, block_dim=D, outlier_frac=0.01, with_scales=True, with_bias=True)
    layer = SplitManifoldLUTLinear(K, M, block_dim=D, bias=True).to(cuda)
    rp, ci, va = w.csr
    rows = np.repeat(np.arange(M), np.diff(rp))
    layer.codebook.copy_(torch.from_numpy(w.codebook))
    layer.codes.copy_(torch.from_numpy(w.codes))
    layer.scales.copy_(torch.from_numpy(w.scales))
    layer.outlier_indices = torch.from_numpy(np.stack([rows, ci.astype(np.int64)])).to(cuda)
    layer.outlier_values = torch.from_numpy(va).to(cuda)
    with torch.no_grad():
        layer.bias.copy_(torch.from_numpy(w.bias))
    x = np.random.default_rng(1).standard_normal((2, 3, K)).astype(np.float32)
    y = layer(torch.from_numpy(x).to(cuda))
    assert y.shape == (2, 3, M)
    want = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x.reshape(-1, K), block_dim=D)
    assert np.array_equal(y.cpu().numpy().reshape(-1, M), want)
    lut = layer.build_lut(torch.from_numpy(x).to(cuda))
    assert lut.shape == (2, 3, K // D, 256)
    assert np.array_equal(lut[1, 2].cpu().numpy(), oracle.build_lut(x[1, 2], w.codebook, block_dim=D))
    assert layer.num_outliers == len(va) and layer.lut_sram_bytes == (K // D) * 256 * 4 and layer.compression_ratio > 1.5
    # encoded from a dense weight on the device, the layer reproduces that weight at its outliers and closely elsewhere
    dense = torch.randn(96, 256, device=cuda) * 0.02
    dense[3, 7] = 1.0
    enc = SplitManifoldLUTLinear.from_dense(dense, block_dim=8)
    xin = torch.randn(4, 256, device=cuda)
    ref = xin @ enc.dequantize_weights().T
    assert torch.allclose(enc(xin), ref, rtol=1e-4, atol=1e-5)
    assert abs(float(enc.dequantize_weights()[3, 7]) - 1.0) < 1e-6 and enc.num_outliers >= 1
