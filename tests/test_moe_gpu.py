"""GPU parity of the MoE path (experts, router) against the CPU oracle."""
import numpy as np
import pytest
import torch

import ojasx_b200
from ojasx_b200 import lut_ctypes, ops, synth

pytestmark = pytest.mark.gpu

# fp32 tolerance of the path (north star): rel 1e-5 / abs 1e-6
RTOL, ATOL = 1e-5, 1e-6


def _oracle_moe(oracle, w, x, idx, wts):
    return np.stack([oracle.moe_forward(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes,
                                        w.down_scales, x[t], idx[t], wts[t], block_dim=w.block_dim,
                                        gu_csr=w.gate_up_csr, dn_csr=w.down_csr) for t in range(x.shape[0])])


def _close(got, want):
    return np.all(np.abs(got - want) <= ATOL + RTOL * np.abs(want))


def test_moe_reference_test_shape_host_abi(cuda, oracle):
    """Shape and routing of the reference's own MoE test (native/tests/test_native_lut.cpp:186-248)
    through the reference's ctypes class bound to this library."""
    w = synth.make_vq_moe(2, 512, 256, 64, block_dim=16, outlier_frac=0, with_router=False)
    moe = lut_ctypes.NativeSplitManifoldMoE(512, 256, 64, 10, 16)
    moe.initialize_weights(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes, w.down_scales)
    x = np.random.default_rng(0).standard_normal(256).astype(np.float32)
    idx = np.array([4, 12, 57, 103, 199, 255, 340, 412, 480, 511], np.int32)
    wts = np.array([0.25, 0.20, 0.15, 0.10, 0.08, 0.07, 0.05, 0.04, 0.03, 0.03], np.float32)
    got = moe.forward(x, idx, wts)
    want = _oracle_moe(oracle, w, x[None], idx[None], wts[None])[0]
    assert _close(got, want), np.abs(got - want).max()
    assert moe.compression_ratio > 20.0


@pytest.mark.parametrize("B", [1, 5, 32])
@pytest.mark.parametrize("frac", [0.0, 0.0038])
def test_moe_device_config2_shape(cuda, oracle, B, frac):
    """Config-2 geometry (hidden 2560, inter 640, block 8, top-10) with 32 experts to keep the CPU oracle quick."""
    w = synth.make_vq_moe(7, 32, 2560, 640, block_dim=8, outlier_frac=frac, unit_scales=(frac == 0.0))
    rng = np.random.default_rng(B)
    x = rng.standard_normal((B, 2560)).astype(np.float32)
    idx = np.stack([rng.choice(32, size=10, replace=False) for _ in range(B)]).astype(np.int32)
    wts = rng.uniform(0.02, 0.3, size=(B, 10)).astype(np.float32)
    if B > 1:
        idx[1, 3] = -1          # out-of-range id: skipped
        idx[1, 4] = 32          # out-of-range id: skipped
        wts[1, 5] = 5e-9        # negligible weight: skipped
    want = _oracle_moe(oracle, w, x, idx, wts)
    moe = ops.VQMoE(w)
    got = moe.forward(torch.from_numpy(x).to(cuda), torch.from_numpy(idx).to(cuda), torch.from_numpy(wts).to(cuda))
    got = got.cpu().numpy()
    assert _close(got, want), np.abs(got - want).max()
    # the only non-bit-exact step is exp() inside silu; report how often that shows
    print(f"B={B} frac={frac}: bit-identical elements {np.mean(got == want):.4f}")


def test_router_index_exact(cuda, oracle):
    w = synth.make_vq_moe(3, 512, 2560, 640, block_dim=8, outlier_frac=0)
    # experts are irrelevant here; only the router weights are used
    x = np.random.default_rng(11).standard_normal((37, 2560)).astype(np.float32)
    want_idx, want_w = oracle.router_topk(x, w.router, 10)
    moe = ops.VQMoE(w)
    idx, wts = moe.route(torch.from_numpy(x).to(cuda), 10)
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert np.array_equal(wts.cpu().numpy(), want_w)
    # torch formula (run_full_48_layers_and_generate.py:172-175) as an independent pin
    p = torch.softmax(torch.from_numpy(x) @ torch.from_numpy(w.router).T, dim=-1)
    tw, ti = torch.topk(p, 10, dim=-1)
    tw = tw / tw.sum(-1, keepdim=True)
    assert np.array_equal(ti.numpy(), want_idx)
    assert np.allclose(tw.numpy(), want_w, rtol=1e-5, atol=1e-7)


def test_moe_routed_and_expert_shards(cuda, oracle):
    """forward_routed == route + forward; two expert shards sum to the whole layer."""
    w = synth.make_vq_moe(5, 16, 256, 64, block_dim=8, outlier_frac=0.01, unit_scales=False)
    x = np.random.default_rng(3).standard_normal((6, 256)).astype(np.float32)
    xt = torch.from_numpy(x).to(cuda)
    full = ops.VQMoE(w)
    idx, wts = full.route(xt, 4)
    y = full.forward(xt, idx, wts)
    y2 = full.forward_routed(xt, 4)
    assert torch.equal(y, y2)
    want = _oracle_moe(oracle, w, x, idx.cpu().numpy(), wts.cpu().numpy())
    assert _close(y.cpu().numpy(), want)
    lo, hi = ops.VQMoE(w, (0, 8)), ops.VQMoE(w, (8, 16))
    ys = lo.forward(xt, idx, wts) + hi.forward(xt, idx, wts)
    assert np.allclose(ys.cpu().numpy(), want, rtol=1e-5, atol=1e-6)


def test_moe_bf16_io(cuda, oracle):
    w = synth.make_vq_moe(8, 8, 256, 64, block_dim=8, outlier_frac=0.0)
    rng = np.random.default_rng(2)
    x = synth.to_bf16_f32(rng.standard_normal((3, 256)).astype(np.float32))
    idx = np.stack([rng.choice(8, size=2, replace=False) for _ in range(3)]).astype(np.int32)
    wts = np.full((3, 2), 0.5, np.float32)
    want = _oracle_moe(oracle, w, x, idx, wts)
    moe = ops.VQMoE(w)
    got = moe.forward(torch.from_numpy(x).to(cuda).to(torch.bfloat16), torch.from_numpy(idx).to(cuda),
                      torch.from_numpy(wts).to(cuda)).float().cpu().numpy()
    # bf16 activation path: rel 2e-2 (north star); here the only loss is the final rounding to bf16
    assert np.allclose(got, want, rtol=2e-2, atol=1e-6)


@pytest.fixture
def fused_everywhere(monkeypatch):
    """Send every batch through the whole-expert kernel (normally used from about a hundred routed pairs)."""
    monkeypatch.setenv("OJASX_B200_MOE_FUSED_MIN_PAIRS", "1")


@pytest.mark.parametrize("H,I,D,E,k,B", [
    (256, 128, 8, 8, 4, 7),      # one table slice per pass; chunks of 4, 2 and 1 tokens; short chains
    (512, 256, 8, 6, 3, 40),     # several slices; about twenty tokens per expert
    (2560, 640, 8, 16, 10, 12),  # benchmark geometry: 10 / 5 / 5 gate-up slices, 80-group down tables with a 16-group tail
    (1024, 512, 16, 4, 2, 9),    # block_dim 16
    (384, 64, 4, 5, 5, 3),       # block_dim 4, every token routed to every expert
])
@pytest.mark.parametrize("frac", [0.0, 0.01])
def test_moe_whole_expert_kernel_shapes(cuda, oracle, fused_everywhere, H, I, D, E, k, B, frac):
    w = synth.make_vq_moe(H + B, E, H, I, block_dim=D, outlier_frac=frac, unit_scales=(frac == 0.0))
    rng = np.random.default_rng(E * B)
    x = rng.standard_normal((B, H)).astype(np.float32)
    idx = np.stack([rng.choice(E, size=k, replace=False) for _ in range(B)]).astype(np.int32)
    wts = rng.uniform(0.02, 0.3, size=(B, k)).astype(np.float32)
    if B > 2:
        idx[1, 0] = -1          # skipped pairs (ojasx_lut_cpu.cpp:284-286)
        idx[2, k - 1] = E
        wts[0, 1] = 5e-9
    want = _oracle_moe(oracle, w, x, idx, wts)
    moe = ops.VQMoE(w)
    n0 = ojasx_b200.launch_count()
    got = moe.forward(torch.from_numpy(x).to(cuda), torch.from_numpy(idx).to(cuda), torch.from_numpy(wts).to(cuda))
    got = got.cpu().numpy()
    assert ojasx_b200.lib().ojasx_b200_take_device_error() == 0
    assert ojasx_b200.launch_count() - n0 == 4          # work list, token tables, experts, combine
    assert _close(got, want), np.abs(got - want).max()
    # expert shards of the same layer (expert-parallel ranks) add up to it
    half = E // 2
    lo, hi = ops.VQMoE(w, (0, half)), ops.VQMoE(w, (half, E))
    args = (torch.from_numpy(x).to(cuda), torch.from_numpy(idx).to(cuda), torch.from_numpy(wts).to(cuda))
    ys = (lo.forward(*args) + hi.forward(*args)).cpu().numpy()
    assert np.allclose(ys, want, rtol=1e-5, atol=1e-6)


def test_moe_config2_full_size_batch_256(cuda, oracle):
    """BASELINE configuration 2 at full size: 512 experts, hidden 2560, inter 640, top-10, 0.38 % outliers on
    every expert matrix, 256 tokens routed by the layer's own router.  The CPU oracle checks a sample of tokens."""
    w = synth.make_vq_moe(77, 512, 2560, 640, block_dim=8, outlier_frac=0.0038)
    rng = np.random.default_rng(256)
    x = rng.standard_normal((256, 2560)).astype(np.float32)
    moe = ops.VQMoE(w)
    xt = torch.from_numpy(x).to(cuda)
    idx, wts = moe.route(xt, 10)
    oi, ow = oracle.router_topk(x, w.router, 10)
    assert np.array_equal(idx.cpu().numpy(), oi) and np.array_equal(wts.cpu().numpy(), ow)
    got = moe.forward_routed(xt, 10).cpu().numpy()
    assert ojasx_b200.lib().ojasx_b200_take_device_error() == 0
    sample = [0, 1, 2, 3, 63, 64, 127, 128, 200, 254, 255]
    want = _oracle_moe(oracle, w, x[sample], oi[sample], ow[sample])
    assert _close(got[sample], want), np.abs(got[sample] - want).max()
    assert np.isfinite(got).all()
    # the same tokens one at a time take the small-batch kernels: both paths agree within the tolerance
    one = moe.forward_routed(xt[:4], 10).cpu().numpy()
    assert _close(one, want[:4])


@pytest.mark.parametrize("H,I,D,E,k,B", [
    (2560, 640, 8, 32, 10, 32),   # benchmark geometry: two full table slices and a 64-group one (two chains per warp)
    (1536, 256, 8, 12, 6, 40),    # a 64-group tail after a full slice; 512 rows per expert (the smallest the walk takes)
    (1024, 512, 16, 8, 4, 50),    # block_dim 16, one 64-group slice only
    (768, 3456, 4, 3, 3, 64),     # block_dim 4; 6912 rows per expert (the most the walk parks); a 64-group tail
])
@pytest.mark.parametrize("frac", [0.0, 0.01])
def test_moe_gate_up_chain_walk_equals_row_walk(cuda, oracle, monkeypatch, H, I, D, E, k, B, frac):
    """From one expected pair per SM the gate/up pass walks a whole expert with 32 lanes per row over table images
    brought in by bulk copies; OJASX_B200_MOE_CHAIN=0 keeps the lane-per-row kernel.  Same sums in the same order:
    the outputs are equal bit for bit (and match the oracle), with outlier rows, skipped pairs, a gate clamp, the
    router in front, and expert shards."""
    w = synth.make_vq_moe(H + I, E, H, I, block_dim=D, outlier_frac=frac, unit_scales=(frac == 0.0))
    rng = np.random.default_rng(E + B)
    x = rng.standard_normal((B, H)).astype(np.float32)
    idx = np.stack([rng.choice(E, size=k, replace=False) for _ in range(B)]).astype(np.int32)
    wts = rng.uniform(0.02, 0.3, size=(B, k)).astype(np.float32)
    idx[1, 0] = -1
    idx[2, k - 1] = E
    wts[0, 1] = 5e-9
    args = (torch.from_numpy(x).to(cuda), torch.from_numpy(idx).to(cuda), torch.from_numpy(wts).to(cuda))
    moe = ops.VQMoE(w)
    n0 = ojasx_b200.launch_count()
    chain = moe.forward(*args)
    launches = ojasx_b200.launch_count() - n0
    routed_chain = moe.forward_routed(args[0], k)
    moe.set_gate_limit(0.05)
    clamp_chain = moe.forward(*args)
    moe.set_gate_limit(0.0)
    assert ojasx_b200.lib().ojasx_b200_take_device_error() == 0
    monkeypatch.setenv("OJASX_B200_MOE_ONE_LAUNCH", "0")   # the same walks as two launches
    assert torch.equal(moe.forward(*args), chain)
    monkeypatch.delenv("OJASX_B200_MOE_ONE_LAUNCH")
    monkeypatch.setenv("OJASX_B200_MOE_CHAIN", "0")
    row = moe.forward(*args)
    routed_row = moe.forward_routed(args[0], k)
    moe.set_gate_limit(0.05)
    clamp_row = moe.forward(*args)
    moe.set_gate_limit(0.0)
    monkeypatch.delenv("OJASX_B200_MOE_CHAIN")
    assert launches == 4                      # work list, table images, experts (gate/up and down from one queue), combine
    assert torch.equal(chain, row) and torch.equal(routed_chain, routed_row) and torch.equal(clamp_chain, clamp_row)
    assert not torch.equal(clamp_chain, chain)
    sample = [0, 1, 2, B - 1]
    want = _oracle_moe(oracle, w, x[sample], idx[sample], wts[sample])
    assert _close(chain.cpu().numpy()[sample], want)
    if E % 2 == 0 and B * k // 2 >= 148 * 2:   # both shards still expect a pair per SM
        lo, hi = ops.VQMoE(w, (0, E // 2)), ops.VQMoE(w, (E // 2, E))
        ys = lo.forward(*args) + hi.forward(*args)
        assert np.allclose(ys.cpu().numpy(), chain.cpu().numpy(), rtol=1e-5, atol=1e-6)
