"""Edge cases of the VQ path on the GPU against the CPU oracle: empty and ragged inputs, odd outlier
layouts, small codebooks, the largest layer of the benchmark set, and size-independent properties at
full size (the reference's own tests cover the plain shapes: native/tests/test_native_lut.cpp:30-248)."""
import ctypes as C

import numpy as np
import pytest
import torch

import ojasx_b200
from ojasx_b200 import lut_ctypes, ops, synth

pytestmark = pytest.mark.gpu


def _lin(oracle, w, x, **kw):
    return oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=w.block_dim, **kw)


def test_empty_batch_and_zero_experts_are_no_ops(cuda):
    """batch_size 0 and k_active 0 return 0 and leave the output alone (ojasx_lut_c_api.cpp:100-118,
    ojasx_lut_cpu.cpp:220)."""
    L = ojasx_b200.lib()
    w = synth.make_vq_linear(1, 64, 32, block_dim=16, outlier_frac=0)
    layer = ops.VQLinear.from_weights(w)
    x = np.ones(64, np.float32)
    y = np.full(32, 7.0, np.float32)
    assert L.ojasx_linear_forward(layer.handle, x.ctypes.data, y.ctypes.data, 0, 0) == 0
    assert np.all(y == 7.0)
    m = synth.make_vq_moe(2, 8, 64, 32, block_dim=8, outlier_frac=0, with_router=False)
    moe = lut_ctypes.NativeSplitManifoldMoE(8, 64, 32, 2, 8)
    moe.initialize_weights(m.codebook, m.down_codebook, m.gate_up_codes, m.gate_up_scales, m.down_codes, m.down_scales)
    idx, wt = np.zeros(2, np.int32), np.ones(2, np.float32)
    out = np.full(64, 3.0, np.float32)
    assert L.ojasx_moe_forward(moe.handle, x.ctypes.data, idx.ctypes.data, wt.ctypes.data, out.ctypes.data, 0) == 0
    assert np.all(out == 3.0)


@pytest.mark.parametrize("K,M,D", [(8, 1, 8), (16, 31, 16), (2560, 33, 8), (64, 1000, 4)])
def test_ragged_row_counts(cuda, oracle, K, M, D):
    """One row, rows that are not a multiple of the 32-row tiles, a single group per row."""
    w = synth.make_vq_linear(K + M, K, M, block_dim=D, outlier_frac=0.02, with_scales=True, with_bias=True)
    x = np.random.default_rng(M).standard_normal((2, K)).astype(np.float32)
    got = ops.VQLinear.from_weights(w)(torch.from_numpy(x).to(cuda)).cpu().numpy()
    assert np.array_equal(got, _lin(oracle, w, x))


def _csr_from_rows(rows):
    rp = np.zeros(len(rows) + 1, np.int32)
    cols, vals = [], []
    for i, r in enumerate(rows):
        cols += [c for c, _ in r]
        vals += [v for _, v in r]
        rp[i + 1] = len(cols)
    return rp, np.asarray(cols, np.int32), np.asarray(vals, np.float32)


@pytest.mark.parametrize("batch", [1, 3])
def test_outlier_layouts(cuda, oracle, batch):
    """Every outlier in one row, empty rows at both ends, a full row, repeated columns (summed in entry
    order, ojasx_lut_cpu.cpp:117-126) and a long row that spans several staging passes."""
    K, M, D = 2560, 96, 8
    rng = np.random.default_rng(3)
    w = synth.make_vq_linear(5, K, M, block_dim=D, outlier_frac=0)
    rows = [[] for _ in range(M)]
    rows[17] = [(int(c), float(v)) for c, v in zip(rng.integers(0, K, 5000), rng.standard_normal(5000))]   # repeats, unsorted
    rows[40] = [(c, 0.5) for c in range(K)]                                                                 # full row
    rows[41] = [(7, 1.0), (7, -1.0), (7, 2.0)]
    rows[94] = [(K - 1, -3.0)]
    csr = _csr_from_rows(rows)
    x = rng.standard_normal((batch, K)).astype(np.float32)
    layer = ops.VQLinear(w.codebook, w.codes, None, None, csr, block_dim=D)
    got = layer(torch.from_numpy(x).to(cuda)).cpu().numpy()
    want = oracle.linear_forward(w.codebook, w.codes, None, None, csr, x, block_dim=D)
    assert np.array_equal(got, want)
    # the same through a row slice that starts inside the long row's neighbourhood
    got = layer(torch.from_numpy(x).to(cuda), 16, 42).cpu().numpy()
    assert np.array_equal(got, want[:, 16:42])


def test_small_codebook(cuda, oracle):
    """codebook_size 16: codes stay below 16 and the table rows above are never touched."""
    rng = np.random.default_rng(8)
    K, M, D, Kcb = 512, 200, 8, 16
    cb = (rng.standard_normal((Kcb, D)) * 0.02).astype(np.float32)
    codes = rng.integers(0, Kcb, size=(M, K // D), dtype=np.uint8)
    x = rng.standard_normal((2, K)).astype(np.float32)
    layer = ops.VQLinear(cb, codes, None, None, None, block_dim=D, codebook_size=Kcb)
    got = layer(torch.from_numpy(x).to(cuda)).cpu().numpy()
    assert np.array_equal(got, oracle.linear_forward(cb, codes, None, None, None, x, block_dim=D, codebook_size=Kcb))


def test_largest_layer_lm_head(cuda, oracle):
    """2560 -> 151936 (the vocabulary projection of the benchmark's decoder stack): every row, bit for bit."""
    w = synth.make_vq_linear(2024, 2560, 151936, block_dim=8, outlier_frac=0.0038)
    x = np.random.default_rng(1).standard_normal((1, 2560)).astype(np.float32)
    got = ops.VQLinear.from_weights(w)(torch.from_numpy(x).to(cuda)).cpu().numpy()
    assert np.array_equal(got, _lin(oracle, w, x))


def test_batch_rows_are_independent_at_full_size(cuda, oracle):
    """Config-1 layer: a batch of 7 (persistent kernel) equals 7 single-row calls (cluster kernel) bit for
    bit, in any row order, and repeated calls give the same bits."""
    w = synth.make_vq_linear(31, 2560, 6912, block_dim=8)
    layer = ops.VQLinear.from_weights(w)
    x = torch.from_numpy(np.random.default_rng(6).standard_normal((7, 2560)).astype(np.float32)).to(cuda)
    whole = layer(x)
    singles = torch.cat([layer(x[i:i + 1]) for i in range(7)])
    assert torch.equal(whole, singles)
    perm = torch.tensor([3, 0, 6, 1, 5, 2, 4], device=cuda)
    assert torch.equal(layer(x[perm]), whole[perm])
    assert torch.equal(layer(x), whole)
    sample = whole[2].cpu().numpy()
    assert np.array_equal(sample, _lin(oracle, w, x[2].cpu().numpy()))


def test_moe_repeated_experts_and_all_skipped(cuda, oracle):
    """The same expert twice in one token's list is evaluated twice (caller order), and a token whose
    weights are all below 1e-8 yields zeros (ojasx_lut_cpu.cpp:284-286)."""
    w = synth.make_vq_moe(9, 16, 256, 64, block_dim=8, outlier_frac=0.01)
    rng = np.random.default_rng(2)
    x = rng.standard_normal((3, 256)).astype(np.float32)
    idx = np.array([[5, 5, 2, 5], [0, 1, 2, 3], [15, 14, 15, 14]], np.int32)
    wts = np.array([[0.4, 0.3, 0.2, 0.1], [1e-9, -1e-9, 0.0, 5e-9], [0.25, 0.25, 0.25, 0.25]], np.float32)
    moe = ops.VQMoE(w)
    got = moe.forward(torch.from_numpy(x).to(cuda), torch.from_numpy(idx).to(cuda), torch.from_numpy(wts).to(cuda)).cpu().numpy()
    want = np.stack([oracle.moe_forward(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes,
                                        w.down_scales, x[t], idx[t], wts[t], block_dim=8, gu_csr=w.gate_up_csr,
                                        dn_csr=w.down_csr) for t in range(3)])
    assert np.all(np.abs(got - want) <= 1e-6 + 1e-5 * np.abs(want)), np.abs(got - want).max()
    assert np.all(got[1] == 0.0)
    again = moe.forward(torch.from_numpy(x).to(cuda), torch.from_numpy(idx).to(cuda), torch.from_numpy(wts).to(cuda)).cpu().numpy()
    assert np.array_equal(again, got)


def test_kv_error_codes(cuda):
    """Head index out of range is -2 for append and attention (ojasx_lut_c_api.cpp:154-160, 166-172)."""
    L = ojasx_b200.lib()
    cache = lut_ctypes.NativeKVCache(2, 64, 8, 16)
    v = np.ones(64, np.float32)
    assert L.ojasx_kv_cache_append(cache._handle, 2, v.ctypes.data, v.ctypes.data) == -2
    assert L.ojasx_kv_cache_append(cache._handle, -1, v.ctypes.data, v.ctypes.data) == -2
    out = np.zeros(64, np.float32)
    assert L.ojasx_kv_cache_attention(cache._handle, 5, v.ctypes.data, out.ctypes.data, C.c_float(1.0)) == -2


def test_concurrent_callers_of_one_handle(cuda, oracle):
    """Several host threads calling ojasx_linear_forward on ONE handle with their own buffers: the calls are
    serialised inside the library, so every caller gets the result of its own input (the reference's CPU
    handle is stateless between calls, ojasx_lut_c_api.cpp:100-118)."""
    import threading

    L = ojasx_b200.lib()
    w = synth.make_vq_linear(77, 512, 384, block_dim=8, outlier_frac=0.01)
    layer = ops.VQLinear.from_weights(w)
    rng = np.random.default_rng(4)
    xs = [rng.standard_normal(512).astype(np.float32) for _ in range(4)]
    want = [_lin(oracle, w, x[None])[0] for x in xs]
    bad = []

    def run(i):
        y = np.zeros(384, np.float32)
        for _ in range(50):
            if L.ojasx_linear_forward(layer.handle, xs[i].ctypes.data, y.ctypes.data, 1, 0) != 0 or not np.array_equal(y, want[i]):
                bad.append(i)
                return

    threads = [threading.Thread(target=run, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not bad


def test_outliers_replaced_after_a_forward(cuda, oracle):
    """ojasx_set_linear_outliers may be called at any time (ojasx_lut_c_api.cpp:67-91): a forward that was
    already recorded for the handle, and a group that already holds the handle, must use the new arrays."""
    L = ojasx_b200.lib()
    K, M, D = 512, 96, 8
    w = synth.make_vq_linear(11, K, M, block_dim=D, outlier_frac=0)
    w2 = synth.make_vq_linear(12, K, M, block_dim=D, outlier_frac=0.02)
    w3 = synth.make_vq_linear(13, K, M, block_dim=D, outlier_frac=0.05)
    x = np.random.default_rng(4).standard_normal((1, K)).astype(np.float32)
    layer = ops.VQLinear(w.codebook, w.codes, None, None, None, block_dim=D)
    other = ops.VQLinear.from_weights(synth.make_vq_linear(14, K, M, block_dim=D, outlier_frac=0.01))
    group = ops.VQLinearGroup([layer, other] * 5)           # 10 members: the persistent grouped kernel
    xd = torch.from_numpy(np.repeat(x, 10, 0)).to(cuda)
    yd = torch.zeros(10, M, device=cuda)
    y = np.zeros((1, M), np.float32)

    def host_forward():
        assert L.ojasx_linear_forward(layer.handle, x.ctypes.data, y.ctypes.data, 1, 0) == 0
        return y.copy()

    base = oracle.linear_forward(w.codebook, w.codes, None, None, None, x, block_dim=D)
    assert np.array_equal(host_forward(), base)
    assert np.array_equal(host_forward(), base)              # second call replays the recorded launch
    group.forward(xd, yd)
    assert np.array_equal(yd[0:1].cpu().numpy(), base)
    for csr in (w2.csr, w3.csr):                             # none -> some -> other (old arrays are freed)
        rp, ci, va = (np.ascontiguousarray(a) for a in csr)
        assert L.ojasx_set_linear_outliers(layer.handle, len(va), rp.ctypes.data, ci.ctypes.data, va.ctypes.data) == 0
        want = oracle.linear_forward(w.codebook, w.codes, None, None, csr, x, block_dim=D)
        assert not np.array_equal(want, base)
        assert np.array_equal(host_forward(), want)
        group.forward(xd, yd)
        torch.cuda.synchronize()
        assert np.array_equal(yd[0:1].cpu().numpy(), want) and np.array_equal(yd[2:3].cpu().numpy(), want)
        assert np.array_equal(layer(torch.from_numpy(x).to(cuda)).cpu().numpy(), want)


def test_static_plan_append_past_capacity_is_reported(cuda):
    """Under the static plan the host cannot refuse an append to a full cache; the kernel drops the token and
    the next ojasx_b200_kvq_sync_len returns -2 once.  (A dropped write, not a fault.)"""
    kv = synth.make_vq_kv(21, 1, 3, kv_heads=4, q_heads=8, head_dim=96)
    cache = ops.VQKVCache(1, 4, 8, 96, 8, 4, kv.k_codebook, kv.v_codebook)
    cache.load(kv.k_codes, kv.v_codes)
    cache.set_static_plan(True)
    k = torch.from_numpy(kv.new_k).to(cuda)
    v = torch.from_numpy(kv.new_v).to(cuda)
    cache.append(k, v)                                       # 3 -> 4: full
    assert cache.sync_len() == 4
    cache.append(k, v)                                       # dropped
    assert cache.sync_len() == -2
    assert cache.sync_len() == 4                             # flag cleared, length unchanged
    out = cache.decode(torch.from_numpy(kv.q).to(cuda))
    assert torch.isfinite(out).all()
    cache.close()
