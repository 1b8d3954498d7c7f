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
    got = layer(xt.to(torch.bfloat16)).float().cpu().numpy()   # batch 4: below the tensor-core switch-over (32)
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


@pytest.mark.parametrize("K,M,D,kcb,dtype", [
    (2560, 1000, 8, 256, "f32"),    # G 320: slices of 128, 128 and 64 groups (two 16-lane chains), ragged last warp
    (768, 600, 16, 256, "f32"),     # G 48: one slice of 48 groups, 12 lanes per chain
    (640, 777, 4, 256, "f32"),      # G 160: 128 + 32
    (6912, 520, 8, 256, "f32"),     # G 864: six full slices and one of 96 groups (24 of 32 lanes)
    (1280, 515, 8, 16, "f32"),      # small codebook: table rows above it are zero
    (9216, 512, 8, 256, "f32"),     # nine slices; x too long to stage for the outlier products
    (2560, 1000, 8, 256, "bf16"),
])
def test_grouped_layers_walk_variants(cuda, oracle, monkeypatch, K, M, D, kcb, dtype):
    """150 layers in one grouped launch (one work item per layer, so every warp walks a long run of rows): the walk
    in which the lanes of a warp share a row and the walk with a row per lane give the same bits as the oracle
    (row sums in ascending group order, ojasx_lut_cpu.cpp:161-175; scale, bias, outliers :178-182, :117-127)."""
    rng = np.random.default_rng(K + M)
    ws = []
    for i in range(3):
        w = synth.make_vq_linear(300 + i, K, M, block_dim=D, outlier_frac=0.01, with_scales=True, with_bias=True)
        if kcb < 256:
            w.codes = (w.codes % kcb).astype(np.uint8)
            w.codebook = w.codebook[:kcb].copy()
        ws.append(w)
    layers = [ops.VQLinear(w.codebook, w.codes, w.scales, w.bias, w.csr, block_dim=D, codebook_size=kcb) for w in ws]
    P = 150
    group = ops.VQLinearGroup([layers[i % 3] for i in range(P)])
    x = rng.standard_normal((P, K)).astype(np.float32)
    if dtype == "bf16":
        x = synth.to_bf16_f32(x)
    xt = torch.from_numpy(x).to(cuda)
    if dtype == "bf16":
        xt = xt.bfloat16()
    want = np.empty((P, M), np.float32)
    for i, w in enumerate(ws):
        want[i::3] = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x[i::3], block_dim=D, codebook_size=kcb)
    if dtype == "bf16":
        want = synth.to_bf16_f32(want)
    for walk in ("chain", "rows"):
        monkeypatch.setenv("OJASX_B200_LINEAR_WALK", walk)
        y = torch.zeros((P, M), device=cuda, dtype=xt.dtype)
        group.forward(xt, y)
        got = y.float().cpu().numpy()
        assert np.array_equal(got, want), (walk, np.abs(got - want).max())


def test_grouped_layers_streamed_outlier_layouts(cuda, oracle):
    """Outlier layouts against the streamed epilogue of the shared-row walk (every warp brings the entries of its
    own rows in 384-entry chunks): rows longer than several chunks, warps without entries, empty rows at chunk
    ends, entry counts that are not multiples of four (the last piece of the arrays comes by plain loads), repeated
    columns; with and without scale and bias.  Bit-exact (entry order of ojasx_lut_cpu.cpp:117-126)."""
    K, M, D, P = 2560, 1000, 8, 150
    rng = np.random.default_rng(9)

    def csr_of(rows):
        rp = np.zeros(M + 1, np.int32)
        cols, vals = [], []
        for i in range(M):
            c, v = rows.get(i, ([], []))
            cols += list(c)
            vals += list(v)
            rp[i + 1] = len(cols)
        return rp, np.asarray(cols, np.int32), np.asarray(vals, np.float32)

    def run(n):
        return rng.integers(0, K, n), rng.standard_normal(n).astype(np.float32)

    layouts = [
        {0: run(1)},                                                            # one entry in the first row
        {M - 1: run(2)},                                                        # two entries in the last row
        {5: run(2001), 6: run(1), 70: run(383), 71: run(385), 500: run(1535), 999: run(7)},   # long rows, odd totals
        {i: run(int(rng.integers(0, 4))) for i in range(0, M, 3)},              # many empty rows
        {i: run(384) for i in range(64, 128)},                                  # every row of one warp is exactly a chunk
        {i: (np.full(5, 11), np.arange(5, dtype=np.float32)) for i in range(M)},  # repeated column everywhere
    ]
    for li, rows in enumerate(layouts):
        for full in (False, True):
            w = synth.make_vq_linear(700 + li, K, M, block_dim=D, outlier_frac=0, with_scales=full, with_bias=full)
            csr = csr_of(rows)
            layer = ops.VQLinear(w.codebook, w.codes, w.scales, w.bias, csr, block_dim=D)
            group = ops.VQLinearGroup([layer] * P)
            x = rng.standard_normal((P, K)).astype(np.float32)
            y = torch.zeros((P, M), device=cuda)
            group.forward(torch.from_numpy(x).to(cuda), y)
            want = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, csr, x, block_dim=D)
            assert np.array_equal(y.cpu().numpy(), want), (li, full)
    assert ojasx_b200.lib().ojasx_b200_take_device_error() == 0


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


@pytest.mark.parametrize("batch", [1, 4, 16])
def test_mlp_block_fp32_and_bf16(cuda, oracle, batch):
    """Config-1 block: gate/up 2560->6912, SiLU gate, down 6912->2560, each with its own codebook and outliers."""
    ws = [synth.make_vq_linear(70 + i, *shape, block_dim=8) for i, shape in enumerate([(2560, 6912), (2560, 6912), (6912, 2560)])]
    mlp = ops.VQMLP(*[ops.VQLinear.from_weights(w) for w in ws])
    x = np.random.default_rng(batch).standard_normal((batch, 2560)).astype(np.float32)

    def lin(w, a):
        return oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, a, block_dim=8)

    def silu(v):
        return (v / (np.float32(1) + np.exp(-v.astype(np.float64)).astype(np.float32))).astype(np.float32)

    g, u = lin(ws[0], x), lin(ws[1], x)
    want = lin(ws[2], (silu(g) * u).astype(np.float32))
    got = mlp(torch.from_numpy(x).to(cuda)).cpu().numpy()
    assert np.all(np.abs(got - want) <= 1e-6 + 1e-5 * np.abs(want)), np.abs(got - want).max()
    # bf16 activations: every stage rounds to bf16 on the way out; tolerance of the bf16 path (rel 2e-2)
    bf = synth.to_bf16_f32
    xb = bf(x)
    gb, ub = bf(lin(ws[0], xb)), bf(lin(ws[1], xb))
    want_b = bf(lin(ws[2], bf(silu(gb) * ub)))
    got_b = mlp(torch.from_numpy(xb).to(cuda).bfloat16()).float().cpu().numpy()
    assert np.allclose(got_b, want_b, rtol=2e-2, atol=2e-3), np.abs(got_b - want_b).max()


@pytest.mark.parametrize("K,M,batch", [(2560, 6912, 64), (6912, 2560, 256), (2560, 2560, 5), (640, 2560, 300), (2560, 200, 33), (1152, 130, 16)])
def test_tensor_core_dequant_gemm_bf16(cuda, oracle, K, M, batch):
    """tcgen05 path: bf16 weights (codebook rounded once) and fp32 accumulation against the fp32 oracle on
    bf16 activations; tolerance of the bf16-activation path (rel 2e-2) plus an absolute term for the
    bf16 rounding of the weights (|y| ~ 1-3 here)."""
    w = synth.make_vq_linear(K + batch, K, M, block_dim=8, with_scales=True, with_bias=True)
    xb = synth.to_bf16_f32(np.random.default_rng(batch).standard_normal((batch, K)).astype(np.float32))
    want = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, xb, block_dim=8)
    layer = ops.VQLinear.from_weights(w)
    got = layer.forward_tensor(torch.from_numpy(xb).to(cuda).bfloat16()).float().cpu().numpy()
    assert ojasx_b200.lib().ojasx_b200_take_device_error() == 0
    err = np.abs(got - want)
    assert np.all(err <= 2e-2 * np.abs(want) + 3e-2), (err.max(), np.abs(want).max())
    # the automatic switch-over (bf16, batch >= 32) takes the same path
    if batch >= 32:
        auto = layer(torch.from_numpy(xb).to(cuda).bfloat16()).float().cpu().numpy()
        assert np.array_equal(auto, got)


@pytest.mark.parametrize("frac", [0.0, 0.08])
def test_tensor_core_outlier_paths(cuda, oracle, frac):
    """No outliers at all, and so many (8 % of the cells) that a row tile's per-K-tile lists do not fit in
    shared memory and the kernel walks the rows instead."""
    K, M, batch = 2560, 300, 40
    w = synth.make_vq_linear(77, K, M, block_dim=8, outlier_frac=frac, with_scales=True, with_bias=True)
    xb = synth.to_bf16_f32(np.random.default_rng(3).standard_normal((batch, K)).astype(np.float32))
    want = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, xb, block_dim=8)
    got = ops.VQLinear.from_weights(w).forward_tensor(torch.from_numpy(xb).to(cuda).bfloat16()).float().cpu().numpy()
    assert ojasx_b200.lib().ojasx_b200_take_device_error() == 0
    err = np.abs(got - want)
    assert np.all(err <= 2e-2 * np.abs(want) + 3e-2 * (1 + 20 * frac)), (err.max(), np.abs(want).max())



@pytest.mark.parametrize("K,M,batch,frac", [(2560, 6912, 256, 0.0038), (6912, 2560, 64, 0.0038), (640, 1000, 300, 0.05), (2560, 700, 40, 0.0),
                                            (2560, 5120, 48, 0.0038),   # three K splits, 16 batch columns each
                                            (1280, 6912, 1100, 0.0038)])   # five batch tiles: the 256-row kernel by itself
def test_tensor_core_feeds_agree(cuda, oracle, monkeypatch, K, M, batch, frac):
    """The X tile by the copy engine against 16-byte copies, and the outlier lists built once per layer against the
    lists every CTA sorts for itself: the same weights meet the same activations in the same order, so with one row
    tile per CTA the outputs are equal bit for bit -- for whole layers, row slices that start off a 128-row boundary
    and a second slice of the same layer (the lists are rebuilt).  The kernel with two row tiles per CTA (forced
    here; by itself it takes batches of several 256-column tiles) splits K differently: same tolerance against the
    oracle, close to the other kernel."""
    w = synth.make_vq_linear(K + M, K, M, block_dim=8, outlier_frac=frac, with_scales=True, with_bias=True)
    layer = ops.VQLinear.from_weights(w)
    xb = synth.to_bf16_f32(np.random.default_rng(batch).standard_normal((batch, K)).astype(np.float32))
    xt = torch.from_numpy(xb).to(cuda).bfloat16()
    slices = [(0, M), (100, M - 37), (3, 131), (256, min(M, 700))]

    def run_all():
        return [layer.forward_tensor(xt, a, b) for a, b in slices]

    monkeypatch.setenv("OJASX_B200_TENSOR_ROWS", "256")
    wide = run_all()
    monkeypatch.setenv("OJASX_B200_TENSOR_ROWS", "128")
    new = run_all()
    monkeypatch.setenv("OJASX_B200_TENSOR_TMA", "0")
    no_tma = run_all()
    monkeypatch.setenv("OJASX_B200_TENSOR_NO_LISTS", "1")
    old = run_all()
    monkeypatch.delenv("OJASX_B200_TENSOR_TMA")
    no_lists = run_all()
    monkeypatch.delenv("OJASX_B200_TENSOR_NO_LISTS")
    monkeypatch.delenv("OJASX_B200_TENSOR_ROWS")
    assert ojasx_b200.lib().ojasx_b200_take_device_error() == 0
    want = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, xb, block_dim=8)
    for i, (a, b) in enumerate(slices):
        assert torch.equal(new[i], no_tma[i]) and torch.equal(new[i], old[i]) and torch.equal(new[i], no_lists[i]), slices[i]
        for y in (new[i], wide[i]):
            got = y.float().cpu().numpy()
            assert np.all(np.abs(got - want[:, a:b]) <= 2e-2 * np.abs(want[:, a:b]) + 3e-2), (slices[i], np.abs(got - want[:, a:b]).max())
        assert torch.allclose(wide[i].float(), new[i].float(), rtol=2e-2, atol=3e-2)
