"""GPU encoder (dense weight -> split-manifold layout) against the reference's own encoder run on the CPU
(tests/golden/encoder_ref.npz, made by tests/golden/make_encoder_fixture.py).  The two run the same steps;
codes can differ where a vector is (nearly) equidistant from two centroids, so agreement is asserted as a
rate and through the reconstruction error, and the layer's arithmetic is then checked bit for bit."""
import os

import numpy as np
import pytest
import torch

from ojasx_b200 import encoder, ops

pytestmark = pytest.mark.gpu
REF = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "encoder_ref.npz"))


def _ref_dense(tag, M, K, D):
    """Dense weight the reference's encoded layer represents."""
    w = (REF[f"{tag}_codebook"][REF[f"{tag}_codes"].astype(np.int64)] * REF[f"{tag}_scales"][:, None, None]).reshape(M, K)
    r, c = REF[f"{tag}_outlier_indices"]
    w[r, c] += REF[f"{tag}_outlier_values"]
    return w


@pytest.mark.parametrize("tag,D", [("d16", 16), ("d8", 8)])
def test_from_dense_matches_the_reference_encoder(cuda, oracle, tag, D):
    W = REF[f"{tag}_W"]
    M, K = W.shape
    enc = encoder.from_dense(torch.from_numpy(W).to(cuda), torch.from_numpy(REF[f"{tag}_bias"]).to(cuda), block_dim=D)
    # same outlier cells, same row scales
    rp, ci, va = enc.csr_numpy()
    rows = np.repeat(np.arange(M), np.diff(rp))
    assert np.array_equal(np.stack([rows, ci]), REF[f"{tag}_outlier_indices"])
    assert np.allclose(enc.scales.cpu().numpy(), REF[f"{tag}_scales"], rtol=1e-6, atol=0)
    # codes: same clustering up to near-ties
    agree = np.mean(enc.codes.cpu().numpy() == REF[f"{tag}_codes"])
    assert agree >= 0.97, agree
    # the represented weight is as close to W as the reference's
    err = np.linalg.norm(enc.dequantize().cpu().numpy() - W)
    err_ref = np.linalg.norm(_ref_dense(tag, M, K, D) - W)
    assert err <= 1.02 * err_ref, (err, err_ref)
    # outlier cells are restored exactly (up to one rounding of the subtraction and the addition)
    deq = enc.dequantize().cpu().numpy()
    r, c = REF[f"{tag}_outlier_indices"]
    assert np.allclose(deq[r, c], W[r, c], rtol=1e-6, atol=1e-7)
    # the encoded layer runs on the table kernels: bit-exact against the oracle on the same arrays, and within the
    # encoder's own error of the reference layer's output
    x = REF[f"{tag}_x"]
    got = enc.to_vq_linear()(torch.from_numpy(x).to(cuda)).cpu().numpy()
    want = oracle.linear_forward(enc.codebook.cpu().numpy(), enc.codes.cpu().numpy(), enc.scales.cpu().numpy(),
                                 enc.bias.cpu().numpy(), enc.csr_numpy(), x, block_dim=D)
    assert np.array_equal(got, want)
    dense = x @ W.T + REF[f"{tag}_bias"]
    assert np.abs(got - dense).max() <= 1.1 * np.abs(REF[f"{tag}_y"] - dense).max() + 1e-4


def test_vq_assign_first_minimum_and_sums(cuda):
    rng = np.random.default_rng(0)
    v = rng.standard_normal((5000, 8)).astype(np.float32)
    cb = rng.standard_normal((256, 8)).astype(np.float32)
    cb[200] = cb[17]                                    # duplicate centroid: the lower index wins
    codes, sums, counts = encoder.vq_assign(torch.from_numpy(v).to(cuda), torch.from_numpy(cb).to(cuda), want_sums=True)
    d = ((v[:, None, :].astype(np.float64) - cb[None].astype(np.float64)) ** 2).sum(-1)
    want = d.argmin(1)
    got = codes.cpu().numpy()
    close = np.sort(d, 1)[:, 1] - np.sort(d, 1)[:, 0] < 1e-5   # fp32 near-ties may go either way
    assert np.all((got == want) | close) and not np.any(got == 200)
    assert int(counts.sum()) == 5000
    s = np.zeros((256, 8)); np.add.at(s, got, v.astype(np.float64))
    assert np.allclose(sums.cpu().numpy(), s, rtol=1e-12, atol=1e-12)
