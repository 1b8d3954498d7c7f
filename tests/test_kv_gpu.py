"""GPU parity of the quantized KV cache: codebook-VQ append/decode and the reference's cache as shipped."""
import numpy as np
import pytest
import torch

from ojasx_b200 import lut_ctypes, ops, synth

pytestmark = pytest.mark.gpu


def _oracle_decode(oracle, kv, kc, vc, q):
    B, Hq, hd = q.shape
    R = Hq // kv.kv_heads
    out = np.zeros((B, Hq, hd), np.float64)
    for b in range(B):
        for h in range(kv.kv_heads):
            out[b, h * R:(h + 1) * R] = oracle.kvq_decode(q[b, h * R:(h + 1) * R], kc[b, h], vc[b, h],
                                                          kv.k_codebook[h], kv.v_codebook[h], block_dim=kv.block_dim)
    return out


@pytest.mark.parametrize("B,ctx", [(1, 2048), (2, 777), (1, 5000), (16, 300)])
def test_kvq_append_then_decode(cuda, oracle, B, ctx):
    kv = synth.make_vq_kv(ctx + B, B, ctx)
    cache = ops.VQKVCache(B, kv.kv_heads, kv.q_heads, kv.head_dim, kv.block_dim, ctx + 8, kv.k_codebook, kv.v_codebook)
    cache.load(kv.k_codes, kv.v_codes)
    cache.append(torch.from_numpy(kv.new_k).to(cuda), torch.from_numpy(kv.new_v).to(cuda))
    assert cache.seq_len == ctx + 1
    # append: index-exact against the oracle's nearest-centroid rule
    gk, gv = cache.read(ctx, ctx + 1)
    for h in range(kv.kv_heads):
        assert np.array_equal(gk[:, h, 0], oracle.kvq_encode(kv.new_k[:, h], kv.k_codebook[h], block_dim=kv.block_dim))
        assert np.array_equal(gv[:, h, 0], oracle.kvq_encode(kv.new_v[:, h], kv.v_codebook[h], block_dim=kv.block_dim))
    kc = np.concatenate([kv.k_codes, gk], axis=2)
    vc = np.concatenate([kv.v_codes, gv], axis=2)
    # decode, fp32 queries: fp32 accumulation against the fp64 online softmax.  Tolerance rel 1e-4 / abs 2e-6, wider
    # than the 1e-5 / 1e-6 of the linear path on purpose: the oracle accumulates in fp64 while the kernel adds a
    # token's 16 partial scores in fp32 in a per-lane rotated group order (the conflict-free table gathers), takes
    # exp() of scores of magnitude ~10 (one fp32 ulp of the score is 1e-6 relative in the probability) and sums
    # probability-weighted values over thousands of tokens in fp32; no reference implementation of the codebook-VQ
    # cache exists whose order could be matched bit for bit.
    want = _oracle_decode(oracle, kv, kc, vc, kv.q)
    got = cache.decode(torch.from_numpy(kv.q).to(cuda)).cpu().numpy()
    assert np.allclose(got, want, rtol=1e-4, atol=2e-6), np.abs(got - want).max()
    # decode, bf16 queries and output: tolerance of the bf16 activation path (rel 2e-2)
    qb = synth.to_bf16_f32(kv.q)
    want_b = _oracle_decode(oracle, kv, kc, vc, qb)
    got_b = cache.decode(torch.from_numpy(qb).to(cuda).to(torch.bfloat16)).float().cpu().numpy()
    assert np.allclose(got_b, want_b, rtol=2e-2, atol=2e-3), np.abs(got_b - want_b).max()


@pytest.mark.parametrize("B,ctx,kv_heads,q_heads,head_dim,block_dim,q_gain", [
    (4, 8192, 8, 32, 128, 8, 6.0),     # ranges of 1024 tokens: two passes per CTA, peaked softmax (running-max rescale)
    (8, 20000, 8, 32, 128, 8, 1.0),    # ranges of several thousand tokens with a ragged tail
    (2, 1500, 4, 4, 64, 4, 3.0),       # one query head per KV head, block_dim 4
    (3, 900, 2, 16, 128, 16, 3.0),     # eight query heads per KV head, block_dim 16 (8 groups: byte code loads)
    (2, 700, 4, 8, 96, 8, 2.0),        # head_dim 96: 12 groups
])
def test_kvq_decode_shapes_and_long_ranges(cuda, oracle, B, ctx, kv_heads, q_heads, head_dim, block_dim, q_gain):
    kv = synth.make_vq_kv(ctx + head_dim, B, ctx, kv_heads=kv_heads, q_heads=q_heads, head_dim=head_dim, block_dim=block_dim)
    q = (kv.q * q_gain).astype(np.float32)
    cache = ops.VQKVCache(B, kv_heads, q_heads, head_dim, block_dim, ctx + 300, kv.k_codebook, kv.v_codebook)
    cache.load(kv.k_codes, kv.v_codes)
    want = _oracle_decode(oracle, kv, kv.k_codes, kv.v_codes, q)
    got = cache.decode(torch.from_numpy(q).to(cuda)).cpu().numpy()
    assert np.allclose(got, want, rtol=1e-4, atol=2e-6), np.abs(got - want).max()
    # planned for the capacity (the CUDA-graph mode): other splits, same tolerance
    cache.set_static_plan(True)
    again = cache.decode(torch.from_numpy(q).to(cuda)).cpu().numpy()
    assert np.allclose(again, want, rtol=1e-4, atol=2e-6), np.abs(again - want).max()


@pytest.mark.parametrize("B,ctx,samples", [(1, 32768, [(0, 0), (0, 5)]), (16, 32768, [(0, 1), (7, 3), (15, 7)]),
                                           (1, 131072, [(0, 2), (0, 7)])])
def test_kvq_decode_baseline_contexts(cuda, oracle, B, ctx, samples):
    """Configuration 3 at its long contexts (32 query / 8 KV heads of 128, 16 codes per vector), one appended token
    then one decode query.  The CPU oracle (fp64 online softmax, pinned to the reference's
    OnlineSoftmaxBlockAttention) checks a sample of (sequence, KV head) pairs to bound its run time.

    Tolerance: the kernel accumulates scores, the softmax normaliser and the context vector in fp32 over `ctx`
    terms while the oracle (like the reference's attention) works in fp64; rounding alone gives about
    sqrt(ctx) * 2^-24 ~ 1e-5 relative to the sum of magnitudes at these lengths, so the comparison allows
    rel 1e-4 / abs 2e-6 and reports the largest deviation it saw."""
    kv = synth.make_vq_kv(ctx + B, B, ctx)
    cache = ops.VQKVCache(B, kv.kv_heads, kv.q_heads, kv.head_dim, kv.block_dim, ctx + 64, kv.k_codebook, kv.v_codebook)
    cache.load(kv.k_codes, kv.v_codes)
    cache.append(torch.from_numpy(kv.new_k).to(cuda), torch.from_numpy(kv.new_v).to(cuda))
    gk, gv = cache.read(ctx, ctx + 1)
    got = cache.decode(torch.from_numpy(kv.q).to(cuda)).cpu().numpy()
    qb = synth.to_bf16_f32(kv.q)
    got_b = cache.decode(torch.from_numpy(qb).to(cuda).to(torch.bfloat16)).float().cpu().numpy()
    R = kv.q_heads // kv.kv_heads
    worst = 0.0
    for b, h in samples:
        assert np.array_equal(gk[b, h, 0], oracle.kvq_encode(kv.new_k[b, h], kv.k_codebook[h], block_dim=kv.block_dim))
        kc = np.concatenate([kv.k_codes[b, h], gk[b, h]], axis=0)
        vc = np.concatenate([kv.v_codes[b, h], gv[b, h]], axis=0)
        want = oracle.kvq_decode(kv.q[b, h * R:(h + 1) * R], kc, vc, kv.k_codebook[h], kv.v_codebook[h], block_dim=kv.block_dim)
        g = got[b, h * R:(h + 1) * R]
        assert np.allclose(g, want, rtol=1e-4, atol=2e-6), np.abs(g - want).max()
        worst = max(worst, float(np.max(np.abs(g - want) / (np.abs(want) + 1e-3))))
        want_b = oracle.kvq_decode(qb[b, h * R:(h + 1) * R], kc, vc, kv.k_codebook[h], kv.v_codebook[h], block_dim=kv.block_dim)
        assert np.allclose(got_b[b, h * R:(h + 1) * R], want_b, rtol=2e-2, atol=2e-3)
    print(f"B={B} ctx={ctx}: largest |got - want| / (|want| + 1e-3) = {worst:.2e}")
    cache.close()


def test_kvq_full_and_errors(cuda):
    kv = synth.make_vq_kv(1, 1, 4)
    cache = ops.VQKVCache(1, 8, 32, 128, 8, 4, kv.k_codebook, kv.v_codebook)
    cache.load(kv.k_codes, kv.v_codes)
    from ojasx_b200 import OjasxB200Error
    with pytest.raises(OjasxB200Error):
        cache.append(torch.from_numpy(kv.new_k).to(cuda), torch.from_numpy(kv.new_v).to(cuda))  # full: -2
    cache.reset()
    with pytest.raises(OjasxB200Error):
        cache.decode(torch.from_numpy(kv.q).to(cuda))  # empty: -2


def test_legacy_kv_cache_matches_reference_semantics(cuda, oracle):
    """ojasx_create_kv_cache / append / attention: the reference's cache as shipped, through the
    reference's ctypes class (shape of native/tests/test_kv_cache_binding.py)."""
    rng = np.random.default_rng(5)
    for D, T in ((16, 500), (8, 1300)):
        G = 128 // D
        cache = lut_ctypes.NativeKVCache(num_heads=2, head_dim=128, max_seq_len=64, block_dim=D)
        ks = rng.standard_normal((T, 128)).astype(np.float32)
        vs = rng.standard_normal((T, 128)).astype(np.float32)
        q = rng.standard_normal(128).astype(np.float32)
        kc, vc = np.zeros((T, G), np.uint8), np.zeros((T, G), np.uint8)
        ksc, vsc = np.zeros(T, np.float32), np.zeros(T, np.float32)
        for t in range(T):
            cache.append(0, ks[t], vs[t])
            kc[t], vc[t], ksc[t], vsc[t] = oracle.kv_legacy_append(ks[t], vs[t], block_dim=D)
        want = oracle.kv_legacy_attention(q, kc, vc, ksc, vsc, block_dim=D)
        got = cache.attention(0, q)
        assert np.allclose(got, want, rtol=1e-4, atol=1e-6), np.abs(got - want).max()
        assert np.all(got.reshape(G, D)[:, 1:] == 0)          # only each block's first coordinate is written
        assert np.all(cache.attention(1, q) == 0)             # empty head: output untouched (zeros)
        assert cache.compression_ratio >= 12.0
