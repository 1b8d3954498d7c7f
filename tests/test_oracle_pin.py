"""CPU tests: the oracle (oracle/oracle_port.c) against the reference's own outputs.

* committed golden vectors (tests/golden/ref_vectors.npz, produced by tests/golden/make_golden.py
  from the reference library) -- always run;
* the reference library itself when oracle/_ref/ was built -- extra random cases;
* torch-CPU formulas for the parts the reference has no implementation of (router, codebook-VQ
  KV cache, CSR on experts).
Linear, MoE-without-outliers and the legacy KV cache are compared bit for bit.
"""
import importlib.util
import os

import numpy as np
import pytest
import torch

from ojasx_b200 import synth

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
mg = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(mg)
GOLD = np.load(os.path.join(HERE, "golden", "ref_vectors.npz"))


@pytest.mark.parametrize("name", list(mg.LINEAR_CASES))
def test_linear_port_equals_golden(oracle, name):
    w, x = mg.linear_inputs(name)
    assert str(GOLD[f"linear/{name}/sha"]) == mg.digest(w.codebook, w.codes, w.scales, w.bias,
                                                        *(w.csr if w.csr else (None,)), x), "inputs drifted"
    y = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=w.block_dim)
    assert np.array_equal(y, GOLD[f"linear/{name}/y"])


def test_linear_reference_test_case(oracle):
    """The reference's own known-answer check (test_native_lut.cpp:61-88): forward vs manual unpack < 1e-4."""
    cb, codes, scales, x = mg.ref_test_linear_inputs()
    assert str(GOLD["linear/ref_test/sha"]) == mg.digest(cb, codes, scales, x)
    y = oracle.linear_forward(cb, codes, scales, None, None, x, block_dim=16)
    assert np.array_equal(y, GOLD["linear/ref_test/y"])
    manual = np.array([(x.reshape(16, 16) * cb[codes[m]]).sum(1).sum() * scales[m] for m in range(128)])
    assert np.abs(y - manual).max() < 1e-4


def test_csr_reference_test_case(oracle):
    """Shape and assertion of test_outliers_and_csr (test_native_lut.cpp:95-126): y[0] >= 4.5."""
    in_f, out_f = 64, 32
    rp = (np.arange(out_f + 1) * 2).astype(np.int32)
    cols = np.stack([(np.arange(out_f) * 2) % in_f, (np.arange(out_f) * 2 + 1) % in_f], 1).reshape(-1).astype(np.int32)
    vals = np.tile(np.array([10.0, -5.0], np.float32), out_f)
    y = oracle.linear_forward(np.zeros((256, 16), np.float32), np.zeros((out_f, 4), np.uint8), None, None,
                              (rp, cols, vals), np.ones(in_f, np.float32), block_dim=16)
    assert np.all(y == 5.0) and y[0] >= 4.5


def test_moe_port_equals_golden(oracle):
    a = mg.ref_test_moe_inputs()
    assert str(GOLD["moe/ref_test/sha"]) == mg.digest(*a)
    cb, cbd, gu, gus, dn, dns, x, idx, wts = a
    y = oracle.moe_forward(cb, cbd, gu, gus, dn, dns, x, idx, wts, block_dim=16)
    assert np.array_equal(y, GOLD["moe/ref_test/y"])
    w, x, idx, wts = mg.moe_seeded_inputs()
    y = oracle.moe_forward(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes,
                           w.down_scales, x, idx, wts, block_dim=8)
    assert np.array_equal(y, GOLD["moe/seeded/y"])


def test_kv_legacy_port_equals_golden(oracle):
    ks, vs, q = mg.kv_legacy_inputs()
    assert str(GOLD["kv_legacy/sha"]) == mg.digest(ks, vs, q)
    for D in (16, 8):
        G = 128 // D
        kc, vc = np.zeros((200, G), np.uint8), np.zeros((200, G), np.uint8)
        ksc, vsc = np.zeros(200, np.float32), np.zeros(200, np.float32)
        for t in range(200):
            kc[t], vc[t], ksc[t], vsc[t] = oracle.kv_legacy_append(ks[t], vs[t], block_dim=D)
        out = oracle.kv_legacy_attention(q, kc, vc, ksc, vsc, block_dim=D)
        assert np.array_equal(out, GOLD[f"kv_legacy/d{D}/out"])


def test_port_equals_live_reference(oracle, reflib):
    """Random extra cases against the compiled reference (skipped where it was not built)."""
    assert reflib.backend() == "Portable_ANSI_C20"
    for seed, (K, M, D) in enumerate([(640, 2560, 8), (2560, 1280, 8), (256, 100, 16), (72, 50, 4)]):
        w = synth.make_vq_linear(50 + seed, K, M, block_dim=D, with_scales=bool(seed & 1), with_bias=bool(seed & 2))
        x = np.random.default_rng(seed).standard_normal((2, K)).astype(np.float32)
        a = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=D)
        for threads in (1, 0):
            b = reflib.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=D, threads=threads)
            assert np.array_equal(a, b)


def test_moe_outlier_extension_is_the_linear_composition(oracle):
    """CSR on experts has no reference implementation; it must equal composing the (pinned) linear layers."""
    w = synth.make_vq_moe(9, 6, 256, 64, block_dim=8, outlier_frac=0.02, unit_scales=False)
    rng = np.random.default_rng(1)
    x = rng.standard_normal(256).astype(np.float32)
    idx, wts = np.array([4, 1, 5], np.int32), np.array([0.5, 0.3, 0.2], np.float32)
    got = oracle.moe_forward(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes, w.down_scales,
                             x, idx, wts, block_dim=8, gu_csr=w.gate_up_csr, dn_csr=w.down_csr)

    def sub_csr(csr, r0, r1):
        rp, ci, va = csr
        lo, hi = rp[r0], rp[r1]
        return (rp[r0:r1 + 1] - lo, ci[lo:hi], va[lo:hi])

    y = np.zeros(256, np.float32)
    for e, we in zip(idx, wts):
        gu = oracle.linear_forward(w.codebook, w.gate_up_codes[e], w.gate_up_scales[e], None,
                                   sub_csr(w.gate_up_csr, e * 128, (e + 1) * 128), x, block_dim=8)
        gate, up = gu[:64], gu[64:]
        e_neg = np.array([np.float32(np.exp(np.float32(-g))) for g in gate], np.float32)  # expf
        inter = ((gate / (np.float32(1.0) + e_neg)).astype(np.float32) * up).astype(np.float32)
        dn = oracle.linear_forward(w.down_codebook, w.down_codes[e], w.down_scales[e], None,
                                   sub_csr(w.down_csr, e * 256, (e + 1) * 256), inter, block_dim=8)
        y = (y + (dn * we).astype(np.float32)).astype(np.float32)
    assert np.allclose(got, y, rtol=1e-6, atol=1e-7)


def test_router_oracle_against_torch(oracle):
    rng = np.random.default_rng(3)
    Wr = (rng.standard_normal((512, 2560)) * 0.02).astype(np.float32)
    x = rng.standard_normal((64, 2560)).astype(np.float32)
    idx, w, probs = oracle.router_topk(x, Wr, 10, return_probs=True)
    p = torch.softmax(torch.from_numpy(x) @ torch.from_numpy(Wr).T, dim=-1)
    tw, ti = torch.topk(p, 10, dim=-1)
    tw = tw / tw.sum(-1, keepdim=True)
    assert np.array_equal(idx, ti.numpy())
    assert np.allclose(w, tw.numpy(), rtol=1e-5, atol=1e-7)
    assert np.allclose(probs, p.numpy(), rtol=1e-5, atol=1e-8)
    assert np.allclose(w.sum(1), 1.0, atol=1e-6)


def test_kvq_encode_against_torch_rule(oracle):
    """codec.py:217-224: argmin of |v|^2 - 2 v.C + |C|^2."""
    rng = np.random.default_rng(0)
    cb = (rng.standard_normal((256, 8)) / np.sqrt(128)).astype(np.float32)
    v = (rng.standard_normal((64, 128)) / np.sqrt(128)).astype(np.float32)
    codes = oracle.kvq_encode(v, cb, block_dim=8)
    vt, ct = torch.from_numpy(v.reshape(-1, 8)), torch.from_numpy(cb)
    d = vt.square().sum(1, keepdim=True) - 2 * vt @ ct.T + ct.square().sum(1).unsqueeze(0)
    assert np.array_equal(codes.reshape(-1), d.argmin(1).numpy().astype(np.uint8))


def test_kvq_decode_against_torch_attention(oracle):
    """Online softmax over dequantised K/V (long_context.py:92-176) == plain fp64 softmax attention."""
    kv = synth.make_vq_kv(4, 1, 700)
    q = kv.q[0, :4]
    got = oracle.kvq_decode(q, kv.k_codes[0, 0], kv.v_codes[0, 0], kv.k_codebook[0], kv.v_codebook[0], block_dim=8,
                            kv_block=256)
    K = torch.from_numpy(kv.k_codebook[0][kv.k_codes[0, 0].astype(np.int64)].reshape(700, 128)).double()
    V = torch.from_numpy(kv.v_codebook[0][kv.v_codes[0, 0].astype(np.int64)].reshape(700, 128)).double()
    s = torch.from_numpy(q).double() @ K.T / np.sqrt(128.0)
    want = (torch.softmax(s, -1) @ V).numpy()
    assert np.allclose(got, want, rtol=1e-12, atol=1e-14)
    # block size must not matter
    got2 = oracle.kvq_decode(q, kv.k_codes[0, 0], kv.v_codes[0, 0], kv.k_codebook[0], kv.v_codebook[0], block_dim=8,
                             kv_block=64)
    assert np.allclose(got, got2, rtol=1e-12, atol=1e-14)


def test_fp32_order_versus_exact_sum(oracle):
    """How far the reference's fp32 order is from the exact sum: the reason the GPU keeps that order."""
    w, x = mg.linear_inputs("cfg1_down_6912x2560")
    y = oracle.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=8)
    f = oracle.linear_forward_f64(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=8)
    assert np.abs(y - f).max() < 5e-5
    viol = int(np.sum(np.abs(y - f) > 1e-6 + 1e-5 * np.abs(f)))
    assert viol > 0  # a result rounded differently from the reference would miss the 1e-5/1e-6 bar here


def test_pack_codes_matches_reference_bit_layout():
    """codec.pack_codes / unpack_codes against bytes produced by the reference's own pack_codes."""
    from ojasx_b200 import codec
    for bits in (1, 2, 4, 8):
        codes = torch.from_numpy(mg.pack_case(bits))
        packed = codec.pack_codes(codes, bits)
        assert np.array_equal(packed.numpy(), GOLD[f"pack/bits{bits}"])
        assert torch.equal(codec.unpack_codes(packed, bits, codes.numel()).long(), codes)
    assert codec.pack_codes(torch.tensor([1, 2, 3, 0]), 2).tolist() == [0b00111001]


def test_kvq_oracle_against_reference_functions(oracle):
    """The codebook-VQ KV oracle against outputs of the reference's own code (tests/golden/kvq_ref.npz, written by
    tests/golden/make_kvq_fixture.py): codes from ojasx_24x96.codec._nearest (codec.py:217-224) and attention from
    OnlineSoftmaxBlockAttention.forward_stream (long_context.py:92-176) over the dequantised cache."""
    ref = np.load(os.path.join(os.path.dirname(__file__), "golden", "kvq_ref.npz"))
    HQ, HKV, HD, D, CTX, TILE = (int(v) for v in ref["shape"])
    codes = oracle.kvq_encode(ref["enc_vectors"], ref["enc_codebook"], block_dim=D)
    assert np.array_equal(codes, ref["enc_codes"])
    R = HQ // HKV
    for tile in (256, TILE, 64):       # the oracle's own tile size must not matter; the reference used TILE
        got = np.concatenate([oracle.kvq_decode(ref["dec_q"][h * R:(h + 1) * R], ref["dec_k_codes"][h], ref["dec_v_codes"][h],
                                                ref["dec_k_codebook"][h], ref["dec_v_codebook"][h], block_dim=D, kv_block=tile)
                              for h in range(HKV)])
        assert np.allclose(got, ref["dec_out"], rtol=1e-11, atol=1e-14), np.abs(got - ref["dec_out"]).max()
