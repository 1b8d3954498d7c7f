"""Generate tests/golden/ref_vectors.npz from the reference's own library.

Run in a container that holds the reference tree:  ``make -C oracle ref`` builds
oracle/_ref/libojasx_lut.so from the reference sources (default flags of the reference
Makefile), then ``python tests/golden/make_golden.py`` runs seeded / formulaic inputs through
it and stores the OUTPUT vectors plus a SHA-256 of every input array.  Inputs are regenerated
from the same seeds at test time (ojasx_b200.synth and the formulas below), so the fixture stays
a few hundred KB.  The formulaic cases restate the inputs of the reference's own tests
(split_manifold_lut_experiment/native/tests/test_native_lut.cpp:30-93 and :186-248).
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
import ojasx_b200  # noqa: E402,F401
from ojasx_b200 import synth  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_vectors.npz")


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        if a is None:
            h.update(b"none")
        else:
            a = np.ascontiguousarray(a)
            h.update(str(a.dtype).encode() + str(a.shape).encode() + a.tobytes())
    return h.hexdigest()


# ---- input builders shared with tests/test_oracle_pin.py -----------------------------------
LINEAR_CASES = {
    # name: (seed, in, out, block_dim, scales, bias, outlier_frac, batch)
    "cfg0_2560x2560": (0, 2560, 2560, 8, False, False, 0.0038, 1),
    "cfg1_gate_2560x6912": (1, 2560, 6912, 8, False, False, 0.0038, 2),
    "cfg1_down_6912x2560": (2, 6912, 2560, 8, True, True, 0.0038, 2),
    "d16_1536x1536": (3, 1536, 1536, 16, True, False, 0.0, 1),
    "ragged_200x77": (4, 200, 77, 8, True, True, 0.01, 3),
}


def linear_inputs(name):
    seed, K, M, D, sc, bi, frac, batch = LINEAR_CASES[name]
    w = synth.make_vq_linear(seed, K, M, block_dim=D, outlier_frac=frac, with_scales=sc, with_bias=bi)
    x = np.random.default_rng(1000 + seed).standard_normal((batch, K)).astype(np.float32)
    return w, x


def ref_test_linear_inputs():
    """Inputs of test_linear_correctness (test_native_lut.cpp:30-59)."""
    in_f, out_f, D = 256, 128, 16
    G = in_f // D
    k = np.arange(256)[:, None]
    d = np.arange(D)[None, :]
    cb = (((k % 17) - 8).astype(np.float32) * np.float32(0.1) + d.astype(np.float32) * np.float32(0.01)).astype(np.float32)
    m = np.arange(out_f)
    scales = (np.float32(1.0) + np.float32(0.01) * m.astype(np.float32)).astype(np.float32)
    codes = ((m[:, None] * 3 + np.arange(G)[None, :] * 7) % 256).astype(np.uint8)
    x = np.sin(np.arange(in_f, dtype=np.float32) * np.float32(0.2)).astype(np.float32)
    return cb, codes, scales, x


def ref_test_moe_inputs():
    """Inputs of test_moe_engine (test_native_lut.cpp:186-231)."""
    E, H, I, D = 512, 256, 64, 16
    G, Gi = H // D, I // D
    k = np.arange(256)
    cb = np.repeat((np.float32(0.05) * ((k % 11) - 5).astype(np.float32))[:, None], D, axis=1).astype(np.float32)
    cbd = np.repeat((np.float32(0.03) * ((k % 7) - 3).astype(np.float32))[:, None], D, axis=1).astype(np.float32)
    gu = (np.arange(E * 2 * I * G, dtype=np.int64) % 256).astype(np.uint8).reshape(E, 2 * I, G)
    dn = ((np.arange(E * H * Gi, dtype=np.int64) * 3) % 256).astype(np.uint8).reshape(E, H, Gi)
    gus, dns = np.ones((E, 2 * I), np.float32), np.ones((E, H), np.float32)
    x = np.full(H, 0.5, np.float32)
    idx = np.array([4, 12, 57, 103, 199, 255, 340, 412, 480, 511], np.int32)
    wts = np.array([0.25, 0.20, 0.15, 0.10, 0.08, 0.07, 0.05, 0.04, 0.03, 0.03], np.float32)
    return cb, cbd, gu, gus, dn, dns, x, idx, wts


def moe_seeded_inputs():
    """Config-2 geometry with 24 experts (the reference MoE has no outliers)."""
    w = synth.make_vq_moe(21, 24, 2560, 640, block_dim=8, outlier_frac=0.0, with_router=False, unit_scales=False)
    rng = np.random.default_rng(22)
    x = rng.standard_normal(2560).astype(np.float32)
    idx = np.array([3, 17, 0, 23, 9, 11, 5, -1, 24, 2], np.int32)     # includes two out-of-range ids
    wts = np.array([.2, .15, .15, .1, .1, .1, .05, .05, .05, 1e-9], np.float32)  # and one negligible weight
    return w, x, idx, wts


def kv_legacy_inputs():
    rng = np.random.default_rng(31)
    return (rng.standard_normal((200, 128)).astype(np.float32), rng.standard_normal((200, 128)).astype(np.float32),
            rng.standard_normal(128).astype(np.float32))


def pack_case(bits):
    return np.random.default_rng(40 + bits).integers(0, 1 << bits, size=1003, dtype=np.int64)


def main():
    ref = O.RefLib()
    assert ref.backend() == "Portable_ANSI_C20", ref.backend()
    out = {}
    for name in LINEAR_CASES:
        w, x = linear_inputs(name)
        y = ref.linear_forward(w.codebook, w.codes, w.scales, w.bias, w.csr, x, block_dim=w.block_dim, threads=1)
        out[f"linear/{name}/y"] = y
        out[f"linear/{name}/sha"] = np.array(digest(w.codebook, w.codes, w.scales, w.bias,
                                                    *(w.csr if w.csr else (None,)), x))
    cb, codes, scales, x = ref_test_linear_inputs()
    out["linear/ref_test/y"] = ref.linear_forward(cb, codes, scales, None, None, x, block_dim=16, threads=1)
    out["linear/ref_test/sha"] = np.array(digest(cb, codes, scales, x))
    a = ref_test_moe_inputs()
    out["moe/ref_test/y"] = ref.moe_forward(*a, block_dim=16)
    out["moe/ref_test/sha"] = np.array(digest(*a))
    w, x, idx, wts = moe_seeded_inputs()
    out["moe/seeded/y"] = ref.moe_forward(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales, w.down_codes,
                                          w.down_scales, x, idx, wts, block_dim=8)
    out["moe/seeded/sha"] = np.array(digest(w.codebook, w.down_codebook, w.gate_up_codes, w.gate_up_scales,
                                            w.down_codes, w.down_scales, x, idx, wts))
    ks, vs, q = kv_legacy_inputs()
    for D in (16, 8):
        out[f"kv_legacy/d{D}/out"] = ref.kv_run(ks, vs, q, block_dim=D)
    out["kv_legacy/sha"] = np.array(digest(ks, vs, q))
    # bit-packing of the package container (ojasx_24x96/codec.py:176-214), from the reference's own Python
    sys.path.insert(0, "/root/reference")
    import torch
    from ojasx_24x96.codec import pack_codes as ref_pack
    for bits in (1, 2, 4, 8):
        codes = torch.from_numpy(pack_case(bits))
        out[f"pack/bits{bits}"] = ref_pack(codes, bits).numpy()
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
