"""Writes tests/golden/kvq_ref.npz: outputs of the REFERENCE's own functions that the codebook-VQ KV oracle
restates, on seeded inputs --

* ``ojasx_24x96.codec._nearest`` (codec.py:217-224): nearest-centroid codes of head vectors, per 8-wide block;
* ``ojasx_24x96.long_context.OnlineSoftmaxBlockAttention.forward_stream`` (long_context.py:92-176): exact
  online-softmax attention (FP64 state, GQA by head expansion) over a stream of K/V tiles, fed with the
  dequantised ``codebook[code]`` keys and values of a coded cache.

    python tests/golden/make_kvq_fixture.py /path/to/reference
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
HQ, HKV, HD, D = 8, 2, 128, 8
CTX, TILE = 1111, 200          # ragged last tile


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from ojasx_24x96.codec import _nearest
    from ojasx_24x96.long_context import OnlineSoftmaxBlockAttention

    rng = np.random.default_rng(20261125)
    sig = 1.0 / np.sqrt(HD)
    out = {"shape": np.array([HQ, HKV, HD, D, CTX, TILE])}
    # --- encode: 96 head vectors against one codebook; a few vectors sit exactly on, or midway between, centroids
    cb = (rng.standard_normal((256, D)) * sig).astype(np.float32)
    vec = (rng.standard_normal((96, HD)) * sig).astype(np.float32)
    vec[0, :D] = cb[17]
    vec[1, :D] = (cb[3] + cb[200]) * 0.5
    vec[2, :] = 0.0
    codes = _nearest(torch.from_numpy(vec.reshape(-1, D)), torch.from_numpy(cb)).numpy().reshape(96, HD // D)
    out.update(enc_codebook=cb, enc_vectors=vec, enc_codes=codes.astype(np.uint8))
    # --- decode: one sequence, GQA 8 query heads over 2 KV heads, keys/values = codebook[code]
    G = HD // D
    kc = rng.integers(0, 256, size=(HKV, CTX, G), dtype=np.uint8)
    vc = rng.integers(0, 256, size=(HKV, CTX, G), dtype=np.uint8)
    kcb = (rng.standard_normal((HKV, 256, D)) * sig).astype(np.float32)
    vcb = (rng.standard_normal((HKV, 256, D)) * sig).astype(np.float32)
    q = (rng.standard_normal((HQ, HD)) * 2.0).astype(np.float32)
    K = np.stack([kcb[h][kc[h].astype(np.int64)].reshape(CTX, HD) for h in range(HKV)])   # [HKV, CTX, HD]
    V = np.stack([vcb[h][vc[h].astype(np.int64)].reshape(CTX, HD) for h in range(HKV)])
    att = OnlineSoftmaxBlockAttention(num_heads=HQ, num_kv_heads=HKV, head_dim=HD, causal=False)
    tiles = [(torch.from_numpy(K[None, :, a:a + TILE]), torch.from_numpy(V[None, :, a:a + TILE])) for a in range(0, CTX, TILE)]
    o, rep = att.forward_stream(torch.from_numpy(q).double()[None, :, None, :], tiles)
    out.update(dec_k_codes=kc, dec_v_codes=vc, dec_k_codebook=kcb, dec_v_codebook=vcb, dec_q=q,
               dec_out=o[0, :, 0, :].numpy(), dec_kv_tokens=np.int64(rep.kv_tokens), dec_blocks=np.int64(rep.num_kv_blocks))
    np.savez_compressed(os.path.join(HERE, "kvq_ref.npz"), **out)
    print("codes", codes[:3, :4].tolist(), "out", o.dtype, tuple(o.shape), "tiles", rep.num_kv_blocks)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
