"""Writes tests/golden/paged_kv_ref.npz: a seeded sequence of appends run through the REFERENCE's
PagedCompressedKVCache (ojasx_24x96/long_context.py:212-279) on the CPU -- the resident pages it ends with
(int8 values, fp16 scales), its counters, and the attention of a seeded query over its dequantised pages.

    python tests/golden/make_paged_kv_fixture.py /path/to/reference
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
APPENDS = (40, 7, 1, 1, 30, 16, 5)     # token counts of the successive append calls
CFG = dict(page_size=16, max_resident_pages=5, sink_pages=1)
B, H, D = 1, 2, 64


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from ojasx_24x96.long_context import PagedCompressedKVCache

    g = torch.Generator().manual_seed(20261104)
    cache = PagedCompressedKVCache(**CFG)
    out = {"appends": np.array(APPENDS), "cfg": np.array([CFG["page_size"], CFG["max_resident_pages"], CFG["sink_pages"]]),
           "shape": np.array([B, H, D])}
    for i, S in enumerate(APPENDS):
        k = torch.randn(B, H, S, D, generator=g)
        v = torch.randn(B, H, S, D, generator=g) * (1.0 + i)
        out[f"k{i}"], out[f"v{i}"] = k.numpy(), v.numpy()
        cache.append(k, v)
    out["total_tokens_seen"] = np.int64(cache.total_tokens_seen)
    out["resident_tokens"] = np.int64(cache.resident_tokens)
    out["storage_bytes"] = np.int64(cache.storage_bytes)
    out["n_pages"] = np.int64(len(cache._pages))
    for j, (qk, sk, qv, sv) in enumerate(cache._pages):
        out[f"p{j}_qk"], out[f"p{j}_sk"], out[f"p{j}_qv"], out[f"p{j}_sv"] = qk.numpy(), sk.numpy(), qv.numpy(), sv.numpy()
    q = torch.randn(B, H, D, generator=g)
    pages = list(cache.iter_dequantized_pages(torch.float32))
    K = torch.cat([p[0] for p in pages], dim=2).double()
    V = torch.cat([p[1] for p in pages], dim=2).double()
    att = torch.softmax(torch.einsum("bhd,bhsd->bhs", q.double(), K) / D ** 0.5, dim=-1)
    out["q"] = q.numpy()
    out["attention"] = torch.einsum("bhs,bhsd->bhd", att, V).numpy()
    np.savez_compressed(os.path.join(HERE, "paged_kv_ref.npz"), **out)
    print("pages", [p[0].shape[2] for p in cache._pages], "resident", cache.resident_tokens, "seen", cache.total_tokens_seen)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
