"""Paged int8 KV cache against the reference's PagedCompressedKVCache run on the CPU
(tests/golden/paged_kv_ref.npz, made by tests/golden/make_paged_kv_fixture.py): page bookkeeping on the CPU,
quantised pages bit for bit and decode attention on the GPU."""
import os

import numpy as np
import pytest
import torch

from ojasx_b200 import long_context

REF = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "paged_kv_ref.npz"))


def test_page_table_follows_the_reference_eviction_rule():
    page_size, max_pages, sinks = (int(v) for v in REF["cfg"])
    table = long_context.PageTable(max_pages, sinks)
    for S in REF["appends"]:
        for start in range(0, int(S), page_size):
            table.push(min(page_size, int(S) - start))
    assert [p[1] for p in table.pages] == [REF[f"p{j}_qk"].shape[2] for j in range(int(REF["n_pages"]))]
    assert table.resident_tokens == int(REF["resident_tokens"])
    assert len({p[0] for p in table.pages}) == len(table.pages) and len(table.free) == 1   # slots are not shared
    with pytest.raises(ValueError):
        long_context.PagedCompressedKVCache(page_size=16, max_resident_pages=2, sink_pages=2)


@pytest.mark.gpu
def test_pages_and_attention_match_the_reference(cuda):
    page_size, max_pages, sinks = (int(v) for v in REF["cfg"])
    cache = long_context.PagedCompressedKVCache(page_size, max_pages, sinks)
    for i in range(len(REF["appends"])):
        cache.append(torch.from_numpy(REF[f"k{i}"]).to(cuda), torch.from_numpy(REF[f"v{i}"]).to(cuda))
    assert cache.total_tokens_seen == int(REF["total_tokens_seen"])
    assert cache.resident_tokens == int(REF["resident_tokens"])
    assert cache.storage_bytes == int(REF["storage_bytes"])
    for j in range(int(REF["n_pages"])):
        qk, sk, qv, sv = cache.page(j)
        assert np.array_equal(qk.cpu().numpy(), REF[f"p{j}_qk"]) and np.array_equal(qv.cpu().numpy(), REF[f"p{j}_qv"])
        assert np.array_equal(sk.cpu().numpy(), REF[f"p{j}_sk"]) and np.array_equal(sv.cpu().numpy(), REF[f"p{j}_sv"])
    q = torch.from_numpy(REF["q"]).to(cuda)
    got = cache.decode_attention(q).cpu().numpy()
    assert np.allclose(got, REF["attention"], rtol=1e-4, atol=1e-5), np.abs(got - REF["attention"]).max()
    again = cache.decode_attention(q).cpu().numpy()
    assert np.array_equal(again, got)
    pages = list(cache.iter_dequantized_pages())
    assert sum(p[0].shape[2] for p in pages) == cache.resident_tokens


@pytest.mark.gpu
@pytest.mark.parametrize("B,Hq,Hkv,D,tokens,dtype", [(1, 32, 8, 128, 9000, torch.float32), (3, 4, 4, 64, 700, torch.bfloat16),
                                                    (2, 8, 2, 256, 1500, torch.float32)])
def test_decode_attention_shapes(cuda, B, Hq, Hkv, D, tokens, dtype):
    """Grouped-query heads, the three head sizes, several context splits, a peaked softmax."""
    g = torch.Generator(device=cuda).manual_seed(D + tokens)
    cache = long_context.PagedCompressedKVCache(page_size=256, max_resident_pages=64, sink_pages=2)
    for start in range(0, tokens, 1000):
        n = min(1000, tokens - start)
        cache.append(torch.randn(B, Hkv, n, D, device=cuda, generator=g), torch.randn(B, Hkv, n, D, device=cuda, generator=g))
    q = (torch.randn(B, Hq, D, device=cuda, generator=g) * 3).to(dtype)
    got = cache.decode_attention(q).float()
    pages = list(cache.iter_dequantized_pages(torch.float64))
    K = torch.cat([p[0] for p in pages], 2).repeat_interleave(Hq // Hkv, 1)
    V = torch.cat([p[1] for p in pages], 2).repeat_interleave(Hq // Hkv, 1)
    att = torch.softmax(torch.einsum("bhd,bhsd->bhs", q.double(), K) / D ** 0.5, -1)
    want = torch.einsum("bhs,bhsd->bhd", att, V).float()
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    assert torch.allclose(got, want, **tol), (got - want).abs().max().item()
