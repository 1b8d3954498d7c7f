"""Paged int8 KV cache resident on the GPU, with the interface of the reference's
``PagedCompressedKVCache`` (``ojasx_24x96/long_context.py:212-279``): ``append(key, value)`` with ``[B, H, S, D]``
tensors quantises every token vector to int8 with one symmetric scale (abs-max / 127, kept as fp16), pages hold
up to ``page_size`` tokens of one ``append`` call, and once more than ``max_resident_pages`` are resident the
oldest page after the ``sink_pages`` first ones is dropped (sliding window plus attention sinks).

Pages live in pools that are allocated once (``max_resident_pages + 1`` slots), so eviction only edits the page
table.  ``decode_attention`` runs one query per (sequence, head) over all resident tokens directly on the int8
pages (``ojasx_b200_paged_kv_decode``); ``iter_dequantized_pages`` yields fp pages like the reference, for callers
that feed their own attention.
"""
from __future__ import annotations

from typing import Iterator, List, Optional, Tuple

import torch

from ._lib import check, lib


class PageTable:
    """Host bookkeeping of the resident pages (pure Python: which pool slot holds which page, in age order)."""

    def __init__(self, max_resident_pages: int, sink_pages: int):
        self.max_resident_pages, self.sink_pages = int(max_resident_pages), int(sink_pages)
        self.pages: List[Tuple[int, int, int]] = []          # (slot, token count, serial number), oldest first
        self.free = list(range(self.max_resident_pages, -1, -1))   # one spare slot: a page is written before one is dropped
        self.serial = 0

    def push(self, n_tokens: int) -> int:
        """Slot for a new page of ``n_tokens``; evicts per the reference's rule (``:250-252``)."""
        slot = self.free.pop()
        self.pages.append((slot, int(n_tokens), self.serial))
        self.serial += 1
        if len(self.pages) > self.max_resident_pages:
            old = self.pages.pop(self.sink_pages)
            self.free.append(old[0])
        return slot

    @property
    def resident_tokens(self) -> int:
        return sum(p[1] for p in self.pages)


class PagedCompressedKVCache:
    def __init__(self, page_size: int = 256, max_resident_pages: int = 64, sink_pages: int = 2) -> None:
        if page_size <= 0 or max_resident_pages <= sink_pages:
            raise ValueError("Invalid page configuration for PagedCompressedKVCache")
        self.page_size = int(page_size)
        self.max_resident_pages = int(max_resident_pages)
        self.sink_pages = int(sink_pages)
        self.total_tokens_seen = 0
        self.table = PageTable(max_resident_pages, sink_pages)
        self._k = self._v = self._ks = self._vs = None       # pools, allocated at the first append
        self._shape: Optional[Tuple[int, int, int]] = None   # (B, H, D)
        self._dev_table = None
        self._scratch = self._counters = None

    # ---------------------------------------------------------------- storage
    def _allocate(self, key: torch.Tensor) -> None:
        B, H, _, D = key.shape
        slots = self.max_resident_pages + 1
        dev = key.device
        self._shape = (B, H, D)
        self._k = torch.empty((slots, B, H, self.page_size, D), dtype=torch.int8, device=dev)
        self._v = torch.empty_like(self._k)
        self._ks = torch.empty((slots, B, H, self.page_size), dtype=torch.float16, device=dev)
        self._vs = torch.empty_like(self._ks)

    def _quantize_into(self, src: torch.Tensor, q8: torch.Tensor, sc: torch.Tensor) -> None:
        """src [B, H, n, D] (fp32 / bf16) -> q8[:, :, :n], sc[:, :, :n] of one pool slot."""
        B, H, n, D = src.shape
        s = src.contiguous()
        if s.dtype not in (torch.float32, torch.bfloat16):
            s = s.float()
        tmp_q = torch.empty((B, H, n, D), dtype=torch.int8, device=s.device)
        tmp_s = torch.empty((B, H, n), dtype=torch.float16, device=s.device)
        check(lib().ojasx_b200_paged_kv_quantize(s.data_ptr(), 0 if s.dtype == torch.float32 else 1, B * H * n, D,
                                                 tmp_q.data_ptr(), tmp_s.data_ptr(),
                                                 torch.cuda.current_stream(s.device).cuda_stream), "ojasx_b200_paged_kv_quantize")
        q8[:, :, :n] = tmp_q
        sc[:, :, :n] = tmp_s

    def append(self, key: torch.Tensor, value: torch.Tensor) -> None:
        """Quantise and append a K/V chunk ``[B, H, S, D]`` (CUDA tensors) into bounded pages."""
        if not key.is_cuda:
            raise ValueError("PagedCompressedKVCache needs CUDA tensors: this package has no CPU path")
        if self._k is None:
            self._allocate(key)
        if tuple(key.shape[:2]) + (key.shape[3],) != self._shape or key.shape != value.shape:
            raise ValueError("key/value shape does not match the cache")
        S = key.shape[2]
        self.total_tokens_seen += S
        for start in range(0, S, self.page_size):
            stop = min(start + self.page_size, S)
            slot = self.table.push(stop - start)
            self._quantize_into(key[:, :, start:stop, :], self._k[slot], self._ks[slot])
            self._quantize_into(value[:, :, start:stop, :], self._v[slot], self._vs[slot])
        self._dev_table = None

    # ---------------------------------------------------------------- reading
    def iter_dequantized_pages(self, dtype: torch.dtype = torch.float32) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        for slot, n, _ in self.table.pages:
            yield ((self._k[slot][:, :, :n].float() * self._ks[slot][:, :, :n, None].float()).to(dtype),
                   (self._v[slot][:, :, :n].float() * self._vs[slot][:, :, :n, None].float()).to(dtype))

    def page(self, index: int):
        """(int8 K, fp16 K scales, int8 V, fp16 V scales) of the ``index``-th resident page, like the reference's tuples."""
        slot, n, _ = self.table.pages[index]
        return self._k[slot][:, :, :n], self._ks[slot][:, :, :n, None], self._v[slot][:, :, :n], self._vs[slot][:, :, :n, None]

    @property
    def resident_tokens(self) -> int:
        return self.table.resident_tokens

    @property
    def storage_bytes(self) -> int:
        B, H, D = self._shape if self._shape else (0, 0, 0)
        return sum(2 * B * H * n * (D + 2) for _, n, _ in self.table.pages)

    def decode_attention(self, q: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
        """``softmax(q K^T * scale) V`` over every resident token; ``q`` is ``[B, Hq, D]`` (or ``[B, Hq, 1, D]``),
        ``Hq`` a multiple of the cache's head count (grouped-query attention).  Returns the shape of ``q``."""
        if self._k is None or not self.table.pages:
            raise ValueError("the cache is empty")
        B, H, D = self._shape
        q3 = q.reshape(q.shape[0], q.shape[1], D).contiguous()
        if q3.dtype not in (torch.float32, torch.bfloat16):
            q3 = q3.float()
        dev = q3.device
        if self._dev_table is None:
            slots = [p[0] for p in self.table.pages]
            starts = [0]
            for p in self.table.pages:
                starts.append(starts[-1] + p[1])
            self._dev_table = (torch.tensor(slots, dtype=torch.int32, device=dev), torch.tensor(starts, dtype=torch.int32, device=dev),
                               len(slots), starts[-1])
        slot_t, start_t, n_pages, total = self._dev_table
        need = lib().ojasx_b200_paged_kv_scratch_floats(B, q3.shape[1], D, self.max_resident_pages * self.page_size)
        if self._scratch is None or self._scratch.numel() < need or self._counters.numel() < B * q3.shape[1]:
            self._scratch = torch.empty(need, dtype=torch.float32, device=dev)
            self._counters = torch.zeros(B * q3.shape[1], dtype=torch.int32, device=dev)
        out = torch.empty_like(q3)
        check(lib().ojasx_b200_paged_kv_decode(q3.data_ptr(), out.data_ptr(), self._k.data_ptr(), self._v.data_ptr(),
                                               self._ks.data_ptr(), self._vs.data_ptr(), slot_t.data_ptr(), start_t.data_ptr(),
                                               n_pages, total, B, q3.shape[1], H, D, self.page_size,
                                               -1.0 if scale is None else float(scale), 0 if q3.dtype == torch.float32 else 1,
                                               self._scratch.data_ptr(), self._counters.data_ptr(),
                                               torch.cuda.current_stream(dev).cuda_stream), "ojasx_b200_paged_kv_decode")
        return out.to(q.dtype).reshape(q.shape)
