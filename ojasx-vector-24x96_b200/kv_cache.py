"""Cache accounting with the reference's entry point: ``OjasXKVCacheManager.update / reset / crop / stats``
(``ojasx_24x96/kv_cache.py:85-266``; the statistics record is ``KVCacheStats``, ``:11-28``).

The reference manager watches whatever a HuggingFace model returns as ``past_key_values`` and only counts
and trims it.  Here the caches are the codebook-quantised ``ops.VQKVCache`` objects of this package (one
per decoder layer): the manager admits a sequence length against ``max_context_length``, reports the bytes
the code storage occupies, and ``crop`` / ``reset`` act on the device-side lengths, so a cropped cache
decodes over the shorter context.  Plain tensor structures (``((k, v), ...)`` tuples, lists, dicts) are
still counted and cropped along their sequence axis, which keeps callers of the reference class working.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Optional, Union

import torch

from .ops import VQKVCache


@dataclass(frozen=True)
class KVCacheStats:
    allocated_bytes: int
    sequence_length: int
    max_context_length: int
    num_cached_layers: int
    dtype: str

    def to_dict(self) -> Dict[str, object]:
        return {"allocated_bytes": self.allocated_bytes, "sequence_length": self.sequence_length,
                "max_context_length": self.max_context_length, "num_cached_layers": self.num_cached_layers,
                "dtype": self.dtype}


def _walk(obj: Any, depth: int = 0) -> Iterable[Any]:
    """Leaves (tensors and quantised caches) of a nested cache structure."""
    if obj is None or depth > 12:
        return
    if isinstance(obj, (torch.Tensor, VQKVCache)):
        yield obj
    elif isinstance(obj, dict):
        for v in obj.values():
            yield from _walk(v, depth + 1)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            yield from _walk(v, depth + 1)
    elif hasattr(obj, "cache") and isinstance(getattr(obj, "cache"), VQKVCache):   # a decoder layer of this package
        yield obj.cache
    elif hasattr(obj, "layers"):
        yield from _walk(getattr(obj, "layers"), depth + 1)


class OjasXKVCacheManager:
    def __init__(self, max_context_length: int = 2048, default_dtype: Union[torch.dtype, str] = torch.float16) -> None:
        if max_context_length <= 0:
            raise ValueError("max_context_length must be positive")
        self.max_context_length = int(max_context_length)
        if isinstance(default_dtype, str):
            default_dtype = getattr(torch, default_dtype.lower().replace("torch.", ""), torch.float16)
        self.default_dtype = default_dtype
        self.past_key_values: Optional[Any] = None
        self._seen_tokens = 0

    # ------------------------------------------------------------------ what is held
    def _leaves(self) -> List[Any]:
        return list(_walk(self.past_key_values))

    def extract_live_tensors(self) -> List[torch.Tensor]:
        """Distinct tensors of a plain tensor structure (quantised caches own their storage inside the library)."""
        seen, out = set(), []
        for leaf in self._leaves():
            if isinstance(leaf, torch.Tensor) and leaf.device.type != "meta":
                key = (str(leaf.device), leaf.untyped_storage().data_ptr())
                if key not in seen:
                    seen.add(key)
                    out.append(leaf)
        return out

    def _infer_sequence_length(self) -> Optional[int]:
        for leaf in self._leaves():
            if isinstance(leaf, VQKVCache):
                return int(leaf.seq_len)
            if isinstance(leaf, torch.Tensor) and leaf.ndim >= 2:
                return int(leaf.shape[-2])
        return None

    @property
    def sequence_length(self) -> int:
        return max(self._seen_tokens, self._infer_sequence_length() or 0)

    @property
    def allocated_bytes(self) -> int:
        caches = [l for l in self._leaves() if isinstance(l, VQKVCache)]
        return sum(c.memory_bytes for c in caches) + sum(t.numel() * t.element_size() for t in self.extract_live_tensors())

    @property
    def num_cached_layers(self) -> int:
        pkv = self.past_key_values
        if pkv is None:
            return 0
        if hasattr(pkv, "layers"):
            return len(getattr(pkv, "layers"))
        if isinstance(pkv, (list, tuple)):
            return len(pkv)
        return len([l for l in self._leaves() if isinstance(l, VQKVCache)])

    @property
    def dtype(self) -> str:
        for leaf in self._leaves():
            if isinstance(leaf, VQKVCache):
                return "uint8_codebook_vq"
            if isinstance(leaf, torch.Tensor):
                return str(leaf.dtype).replace("torch.", "")
        return str(self.default_dtype).replace("torch.", "")

    # ------------------------------------------------------------------ the reference's four calls
    def update(self, past_key_values: Any, sequence_length: Optional[int] = None) -> None:
        self.past_key_values = past_key_values
        if sequence_length is not None:
            self._seen_tokens = int(sequence_length)
        else:
            inferred = self._infer_sequence_length()
            if inferred:
                self._seen_tokens = inferred
        if self.sequence_length > self.max_context_length:
            raise ValueError(f"KV cache sequence length ({self.sequence_length}) exceeds admission bound "
                             f"max_context_length ({self.max_context_length})")

    def reset(self) -> None:
        for leaf in self._leaves():
            if isinstance(leaf, VQKVCache):
                leaf.reset()
        if self.past_key_values is not None and hasattr(self.past_key_values, "reset"):
            try:
                self.past_key_values.reset()
            except Exception:
                pass
        self.past_key_values = None
        self._seen_tokens = 0

    def crop(self, max_length: int) -> None:
        if max_length < 0:
            raise ValueError("max_length must be nonnegative")

        def trim(obj: Any) -> Any:
            if isinstance(obj, VQKVCache):
                obj.crop(max_length)
                return obj
            if isinstance(obj, torch.Tensor):
                return obj[..., :max_length, :] if obj.ndim >= 2 and obj.shape[-2] > max_length else obj
            if isinstance(obj, tuple):
                return tuple(trim(v) for v in obj)
            if isinstance(obj, list):
                obj[:] = [trim(v) for v in obj]
                return obj
            if isinstance(obj, dict):
                for k in obj:
                    obj[k] = trim(obj[k])
                return obj
            if hasattr(obj, "cache") and isinstance(getattr(obj, "cache"), VQKVCache):
                obj.cache.crop(max_length)
            elif hasattr(obj, "layers"):
                trim(getattr(obj, "layers"))
            return obj

        if self.past_key_values is not None:
            self.past_key_values = trim(self.past_key_values)
        self._seen_tokens = min(self._seen_tokens, max_length)

    def stats(self) -> KVCacheStats:
        return KVCacheStats(self.allocated_bytes, self.sequence_length, self.max_context_length, self.num_cached_layers,
                            self.dtype)
