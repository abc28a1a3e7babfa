"""Interface every KV cache handed to the attention layers implements.

Same contract as the reference's ``falcon_perception/kv_cache.py:12-31``:
``insert_kv(layer_id, k, v, **kwargs)`` appends new keys/values and returns
what the attention call should read.
"""

from __future__ import annotations

from abc import ABC, abstractmethod

from torch import Tensor


class KVCacheBase(ABC):
    kv_cache: Tensor | None

    @abstractmethod
    def insert_kv(self, layer_id: int, k: Tensor, v: Tensor, **kwargs) -> tuple[Tensor, Tensor]:
        """Insert new keys/values and return the cached K/V the caller attends over."""
        ...
