"""The static, non-paged KV cache in HBM: [layer, sequence, kv_head, position, head_dim].

The reference preallocates max-shape K/V tensors once and never frees them
(src/memory/allocator.rs:16-27; per-layer buffers by name,
src/memory/cache.rs:69-75) and hands the operator a stride vector
(src/qwen3_moe/attention.rs:149-166).  The device memory belongs to the library's own cache
object (ellm_kv_cache_create: one zero-filled allocation per K and V); this class is its
host-side mirror and wraps the two allocations as torch tensors (views, no copy) so that tests
and the benchmark can fill and read them.
"""
import ctypes as C

import torch

from . import _lib as L


class _DeviceArray:
    """Device memory owned elsewhere, described for torch.as_tensor (16-bit words)."""

    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<i2", "data": (ptr, False), "version": 2}


class StaticKVCache:
    def __init__(self, layers, max_batch, kv_heads, max_seq, head_dim=128, device="cuda:0",
                 dtype=torch.bfloat16):
        if dtype != torch.bfloat16:
            raise ValueError("the cache holds bf16")
        dev = torch.device(device)
        self._lib = L.load()
        self._h = C.c_void_p()
        L.check(self._lib.ellm_kv_cache_create(dev.index or 0, layers, max_batch, kv_heads, max_seq, head_dim,
                                               C.byref(self._h)))
        shape = (layers, max_batch, kv_heads, max_seq, head_dim)
        k, v = C.c_void_p(), C.c_void_p()
        strides = (C.c_size_t * 4)()
        L.check(self._lib.ellm_kv_cache_layer(self._h, 0, C.byref(k), C.byref(v), strides))
        self._strides = [int(x) for x in strides]
        with torch.cuda.device(dev):
            self.k = torch.as_tensor(_DeviceArray(k.value, shape), device=dev).view(torch.bfloat16)
            self.v = torch.as_tensor(_DeviceArray(v.value, shape), device=dev).view(torch.bfloat16)
        self.layers, self.max_batch, self.kv_heads, self.max_seq, self.head_dim = shape

    @property
    def strides(self):
        """kv_strides of one layer, in elements: (sequence, kv_head, position, head_dim)."""
        return list(self._strides)

    def layer(self, i):
        return self.k[i], self.v[i]

    def bytes(self):
        return 2 * self.k.numel() * self.k.element_size()

    def close(self):
        """Frees the device memory; the tensors handed out before must not be used afterwards."""
        if self._h:
            self.k = self.v = None
            self._lib.ellm_kv_cache_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
