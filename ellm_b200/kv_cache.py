"""The static, non-paged KV cache in HBM: [layer, sequence, kv_head, position, head_dim].

The reference preallocates max-shape K/V tensors once and never frees them
(src/memory/allocator.rs:16-27; per-layer buffers by name,
src/memory/cache.rs:69-75) and hands the operator a stride vector
(src/qwen3_moe/attention.rs:149-166).  This class does the same on the device:
one allocation per K and V, `strides` in the operator's (sequence, kv_head,
position, head_dim) order.  torch is used only to own the device memory.
"""
import torch


class StaticKVCache:
    def __init__(self, layers, max_batch, kv_heads, max_seq, head_dim=128, device="cuda:0",
                 dtype=torch.bfloat16):
        shape = (layers, max_batch, kv_heads, max_seq, head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.layers, self.max_batch, self.kv_heads, self.max_seq, self.head_dim = shape

    @property
    def strides(self):
        """kv_strides of one layer, in elements: (sequence, kv_head, position, head_dim)."""
        return [self.kv_heads * self.max_seq * self.head_dim, self.max_seq * self.head_dim,
                self.head_dim, 1]

    def layer(self, i):
        return self.k[i], self.v[i]

    def bytes(self):
        return 2 * self.k.numel() * self.k.element_size()
