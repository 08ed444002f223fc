"""RoPE table: host-side mirror of the reference's `precompute_freqs_cis`
(src/qwen3_moe/rope.rs:7-28).

freq_j = 1 / theta^(2j/dim) and angle = t * freq_j, both in float32 as in the reference; row t
holds the interleaved pairs (cos angle, sin angle) that the interleaved complex multiply of
src/kernel/generic/complex_mul.rs:3-20 expects.  The reference builds the entries with
`Complex::new(1, angle).to_polar()`, which gives (sqrt(1+angle^2), atan(angle)) instead of a
unit phasor (and never uses the table in that snapshot); this mirror writes the phasor.
"""
import numpy as np


def precompute_freqs_cis(dim, rows, theta):
    """float32 [rows, dim] table, row = absolute position."""
    x = np.arange(0, dim, 2, dtype=np.float32)
    freqs = (np.float32(1.0) / np.power(np.float32(theta), x / np.float32(dim), dtype=np.float32)).astype(np.float32)
    t = np.arange(rows, dtype=np.float32)
    ang = (t[:, None] * freqs[None, :]).astype(np.float32)
    out = np.empty((rows, dim), dtype=np.float32)
    out[:, 0::2] = np.cos(ang, dtype=np.float32)
    out[:, 1::2] = np.sin(ang, dtype=np.float32)
    return out
