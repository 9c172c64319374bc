"""The host-side position checks the glue wrappers share with the reference's decode engine
(python/caminus/engine/k3.py:413-433, 535-540): refused on the host before any launch, nothing is written."""
import numpy as np

YARN_TABLE_FLOATS = 65   # freq [64] | mscale after the decode block's eps (python/caminus/engine/k3.py:130)


class ContextBoundsError(IndexError):
    """a position outside what the KV cache holds: refused on the host before any launch"""


def check_span(i0, n, max_ctx, what='pass'):
    """positions i0 .. i0 + n - 1 must lie in [0, max_ctx)"""
    if isinstance(i0, bool) or not isinstance(i0, (int, np.integer)):
        raise ContextBoundsError(f'k3 {what}: position {i0!r} is not an int')
    i0, n = int(i0), int(n)
    if i0 < 0 or n < 1 or i0 + n > max_ctx:
        raise ContextBoundsError(f'k3 {what}: positions {i0} .. {i0 + n - 1} outside the KV cache [0, {max_ctx})')


def kv_pos_bytes(M, q8=False):
    """bytes of one position's K | V row: 2 M fp16 values, or 2 (M / 32) Q8_0 blocks of 34 bytes"""
    return 2 * (M // 32) * 34 if q8 else 2 * M * 2


def kv_rows(cache, M, q8=False):
    """positions a KV cache holds, from its allocation"""
    pb = kv_pos_bytes(M, q8); nb = cache.numel() * cache.element_size()
    if q8 and M % 32: raise ValueError(f'k3 KV cache: {M} values per position is not a whole number of q8_0 blocks')
    if nb % pb or not 0 < nb // pb < 2 ** 31: raise ValueError(f'k3 KV cache: {nb} bytes is not a whole number of {pb}-byte positions')
    return nb // pb
