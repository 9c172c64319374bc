"""The reference's host-side NumPy path for the four benchmarked ops, restated: TEST INFRASTRUCTURE, not product code.

The reference (jdominick05/caminus) has no CPU build of its glue kernels; what it runs on a CPU is the NumPy code its tests and
its GGUF loader use as ground truth. These functions restate that code's arithmetic so the benchmark's CPU legs can time "the
reference's CPU/NumPy path" on the box's host cores (NumPy elementwise work: one core), and the CPU tests pin each of them to the
fixtures the reference's own code produced (tests/golden/):

    add_rms_f32        the float32 x / sqrt(mean(x^2) + eps) * w of Q3MoERef.rms (python/caminus/ref_q3moe.py:51-52) on x + d
    qk_norm_rope_f64   the per-head norm + NeoX rotation `nr` of tests/prefill/test_q3m_ops.py:204-208 (float64)
    swiglu_q8_1        silu(g) u with silu(x) = x / (1 + exp(-x)) (python/caminus/ref_q35.py) quantised as
                       tests/engine/golden_util.py:101-108 does (d = amax / 127 in float32, round half away from zero)
    q4k_rows           the Q4_K decoder of python/caminus/own_dequant.py:19-37 on the gathered raw rows
"""
import numpy as np

F32 = np.float32


def add_rms_f32(x, d, w, eps=1e-6):
    """x + d, and its RMS-normalised rows times w, all in float32"""
    xs = (x.astype(F32) + d.astype(F32)).astype(F32)
    ms = (xs * xs).mean(axis=-1, keepdims=True, dtype=F32)
    return xs, (xs / np.sqrt(ms + F32(eps)) * w.astype(F32)).astype(F32)


def qk_norm_rope_f64(x, w, pos, theta=1e6, eps=1e-6):
    """x [n, heads, hd] at positions pos [n]: per-head RMS norm with weights w [hd], then the NeoX rotation of the pairs
    (j, j + hd / 2) by pos * theta^(-2 j / hd); float64 throughout"""
    x = x.astype(np.float64); hd = x.shape[-1]; half = hd // 2
    x = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w.astype(np.float64)
    ang = np.asarray(pos, np.float64).reshape(-1, 1, 1) * (np.float64(theta) ** (-2.0 * np.arange(half) / hd))
    c, s = np.cos(ang), np.sin(ang)
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * c - b * s, b * c + a * s], -1)


def silu(x):
    x = x.astype(F32)
    return (x / (F32(1) + np.exp(-x))).astype(F32)


def q8_1_blocks(x):
    """float32 values -> Q8_1 blocks of 32: (d float16 [nb], s float16 [nb], q int8 [nb, 32]); d = amax / 127 in float32,
    q = x / d rounded half away from zero, s = the block's float32 sum"""
    x = np.asarray(x, F32).reshape(-1); nb = -(-x.size // 32)
    xb = np.zeros(nb * 32, F32); xb[:x.size] = x; xb = xb.reshape(nb, 32)
    d = (np.abs(xb).max(1) / F32(127)).astype(F32)
    safe = np.where(d > 0, d, F32(1))
    v = np.where(d[:, None] > 0, xb / safe[:, None], F32(0)).astype(F32)
    q = (np.sign(v) * np.floor(np.abs(v.astype(np.float64)) + 0.5)).astype(np.int8)
    return d.astype(np.float16), xb.sum(1, dtype=F32).astype(np.float16), q


def swiglu_q8_1(g, u):
    return q8_1_blocks(silu(g) * u.astype(F32))


def q4k_rows(table, ids):
    """table uint8 [vocab, nblk, 144] (Q4_K super-blocks of 256 values), ids [n] -> float32 [n, nblk * 256]: per super-block fp16 d
    and dmin, eight 6-bit (scale, min) pairs packed in 12 bytes, 128 bytes of nibbles (64 values per 32 bytes: low nibbles, then
    high); value = (d * scale) * q - (dmin * min)"""
    vocab, nblk = table.shape[:2]
    b = table[np.clip(np.asarray(ids, np.int64), 0, vocab - 1)].reshape(-1, 144)
    d = b[:, 0:2].copy().view(np.float16).astype(F32).reshape(-1); dmin = b[:, 2:4].copy().view(np.float16).astype(F32).reshape(-1)
    p = b[:, 4:16]
    sc = np.concatenate([p[:, 0:4] & 63, (p[:, 8:12] & 15) | ((p[:, 0:4] >> 6) << 4)], 1).astype(F32)
    mn = np.concatenate([p[:, 4:8] & 63, (p[:, 8:12] >> 4) | ((p[:, 4:8] >> 6) << 4)], 1).astype(F32)
    nib = b[:, 16:].reshape(-1, 4, 1, 32)
    q = np.concatenate([nib & 15, nib >> 4], 2).reshape(-1, 8, 32).astype(F32)
    out = (d[:, None] * sc)[:, :, None] * q - (dmin[:, None] * mn)[:, :, None]
    return out.reshape(len(ids), nblk * 256).astype(F32)
