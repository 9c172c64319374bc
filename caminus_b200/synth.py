"""Seeded synthetic inputs of the benchmark configurations (numpy, host side): `numpy.random.default_rng(seed)`, one
generator per tensor in the listed order, so that tests, the benchmark and a CPU baseline all see the same bytes.
No dataset or model file is involved anywhere in this library's measurements."""
import numpy as np


def _rng(seed, k):
    return np.random.default_rng([seed, k])


def _normal(g, shape, scale=1.0, dtype=np.float32, chunk=1 << 24):
    """N(0, scale) of `shape` drawn in float32 pieces (a float64 draw of the large configs would not fit beside them)"""
    n = int(np.prod(shape)); out = np.empty(n, dtype)
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        v = g.standard_normal(b - a, dtype=np.float32)
        if scale != 1.0: v *= np.float32(scale)
        out[a:b] = v
    return out.reshape(shape)


def add_rms_inputs(T, N, seed=0, dtype=np.float32):
    """x, residual ~ N(0, 1) [T, N]; weight = 1 + N(0, 0.05) fp32 [N]"""
    x = _normal(_rng(seed, 0), (T, N), 1.0, dtype); r = _normal(_rng(seed, 1), (T, N), 1.0, dtype)
    w = (1.0 + 0.05 * _rng(seed, 2).standard_normal(N)).astype(np.float32)
    return x, r, w


def rope_par(seed=0, theta=1e6, eps=1e-6, hd=128, yarn_table=None):
    """q_norm | k_norm = 1 + N(0, 0.05) | theta_scale = fp32(fp32(theta)^fp32(-2 / hd)) | eps (| freq[64] | mscale)"""
    qn = (1.0 + 0.05 * _rng(seed, 10).standard_normal(hd)).astype(np.float32)
    kn = (1.0 + 0.05 * _rng(seed, 11).standard_normal(hd)).astype(np.float32)
    ts = np.float32(np.float32(theta) ** np.float32(-2.0 / hd))
    par = np.concatenate([qn, kn, np.array([ts, eps], np.float32)])
    if yarn_table is not None: par = np.concatenate([par, np.asarray(yarn_table, np.float32)])
    return par.astype(np.float32)


def yarn_table(n_rot=128, base=1e6, factor=4.0, n_ctx_orig=32768, beta_fast=32.0, beta_slow=1.0):
    """freq[n_rot / 2] | mscale in fp32: the YaRN recipe of llama.cpp's rope_yarn as the reference tabulates it on the host
    (python/caminus/rope.py:27-50), in float64 rounded once"""
    import math
    dim = lambda beta: n_rot * math.log(n_ctx_orig / (beta * 2 * math.pi)) / (2 * math.log(base))
    lo, hi = max(0.0, float(math.floor(dim(beta_fast)))), min(float(n_rot - 1), float(math.ceil(dim(beta_slow))))
    j = np.arange(n_rot // 2, dtype=np.float64)
    inv = base ** (-2.0 * j / n_rot)
    ramp = 1.0 - np.clip((j - lo) / max(0.001, hi - lo), 0.0, 1.0)
    ms = 1.0 if factor <= 1.0 else 1.0 + 0.1 * math.log(factor)
    return np.concatenate([inv * (ramp + (1.0 - ramp) / factor), [ms]]).astype(np.float32)


def qk_inputs(T, nh, nkv, seed=0):
    """Q fp16 [T, nh, 128], K fp16 [T, nkv, 128] ~ N(0, 1)"""
    return _normal(_rng(seed, 20), (T, nh, 128), 1.0, np.float16), _normal(_rng(seed, 21), (T, nkv, 128), 1.0, np.float16)


def swiglu_inputs(T, I, seed=0, dtype=np.float16):
    """gate, up ~ N(0, 1.5) [T, I]"""
    return _normal(_rng(seed, 30), (T, I), 1.5, dtype), _normal(_rng(seed, 31), (T, I), 1.5, dtype)


def q4k_table(vocab, N, seed=0):
    """uint8 [vocab, N / 256, 144]: bytes uniform in [0, 256), each block's d and dmin = fp16 |N(0, 1e-3)|"""
    g = _rng(seed, 40); nb = N // 256
    W = g.integers(0, 256, (vocab, nb, 144), dtype=np.uint8)
    dd = np.abs(_rng(seed, 41).standard_normal((vocab, nb, 2), dtype=np.float32) * np.float32(1e-3)).astype(np.float16)
    W[:, :, 0:4] = dd.view(np.uint8).reshape(vocab, nb, 4)
    return W


def token_ids(n, vocab, seed=0):
    return _rng(seed, 42).integers(0, vocab, n, dtype=np.int32)
