"""CPU oracle for the fused glue ops: TEST INFRASTRUCTURE, not product code.

ctypes front of oracle/cam_oracle.c (the C restatement of the reference's HIP glue kernels, one IEEE operation per
statement) plus the float64 references the reference's own tests use. Imported only by tests/, __graft_entry__.smoke() and
bench.py's CPU-baseline legs; the package caminus_b200 never imports it.

Every function takes and returns numpy arrays. Row-parallel work is split over host threads here (ctypes releases the GIL
for the duration of a call; the C side is single-threaded); `threads=1` gives the scalar port.
"""
import ctypes
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_DIR, 'libcam_oracle.so')
_lib = None


def build(force=False):
    """compile cam_oracle.c with the Makefile beside it (gcc only)"""
    src = os.path.join(_DIR, 'cam_oracle.c')
    if force or not os.path.isfile(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(['make', '-C', _DIR, '-B'], check=True, stdout=subprocess.DEVNULL)
    return _SO


def _has_fma():
    try:
        return ' fma ' in open('/proc/cpuinfo').read()
    except OSError:
        return True


def lib():
    global _lib
    if _lib is None:
        build()
        if not _has_fma():   # a library built for x86-64-v3 would trap here: rebuild without -march
            subprocess.run(['gcc', '-O2', '-fPIC', '-shared', '-ffp-contract=off', '-fno-fast-math', '-std=gnu11', '-o', _SO,
                            os.path.join(_DIR, 'cam_oracle.c'), '-lm'], check=True)
        L = ctypes.CDLL(_SO)
        L.orc_expf.restype = ctypes.c_float; L.orc_expf.argtypes = [ctypes.c_float]
        L.orc_silu.restype = ctypes.c_float; L.orc_silu.argtypes = [ctypes.c_float]
        L.orc_rsqrt.restype = ctypes.c_float; L.orc_rsqrt.argtypes = [ctypes.c_float]
        L.orc_powi.restype = ctypes.c_float; L.orc_powi.argtypes = [ctypes.c_float, ctypes.c_int]
        L.orc_sincos.restype = None
        L.orc_sincos.argtypes = [ctypes.c_float, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float)]
        _lib = L
    return _lib


def default_threads():
    return len(os.sched_getaffinity(0)) if hasattr(os, 'sched_getaffinity') else (os.cpu_count() or 1)


P, I, L_, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float


def _p(a, off=0):
    return P(0) if a is None else P(a.ctypes.data + off)


def _chunks(n, threads):
    threads = max(1, min(int(threads), n))
    edges = [n * i // threads for i in range(threads + 1)]
    return [(a, b) for a, b in zip(edges[:-1], edges[1:]) if b > a]


def _run(n, threads, fn):
    """fn(a, b) on row ranges [a, b) covering [0, n)"""
    ch = _chunks(n, threads)
    if len(ch) <= 1:
        for a, b in ch: fn(a, b)
        return
    with ThreadPoolExecutor(len(ch)) as ex:
        list(ex.map(lambda ab: fn(*ab), ch))


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


# ---- scalar sequences -------------------------------------------------------------------------------------------------
def expf(a): return float(lib().orc_expf(F(float(a))))
def silu(x): return float(lib().orc_silu(F(float(x))))
def rsqrt(v): return float(lib().orc_rsqrt(F(float(v))))
def powi(b, e): return float(lib().orc_powi(F(float(b)), I(int(e))))


def sincos(theta):
    s, c = F(), F()
    lib().orc_sincos(F(float(theta)), ctypes.byref(s), ctypes.byref(c))
    return s.value, c.value


# ---- ops --------------------------------------------------------------------------------------------------------------
def q4k_get_rows(W, rb, vocab, toks, N, threads=None):
    """W: uint8 table (vocab rows of rb bytes of Q4_K blocks); toks int32 [n] -> float32 [n, N]"""
    W = _c(W, np.uint8).reshape(-1); toks = _c(toks, np.int32).reshape(-1); n = toks.size
    x = np.empty((n, N), np.float32)
    f = lib().orc_q4k_get_rows
    _run(n, threads or default_threads(),
         lambda a, b: f(_p(W), I(rb), I(vocab), _p(toks, 4 * a), _p(x, 4 * a * N), I(b - a), I(N)))
    return x


def add_rms16(x, nw, eps, d=None, w=None, S=0, want_h=True, threads=None):
    """q3p_add_rms16: returns (x updated, h or None, h16 as float16)"""
    x = _c(x, np.float32).copy(); n, N = x.shape
    d = None if d is None else _c(d, np.float32); w = None if w is None else _c(w, np.float32); nw = _c(nw, np.float32)
    h = np.empty((n, N), np.float32) if want_h else None; h16 = np.empty((n, N), np.uint16)
    f = lib().orc_add_rms16
    _run(n, threads or default_threads(),
         lambda a, b: f(_p(x, 4 * a * N), _p(d, 4 * a * S * N), _p(w, 4 * a * S), I(S), _p(nw), F(eps), _p(h, 4 * a * N),
                        _p(h16, 2 * a * N), I(b - a), I(N)))
    return x, h, h16.view(np.float16)


def add_rms16_q35(x, nw, eps, d=None, threads=None):
    x = _c(x, np.float32).copy(); n, N = x.shape
    d = None if d is None else _c(d, np.float32); nw = _c(nw, np.float32)
    h = np.empty((n, N), np.float32); h16 = np.empty((n, N), np.uint16)
    f = lib().orc_add_rms16_q35
    _run(n, threads or default_threads(),
         lambda a, b: f(_p(x, 4 * a * N), _p(d, 4 * a * N), _p(nw), F(eps), _p(h, 4 * a * N), _p(h16, 2 * a * N), I(b - a), I(N)))
    return x, h, h16.view(np.float16)


def add_rms_f16(x16, nw, eps, d16=None, threads=None):
    """fp16-storage form: returns (x updated float16, h16 float16)"""
    x = _c(x16, np.float16).copy(); n, N = x.shape
    d = None if d16 is None else _c(d16, np.float16); nw = _c(nw, np.float32)
    h16 = np.empty((n, N), np.uint16)
    f = lib().orc_add_rms_f16
    _run(n, threads or default_threads(),
         lambda a, b: f(_p(x, 2 * a * N), _p(d, 2 * a * N), _p(nw), F(eps), _p(h16, 2 * a * N), I(b - a), I(N)))
    return x, h16.view(np.float16)


def rms_partial_f16(x16, d16=None, threads=None):
    x = _c(x16, np.float16); n, Ns = x.shape
    d = None if d16 is None else _c(d16, np.float16)
    ss = np.empty(n, np.float32)
    f = lib().orc_rms_partial_f16
    _run(n, threads or default_threads(), lambda a, b: f(_p(x, 2 * a * Ns), _p(d, 2 * a * Ns), _p(ss, 4 * a), I(b - a), I(Ns)))
    return ss


def rms_apply_f16(x16, tot, nw, eps, Nfull, d16=None, threads=None):
    x = _c(x16, np.float16).copy(); n, Ns = x.shape
    d = None if d16 is None else _c(d16, np.float16); nw = _c(nw, np.float32); tot = _c(tot, np.float32)
    h16 = np.empty((n, Ns), np.uint16)
    f = lib().orc_rms_apply_f16
    _run(n, threads or default_threads(),
         lambda a, b: f(_p(x, 2 * a * Ns), _p(d, 2 * a * Ns), _p(tot, 4 * a), _p(nw), F(eps), _p(h16, 2 * a * Ns), I(b - a),
                        I(Ns), I(Nfull)))
    return x, h16.view(np.float16)


def swiglu16(g, u, threads=None):
    g = _c(g, np.float32).reshape(-1); u = _c(u, np.float32).reshape(-1); n = g.size
    y = np.empty(n, np.uint16); f = lib().orc_swiglu16
    _run(n, threads or default_threads(), lambda a, b: f(_p(g, 4 * a), _p(u, 4 * a), _p(y, 2 * a), L_(b - a)))
    return y.view(np.float16)


def silu_mul(g, u, threads=None):
    g = _c(g, np.float32).reshape(-1); u = _c(u, np.float32).reshape(-1); n = g.size
    h = np.empty(n, np.float32); f = lib().orc_silu_mul
    _run(n, threads or default_threads(), lambda a, b: f(_p(g, 4 * a), _p(u, 4 * a), _p(h, 4 * a), L_(b - a)))
    return h


def _blocks(n, threads, fn):
    """split n values at multiples of 32"""
    nb = (n + 31) // 32
    _run(nb, threads, lambda a, b: fn(a * 32, min(b * 32, n)))


def q8_1(x, sum_order=0, threads=None):
    """gg_quantize_q8_1: float32 [n] -> uint8 [ceil(n / 32) * 36]"""
    x = _c(x, np.float32).reshape(-1); n = x.size
    y = np.empty((n + 31) // 32 * 36, np.uint8); f = lib().orc_q8_1
    _blocks(n, threads or default_threads(), lambda a, b: f(_p(x, 4 * a), _p(y, a // 32 * 36), L_(b - a), I(sum_order)))
    return y


def swiglu_q8_1(g, u, sum_order=0, threads=None):
    """silu(g) * u quantised to Q8_1; g, u both float32 or both float16"""
    f16 = g.dtype == np.float16
    dt, es = (np.float16, 2) if f16 else (np.float32, 4)
    g = _c(g, dt).reshape(-1); u = _c(u, dt).reshape(-1); n = g.size
    y = np.empty((n + 31) // 32 * 36, np.uint8)
    f = lib().orc_swiglu_q8_1_f16 if f16 else lib().orc_swiglu_q8_1
    _blocks(n, threads or default_threads(),
            lambda a, b: f(_p(g, es * a), _p(u, es * a), _p(y, a // 32 * 36), L_(b - a), I(sum_order)))
    return y


def silu_scale_q8_1(x, rs, sum_order=0):
    """silu(x * rs) quantised to Q8_1 (the tape op OP_GG_Q8_1 with work = 1, kernels/k3_gguf_ops.h:70): uint8 [ceil(n / 32) * 36]"""
    x = _c(x, np.float32).reshape(-1); n = x.size
    y = np.empty((n + 31) // 32 * 36, np.uint8)
    lib().orc_silu_scale_q8_1(_p(x), F(rs), _p(y), L_(n), I(sum_order))
    return y


def swiglu_f32_from_f16(g, u, threads=None):
    g = _c(g, np.float16).reshape(-1); u = _c(u, np.float16).reshape(-1); n = g.size
    h = np.empty(n, np.float32); f = lib().orc_swiglu_f32_from_f16
    _run(n, threads or default_threads(), lambda a, b: f(_p(g, 2 * a), _p(u, 2 * a), _p(h, 4 * a), L_(b - a)))
    return h


def qk_rope(qkv, ldq, nh, nkv, par, pos0, cache, n, yarn=False, sum_order=0, threads=None):
    """q3p_qk_rope: qkv float32 [n * ldq]; cache float16 (flat; rows of 2 nkv 128) is copied and updated.
    sum_order 0: the reference's order of the head's sum of squares; 1: the CUDA kernel's (see cam_oracle.c).
    Returns (q16 float16 [n, nh, 128], cache)"""
    qkv = _c(qkv, np.float32).reshape(-1); par = _c(par, np.float32); cache = _c(cache, np.float16).reshape(-1).copy()
    q16 = np.empty((n, nh, 128), np.uint16); f = lib().orc_qk_rope
    _run(n, threads or default_threads(),
         lambda a, b: f(_p(qkv, 4 * a * ldq), I(ldq), I(nh), I(nkv), _p(par), I(pos0 + a), _p(q16, 2 * a * nh * 128), _p(cache),
                        I(b - a), I(int(yarn)), I(int(sum_order))))
    return q16.view(np.float16), cache


def qk_rope_f16(q, k, par, pos0, yarn=False, sum_order=0, threads=None):
    """fp16 q [n, nh, 128], k [n, nkv, 128] -> (q out, k out) float16"""
    q = _c(q, np.float16); k = _c(k, np.float16); par = _c(par, np.float32)
    n, nh, _ = q.shape; nkv = k.shape[1]
    qo = np.empty(q.shape, np.uint16); ko = np.empty(k.shape, np.uint16); f = lib().orc_qk_rope_f16
    _run(n, threads or default_threads(),
         lambda a, b: f(_p(q, 2 * a * nh * 128), _p(k, 2 * a * nkv * 128), I(nh), I(nkv), _p(par), I(pos0 + a),
                        _p(qo, 2 * a * nh * 128), _p(ko, 2 * a * nkv * 128), I(b - a), I(int(yarn)), I(int(sum_order))))
    return qo.view(np.float16), ko.view(np.float16)


# ---- float64 references, as the reference's tests state them ----------------------------------------------------------------
def rms_f64(x, nw, eps):
    """tests/prefill/test_q3m_ops.py:160-161: x / sqrt(mean(x^2) + eps) * nw in float64"""
    x = np.asarray(x, np.float64)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * np.asarray(nw, np.float64)


def norm_rope_f64(x, w, theta, eps, mscale=1.0):
    """tests/engine/test_q3m_yarn_rope.py:102-108: float64 norm + NeoX RoPE of rows x [..., 128] with the angles theta [64]
    (the caller passes the kernel's fp32 angles, or float64 ones for the looser test_q3m_ops.py:204-208 form)"""
    x = np.asarray(x, np.float64)
    y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * np.asarray(w, np.float64)
    th = np.asarray(theta, np.float64)
    c, s = np.cos(th) * mscale, np.sin(th) * mscale
    return np.concatenate([y[..., :64] * c - y[..., 64:] * s, y[..., 64:] * c + y[..., :64] * s], -1)


def q8_split(q8):
    """tests/engine/golden_util.py:92-98: Q8_1 bytes -> (d float16 [nb], s float16 [nb], qs int8 [nb, 32])"""
    b = np.asarray(q8, np.uint8).reshape(-1, 36)
    return (b[:, 0:2].copy().view(np.float16).reshape(-1), b[:, 2:4].copy().view(np.float16).reshape(-1),
            b[:, 4:].copy().view(np.int8))


# ---- the hyper-connection line and the training line's forwards (single-threaded calls; small test sizes) -----------------------
def _f32(a): return None if a is None else _c(a, np.float32)


def pf_rms_mul(x, w, eps, K, want=('y', 'ybf', 'scl')):
    """returns (y float32 [R, K] or None, ybf uint16 or None, scl float32 [R] or None)"""
    x = _f32(x).reshape(-1, K); w = _f32(w).reshape(-1, K); R, wr = x.shape[0], w.shape[0]
    y = np.empty((R, K), np.float32) if 'y' in want else None
    ybf = np.empty((R, K), np.uint16) if 'ybf' in want else None
    scl = np.empty(R, np.float32) if 'scl' in want else None
    lib().orc_pf_rms_mul(_p(x), _p(w), _p(y), _p(ybf), _p(scl), I(R), I(wr), F(eps), I(K))
    return y, ybf, scl


def pf_hc_post_rms(b, inj, res, w, T, HC, rs, eps, N):
    """returns (res updated, xn float32, xnbf uint16, scl)"""
    b = _f32(b); inj = _f32(inj); res = _f32(res).copy(); w = _f32(w)
    xn = np.empty((T * HC, N), np.float32); xnbf = np.empty((T * HC, N), np.uint16); scl = np.empty(T * HC, np.float32)
    lib().orc_pf_hc_post_rms(_p(b), _p(inj), _p(res), _p(w), _p(xn), _p(xnbf), _p(scl), I(T), I(HC), F(rs), F(eps), I(N))
    return res, xn, xnbf, scl


def pf_hc_post(b, inj, res, T, HC, D, rs):
    b = _f32(b); inj = _f32(inj); res = _f32(res).copy()
    lib().orc_pf_hc_post(_p(b), _p(inj), _p(res), I(T), I(HC), I(D), F(rs))
    return res


def pf_hc_mean(x, g, T, HC, D, rs, scl=None, w=None):
    x = _f32(x); g = _f32(g); scl = _f32(scl); w = _f32(w); out = np.empty((T, D), np.float32)
    lib().orc_pf_hc_mean(_p(x), _p(scl), _p(w), _p(g), _p(out), I(T), I(HC), I(D), F(rs))
    return out


def pf_add_sum(a, b, y):
    a = _f32(a).reshape(-1); b = _f32(b).reshape(-1); y = _f32(y).reshape(-1).copy()
    lib().orc_pf_add_sum(_p(a), _p(b), _p(y), L_(y.size))
    return y


def pf_swiglu(g, u):
    g = _f32(g).reshape(-1); u = _f32(u).reshape(-1); y = np.empty(g.size, np.float32)
    lib().orc_pf_swiglu(_p(g), _p(u), _p(y), L_(g.size))
    return y


def pf_to_bf16(x, ldx, T, Tpad, K, rs=None):
    """rs None: pf_to_bf16; else pf_silu_bf16. Returns uint16 [Tpad, K]"""
    x = _f32(x).reshape(-1); y = np.empty((Tpad, K), np.uint16)
    if rs is None: lib().orc_pf_to_bf16(_p(x), I(ldx), _p(y), I(T), I(Tpad), I(K))
    else: lib().orc_pf_silu_bf16(_p(x), I(ldx), _p(y), I(T), I(Tpad), I(K), F(rs))
    return y


def embedding_f32(tok, emb):
    tok = _c(tok, np.int32); emb = _f32(emb); D = emb.shape[1]; out = np.empty((tok.size, D), np.float32)
    lib().orc_embedding_f32(_p(tok), _p(emb), _p(out), I(D), I(tok.size))
    return out


def rmsnorm_f32(x, w, eps):
    x = _f32(x); w = _f32(w); R, D = x.shape; out = np.empty((R, D), np.float32)
    lib().orc_rmsnorm_f32(_p(x), _p(w), _p(out), I(D), F(eps), I(R))
    return out


def silu_mul_bf16(gu, H):
    gu = _c(gu, np.uint16); n = gu.size // 2; act = np.empty(n, np.uint16)
    lib().orc_silu_mul_bf16(_p(gu), _p(act), I(H), L_(n))
    return act


def residual3(x, m, y):
    x = _f32(x).reshape(-1); m = _c(m, np.uint16).reshape(-1); y = _c(y, np.uint16).reshape(-1); out = np.empty(x.size, np.float32)
    lib().orc_residual3(_p(x), _p(m), _p(y), _p(out), L_(x.size))
    return out


def cast_bf16(x):
    x = _f32(x).reshape(-1); out = np.empty(x.size, np.uint16)
    lib().orc_cast_bf16(_p(x), _p(out), L_(x.size))
    return out


def residual_slices_fwd(x, m, mlp, ys, pos, d):
    x = _f32(x).reshape(-1); m = _c(m, np.uint16).reshape(-1); mlp = _c(mlp, np.uint16).reshape(-1)
    ys = None if ys is None else _c(ys, np.uint16); pos = None if pos is None else _c(pos, np.int32)
    out = np.empty(x.size, np.float32)
    lib().orc_residual_slices_fwd(_p(x), _p(m), _p(mlp), _p(ys), _p(pos), _p(out), I(d), L_(x.size // 4))
    return out


def pf_qk_nr(xin, head_stride, heads, w, D, nrot, theta_scale, eps, pos0, nblocks):
    xin = _f32(xin).reshape(-1); w = _f32(w); out = np.empty((nblocks, D), np.float32)
    lib().orc_pf_qk_nr(_p(xin), I(head_stride), I(heads), _p(w), I(D), I(nrot), F(theta_scale), F(eps), I(pos0), _p(out), I(nblocks))
    return out


def mmq_q8_1(x, kvalid, Kpad, layout, u=None):
    """Q8_1 in the MMQ layout of rows x [rows, ld] (float32, or float16 with u: SwiGLU): uint8 [Kpad / 128, rows, 144].
    u given: the values are silu(x) * u."""
    rows, ld = x.shape; y = np.empty((Kpad // 128, rows, 144), np.uint8)
    if x.dtype == np.float16:
        x = _c(x, np.float16); u = _c(u, np.float16)
        lib().orc_mmq_q8_1_f16(_p(x), _p(u), _p(y), I(kvalid), I(Kpad), L_(ld), I(rows), I(layout))
    else:
        x = _f32(x); u = _f32(u)
        lib().orc_mmq_q8_1(_p(x), _p(u), _p(y), I(kvalid), I(Kpad), L_(ld), I(rows), I(layout), I(0 if u is None else 1))
    return y


def qk_rope_q8(qkv, ldq, nh, nkv, par, pos0, cache, n, yarn=False, sum_order=0):
    """q3p_qk_rope_q8: cache uint8 (flat; rows of 2 (nkv 128 / 32) 34 bytes) is copied and updated.
    Returns (q16 float16 [n, nh, 128], cache, err)"""
    qkv = _f32(qkv).reshape(-1); par = _f32(par); cache = _c(cache, np.uint8).reshape(-1).copy()
    q16 = np.empty((n, nh, 128), np.uint16); err = np.zeros(1, np.int32)
    lib().orc_qk_rope_q8(_p(qkv), I(ldq), I(nh), I(nkv), _p(par), I(pos0), _p(q16), _p(cache), _p(err), I(n), I(int(yarn)), I(int(sum_order)))
    return q16.view(np.float16), cache, int(err[0])


def hadamard128(x):
    y = _f32(x).copy().reshape(-1, 128)
    lib().orc_hadamard128(_p(y), I(y.shape[0]))
    return y.reshape(np.shape(x))


def q8_kv_rows(k, v):
    """K, V float32 [rows, nkv, 128] -> (uint8 [rows, 2 (nkv 128 / 32) 34], refused blocks)"""
    k = _f32(k); v = _f32(v); rows, nkv, _ = k.shape
    out = np.zeros((rows, 2 * (nkv * 128 // 32) * 34), np.uint8)
    lib().orc_q8_kv_rows.restype = ctypes.c_int
    bad = lib().orc_q8_kv_rows(_p(k), _p(v), _p(out), I(rows), I(nkv))
    return out, int(bad)


def actq_fwd(x, clip, qmax):
    """x [M, K] float32, or uint16 (bf16 bits) -> (y uint16 [M, K], s float32 [M], codes uint16 [M, K / 4])"""
    is_bf = x.dtype == np.uint16; x = _c(x, np.uint16 if is_bf else np.float32); M, K = x.shape
    y = np.empty((M, K), np.uint16); s = np.empty(M, np.float32); codes = np.empty((M, K // 4), np.uint16)
    lib().orc_actq_fwd(_p(x), I(int(is_bf)), _p(y), _p(s), _p(codes), I(M), I(K), F(clip), I(qmax))
    return y, s, codes


def silu_mul_actq_fwd(gu, Fw, clip, qmax):
    gu = _c(gu, np.uint16); M, ld = gu.shape
    y = np.empty((M, Fw), np.uint16); s = np.empty(M, np.float32); codes = np.empty((M, Fw // 4), np.uint16)
    lib().orc_silu_mul_actq_fwd(_p(gu), I(ld), I(Fw), _p(y), _p(s), _p(codes), I(M), F(clip), I(qmax))
    return y, s, codes


def block_entry_fwd(x, nw, wab, eps, clip, qmax):
    x = _f32(x); nw = _f32(nw); M, d = x.shape; nab = 0 if wab is None else wab.shape[0]
    wab = None if wab is None else _c(wab, np.uint16)
    y = np.empty((M, d), np.uint16); s = np.empty(M, np.float32); codes = np.empty((M, d // 4), np.uint16)
    ab = np.empty((M, nab), np.uint16); rstd = np.empty(M, np.float32)
    lib().orc_block_entry_fwd(_p(x), _p(nw), _p(wab), I(nab), F(eps), _p(y), _p(s), _p(codes), _p(ab), _p(rstd), I(M), I(d), F(clip), I(qmax))
    return y, s, codes, ab, rstd


def router(h, Wr):
    h = _f32(h); Wr = _f32(Wr); n, K = h.shape; E = Wr.shape[0]; out = np.empty((n, E), np.float32)
    lib().orc_router(_p(h), _p(Wr), I(E), I(K), _p(out), I(n))
    return out


def topk(logits, k, floor_):
    lg = _f32(logits); n, E = lg.shape
    ids = np.empty((n, k), np.int32); wts = np.empty((n, k), np.float32); err = np.zeros(1, np.int32)
    lib().orc_topk(_p(lg), I(E), I(k), F(floor_), _p(ids), _p(wts), _p(err), I(n))
    return ids, wts, int(err[0])


def pf_router(logits, k, clamp):
    """softmax + top-k of the hyper-connection line's router (kernels/prefill_glue.hip:242-308): ids [n, k], wts [n, k], the error word"""
    lg = _f32(logits); n, E = lg.shape
    ids = np.empty((n, k), np.int32); wts = np.empty((n, k), np.float32); err = np.zeros(1, np.int32)
    lib().orc_pf_router(_p(lg), I(E), I(k), F(clamp), _p(ids), _p(wts), _p(err), I(n))
    return ids, wts, int(err[0])


def group(ids, k, E):
    """the grouping of the (token, slot) pairs by expert (kernels/q3m_prefill.hip:490-513) with every expert's list in ascending pair
    order (the reference leaves the order inside a list to its atomics and states that it changes no bit downstream):
    xs, yd [npairs], items [nitems, 4] = (expert, first, count, 0) of at most 64 pairs, the error word (2: an id outside [0, E), which
    counts as expert 0)"""
    ids = _c(ids, np.int32).reshape(-1); bad = (ids < 0) | (ids >= E)
    e = np.where(bad, 0, ids)
    yd = np.argsort(e, kind='stable').astype(np.int32); xs = (yd // k).astype(np.int32)
    cnt = np.bincount(e, minlength=E); first = np.concatenate([[0], np.cumsum(cnt)[:-1]])
    items = [(x, int(first[x]) + 64 * j, min(64, int(cnt[x]) - 64 * j), 0) for x in range(E) for j in range(-(-int(cnt[x]) // 64))]
    return xs, yd, np.array(items, np.int32).reshape(-1, 4), 2 if bad.any() else 0


def embd_rows_iq4xs(table, tok, nvocab, nblk):
    table = _c(table, np.uint8).reshape(-1); tok = _c(tok, np.int32); out = np.empty((tok.size, nblk * 256), np.float32); err = np.zeros(1, np.int32)
    lib().orc_embd_rows_iq4xs(_p(table), _p(tok), I(nvocab), I(tok.size), I(nblk), _p(out), _p(err))
    return out, int(err[0])


def ple_rows_iq4nl(raw, inv, nuniq, bpr):
    raw = _c(raw, np.uint8).reshape(-1); inv = _c(inv, np.int32); out = np.empty((inv.size, bpr * 32), np.float32); err = np.zeros(1, np.int32)
    lib().orc_ple_rows_iq4nl(_p(raw), _p(inv), I(nuniq), I(inv.size), I(bpr), _p(out), _p(err))
    return out, int(err[0])


def pack_iq2s_grid(mags):
    """uint8 [1024, 8] magnitudes (8 / 25 / 43: the form of the reference's iq_tables.GRID_IQ2_S) -> uint32 [512], the packing of the
    reference's kernels/iq2s_grid.h (python/caminus/iq_tables.py:747-768): 2-bit codes 0 / 1 / 2 at bits 2 k, entry 2 w in word w's low half"""
    m = np.asarray(mags, np.uint8).reshape(1024, 8)
    code = np.where(m == 8, 0, np.where(m == 25, 1, 2)).astype(np.uint32)
    e = (code << (2 * np.arange(8, dtype=np.uint32))).sum(axis=1).astype(np.uint32)
    return (e[0::2] | (e[1::2] << 16)).astype(np.uint32)


def emb_rows_iq2s(W, rb, vocab, toks, N, grid):
    W = _c(W, np.uint8).reshape(-1); toks = _c(toks, np.int32); grid = _c(grid, np.uint32); x = np.empty((toks.size, N), np.float32)
    lib().orc_emb_rows_iq2s(_p(W), I(rb), I(vocab), _p(toks), _p(x), I(toks.size), I(N), _p(grid))
    return x


def emb_rows_q6k(W, rb, vocab, toks, N):
    W = _c(W, np.uint8).reshape(-1); toks = _c(toks, np.int32); x = np.empty((toks.size, N), np.float32)
    lib().orc_emb_rows_q6k(_p(W), I(rb), I(vocab), _p(toks), _p(x), I(toks.size), I(N))
    return x
