"""Generates the golden fixtures of tests/golden/ by running the REFERENCE's own CPU code on seeded inputs.

Run it where the reference checkout is present:   python tests/golden/make_golden.py /path/to/caminus
It imports, from that checkout: caminus.own_dequant (the bitwise host decoder of Q4_K the reference gates q3p_emb against),
the vendored gguf-py dequantizer (the decoder's own oracle), tests/engine/golden_util.q8_host and
tests/engine/test_gguf_mv.q8_1_numpy's arithmetic (the Q8_1 host quantisers its GPU quantiser is gated against),
caminus.rope.yarn_table, caminus.ref_q35.silu, and restates the float64 references of tests/prefill/test_q3m_ops.py and
tests/engine/test_q3m_yarn_rope.py. The outputs are stored as .npz next to this file; the test-suite reads only those.
"""
import os
import sys

import numpy as np

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get('CAMINUS_REFERENCE', '')
if not os.path.isdir(os.path.join(REF, 'python', 'caminus')): sys.exit('usage: python tests/golden/make_golden.py /path/to/caminus   (or CAMINUS_REFERENCE=...)')
sys.path.insert(0, os.path.join(REF, 'python'))
sys.path.insert(0, os.path.join(REF, 'python', 'caminus', '_vendor'))
sys.path.insert(0, os.path.join(REF, 'tests', 'engine'))
OUT = os.path.dirname(os.path.abspath(__file__))

from caminus import own_dequant, rope, ref_q35, ref_kv   # noqa: E402
import golden_util                                 # noqa: E402
from gguf import quants as gq                      # noqa: E402
from gguf.constants import GGMLQuantizationType as QT   # noqa: E402


def q4k_table(g, rows, blocks):
    """random Q4_K bytes with small finite fp16 d / dmin (as tests/io/test_own_dequant.py:13-25 draws them)"""
    W = g.integers(0, 256, (rows, blocks, 144), dtype=np.uint8)
    dd = np.abs(g.standard_normal((rows, blocks, 2)) * 1e-3).astype(np.float16)
    W[:, :, 0:4] = dd.view(np.uint8).reshape(rows, blocks, 4)
    return W


def make_q4k():
    g = np.random.default_rng(20261110)
    vocab, blocks = 61, 2
    W = q4k_table(g, vocab, blocks)
    W[5, 0, 0:4] = 0                                                  # d = dmin = 0
    W[6, 1, 0:2] = np.array([0x7bff], np.uint16).view(np.uint8)       # the largest finite fp16 scale
    W[7, 0, 4:16] = 255                                               # every 6-bit scale / min at 63
    toks = np.array([0, 1, 60, 59, 99999, -3, 200000, 5, 6, 7, 7, 30], np.int32)   # out-of-range ids as test_q3m_ops.py:148
    cl = np.clip(toks, 0, vocab - 1)
    want = np.stack([own_dequant.q4_k(W[t].reshape(-1)) for t in cl]).astype(np.float32)
    gg = np.stack([gq.dequantize(W[t].reshape(1, -1), QT.Q4_K).reshape(-1) for t in cl]).astype(np.float32)
    assert np.array_equal(want.view(np.uint32), gg.view(np.uint32)), 'own_dequant.q4_k != gguf-py'
    np.savez_compressed(os.path.join(OUT, 'q4k_rows.npz'), W=W, toks=toks, vocab=vocab, want=want)


def q8_1_numpy(x):
    """tests/engine/test_gguf_mv.py:18-25, restated: d = amax / 127, q = roundf(x / d) in float32"""
    xb = x.astype(np.float32).reshape(-1, 32)
    amax = np.abs(xb).max(1); d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide='ignore', invalid='ignore'):
        v = np.where(d[:, None] > 0, xb / d[:, None], 0).astype(np.float32)
    q = (np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))).astype(np.int8)
    return q, d.astype(np.float16)


def make_q8():
    g = np.random.default_rng(7)
    x = (g.standard_normal(64 * 32) * 0.5).astype(np.float32)
    x[0:32] = 0.0                                                     # an all-zero block
    x[32:64] = np.float32(1.0)                                        # every value the maximum
    x[64:96] = (np.arange(32, dtype=np.float32) - 16) * np.float32(0.5)   # exact .5 code boundaries: x / d = k + 0.5 ...
    x[64 + 31] = np.float32(127 * 0.5)                                # ... with d = 0.5 exactly (amax = 63.5)
    x[96:128] = np.array([30, -30, 0, -0.0, 1e-3, -88, 88, 3] * 4, np.float32)   # tests/train/test_silu_mul_actq.py:24
    x[128:160] *= np.float32(1e-30)                                   # a tiny block (d in fp16's subnormal range / zero)
    x[160:192] *= np.float32(1e4)                                     # a large one
    n_odd = 64 * 32 - 13                                              # a length that is not a multiple of 32
    d32, d16, v, q = golden_util.q8_host(x)
    q2, d2 = q8_1_numpy(x)
    assert np.array_equal(q, q2) and np.array_equal(d16.view(np.uint16), d2.view(np.uint16)), 'the two host quantisers differ'
    _, d16o, _, qo = golden_util.q8_host(x[:n_odd])
    np.savez_compressed(os.path.join(OUT, 'q8_1.npz'), x=x, d16=d16, q=q, n_odd=n_odd, d16_odd=d16o, q_odd=qo)


def make_swiglu():
    g = np.random.default_rng(11)
    n = 4096
    gate = (g.standard_normal(n) * 1.5).astype(np.float16); up = (g.standard_normal(n) * 1.5).astype(np.float16)
    gate[:8] = np.array([30, -30, 0, -0.0, 1e-3, -88, 88, 3], np.float16)
    g32, u32 = gate.astype(np.float32), up.astype(np.float32)
    h64 = ref_q35.silu(g32.astype(np.float64)) * u32.astype(np.float64)          # the reference's float64 silu
    with np.errstate(over='ignore'):
        h32 = (g32 / (np.float32(1.0) + np.exp(-g32)) * u32).astype(np.float32)   # the device statement in numpy float32
    _, d16, _, q = golden_util.q8_host(h32)
    # the wider test inputs of tests/prefill/test_q3m_ops.py:184-187 (gate x 4), fp32
    gg = (g.standard_normal(5000) * 4).astype(np.float32); uu = g.standard_normal(5000).astype(np.float32)
    sr = gg.astype(np.float64) / (1 + np.exp(-gg.astype(np.float64))) * uu
    np.savez_compressed(os.path.join(OUT, 'swiglu.npz'), gate=gate, up=up, h64=h64, h32=h32, d16=d16, q=q, gg=gg, uu=uu, sr=sr)


def make_rms():
    g = np.random.default_rng(3)
    n, S, D = 3, 8, 2048                                              # tests/prefill/test_q3m_ops.py:154-163 at fewer rows
    x0 = (g.standard_normal((n, D)) * 3).astype(np.float32); dd = g.standard_normal((n, S, D)).astype(np.float32)
    ww = g.random((n, S)).astype(np.float32); nw = (g.random(D) + 0.5).astype(np.float32)
    xr = x0.astype(np.float64) + np.einsum('ns,nsd->nd', ww.astype(np.float64), dd.astype(np.float64))
    hr = xr / np.sqrt((xr ** 2).mean(-1, keepdims=True) + 1e-6) * nw
    # the decode-token case of the benchmark: hidden 2048, T = 1, seed 0, one generator per tensor in the listed order
    x1 = np.random.default_rng(0).standard_normal((1, 2048)).astype(np.float32)
    r1 = np.random.default_rng(0).standard_normal((1, 2048)).astype(np.float32)
    w1 = (1 + 0.05 * np.random.default_rng(0).standard_normal(2048)).astype(np.float32)
    s1 = x1.astype(np.float64) + r1
    h1 = s1 / np.sqrt((s1 ** 2).mean(-1, keepdims=True) + 1e-6) * w1
    np.savez_compressed(os.path.join(OUT, 'add_rms.npz'), x0=x0, dd=dd, ww=ww, nw=nw, xr=xr, hr=hr, x1=x1, r1=r1, w1=w1, s1=s1, h1=h1)


def make_rope():
    g = np.random.default_rng(23)
    nh, nkv, hd = 4, 2, 128
    M = nkv * hd
    POS = (0, 1, 63, 64, 1000, 4095, 32767, 32768, 40960, 65536, 100000, 131071)   # test_q3m_yarn_rope.py:49 (+ 4095)
    eps = 1e-6
    theta_scale = np.float32(np.float32(1e6) ** np.float32(-2.0 / hd))              # test_q3m_ops.py:195
    qn = (0.5 + g.random(hd)).astype(np.float32); kn = (0.5 + g.random(hd)).astype(np.float32)
    tab = rope.yarn_table(hd, 1e6, 4.0, 32768)
    par = np.concatenate([qn, kn, np.array([theta_scale, eps], np.float32), tab]).astype(np.float32)
    qkv = (g.standard_normal((len(POS), nh * hd + 2 * M)) * 1.3).astype(np.float32)
    inv64 = np.float64(1e6) ** (-2.0 * np.arange(hd // 2) / hd)

    def nr(x, w, th, ms=1.0):   # float64 norm + NeoX RoPE (test_q3m_ops.py:204-208; test_q3m_yarn_rope.py:102-108)
        x = x.astype(np.float64); y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w.astype(np.float64)
        c, s = np.cos(th) * ms, np.sin(th) * ms
        return np.concatenate([y[..., :64] * c - y[..., 64:] * s, y[..., 64:] * c + y[..., :64] * s], -1)

    q_plain = np.stack([nr(qkv[i, :nh * hd].reshape(nh, hd), qn, p * inv64) for i, p in enumerate(POS)])
    k_plain = np.stack([nr(qkv[i, nh * hd:nh * hd + M].reshape(nkv, hd), kn, p * inv64) for i, p in enumerate(POS)])
    # the YaRN form on the kernel's fp32 angle (float32(pos) * table), the factor on cos and sin
    th32 = [(np.float32(p) * tab[:64]).astype(np.float64) for p in POS]
    q_yarn = np.stack([nr(qkv[i, :nh * hd].reshape(nh, hd), qn, th32[i], float(tab[64])) for i in range(len(POS))])
    k_yarn = np.stack([nr(qkv[i, nh * hd:nh * hd + M].reshape(nkv, hd), kn, th32[i], float(tab[64])) for i in range(len(POS))])
    np.savez_compressed(os.path.join(OUT, 'qk_rope.npz'), pos=np.array(POS, np.int64), nh=nh, nkv=nkv, par=par, qkv=qkv,
                        q_plain=q_plain, k_plain=k_plain, q_yarn=q_yarn, k_yarn=k_yarn, tab=tab)


def make_q8_kv():
    """the Q8_0 KV rows of fp16-valued K / V: encode_q8_kv(hadamard128(K), V) (python/caminus/ref_kv.py), the statement the
    reference gates its Q8 prefill rows with (tests/engine/test_q3m_yarn_rope.py:121-123)"""
    g = np.random.default_rng(31); rows, nkv = 9, 2
    K = (g.standard_normal((rows, nkv, 128)) * 0.8).astype(np.float16).astype(np.float32)
    V = (g.standard_normal((rows, nkv, 128)) * 0.5).astype(np.float16).astype(np.float32)
    K[0, 0, :32] = 0; V[1, 1, 32:64] = 0                         # all-zero blocks
    K[2, 0, 5] = 30.0; V[3, 0] *= np.float32(1e-3)               # an outlier; a small block
    H = ref_kv.hadamard128(K)
    raw = ref_kv.encode_q8_kv(H, V, ref_kv.Q8KVLayout(nkv, 128))
    np.savez_compressed(os.path.join(OUT, 'q8_kv.npz'), K=K, V=V, H=H, raw=raw)


def make_iq4():
    """IQ4_XS and IQ4_NL rows: own_dequant's decoders (bitwise gguf-py upstream, tests/io/test_own_dequant.py), small finite scales"""
    g = np.random.default_rng(20261110); vocab, nblk = 23, 2
    T = g.integers(0, 256, (vocab, nblk, 136), dtype=np.uint8)
    T[:, :, 0:2] = (g.standard_normal((vocab, nblk, 1)) * 1e-2).astype(np.float16).view(np.uint8).reshape(vocab, nblk, 2)
    xs = np.stack([own_dequant.iq4_xs(T[t].reshape(-1)) for t in range(vocab)]).astype(np.float32)
    assert np.array_equal(xs.view(np.uint32), np.stack([gq.dequantize(T[t].reshape(1, -1), QT.IQ4_XS).reshape(-1) for t in range(vocab)]).astype(np.float32).view(np.uint32))
    nuniq, bpr = 11, 5
    R = g.integers(0, 256, (nuniq, bpr, 18), dtype=np.uint8)
    R[:, :, 0:2] = (g.standard_normal((nuniq, bpr, 1)) * 1e-2).astype(np.float16).view(np.uint8).reshape(nuniq, bpr, 2)
    nl = np.stack([gq.dequantize(R[u].reshape(1, -1), QT.IQ4_NL).reshape(-1) for u in range(nuniq)]).astype(np.float32)
    np.savez_compressed(os.path.join(OUT, 'iq4_rows.npz'), T=T, xs=xs, R=R, nl=nl)


def make_q6k():
    """Q6_K rows: own_dequant.q6_k (python/caminus/own_dequant.py:40-53), bitwise the vendored gguf-py dequantiser; small finite scales"""
    g = np.random.default_rng(20261125); vocab, nblk = 19, 3
    T = g.integers(0, 256, (vocab, nblk, 210), dtype=np.uint8)
    T[:, :, 208:210] = (g.standard_normal((vocab, nblk, 1)) * 1e-3).astype(np.float16).view(np.uint8).reshape(vocab, nblk, 2)
    rows = np.stack([own_dequant.q6_k(T[t].reshape(-1)) for t in range(vocab)]).astype(np.float32)
    assert np.array_equal(rows.view(np.uint32), np.stack([gq.dequantize(T[t].reshape(1, -1), QT.Q6_K).reshape(-1) for t in range(vocab)]).astype(np.float32).view(np.uint32))
    np.savez_compressed(os.path.join(OUT, 'q6k_rows.npz'), T=T, rows=rows)


def make_iq2s():
    """IQ2_S rows: own_dequant.iq2_s (python/caminus/own_dequant.py:128-137), the decoder the reference gates q35t_emb_iq2s against.
    The 1024-entry grid is ggml's data and is not carried by this repository: for the stored fixture the decoder runs over a seeded
    stand-in grid (magnitudes drawn from 8 / 25 / 43, as the real entries are), which pins every statement of the decoder (index
    assembly, scales, signs, the order of the float32 products). With the checkout present this function also checks, without storing
    anything, that the oracle over the reference's real grid equals the decoder and gguf-py on the same bytes."""
    from caminus import iq_tables
    sys.path.insert(0, os.path.join(OUT, '..', '..'))
    import oracle
    g = np.random.default_rng(20261126); vocab, nblk = 23, 3
    T = g.integers(0, 256, (vocab, nblk, 82), dtype=np.uint8)
    T[:, :, 0:2] = (g.standard_normal((vocab, nblk, 1)) * 1e-2).astype(np.float16).view(np.uint8).reshape(vocab, nblk, 2)
    T[3, 0, 0:2] = 0; T[4, 1, 0:2] = np.array([0x8000], np.uint16).view(np.uint8); T[5, 2, 0:2] = np.array([0x7bff], np.uint16).view(np.uint8)
    real = iq_tables.GRID_IQ2_S
    toks = np.arange(vocab, dtype=np.int32)
    rows_real = np.stack([own_dequant.iq2_s(T[t].reshape(-1)) for t in range(vocab)]).astype(np.float32)
    assert np.array_equal(rows_real.view(np.uint32), np.stack([gq.dequantize(T[t].reshape(1, -1), QT.IQ2_S).reshape(-1) for t in range(vocab)]).astype(np.float32).view(np.uint32))
    assert np.array_equal(rows_real.view(np.uint32), oracle.emb_rows_iq2s(T, nblk * 82, vocab, toks, nblk * 256, oracle.pack_iq2s_grid(real)).view(np.uint32))
    grid = np.array([8, 25, 43], np.uint8)[g.integers(0, 3, (1024, 8))]
    iq_tables.GRID_IQ2_S = grid
    try:
        rows = np.stack([own_dequant.iq2_s(T[t].reshape(-1)) for t in range(vocab)]).astype(np.float32)
    finally:
        iq_tables.GRID_IQ2_S = real
    np.savez_compressed(os.path.join(OUT, 'iq2s_rows.npz'), T=T, rows=rows, grid=grid)


if __name__ == '__main__':
    make_iq2s(); make_q6k(); make_iq4(); make_q4k(); make_q8(); make_swiglu(); make_rms(); make_rope(); make_q8_kv()
    for f in sorted(os.listdir(OUT)):
        if f.endswith('.npz'): print(f, os.path.getsize(os.path.join(OUT, f)), 'bytes')
