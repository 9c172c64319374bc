"""Pins the CPU oracle (oracle/cam_oracle.c) to the reference's own CPU code, through the fixtures that
tests/golden/make_golden.py produced by running that code: own_dequant.q4_k (bitwise), the q8_host / q8_1_numpy host
quantisers (bitwise d and codes), the float64 norm, SwiGLU and norm + RoPE references with the reference's own bounds."""
import numpy as np

import oracle


def ulp16(v):
    return np.abs(np.spacing(np.abs(v).astype(np.float16))).astype(np.float64)


def test_q4k_rows_bitwise(golden):
    f = golden('q4k_rows')
    W = f['W']; vocab = int(f['vocab']); rb = W.shape[1] * 144; N = W.shape[1] * 256
    got = oracle.q4k_get_rows(W, rb, vocab, f['toks'], N)
    assert np.array_equal(got.view(np.uint32), f['want'].view(np.uint32))       # tests/prefill/test_q3m_ops.py:147-152
    assert np.array_equal(oracle.q4k_get_rows(W, rb, vocab, f['toks'], N, threads=1).view(np.uint32), got.view(np.uint32))


def test_q8_1_codes_and_scales_bitwise(golden):
    f = golden('q8_1')
    for order in (0, 1):
        d, s, q = oracle.q8_split(oracle.q8_1(f['x'], sum_order=order))
        assert np.array_equal(q, f['q']) and np.array_equal(d.view(np.uint16), f['d16'].view(np.uint16))   # 0 mismatches
    n = int(f['n_odd'])
    d, s, q = oracle.q8_split(oracle.q8_1(f['x'][:n]))
    assert np.array_equal(q, f['q_odd']) and np.array_equal(d.view(np.uint16), f['d16_odd'].view(np.uint16))
    # the block sum: fp16 of the fp32 sum, both orders within one fp16 ulp of the float64 sum (reported, not gated, upstream)
    x = f['x'].astype(np.float64).reshape(-1, 32)
    for order in (0, 1):
        _, s, _ = oracle.q8_split(oracle.q8_1(f['x'], sum_order=order))
        ref = x.sum(1)
        assert (np.abs(s.astype(np.float64) - ref) <= ulp16(ref) + 32 * 2.0 ** -24 * np.abs(x).sum(1)).all()


def test_silu_extremes_and_accuracy():
    # the explicit exp sequence against float64: silu within 3 fp32 ulp over the range fp16 inputs reach
    g = np.concatenate([np.linspace(-90, 90, 200001), [30, -30, 0, -0.0, 1e-3, -88, 88, 3, 65504, -65504]]).astype(np.float32)
    got = oracle.silu_mul(g, np.ones_like(g)).astype(np.float64)
    ref = g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64)))
    err = np.abs(got - ref)
    tiny = np.abs(ref) < 1e-30          # g below -87: exp is clamped; the value is ~1e-36 either way
    assert (err[~tiny] <= 3 * np.spacing(np.abs(ref[~tiny]).astype(np.float32))).all()
    assert (np.abs(got[tiny]) < 1e-30).all()
    e = np.array([oracle.expf(a) for a in np.linspace(-87, 88, 5001)])
    r = np.exp(np.linspace(-87, 88, 5001).astype(np.float32).astype(np.float64))
    assert (np.abs(e / r - 1) < 2 ** -23).all()


def test_swiglu_q8_against_reference_host_path(golden):
    """The reference's rule for a chain crossing a Q8_1 quantisation (tests/engine/golden_util.py:132-173): the float is
    within 1e-6 of max; d differs by at most one half-ulp; codes differ by at most 1 and only where the two x / d values
    straddle the .5 boundary."""
    f = golden('swiglu')
    gate, up = f['gate'], f['up']
    h = oracle.swiglu_f32_from_f16(gate, up)
    h64, h32 = f['h64'], f['h32']
    assert np.abs(h - h64).max() <= 1e-6 * np.abs(h64).max()
    assert np.abs(h.astype(np.float64) - h32).max() <= 1e-6 * np.abs(h32).max()
    for order in (0, 1):
        d, s, q = oracle.q8_split(oracle.swiglu_q8_1(gate, up, sum_order=order))
        # exact: our bytes are the host quantiser's of our float
        d2, _, q2 = oracle.q8_split(oracle.q8_1(h))
        assert np.array_equal(d.view(np.uint16), d2.view(np.uint16)) and np.array_equal(q, q2)
        dr, qr = f['d16'], f['q']
        assert np.abs(d.view(np.int16).astype(np.int32) - dr.view(np.int16).astype(np.int32)).max() <= 1
        dq = q.astype(np.int32) - qr.astype(np.int32); diff = dq != 0
        assert np.abs(dq).max() <= 1
        if diff.any():
            def v_of(x):
                xb = x.reshape(-1, 32); dd = (np.abs(xb).max(1) / np.float32(127)).astype(np.float32)
                return np.where(dd[:, None] > 0, xb / np.where(dd > 0, dd, 1)[:, None], 0).astype(np.float64)
            a, b = v_of(h)[diff], v_of(h32)[diff]
            bnd = np.minimum(q, qr)[diff].astype(np.float64) + 0.5
            assert ((np.minimum(a, b) <= bnd) & (bnd <= np.maximum(a, b))).all()
        assert diff.mean() < 1e-3
    # unfused fp16 form: within fp16 rounding of float64 (tests/prefill/test_q3m_ops.py:184-187)
    y = oracle.swiglu16(f['gg'], f['uu']).astype(np.float64)
    assert np.abs(y - f['sr']).max() <= np.abs(f['sr']).max() * 2.0 ** -10


def test_add_rms_against_float64(golden):
    f = golden('add_rms')
    rel = lambda a, b: float(np.abs(a - b).max() / np.sqrt((np.asarray(b, np.float64) ** 2).mean()))
    x, h, h16 = oracle.add_rms16(f['x0'], f['nw'], 1e-6, d=f['dd'], w=f['ww'], S=8)
    assert rel(x, f['xr']) < 1e-6 and rel(h, f['hr']) < 2e-6 and rel(h16.astype(np.float64), f['hr']) < 2e-3   # test_q3m_ops.py:162
    # the decode-token case: one added row, the q3p (S = 1, no weights) and q35p forms agree bit for bit here
    x1, h1, h116 = oracle.add_rms16(f['x1'], f['w1'], 1e-6, d=f['r1'].reshape(1, 1, -1), S=1)
    x2, h2, h216 = oracle.add_rms16_q35(f['x1'], f['w1'], 1e-6, d=f['r1'])
    assert np.abs(h1 - f['h1']).max() <= 1e-5 * np.abs(f['h1']).max() and np.array_equal(x1, f['s1'].astype(np.float32))
    assert np.array_equal(h1.view(np.uint32), h2.view(np.uint32)) and np.array_equal(h116.view(np.uint16), h216.view(np.uint16))
    # no addend: x untouched
    x3, h3, _ = oracle.add_rms16(f['x1'], f['w1'], 1e-6)
    assert np.array_equal(x3, f['x1'])
    # fp16 storage form within 2 fp16 ulp of float64 on the same fp16 inputs
    a16, d16 = f['x1'].astype(np.float16), f['r1'].astype(np.float16)
    xo, ho = oracle.add_rms_f16(a16, f['w1'], 1e-6, d16)
    s = a16.astype(np.float64) + d16.astype(np.float64)
    ref = oracle.rms_f64(s, f['w1'], 1e-6)
    assert (np.abs(ho.astype(np.float64) - ref) <= 2 * ulp16(ref) + 1e-5 * np.abs(ref).max()).all()
    assert np.array_equal(xo.view(np.uint16), s.astype(np.float32).astype(np.float16).view(np.uint16))


def test_qk_rope_against_float64(golden):
    """fp32 qkv entry at positions whose cache rows fit in memory, against the fixture's float64 rows; the fp16 entry at
    every position of tests/engine/test_q3m_yarn_rope.py:49 against float64 on the same fp16-rounded inputs."""
    f = golden('qk_rope')
    pos, nh, nkv, par, qkv, tab = f['pos'], int(f['nh']), int(f['nkv']), f['par'], f['qkv'], f['tab']
    M = nkv * 128; ldq = nh * 128 + 2 * M
    inv64 = np.float64(1e6) ** (-2.0 * np.arange(64) / 128)

    def bound(ref, p, yarn):
        # test_q3m_yarn_rope.py:132-135: 1 fp16 ulp + 1e-5 max of float64 on the kernel's fp32 angle (the YaRN table form).
        # The plain form is checked against the float64 angle pos * base^(-2j/128); the kernel's angle is that rounded to
        # fp32 (frequency and product, <= 2^-23 relative), which moves the result by at most angle * 2^-23 * max.
        return ulp16(ref) + 1e-5 * np.abs(ref).max() + (0 if yarn else 2.0 ** -23 * p * np.abs(ref).max())

    for yarn, qk, kk in ((False, 'q_plain', 'k_plain'), (True, 'q_yarn', 'k_yarn')):
        for i, p in enumerate(int(v) for v in pos):
            if p < 5000:
                cache = np.zeros((p + 1) * 2 * M, np.float16)
                q16, cache = oracle.qk_rope(qkv[i], ldq, nh, nkv, par, p, cache, 1, yarn=yarn)
                row = cache[p * 2 * M:(p + 1) * 2 * M]
                assert np.array_equal(row[M:], qkv[i, nh * 128 + M:].astype(np.float16))            # V rows exact
                assert not cache[:p * 2 * M].any()                                                  # rows below untouched
                for got, ref in ((q16[0], f[qk][i]), (row[:M].reshape(nkv, 128), f[kk][i])):
                    assert (np.abs(got.astype(np.float64) - ref) <= bound(ref, p, yarn)).all(), (yarn, p)
            qh = qkv[i, :nh * 128].astype(np.float16).reshape(1, nh, 128)
            kh = qkv[i, nh * 128:nh * 128 + M].astype(np.float16).reshape(1, nkv, 128)
            th = (np.float32(p) * tab[:64]).astype(np.float64) if yarn else p * inv64
            ms = float(tab[64]) if yarn else 1.0
            outs = []
            for order in (0, 1):      # the reference's order of the head's sum of squares, and the CUDA kernel's: both inside the bound
                qo, ko = oracle.qk_rope_f16(qh, kh, par, p, yarn=yarn, sum_order=order)
                outs.append((qo, ko))
                for got, x, w in ((qo[0], qh[0], par[:128]), (ko[0], kh[0], par[128:256])):
                    ref = oracle.norm_rope_f64(x, w, th, 1e-6, ms)
                    assert (np.abs(got.astype(np.float64) - ref) <= bound(ref, p, yarn)).all(), (yarn, p, order)
            for a, b in zip(outs[0], outs[1]):     # the two orders: at most one fp16 ulp apart, nearly always equal
                da = np.abs(a.view(np.int16).astype(np.int32) - b.view(np.int16).astype(np.int32))
                assert da.max() <= 1 and (da != 0).mean() < 0.02


def test_sincos_and_powi_sequences():
    th = np.concatenate([np.linspace(0, 10, 20001), np.linspace(0, 131071, 50001), np.linspace(-4000, 4000, 10001)]).astype(np.float32)
    sc = np.array([oracle.sincos(t) for t in th], np.float64)
    t64 = th.astype(np.float64)
    assert np.abs(sc[:, 0] - np.sin(t64)).max() < 2.5e-7 and np.abs(sc[:, 1] - np.cos(t64)).max() < 2.5e-7
    ts = np.float32(np.float32(1e6) ** np.float32(-2.0 / 128))
    for j in range(64):
        want = np.float32(np.float64(ts) ** j)
        assert oracle.powi(ts, j) == float(want)
    assert all(abs(oracle.rsqrt(v) * np.sqrt(np.float64(np.float32(v))) - 1) < 1.2e-7 for v in (1e-6, 0.5, 1.0, 3.7, 1e4))


def test_q8_kv_rows_bitwise(golden):
    """the Q8_0 KV row bytes and the 128-point Hadamard transform: the reference's CPU reference (python/caminus/ref_kv.py), bit for bit"""
    f = golden('q8_kv')
    assert np.array_equal(oracle.hadamard128(f['K']).view(np.uint32), f['H'].view(np.uint32))
    raw, bad = oracle.q8_kv_rows(f['H'], f['V'])
    assert bad == 0 and np.array_equal(raw, f['raw'])
    # the Q8 object's row = encode(hadamard(K16), V16) of the F16 object's halves (tests/engine/test_q3m_yarn_rope.py:121-123)
    g = np.random.default_rng(3); nh, nkv, n, pos0 = 4, 2, 5, 7; M = nkv * 128; ldq = nh * 128 + 2 * M
    qkv = (g.standard_normal((n, ldq)) * 1.3).astype(np.float32)
    par = np.concatenate([(0.5 + g.random(256)), [np.float32(np.float32(1e6) ** np.float32(-2.0 / 128)), 1e-6]]).astype(np.float32)
    q16, c16 = oracle.qk_rope(qkv, ldq, nh, nkv, par, pos0, np.zeros((pos0 + n) * 2 * M, np.float16), n)
    q8, c8, err = oracle.qk_rope_q8(qkv, ldq, nh, nkv, par, pos0, np.zeros((pos0 + n) * 2 * (M // 32) * 34, np.uint8), n)
    rows16 = c16.reshape(-1, 2, nkv, 128)[pos0:].astype(np.float32)
    want, _ = oracle.q8_kv_rows(oracle.hadamard128(rows16[:, 0]), rows16[:, 1])
    assert err == 0 and np.array_equal(c8.reshape(pos0 + n, -1)[pos0:], want) and not c8.reshape(pos0 + n, -1)[:pos0].any()
    assert np.array_equal(q8.view(np.uint16), oracle.hadamard128(q16.astype(np.float32)).astype(np.float16).view(np.uint16))
    bad = qkv.copy(); bad[1, nh * 128 + 3] = np.inf
    _, _, err = oracle.qk_rope_q8(bad, ldq, nh, nkv, par, pos0, np.zeros((pos0 + n) * 2 * (M // 32) * 34, np.uint8), n)
    assert err == 2                                                    # a refused block sets the prefill's error word


def test_iq4_rows_bitwise(golden):
    """IQ4_XS / IQ4_NL row gathers: the reference's host decoders (own_dequant.iq4_xs, gguf-py), bit for bit; clamped ids reported"""
    f = golden('iq4_rows'); T, R = f['T'], f['R']; vocab, nblk = T.shape[:2]; nuniq, bpr = R.shape[:2]
    tok = np.array([0, 22, 5, 99, -1, 7], np.int32)
    out, err = oracle.embd_rows_iq4xs(T, tok, vocab, nblk)
    assert err == 2 and np.array_equal(out.view(np.uint32), f['xs'][np.clip(tok, 0, vocab - 1)].view(np.uint32))
    inv = np.array([3, 0, 10, 11, -2, 4], np.int32)
    out, err = oracle.ple_rows_iq4nl(R, inv, nuniq, bpr)
    assert err == 1 and np.array_equal(out.view(np.uint32), f['nl'][np.clip(inv, 0, nuniq - 1)].view(np.uint32))


def test_q6k_rows_bitwise(golden):
    """the Q6_K decoder of the oracle == the reference's own_dequant.q6_k (== gguf-py) on the fixture, clamped ids included"""
    f = golden('q6k_rows'); T = f['T']; vocab, nblk = T.shape[:2]
    toks = np.array([0, 7, 18, -2, 50, 3], np.int32)
    x = oracle.emb_rows_q6k(T, nblk * 210, vocab, toks, nblk * 256)
    assert np.array_equal(x.view(np.uint32), f['rows'][np.clip(toks, 0, vocab - 1)].view(np.uint32))


def test_iq2s_rows_bitwise(golden):
    """the IQ2_S decoder of the oracle == the reference's own_dequant.iq2_s on the fixture (decoded over the fixture's stand-in grid:
    the real grid is ggml's data and not carried here; the generator also checks the real grid, unstored), clamped ids included"""
    f = golden('iq2s_rows'); T = f['T']; vocab, nblk = T.shape[:2]
    toks = np.array([0, 7, 22, -2, 50, 3], np.int32)
    x = oracle.emb_rows_iq2s(T, nblk * 82, vocab, toks, nblk * 256, oracle.pack_iq2s_grid(f['grid']))
    assert np.array_equal(x.view(np.uint32), f['rows'][np.clip(toks, 0, vocab - 1)].view(np.uint32))


def test_numpy_path_against_the_fixtures(golden):
    """the NumPy restatement of the reference's host path (the benchmark's second CPU leg) against what the reference's own code
    produced: Q4_K rows and Q8_1 scales / codes bit for bit, the norms and the rotation within float32 rounding of float64"""
    from oracle import numpy_path as NP
    f = golden('q4k_rows')
    assert np.array_equal(NP.q4k_rows(f['W'], f['toks']).view(np.uint32), f['want'].view(np.uint32))
    f = golden('q8_1')
    d, s, q = NP.q8_1_blocks(f['x'])
    assert np.array_equal(d.view(np.uint16), f['d16'].view(np.uint16)) and np.array_equal(q, f['q'])
    d, s, q = NP.q8_1_blocks(f['x'][:int(f['n_odd'])])
    assert np.array_equal(d.view(np.uint16), f['d16_odd'].view(np.uint16)) and np.array_equal(q, f['q_odd'])
    f = golden('swiglu')
    h = NP.silu(f['gate']) * f['up'].astype(np.float32)
    assert np.abs(h - f['h64']).max() <= 1e-6 * np.abs(f['h64']).max()
    d, s, q = NP.swiglu_q8_1(f['gate'], f['up'])
    assert (np.abs(q.astype(int) - f['q'].astype(int)) <= 1).all() and (q != f['q']).mean() < 2e-3      # the reference's flip rule: a code may move by one at a .5 boundary
    f = golden('add_rms')
    xs, hh = NP.add_rms_f32(f['x1'], f['r1'], f['w1'])
    assert np.abs(xs - f['s1']).max() <= 1e-6 * np.abs(f['s1']).max() and np.abs(hh - f['h1']).max() <= 2e-6 * np.sqrt((f['h1'] ** 2).mean()) * 10
    f = golden('qk_rope'); nh, nkv = int(f['nh']), int(f['nkv']); par = f['par']
    q = f['qkv'][:, :nh * 128].reshape(-1, nh, 128)
    got = NP.qk_norm_rope_f64(q, par[:128], f['pos'], theta=1e6, eps=float(par[257]))
    assert np.abs(got - f['q_plain']).max() <= 1e-12


def test_silu_scale_q8_1_against_the_host_path():
    """the tape op's work = 1, silu(x * rs) then Q8_1, against the NumPy host path under the reference's flip rule (a code may move by
    one where the quotient sits on a .5 boundary, tests/engine/golden_util.py:132-173); rs = 1 with u = 1 is the SwiGLU form's bytes"""
    from oracle import numpy_path as NP
    g = np.random.default_rng(8); x = (g.standard_normal(4096 + 19) * 3).astype(np.float32); rs = 0.37
    y = oracle.silu_scale_q8_1(x, rs, sum_order=1)
    d, s, q = oracle.q8_split(y)
    dn, sn, qn = NP.q8_1_blocks(NP.silu((x * np.float32(rs)).astype(np.float32)))
    assert (np.abs(q.astype(int) - qn.astype(int)) <= 1).all() and (q != qn).mean() < 2e-3
    assert np.abs(d.view(np.int16).astype(int) - dn.view(np.int16).astype(int)).max() <= 1
    assert np.array_equal(oracle.silu_scale_q8_1(x, 1.0, sum_order=1), oracle.swiglu_q8_1(x, np.ones_like(x), sum_order=1))
