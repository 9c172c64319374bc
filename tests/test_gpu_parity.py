"""Parity of the CUDA path (called through the C ABI / the reference-shaped wrappers) with the CPU oracle on the same
seeded inputs: bit for bit for every stored byte, plus the reference's own tolerance against float64 where it states one."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip('torch')
pytestmark = pytest.mark.gpu

import oracle   # noqa: E402
from caminus_b200 import glue, synth   # noqa: E402
from caminus_b200.engine import gguf, k3   # noqa: E402
from caminus_b200.prefill import q3m_ops, q35own   # noqa: E402

DEV = 'cuda:0'


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def bits(a):
    a = a.detach().cpu().numpy() if torch.is_tensor(a) else np.asarray(a)
    return a.view({2: np.uint16, 4: np.uint32, 1: np.uint8}[a.dtype.itemsize]).reshape(-1)


def same(a, b):
    return np.array_equal(bits(a), bits(b))


def ulp16(v):
    return np.abs(np.spacing(np.abs(v).astype(np.float16))).astype(np.float64)


@pytest.fixture(scope='module')
def O():
    return q3m_ops.Ops(DEV)


# ---- Q4_K embedding rows ------------------------------------------------------------------------------------------------
def test_emb_golden_bitwise(O, golden):
    f = golden('q4k_rows')
    W = f['W']; vocab = int(f['vocab']); rb = W.shape[1] * 144; N = W.shape[1] * 256; toks = f['toks']
    x = torch.zeros(len(toks), N, device=DEV)
    O.emb(cu(W.reshape(-1)), rb, vocab, cu(toks), x, len(toks), N)
    assert same(x, f['want'])                                       # the reference decoder's bits, ids clamped


@pytest.mark.parametrize('n,vocab,N', [(1, 7, 256), (33, 1000, 2048), (16384, 151936, 2048), (257, 300, 5120)])
def test_emb_vs_oracle(O, n, vocab, N):
    W = synth.q4k_table(vocab, N, seed=1); toks = synth.token_ids(n, vocab, seed=1)
    if n > 8: toks[:4] = [-1, vocab, vocab - 1, 0]
    x = torch.full((n, N), float('nan'), device=DEV)
    O.emb(cu(W.reshape(-1)), N // 256 * 144, vocab, cu(toks), x, n, N)
    assert same(x, oracle.q4k_get_rows(W, N // 256 * 144, vocab, toks, N))


# ---- residual add + RMSNorm ---------------------------------------------------------------------------------------------
def test_add_rms16_golden(O, golden):
    f = golden('add_rms')
    x0, dd, ww, nw = f['x0'], f['dd'], f['ww'], f['nw']; n, D = x0.shape
    x = cu(x0); h = torch.zeros(n, D, device=DEV); h16 = torch.zeros(n, D, dtype=torch.float16, device=DEV)
    O.add_rms16(x, cu(nw), 1e-6, h16, n, D, d=cu(dd), w=cu(ww), S=8, h=h)
    xo, ho, h16o = oracle.add_rms16(x0, nw, 1e-6, d=dd, w=ww, S=8)
    assert same(x, xo) and same(h, ho) and same(h16, h16o)
    rel = lambda a, b: float(np.abs(a - b).max() / np.sqrt((b ** 2).mean()))
    assert rel(x.cpu().numpy(), f['xr']) < 1e-6 and rel(h.cpu().numpy(), f['hr']) < 2e-6        # tests/prefill/test_q3m_ops.py:162
    assert rel(h16.float().cpu().numpy(), f['hr']) < 2e-3
    # the decode-token case: T = 1, hidden 2048, one added row
    x = cu(f['x1']); h = torch.zeros(1, 2048, device=DEV); h16 = torch.zeros(1, 2048, dtype=torch.float16, device=DEV)
    O.add_rms16(x, cu(f['w1']), 1e-6, h16, 1, 2048, d=cu(f['r1']), S=1, h=h)
    xo, ho, h16o = oracle.add_rms16(f['x1'], f['w1'], 1e-6, d=f['r1'].reshape(1, 1, -1), S=1)
    assert same(x, xo) and same(h, ho) and same(h16, h16o)
    assert np.abs(h.cpu().numpy() - f['h1']).max() <= 1e-5 * np.abs(f['h1']).max()


@pytest.mark.parametrize('N', [256, 512, 768, 1024, 1280, 1536, 1792, 2048])
@pytest.mark.parametrize('S,weighted', [(0, False), (1, False), (3, True)])
def test_add_rms16_shapes(O, N, S, weighted):
    g = np.random.default_rng(N + S)
    n = 37
    x0 = (g.standard_normal((n, N)) * 3).astype(np.float32); nw = (g.random(N) + 0.5).astype(np.float32)
    dd = g.standard_normal((n, max(S, 1), N)).astype(np.float32) if S else None
    ww = g.random((n, S)).astype(np.float32) if weighted else None
    x = cu(x0); h16 = torch.zeros(n, N, dtype=torch.float16, device=DEV); h = torch.zeros(n, N, device=DEV)
    O.add_rms16(x, cu(nw), 1e-6, h16, n, N, d=None if dd is None else cu(dd), w=None if ww is None else cu(ww), S=S, h=h)
    xo, ho, h16o = oracle.add_rms16(x0, nw, 1e-6, d=dd, w=ww, S=S)
    assert same(x, xo) and same(h, ho) and same(h16, h16o)
    # h omitted: the same h16
    x = cu(x0); h16b = torch.zeros(n, N, dtype=torch.float16, device=DEV)
    O.add_rms16(x, cu(nw), 1e-6, h16b, n, N, d=None if dd is None else cu(dd), w=None if ww is None else cu(ww), S=S)
    assert same(h16b, h16o)


@pytest.mark.parametrize('N', [256, 2048, 2560, 5120, 8192, 65536])
@pytest.mark.parametrize('add', [True, False])
def test_add_rms16_q35(N, add):
    Q = q35own.Ops(DEV)
    g = np.random.default_rng(N)
    n = 9 if N > 8192 else 133
    x0 = (g.standard_normal((n, N)) * 3).astype(np.float32); nw = (g.random(N) + 0.5).astype(np.float32)
    dd = g.standard_normal((n, N)).astype(np.float32) if add else None
    x = cu(x0); h = torch.zeros(n, N, device=DEV); h16 = torch.zeros(n, N, dtype=torch.float16, device=DEV)
    Q.add_rms16(x, cu(nw), 1e-6, h16, n, N, d=None if dd is None else cu(dd), h=h)
    xo, ho, h16o = oracle.add_rms16_q35(x0, nw, 1e-6, d=dd)
    assert same(x, xo) and same(h, ho) and same(h16, h16o)
    with pytest.raises(ValueError): Q.add_rms16(x, cu(nw), 1e-6, h16, n, N)          # h is required (q35own.py:139)


@pytest.mark.parametrize('T,N', [(1, 2048), (5, 256), (777, 5120), (4096, 5120), (64, 8192), (3, 28672),
                                 (70, 512), (99, 768), (130, 1280), (65, 1536), (77, 3072), (66, 3584),       # rows held in one warp's registers
                                 (71, 6144), (67, 7168), (90, 8192), (65, 10240), (64, 12288), (69, 14336), (66, 16384), (65, 20480),   # in two or four warps'
                                 (63, 8192), (200, 3328)])                                                      # few rows / another length: the staged kernel
@pytest.mark.parametrize('add', [True, False])
def test_add_rms_f16(T, N, add):
    x0, r0, w = synth.add_rms_inputs(T, N, seed=T, dtype=np.float16)
    x = cu(x0); h16 = torch.zeros(T, N, dtype=torch.float16, device=DEV)
    glue.add_rms_f16(x, cu(w), 1e-6, h16=h16, d=cu(r0) if add else None)
    xo, ho = oracle.add_rms_f16(x0, w, 1e-6, r0 if add else None)
    assert same(x, xo) and same(h16, ho)
    s = x0.astype(np.float64) + (r0.astype(np.float64) if add else 0)
    ref = oracle.rms_f64(s, w, 1e-6)
    assert (np.abs(h16.float().cpu().numpy() - ref) <= 2 * ulp16(ref) + 1e-5 * np.abs(ref).max()).all()   # 2 fp16 ulp / 1e-5


@pytest.mark.parametrize('N', [28672, 29184, 57600, 58112, 65536])
@pytest.mark.parametrize('add', [True, False])
def test_add_rms_f16_rows_around_the_staging_limit(N, add):
    """row lengths on both sides of what a warp can stage in shared memory (two stages of x and d: about 28 900 values with an addend,
    57 800 without): the staged kernel below, the two-pass kernel above, one set of bytes; through the direct entry, the partial / apply
    pair and the entry that keeps the sums in the library's static array"""
    from caminus_b200 import lib
    T = 5
    x0, r0, w = synth.add_rms_inputs(T, N, seed=N, dtype=np.float16)
    xo, ho = oracle.add_rms_f16(x0, w, 1e-6, r0 if add else None)
    x = cu(x0); d = cu(r0) if add else None; nw = cu(w)
    h16 = glue.add_rms_f16(x, nw, 1e-6, d=d)
    assert same(x, xo) and same(h16, ho)
    L = lib.load(); s = torch.cuda.current_stream().cuda_stream
    x2 = cu(x0); ss = torch.zeros(T, device=DEV); h2 = torch.zeros_like(x2); dp = 0 if d is None else d.data_ptr()
    lib.check(L.cam_rms_partial_f16(T, x2.data_ptr(), dp, ss.data_ptr(), N, s))
    assert same(ss, oracle.rms_partial_f16(x0, r0 if add else None))
    lib.check(L.cam_rms_apply_f16(T, x2.data_ptr(), dp, ss.data_ptr(), nw.data_ptr(), 1e-6, h2.data_ptr(), N, N, s))
    assert same(x2, xo) and same(h2, ho)
    x3 = cu(x0); h3 = torch.zeros_like(x3)
    lib.check(L.cam_rms_norm_f16_static(T, x3.data_ptr(), dp, nw.data_ptr(), 1e-6, h3.data_ptr(), N, s))
    assert same(x3, xo) and same(h3, ho)


# ---- SwiGLU and Q8_1 ------------------------------------------------------------------------------------------------------
def test_q8_1_golden(golden):
    f = golden('q8_1')
    for x, dk, qk in ((f['x'], 'd16', 'q'), (f['x'][:int(f['n_odd'])], 'd16_odd', 'q_odd')):
        y = gguf.quantize_q8_1(cu(x))
        d, s, q = oracle.q8_split(y.cpu().numpy())
        assert np.array_equal(q, f[qk]) and same(d, f[dk])                       # 0 mismatches (tests/engine/test_gguf_mv.py:33-45)
        assert same(y, oracle.q8_1(x, sum_order=1))                              # every byte, the block sums included


def test_q8_1_plain_every_byte_on_hard_inputs():
    """the plain quantiser's division-free codes: all 36 bytes of every block are the exact statements' on scales from 1e-35 to
    1e35, quotients on exact .5 boundaries, zero blocks, infinities and NaNs, and a ragged tail"""
    g_ = np.random.default_rng(5); n = (1 << 20) + 19
    x = (g_.standard_normal(n) * 2.0).astype(np.float32)
    x[:32768] *= (10.0 ** g_.integers(-35, 35, 32768 // 32).repeat(32)).astype(np.float32)      # a scale per block
    blk = x[32768:65536].reshape(-1, 32); blk[:] = np.round(blk * 8) / 8; blk[:, 0] = 127.0 / 8 * 8    # amax 127: d = 1, codes = values: ties at .5
    x[65536:65536 + 64] = 0.0
    x[70000] = np.inf; x[70100] = -np.inf; x[70200] = np.nan; x[80000:80032] = 3e38
    y = gguf.quantize_q8_1(cu(x)).cpu().numpy(); want = oracle.q8_1(x, sum_order=1)
    d, s_, q = oracle.q8_split(y); d1, s1, q1 = oracle.q8_split(want)
    ok = ~np.isnan(d1.astype(np.float32)) & ~np.isnan(s1.astype(np.float32))        # (a NaN has no fixed bit pattern)
    assert np.array_equal(q, q1) and np.array_equal(d.view(np.uint16)[ok], d1.view(np.uint16)[ok]) and np.array_equal(s_.view(np.uint16)[ok], s1.view(np.uint16)[ok])


def sums_close(y, want, h):
    """the block sums of the fast pass: within one fp16 ulp of the exact statements' sum, or 2e-6 sum |h| when the values cancel"""
    _, s, _ = oracle.q8_split(y); _, s0, _ = oracle.q8_split(want)
    n = h.size; hp = np.zeros((n + 31) // 32 * 32); hp[:n] = np.abs(h.astype(np.float64))
    tol = ulp16(s0.astype(np.float64)) + 2e-6 * hp.reshape(-1, 32).sum(1)
    return bool((np.abs(s.astype(np.float64) - s0.astype(np.float64)) <= tol).all())


@pytest.mark.parametrize('dtype', [np.float16, np.float32])
@pytest.mark.parametrize('n', [32, 64, 31, 1, 8 * 25600, 1000003])
def test_swiglu_q8_1_vs_oracle(dtype, n):
    g, u = synth.swiglu_inputs(1, n, seed=n, dtype=dtype)
    g = g.reshape(-1); u = u.reshape(-1)
    if n >= 64: g[:8] = np.array([30, -30, 0, -0.0, 1e-3, -88, 88, 3], dtype); u[32:64] = 0   # silu extremes; an all-zero block
    want = oracle.swiglu_q8_1(g, u, sum_order=1)
    ys = gguf.swiglu_q8_1(cu(g), cu(u), strict=True)
    assert same(ys, want)                                                        # strict: every byte
    assert same(gguf.swiglu_q8_1(cu(g), cu(u), sums=True), want)                 # the fast pass with the sum test: every byte too
    y = gguf.swiglu_q8_1(cu(g), cu(u)).cpu().numpy()
    d, s, q = oracle.q8_split(y); d1, s1, q1 = oracle.q8_split(want)
    assert np.array_equal(q, q1) and same(d, d1)                                 # the fused kernel: d and codes exact, always
    h = oracle.swiglu_f32_from_f16(g, u) if dtype == np.float16 else oracle.silu_mul(g, u)
    assert sums_close(y, want, h)
    d0, s0, q0 = oracle.q8_split(oracle.swiglu_q8_1(g, u, sum_order=0))        # the lane-butterfly sum order: d, codes identical,
    assert np.array_equal(q, q0) and same(d, d0)                                 # the sums within one fp16 ulp
    assert (np.abs(s1.astype(np.float64) - s0.astype(np.float64)) <= ulp16(s0.astype(np.float64)) + 1e-6).all()


@pytest.mark.parametrize('kind', ['wide_gate', 'outliers', 'tiny', 'huge', 'negative_gate', 'nonfinite', 'ties'])
def test_swiglu_q8_1_hard_inputs(kind):
    """inputs that stress the fast pass's margins: the fused kernel's d and codes stay the exact statements' bytes"""
    g_ = np.random.default_rng(sum(map(ord, kind)))
    n = 1 << 20
    gate = (g_.standard_normal(n) * 1.5).astype(np.float32); up = (g_.standard_normal(n) * 1.5).astype(np.float32)
    if kind == 'wide_gate': gate *= 4                                            # tests/prefill/test_q3m_ops.py:184
    if kind == 'outliers': m = g_.random(n) < 0.002; gate[m] *= 30; up[m] *= 30   # tests/prefill/test_prefill_glue.py:125-128
    if kind == 'tiny': gate *= 1e-3; up *= 1e-4
    if kind == 'huge': up *= 1e3
    if kind == 'negative_gate': gate = -np.abs(gate) * 3
    if kind == 'ties': gate = np.round(gate * 2) / 2; up = np.round(up * 4) / 4   # few distinct values: exact .5 quotients occur
    gate = gate.astype(np.float16); up = up.astype(np.float16)
    if kind == 'nonfinite':
        gate[5] = np.inf; up[100] = np.nan; gate[200] = -np.inf; up[300] = np.inf; gate[400] = np.nan
    want = oracle.swiglu_q8_1(gate, up, sum_order=1)
    y = gguf.swiglu_q8_1(cu(gate), cu(up)).cpu().numpy()
    d, s, q = oracle.q8_split(y); d1, s1, q1 = oracle.q8_split(want)
    ok = ~(np.isnan(d1.astype(np.float32)))                                      # (a NaN scale has no fixed bit pattern)
    assert np.array_equal(q, q1) and np.array_equal(d.view(np.uint16)[ok], d1.view(np.uint16)[ok]) and np.isnan(d.astype(np.float32)[~ok]).all()
    if kind != 'nonfinite': assert sums_close(y, want, oracle.swiglu_f32_from_f16(gate, up))
    if kind != 'nonfinite': assert np.array_equal(gguf.swiglu_q8_1(cu(gate), cu(up), sums=True).cpu().numpy(), want)     # all 36 bytes


@pytest.mark.parametrize('n', [32, 1, 4096 + 7, 1 << 20])
@pytest.mark.parametrize('rs', [1.0, 0.25, -3.0, 1e-3, 40.0])
def test_silu_scale_q8_1(n, rs):
    """gg_silu_scale_q8_1 (the tape op's work = 1: ggml_scale, ggml_silu, the quantiser): scale and codes are the oracle's bytes, the
    _sums form all 36 bytes; gates scaled below -8 and above the exponential's range, zeros, a zero block, a ragged tail"""
    g_ = np.random.default_rng(n + int(abs(rs) * 7)); x = (g_.standard_normal(n) * 4).astype(np.float32)
    if n >= 64: x[:8] = np.array([30, -30, 0, -0.0, 1e-3, -88, 88, 3], np.float32); x[32:64] = 0
    want = oracle.silu_scale_q8_1(x, rs, sum_order=1)
    assert same(gguf.silu_scale_q8_1(cu(x), rs, sums=True), want)
    d, s, q = oracle.q8_split(gguf.silu_scale_q8_1(cu(x), rs).cpu().numpy()); d1, s1, q1 = oracle.q8_split(want)
    assert np.array_equal(q, q1) and same(d, d1)
    assert (np.abs(s.astype(np.float64) - s1.astype(np.float64)) <= ulp16(s1.astype(np.float64)) + 1e-5).all()


def test_swiglu_q8_1_f32_denormal_gates():
    """fp32 gates so small that the exact statements' g / (1 + e) is a denormal (its rounding is not the fast product's), next to
    huge ups that bring the product back to the block's scale; zero gates; the fused entries still give the exact statements' bytes"""
    g_ = np.random.default_rng(77); n = 1 << 16
    gate = (g_.standard_normal(n) * 1.5).astype(np.float32); up = (g_.standard_normal(n) * 1.5).astype(np.float32)
    idx = np.arange(0, n, 37)
    gate[idx] = (g_.integers(1, 1 << 20, idx.size) * np.float64(1.4e-45)).astype(np.float32) * np.where(g_.random(idx.size) < 0.5, -1, 1).astype(np.float32)
    up[idx] = (g_.random(idx.size).astype(np.float32) + 0.5) * np.float32(2e38)
    gate[5::101] = 0.0
    want = oracle.swiglu_q8_1(gate, up, sum_order=1)
    for strict in (False, True):
        y = gguf.swiglu_q8_1(cu(gate), cu(up), strict=strict).cpu().numpy()
        d, s_, q = oracle.q8_split(y); d1, s1, q1 = oracle.q8_split(want)
        assert np.array_equal(q, q1) and np.array_equal(d.view(np.uint16), d1.view(np.uint16))
        if strict: assert np.array_equal(y, want)
    assert np.array_equal(gguf.swiglu_q8_1(cu(gate), cu(up), sums=True).cpu().numpy(), want)


def test_swiglu_golden_reference_host_path(golden):
    """against the reference's host path (numpy float32 silu, q8_host): the flip rule of tests/engine/golden_util.py:132-173"""
    f = golden('swiglu')
    y = gguf.swiglu_q8_1(cu(f['gate']), cu(f['up']))
    d, s, q = oracle.q8_split(y.cpu().numpy())
    dq = q.astype(np.int32) - f['q'].astype(np.int32)
    assert np.abs(dq).max() <= 1 and (dq != 0).mean() < 1e-3
    assert np.abs(d.view(np.int16).astype(np.int32) - f['d16'].view(np.int16).astype(np.int32)).max() <= 1
    y16 = torch.zeros(5000, dtype=torch.float16, device=DEV)
    q3m_ops.Ops(DEV).swiglu(cu(f['gg']), cu(f['uu']), y16, 5000)
    assert np.abs(y16.float().cpu().numpy() - f['sr']).max() <= np.abs(f['sr']).max() * 2.0 ** -10    # test_q3m_ops.py:184-187
    assert same(y16, oracle.swiglu16(f['gg'], f['uu']))
    assert same(gguf.silu_mul(cu(f['gg']), cu(f['uu'])), oracle.silu_mul(f['gg'], f['uu']))


def test_swiglu_q8_1_full_size_config():
    """The SwiGLU + Q8_1 benchmark workload (T = 8192, I = 25600): the whole output against the oracle on a strided sample of rows, and
    size-independent properties of all of it: |q| <= 127, d >= 0, |x - d q| <= d / 2 up to fp16 rounding of d."""
    T, I = 8192, 25600
    g, u = synth.swiglu_inputs(T, I, seed=0)
    gd, ud = cu(g), cu(u)
    y = gguf.swiglu_q8_1(gd.reshape(-1), ud.reshape(-1))
    ystrict = gguf.swiglu_q8_1(gd.reshape(-1), ud.reshape(-1), strict=True)
    yb, ysb = y.view(T, I // 32, 36), ystrict.view(T, I // 32, 36)
    rows = np.arange(0, T, 61)
    want = oracle.swiglu_q8_1(g[rows].reshape(-1), u[rows].reshape(-1), sum_order=1).reshape(len(rows), I // 32, 36)
    assert np.array_equal(ysb[torch.from_numpy(rows).to(DEV)].cpu().numpy(), want)     # the exact statements: the oracle's bytes
    assert torch.equal(gguf.swiglu_q8_1(gd.reshape(-1), ud.reshape(-1), sums=True), ystrict)       # the sum test: all 36 bytes of all 6.5 M blocks
    # the fused kernel against the exact statements over ALL 6.5 M blocks: d and the 32 codes identical, sums within one fp16 ulp
    assert torch.equal(yb[:, :, 0:2], ysb[:, :, 0:2]) and torch.equal(yb[:, :, 4:], ysb[:, :, 4:])
    sf, ss_ = yb[:, :, 2:4].contiguous().view(torch.float16).float(), ysb[:, :, 2:4].contiguous().view(torch.float16).float()
    assert bool(((sf - ss_).abs() <= ss_.abs() * 2.0 ** -10 + 1e-3).all())
    qs = yb[:, :, 4:].contiguous().view(torch.int8)
    assert int(qs.min()) >= -127 and int(qs.max()) <= 127
    d = yb[:, :, 0:2].contiguous().view(torch.float16).float().squeeze(-1)
    assert bool((d >= 0).all()) and bool((qs.abs().amax(-1) == 127)[d > 0].all())      # the largest value of a block codes to 127
    y2 = gguf.swiglu_q8_1(gd.reshape(-1), ud.reshape(-1))
    assert torch.equal(y, y2)                                                          # run to run identical


# ---- q/k RMSNorm + RoPE -----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize('yarn', [False, True])
def test_qk_rope_golden(golden, yarn):
    f = golden('qk_rope')
    pos, nh, nkv, par, qkv = f['pos'], int(f['nh']), int(f['nkv']), f['par'], f['qkv']
    M = nkv * 128; ldq = nh * 128 + 2 * M
    R = q3m_ops.Ops(DEV, yarn=yarn)
    pd = cu(par if yarn else par[:258])
    for i, p in enumerate(int(v) for v in pos):
        if p >= 5000: continue
        cache0 = (np.random.default_rng(p).standard_normal((p + 3) * 2 * M) * 1.5).astype(np.float16)
        cache = cu(cache0); q16 = torch.zeros(1, nh, 128, dtype=torch.float16, device=DEV)
        R.qk_rope(cu(qkv[i]), ldq, nh, nkv, pd, p, q16, cache, 1)
        qo, co = oracle.qk_rope(qkv[i], ldq, nh, nkv, par, p, cache0, 1, yarn=yarn, sum_order=1)
        assert same(q16, qo) and same(cache, co)                       # K | V row written, every other row untouched
        ref = f['q_yarn' if yarn else 'q_plain'][i]
        bound = ulp16(ref) + 1e-5 * np.abs(ref).max() + (0 if yarn else 2.0 ** -23 * p * np.abs(ref).max())
        assert (np.abs(q16[0].float().cpu().numpy() - ref) <= bound).all()     # tests/engine/test_q3m_yarn_rope.py:132-135


@pytest.mark.parametrize('n,nh,nkv,pos0', [(75, 32, 4, 1000), (1, 32, 4, 0), (130, 64, 8, 7), (19, 5, 1, 3), (40, 16, 2, 131000), (5000, 32, 4, 3), (77, 40, 8, 0),
                                           (33, 32, 8, 9), (2500, 64, 8, 1)])
def test_qk_rope_chunk(O, n, nh, nkv, pos0):
    """a chunk at pos0 as tests/prefill/test_q3m_ops.py:189-217 runs it, with a padded row stride"""
    g = np.random.default_rng(n); M = nkv * 128; ldq = nh * 128 + 2 * M + 64; rows = 9 if pos0 > 100000 else pos0 + n + 2
    base = pos0 if pos0 > 100000 else 0
    par = synth.rope_par(seed=n)
    qkv = (g.standard_normal((n, ldq)) * 3).astype(np.float32)
    cache0 = (g.standard_normal((rows if base == 0 else n + 2) * 2 * M) * 1.5).astype(np.float16)
    if base:   # a cache this large is not needed: check the positions with the fp16 entry instead
        q = qkv[:, :nh * 128].astype(np.float16).reshape(n, nh, 128); k = qkv[:, nh * 128:nh * 128 + M].astype(np.float16).reshape(n, nkv, 128)
        qo, ko = glue.qk_rope_f16(cu(q), cu(k), cu(par), pos0, qo=torch.zeros(n, nh, 128, dtype=torch.float16, device=DEV),
                                  ko=torch.zeros(n, nkv, 128, dtype=torch.float16, device=DEV))
        qr, kr = oracle.qk_rope_f16(q, k, par, pos0, sum_order=1)
        assert same(qo, qr) and same(ko, kr)
        return
    cache = cu(cache0); q16 = torch.zeros(n, nh, 128, dtype=torch.float16, device=DEV)
    O.qk_rope(cu(qkv.reshape(-1)), ldq, nh, nkv, cu(par), pos0, q16, cache, n)
    qo, co = oracle.qk_rope(qkv.reshape(-1), ldq, nh, nkv, par, pos0, cache0, n, sum_order=1)
    assert same(q16, qo) and same(cache, co)
    assert np.array_equal(cache.cpu().numpy()[:pos0 * 2 * M], cache0[:pos0 * 2 * M])                 # rows below the chunk untouched
    assert np.array_equal(cache.cpu().numpy().reshape(-1, 2, M)[pos0:pos0 + n, 1], qkv[:, nh * 128 + M:nh * 128 + 2 * M].astype(np.float16))


@pytest.mark.parametrize('yarn', [False, True])
def test_qk_rope_f16_config(yarn):
    """The q/k norm + RoPE benchmark workload: T = 4096, 32 q + 4 kv heads, positions 0 .. 4095; in place and out of place"""
    T, nh, nkv = 4096, 32, 4
    q, k = synth.qk_inputs(T, nh, nkv, seed=0)
    par = synth.rope_par(seed=0, yarn_table=synth.yarn_table() if yarn else None)
    qr, kr = oracle.qk_rope_f16(q, k, par, 0, yarn=yarn, sum_order=1)
    qd, kd = cu(q), cu(k)
    qo, ko = glue.qk_rope_f16(qd, kd, cu(par), 0, qo=torch.empty_like(qd), ko=torch.empty_like(kd), yarn=yarn)
    assert same(qo, qr) and same(ko, kr) and same(qd, q)
    glue.qk_rope_f16(qd, kd, cu(par), 0, yarn=yarn)
    assert same(qd, qr) and same(kd, kr)
    # float64 on the kernel's fp32 angle: 1 fp16 ulp + 1e-5 max (tests/engine/test_q3m_yarn_rope.py:132-135), sampled tokens
    for t in (0, 1, 63, 64, 1000, 4095):
        fr = par[258:322] if yarn else np.array([oracle.powi(par[256], j) for j in range(64)], np.float32)
        th = (np.float32(t) * fr).astype(np.float64)
        ref = oracle.norm_rope_f64(q[t], par[:128], th, 1e-6, float(par[322]) if yarn else 1.0)
        assert (np.abs(qr[t].astype(np.float64) - ref) <= ulp16(ref) + 1e-5 * np.abs(ref).max()).all()


def test_qk_rope_refusals(O):
    """a span outside the cache: refused on the host, nothing launched, buffers keep their bytes (test_q3m_ops.py:241-257)"""
    nh, nkv, n = 32, 4, 75; M = nkv * 128; ctx = 1075
    par = cu(synth.rope_par()); qkv = torch.randn(n * (nh * 128 + 2 * M), device=DEV)
    cache = torch.randn(ctx * 2 * M, device=DEV).half(); q16 = torch.zeros(n, nh, 128, dtype=torch.float16, device=DEV)
    keep = (cache.clone(), q16.clone())
    for fn in (lambda: O.qk_rope(qkv, nh * 128 + 2 * M, nh, nkv, par, -1, q16, cache, n),
               lambda: O.qk_rope(qkv, nh * 128 + 2 * M, nh, nkv, par, ctx - n + 1, q16, cache, n),
               lambda: O.qk_rope(qkv, nh * 128 + 2 * M, nh, nkv, par, ctx - 64 - n + 1, q16, cache, n, rows=ctx - 64),
               lambda: O.qk_rope(qkv, nh * 128 + 2 * M, nh, nkv, par, 1000.5, q16, cache, n)):
        with pytest.raises(k3.ContextBoundsError): fn()
    torch.cuda.synchronize()
    assert torch.equal(cache, keep[0]) and torch.equal(q16, keep[1])
    with pytest.raises(ValueError): O.qk_rope(qkv, nh * 128, nh, nkv, par, 0, q16, cache, n)              # row stride too short
    with pytest.raises(ValueError): O.qk_rope(qkv, nh * 128 + 2 * M, nh, nkv, par[:200], 0, q16, cache, n)


# ---- the loader interface -----------------------------------------------------------------------------------------------
def test_module_interface():
    from caminus_b200.device import cuda as hip
    with pytest.raises(FileNotFoundError): hip.Module('no_such_object')
    m = hip.Module('q3m_prefill')
    with pytest.raises(RuntimeError): m.q3p_attn
    x = torch.zeros(4, 256, device=DEV)
    with pytest.raises(ValueError):   # a misaligned row pointer is refused, nothing is launched
        m.q3p_emb((1,), (256,), torch.zeros(144, dtype=torch.uint8, device=DEV), ctypes.c_int(144), ctypes.c_int(1),
                  torch.zeros(1, dtype=torch.int32, device=DEV), x.view(-1)[1:], ctypes.c_int(256))
    with pytest.raises(ValueError):   # grid.y must be nh + nkv
        m.q3p_qk_rope((1, 5), (128,), x, ctypes.c_int(768), ctypes.c_int(2), ctypes.c_int(2), x, ctypes.c_int(0), x, x)
    assert 'q3m_prefill' in hip.LOADED


def test_layer_glue_sequence():
    """the per-layer order of the benchmarked sequence (Qwen3-32B shape) at a small T: each op's bytes are the oracle's"""
    T, N, nh, nkv, I = 96, 5120, 64, 8, 25600
    x0, r0, w = synth.add_rms_inputs(T, N, seed=5, dtype=np.float16)
    q0, k0 = synth.qk_inputs(T, nh, nkv, seed=5); g0, u0 = synth.swiglu_inputs(T, I, seed=5); par = synth.rope_par(seed=5)
    L = glue.LayerGlue(cu(w), cu(par))
    x, q, k = cu(x0), cu(q0), cu(k0)
    h16 = torch.empty_like(x); yq = torch.empty(T * I // 32 * 36, dtype=torch.uint8, device=DEV)
    L(x, cu(r0), q, k, cu(g0), cu(u0), h16, yq, pos0=11)
    xo, ho = oracle.add_rms_f16(x0, w, 1e-6, r0); qo, ko = oracle.qk_rope_f16(q0, k0, par, 11, sum_order=1)
    assert same(x, xo) and same(h16, ho) and same(q, qo) and same(k, ko)
    d, s, q_ = oracle.q8_split(yq.cpu().numpy()); d1, s1, q1 = oracle.q8_split(oracle.swiglu_q8_1(g0.reshape(-1), u0.reshape(-1), sum_order=1))
    assert same(d, d1) and np.array_equal(q_, q1)


def test_config5_full_size_properties():
    """The benchmarked per-layer sequence at its full per-GPU size (T = 65536 rows, 13.7 GB per pass), through size-independent properties:
    chunk-split invariance (one launch == three launches over row ranges, bit for bit: the reference's own gate for its prefill),
    the updated residual == fp16(x + r) computed by torch, fast == strict SwiGLU blocks (d and codes) over all 52 M blocks,
    and rows sampled across the batch == the oracle"""
    T, N, nh, nkv, I = 65536, 5120, 64, 8, 25600
    gen = torch.Generator(device=DEV); gen.manual_seed(55)
    rn = lambda *sh, sc=1.0: (torch.randn(*sh, device=DEV, generator=gen) * sc).half()
    x0, r0 = rn(T, N), rn(T, N); q0, k0 = rn(T, nh, 128), rn(T, nkv, 128)
    w = (1 + 0.05 * torch.randn(N, device=DEV, generator=gen)); par = cu(synth.rope_par(seed=55))
    L = glue.LayerGlue(w, par)
    g0, u0 = rn(T, I, sc=1.5), rn(T, I, sc=1.5)
    def run(cuts):
        x, q, k = x0.clone(), q0.clone(), k0.clone()
        h16 = torch.empty_like(x); yq = torch.empty(T * I // 32 * 36, dtype=torch.uint8, device=DEV); rb = I // 32 * 36
        for a, b in zip(cuts[:-1], cuts[1:]):
            L(x[a:b], r0[a:b], q[a:b], k[a:b], g0[a:b], u0[a:b], h16[a:b], yq[a * rb:b * rb], pos0=7 + a)
        return x, h16, q, k, yq
    one = run([0, T]); three = run([0, 20001, 20002, T])
    for a, b in zip(one, three): assert torch.equal(a, b)
    x, h16, q, k, yq = one
    del three
    assert torch.equal(x, (x0.float() + r0.float()).half())
    strict = gguf.swiglu_q8_1(g0.view(-1), u0.view(-1), strict=True).view(-1, 36); fast = yq.view(-1, 36)
    assert torch.equal(fast[:, :2], strict[:, :2]) and torch.equal(fast[:, 4:], strict[:, 4:])
    del strict
    rows = np.unique(np.concatenate([[0, 1, T - 1], np.random.default_rng(9).integers(0, T, 29)]))
    xs, rs = x0[rows].cpu().numpy(), r0[rows].cpu().numpy()
    xo, ho = oracle.add_rms_f16(xs, w.cpu().numpy(), 1e-6, rs)
    assert same(x[rows], xo) and same(h16[rows], ho)
    for i, t in enumerate(rows):
        qo, ko = oracle.qk_rope_f16(q0[t:t + 1].cpu().numpy(), k0[t:t + 1].cpu().numpy(), par.cpu().numpy(), 7 + int(t), sum_order=1)
        assert same(q[t:t + 1], qo) and same(k[t:t + 1], ko)
    want = oracle.swiglu_q8_1(g0[rows].cpu().numpy().reshape(-1), u0[rows].cpu().numpy().reshape(-1), sum_order=1).reshape(len(rows), -1, 36)
    got = yq.view(T, -1, 36)[rows].cpu().numpy()
    assert np.array_equal(got[:, :, :2], want[:, :, :2]) and np.array_equal(got[:, :, 4:], want[:, :, 4:])


# ---- tensor-parallel RMSNorm (hidden sharded) ---------------------------------------------------------------------------------
@pytest.mark.parametrize('T,N,G', [(300, 5120, 8), (64, 2048, 2), (1000, 5120, 4)])
@pytest.mark.parametrize('add', [True, False])
def test_tp_rmsnorm_pieces(T, N, G, add):
    """the two kernels of the hidden-sharded norm on the G column shards of one row batch (all on this GPU): each shard's
    partial and its apply are the oracle's bytes; the whole agrees with the unsharded kernel within 1e-5 relative (the
    order of the sum over shards differs from the unsharded row sum)"""
    from caminus_b200 import dist as D
    x0, r0, w = synth.add_rms_inputs(T, N, seed=T + G, dtype=np.float16)
    parts, shards = [], []
    for r in range(G):
        a, b = D.col_shard(N, r, G)
        xs = np.ascontiguousarray(x0[:, a:b]); rs = np.ascontiguousarray(r0[:, a:b]) if add else None
        norm = D.TPRmsNorm(cu(w[a:b]), N, 1e-6, all_reduce=lambda t: None)
        ss = norm.partial(cu(xs), cu(rs) if add else None).clone()
        assert same(ss, oracle.rms_partial_f16(xs, rs))
        parts.append(ss); shards.append((a, b, xs, rs, norm))
    tot = torch.zeros(T, device=DEV)
    for ss in parts: tot += ss                                       # rank order, as a ring all-reduce would not guarantee
    full_x, full_h = oracle.add_rms_f16(x0, w, 1e-6, r0 if add else None)
    for a, b, xs, rs, norm in shards:
        xd = cu(xs)
        h16 = norm.apply(xd, tot, d=cu(rs) if add else None)
        xo, ho = oracle.rms_apply_f16(xs, tot.cpu().numpy(), w[a:b], 1e-6, N, rs)
        assert same(xd, xo) and same(h16, ho)
        assert same(xd, full_x[:, a:b].copy())                       # the residual update does not depend on the sharding
        ref = full_h[:, a:b].astype(np.float64)
        assert (np.abs(h16.float().cpu().numpy() - ref) <= ulp16(ref) + 1e-5 * np.abs(ref).max()).all()


def test_add_rms16_single_row_kernel_and_many_rows_agree(O):
    """n <= 2 x multiprocessors takes the block-per-row kernel, more rows the warp-per-row kernel: the same bytes"""
    g = np.random.default_rng(9); N = 2048; n = 700
    x0 = (g.standard_normal((n, N)) * 3).astype(np.float32); dd = g.standard_normal((n, 2, N)).astype(np.float32)
    ww = g.random((n, 2)).astype(np.float32); nw = (g.random(N) + 0.5).astype(np.float32)
    outs = []
    for rows in (n, 5):
        x = cu(x0[:rows]); h = torch.zeros(rows, N, device=DEV); h16 = torch.zeros(rows, N, dtype=torch.float16, device=DEV)
        O.add_rms16(x, cu(nw), 1e-6, h16, rows, N, d=cu(dd[:rows]), w=cu(ww[:rows]), S=2, h=h)
        outs.append((x.cpu().numpy(), h.cpu().numpy(), h16.cpu().numpy()))
    for a, b in zip(outs[0], outs[1]): assert same(a[:5], b)
    xo, ho, h16o = oracle.add_rms16(x0[:5], nw, 1e-6, d=dd[:5], w=ww[:5], S=2)
    assert same(outs[1][0], xo) and same(outs[1][1], ho) and same(outs[1][2], h16o)


# ---- the Q8_0 KV cache form ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize('yarn', [False, True])
@pytest.mark.parametrize('n,nh,nkv,pos0', [(75, 32, 4, 1000), (1, 32, 4, 0), (33, 16, 2, 5), (20, 5, 3, 2), (5000, 32, 4, 3), (130, 64, 8, 7), (41, 40, 8, 2), (9, 32, 8, 0)])
def test_qk_rope_q8(n, nh, nkv, pos0, yarn):
    """q3p_qk_rope_q8: q16 and the Q8_0 row bytes are the oracle's; the row is encode(hadamard(K16), V16) of the F16 object's
    halves (tests/engine/test_q3m_yarn_rope.py:121-123); rows below the chunk untouched; a refused block sets bit 2 of err"""
    g = np.random.default_rng(n + nh); M = nkv * 128; ldq = nh * 128 + 2 * M; rowb = 2 * (M // 32) * 34
    par = synth.rope_par(seed=n, yarn_table=synth.yarn_table() if yarn else None)
    qkv = (g.standard_normal((n, ldq)) * 3).astype(np.float32)
    tie = ((g.integers(-126, 126, 32) + 0.5) / 4).astype(np.float32); tie[3] = 127 / 4         # a V block whose quotients sit on .5 (scale 1 / 4):
    qkv[n // 3, nh * 128 + M + 32:nh * 128 + M + 64] = tie                                     # roundf rounds those away from zero
    cache0 = g.integers(0, 256, (pos0 + n + 2) * rowb, dtype=np.uint8)
    R = q3m_ops.Ops(DEV, q8=True, yarn=yarn)
    cache = cu(cache0); q16 = torch.zeros(n, nh, 128, dtype=torch.float16, device=DEV); err = torch.zeros(1, dtype=torch.int32, device=DEV)
    R.qk_rope(cu(qkv.reshape(-1)), ldq, nh, nkv, cu(par), pos0, q16, cache, n, err=err)
    qo, co, eo = oracle.qk_rope_q8(qkv, ldq, nh, nkv, par, pos0, cache0, n, yarn=yarn, sum_order=1)
    assert int(err.item()) == 0 == eo and same(q16, qo) and np.array_equal(cache.cpu().numpy(), co)
    F16 = q3m_ops.Ops(DEV, yarn=yarn)
    c16 = torch.zeros((pos0 + n) * 2 * M, dtype=torch.float16, device=DEV); q16f = torch.zeros_like(q16)
    F16.qk_rope(cu(qkv.reshape(-1)), ldq, nh, nkv, cu(par), pos0, q16f, c16, n)
    rows16 = c16.cpu().numpy().reshape(-1, 2, nkv, 128)[pos0:].astype(np.float32)
    want, _ = oracle.q8_kv_rows(oracle.hadamard128(rows16[:, 0]), rows16[:, 1])
    assert np.array_equal(cache.cpu().numpy().reshape(-1, rowb)[pos0:pos0 + n], want)
    bad = qkv.copy(); bad[n // 2, nh * 128 + M + 7] = np.nan          # a NaN in V: that block is refused and keeps its bytes
    cache = cu(cache0); err.zero_()
    R.qk_rope(cu(bad.reshape(-1)), ldq, nh, nkv, cu(par), pos0, q16, cache, n, err=err)
    _, co, eo = oracle.qk_rope_q8(bad, ldq, nh, nkv, par, pos0, cache0, n, yarn=yarn, sum_order=1)
    assert int(err.item()) == 2 == eo and np.array_equal(cache.cpu().numpy(), co)
    from caminus_b200.errors import InvalidKVEncoding, NumericalFailure
    with pytest.raises(InvalidKVEncoding): R.check_kv_code(err)                     # the host's reading of the word: terminal, and sticky
    assert int(err.item()) == 2 and issubclass(InvalidKVEncoding, NumericalFailure)
    with pytest.raises(ValueError): R.qk_rope(cu(qkv.reshape(-1)), ldq, nh, nkv, cu(par), pos0, q16, cache, n)          # err is required
    with pytest.raises(k3.ContextBoundsError): R.qk_rope(cu(qkv.reshape(-1)), ldq, nh, nkv, cu(par), pos0 + 3, q16, cache, n, err=err)


# ---- the one-kernel tensor-parallel RMSNorm on ONE GPU: a single rank; two ranks with the other rank's words written beforehand
# (no kernel waits for another kernel); a wait that nothing answers (bounded: the status word reports it)
def _tp_words(part, tag):
    return (np.uint64(tag) << np.uint64(32)) | part.view(np.uint32).astype(np.uint64)


def test_tp_rms_fused_single_rank_is_the_unsharded_norm():
    from caminus_b200 import dist as D
    T, N = 700, 5120
    x0, r0, w = synth.add_rms_inputs(T, N, seed=11, dtype=np.float16)
    F_ = D.TPRmsNormFused(cu(w), N, T, 1e-6, device=DEV)
    for rep in range(3):                                            # (tags 1, 2, 3: both halves of the buffer)
        x = cu(x0); h = F_(x, cu(r0)); F_.check()
        xo, ho = oracle.add_rms_f16(x0, w, 1e-6, r0)
        assert same(x, xo) and same(h, ho)
    with pytest.raises(ValueError): F_(cu(np.zeros((T + 1, N), np.float16)))
    # a call without rows launches nothing and leaves the tag alone (two launches in a row must not share a half of the buffer)
    before = F_.tag; F_(torch.zeros(0, N, dtype=torch.float16, device=DEV)); assert F_.tag == before
    # two norms over one exchange (one buffer, one tag sequence), called alternately
    ex = D.TPExchange(T, group=D.SOLO, device=DEV)
    wa, wb = cu(w), cu((w * 0.5).astype(np.float32)); Fa, Fb = D.TPRmsNormFused(wa, N, exchange=ex), D.TPRmsNormFused(wb, N, exchange=ex)
    for rep in range(4):
        Fn, wn = (Fa, w) if rep % 2 == 0 else (Fb, (w * 0.5).astype(np.float32))
        x = cu(x0); h = Fn(x, cu(r0)); Fn.check()
        xo, ho = oracle.add_rms_f16(x0, wn, 1e-6, r0)
        assert same(x, xo) and same(h, ho) and ex.tag == rep + 1
    ex.close()
    for N2 in (2048, 640, 1288):                                       # rows held in registers (one row / two rows deep), a short last chunk
        x0, r0, w = synth.add_rms_inputs(T, N2, seed=N2, dtype=np.float16)
        F2 = D.TPRmsNormFused(cu(w), N2, T, 1e-6, device=DEV)
        for dd in (r0, None):
            x = cu(x0); h = F2(x, None if dd is None else cu(dd)); F2.check()
            tot = np.float32(0) + oracle.rms_partial_f16(x0, dd)
            xo, ho = oracle.rms_apply_f16(x0, tot, w, 1e-6, N2, dd)
            assert same(x, xo) and same(h, ho)


@pytest.mark.parametrize('N', [2560, 1024, 1296])                      # shards of 1280 (a warp per row), 512 and 648 (a half-warp per row)
def test_tp_rms_fused_two_ranks_with_the_peer_words_in_place(N):
    from caminus_b200 import lib
    T, world, tag = 300, 2, 5
    x0, r0, w = synth.add_rms_inputs(T, N, seed=12, dtype=np.float16)
    Ns = N // world; L = lib.load(); words = L.cam_tp_rms_words(T, world)
    parts = [oracle.rms_partial_f16(x0[:, r * Ns:(r + 1) * Ns], r0[:, r * Ns:(r + 1) * Ns]) for r in range(world)]
    tot = (np.float32(0) + parts[0]) + parts[1]
    for rank in range(world):
        other = 1 - rank
        own = np.zeros(words, np.uint64); half = (tag & 1) * world * T
        own[half + other * T: half + other * T + T] = _tp_words(parts[other], tag)      # the other rank's partials, as its kernel would have stored them
        own_d = torch.from_numpy(own.view(np.int64)).to(DEV); peer_d = torch.zeros(words, dtype=torch.int64, device=DEV)
        ptrs = [0, 0]; ptrs[rank] = own_d.data_ptr(); ptrs[other] = peer_d.data_ptr()
        peers = torch.tensor(ptrs, dtype=torch.int64, device=DEV); status = torch.zeros(1, dtype=torch.int32, device=DEV)
        xs = cu(np.ascontiguousarray(x0[:, rank * Ns:(rank + 1) * Ns])); ds = cu(np.ascontiguousarray(r0[:, rank * Ns:(rank + 1) * Ns]))
        nw = cu(w[rank * Ns:(rank + 1) * Ns].copy()); h = torch.zeros_like(xs)
        lib.check(L.cam_tp_rms_norm_f16(T, xs.data_ptr(), ds.data_ptr(), nw.data_ptr(), 1e-6, h.data_ptr(), Ns, N, peers.data_ptr(), rank, world, T, tag,
                                        status.data_ptr(), torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        xo, ho = oracle.rms_apply_f16(x0[:, rank * Ns:(rank + 1) * Ns], tot, w[rank * Ns:(rank + 1) * Ns], 1e-6, N, r0[:, rank * Ns:(rank + 1) * Ns])
        assert int(status.item()) == 0 and same(xs, xo) and same(h, ho)
        sent = peer_d.cpu().numpy().view(np.uint64)[half + rank * T: half + rank * T + T]   # what this rank stored into the peer's buffer
        assert np.array_equal(sent, _tp_words(parts[rank], tag))
        assert np.array_equal(own_d.cpu().numpy().view(np.uint64)[half + rank * T: half + rank * T + T], _tp_words(parts[rank], tag))


@pytest.mark.parametrize('Ns', [256, 640])                             # the staged kernel and the lean one
def test_tp_rms_fused_wait_runs_out_and_reports(Ns):
    """a peer that never writes: every wait ends at its limit, the status word says so, the rows are left alone, the context lives on"""
    from caminus_b200 import lib
    T, world = 16, 2
    L = lib.load(); words = L.cam_tp_rms_words(T, world)
    own = torch.zeros(words, dtype=torch.int64, device=DEV); peer = torch.zeros(words, dtype=torch.int64, device=DEV)
    peers = torch.tensor([own.data_ptr(), peer.data_ptr()], dtype=torch.int64, device=DEV); status = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = torch.ones(T, Ns, dtype=torch.float16, device=DEV); nw = torch.ones(Ns, device=DEV); h = torch.zeros_like(x)
    lib.check(L.cam_tp_rms_norm_f16(T, x.data_ptr(), 0, nw.data_ptr(), 1e-6, h.data_ptr(), Ns, 2 * Ns, peers.data_ptr(), 0, world, T, 1, status.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(status.item()) == 1 and not h.any().item()
    assert float((x + 1).sum().item()) == 2.0 * T * Ns                 # (the context still runs kernels)
    assert L.cam_tp_rms_norm_f16(T + 1, x.data_ptr(), 0, nw.data_ptr(), 1e-6, h.data_ptr(), Ns, 2 * Ns, peers.data_ptr(), 0, world, T, 1, status.data_ptr(), 0) == -4


def test_q6k_rows(golden):
    """cam_emb_rows_q6k: the fixture's rows (the reference's host decoder) bit for bit, clamped ids; a larger random table against the oracle"""
    f = golden('q6k_rows'); T = f['T']; vocab, nblk = T.shape[:2]; N = nblk * 256
    O = q3m_ops.Ops(DEV)
    toks = np.concatenate([[0, 18, -4, 77], np.random.default_rng(3).integers(0, vocab, 200)]).astype(np.int32)
    x = torch.zeros(len(toks), N, device=DEV)
    O.emb_q6k(cu(T.reshape(-1)), nblk * 210, vocab, cu(toks), x, len(toks), N)
    assert same(x, f['rows'][np.clip(toks, 0, vocab - 1)])
    g_ = np.random.default_rng(8); vocab2, nblk2 = 300, 8
    W = g_.integers(0, 256, (vocab2, nblk2, 210), dtype=np.uint8)
    W[:, :, 208:210] = (g_.standard_normal((vocab2, nblk2, 1)) * 1e-3).astype(np.float16).view(np.uint8).reshape(vocab2, nblk2, 2)
    toks2 = g_.integers(0, vocab2, 1000).astype(np.int32); x2 = torch.zeros(1000, nblk2 * 256, device=DEV)
    O.emb_q6k(cu(W.reshape(-1)), nblk2 * 210, vocab2, cu(toks2), x2, 1000, nblk2 * 256)
    assert same(x2, oracle.emb_rows_q6k(W, nblk2 * 210, vocab2, toks2, nblk2 * 256))
    with pytest.raises(ValueError): O.emb_q6k(cu(W.reshape(-1)), 100, vocab2, cu(toks2), x2, 1000, nblk2 * 256)


def test_iq2s_rows(golden):
    """q35t_emb_iq2s: the fixture's rows (the reference's host decoder over the fixture's grid) bit for bit, clamped ids; a larger random
    table against the oracle; the grid handed over in either form; refused without one"""
    from caminus_b200.prefill import q35own
    from caminus_b200.device import cuda as hip
    f = golden('iq2s_rows'); T = f['T']; vocab, nblk = T.shape[:2]; N = nblk * 256
    O = q35own.Ops(DEV, module=q35own.MODULE_TCAP)
    toks = np.concatenate([[0, 22, -4, 77], np.random.default_rng(3).integers(0, vocab, 200)]).astype(np.int32)
    x = torch.zeros(len(toks), N, device=DEV)
    hip._IQ2S.clear()
    with pytest.raises(RuntimeError): O.emb_iq2s(cu(T.reshape(-1)), nblk * 82, vocab, cu(toks), x, len(toks), N)
    hip.set_iq2s_grid(f['grid'])                                        # the magnitudes, [1024, 8]
    O.emb_iq2s(cu(T.reshape(-1)), nblk * 82, vocab, cu(toks), x, len(toks), N)
    assert same(x, f['rows'][np.clip(toks, 0, vocab - 1)])
    g_ = np.random.default_rng(9); vocab2, nblk2 = 300, 20
    grid2 = np.array([8, 25, 43], np.uint8)[g_.integers(0, 3, (1024, 8))]
    hip.set_iq2s_grid(oracle.pack_iq2s_grid(grid2))                     # the packed words
    W = g_.integers(0, 256, (vocab2, nblk2, 82), dtype=np.uint8)
    W[:, :, 0:2] = (g_.standard_normal((vocab2, nblk2, 1)) * 1e-2).astype(np.float16).view(np.uint8).reshape(vocab2, nblk2, 2)
    toks2 = g_.integers(-3, vocab2 + 3, 1000).astype(np.int32); x2 = torch.zeros(1000, nblk2 * 256, device=DEV)
    O.emb_iq2s(cu(W.reshape(-1)), nblk2 * 82, vocab2, cu(toks2), x2, 1000, nblk2 * 256)
    assert same(x2, oracle.emb_rows_iq2s(W, nblk2 * 82, vocab2, toks2, nblk2 * 256, oracle.pack_iq2s_grid(grid2)))
    for nblk3, n3 in ((8, 20011), (16, 700), (24, 9)):                  # row strides that are multiples of 16 bytes: the staged kernel, several rows per warp
        W3 = g_.integers(0, 256, (vocab2, nblk3, 82), dtype=np.uint8)
        W3[:, :, 0:2] = (g_.standard_normal((vocab2, nblk3, 1)) * 1e-2).astype(np.float16).view(np.uint8).reshape(vocab2, nblk3, 2)
        toks3 = g_.integers(-3, vocab2 + 3, n3).astype(np.int32); x3 = torch.zeros(n3, nblk3 * 256, device=DEV)
        O.emb_iq2s(cu(W3.reshape(-1)), nblk3 * 82, vocab2, cu(toks3), x3, n3, nblk3 * 256)
        assert same(x3, oracle.emb_rows_iq2s(W3, nblk3 * 82, vocab2, toks3, nblk3 * 256, oracle.pack_iq2s_grid(grid2)))
    with pytest.raises(ValueError): O.emb_iq2s(cu(W.reshape(-1)), 100, vocab2, cu(toks2), x2, 1000, nblk2 * 256)
    with pytest.raises(ValueError): q35own.Ops(DEV).emb_iq2s(cu(W.reshape(-1)), nblk2 * 82, vocab2, cu(toks2), x2, 1000, nblk2 * 256)
    with pytest.raises(ValueError): hip.set_iq2s_grid(np.zeros((1024, 8), np.uint8))
