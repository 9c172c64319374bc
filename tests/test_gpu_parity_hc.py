"""GPU parity of the hyper-connection line's glue and the training line's forwards with the CPU oracle: every output byte
equal, on the reference tests' input recipe (N(0, s) with 0.2 % of entries x 30), row counts 1 ... 777 and every glue object
width (tests/prefill/test_prefill_glue.py runs T in {1, 4, 512, 777, 2048})."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip('torch')
pytestmark = pytest.mark.gpu

import oracle   # noqa: E402
from caminus_b200.device import cuda as hip   # noqa: E402
from caminus_b200.prefill import glue as G   # noqa: E402

DEV = 'cuda:0'
I, F, L = ctypes.c_int, ctypes.c_float, ctypes.c_long


def cu(a): return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
def bfz(*s): return torch.zeros(*s, dtype=torch.bfloat16, device=DEV)


def bits(a):
    if torch.is_tensor(a):
        a = a.detach().cpu()
        a = a.view(torch.int16).numpy() if a.dtype == torch.bfloat16 else a.numpy()
    return np.ascontiguousarray(a).view({1: np.uint8, 2: np.uint16, 4: np.uint32}[a.dtype.itemsize]).reshape(-1)


def same(a, b): return np.array_equal(bits(a), bits(b))


def acts(g, shape, scale=1.0):
    x = g.standard_normal(shape) * scale
    x[g.random(shape) < 0.002] *= 30
    return x.astype(np.float32)


@pytest.mark.parametrize('module', ['prefill_glue', 'prefill_glue_q35', 'prefill_glue_q35d'])
@pytest.mark.parametrize('R,wr', [(1, 1), (4, 4), (777, 1), (512, 4)])
def test_rms_mul(module, R, wr):
    gl = G.Glue(DEV, module=module); K = gl.D
    g = np.random.default_rng(R + K)
    x = acts(g, (R, K), 3.0); w = (g.random((wr, K)) + 0.5).astype(np.float32)
    yo, ybfo, sclo = oracle.pf_rms_mul(x, w, 1e-6, K)
    xd = cu(x); y = torch.zeros(R, K, device=DEV); ybf = bfz(R, K); scl = torch.zeros(R, device=DEV)
    gl.rms_mul(xd, cu(w), y, R, 1e-6, ybf=ybf, scale=scl)
    assert same(y, yo) and same(ybf, ybfo) and same(scl, sclo)
    gl.rms_mul(xd, cu(w), xd, R, 1e-6)                                   # in place, y is x; the other outputs omitted
    assert same(xd, yo)
    with pytest.raises(ValueError): gl.rms_mul(xd, cu(w), None, R, 1e-6)  # no output


@pytest.mark.parametrize('T,HC', [(1, 4), (4, 4), (130, 4), (33, 2)])
def test_hc_post_rms_post_mean(T, HC):
    gl = G.Glue(DEV); D = gl.D
    g = np.random.default_rng(T)
    b = acts(g, (T, D)); inj = (g.standard_normal((T, HC)) * 3).astype(np.float32); res = acts(g, (T * HC, D), 2.0)
    w = (g.random((HC, D)) + 0.5).astype(np.float32); gate = (g.standard_normal((T * HC, D)) * 2).astype(np.float32)
    ro, xno, xnbfo, sclo = oracle.pf_hc_post_rms(b, inj, res, w, T, HC, 0.25, 1e-6, D)
    rd = cu(res); xn = torch.zeros(T * HC, D, device=DEV); xnbf = bfz(T * HC, D); scl = torch.zeros(T * HC, device=DEV)
    gl.hc_post_rms(cu(b), cu(inj), rd, cu(w), T, HC, 1e-6, xn=xn, xnbf=xnbf, scale=scl)
    assert same(rd, ro) and same(xn, xno) and same(xnbf, xnbfo) and same(scl, sclo)
    rd2 = cu(res); gl.hc_post(cu(b), cu(inj), rd2, T, HC)
    assert same(rd2, ro)
    out = torch.zeros(T, D, device=DEV)
    gl.hc_mean(xn, cu(gate), out, T, HC)
    mo = oracle.pf_hc_mean(xno, gate, T, HC, D, 0.25)
    assert same(out, mo)
    out2 = torch.zeros(T, D, device=DEV)
    gl.hc_mean(rd, cu(gate), out2, T, HC, scale=scl, w=cu(w))             # the norm recomputed from (res, scale, w): the same bits
    assert same(out2, mo)
    y = acts(g, (T * D,)); a = acts(g, (T * D,)); c = acts(g, (T * D,))
    yd = cu(y); gl.add_sum(cu(a), cu(c), yd, T * D)
    assert same(yd, oracle.pf_add_sum(a, c, y))


def test_bf16_operands_and_swiglu():
    gl = G.Glue(DEV); g = np.random.default_rng(4)
    T, K, ldx = 130, 320, 352
    x = acts(g, (T, ldx), 2.0); Tp = G.tpad(T)
    y = torch.full((Tp, K), 7.0, dtype=torch.bfloat16, device=DEV)
    gl.to_bf16(cu(x), y, T, K, ldx=ldx)
    assert same(y, oracle.pf_to_bf16(x, ldx, T, Tp, K))
    gl.silu_bf16(cu(x), y, T, K, 0.5, ldx=ldx)
    assert same(y, oracle.pf_to_bf16(x, ldx, T, Tp, K, rs=0.5))
    m = hip.Module('prefill_tp')
    gg = acts(g, (5000,), 4.0); uu = acts(g, (5000,)); yy = torch.zeros(5000, device=DEV)
    m.pf_swiglu((20,), (256,), cu(gg), cu(uu), yy, L(5000))
    assert same(yy, oracle.pf_swiglu(gg, uu))


@pytest.mark.parametrize('rows,heads,D,nrot,stride', [(7, 3, 256, 64, 512), (1, 24, 256, 64, 512), (40, 2, 128, 128, 128), (3, 1, 512, 0, 512),
                                                      (64, 4, 256, 256, 256), (10, 6, 128, 8, 132), (500, 16, 256, 0, 256), (9, 2, 256, 136, 260)])   # pairs of heads: both chunks rotated, a rotated range of 8, none, one that ends inside the second chunk
def test_qk_nr(rows, heads, D, nrot, stride):
    g = np.random.default_rng(rows + D)
    x = acts(g, (rows * heads, stride), 1.5); w = (g.random(D) + 0.5).astype(np.float32)
    ts = float(np.float32(np.float32(1e7) ** np.float32(-2.0 / max(nrot, 2)))); pos0 = 1000
    out = torch.zeros(rows * heads, D, device=DEV)
    hip.Module('prefill_attn').pf_qk_nr((rows * heads,), (256,), cu(x), I(stride), I(heads), cu(w), I(D), I(nrot), F(ts), F(1e-6), I(pos0), out)
    assert same(out, oracle.pf_qk_nr(x, stride, heads, w, D, nrot, ts, 1e-6, pos0, rows * heads))


def test_training_line_forwards():
    g = np.random.default_rng(6); n, d, H = 300, 896, 448
    core, fuse = hip.Module('core'), hip.Module('fuse')
    x = acts(g, (n, d)); w = (g.random(d) + 0.5).astype(np.float32)
    out = torch.zeros(n, d, device=DEV)
    core.rmsnorm_f32((n,), (256,), cu(x), cu(w), out, I(d), F(1e-5))
    assert same(out, oracle.rmsnorm_f32(x, w, 1e-5))
    tok = g.integers(0, n, 50).astype(np.int32); eo = torch.zeros(50, d, device=DEV)
    core.embedding_f32((50,), (256,), cu(tok), cu(x), eo, I(d))
    assert same(eo, x[tok])
    m = torch.from_numpy(acts(g, (n, d))).bfloat16().to(DEV); mlp = torch.from_numpy(acts(g, (n, d))).bfloat16().to(DEV)
    r3 = torch.zeros(n * d, device=DEV)
    core.residual3(((n * d + 255) // 256,), (256,), cu(x), m, mlp, r3, ctypes.c_int64(n * d))
    assert same(r3, oracle.residual3(x, bits(m), bits(mlp))) and same(r3, ((cu(x) + m) + mlp))              # torch's own add order
    cb = bfz(n * d); core.cast_bf16(((n * d + 255) // 256,), (256,), cu(x), cb, ctypes.c_int64(n * d))
    assert same(cb, oracle.cast_bf16(x)) and same(cb, cu(x).bfloat16())
    gu = torch.from_numpy(acts(g, (n, 2 * H), 2.0)).bfloat16().to(DEV); act = bfz(n * H)
    core.silu_mul_bf16(((n * H + 255) // 256,), (256,), gu, act, I(H), ctypes.c_int64(n * H))
    assert same(act, oracle.silu_mul_bf16(bits(gu), H))
    ys = torch.from_numpy(acts(g, (40, d))).bfloat16().to(DEV)
    pos = np.full(n, -1, np.int32); pos[g.choice(n, 40, replace=False)] = np.arange(40, dtype=np.int32)
    ro = torch.zeros(n * d, device=DEV); NUL = ctypes.c_void_p(None)
    fuse.residual_slices_fwd(((n * d // 4 + 255) // 256,), (256,), cu(x), m, mlp, ys, cu(pos), ro, I(d), L(n * d // 4))
    assert same(ro, oracle.residual_slices_fwd(x, bits(m), bits(mlp), bits(ys), pos, d))
    fuse.residual_slices_fwd(((n * d // 4 + 255) // 256,), (256,), cu(x), m, mlp, NUL, NUL, ro, I(d), L(n * d // 4))
    assert same(ro, r3)


def specials32():
    """fp32 values the fast evaluations must hand to the exact statements or get right: zeros, denormals, the -8 gate bound, the
    exp clamps, huge values, infinities, NaNs"""
    v = np.array([0.0, -0.0, 1e-45, -1e-45, 1e-39, -3e-39, 2.9e-38, 3.1e-38, -8.0, -8.000001, -7.999999, -20.0, -87.0, -88.5, -104.0, 87.0, 88.0, 89.0,
                  1e30, -1e30, 3.3e38, -3.3e38, np.inf, -np.inf, np.nan, 1.0, -1.0, 0.5, 65504.0], np.float32)
    nan2 = np.array([0x7fa00001, 0xffc12345, 0x7f800001], np.uint32).view(np.float32)       # signalling and payload NaNs
    return np.concatenate([v, nan2])


def same_but_nan(a, b):
    """bit-equal where the oracle's value is a number; where it is a NaN the device's must be one too (the payload of a computed NaN
    is the arithmetic unit's: 0x7fffffff on this device, the operand's quieted payload on the CPU)"""
    a, b = bits(a), bits(b)
    if a.dtype == np.uint32: na, nb = (a & 0x7fffffff) > 0x7f800000, (b & 0x7fffffff) > 0x7f800000
    else: na, nb = (a & 0x7fff) > 0x7f80, (b & 0x7fff) > 0x7f80
    return np.array_equal(na, nb) and np.array_equal(a[~nb], b[~nb])


def test_silu_mul_bf16_every_gate():
    """every one of the 65536 bf16 gate patterns through the vector kernel (its proof-or-exact rounding), against a few ups"""
    core = hip.Module('core'); H = 65536
    gpat = np.arange(H, dtype=np.uint16); g = np.random.default_rng(40)
    ups = [np.full(H, 0x3f80, np.uint16), (g.standard_normal(H) * 2).astype(np.float32).view(np.uint32) >> 16,
           np.resize(np.array([0x7f80, 0xff80, 0x7fc0, 0x0000, 0x8000, 0x0001, 0x7f7f, 0xc2f0], np.uint16), H)]
    gu = np.concatenate([np.concatenate([gpat, np.asarray(u, np.uint16)]) for u in ups]).reshape(3, 2 * H)
    gd = torch.from_numpy(gu.view(np.int16)).to(DEV).view(torch.bfloat16); act = bfz(3 * H)
    core.silu_mul_bf16(((3 * H + 255) // 256,), (256,), gd, act, I(H), ctypes.c_int64(3 * H))
    assert same(act, oracle.silu_mul_bf16(gu, H))
    n = 2 * H + 1000                                                       # whole rows by vectors, the partial third row by elements
    act2 = bfz(3 * H)
    core.silu_mul_bf16(((n + 255) // 256,), (256,), gd, act2, I(H), ctypes.c_int64(n))
    assert same(act2[:n], bits(act)[:n]) and not bits(act2)[n:].any()
    H2 = 100                                                               # a row length the vector kernel does not take
    gu2 = gu.reshape(-1)[:40 * 2 * H2].copy(); a3 = bfz(40 * H2)
    core.silu_mul_bf16(((40 * H2 + 255) // 256,), (256,), torch.from_numpy(gu2.view(np.int16)).to(DEV).view(torch.bfloat16), a3, I(H2), ctypes.c_int64(40 * H2))
    assert same(a3, oracle.silu_mul_bf16(gu2, H2))


@pytest.mark.parametrize('T,K,ldx,rs', [(1500, 1024, 1024, 1.0), (700, 896, 1000, 0.5), (130, 322, 322, 0.25)])
def test_bf16_operands_hard_inputs(T, K, ldx, rs):
    """pf_silu_bf16 / pf_to_bf16 on wide-ranging inputs and the special values: dense rows, strided rows, a width without the vector path"""
    gl = G.Glue(DEV); g = np.random.default_rng(T)
    x = (g.standard_normal((T, ldx)) * np.exp(g.uniform(-6, 4, (T, ldx)))).astype(np.float32)
    sp = specials32()
    with np.errstate(all='ignore'):
        x.reshape(-1)[: 40 * sp.size] = np.tile(sp, 40) / np.float32(rs) * np.repeat(np.linspace(0.999, 1.001, 40, dtype=np.float32), sp.size)
    x.reshape(-1)[40 * sp.size: 41 * sp.size] = sp
    Tp = G.tpad(T); y = torch.full((Tp, K), 7.0, dtype=torch.bfloat16, device=DEV)
    gl.silu_bf16(cu(x), y, T, K, rs, ldx=ldx)
    assert same_but_nan(y, oracle.pf_to_bf16(x, ldx, T, Tp, K, rs=rs))
    y.fill_(7.0); gl.to_bf16(cu(x), y, T, K, ldx=ldx)
    assert same(y, oracle.pf_to_bf16(x, ldx, T, Tp, K))


def test_elementwise_tails_and_unaligned():
    """the four-element kernels with n % 4 != 0 and the special values; buffers offset by one element take the element kernels"""
    g = np.random.default_rng(41); n = 4 * 70001 + 3; sp = specials32()
    core, tp, gl = hip.Module('core'), hip.Module('prefill_tp'), G.Glue(DEV)
    a = acts(g, (n + 1,), 3.0); b = acts(g, (n + 1,)); c = acts(g, (n + 1,))
    a[: sp.size] = sp; a[-sp.size:] = sp; b[5: 5 + sp.size] = sp
    mb = torch.from_numpy(b).bfloat16().to(DEV); lb = torch.from_numpy(c).bfloat16().to(DEV)
    grid = ((n + 255) // 256,)
    for off in (0, 1):
        av, bv, cv = a[off: off + n], b[off: off + n], c[off: off + n]
        ad, bd = cu(a)[off: off + n], cu(b)[off: off + n]
        y = cu(c)[off: off + n]
        gl.add_sum(ad, bd, y, n)
        assert same_but_nan(y, oracle.pf_add_sum(av, bv, cv))
        out = torch.zeros(n + 1, device=DEV)[off: off + n]
        tp.pf_swiglu(grid, (256,), ad, bd, out, L(n))
        assert same_but_nan(out, oracle.pf_swiglu(av, bv))
        core.residual3(grid, (256,), ad, mb[off: off + n], lb[off: off + n], out, ctypes.c_int64(n))
        assert same_but_nan(out, oracle.residual3(av, bits(mb)[off: off + n], bits(lb)[off: off + n]))
        cb = bfz(n + 1)[off: off + n]
        core.cast_bf16(grid, (256,), ad, cb, ctypes.c_int64(n))
        assert same(cb, oracle.cast_bf16(av))


@pytest.mark.parametrize('rows,d', [(1000, 512), (600, 1024), (400, 3584), (333, 4096), (300, 704), (20, 896)])
def test_rmsnorm_f32_row_lengths(rows, d):
    """the warp-per-row path (multiples of 128 with enough rows) and the block-per-row path give the oracle's bits"""
    g = np.random.default_rng(d); x = acts(g, (rows, d), 2.0); w = (g.random(d) + 0.5).astype(np.float32)
    out = torch.zeros(rows, d, device=DEV)
    hip.Module('core').rmsnorm_f32((rows,), (256,), cu(x), cu(w), out, I(d), F(1e-5))
    assert same(out, oracle.rmsnorm_f32(x, w, 1e-5))


def test_embedding_f32_and_qk_nr_other_paths():
    g = np.random.default_rng(42); core = hip.Module('core')
    for V, d, T in ((500, 896, 3000), (64, 30, 100)):
        emb = acts(g, (V, d)); tok = g.integers(0, V, T).astype(np.int32); eo = torch.zeros(T, d, device=DEV)
        core.embedding_f32((T,), (256,), cu(tok), cu(emb), eo, I(d))
        assert same(eo, emb[tok])
    for rows, heads, D, nrot, stride in ((300, 16, 256, 64, 256), (50, 5, 384, 384, 400), (9, 2, 130, 64, 131), (64, 8, 64, 32, 64), (33, 4, 512, 512, 512), (17, 3, 128, 20, 128), (21, 2, 256, 250, 260)):
        x = acts(g, (rows * heads, stride), 1.5); w = (g.random(D) + 0.5).astype(np.float32)
        ts = float(np.float32(np.float32(1e6) ** np.float32(-2.0 / nrot))); pos0 = 70000
        out = torch.zeros(rows * heads, D, device=DEV)
        hip.Module('prefill_attn').pf_qk_nr((rows * heads,), (256,), cu(x), I(stride), I(heads), cu(w), I(D), I(nrot), F(ts), F(1e-6), I(pos0), out)
        assert same(out, oracle.pf_qk_nr(x, stride, heads, w, D, nrot, ts, 1e-6, pos0, rows * heads)), (rows, heads, D, nrot)


@pytest.mark.parametrize('layout', ['D4', 'DS4'])
@pytest.mark.parametrize('rows,K', [(1, 128), (37, 768), (150, 2560), (9, 300)])
def test_mmq_q8_1(layout, rows, K):
    """the MMQ-layout quantiser and its fused SwiGLU form: the oracle's bytes (tests/prefill/test_prefill_moe.py:135 gates the
    reference's fused bytes against its unfused path the same way)"""
    from caminus_b200.engine import gguf
    g = np.random.default_rng(rows + K); lay = gguf.MMQ_LAYOUTS[layout]; Kp = (K + 127) // 128 * 128
    x = acts(g, (rows, K), 0.7); u = acts(g, (rows, K))
    if rows > 1: x[1, :32] = 0
    assert same(gguf.quantize_mmq_q8_1(cu(x), layout), oracle.mmq_q8_1(x, K, Kp, lay))
    assert same(gguf.quantize_mmq_q8_1(cu(x), layout, u=cu(u)), oracle.mmq_q8_1(x, K, Kp, lay, u=u))
    xh, uh = x.astype(np.float16), u.astype(np.float16)
    fused = gguf.quantize_mmq_q8_1(cu(xh), layout, u=cu(uh))
    assert same(fused, oracle.mmq_q8_1(xh, K, Kp, lay, u=uh))
    # fused == unfused: silu(g) * u written as fp32 by pf_swiglu's statements, then the plain quantiser
    h = oracle.swiglu_f32_from_f16(xh.reshape(-1), uh.reshape(-1)).reshape(rows, K)
    assert same(fused, gguf.quantize_mmq_q8_1(cu(h), layout))


@pytest.mark.parametrize('layout', ['D4', 'DS4'])
@pytest.mark.parametrize('rows,K,pad', [(5, 384, 0), (40, 5120, 0), (7, 640, 4), (6, 300, 0), (9, 1024, 8)])
def test_mmq_q8_1_ties_and_specials(layout, rows, K, pad):
    """the plain MMQ quantiser on quotients that sit on .5 (roundf rounds them away from zero, the device's add-a-large-number rounding
    to even: those lanes take the reference's statements), NaN, infinities, a maximum so small that 127 / amax overflows, zero groups;
    rows 32-byte aligned (256-bit loads) and not (row stride K + 4)"""
    from caminus_b200.engine import gguf
    rng = np.random.default_rng(rows + K + pad); lay = gguf.MMQ_LAYOUTS[layout]; Kp = (K + 127) // 128 * 128
    full = np.zeros((rows, K + pad), np.float32); x = full[:, :K]
    x[:] = acts(rng, (rows, K), 0.7)
    x[0, :32] = np.arange(32, dtype=np.float32) - 15.5; x[0, 0] = 127.0            # amax 127: the quotients are the values, halves are ties
    x[0, 32:64] = (rng.integers(-126, 126, 32).astype(np.float32) + 0.5) / 8; x[0, 40] = 127.0 / 8
    x[1, 64:96] = np.round(x[1, 64:96] * 40) / 2; x[1, 70] = 63.5                  # amax 63.5: the quotients are twice the values
    if rows > 2: x[2, 5] = np.nan; x[2, 40] = np.inf; x[2, 64:96] = 0; x[2, 100] = -np.inf; x[2, 130] = 3e38
    if rows > 3: x[3, :32] = 1e-42; x[3, 32:64] *= 1e-38; x[3, 64:96] = -0.0
    got = gguf.quantize_mmq_q8_1(cu(full)[:, :K], layout)
    want = oracle.mmq_q8_1(np.ascontiguousarray(x), K, Kp, lay)
    if layout == 'DS4':                                                            # (a NaN sum has the arithmetic unit's payload)
        gb, wb = bits(got).reshape(-1, 144), bits(want).reshape(-1, 144)
        gh, wh = gb[:, :16].copy().view(np.uint16), wb[:, :16].copy().view(np.uint16)
        nan = (wh & 0x7fff) > 0x7c00
        assert np.array_equal(gb[:, 16:], wb[:, 16:]) and np.array_equal(gh[~nan], wh[~nan]) and ((gh[nan] & 0x7fff) > 0x7c00).all()
    else: assert same(got, want)


@pytest.mark.parametrize('layout', ['D4', 'DS4'])
@pytest.mark.parametrize('dt', [np.float16, np.float32])
@pytest.mark.parametrize('rows,K,kvalid', [(1, 128, 128), (3, 384, 384), (6, 640, 592), (13, 1024, 1024), (5, 896, 888), (64, 2560, 2560)])
def test_swiglu_mmq_hard_inputs(layout, dt, rows, K, kvalid):
    """the D4 and DS4 fast passes: every byte is the exact statements' byte on inputs built to sit on its margins: duplicated and nearly
    equal maxima, products on rounding boundaries, gates below -8, zero groups, tiny and huge values, NaN and infinities; odd
    K-block counts, row counts that do not fill a warp's four rows, kvalid below K"""
    from caminus_b200.engine import gguf
    rng = np.random.default_rng(rows * 7 + K)
    g = acts(rng, (rows, K), 1.5).astype(dt); u = acts(rng, (rows, K)).astype(dt)
    r = np.arange(rows)
    g[r, (r * 37) % K] = -9.5; g[r, (r * 11 + 5) % K] = 30.0
    g[:, 32:40] = g[:, 40:48]; u[:, 32:40] = u[:, 40:48]                        # every value of these lanes twice: duplicated maxima
    if K >= 384: g[:, 256:288] = 0; u[:, 300:310] = 0                          # a zero group
    if K >= 640:
        g[:, 512:544] = (g[:, 512:544].astype(np.float32) * 1e-3).astype(dt); u[:, 512:544] = (u[:, 512:544].astype(np.float32) * 1e-3).astype(dt)
        u[:, 544:576] = 60000.0 if dt == np.float16 else 1e30
    if rows > 2: g[2, 70] = np.nan; u[2, 100] = np.inf; g[1, 3] = np.inf
    if dt == np.float32 and rows > 4: g[4, 200 % K] = 1e-40; u[4, 200 % K] = 3e38; g[3, :64] *= 1e-20
    # halves of the maximum: codes on the .5 boundaries
    h = oracle.swiglu_f32_from_f16(g.reshape(-1), u.reshape(-1)).reshape(rows, K) if dt == np.float16 else None
    Kp = (K + 127) // 128 * 128
    got = gguf.quantize_mmq_q8_1(cu(g), layout, u=cu(u), kvalid=kvalid)
    want = oracle.mmq_q8_1(g, kvalid, Kp, gguf.MMQ_LAYOUTS[layout], u=u)
    if layout == 'DS4':                                                            # (a NaN sum or scale has the arithmetic unit's payload)
        gb, wb = bits(got).reshape(-1, 144), bits(want).reshape(-1, 144)
        gh, wh = gb[:, :16].copy().view(np.uint16), wb[:, :16].copy().view(np.uint16)
        nan = (wh & 0x7fff) > 0x7c00
        assert np.array_equal(gb[:, 16:], wb[:, 16:]) and np.array_equal(gh[~nan], wh[~nan]) and ((gh[nan] & 0x7fff) > 0x7c00).all()
    else: assert same(got, want)
    if h is not None and kvalid == K and not np.isnan(h).any(): assert same(got, gguf.quantize_mmq_q8_1(cu(h), layout))


@pytest.mark.parametrize('layout', ['D4', 'DS4'])
def test_swiglu_mmq_fast_equals_unfused_large(layout):
    """2048 x 25600 fp16 values: the fused D4 / DS4 blocks equal the plain quantiser's over gg_silu_mul's fp32 products (both the exact
    statements for every value), byte for byte"""
    from caminus_b200.engine import gguf
    gen = torch.Generator(device=DEV); gen.manual_seed(5)
    T, K = 2048, 25600
    g = (torch.randn(T, K, device=DEV, generator=gen) * 1.5).half(); u = torch.randn(T, K, device=DEV, generator=gen).half()
    fused = gguf.quantize_mmq_q8_1(g, layout, u=u)
    h = gguf.silu_mul(g.float().reshape(-1), u.float().reshape(-1)).reshape(T, K)
    assert torch.equal(fused, gguf.quantize_mmq_q8_1(h, layout))


@pytest.mark.parametrize('layout', [0, 1])
def test_mmq_quantize_ids_and_scatter(layout):
    """Mmq.quantize with a row index and Mmq.quantize_scatter: every column holds the oracle's block of the row it names
    (the reference runs both forms through its MMQ and compares the products, tests/prefill/test_prefill_mmq.py:226-233)"""
    from caminus_b200.prefill import mmq
    g = np.random.default_rng(31 + layout); ntok, k, K, s01 = 37, 4, 600, 640
    M = mmq.Mmq(DEV); Kp = mmq.k_pad(K)
    x = acts(g, (ntok * k, s01), 2.0); x[3, :40] = 0
    plain = oracle.mmq_q8_1(x, K, Kp, layout)                                   # [Kp / 128, rows, 144] of the rows in order
    xd = cu(x.reshape(-1))
    def run(fn, ncols):
        y = torch.zeros(mmq.y_bytes(K, ncols), dtype=torch.uint8, device=DEV); fn(y)
        return y[:Kp // 128 * ncols * 144].cpu().numpy().reshape(Kp // 128, ncols, 144)
    ncols = ntok * k
    assert np.array_equal(run(lambda y: M.quantize(xd, K, ncols, y, layout, s01=s01), ncols), plain)
    ids = g.permutation(ncols).astype(np.int32); idd = cu(ids)
    assert np.array_equal(run(lambda y: M.quantize(xd, K, ncols, y, layout, s01=s01, ids=idd), ncols), plain[:, ids])
    inv = g.permutation(ncols).astype(np.int32); invd = cu(inv)                # token t's k columns
    got = run(lambda y: M.quantize_scatter(xd, K, ntok, invd, k, y, layout, s_tok=s01), ncols)
    want = np.zeros_like(got)
    for t in range(ntok): want[:, inv[t * k:(t + 1) * k]] = plain[:, t:t + 1]
    assert np.array_equal(got, want)
    with pytest.raises(ValueError): M.quantize(xd, K + 2, ncols, torch.zeros(mmq.y_bytes(K, ncols), dtype=torch.uint8, device=DEV), layout)
    with pytest.raises(ValueError): M.quantize(xd, K, ncols, torch.zeros(100, dtype=torch.uint8, device=DEV), layout)


@pytest.mark.parametrize('layout', [0, 1])
@pytest.mark.parametrize('dt', [np.float16, np.float32])
@pytest.mark.parametrize('ncols,K,s01', [(37, 600, 640), (150, 2560, 2560), (5, 128, 128), (64, 1000, 1008)])
def test_swiglu_mmq_with_a_row_index(layout, dt, ncols, K, s01):
    """Mmq.swiglu_quantize: the fused SwiGLU blocks gathered through a row index: column c holds the oracle's block of row ids[c]
    (with and without an index, aligned rows on the fast pass and odd strides on the exact kernel, ids out of range clamped)"""
    from caminus_b200.prefill import mmq
    g = np.random.default_rng(ncols + K + layout); M = mmq.Mmq(DEV); Kp = mmq.k_pad(K)
    gt = acts(g, (ncols, s01), 1.5).astype(dt); up = acts(g, (ncols, s01)).astype(dt)
    gt[1, :40] = 0; gt[2 % ncols, 5] = -9.5
    plain = oracle.mmq_q8_1(gt, K, Kp, layout, u=up)                             # [Kp / 128, rows, 144] of the rows in order
    gd, ud = cu(gt.reshape(-1)), cu(up.reshape(-1))
    def run(ids):
        y = torch.zeros(mmq.y_bytes(K, ncols), dtype=torch.uint8, device=DEV)
        M.swiglu_quantize(gd, ud, K, ncols, y, layout, s01=s01, ids=ids)
        return y[:Kp // 128 * ncols * 144].cpu().numpy().reshape(Kp // 128, ncols, 144)
    assert np.array_equal(run(None), plain)
    ids = g.permutation(ncols).astype(np.int32); ids[0] = ids[-1]                # a row used twice
    assert np.array_equal(run(cu(ids)), plain[:, ids])
    wild = ids.copy(); wild[1 % ncols] = -4; wild[2 % ncols] = ncols + 9
    assert np.array_equal(run(cu(wild)), plain[:, np.clip(wild, 0, ncols - 1)])
    with pytest.raises(ValueError): M.swiglu_quantize(gd, ud, K + 2, ncols, torch.zeros(mmq.y_bytes(K, ncols), dtype=torch.uint8, device=DEV), layout)
    with pytest.raises(ValueError): M.swiglu_quantize(gd, ud.float() if dt == np.float16 else ud.half(), K, ncols, torch.zeros(mmq.y_bytes(K, ncols), dtype=torch.uint8, device=DEV), layout)


@pytest.mark.parametrize('M,K', [(1, 128), (37, 896), (300, 1024), (5, 8192), (20, 2048), (9, 4096), (3, 384), (11, 4224), (6, 2304), (70, 6144)])
def test_actq_family(M, K):
    """actq_fwd_*, silu_mul_actq_fwd, block_entry_fwd: values, scales and packed codes are the oracle's bytes; silu extremes and a
    row-strided view as tests/train/test_silu_mul_actq.py:21-47"""
    from caminus_b200.train import actq as A
    g = np.random.default_rng(M + K)
    x = acts(g, (M, K), 2.0)
    xs = x.copy()
    if M >= 5: xs[1] = 0; xs[2, 3] = np.inf; xs[3, 5] = np.nan; xs[4] *= 1e-20      # a zero row, rows with an infinity / a NaN, a tiny row
    for xin in (cu(xs), cu(xs).bfloat16()):
        y, c, s = A.actq_codes(xin, 4, 1.0)
        ref = xs if xin.dtype == torch.float32 else bits(xin).reshape(M, K)
        yo, so, co = oracle.actq_fwd(ref, 1.0, 7)
        assert same(y, yo) and same(s, so) and np.array_equal(c.cpu().numpy().view(np.uint16).reshape(-1), co.reshape(-1))
        assert same(A.actq(xin, 4, 1.0), yo)
        for nbits, clip in ((3, 1.5), (4, 0.7), (2, 1.0)):           # clips on both sides of 1 (above it no quotient passes qmax), other code widths
            y, c, s = A.actq_codes(xin, nbits, clip)
            yo2, so2, co2 = oracle.actq_fwd(ref, clip, 2 ** (nbits - 1) - 1)
            assert same(y, yo2) and same(s, so2) and np.array_equal(c.cpu().numpy().view(np.uint16).reshape(-1), co2.reshape(-1))
    wide = torch.from_numpy(acts(g, (M, 2 * K + 64), 2.0)).bfloat16().to(DEV)
    wide[0, :8] = torch.tensor([30, -30, 0, -0.0, 1e-3, -88, 88, 3]).bfloat16()
    gu = wide[:, :2 * K]                                              # a row-strided view
    y, c, s = A.silu_mul_actq(gu, 4, 0.9)
    yo, so, co = oracle.silu_mul_actq_fwd(bits(wide.cpu()).reshape(M, -1), K, 0.9, 7)
    assert same(y, yo) and same(s, so) and np.array_equal(c.cpu().numpy().view(np.uint16).reshape(-1), co.reshape(-1))
    y, c, s = A.silu_mul_actq(wide[:, 64:], 4, 1.0)                   # (16-byte aligned rows of the same stride, no clamp)
    yo, so, co = oracle.silu_mul_actq_fwd(bits(wide[:, 64:].contiguous().cpu()).reshape(M, -1), K, 1.0, 7)
    assert same(y, yo) and same(s, so) and np.array_equal(c.cpu().numpy().view(np.uint16).reshape(-1), co.reshape(-1))
    if K <= 1024:
        nw = (g.random(K) + 0.5).astype(np.float32); wab = torch.from_numpy(acts(g, (6, K), 0.05)).bfloat16().to(DEV)
        for w_ in (wab, None):
            y, c, s, ab, rstd = A.block_entry(cu(x), cu(nw), w_, 1e-6, 4, 1.0)
            yo, so, co, abo, ro = oracle.block_entry_fwd(x, nw, None if w_ is None else bits(w_).reshape(6, K), 1e-6, 1.0, 7)
            assert same(y, yo) and same(s, so) and same(rstd, ro) and np.array_equal(c.cpu().numpy().view(np.uint16).reshape(-1), co.reshape(-1))
            if w_ is not None: assert same(ab, abo)
        # an odd number of projections (the wrapper takes even counts as upstream; the entry itself takes any up to 16)
        import ctypes
        from caminus_b200.device import cuda as hip
        w5 = torch.from_numpy(acts(g, (5, K), 0.05)).bfloat16().to(DEV); xd = cu(x); nwd = cu(nw)
        y5 = torch.empty(M, K, dtype=torch.bfloat16, device=DEV); s5 = torch.empty(M, device=DEV); c5 = torch.empty(M, K // 4, dtype=torch.int16, device=DEV)
        ab5 = torch.empty(M, 5, dtype=torch.bfloat16, device=DEV); r5 = torch.empty(M, device=DEV)
        hip.Module('actq').block_entry_fwd((M,), (256,), xd, nwd, w5, ctypes.c_int(5), ctypes.c_float(1e-6), y5, s5, c5, ab5, r5, ctypes.c_int(K), ctypes.c_float(1.0), ctypes.c_int(7))
        yo, so, co, abo, ro = oracle.block_entry_fwd(x, nw, bits(w5).reshape(5, K), 1e-6, 1.0, 7)
        assert same(y5, yo) and same(s5, so) and same(r5, ro) and same(ab5, abo)


def test_router_topk_group():
    """the router glue: logits, ids and weights are the oracle's bytes; the grouping puts every pair once under its expert
    (tests/prefill/test_q3m_ops.py:118-129, 165-182)"""
    from caminus_b200.prefill import q3m_ops
    O = q3m_ops.Ops(DEV); g = np.random.default_rng(21); n, D, E, k = 150, 2048, 128, 8
    hh = g.standard_normal((n, D)).astype(np.float32); Wr = (g.standard_normal((E, D)) * 0.05).astype(np.float32)
    lg = torch.zeros(n, E, device=DEV)
    O.router(cu(hh), cu(Wr), E, D, lg, n)
    lo = oracle.router(hh, Wr)
    assert same(lg, lo)
    for n2, E2, D2 in ((5, 128, 2048), (70, 61, 256), (64, 4, 128), (1, 128, 2048), (63, 13, 384), (2, 1, 128)):          # few tokens (a block per token); tiles that overhang n and E
        h2 = g.standard_normal((n2, D2)).astype(np.float32); W2 = g.standard_normal((E2, D2)).astype(np.float32)
        l2 = torch.zeros(n2, E2, device=DEV); hd, wd = cu(h2), cu(W2)
        O.router(hd, wd, E2, D2, l2, n2)
        assert same(l2, oracle.router(h2, W2))
    lo[3, 7] = lo[3, 9] = lo[3].max() + 1.0
    ids = torch.zeros(n * k, dtype=torch.int32, device=DEV); wts = torch.zeros(n * k, device=DEV); err = torch.zeros(1, dtype=torch.int32, device=DEV)
    O.topk(cu(lo), E, k, 6.103515625e-5, ids, wts, err, n)
    io, wo, eo = oracle.topk(lo, k, 6.103515625e-5)
    assert int(err.item()) == 0 == eo and np.array_equal(ids.cpu().numpy().reshape(n, k), io) and same(wts, wo)
    lo[5, 2] = np.nan; err.zero_()
    O.topk(cu(lo), E, k, 6.103515625e-5, ids, wts, err, n)
    assert int(err.item()) & 1
    from caminus_b200.engine import k3
    with pytest.raises(k3.ContextBoundsError): O.check_flags(err)                   # the host's reading of the flag word: raises and clears
    assert int(err.item()) == 0
    O.check_flags(err)
    use = g.choice(E, 12, replace=False)
    ids_np = np.stack([g.choice(use, k, replace=False) for _ in range(n)]).astype(np.int32)
    _group_case(O, ids_np.reshape(-1), k, E)
    bad = ids_np.reshape(-1).copy(); bad[10] = E + 5; bad[77] = -3
    assert _group_case(O, bad, k, E) & 2


def _group_case(O, ids_np, k, E):
    """one grouping launch held to the oracle on every word: xs, yd, the items and their count, the error word (returned)"""
    from caminus_b200.prefill import q3m_ops
    npairs = ids_np.size; bound = q3m_ops.items_bound(npairs, E)
    xs, yd = (torch.full((max(npairs, 1),), -7, dtype=torch.int32, device=DEV) for _ in range(2))
    items = torch.full((bound + 1, 4), -7, dtype=torch.int32, device=DEV); nitems = torch.full((1,), -7, dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    idd = cu(ids_np) if npairs else torch.zeros(1, dtype=torch.int32, device=DEV)
    O.group(idd, npairs, k, E, xs, yd, items, nitems, err)
    xo, yo, io, eo = oracle.group(ids_np, k, E)
    ni = int(nitems.item())
    assert ni == len(io) <= bound and int(err.item()) == eo
    assert np.array_equal(xs.cpu().numpy()[:npairs], xo) and np.array_equal(yd.cpu().numpy()[:npairs], yo)
    assert np.array_equal(items.cpu().numpy()[:ni], io) and (items.cpu().numpy()[ni:] == -7).all()      # nothing written past the count
    return int(err.item())


@pytest.mark.parametrize('npairs,k,E', [(0, 8, 128), (1, 8, 128), (31, 1, 7), (65536, 8, 128), (65537, 8, 1024), (8191, 7, 1000),
                                        (200000, 8, 128), (300001, 10, 256), (4096, 8, 1)])
def test_group_sizes(npairs, k, E):
    """the grouping over its launch shapes: no pair, one pair, odd counts, one to eight blocks in the cluster, runs longer than the
    eight steps a warp keeps in registers, 1 to 1024 experts, lists skewed to a few experts and lists that stay empty"""
    from caminus_b200.prefill import q3m_ops
    O = q3m_ops.Ops(DEV); g = np.random.default_rng(npairs + E)
    ids = g.integers(0, E, npairs).astype(np.int32)
    if npairs > 100: ids[g.random(npairs) < 0.5] = E // 3                       # half of all pairs under one expert: hundreds of items for it
    if E > 16: ids[ids == 5] = 6                                                 # an expert nobody routes to
    assert _group_case(O, ids, k, E) == 0
    assert _group_case(O, ids, k, E) == 0                                        # and again: nothing is carried between launches


@pytest.mark.parametrize('T,E,k', [(777, 256, 10), (5, 128, 8), (64, 1000, 64), (33, 33, 5), (2048, 512, 12), (9, 1024, 33), (3, 8, 8)])
def test_pf_router(T, E, k):
    """the hyper-connection line's softmax + top-k (a warp per token here, a workgroup per token in the reference): ids and weights are
    the oracle's bytes, with exact ties, equal rows and a row of large logits; a row with a logit that is not finite sets bit 0 and
    still carries k distinct experts below E"""
    gl = G.Glue(DEV); g = np.random.default_rng(T + E + k)
    lg = (g.standard_normal((T, E)) * 3).astype(np.float32)
    lg[0, min(7, E - 1)] = lg[0, 2] = lg[0].max() + 1.0; lg[1, :] = 0.5; lg[2] *= 40
    ids = torch.full((T, k), -1, dtype=torch.int32, device=DEV); wts = torch.zeros(T, k, device=DEV); err = torch.zeros(1, dtype=torch.int32, device=DEV)
    gl.router(cu(lg), T, E, k, ids, wts, err)
    io, wo, eo = oracle.pf_router(lg, k, 6.103515625e-5)
    assert int(err.item()) == 0 == eo and np.array_equal(ids.cpu().numpy(), io) and same(wts, wo)
    if T > 4:
        lg[3, 1] = np.nan; lg[4, 0] = -np.inf
        gl.router(cu(lg), T, E, k, ids, wts, err)
        got = ids.cpu().numpy()
        assert int(err.item()) == 1 and all(len(set(r.tolist())) == k and r.min() >= 0 and r.max() < E for r in got)
        keep = np.ones(T, bool); keep[3:5] = False
        assert np.array_equal(got[keep], io[keep]) and same(wts[torch.from_numpy(keep).to(DEV)], wo[keep])
    with pytest.raises(ValueError): gl.router(cu(lg), T, E, E + 1, ids, wts, err)
    with pytest.raises(ValueError): gl.router(cu(lg), T, E, k, ids[:-1], wts, err)


def test_iq4_row_gathers(golden):
    f = golden('iq4_rows'); T, R = f['T'], f['R']; vocab, nblk = T.shape[:2]; nuniq, bpr = R.shape[:2]
    m = hip.Module('prefill_feed'); g = np.random.default_rng(1)
    tok = np.concatenate([[0, 22, 99, -1], g.integers(0, vocab, 300)]).astype(np.int32)
    out = torch.zeros(len(tok), nblk * 256, device=DEV); err = torch.zeros(1, dtype=torch.int32, device=DEV)
    m.embd_rows_iq4xs((1,), (256,), cu(T.reshape(-1)), cu(tok), I(vocab), I(len(tok)), I(nblk), out, err)
    oo, eo = oracle.embd_rows_iq4xs(T, tok, vocab, nblk)
    assert same(out, oo) and int(err.item()) == eo == 2 and same(out, f['xs'][np.clip(tok, 0, vocab - 1)])
    inv = np.concatenate([[3, 11, -2], g.integers(0, nuniq, 200)]).astype(np.int32)
    out = torch.zeros(len(inv), bpr * 32, device=DEV); err.zero_()
    m.ple_rows_iq4nl((1,), (256,), cu(R.reshape(-1)), cu(inv), I(nuniq), I(len(inv)), I(bpr), out, err)
    oo, eo = oracle.ple_rows_iq4nl(R, inv, nuniq, bpr)
    assert same(out, oo) and int(err.item()) == eo == 1 and same(out, f['nl'][np.clip(inv, 0, nuniq - 1)])
    # tables at odd addresses take the byte-wise kernels: the same floats
    Tb = torch.zeros(T.size + 16, dtype=torch.uint8, device=DEV); Tb[4:4 + T.size] = cu(T.reshape(-1))
    o2 = torch.zeros(len(tok), nblk * 256, device=DEV)
    m.embd_rows_iq4xs((1,), (256,), Tb[4:], cu(tok), I(vocab), I(len(tok)), I(nblk), o2, err)
    assert same(o2, f['xs'][np.clip(tok, 0, vocab - 1)])
    Rb = torch.zeros(R.size + 16, dtype=torch.uint8, device=DEV); Rb[1:1 + R.size] = cu(R.reshape(-1))
    o3 = torch.zeros(len(inv), bpr * 32, device=DEV)
    m.ple_rows_iq4nl((1,), (256,), Rb[1:], cu(inv), I(nuniq), I(len(inv)), I(bpr), o3, err)
    assert same(o3, f['nl'][np.clip(inv, 0, nuniq - 1)])


@pytest.mark.parametrize('R,K,wr', [(5, 2560, 1), (300, 2048, 4), (7, 320, 1), (1000, 2560, 1), (601, 5120, 2)])
def test_rms_mul_q8_1_copy(R, K, wr):
    """the norm that also emits the Q8_1 copy: the bytes of the plain quantiser run on the normed rows (fused == unfused)"""
    from caminus_b200 import lib
    g = np.random.default_rng(R + K); x = acts(g, (R, K), 3.0); w = (g.random((wr, K)) + 0.5).astype(np.float32)
    x[R // 2] = 0; x[R // 3, 64:96] = 0; x[R // 4, 5] = 1e15; x[R - 1, :32] *= 1e-30       # a zero row, a zero block, a dominated row, a tiny block
    y = torch.zeros(R, K, device=DEV); yq = torch.zeros(R * K // 32 * 36, dtype=torch.uint8, device=DEV)
    xd, wd = cu(x), cu(w)      # (kept alive until the launch has run)
    lib.check(lib.load().cam_rms_mul_q8_1(xd.data_ptr(), wd.data_ptr(), y.data_ptr(), yq.data_ptr(), R, wr, 1e-6, K, torch.cuda.current_stream().cuda_stream))
    yo, _, _ = oracle.pf_rms_mul(x, w, 1e-6, K)
    assert same(y, yo) and same(yq, oracle.q8_1(yo.reshape(-1), sum_order=0))
