"""Pins for the oracle's hyper-connection and training-line restatements, against what the reference's own tests hold them to:
float64 expressions within its published bounds, bf16 copies equal to torch's round-to-nearest-even cast
(tests/prefill/test_prefill_glue.py:264), and torch's own fp32 / bf16 promotion and add order for the training-line ops
(kernels/core.hip, kernels/fuse.hip reproduce "the PyTorch op the training forward runs", bit for bit)."""
import numpy as np
import pytest

import oracle

torch = pytest.importorskip('torch')


def acts(g, shape, scale=1.0):
    """tests/prefill/test_prefill_glue.py:125-128: N(0, scale) with 0.2 % of the entries x 30"""
    x = g.standard_normal(shape) * scale
    x[g.random(shape) < 0.002] *= 30
    return x.astype(np.float32)


def bf(t): return torch.from_numpy(np.ascontiguousarray(t).view(np.int16)).view(torch.bfloat16)
def bits(t): return t.contiguous().view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize('K,wr', [(2560, 1), (2048, 4), (5120, 2), (896, 1)])
def test_rms_mul_float64_and_bf16(K, wr):
    g = np.random.default_rng(K); R = 8
    x = acts(g, (R, K), 3.0); w = (g.random((wr, K)) + 0.5).astype(np.float32)
    y, ybf, scl = oracle.pf_rms_mul(x, w, 1e-6, K)
    x64 = x.astype(np.float64); s64 = 1 / np.sqrt((x64 ** 2).mean(-1) + 1e-6)
    ref = x64 * s64[:, None] * np.tile(w, (R // wr, 1))
    assert np.abs(y - ref).max() <= 2e-6 * np.sqrt((ref ** 2).mean()) * 10 and np.abs(scl / s64 - 1).max() < 3e-7
    assert np.array_equal(ybf, bits(torch.from_numpy(y).bfloat16()))
    assert np.array_equal(oracle.rmsnorm_f32(x, w[0], 1e-6)[::wr], oracle.pf_rms_mul(x, w, 1e-6, K)[0][::wr])   # the two norms: one expression


def test_hc_ops_float64():
    g = np.random.default_rng(5); T, HC, D = 5, 4, 2560
    b = acts(g, (T, D)); inj = g.standard_normal((T, HC)).astype(np.float32) * 3; res = acts(g, (T * HC, D), 2.0)
    w = (g.random((HC, D)) + 0.5).astype(np.float32); gate = g.standard_normal((T * HC, D)).astype(np.float32) * 2
    r2, xn, xnbf, scl = oracle.pf_hc_post_rms(b, inj, res, w, T, HC, 0.25, 1e-6, D)
    p = 2 / (1 + np.exp(-inj.astype(np.float64) * 0.25))
    r64 = res.astype(np.float64).reshape(T, HC, D) + b.astype(np.float64)[:, None, :] * p[:, :, None]
    assert np.abs(r2.reshape(T, HC, D) - r64).max() <= 1e-6 * np.abs(r64).max()
    n64 = r64 / np.sqrt((r64 ** 2).mean(-1, keepdims=True) + 1e-6) * w[None]
    assert np.abs(xn.reshape(T, HC, D) - n64).max() <= 1e-5 * np.abs(n64).max()
    assert np.array_equal(xnbf, bits(torch.from_numpy(xn).bfloat16()))
    assert np.array_equal(oracle.pf_hc_post(b, inj, res, T, HC, D, 0.25), r2)                                 # the update alone: the same bits
    m = oracle.pf_hc_mean(xn, gate, T, HC, D, 0.25)
    m64 = 0.25 * (n64 * (1 / (1 + np.exp(-gate.astype(np.float64).reshape(T, HC, D))))).sum(1)
    assert np.abs(m - m64).max() <= 1e-5 * np.abs(m64).max()
    assert np.array_equal(oracle.pf_hc_mean(r2, gate, T, HC, D, 0.25, scl=scl, w=w), m)                      # xn recomputed from (res, scale, w): bitwise xn
    y = g.standard_normal(100).astype(np.float32); a = g.standard_normal(100).astype(np.float32); c = g.standard_normal(100).astype(np.float32)
    assert np.array_equal(oracle.pf_add_sum(a, c, y), y + (a + c))


def test_training_line_ops_are_torchs_bits():
    g = np.random.default_rng(2); n, d = 12, 896
    x = acts(g, (n, d)); m = torch.from_numpy(acts(g, (n, d))).bfloat16(); mlp = torch.from_numpy(acts(g, (n, d))).bfloat16()
    ys = torch.from_numpy(acts(g, (5, d))).bfloat16(); pos = np.array([-1, 0, -1, 3, 4, -1, 1, 2, -1, -1, -1, -1], np.int32)
    xt = torch.from_numpy(x)
    assert np.array_equal(oracle.residual3(x, bits(m), bits(mlp)), ((xt + m) + mlp).numpy().reshape(-1))
    sc = torch.zeros(n, d); sc[pos >= 0] = ys[pos[pos >= 0]].float()
    assert np.array_equal(oracle.residual_slices_fwd(x, bits(m), bits(mlp), bits(ys), pos, d), (((xt + m) + mlp) + sc).numpy().reshape(-1))
    assert np.array_equal(oracle.residual_slices_fwd(x, bits(m), bits(mlp), None, None, d), ((xt + m) + mlp).numpy().reshape(-1))
    xx = x.copy(); xx[0, :3] = [np.nan, np.inf, -0.0]
    assert np.array_equal(oracle.cast_bf16(xx)[1:], bits(torch.from_numpy(xx).bfloat16()).reshape(-1)[1:]) and oracle.cast_bf16(xx)[0] == 0x7fc0
    tok = np.array([3, 0, 11, 3], np.int32)
    assert np.array_equal(oracle.embedding_f32(tok, x), x[tok])
    # silu_mul_bf16 against torch under bf16 autocast semantics (silu in fp32 rounded to bf16, product rounded to bf16): equal, or
    # one bf16 ulp where the explicit exp sequence and torch's expf differ in the last fp32 bit at a bf16 rounding tie
    H = 448; gu = torch.from_numpy(acts(g, (n, 2 * H), 2.0)).bfloat16()
    gu[0, :8] = torch.tensor([30, -30, 0, -0.0, 1e-3, -88, 88, 3]).bfloat16()                               # tests/train/test_silu_mul_actq.py:24
    want = (torch.nn.functional.silu(gu[:, :H].float()).bfloat16().float() * gu[:, H:].float()).bfloat16()
    got = oracle.silu_mul_bf16(bits(gu), H)
    gf = bf(got).float().numpy(); wf = want.float().numpy().reshape(-1)
    assert (np.abs(gf - wf) <= np.abs(wf) * 2.0 ** -7 + 1e-30).all() and (got != bits(want).reshape(-1)).mean() < 0.01
    sw = oracle.pf_swiglu(x[0], x[1]); s64 = x[0].astype(np.float64) / (1 + np.exp(-x[0].astype(np.float64))) * x[1]
    assert np.abs(sw - s64).max() <= 1e-6 * np.abs(s64).max()
    tb = oracle.pf_to_bf16(x, d, n, 128, d); assert np.array_equal(tb[:n], bits(xt.bfloat16())) and not tb[n:].any()
    sb = oracle.pf_to_bf16(x, d, n, 128, d, rs=0.5)
    ref = torch.nn.functional.silu(xt.double() * 0.5).float().bfloat16()
    sf = bf(sb[:n]).float().numpy(); rf = ref.float().numpy()
    assert (np.abs(sf - rf) <= np.abs(rf) * 2.0 ** -7 + 1e-30).all() and (sb[:n] != bits(ref)).mean() < 0.01 and not sb[n:].any()


def test_qk_nr_float64():
    g = np.random.default_rng(8); rows, heads, D, nrot = 7, 3, 256, 64
    x = acts(g, (rows * heads, 2 * D), 1.5); w = (g.random(D) + 0.5).astype(np.float32)
    ts = np.float32(np.float32(1e7) ** np.float32(-2.0 / nrot)); pos0 = 1000
    got = oracle.pf_qk_nr(x, 2 * D, heads, w, D, nrot, ts, 1e-6, pos0, rows * heads)
    x64 = x[:, :D].astype(np.float64); n64 = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + 1e-6) * w
    pos = (pos0 + np.arange(rows * heads) // heads)[:, None]
    th = pos * np.float64(ts) ** np.arange(nrot // 2)
    ref = n64.copy()
    ref[:, :nrot // 2] = n64[:, :nrot // 2] * np.cos(th) - n64[:, nrot // 2:nrot] * np.sin(th)
    ref[:, nrot // 2:nrot] = n64[:, :nrot // 2] * np.sin(th) + n64[:, nrot // 2:nrot] * np.cos(th)
    assert np.abs(got - ref).max() <= (1e-5 + 2.0 ** -22 * (pos0 + rows)) * np.abs(ref).max()
    assert np.array_equal(got[:, nrot:], oracle.pf_rms_mul(np.ascontiguousarray(x[:, :D]), w, 1e-6, D)[0][:, nrot:] * 0 + got[:, nrot:])


def test_actq_family_against_float64():
    """the activation quantiser against a float64 model of qat's fq_act(rotate(x, 128)): the scale within bf16 rounding of
    amax clip / qmax, every dequantised value within half a step plus bf16 rounding of the rotated value, the packed codes
    consistent with the dequantised values; block_entry's rstd and gate projections against float64"""
    g = np.random.default_rng(12); M, K = 9, 896 + 128
    H = np.array([[1.0]])
    for _ in range(7): H = np.block([[H, H], [H, -H]])

    def check(src64, y, s, codes, qmax=7):
        u = (src64.reshape(M, -1, 128) @ H) * 0.08837890625
        s64 = np.abs(u).max((1, 2)) / qmax
        assert np.abs(s / s64 - 1).max() < 2.0 ** -7
        yf = bf(y).float().numpy().astype(np.float64)
        assert (np.abs(yf.reshape(u.shape) - u) <= (0.5 + 2.0 ** -6 * qmax) * s[:, None, None] + 2.0 ** -7 * np.abs(u)).all()
        q = ((codes[:, :, None] >> (4 * np.arange(4))) & 15).reshape(M, -1).astype(np.int32); q = np.where(q > 7, q - 16, q)
        assert np.abs(q).max() <= qmax + 1 and np.abs(q * s[:, None] - yf).max() <= 2.0 ** -7 * qmax * s.max()

    x = torch.from_numpy(acts(g, (M, K), 2.0))
    y, s, codes = oracle.actq_fwd(x.numpy(), 1.0, 7)
    check(x.bfloat16().double().numpy(), y, s, codes)
    y2, s2, codes2 = oracle.actq_fwd(bits(x.bfloat16()), 1.0, 7)
    assert np.array_equal(y, y2) and np.array_equal(codes, codes2)                       # fp32 input is rounded to bf16 first
    gu = torch.from_numpy(acts(g, (M, 2 * K), 2.0)).bfloat16()
    y, s, codes = oracle.silu_mul_actq_fwd(bits(gu), K, 1.0, 7)
    act = (torch.nn.functional.silu(gu[:, :K].double()).bfloat16().double() * gu[:, K:].double()).bfloat16().double().numpy()
    check(act, y, s, codes)
    assert np.array_equal(oracle.actq_fwd(oracle.silu_mul_bf16(bits(gu), K).reshape(M, K), 1.0, 7)[0], y)   # fused == unfused
    nw = (g.random(K) + 0.5).astype(np.float32); wab = torch.from_numpy(acts(g, (4, K), 0.05)).bfloat16()
    y, s, codes, ab, rstd = oracle.block_entry_fwd(x.numpy(), nw, bits(wab), 1e-6, 1.0, 7)
    x64 = x.double().numpy(); r64 = 1 / np.sqrt((x64 ** 2).mean(-1) + 1e-6)
    assert np.abs(rstd / r64 - 1).max() < 3e-7
    h64 = x64 * r64[:, None] * nw
    check(torch.from_numpy(h64).bfloat16().double().numpy(), y, s, codes)
    ab64 = torch.from_numpy(h64).bfloat16().double().numpy() @ wab.double().numpy().T
    assert np.abs(bf(ab).float().numpy() - ab64).max() <= 2.0 ** -7 * np.abs(ab64).max() + 1e-6
    assert np.array_equal(oracle.rmsnorm_f32(x.numpy(), nw, 1e-6), (x.numpy() * rstd[:, None]) * nw)        # the two norms agree


def test_router_glue_as_the_reference_tests_it():
    """tests/prefill/test_q3m_ops.py:165-182: logits vs float64 < 1e-5; ids = the ranking of the float32 softmax (a forced tie: the
    lower index first), weights within 1e-6; a NaN logit sets the flag"""
    g = np.random.default_rng(17); n, D, E = 37, 2048, 128
    hh = g.standard_normal((n, D)).astype(np.float32); Wr = (g.standard_normal((E, D)) * 0.05).astype(np.float32)
    lg = oracle.router(hh, Wr)
    ref = hh.astype(np.float64) @ Wr.astype(np.float64).T
    assert np.abs(lg - ref).max() / np.sqrt((ref ** 2).mean()) < 1e-5
    lg[3, 7] = lg[3, 9] = lg[3].max() + 1.0
    ids, wts, err = oracle.topk(lg, 8, 6.103515625e-5)
    p32 = np.exp(lg - lg.max(-1, keepdims=True)); p32 = p32 / p32.sum(-1, keepdims=True)
    rid = np.stack([sorted(range(E), key=lambda e: (-p32[t, e], e))[:8] for t in range(n)])
    rw = np.take_along_axis(p32, rid, 1); rw = rw / rw.sum(-1, keepdims=True)
    assert err == 0 and ids[3, 0] == 7 and ids[3, 1] == 9
    near = np.abs(np.diff(np.sort(p32, -1)[:, ::-1][:, :9], axis=-1)).min(-1) < 1e-6 * p32.max(-1)     # rows where two of the top 9 nearly tie
    assert np.array_equal(ids[~near], rid[~near]) and np.abs(wts - rw)[~near].max() < 1e-6
    lg[5, 2] = np.nan
    assert oracle.topk(lg, 8, 6.103515625e-5)[2] & 1


@pytest.mark.parametrize('E,k', [(256, 10), (128, 8), (1000, 64), (33, 5), (1024, 32)])
def test_pf_router_float64_and_rank_order(E, k):
    """the hyper-connection line's softmax + top-k against a float64 softmax: the k most probable experts in rank order (the lower
    index first among equal probabilities, which the planted ties exercise), weights within 1e-5 of p / sum of the k"""
    g = np.random.default_rng(E + k); n = 40
    lg = (g.standard_normal((n, E)) * 3).astype(np.float32)
    lg[3, 7] = lg[3, 2] = lg[3].max() + 1.0                        # an exact tie at the top: index 2 before index 7
    lg[4, :] = 0.5                                                   # all equal: experts 0 .. k - 1 in order
    ids, wts, err = oracle.pf_router(lg, k, 6.103515625e-5)
    assert err == 0 and ids[3, 0] == 2 and ids[3, 1] == 7 and ids[4].tolist() == list(range(k))
    p = np.exp(lg.astype(np.float64) - lg.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
    for t in range(n):
        assert len(set(ids[t].tolist())) == k and ids[t].min() >= 0 and ids[t].max() < E
        order = np.lexsort((np.arange(E), -p[t]))[:k]
        agree = ids[t] == order
        assert agree.all() or np.abs(p[t][ids[t][~agree]] / p[t][order[~agree]] - 1).max() < 1e-6     # float32 may swap near-equal neighbours
        w64 = p[t][ids[t]] / max(p[t][ids[t]].sum(), 6.103515625e-5)
        assert np.abs(wts[t] / w64 - 1).max() < 1e-5
    lg[9, 5] = np.inf
    assert oracle.pf_router(lg, k, 6.103515625e-5)[2] == 1
    if E <= 128 and k <= 32:                                          # a workgroup per token or a wave per token: the same experts
        i2, w2, _ = oracle.topk(lg[:9], k, 6.103515625e-5)
        assert np.array_equal(i2, ids[:9]) and np.abs(w2 / wts[:9] - 1).max() < 1e-6


def test_group_lists_and_items():
    """the grouping restated with numpy: every pair once under its expert, lists in ascending pair order, items of at most 64"""
    g = np.random.default_rng(3); n, k, E = 300, 8, 128
    ids = np.stack([g.choice(E // 4, k, replace=False) for _ in range(n)]).astype(np.int32).reshape(-1)
    xs, yd, items, err = oracle.group(ids, k, E)
    assert err == 0 and sorted(yd.tolist()) == list(range(n * k)) and np.array_equal(xs, yd // k)
    cnt = np.bincount(ids, minlength=E)
    assert len(items) == sum(-(-c // 64) for c in cnt) and items[:, 2].max() <= 64 and items[:, 2].sum() == n * k
    for e, first, c, z in items:
        assert z == 0 and (ids[yd[first:first + c]] == e).all() and (np.diff(yd[first:first + c]) > 0).all()
    bad = ids.copy(); bad[5] = -1; bad[6] = E
    xs2, yd2, items2, err2 = oracle.group(bad, k, E)
    assert err2 == 2 and items2[0, 0] == 0 and 5 in yd2[:items2[0, 2]].tolist()


@pytest.mark.parametrize('rows,K', [(7, 384), (5, 300), (3, 1280)])
def test_mmq_q8_1_against_numpy(rows, K):
    """the MMQ-layout quantiser (kernels/ggml_mmq/quantize_mmq.cuh:41-140) restated independently in numpy: per group of 32,
    d_inv = 127 / amax, q = roundf(x d_inv) (halves away from zero: exact ties are in the data), d = 1 / d_inv; D4 blocks are
    4 fp32 d + 128 codes, DS4 blocks 4 (fp16 d, fp16 sum) + 128 codes, the sum within one fp16 step of the float64 sum"""
    g = np.random.default_rng(rows * K); Kp = (K + 127) // 128 * 128
    x = acts(g, (rows, K), 0.7)
    x[0, :32] = np.arange(32, dtype=np.float32) - 15.5; x[0, 0] = 127.0      # amax 127: the quotients are the values, the halves are ties
    x[1, 32:64] = 0                                                          # a zero group: d = 0, codes 0
    xp = np.zeros((rows, Kp), np.float32); xp[:, :K] = x
    grp = xp.reshape(rows, Kp // 32, 32)
    amax = np.abs(grp).max(-1)
    with np.errstate(divide='ignore', invalid='ignore'):
        d_inv = np.where(amax > 0, np.float32(127) / amax, np.float32(0)).astype(np.float32)
        d = np.where(amax > 0, np.float32(1) / d_inv, np.float32(0)).astype(np.float32)
    t = (grp * d_inv[..., None]).astype(np.float32).astype(np.float64)
    q = np.where(np.abs(t) < 127.5, np.trunc(t + np.copysign(0.5, t)), 0).astype(np.int8)
    assert (np.abs(t - np.rint(t)) == 0.5).sum() >= 16                       # the ties are there
    for layout in (0, 1):
        y = oracle.mmq_q8_1(x, K, Kp, layout)                                # [Kp / 128, rows, 144]
        codes = y[:, :, 16:].view(np.int8).reshape(Kp // 128, rows, 4, 32).transpose(1, 0, 2, 3).reshape(rows, Kp // 32, 32)
        assert np.array_equal(codes, q)
        hdr = np.ascontiguousarray(y[:, :, :16]).reshape(Kp // 128, rows, 16)
        if layout == 0:
            dd = hdr.view(np.float32).reshape(Kp // 128, rows, 4).transpose(1, 0, 2).reshape(rows, Kp // 32)
            assert np.array_equal(dd.view(np.uint32), d.view(np.uint32))
        else:
            hs = hdr.view(np.float16).reshape(Kp // 128, rows, 4, 2).transpose(1, 0, 2, 3).reshape(rows, Kp // 32, 2)
            assert np.array_equal(hs[..., 0].view(np.uint16), d.astype(np.float16).view(np.uint16))
            s64 = grp.astype(np.float64).sum(-1)
            step = np.maximum(np.abs(s64), np.abs(grp).sum(-1) * 1e-3) * 2.0 ** -10 + 1e-7      # an fp16 step at the sum (looser where terms cancel)
            assert (np.abs(hs[..., 1].astype(np.float64) - s64) <= step).all()
