"""The fast passes held to the exact statements on EVERY gate, not on samples. A kernel that stores the special-function unit's value
where it has proven the stored bytes cannot depend on it (SwiGLU + Q8_1 in its default and all-bytes forms, the MMQ-layout SwiGLU in
both layouts, the training line's fused SiLU quantiser) is run on all 65 536 bit patterns of a 16-bit gate (finite, both zeros, both
infinities, every NaN, every subnormal), each against 256 up values, in two block compositions, and compared with the kernel that runs
the exact statements for every value. 2 x 16.7 M values per form: about 300 000 of the codes lie within a few fp32 ulps of a .5
boundary and a few hundred block scales within an ulp of an fp16 tie, which is where a wrong proof would show. The reference's own
gate for these bytes is 0 mismatches (tests/engine/test_gguf_mv.py:33-45)."""
import numpy as np
import pytest

torch = pytest.importorskip('torch')
pytestmark = pytest.mark.gpu

from caminus_b200.engine import gguf   # noqa: E402

DEV = 'cuda:0'
U = 256


def every_gate(dtype, layout, finite_ups=False):
    """gate [65536 * U] = every 16-bit pattern U times, up [65536 * U]: a quarter N(0, 1.5), a quarter log-uniform over the type's range
    with random signs, a quarter multiples of 1 / 8 (few distinct products: exact .5 quotients occur), a quarter specials (zeros, the
    largest and smallest normals, subnormals, infinities, NaN) mixed into N(0, 1). layout 'runs': a block of 32 is 32 consecutive gate
    patterns under one up value (equal magnitudes: every code between 64 and 127); 'mixed': gates and ups shuffled over all blocks"""
    gen = torch.Generator(device=DEV); gen.manual_seed(11)
    pat = torch.arange(65536, device=DEV, dtype=torch.int32).to(torch.int16).view(dtype)
    q = U // 4
    ups = torch.empty(U, 65536, device=DEV, dtype=torch.float32)
    ups[:q] = torch.randn(q, 65536, device=DEV, generator=gen) * 1.5
    lo, hi = (-14.0, 15.0) if dtype == torch.float16 else (-20.0, 20.0)
    mag = torch.exp2(torch.rand(q, 65536, device=DEV, generator=gen) * (hi - lo) + lo)
    ups[q:2 * q] = mag * (torch.randint(0, 2, (q, 65536), device=DEV, generator=gen) * 2 - 1)
    ups[2 * q:3 * q] = torch.round(torch.randn(q, 65536, device=DEV, generator=gen) * 12) / 8
    sp = torch.randn(q, 65536, device=DEV, generator=gen)
    big, tiny = (65504.0, 6.1e-5) if dtype == torch.float16 else (3.38e38, 1.2e-38)
    specials = torch.tensor([0.0, -0.0, big, -big, tiny, -tiny, tiny / 64, 1.0, -1.0] + ([] if finite_ups else [float('inf'), float('-inf'), float('nan')]), device=DEV)
    pick = torch.randint(0, 40 * len(specials), (q, 65536), device=DEV, generator=gen)
    sp = torch.where(pick < len(specials), specials[pick.clamp(max=len(specials) - 1)], sp)
    ups[3 * q:] = sp
    g = pat.unsqueeze(0).expand(U, 65536).contiguous().view(-1)
    u = ups.to(dtype).view(-1)
    if layout == 'mixed':
        p1 = torch.randperm(g.numel(), device=DEV, generator=gen); p2 = torch.randperm(g.numel(), device=DEV, generator=gen)
        g, u = g[p1].contiguous(), u[p2].contiguous()
    return g, u


def q8_fields(y):
    b = y.view(-1, 36)
    return b[:, 0:2].contiguous().view(torch.int16).view(-1), b[:, 2:4].contiguous().view(torch.int16).view(-1), b[:, 4:]


def is_nan16(h): return (h & 0x7fff) > 0x7c00


@pytest.mark.parametrize('layout', ['runs', 'mixed'])
def test_swiglu_q8_1_f16_every_gate(layout):
    """gg_swiglu_q8_1_f16: scale and codes of every block are the exact statements'; gg_swiglu_q8_1_f16_sums: all 36 bytes"""
    g, u = every_gate(torch.float16, layout)
    strict = gguf.swiglu_q8_1(g, u, strict=True)
    d0, s0, q0 = q8_fields(strict)
    nan_d = is_nan16(d0)                                     # (a NaN scale has no fixed bit pattern; its block's codes are not gated either)
    for sums in (False, True):
        d, s, q = q8_fields(gguf.swiglu_q8_1(g, u, sums=sums))
        assert torch.equal(d[~nan_d], d0[~nan_d]) and bool(is_nan16(d[nan_d]).all())
        assert torch.equal(q[~nan_d], q0[~nan_d])
        if sums:
            nan_s = is_nan16(s0)
            assert torch.equal(s[~nan_s], s0[~nan_s]) and bool(is_nan16(s[nan_s]).all())
    assert int((~nan_d).sum()) > 400000                      # the comparison covered what it should


@pytest.mark.parametrize('layout', ['runs', 'mixed'])
@pytest.mark.parametrize('mmq', ['D4', 'DS4'])
def test_swiglu_mmq_f16_every_gate(layout, mmq):
    """cam_swiglu_mmq_q8_1_f16 in both layouts: every byte equals the plain quantiser's over the fp32 products silu(g) u formed by the
    exact statements (fused == unfused)"""
    g, u = every_gate(torch.float16, layout)
    K = 4096; rows = g.numel() // K
    g2, u2 = g.view(rows, K), u.view(rows, K)
    fused = gguf.quantize_mmq_q8_1(g2, mmq, u=u2)
    h = gguf.silu_mul(g.float(), u.float()).view(rows, K)
    plain = gguf.quantize_mmq_q8_1(h, mmq)
    fb, pb = fused.view(-1, 144), plain.view(-1, 144)
    if mmq == 'D4':
        fd, pd = fb[:, :16].contiguous().view(torch.int32), pb[:, :16].contiguous().view(torch.int32)
        nan = (pd & 0x7fffffff) > 0x7f800000
        grp_ok = ~nan                                                        # [blocks, 4]: the groups of 32 with a number for a scale
        assert torch.equal(fd[grp_ok], pd[grp_ok]) and bool(((fd[nan] & 0x7fffffff) > 0x7f800000).all())
    else:
        fd, pd = fb[:, :16].contiguous().view(torch.int16), pb[:, :16].contiguous().view(torch.int16)      # (d, sum) x 4
        nan = is_nan16(pd)
        assert torch.equal(fd[~nan], pd[~nan]) and bool(is_nan16(fd[nan]).all())
        grp_ok = ~nan.view(-1, 4, 2)[:, :, 0]
    fq, pq = fb[:, 16:].view(-1, 4, 32), pb[:, 16:].view(-1, 4, 32)
    assert torch.equal(fq[grp_ok], pq[grp_ok])


def test_silu_mul_actq_every_bf16_gate():
    """silu_mul_actq_fwd: values, scales and packed codes equal the unfused pair (silu_mul_bf16, then actq_fwd_codes_bf16) on every bf16
    gate against 256 ups (the unfused pair is held to the oracle on every gate in test_gpu_parity_hc.py)"""
    import ctypes
    from caminus_b200.device import cuda as hip
    from caminus_b200.train import actq as A
    g, u = every_gate(torch.bfloat16, 'runs', finite_ups=True)      # (rows of 4096 consecutive patterns: the NaN and infinity gates keep to 2 rows in 16)
    F = 4096; M = g.numel() // F
    gu = torch.cat([g.view(M, F), u.view(M, F)], dim=1).contiguous()
    y, c, s = A.silu_mul_actq(gu, 4, 1.0)
    act = torch.empty(M, F, dtype=torch.bfloat16, device=DEV)
    hip.Module('core').silu_mul_bf16(((M * F + 255) // 256,), (256,), gu, act, ctypes.c_int(F), ctypes.c_int64(M * F))
    y2, c2, s2 = A.actq_codes(act, 4, 1.0)
    fin = torch.isfinite(s2)                                  # a row whose activation holds a NaN or an infinity has no number for a scale
    assert int(fin.sum()) > M // 2
    assert torch.equal(s.view(torch.int32)[fin], s2.view(torch.int32)[fin])
    assert torch.equal(y.view(torch.int16)[fin], y2.view(torch.int16)[fin]) and torch.equal(c[fin], c2[fin])


def test_fast_silu_bound_over_every_fp16_gate():
    """the bound the fp16 entries' proofs rest on, measured on this device: over every fp16 gate >= -8 (zeros aside) the special-function
    evaluation of silu is within 5.6e-7 of the exact statements' value (5.43e-7 on sm_100a; the proofs allow 7.0e-7 after the product)"""
    from caminus_b200 import lib
    pat = torch.arange(65536, device=DEV, dtype=torch.int32).to(torch.int16)
    fast = torch.empty(65536, device=DEV); exact = torch.empty(65536, device=DEV)
    lib.check(lib.load().cam_probe_silu_f16(pat.data_ptr(), fast.data_ptr(), exact.data_ptr(), 65536, torch.cuda.current_stream().cuda_stream))
    g = pat.view(torch.float16).double()
    ok = torch.isfinite(g) & (g >= -8.0) & (g != 0)
    rel = ((fast.double() - exact.double()).abs() / exact.double().abs())[ok]
    assert int(ok.sum()) == 50175 and float(rel.max()) <= 5.6e-7, float(rel.max())
    true = g[ok] / (1 + torch.exp(-g[ok]))
    assert float(((exact.double()[ok] - true).abs() / true.abs()).max()) <= 2.5e-7      # the exact statements against float64
