"""Forward halves of the reference's fused activation-quant wrappers (python/caminus/train/actq.py: actq, actq_codes,
silu_mul_actq, block_entry), same argument meaning and shape checks. The reference wraps each in a torch.autograd.Function
whose backward is another kernel; the backward kernels (training is dormant upstream) are not part of this library, so these
return plain tensors."""
import ctypes

import torch

from ..device.cuda import Module

_mod = {}


def _m():
    dev = torch.cuda.current_device()
    if dev not in _mod: _mod[dev] = Module('actq')
    return _mod[dev]


I, F = ctypes.c_int, ctypes.c_float


def actq_codes(x, bits=4, clip=1.0):
    """(xq bf16, codes uint8 [M, K / 2], scales fp32 [M]) of x [..., K] (bf16 or fp32): fq_act(rotate(x, 128), bits, clip)"""
    K = x.shape[-1]; x2 = x.reshape(-1, K).contiguous(); M = x2.shape[0]
    assert x2.dtype in (torch.bfloat16, torch.float32) and K % 128 == 0 and K <= 8192 and bits <= 4
    y = torch.empty(M, K, device=x.device, dtype=torch.bfloat16)
    c = torch.empty(M, K // 2, device=x.device, dtype=torch.uint8); s = torch.empty(M, device=x.device)
    if M:
        fn = _m().actq_fwd_codes_bf16 if x2.dtype == torch.bfloat16 else _m().actq_fwd_codes_f32
        fn((M,), (256,), x2, y, s, c, I(K), F(clip), I(2 ** (bits - 1) - 1))
    return y.view(*x.shape), c, s


def actq(x, bits=4, clip=1.0):
    """the dequantised bf16 values alone"""
    K = x.shape[-1]; x2 = x.reshape(-1, K).contiguous(); M = x2.shape[0]
    assert x2.dtype in (torch.bfloat16, torch.float32) and K % 128 == 0 and K <= 8192
    y = torch.empty(M, K, device=x.device, dtype=torch.bfloat16); s = torch.empty(M, device=x.device)
    if M:
        fn = _m().actq_fwd_bf16 if x2.dtype == torch.bfloat16 else _m().actq_fwd_f32
        fn((M,), (256,), x2, y, s, I(K), F(clip), I(2 ** (bits - 1) - 1))
    return y.view(*x.shape)


def silu_mul_actq(gu, bits=4, clip=1.0):
    """(xq, codes, scales) = actq_codes(silu(g) * u) for gu [M, 2F] bf16 (may be a row-strided view), fused"""
    M, F2 = gu.shape; Fw = F2 // 2
    assert gu.dtype == torch.bfloat16 and gu.stride(1) == 1 and Fw % 128 == 0 and Fw <= 8192 and bits <= 4
    y = torch.empty(M, Fw, device=gu.device, dtype=torch.bfloat16)
    c = torch.empty(M, Fw // 2, device=gu.device, dtype=torch.uint8); s = torch.empty(M, device=gu.device)
    if M: _m().silu_mul_actq_fwd((M,), (256,), gu, I(gu.stride(0)), I(Fw), y, s, c, F(clip), I(2 ** (bits - 1) - 1))
    return y, c, s


def block_entry(x, nw, wab, eps, bits=4, clip=1.0):
    """(xq, codes, scales, ab, rstd) for h = RMSNorm(x; nw, eps), fused; wab bf16 [nab, d] or None"""
    d = x.shape[-1]; x2 = x.reshape(-1, d).contiguous(); M = x2.shape[0]
    assert x2.dtype == torch.float32 and d % 128 == 0 and d <= 1024 and bits <= 4
    nab = 0 if wab is None else wab.shape[0]
    assert nab <= 16 and nab % 2 == 0
    y = torch.empty(M, d, device=x.device, dtype=torch.bfloat16)
    c = torch.empty(M, d // 2, device=x.device, dtype=torch.uint8); s = torch.empty(M, device=x.device)
    ab = torch.empty(M, nab, device=x.device, dtype=torch.bfloat16); rstd = torch.empty(M, device=x.device)
    nul = ctypes.c_void_p(None)
    if M:
        _m().block_entry_fwd((M,), (256,), x2, nw, wab if nab else nul, I(nab), F(eps), y, s, c, ab if nab else nul, rstd, I(d), F(clip),
                             I(2 ** (bits - 1) - 1))
    return y.view(*x.shape), c, s, ab.view(*x.shape[:-1], nab), rstd
