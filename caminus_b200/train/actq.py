"""The forward launches of the training line's fused activation quantiser, with the function names and argument meaning of the
reference's wrappers (python/caminus/train/actq.py: actq, actq_codes, silu_mul_actq, block_entry). Upstream each is the
forward of a torch.autograd.Function whose backward is another kernel; the backward kernels are not part of this library
(training is dormant upstream), so these functions return plain tensors."""
import ctypes

import torch

from ..device.cuda import Module

_modules = {}                      # the 'actq' object per device index


def _kernels():
    idx = torch.cuda.current_device()
    mod = _modules.get(idx)
    if mod is None: mod = _modules[idx] = Module('actq')
    return mod


def _qmax(bits):
    return (1 << (bits - 1)) - 1


def _rows(x, what, dtypes, limit=8192):
    """x [..., K] as contiguous rows [M, K]; K a multiple of 128 up to `limit`"""
    K = x.shape[-1]
    if x.dtype not in dtypes or K % 128 or K > limit:
        raise AssertionError(f'{what}: rows of {K} {x.dtype} values (a multiple of 128 up to {limit}; {" / ".join(map(str, dtypes))})')
    x2 = x.reshape(-1, K).contiguous()
    return x2, x2.shape[0], K


def _outputs(M, K, dev, codes=True):
    y = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    s = torch.empty(M, dtype=torch.float32, device=dev)
    c = torch.empty(M, K // 2, dtype=torch.uint8, device=dev) if codes else None
    return y, s, c


def actq_codes(x, bits=4, clip=1.0):
    """x [..., K] (bf16 or fp32) -> (xq bf16 like x, codes uint8 [M, K / 2], scales fp32 [M]): the rows rotated by the 128-point
    Hadamard transform and fake-quantised to `bits` with the row scale amax * clip / qmax"""
    assert bits <= 4
    x2, M, K = _rows(x, 'actq_codes', (torch.bfloat16, torch.float32))
    y, s, c = _outputs(M, K, x.device)
    if M > 0:
        k = _kernels()
        launch = k.actq_fwd_codes_bf16 if x2.dtype == torch.bfloat16 else k.actq_fwd_codes_f32
        launch((M,), (256,), x2, y, s, c, ctypes.c_int(K), ctypes.c_float(clip), ctypes.c_int(_qmax(bits)))
    return y.view(x.shape), c, s


def actq(x, bits=4, clip=1.0):
    """the dequantised bf16 values of actq_codes alone"""
    x2, M, K = _rows(x, 'actq', (torch.bfloat16, torch.float32))
    y, s, _ = _outputs(M, K, x.device, codes=False)
    if M > 0:
        k = _kernels()
        launch = k.actq_fwd_bf16 if x2.dtype == torch.bfloat16 else k.actq_fwd_f32
        launch((M,), (256,), x2, y, s, ctypes.c_int(K), ctypes.c_float(clip), ctypes.c_int(_qmax(bits)))
    return y.view(x.shape)


def silu_mul_actq(gu, bits=4, clip=1.0):
    """gu [M, 2 F] bf16 = [gate | up] rows (a row-strided view is fine) -> actq_codes(bf16(bf16(silu(gate)) * up)) in one launch"""
    M, width = gu.shape
    Fw = width // 2
    assert bits <= 4 and gu.dtype == torch.bfloat16 and gu.stride(1) == 1 and Fw % 128 == 0 and Fw <= 8192
    y, s, c = _outputs(M, Fw, gu.device)
    if M > 0:
        _kernels().silu_mul_actq_fwd((M,), (256,), gu, ctypes.c_int(gu.stride(0)), ctypes.c_int(Fw), y, s, c, ctypes.c_float(clip),
                                     ctypes.c_int(_qmax(bits)))
    return y, c, s


def block_entry(x, nw, wab, eps, bits=4, clip=1.0):
    """x [..., d] fp32 -> (xq, codes, scales, ab, rstd): actq_codes of h = RMSNorm(x; nw, eps), h never stored, plus the thin
    projections ab = bf16(h @ wab^T) for wab bf16 [nab, d] (None: none) and the rows' rstd"""
    assert bits <= 4
    x2, M, d = _rows(x, 'block_entry', (torch.float32,), limit=1024)
    nab = wab.shape[0] if wab is not None else 0
    assert nab % 2 == 0 and nab <= 16
    y, s, c = _outputs(M, d, x.device)
    ab = torch.empty(M, nab, dtype=torch.bfloat16, device=x.device)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    if M > 0:
        none = ctypes.c_void_p(None)
        _kernels().block_entry_fwd((M,), (256,), x2, nw, wab if nab else none, ctypes.c_int(nab), ctypes.c_float(eps), y, s, c,
                                   ab if nab else none, rstd, ctypes.c_int(d), ctypes.c_float(clip), ctypes.c_int(_qmax(bits)))
    return y.view(x.shape), c, s, ab.view(*x.shape[:-1], nab), rstd
