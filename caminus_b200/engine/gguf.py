"""Q8_1 activation quantiser and SwiGLU, with the reference's host functions (python/caminus/engine/gguf.py:39-61) plus the
fused form the decode tape builds with Engine.gg_q8_1(x, yq, mul=u) (python/caminus/engine/k3.py:649-659)."""
import ctypes

import torch

from ..device.cuda import Module
from .. import lib as _lib

Q8_1_BYTES = 36          # block_q8_1: half d, half sum, 32 int8
_mod = {}


def _m(module='k3_gguf'):
    key = (torch.cuda.current_device(), module)
    if key not in _mod: _mod[key] = Module(module)
    return _mod[key]


def quantize_q8_1(x):
    """x fp32 [n] (cuda) -> q8_1 blocks (uint8 [ceil(n / 32) * 36]); values past n quantize as 0"""
    n = x.numel(); nb = (n + 31) // 32
    y = torch.empty(nb * Q8_1_BYTES, dtype=torch.uint8, device=x.device)
    _m().gg_quantize_q8_1(((nb * 32 + 255) // 256,), (256,), x.contiguous(), y, ctypes.c_int(n))
    return y


def silu_mul(g, u):
    """h = silu(g) * u in fp32"""
    n = g.numel(); h = torch.empty_like(g)
    _m('k3_gguf_gsq').gg_silu_mul(((n + 255) // 256,), (256,), g.contiguous(), u.contiguous(), h, ctypes.c_int(n))
    return h


def swiglu_q8_1(g, u, yq=None, strict=False, sums=False):
    """q8_1 blocks of silu(g) * u in one launch; g, u both fp32 or both fp16 (cuda), same numel. d and the codes are always
    the exact statements' bytes; sums=True proves the block sums as well (all 36 bytes exact, about four fifths of the default's
    throughput); strict=True runs the exact statements for every value (the same bytes as sums=True, slower still)"""
    if g.dtype != u.dtype or g.dtype not in (torch.float32, torch.float16) or g.numel() != u.numel() or g.device != u.device:
        raise ValueError(f'swiglu_q8_1: gate {g.dtype} [{g.numel()}] and up {u.dtype} [{u.numel()}] (both fp32 or both fp16, one size)')
    if not (g.is_contiguous() and u.is_contiguous()): raise ValueError('swiglu_q8_1: gate and up must be contiguous')
    n = g.numel(); nb = (n + 31) // 32
    if yq is None: yq = torch.empty(nb * Q8_1_BYTES, dtype=torch.uint8, device=g.device)
    elif yq.dtype != torch.uint8 or yq.numel() < nb * Q8_1_BYTES or not yq.is_contiguous():
        raise ValueError(f'swiglu_q8_1: yq needs {nb * Q8_1_BYTES} contiguous uint8')
    fn = getattr(_lib.load(), ('gg_swiglu_q8_1_f16' if g.dtype == torch.float16 else 'gg_swiglu_q8_1') + ('_strict' if strict else '_sums' if sums else ''))
    with torch.cuda.device(g.device):
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(fn(g.data_ptr(), u.data_ptr(), yq.data_ptr(), n, s), 'gg_swiglu_q8_1')
    return yq


def silu_scale_q8_1(x, rs, yq=None, sums=False):
    """q8_1 blocks of silu(x * rs) in one launch (x fp32, cuda): the decode tape's Engine.gg_q8_1(x, yq, silu_scale=rs)
    (python/caminus/engine/k3.py:649-659). sums=True proves the block sums too (all 36 bytes the exact statements')"""
    if x.dtype != torch.float32 or not x.is_contiguous(): raise ValueError(f'silu_scale_q8_1: x must be contiguous fp32, not {x.dtype}')
    n = x.numel(); nb = (n + 31) // 32
    if yq is None: yq = torch.empty(nb * Q8_1_BYTES, dtype=torch.uint8, device=x.device)
    elif yq.dtype != torch.uint8 or yq.numel() < nb * Q8_1_BYTES or not yq.is_contiguous(): raise ValueError(f'silu_scale_q8_1: yq needs {nb * Q8_1_BYTES} contiguous uint8')
    fn = _lib.load().gg_silu_scale_q8_1_sums if sums else _lib.load().gg_silu_scale_q8_1
    with torch.cuda.device(x.device):
        _lib.check(fn(x.data_ptr(), float(rs), yq.data_ptr(), n, torch.cuda.current_stream().cuda_stream), 'gg_silu_scale_q8_1')
    return yq


MMQ_BLOCK_BYTES = 144     # block_q8_1_mmq: 16 bytes of scales + 128 int8
MMQ_LAYOUTS = {'D4': 0, 'DS4': 1}


def quantize_mmq_q8_1(x, layout='D4', u=None, y=None, kvalid=None):
    """rows of x [rows, K] (cuda; fp32, or fp16 with u) -> Q8_1 in the MMQ layout, uint8 [ceil(K / 128), rows, 144].
    u given: the blocks of silu(x) * u (the fused gate / up epilogue's bytes). kvalid: values per row that count (default K)"""
    if x.dim() != 2 or x.stride(1) != 1 or x.dtype not in (torch.float32, torch.float16): raise ValueError('quantize_mmq_q8_1: x must be [rows, K] fp32 / fp16')
    if u is None and x.dtype != torch.float32: raise ValueError('quantize_mmq_q8_1: plain quantisation takes fp32')
    if u is not None and (u.shape != x.shape or u.dtype != x.dtype or u.stride() != x.stride()): raise ValueError('quantize_mmq_q8_1: u must match x')
    if layout not in MMQ_LAYOUTS: raise ValueError(f'quantize_mmq_q8_1: layout {layout!r} ({sorted(MMQ_LAYOUTS)})')
    rows, K = x.shape; kvalid = K if kvalid is None else int(kvalid); Kpad = (K + 127) // 128 * 128
    if y is None: y = torch.empty(Kpad // 128, rows, MMQ_BLOCK_BYTES, dtype=torch.uint8, device=x.device)
    elif y.dtype != torch.uint8 or y.numel() < Kpad // 128 * rows * MMQ_BLOCK_BYTES or not y.is_contiguous(): raise ValueError('quantize_mmq_q8_1: y too small')
    L = _lib.load()
    with torch.cuda.device(x.device):
        s = torch.cuda.current_stream().cuda_stream
        if u is None: r = L.cam_quantize_mmq_q8_1(x.data_ptr(), y.data_ptr(), kvalid, Kpad, x.stride(0), rows, MMQ_LAYOUTS[layout], s)
        elif x.dtype == torch.float16: r = L.cam_swiglu_mmq_q8_1_f16(x.data_ptr(), u.data_ptr(), y.data_ptr(), kvalid, Kpad, x.stride(0), rows, MMQ_LAYOUTS[layout], s)
        else: r = L.cam_swiglu_mmq_q8_1(x.data_ptr(), u.data_ptr(), y.data_ptr(), kvalid, Kpad, x.stride(0), rows, MMQ_LAYOUTS[layout], s)
    _lib.check(r, 'quantize_mmq_q8_1')
    return y
