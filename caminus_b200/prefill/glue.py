"""The hyper-connection part of the reference's prefill glue wrapper (python/caminus/prefill/glue.py:96-313: Glue.rms_mul,
hc_post_rms, hc_post, hc_mean, add_sum, silu_bf16, to_bf16), same names, argument meaning and refusals, over the B200
kernels. The router, GDN, PLE and BF16-matrix methods of the reference's class are outside this library's path."""
import ctypes

import torch

from ..device.cuda import Module

D_GLUE = 2560          # the default glue object's row width
TPAD = 128             # the GEMMs' token padding
GLUE_MODULES = {'prefill_glue': 2560, 'prefill_glue_q35': 2048, 'prefill_glue_q35d': 5120}
F32, BF16 = torch.float32, torch.bfloat16


def tpad(T):
    return (int(T) + TPAD - 1) // TPAD * TPAD


def _check(dev, what, bufs, opt=()):
    """each buffer stated once as (tensor, dtype, elements): on this device, contiguous, of that dtype and at least that long
    (the reference's device/bufcheck.LaunchCheck, python/caminus/device/bufcheck.py:1-27, without its overlap analysis)"""
    for name, (t, dt, n) in bufs.items():
        if t is None:
            if name in opt: continue
            raise ValueError(f'{what}: {name} is required')
        if not torch.is_tensor(t) or t.dtype != dt or t.numel() < n or not t.is_contiguous() or t.device != dev:
            raise ValueError(f'{what}: {name} needs a contiguous {dt} tensor of {n} elements on {dev}')


class Glue:
    module, D = 'prefill_glue', D_GLUE

    def __init__(self, device, module='prefill_glue'):
        self.dev = torch.device(device)
        if self.dev.index is None: self.dev = torch.device('cuda', torch.cuda.current_device())
        if module not in GLUE_MODULES: raise ValueError(f'Glue: module {module!r} ({sorted(GLUE_MODULES)})')
        self.module, self.D = module, GLUE_MODULES[module]
        with torch.cuda.device(self.dev): self.m = Module(module)

    def _go(self, fn, n, *args, threads=256):
        with torch.cuda.device(self.dev):
            getattr(self.m, fn)(((int(n) + threads - 1) // threads,), (threads,), *args)

    @staticmethod
    def _nul(t):
        return t if t is not None else ctypes.c_void_p(0)

    def rms_mul(self, x, w, y, R, eps, ybf=None, scale=None):
        """y[r] = rms_norm(x[r]) * w[r % wr] for R rows of D (w [wr, D], wr divides R). Outputs, each optional (at least one):
        y fp32 (y is x allowed), ybf its bf16 copy, scale [R] the row's rsqrt(mean(x^2) + eps)"""
        K = self.D; R = int(R); wr = w.numel() // K
        if R < 1 or wr < 1 or w.numel() != wr * K or R % wr: raise ValueError(f'rms_mul: R {R}, w {w.numel()} (rows of {K})')
        if y is None and ybf is None and scale is None: raise ValueError('rms_mul: no output')
        _check(self.dev, 'rms_mul', dict(x=(x, F32, R * K), w=(w, F32, wr * K), y=(y, F32, R * K), ybf=(ybf, BF16, R * K), scale=(scale, F32, R)),
               opt=('y', 'ybf', 'scale'))
        with torch.cuda.device(self.dev):
            self.m.pf_rms_mul((R,), (256,), x, w, self._nul(y), self._nul(ybf), self._nul(scale), ctypes.c_int(R), ctypes.c_int(wr), ctypes.c_float(eps))

    def hc_post_rms(self, block, inj, res, w, T, HC, eps, rs=0.25, xn=None, xnbf=None, scale=None):
        """res[t, h] += block[t] * 2 sigmoid(inj[t, h] * rs) (in place), then the norm of each (token, stream) row"""
        T, HC, D = int(T), int(HC), self.D
        _check(self.dev, 'hc_post_rms', dict(block=(block, F32, T * D), inj=(inj, F32, T * HC), res=(res, F32, T * HC * D), w=(w, F32, HC * D),
                                             xn=(xn, F32, T * HC * D), xnbf=(xnbf, BF16, T * HC * D), scale=(scale, F32, T * HC)), opt=('xn', 'xnbf', 'scale'))
        with torch.cuda.device(self.dev):
            self.m.pf_hc_post_rms((T * HC,), (256,), block, inj, res, w, self._nul(xn), self._nul(xnbf), self._nul(scale), ctypes.c_int(T),
                                  ctypes.c_int(HC), ctypes.c_float(rs), ctypes.c_float(eps))

    def hc_post(self, block, inj, res, T, HC, D=None, rs=0.25):
        T, HC, D = int(T), int(HC), int(self.D if D is None else D)
        _check(self.dev, 'hc_post', dict(block=(block, F32, T * D), inj=(inj, F32, T * HC), res=(res, F32, T * HC * D)))
        self._go('pf_hc_post', T * D, block, inj, res, ctypes.c_int(T), ctypes.c_int(HC), ctypes.c_int(D), ctypes.c_float(rs))

    def hc_mean(self, xn, gate, out, T, HC, D=None, rs=0.25, scale=None, w=None):
        T, HC, D = int(T), int(HC), int(self.D if D is None else D)
        if (scale is None) != (w is None): raise ValueError('hc_mean: scale and w go together')
        _check(self.dev, 'hc_mean', dict(xn=(xn, F32, T * HC * D), gate=(gate, F32, T * HC * D), out=(out, F32, T * D), scale=(scale, F32, T * HC),
                                         w=(w, F32, HC * D)), opt=('scale', 'w'))
        self._go('pf_hc_mean', T * D, xn, self._nul(scale), self._nul(w), gate, out, ctypes.c_int(T), ctypes.c_int(HC), ctypes.c_int(D), ctypes.c_float(rs))

    def add_sum(self, a, b, y, n):
        """y += a + b"""
        n = int(n)
        _check(self.dev, 'add_sum', dict(a=(a, F32, n), b=(b, F32, n), y=(y, F32, n)))
        self._go('pf_add_sum', n, a, b, y, ctypes.c_long(n))

    def silu_bf16(self, x, y, T, K, rs, ldx=None):
        """y [tpad(T), K] bf16 = bf16(silu(fma(rs, x, 0))) for the T rows of x (row stride ldx), zero rows to tpad(T)"""
        T, K = int(T), int(K); ldx = K if ldx is None else int(ldx); Tp = tpad(T)
        _check(self.dev, 'silu_bf16', dict(x=(x, F32, (T - 1) * ldx + K), y=(y, BF16, Tp * K)))
        self._go('pf_silu_bf16', Tp * K, x, ctypes.c_int(ldx), y, ctypes.c_int(T), ctypes.c_int(Tp), ctypes.c_int(K), ctypes.c_float(rs))

    def to_bf16(self, x, y, T, K, ldx=None):
        T, K = int(T), int(K); ldx = K if ldx is None else int(ldx); Tp = tpad(T)
        _check(self.dev, 'to_bf16', dict(x=(x, F32, (T - 1) * ldx + K), y=(y, BF16, Tp * K)))
        self._go('pf_to_bf16', Tp * K, x, ctypes.c_int(ldx), y, ctypes.c_int(T), ctypes.c_int(Tp), ctypes.c_int(K))
