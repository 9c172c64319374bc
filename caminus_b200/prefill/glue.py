"""Host side of the hyper-connection ("Coder") glue: the methods rms_mul, hc_post_rms, hc_post, hc_mean, router, add_sum, silu_bf16
and to_bf16 of the reference's class Glue (python/caminus/prefill/glue.py:96-313) with its names, argument meaning and refusals,
over the B200 kernels. The router-logit matrices, GDN, PLE and BF16-matrix methods of that class are outside this library's path."""
import ctypes

import torch

from ..device.cuda import Module

TPAD = 128                                         # rows of the GEMM operands come in multiples of this
GLUE_MODULES = {'prefill_glue': 2560, 'prefill_glue_q35': 2048, 'prefill_glue_q35d': 5120}     # code object -> row width
D_GLUE = GLUE_MODULES['prefill_glue']
F32, BF16, I32 = torch.float32, torch.bfloat16, torch.int32
_i, _f, _l = ctypes.c_int, ctypes.c_float, ctypes.c_long
_NULL = ctypes.c_void_p(0)


def tpad(T):
    """T rounded up to the GEMMs' row padding"""
    return -(-int(T) // TPAD) * TPAD


def _check(dev, what, bufs, opt=()):
    """refuses a launch whose buffers do not fit: every entry of bufs is (tensor, dtype, least number of elements); a tensor must
    live on dev, be contiguous, have that dtype and at least that many elements; names in opt may be None. (The reference states
    the same per launch with device/bufcheck.LaunchCheck, python/caminus/device/bufcheck.py:1-27, which also analyses overlaps.)"""
    for name, (t, dtype, least) in bufs.items():
        if t is None and name in opt: continue
        if t is None: raise ValueError(f'{what}: {name} is missing')
        ok = torch.is_tensor(t) and t.device == dev and t.dtype == dtype and t.is_contiguous() and t.numel() >= least
        if not ok: raise ValueError(f'{what}: {name} must be a contiguous {dtype} tensor on {dev} with at least {least} elements')


class Glue:
    module, D = 'prefill_glue', D_GLUE

    def __init__(self, device, module='prefill_glue'):
        dev = torch.device(device)
        self.dev = dev if dev.index is not None else torch.device('cuda', torch.cuda.current_device())
        if module not in GLUE_MODULES: raise ValueError(f'Glue: no glue object {module!r}; there are {sorted(GLUE_MODULES)}')
        self.module, self.D = module, GLUE_MODULES[module]
        with torch.cuda.device(self.dev): self.m = Module(module)

    def _go(self, kernel, units, *args, threads=256):
        """launch `kernel` over `units` work units of the reference's grid (threads per block as there)"""
        blocks = -(-int(units) // threads)
        with torch.cuda.device(self.dev): getattr(self.m, kernel)((blocks,), (threads,), *args)

    @staticmethod
    def _nul(t):
        return _NULL if t is None else t

    # ---- norms -------------------------------------------------------------------------------------------------------------
    def rms_mul(self, x, w, y, R, eps, ybf=None, scale=None):
        """R rows of D: y[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * w[r % wr], w holding wr rows (wr divides R). Any of the outputs
        may be left out, not all: y fp32 (may be x itself), ybf the bf16 copy, scale [R] the rows' rsqrt factors"""
        R, K = int(R), self.D
        wr = w.numel() // K
        if R < 1 or wr < 1 or wr * K != w.numel() or R % wr: raise ValueError(f'rms_mul: {R} rows with weights of {w.numel()} values (rows of {K})')
        if (y, ybf, scale) == (None, None, None): raise ValueError('rms_mul: asks for no output')
        _check(self.dev, 'rms_mul', {'x': (x, F32, R * K), 'w': (w, F32, wr * K), 'y': (y, F32, R * K), 'ybf': (ybf, BF16, R * K),
                                     'scale': (scale, F32, R)}, opt=('y', 'ybf', 'scale'))
        self._go('pf_rms_mul', R * 256, x, w, self._nul(y), self._nul(ybf), self._nul(scale), _i(R), _i(wr), _f(eps))

    def hc_post_rms(self, block, inj, res, w, T, HC, eps, rs=0.25, xn=None, xnbf=None, scale=None):
        """the stream update res[t, h] += block[t] * 2 sigmoid(rs * inj[t, h]) in place, followed by the norm of every
        (token, stream) row with w[h]; outputs as rms_mul's"""
        T, HC, D = int(T), int(HC), self.D
        rows = T * HC
        _check(self.dev, 'hc_post_rms', {'block': (block, F32, T * D), 'inj': (inj, F32, rows), 'res': (res, F32, rows * D), 'w': (w, F32, HC * D),
                                         'xn': (xn, F32, rows * D), 'xnbf': (xnbf, BF16, rows * D), 'scale': (scale, F32, rows)}, opt=('xn', 'xnbf', 'scale'))
        self._go('pf_hc_post_rms', rows * 256, block, inj, res, w, self._nul(xn), self._nul(xnbf), self._nul(scale), _i(T), _i(HC), _f(rs), _f(eps))

    # ---- stream updates and the gated mean ---------------------------------------------------------------------------------------
    def hc_post(self, block, inj, res, T, HC, D=None, rs=0.25):
        T, HC = int(T), int(HC); D = self.D if D is None else int(D)
        _check(self.dev, 'hc_post', {'block': (block, F32, T * D), 'inj': (inj, F32, T * HC), 'res': (res, F32, T * HC * D)})
        self._go('pf_hc_post', T * D, block, inj, res, _i(T), _i(HC), _i(D), _f(rs))

    def hc_mean(self, xn, gate, out, T, HC, D=None, rs=0.25, scale=None, w=None):
        T, HC = int(T), int(HC); D = self.D if D is None else int(D)
        if (scale is None) is not (w is None): raise ValueError('hc_mean: scale and w are given together or not at all')
        _check(self.dev, 'hc_mean', {'xn': (xn, F32, T * HC * D), 'gate': (gate, F32, T * HC * D), 'out': (out, F32, T * D),
                                     'scale': (scale, F32, T * HC), 'w': (w, F32, HC * D)}, opt=('scale', 'w'))
        self._go('pf_hc_mean', T * D, xn, self._nul(scale), self._nul(w), gate, out, _i(T), _i(HC), _i(D), _f(rs))

    # ---- the router: softmax + top-k of a token's expert logits ---------------------------------------------------------------
    def router(self, logits, T, E, k, ids, wts, err, clamp=6.103515625e-5):
        """logits [T, E] -> ids [T, k] int32 and wts [T, k] = p / max(sum of the k, clamp), in rank order (most probable first, ties
        to the lower index); err: the sticky routing flag word (bit 0: a logit was NaN or infinite)"""
        T, E, k = int(T), int(E), int(k)
        if T < 1 or not (1 <= E <= 1024 and 1 <= k <= min(64, E)): raise ValueError(f'router: T {T}, E {E}, k {k}')
        _check(self.dev, 'router', {'logits': (logits, F32, T * E), 'ids': (ids, I32, T * k), 'wts': (wts, F32, T * k), 'err': (err, I32, 1)})
        with torch.cuda.device(self.dev): self.m.pf_router((T,), (256,), logits, _i(E), _i(k), _f(clamp), ids, wts, err)

    def add_sum(self, a, b, y, n):
        """y[i] += a[i] + b[i] for n values"""
        n = int(n)
        _check(self.dev, 'add_sum', {'a': (a, F32, n), 'b': (b, F32, n), 'y': (y, F32, n)})
        self._go('pf_add_sum', n, a, b, y, _l(n))

    # ---- bf16 operands of the GEMMs -------------------------------------------------------------------------------------------
    def _rows_to_bf16(self, kernel, x, y, T, K, ldx, *tail):
        T, K = int(T), int(K); ldx = K if ldx is None else int(ldx)
        Tp = tpad(T)
        _check(self.dev, kernel[3:], {'x': (x, F32, (T - 1) * ldx + K), 'y': (y, BF16, Tp * K)})
        self._go(kernel, Tp * K, x, _i(ldx), y, _i(T), _i(Tp), _i(K), *tail)

    def silu_bf16(self, x, y, T, K, rs, ldx=None):
        """y [tpad(T), K] bf16: rows t < T are bf16(silu(fma(rs, x[t], 0))) (x has row stride ldx), the padding rows zero"""
        self._rows_to_bf16('pf_silu_bf16', x, y, T, K, ldx, _f(rs))

    def to_bf16(self, x, y, T, K, ldx=None):
        """y [tpad(T), K] bf16: the bf16 copy of x's T rows, the padding rows zero"""
        self._rows_to_bf16('pf_to_bf16', x, y, T, K, ldx)
