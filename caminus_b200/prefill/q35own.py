"""The add + norm and IQ2_S embedding wrappers of the reference's dense-model prefill (python/caminus/prefill/q35own.py:130-140)."""
import ctypes

import torch

from ..device import cuda as hip

I, F = ctypes.c_int, ctypes.c_float
NULL = ctypes.c_void_p(0)
MODULE = 'q35_prefill'
MODULE_TCAP = 'q35_prefill_tcap'      # (the objects that hold the IQ2_S embedding kernel)
MODULE_GSQ = 'q35_prefill_gsq'


class Ops:
    def __init__(self, dev, module=MODULE):
        self.dev = torch.device(dev) if not isinstance(dev, torch.device) else dev
        self.module = module
        with torch.cuda.device(self.dev):
            self.mod = hip.Module(module)

    def add_rms16(self, x, nw, eps, h16, n, N, d=None, h=None):
        """per row: x += d (d None: no add); h = rms_norm(x) * nw (fp32, always written); h16 = its fp16 copy"""
        if N % 256 or not 256 <= N <= 65536: raise ValueError(f'q35 add_rms16: N {N} (a multiple of 256)')
        if h is None: raise ValueError('q35 add_rms16: h (the fp32 output) is required')
        with torch.cuda.device(self.dev):
            self.mod.q35p_add_rms16((int(n),), (256,), x, NULL if d is None else d, nw, F(eps), h, h16, I(N))

    def emb_iq2s(self, W, rb, vocab, toks, x, n, N):
        """x [n][N] = the IQ2_S embedding rows toks[i], the floats of the host decoder; the grid table comes from
        device.cuda.set_iq2s_grid (the reference's code object carries it as a constant)"""
        if self.module not in (MODULE_TCAP, MODULE_GSQ): raise ValueError(f'q35 emb_iq2s: the {MODULE_TCAP} / {MODULE_GSQ} objects only')
        with torch.cuda.device(self.dev):
            self.mod.q35t_emb_iq2s((int(n),), (256,), W, I(rb), I(vocab), toks, x, I(N))
