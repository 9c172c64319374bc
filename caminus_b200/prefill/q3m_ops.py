"""Launch wrappers of the glue ops of Qwen3-30B-A3B's batched prefill with the names, argument order and refusals of the
reference's class (python/caminus/prefill/q3m_ops.py:61-139: Ops.emb / add_rms16 / router / topk / group / swiglu / qk_rope),
over the B200 kernels. The GEMM and attention methods of the reference's class are not part of this library."""
import contextlib
import ctypes

import torch

from ..device import cuda as hip
from ..engine import k3

I, F = ctypes.c_int, ctypes.c_float
NULL = ctypes.c_void_p(0)
KVQ8_MODULE = 'q3m_prefill_kvq8'
YARN_MODULE = {False: 'q3m_prefill_yarn', True: 'q3m_prefill_kvq8_yarn'}
PLAIN_PAR = 2 * 128 + 2                            # q_norm | k_norm | theta_scale, eps
YARN_PAR = PLAIN_PAR + k3.YARN_TABLE_FLOATS        # ... | freq [64] | mscale
MM_M = 64                                          # pairs per grouped work item


def items_bound(npairs, n_exp):
    """an upper bound of the work items q3p_group writes: every expert may end in one partly filled item"""
    return (npairs + MM_M - 1) // MM_M + n_exp


def _opt(t):
    """an optional tensor argument: the null pointer when absent"""
    return NULL if t is None else t


class Ops:
    def __init__(self, dev, module='q3m_prefill', q8=False, yarn=False):
        """q8: the Q8_0 KV cache objects; yarn: the long-context objects (par then carries the YaRN table: YARN_PAR floats)"""
        self.dev = dev if isinstance(dev, torch.device) else torch.device(dev)
        self.module, self.q8, self.yarn = module, bool(q8), bool(yarn)
        if self.yarn and module != 'q3m_prefill':
            raise ValueError(f'q3m Ops: the long-context mode exists for q3m_prefill only, not for {module}')
        with torch.cuda.device(self.dev):
            self.mod = hip.Module(module)
            self.kvmod = hip.Module(KVQ8_MODULE) if self.q8 else None
            if self.yarn: self.ropemod = hip.Module(YARN_MODULE[self.q8])
            else: self.ropemod = self.kvmod if self.q8 else self.mod

    @contextlib.contextmanager
    def _here(self):
        """the launch's device is current inside the block (no switch when it already is)"""
        idx = self.dev.index
        if idx is None or torch.cuda.current_device() == idx:
            yield
        else:
            with torch.cuda.device(self.dev): yield

    def _go(self, mod, kernel, grid, block, *args):
        idx = self.dev.index
        if idx is None or torch.cuda.current_device() == idx: getattr(mod, kernel)(grid, block, *args)      # (the usual case: no context to enter)
        else:
            with torch.cuda.device(self.dev): getattr(mod, kernel)(grid, block, *args)

    # ---- embedding rows ---------------------------------------------------------------------------------------------------
    def emb(self, W, rb, vocab, toks, x, n, N):
        self._go(self.mod, 'q3p_emb', (n,), (256,), W, I(rb), I(vocab), toks, x, I(N))

    def emb_q6k(self, W, rb, vocab, toks, x, n, N):
        """as emb for a Q6_K table (rows of N / 256 * 210 bytes): the floats of own_dequant.q6_k (python/caminus/own_dequant.py:40-53)"""
        from .. import lib as _lib
        if N % 256 or rb < N // 256 * 210: raise ValueError(f'q3m emb_q6k: N {N} (a multiple of 256), rb {rb}')
        with self._here():
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(_lib.load().cam_emb_rows_q6k(n, W.data_ptr(), rb, vocab, toks.data_ptr(), x.data_ptr(), N, stream), 'cam_emb_rows_q6k')

    # ---- residual add + RMSNorm -----------------------------------------------------------------------------------------
    def add_rms16(self, x, nw, eps, h16, n, N, d=None, w=None, S=0, h=None):
        if N > 2048 or N % 256: raise ValueError(f'q3m add_rms16: row length {N} is not a multiple of 256 up to 2048')
        self._go(self.mod, 'q3p_add_rms16', (n,), (256,), x, _opt(d), _opt(w), I(S), nw, F(eps), _opt(h), h16, I(N))

    # ---- router glue -------------------------------------------------------------------------------------------------------
    def router(self, h, Wr, E, K, logits, n):
        if K % 128: raise ValueError(f'q3m router: row length {K} is not a multiple of 128')
        self._go(self.mod, 'q3p_router', (n,), (256,), h, Wr, I(E), I(K), logits)

    def topk(self, logits, E, k, floor_, ids, wts, err, n):
        if not (E <= 128 and k <= 32): raise ValueError(f'q3m topk: {E} experts (at most 128), top {k} (at most 32)')
        self._go(self.mod, 'q3p_topk', (n,), (32,), logits, I(E), I(k), F(floor_), ids, wts, err)

    def group(self, ids, npairs, k, E, xs, yd, items, nitems, err):
        if E > 1024: raise ValueError(f'q3m group: {E} experts (at most 1024)')
        self._go(self.mod, 'q3p_group', (1,), (1024,), ids, I(npairs), I(k), I(E), xs, yd, items, nitems, err)

    def check_flags(self, err, what='prefill'):
        """after the stream has drained: raise if a launch set the routing flag word (1: a router logit not finite; 2: an expert
        id out of range), and clear it (python/caminus/prefill/q3m.py:167-173)"""
        word = int(err.item())
        if word == 0: return
        err.zero_()
        raise k3.ContextBoundsError(f'{what}: routing flag word {word:#x} (bit 0: a router logit was not finite; bit 1: an expert id out of range)')

    def check_kv_code(self, err):
        """after the stream has drained: a Q8_0 KV encoder's error word (q3p_qk_rope_q8 ORs 2 into it for a refused block) raises
        InvalidKVEncoding; the word stays set (python/caminus/engine/k3.py:1653-1659)"""
        word = int(err.item())
        if word == 0: return
        from ..errors import InvalidKVEncoding
        raise InvalidKVEncoding(f'{getattr(self, "module", "q3m_prefill")}: a Q8_0 KV block was refused (error word {word:#x}); the appended cache rows are unusable')

    # ---- SwiGLU --------------------------------------------------------------------------------------------------------------
    def swiglu(self, g, u, y16, n):
        blocks = min((n + 255) // 256, 4096)
        self._go(self.mod, 'q3p_swiglu', (blocks,), (256,), g, u, y16, I(n))

    # ---- q/k norm + RoPE into the KV cache --------------------------------------------------------------------------------------
    def _span(self, what, cache, pos0, n, nkv, rows):
        """positions pos0 .. pos0 + n - 1 must be among the cache's first `rows` positions (None: every row of the allocation),
        else k3.ContextBoundsError and nothing is launched"""
        if n < 1 or nkv < 1: raise ValueError(f'q3m {what}: n {n}, nkv {nkv}')
        kind, dtype = ('Q8', torch.uint8) if self.q8 else ('F16', torch.float16)
        if cache.dtype != dtype: raise ValueError(f'q3m {what}: the {kind} prefill writes a {dtype} cache; this one is {cache.dtype}')
        held = k3.kv_rows(cache, nkv * 128, self.q8)
        if rows is not None and not 0 <= int(rows) <= held: raise ValueError(f'q3m {what}: rows {rows}, the cache holds {held}')
        k3.check_span(pos0, n, held if rows is None else int(rows), what=f'q3m {what}')

    def qk_rope(self, qkv, ldq, nh, nkv, par, pos0, q16, cache, n, rows=None, err=None):
        self._span('qk_rope', cache, pos0, n, nkv, rows)
        width = 128 * (nh + 2 * nkv)
        if ldq < width or qkv.numel() < (n - 1) * ldq + width or q16.numel() < n * nh * 128:
            raise ValueError(f'q3m qk_rope: {n} tokens take qkv rows of {width} values at stride {ldq} and {n * nh * 128} values of q16')
        need = YARN_PAR if self.yarn else PLAIN_PAR
        if par.dtype != torch.float32 or par.numel() < need:
            layout = 'q_norm | k_norm | theta_scale, eps' + (' | freq[64] | mscale' if self.yarn else '')
            raise ValueError(f'q3m qk_rope: par must hold {need} fp32 values ({layout}); got {par.numel()} of {par.dtype}')
        args = (qkv, I(ldq), I(nh), I(nkv), par, I(pos0), q16, cache)
        if not self.q8:
            if err is not None: raise ValueError('q3m qk_rope: an error word belongs to the Q8 cache form only')
            self._go(self.ropemod, 'q3p_qk_rope', (n, nh + nkv), (128,), *args)
            return
        if err is None or err.dtype != torch.int32 or err.numel() < 1: raise ValueError('q3m qk_rope: the Q8 cache form needs its int32 error word')
        if cache.data_ptr() % 4 or not cache.is_contiguous(): raise ValueError('q3m qk_rope: the Q8 cache must be contiguous and 4-byte aligned')
        self._go(self.ropemod, 'q3p_qk_rope_q8', (n, nh + nkv), (128,), *args, err)
