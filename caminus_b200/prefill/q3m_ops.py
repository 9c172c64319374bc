"""The glue part of the reference's launch wrappers for Qwen3-30B-A3B's batched prefill
(python/caminus/prefill/q3m_ops.py:61-139: Ops.emb / add_rms16 / swiglu / qk_rope), same names, argument meaning and
refusals, over the B200 kernels. The GEMM, router and attention methods of the reference's class are not part of this
library (contractions and the scheduler are outside its path)."""
import ctypes

import torch

from ..device import cuda as hip
from ..engine import k3

I, F = ctypes.c_int, ctypes.c_float
NULL = ctypes.c_void_p(0)
KVQ8_MODULE = 'q3m_prefill_kvq8'
YARN_MODULE = {False: 'q3m_prefill_yarn', True: 'q3m_prefill_kvq8_yarn'}
YARN_PAR = 2 * 128 + 2 + k3.YARN_TABLE_FLOATS      # q_norm | k_norm | theta_scale, eps | freq [64] | mscale


MM_M = 64                    # pairs per grouped work item


def items_bound(npairs, n_exp):
    """the most work items q3p_group can write for npairs pairs over n_exp experts"""
    return -(-npairs // MM_M) + n_exp


class _On:
    """`with _On(dev):` makes dev the current device for a launch; free when it already is (the common case)"""
    __slots__ = ('dev', 'ctx')

    def __init__(self, dev): self.dev, self.ctx = dev, None

    def __enter__(self):
        if self.dev.index is not None and torch.cuda.current_device() != self.dev.index:
            self.ctx = torch.cuda.device(self.dev); self.ctx.__enter__()

    def __exit__(self, *a):
        if self.ctx is not None: self.ctx.__exit__(*a); self.ctx = None


class Ops:
    def __init__(self, dev, module='q3m_prefill', q8=False, yarn=False):
        """yarn: the long-context mode: qk_rope reads the YaRN table after eps in par (YARN_PAR floats)"""
        self.dev = torch.device(dev) if not isinstance(dev, torch.device) else dev
        self.module, self.q8, self.yarn = module, bool(q8), bool(yarn)
        if self.yarn and module != 'q3m_prefill': raise ValueError(f'q3m Ops: the long-context mode runs with q3m_prefill only (not {module})')
        with torch.cuda.device(self.dev):
            self.mod = hip.Module(module)
            self.kvmod = hip.Module(KVQ8_MODULE) if self.q8 else None
            self.ropemod = hip.Module(YARN_MODULE[self.q8]) if self.yarn else (self.kvmod if self.q8 else self.mod)

    # -- the glue ----------------------------------------------------------------------------------------------------------
    def emb(self, W, rb, vocab, toks, x, n, N):
        with _On(self.dev):
            self.mod.q3p_emb((n,), (256,), W, I(rb), I(vocab), toks, x, I(N))

    def emb_q6k(self, W, rb, vocab, toks, x, n, N):
        """as emb for a Q6_K table (rows of N / 256 * 210 bytes): the floats of own_dequant.q6_k (python/caminus/own_dequant.py:40-53)"""
        from .. import lib as _lib
        if N % 256 or rb < N // 256 * 210: raise ValueError(f'q3m emb_q6k: N {N} (a multiple of 256), rb {rb}')
        with _On(self.dev):
            _lib.check(_lib.load().cam_emb_rows_q6k(n, W.data_ptr(), rb, vocab, toks.data_ptr(), x.data_ptr(), N, torch.cuda.current_stream().cuda_stream), 'cam_emb_rows_q6k')

    def add_rms16(self, x, nw, eps, h16, n, N, d=None, w=None, S=0, h=None):
        if N % 256 or N > 2048: raise ValueError(f'q3m add_rms16: N {N} (a multiple of 256, <= 2048)')
        with _On(self.dev):
            self.mod.q3p_add_rms16((n,), (256,), x, NULL if d is None else d, NULL if w is None else w, I(S), nw, F(eps),
                                   NULL if h is None else h, h16, I(N))

    def router(self, h, Wr, E, K, logits, n):
        if K % 128: raise ValueError(f'q3m router: K {K} (a multiple of 128)')
        with _On(self.dev): self.mod.q3p_router((n,), (256,), h, Wr, I(E), I(K), logits)

    def topk(self, logits, E, k, floor_, ids, wts, err, n):
        if E > 128 or k > 32: raise ValueError(f'q3m topk: E {E} (<= 128), k {k} (<= 32)')
        with _On(self.dev): self.mod.q3p_topk((n,), (32,), logits, I(E), I(k), F(floor_), ids, wts, err)

    def group(self, ids, npairs, k, E, xs, yd, items, nitems, err):
        if E > 1024: raise ValueError(f'q3m group: E {E} (<= 1024)')
        with _On(self.dev): self.mod.q3p_group((1,), (1024,), ids, I(npairs), I(k), I(E), xs, yd, items, nitems, err)

    def check_flags(self, err, what='prefill'):
        """after the stream has drained: raise if a launch set the routing flag word (1: a router logit not finite; 2: an expert
        id out of range), and clear it (python/caminus/prefill/q3m.py:167-173)"""
        e = int(err.item())
        if e:
            err.zero_()
            raise k3.ContextBoundsError(f'{what}: the routing flag word is {e:#x} (1: a router logit not finite, 2: an id out of range)')

    def check_kv_code(self, err):
        """after the stream has drained: a Q8_0 KV encoder's error word (q3p_qk_rope_q8 ORs 2 into it for a refused block) raises
        InvalidKVEncoding; the word stays set (python/caminus/engine/k3.py:1653-1659)"""
        code = int(err.item())
        if code:
            from ..errors import InvalidKVEncoding
            raise InvalidKVEncoding(f'q3m_prefill: invalid KV encoding (error {code:#x}); cache result is unusable')

    def swiglu(self, g, u, y16, n):
        with _On(self.dev):
            self.mod.q3p_swiglu((min(-(-n // 256), 4096),), (256,), g, u, y16, I(n))

    def _span(self, what, cache, pos0, n, nkv, rows):
        """positions pos0 .. pos0 + n - 1 must be among the cache's first `rows` positions (2 * nkv * 128 fp16 per row; None:
        every row of the allocation), else k3.ContextBoundsError and nothing is launched"""
        if n < 1 or nkv < 1: raise ValueError(f'q3m {what}: n {n}, nkv {nkv}')
        want = torch.uint8 if self.q8 else torch.float16
        if cache.dtype != want: raise ValueError(f'q3m {what}: a {"Q8" if self.q8 else "F16"} prefill needs a {want} cache, not {cache.dtype}')
        alloc = k3.kv_rows(cache, nkv * 128, self.q8)
        if rows is not None and not 0 <= int(rows) <= alloc: raise ValueError(f'q3m {what}: rows {rows} of a cache of {alloc}')
        k3.check_span(pos0, n, alloc if rows is None else int(rows), what=f'q3m {what}')

    def qk_rope(self, qkv, ldq, nh, nkv, par, pos0, q16, cache, n, rows=None, err=None):
        self._span('qk_rope', cache, pos0, n, nkv, rows)
        if ldq < (nh + 2 * nkv) * 128 or qkv.numel() < (n - 1) * ldq + (nh + 2 * nkv) * 128 or q16.numel() < n * nh * 128:
            raise ValueError(f'q3m qk_rope: {n} tokens need qkv rows of {(nh + 2 * nkv) * 128} (stride {ldq}) and {n * nh * 128} q16')
        if par.dtype != torch.float32 or par.numel() < (YARN_PAR if self.yarn else 2 * 128 + 2):
            raise ValueError(f'q3m qk_rope: par needs {YARN_PAR if self.yarn else 2 * 128 + 2} fp32 values'
                             f'{" (q_norm | k_norm | theta_scale, eps | the YaRN table)" if self.yarn else ""}, not {par.numel()} {par.dtype}')
        if self.q8:
            if err is None or err.dtype != torch.int32 or err.numel() < 1: raise ValueError('q3m qk_rope: a Q8 cache needs its int32 error word')
            if not cache.is_contiguous() or cache.data_ptr() % 4: raise ValueError('q3m qk_rope: the Q8 cache must be contiguous and 4-byte aligned')
            with _On(self.dev):
                self.ropemod.q3p_qk_rope_q8((n, nh + nkv), (128,), qkv, I(ldq), I(nh), I(nkv), par, I(pos0), q16, cache, err)
            return
        if err is not None: raise ValueError('q3m qk_rope: err is the Q8 cache\'s word')
        with _On(self.dev):
            self.ropemod.q3p_qk_rope((n, nh + nkv), (128,), qkv, I(ldq), I(nh), I(nkv), par, I(pos0), q16, cache)
