"""Multi-GPU forms: token rows sharded over ranks (no communication), and the tensor-parallel RMSNorm.

One process per GPU with torch.distributed. Row sharding needs no collective: every op of this library works on
independent rows, so rank r of G takes rows [r T / G, (r + 1) T / G) and the norm weights, the par block and the Q4_K table
are replicated. The tensor-parallel RMSNorm shards the hidden dimension instead: each rank reduces its columns to one fp32
sum of squares per row, the [T] partials are all-reduced (the only bytes that cross NVLink), and each rank normalises its
own columns. The reference has no counterpart: it replicates norms and the residual on both of its cards
(python/caminus/engine/q3moe_tp.py:18-20).
"""
import torch
import torch.distributed as dist

from . import lib as _lib


def row_shard(T, rank, world):
    """[a, b): the token rows of `rank` when T rows are split over `world` ranks in order (sizes differ by at most one)"""
    if not 0 <= rank < world: raise ValueError(f'row_shard: rank {rank} of {world}')
    return T * rank // world, T * (rank + 1) // world


def col_shard(N, rank, world, multiple=8):
    """[a, b): the hidden columns of `rank`; every shard a multiple of `multiple` columns (the kernels read 16 bytes at a time)"""
    if N % (world * multiple): raise ValueError(f'col_shard: {N} columns do not split into {world} shards of a multiple of {multiple}')
    w = N // world
    return rank * w, (rank + 1) * w


class TPRmsNorm:
    """RMSNorm over a hidden dimension sharded across the ranks of `group`.

    __call__(x, d): x fp16 [T, Ns] is this rank's column shard (updated in place to fp16(x + d) when d is given);
    returns h16 fp16 [T, Ns]. ss is a reusable fp32 [T] buffer (allocated on first use per T and device).
    `all_reduce` may be replaced (tests inject a gloo group or a stub)."""

    def __init__(self, nw_shard, Nfull, eps=1e-6, group=None, all_reduce=None):
        self.nw, self.Nfull, self.eps, self.group = nw_shard, int(Nfull), float(eps), group
        self._ss = None
        self._all_reduce = all_reduce or (lambda t: dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group))

    def partial(self, x, d=None):
        T, Ns = x.shape
        if self._ss is None or self._ss.numel() != T or self._ss.device != x.device:
            self._ss = torch.empty(T, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            s = torch.cuda.current_stream().cuda_stream
            _lib.check(_lib.load().cam_rms_partial_f16(T, x.data_ptr(), 0 if d is None else d.data_ptr(), self._ss.data_ptr(), Ns, s),
                       'cam_rms_partial_f16')
        return self._ss

    def apply(self, x, tot, h16=None, d=None):
        T, Ns = x.shape
        if h16 is None: h16 = torch.empty_like(x)
        with torch.cuda.device(x.device):
            s = torch.cuda.current_stream().cuda_stream
            _lib.check(_lib.load().cam_rms_apply_f16(T, x.data_ptr(), 0 if d is None else d.data_ptr(), tot.data_ptr(),
                                                     self.nw.data_ptr(), self.eps, h16.data_ptr(), Ns, self.Nfull, s), 'cam_rms_apply_f16')
        return h16

    def __call__(self, x, d=None, h16=None):
        if x.dtype != torch.float16 or not x.is_contiguous() or x.dim() != 2 or x.shape[1] % 8:
            raise ValueError(f'TPRmsNorm: x must be contiguous fp16 [T, Ns] with Ns a multiple of 8, not {tuple(x.shape)} {x.dtype}')
        if d is not None and (d.shape != x.shape or d.dtype != x.dtype or not d.is_contiguous()):
            raise ValueError('TPRmsNorm: d must match x')
        if self.nw.numel() != x.shape[1]: raise ValueError(f'TPRmsNorm: {self.nw.numel()} weights for {x.shape[1]} columns')
        ss = self.partial(x, d)
        self._all_reduce(ss)
        return self.apply(x, ss, h16, d)
