"""Multi-GPU forms: token rows sharded over ranks (no communication), and the tensor-parallel RMSNorm.

One process per GPU with torch.distributed. Row sharding needs no collective: every op of this library works on
independent rows, so rank r of G takes rows [r T / G, (r + 1) T / G) and the norm weights, the par block and the Q4_K table
are replicated. The tensor-parallel RMSNorm shards the hidden dimension instead: each rank reduces its columns to one fp32
sum of squares per row, the [T] partials are all-reduced (the only bytes that cross NVLink), and each rank normalises its
own columns. The reference has no counterpart: it replicates norms and the residual on both of its cards
(python/caminus/engine/q3moe_tp.py:18-20). TPRmsNormFused is the same norm as one kernel per rank: the partials go straight into
every rank's exchange buffer by peer stores over NVLink and a row is normalised as soon as its partials have arrived.
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


SOLO = object()      # group=SOLO: a single-rank exchange (world 1) even when torch.distributed is initialised


class TPExchange:
    """The per-rank side of the one-kernel tensor-parallel norm that does not depend on a layer: this rank's exchange buffer
    (2 * world * cap 64-bit words, zeroed), the other ranks' buffers mapped into this process through CUDA IPC (torch's tensor
    sharing; the handles travel by all_gather_object), the call counter (the tag every rank stamps its partials with) and the status
    word. ONE exchange per rank and group serves every layer's norm: the norms differ only in their weights, and an allocation
    exported once is mapped once by each peer. Every rank of `group` constructs it with the same `cap` (rows per call at most);
    construction ends with a collective, so no rank launches before all have mapped. One rank per GPU: two ranks' kernels on one
    GPU would wait for each other. close() after the last call has finished on every rank (the caller's barrier)."""

    def __init__(self, cap, group=None, device=None):
        self.cap, self.group = int(cap), None if group is SOLO else group
        self.dev = torch.device(device) if device is not None else torch.device('cuda', torch.cuda.current_device())
        one = group is SOLO or (group is None and not dist.is_initialized())
        self.world = 1 if one else dist.get_world_size(self.group)
        self.rank = 0 if one else dist.get_rank(self.group)
        L = _lib.load()
        words = L.cam_tp_rms_words(self.cap, self.world)
        if words < 0: raise ValueError(f'TPExchange: cap {cap}, world {self.world}')
        self.buf = torch.zeros(words, dtype=torch.int64, device=self.dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.tag = 0
        self._mapped = []                                        # bases of the peers' allocations mapped into this process
        self._export = None
        ptrs = [0] * self.world
        if self.world > 1:
            import ctypes
            torch.cuda.synchronize(self.dev)                     # the zeros are in place before any peer can write
            # CUDA IPC: the handle of the allocation that holds buf and buf's offset in it (torch's own export call, which also
            # keeps the allocation from being reused while it is shared)
            shared = self.buf.untyped_storage()._share_cuda_()
            raw = bytes(shared[1])
            # (torch wraps the 64-byte cudaIpcMemHandle_t: a version byte and a kind byte, 'c' = a cudaMalloc block, in front)
            if len(raw) < 64 or (len(raw) > 64 and raw[-65:-64] != b'c'):
                raise RuntimeError(f'TPExchange: the allocator exported a handle this code does not map ({len(raw)} bytes, kind {raw[-65:-64]!r}): '
                                   'expandable segments are not supported')
            self._export = (shared[4], shared[5])                # the allocator's count of importers for this export (released in close)
            mine = (raw[-64:], int(shared[3]))
            everyone = [None] * self.world
            dist.all_gather_object(everyone, mine, group=self.group)
            failed = None
            try:
                with torch.cuda.device(self.dev):
                    for r, (handle, offset) in enumerate(everyone):
                        if r == self.rank: continue
                        base = ctypes.c_void_p()
                        _lib.check(L.cam_ipc_open(handle, ctypes.byref(base)), f'cam_ipc_open (rank {r})')
                        self._mapped.append(base)
                        ptrs[r] = base.value + offset
            except Exception as e:                               # (reported below on every rank: no rank is left waiting for this one)
                failed = e
            # every rank has mapped every buffer before the first launch, or every rank learns that one could not
            flag = torch.tensor([0 if failed is None else 1], dtype=torch.int32, device=self.dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
            if int(flag.item()):
                self.close()
                raise RuntimeError('TPExchange: a rank could not map a peer\'s exchange buffer' + (f': {failed}' if failed else '')) from failed
        ptrs[self.rank] = self.buf.data_ptr()
        self.peers = torch.tensor(ptrs, dtype=torch.int64, device=self.dev)

    def next_tag(self):
        """the tag of the next launch: 1, 2, .. (never 0; consecutive launches alternate parity). Taken only for a call that
        launches: a call without rows must not advance it, or two launches in a row would share a half of the buffer"""
        self.tag = self.tag % 0xfffffffe + 1
        return self.tag

    def close(self):
        """unmap the peers' buffers (after the last call has finished on every rank: the caller's barrier). Keep this object (its
        buffer) alive until every rank has closed"""
        torch.cuda.synchronize(self.dev)
        with torch.cuda.device(self.dev):
            for base in self._mapped: _lib.load().cam_ipc_close(base)
        self._mapped = []
        if self._export is not None:
            # the export counted one importer that the allocator expects to report back; the peers map the block through this library
            # instead, so the exporter reports for them (else the allocator warns at exit that the block was still shared)
            handle, offset = self._export
            self._export = None
            try: torch.UntypedStorage._release_ipc_counter(handle, offset, device=self.dev)
            except Exception: pass                               # (bookkeeping only)

    def check(self):
        """synchronises and raises if a wait ran out (a rank that did not make the matching call). After that the rows of the failed
        call are in an unknown state: some hold fp16(x + d) and their norm, the rest are untouched; restore x from a copy to retry"""
        torch.cuda.synchronize(self.dev)
        if int(self.status.item()) != 0:
            self.status.zero_()
            raise RuntimeError('TPRmsNormFused: a wait for another rank ran out (a rank did not make the matching call); the call\'s rows are partly updated')


class TPRmsNormFused:
    """The tensor-parallel RMSNorm as ONE launch per rank (cam_tp_rms_norm_f16): no collective call, no second pass over HBM.

    A norm is its weights plus a TPExchange. Pass `exchange` to share one exchange among all the norms of a model (the ranks then
    make the same sequence of calls over all of them); without it the norm builds its own from `cap` and `group`, which is meant
    for a single norm: every further exchange is another allocation exported to and mapped by every peer.
    __call__(x, d) as TPRmsNorm.__call__. check() synchronises and raises if a wait ran out (a rank that did not take part)."""

    def __init__(self, nw_shard, Nfull, cap=None, eps=1e-6, group=None, device=None, exchange=None):
        self.nw, self.Nfull, self.eps = nw_shard, int(Nfull), float(eps)
        if exchange is None:
            if cap is None: raise ValueError('TPRmsNormFused: give cap (rows per call at most) or an exchange')
            exchange = TPExchange(cap, group, device if device is not None else nw_shard.device); self._own = True
        else:
            self._own = False
        self.ex = exchange
        self.dev, self.cap, self.world, self.rank = exchange.dev, exchange.cap, exchange.world, exchange.rank

    @property
    def tag(self): return self.ex.tag

    def __call__(self, x, d=None, h16=None):
        if x.dtype != torch.float16 or not x.is_contiguous() or x.dim() != 2 or x.shape[1] % 8 or x.device != self.dev:
            raise ValueError(f'TPRmsNormFused: x must be contiguous fp16 [T, Ns] on {self.dev} with Ns a multiple of 8, not {tuple(x.shape)} {x.dtype}')
        if d is not None and (d.shape != x.shape or d.dtype != x.dtype or not d.is_contiguous()):
            raise ValueError('TPRmsNormFused: d must match x')
        if self.nw.numel() != x.shape[1]: raise ValueError(f'TPRmsNormFused: {self.nw.numel()} weights for {x.shape[1]} columns')
        T, Ns = x.shape
        if T > self.cap: raise ValueError(f'TPRmsNormFused: {T} rows, built for {self.cap}')
        if h16 is None: h16 = torch.empty_like(x)
        if T == 0: return h16                                    # (nothing launches: the tag stays)
        ex = self.ex
        tag = ex.next_tag()
        with torch.cuda.device(self.dev):
            s = torch.cuda.current_stream().cuda_stream
            _lib.check(_lib.load().cam_tp_rms_norm_f16(T, x.data_ptr(), 0 if d is None else d.data_ptr(), self.nw.data_ptr(), self.eps, h16.data_ptr(),
                                                       Ns, self.Nfull, ex.peers.data_ptr(), ex.rank, ex.world, ex.cap, tag,
                                                       ex.status.data_ptr(), s), 'cam_tp_rms_norm_f16')
        return h16

    def close(self):
        """closes the exchange this norm built itself (a shared one is closed by whoever built it)"""
        if self._own: self.ex.close()

    def check(self):
        self.ex.check()
