"""Launch the B200 glue kernels with the reference's loader interface.

The reference loads a gfx1100 code object per module and launches `extern "C"` kernels through hipModuleLaunchKernel:
    Module(name).<kernel>(grid, block, *args, shmem=0, stream=None)
(python/caminus/device/hip.py:77-123), each argument a torch tensor (passed as its device pointer) or a ctypes scalar.
This module gives the same two classes over libcaminus_b200.so, so the reference's op wrappers run on CUDA tensors by
assigning `caminus.device.hip.Module = caminus_b200.device.cuda.Module` (and the by-name imports of its wrappers).

What changes under the call: the AMD block shape is dropped (the kernels choose their own launch shape); where the
reference carries a row or head count only in the launch grid, it is read from `grid` and passed as the C entry's leading
argument; the module name selects the build variant the reference bakes into separate code objects (the YaRN RoPE).
Errors: an unknown module raises FileNotFoundError as a missing code object does; a refused argument ValueError; a
launch failure RuntimeError('CUDA error ...') (the reference: RuntimeError('HIP error ...'), device/hip.py:35-37).
"""
import ctypes

from .. import lib as _lib

# caminus.prefill.graph's recorder hook of the reference (device/hip.py:12-14): an object with intercept(...) / launched(...)
RECORD = None
LOADED = []    # module names this process asked for, in order (the reference's LOADED, device/hip.py:16)
CHECK_DEVICE = True   # refuse host tensors as kernel arguments (a test that records launches without a GPU clears it)

# kernel -> (C entry, how many leading counts come from the launch grid)
_Q3M = {'q3p_emb': ('q3p_emb', 1), 'q3p_add_rms16': ('q3p_add_rms16', 1), 'q3p_swiglu': ('q3p_swiglu', 0),
        'q3p_qk_rope': ('q3p_qk_rope', 1), 'q3p_router': ('q3p_router', 1), 'q3p_topk': ('q3p_topk', 1), 'q3p_group': ('q3p_group', 0)}
def _glue(K):
    """the hyper-connection glue object of row width K (the reference bakes K into the code object: GLUE_NI x 256)"""
    return {'pf_rms_mul': ('pf_rms_mul', 0, (K,)), 'pf_hc_post_rms': ('pf_hc_post_rms', 0, (K,)), 'pf_hc_post': ('pf_hc_post', 0),
            'pf_hc_mean': ('pf_hc_mean', 0), 'pf_router': ('pf_router', 1), 'pf_add_sum': ('pf_add_sum', 0), 'pf_silu_bf16': ('pf_silu_bf16', 0), 'pf_to_bf16': ('pf_to_bf16', 0)}


MODULES = {
    'prefill_glue': _glue(2560), 'prefill_glue_q35': _glue(2048), 'prefill_glue_q35d': _glue(5120),
    'prefill_tp': {'pf_swiglu': ('pf_swiglu', 0)},
    'prefill_attn': {'pf_qk_nr': ('pf_qk_nr', 1)},
    'core': {'embedding_f32': ('embedding_f32', 1), 'rmsnorm_f32': ('rmsnorm_f32', 1), 'silu_mul_bf16': ('silu_mul_bf16', 0),
             'residual3': ('residual3', 0), 'cast_bf16': ('cast_bf16', 0)},
    'fuse': {'residual_slices_fwd': ('residual_slices_fwd', 0)},
    'prefill_feed': {'embd_rows_iq4xs': ('embd_rows_iq4xs', 0), 'ple_rows_iq4nl': ('ple_rows_iq4nl', 0)},
    'actq': {k: (k, 1) for k in ('actq_fwd_bf16', 'actq_fwd_f32', 'actq_fwd_codes_bf16', 'actq_fwd_codes_f32', 'silu_mul_actq_fwd', 'block_entry_fwd')},
    'q3m_prefill': _Q3M,
    'q3m_prefill_yarn': dict(_Q3M, q3p_qk_rope=('q3p_qk_rope_yarn', 1)),
    'q3m_prefill_kvq8': {'q3p_qk_rope_q8': ('q3p_qk_rope_q8', 1)},
    'q3m_prefill_kvq8_yarn': {'q3p_qk_rope_q8': ('q3p_qk_rope_q8_yarn', 1)},
    'q35_prefill': {'q35p_add_rms16': ('q35p_add_rms16', 1)},
    'q35_prefill_tcap': {'q35p_add_rms16': ('q35p_add_rms16', 1), 'q35t_emb_iq2s': ('q35t_emb_iq2s', 1, (lambda: _iq2s_grid(),))},
    'q35_prefill_gsq': {'q35p_add_rms16': ('q35p_add_rms16', 1), 'q35t_emb_iq2s': ('q35t_emb_iq2s', 1, (lambda: _iq2s_grid(),))},
    'k3_gguf': {'gg_quantize_q8_1': ('gg_quantize_q8_1', 0), 'gg_silu_mul': ('gg_silu_mul', 0)},
    'k3_gguf_gsq': {'gg_quantize_q8_1': ('gg_quantize_q8_1', 0), 'gg_silu_mul': ('gg_silu_mul', 0)},
}


def check(err):
    _lib.check(err)


# GGUF's IQ2_S grid, a constant of the reference's q35_prefill_tcap / _gsq code objects (kernels/iq2s_grid.h, generated from
# python/caminus/iq_tables.py:747-768). This library does not carry the table: the caller hands it over once per device.
_IQ2S = {}


def pack_iq2s_grid(grid):
    """grid: the reference's iq_tables.GRID_IQ2_S (uint8 [1024, 8], magnitudes 8 / 25 / 43) or its packed form (uint32 / int32 [512]);
    returns the packed words (uint32 [512]: 2-bit codes 0 / 1 / 2 at bits 2 k, entry 2 w in word w's low half, kernels/iq2s_grid.h)"""
    import numpy as np
    g = np.asarray(grid)
    if g.size == 8192:
        m = g.astype(np.uint8).reshape(1024, 8)
        if not np.isin(m, (8, 25, 43)).all(): raise ValueError('IQ2_S grid: magnitudes other than 8 / 25 / 43')
        code = np.where(m == 8, 0, np.where(m == 25, 1, 2)).astype(np.uint32)
        e = (code << (2 * np.arange(8, dtype=np.uint32))).sum(axis=1).astype(np.uint32)
        return (e[0::2] | (e[1::2] << 16)).astype(np.uint32)
    if g.size != 512 or g.dtype.itemsize != 4:
        raise ValueError(f'IQ2_S grid: {g.size} values of {g.dtype}; expected uint8 [1024, 8] or 512 packed words')
    return np.ascontiguousarray(g).view(np.uint32).reshape(512).copy()


def set_iq2s_grid(grid, device=None):
    """hands the IQ2_S grid (either form pack_iq2s_grid takes, as a numpy array or tensor) to the library's launches on `device`
    (default: the current one)"""
    import numpy as np
    import torch
    g = pack_iq2s_grid(grid.detach().cpu().numpy() if torch.is_tensor(grid) else grid)
    dev = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    _IQ2S[idx] = torch.from_numpy(g.view(np.int32)).to(torch.device('cuda', idx))


def _iq2s_grid():
    import torch
    t = _IQ2S.get(torch.cuda.current_device())
    if t is None: raise RuntimeError('caminus_b200: q35t_emb_iq2s needs the IQ2_S grid: call caminus_b200.device.cuda.set_iq2s_grid(iq_tables.GRID_IQ2_S) once per device')
    return ctypes.c_void_p(t.data_ptr())


_torch = None
_Tensor = None


def _bind_torch():
    global _torch, _Tensor
    import torch
    _torch, _Tensor = torch, torch.Tensor


def _current_stream():
    if _torch is None: _bind_torch()
    return _torch.cuda.current_stream().cuda_stream


class Kernel:
    """one kernel of a code object: __call__(grid, block, *args, shmem=0, stream=None) as the reference's hip.Kernel. The call is the
    whole host cost of a decode-sized launch, so its path is short: tensors go down as their device addresses (plain integers),
    ctypes scalars as they are, and nothing is built that the launch does not need."""

    def __init__(self, module, name, entry, ngrid, tail=()):
        """tail: constants the reference bakes into the code object, passed as the entry's last arguments before the stream"""
        self.module, self.name, self.entry, self.ngrid, self.tail = module, name, entry, ngrid, tuple(tail)
        self.fn = getattr(_lib.load(), entry)
        self._heads = name in ('q3p_qk_rope', 'q3p_qk_rope_q8')      # grid.y is the reference's nh + nkv: checked against the arguments
        self._lazy_tail = any(callable(t) for t in self.tail)
        if _Tensor is None: _bind_torch()

    def __call__(self, grid, block, *args, shmem=0, stream=None):
        """args: torch tensors (passed as device pointers) or ctypes scalars (c_int, c_float, c_void_p(0) for null)"""
        T = _Tensor
        vals = []
        for a in args:
            if type(a) is T:
                if CHECK_DEVICE and not a.is_cuda: raise ValueError('caminus_b200: a kernel argument is a CPU tensor')
                vals.append(a.data_ptr())
            elif hasattr(a, 'data_ptr'):                             # (a tensor subclass or another array with a device address)
                if CHECK_DEVICE and getattr(a, 'is_cuda', True) is False: raise ValueError('caminus_b200: a kernel argument is a CPU tensor')
                vals.append(a.data_ptr())
            else:
                vals.append(a)
        s = _torch.cuda.current_stream().cuda_stream if stream is None else stream
        r = RECORD
        if r is not None:                                            # the recorder sees what the reference's loader hands it: c_void_p for tensors, 3-tuples
            vals = [ctypes.c_void_p(v) if type(v) is int else v for v in vals]
            grid, block = (tuple(grid) + (1, 1))[:3], (tuple(block) + (1, 1))[:3]
            if r.intercept(self, grid, block, vals, shmem, s): return
        if self._heads:
            nh, nkv = int(getattr(vals[2], 'value', vals[2])), int(getattr(vals[3], 'value', vals[3]))
            gy = grid[1] if len(grid) > 1 else 1
            if gy != nh + nkv: raise ValueError(f'{self.name}: grid.y {gy} is not nh + nkv = {nh + nkv}')
        tail = [t() if callable(t) else t for t in self.tail] if self._lazy_tail else self.tail      # (a callable: a per-device constant looked up at the launch)
        n = self.ngrid
        if n == 0: rc = self.fn(*vals, *tail, s)
        elif n == 1: rc = self.fn(int(grid[0]), *vals, *tail, s)
        else: rc = self.fn(*[int(grid[i]) for i in range(n)], *vals, *tail, s)
        if rc: _lib.check(rc, self.name)
        if r is not None: r.launched(self, grid, block, vals, shmem, s)


class Module:
    """one of the reference's code objects by name, served by the entries of libcaminus_b200.so"""

    def __init__(self, name):
        if name not in MODULES:
            raise FileNotFoundError(f'caminus_b200: no kernels for the code object {name!r} (have {", ".join(sorted(MODULES))}); '
                                    f'library {_lib.path()}')
        _lib.load()
        self._name, self._fns = name, {}
        if name not in LOADED: LOADED.append(name)

    def __getattr__(self, name):
        if name.startswith('_'): raise AttributeError(name)
        if name not in self._fns:
            spec = MODULES[self._name].get(name)
            if spec is None: raise RuntimeError(f'CUDA error: the code object {self._name} has no kernel {name}')
            self._fns[name] = Kernel(self._name, name, *spec)
        return self._fns[name]
