"""The fp16-storage forms of the glue ops (the shapes the benchmark configs name) and the per-layer sequence.

The reference's glue kernels take fp32 activations (GEMM outputs); these entries run the same statements between an exact
fp16 load and a rounded fp16 store. Every function launches on the tensors' device and torch's current stream, allocates
nothing unless an output is omitted, and refuses bad shapes on the host before any launch.
"""
import torch

from . import lib as _lib
from .engine import gguf as _gguf
from .engine import k3


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _need(t, dtype, numel, what):
    if t.dtype != dtype or t.numel() < numel or not t.is_contiguous() or not t.is_cuda:
        raise ValueError(f'{what}: needs a contiguous CUDA {dtype} tensor of {numel} values, not {tuple(t.shape)} {t.dtype} on {t.device}')


def add_rms_f16(x, nw, eps, h16=None, d=None):
    """x fp16 [n, N] (updated in place to fp16(x + d) when d is given), nw fp32 [N] -> h16 fp16 [n, N] = the normed rows"""
    n, N = x.shape
    if N % 256: raise ValueError(f'add_rms_f16: N {N} (a multiple of 256)')
    _need(x, torch.float16, n * N, 'add_rms_f16 x'); _need(nw, torch.float32, N, 'add_rms_f16 nw')
    if d is not None: _need(d, torch.float16, n * N, 'add_rms_f16 d')
    if h16 is None: h16 = torch.empty_like(x)
    else: _need(h16, torch.float16, n * N, 'add_rms_f16 h16')
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().cam_add_rms_f16(n, x.data_ptr(), 0 if d is None else d.data_ptr(), nw.data_ptr(), float(eps),
                                               h16.data_ptr(), N, _stream(x)), 'cam_add_rms_f16')
    return h16


def qk_rope_f16(q, k, par, pos0, qo=None, ko=None, yarn=False):
    """q fp16 [n, nh, 128], k fp16 [n, nkv, 128] at positions pos0 .. pos0 + n - 1 -> (qo, ko) fp16 (None: in place).
    par fp32: q_norm[128] | k_norm[128] | theta_scale | eps (yarn: then freq[64] | mscale)."""
    n, nh, hd = q.shape; nkv = k.shape[1]
    if hd != 128 or k.shape[0] != n or k.shape[2] != 128: raise ValueError(f'qk_rope_f16: q {tuple(q.shape)}, k {tuple(k.shape)} (heads of 128)')
    k3.check_span(pos0, n, 1 << 22, what='qk_rope_f16')
    _need(q, torch.float16, n * nh * 128, 'qk_rope_f16 q'); _need(k, torch.float16, n * nkv * 128, 'qk_rope_f16 k')
    _need(par, torch.float32, 258 + (k3.YARN_TABLE_FLOATS if yarn else 0), 'qk_rope_f16 par')
    qo = q if qo is None else qo; ko = k if ko is None else ko
    _need(qo, torch.float16, n * nh * 128, 'qk_rope_f16 qo'); _need(ko, torch.float16, n * nkv * 128, 'qk_rope_f16 ko')
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().cam_qk_rope_f16(n, q.data_ptr(), k.data_ptr(), nh, nkv, par.data_ptr(), int(pos0), qo.data_ptr(),
                                               ko.data_ptr(), int(bool(yarn)), _stream(q)), 'cam_qk_rope_f16')
    return qo, ko


swiglu_q8_1 = _gguf.swiglu_q8_1


class LayerGlue:
    """One transformer layer's glue in the prefill's order (python/caminus/prefill/q3m.py:146-164 with the GEMMs and the
    attention left out): add + RMSNorm -> q/k norm + RoPE -> SwiGLU + Q8_1, on one device, for T token rows."""

    def __init__(self, nw, par, eps=1e-6, yarn=False):
        self.nw, self.par, self.eps, self.yarn = nw, par, float(eps), bool(yarn)

    def __call__(self, x, resid, q, k, gate, up, h16, yq, pos0=0):
        add_rms_f16(x, self.nw, self.eps, h16=h16, d=resid)
        qk_rope_f16(q, k, self.par, pos0, yarn=self.yarn)
        swiglu_q8_1(gate.reshape(-1), up.reshape(-1), yq)
        return h16, q, k, yq
