"""The reference's OWN wrapper classes over this library's loader, without a GPU. With CAMINUS_REFERENCE naming a checkout of the
reference, its Python package is imported, the assignments a maintainer makes (one Module class for another) are applied, and its
wrappers are called: caminus.prefill.q3m_ops.Ops, caminus.prefill.q35own.Ops, caminus.prefill.glue.Glue, caminus.engine.gguf, the
forwards of caminus.train.actq and caminus.train.fuse. The library's entries are replaced by recorders, so nothing computes: what is
checked is that every launch those wrappers make resolves to an entry of include/caminus_b200.h and hands it exactly the arguments the
entry declares: their number, their order and the ctypes kind of each (pointer, int, long, float), with the counts the reference
carries in its launch grid as the leading arguments. Skipped when CAMINUS_REFERENCE is not set."""
import contextlib
import ctypes
import os
import sys

import pytest

torch = pytest.importorskip('torch')

REF = os.environ.get('CAMINUS_REFERENCE', '')
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, 'python', 'caminus')), reason='CAMINUS_REFERENCE does not name a checkout of the reference')

from caminus_b200 import lib   # noqa: E402
from caminus_b200.device import cuda as b200   # noqa: E402

KIND = {lib.P: 'pointer', lib.I: 'int', lib.L: 'long', lib.F: 'float', lib.U: 'unsigned'}


def kind_of(a):
    if isinstance(a, (ctypes.c_void_p,)): return 'pointer'
    if isinstance(a, int): return 'pointer-or-int'                    # a tensor's address, the stream, or a count read from the grid
    if isinstance(a, ctypes.c_float): return 'float'
    if isinstance(a, ctypes.c_int): return 'int'
    if isinstance(a, (ctypes.c_long, ctypes.c_longlong)): return 'long'
    if isinstance(a, ctypes.c_uint): return 'unsigned'
    return type(a).__name__


class Recorder:
    """stands in for one entry of the library: checks a call against the entry's declared arguments, keeps it, launches nothing"""
    log = []

    def __init__(self, entry): self.entry = entry

    def __call__(self, *args):
        want = lib.SIGNATURES[self.entry]
        assert len(args) == len(want), f'{self.entry}: {len(args)} arguments for {len(want)} declared'
        for i, (a, w) in enumerate(zip(args, want)):
            k = kind_of(a)
            ok = k == KIND[w] or (k == 'pointer-or-int' and KIND[w] in ('pointer', 'int', 'long'))
            assert ok, f'{self.entry}: argument {i} is a {k}, the entry declares a {KIND[w]}'
        Recorder.log.append((self.entry, args))
        return 0


class RecordingModule(b200.Module):
    def __getattr__(self, name):
        k = super().__getattr__(name)
        if not isinstance(k.fn, Recorder): k.fn = Recorder(k.entry)
        return k


@pytest.fixture
def ref(monkeypatch):
    """the reference's package importable, torch's CUDA calls stubbed (no device here), the maintainer's install() applied"""
    monkeypatch.syspath_prepend(os.path.join(REF, 'python'))
    monkeypatch.setattr(torch.cuda, 'device', lambda d: contextlib.nullcontext())
    monkeypatch.setattr(torch.cuda, 'current_device', lambda: 0)
    monkeypatch.setattr(torch.cuda, 'current_stream', lambda *a: type('S', (), {'cuda_stream': 0})())
    monkeypatch.setattr(torch.cuda, 'get_device_properties', lambda d: type('Props', (), {'multi_processor_count': 148})())
    monkeypatch.setattr(b200, 'CHECK_DEVICE', False)
    from caminus.device import hip
    from caminus.engine import gguf
    from caminus.prefill import glue, q35own, q3m_ops
    from caminus.train import actq, fuse
    for m in (hip, gguf, glue, actq, fuse): monkeypatch.setattr(m, 'Module', RecordingModule)
    for m in (gguf, actq, fuse): monkeypatch.setattr(m, '_mod', {})
    b200._IQ2S[0] = torch.zeros(512, dtype=torch.int32)
    Recorder.log.clear()
    yield type('Ref', (), dict(hip=hip, gguf=gguf, glue=glue, q35own=q35own, q3m_ops=q3m_ops, actq=actq, fuse=fuse))
    b200._IQ2S.pop(0, None)


def entries(): return [e for e, _ in Recorder.log]
def f32(*s): return torch.zeros(*s)
def i32(*s): return torch.zeros(*s, dtype=torch.int32)
def f16(*s): return torch.zeros(*s, dtype=torch.float16)
def bf(*s): return torch.zeros(*s, dtype=torch.bfloat16)
def u8(*s): return torch.zeros(*s, dtype=torch.uint8)


def test_q3m_ops_wrappers(ref):
    n, N, E, k, nh, nkv = 5, 2048, 128, 8, 32, 4
    O = ref.q3m_ops.Ops('cpu')
    O.emb(u8(100 * 1152), 1152, 100, i32(n), f32(n, N), n, N)
    O.add_rms16(f32(n, N), f32(N), 1e-6, f16(n, N), n, N, d=f32(n, 2, N), w=f32(n, 2), S=2, h=f32(n, N))
    O.add_rms16(f32(n, N), f32(N), 1e-6, f16(n, N), n, N)                        # the optional arguments as null pointers
    O.router(f32(n, N), f32(E, N), E, N, f32(n, E), n)
    O.topk(f32(n, E), E, k, 6.1e-5, i32(n, k), f32(n, k), i32(1), n)
    O.group(i32(n * k), n * k, k, E, i32(n * k), i32(n * k), i32(ref.q3m_ops.items_bound(n * k, E), 4), i32(1), i32(1))
    O.swiglu(f32(n * 768), f32(n * 768), f16(n * 768), n * 768)
    ldq = (nh + 2 * nkv) * 128
    O.qk_rope(f32(n, ldq), ldq, nh, nkv, f32(258), 3, f16(n, nh, 128), f16(64, 2, nkv * 128), n)
    assert entries() == ['q3p_emb', 'q3p_add_rms16', 'q3p_add_rms16', 'q3p_router', 'q3p_topk', 'q3p_group', 'q3p_swiglu', 'q3p_qk_rope']
    assert Recorder.log[0][1][0] == n and Recorder.log[7][1][0] == n            # the row counts of the launch grids lead
    Recorder.log.clear()
    Y = ref.q3m_ops.Ops('cpu', yarn=True)
    Y.qk_rope(f32(n, ldq), ldq, nh, nkv, f32(ref.q3m_ops.YARN_PAR), 3, f16(n, nh, 128), f16(64, 2, nkv * 128), n)
    Q = ref.q3m_ops.Ops('cpu', q8=True)
    Q.qk_rope(f32(n, ldq), ldq, nh, nkv, f32(258), 3, f16(n, nh, 128), u8(64 * 2 * (nkv * 128 // 32) * 34), n, err=i32(1))
    assert entries() == ['q3p_qk_rope_yarn', 'q3p_qk_rope_q8']
    with pytest.raises(ValueError): O.mod.q3p_qk_rope((n, nh + nkv + 1), (128,), f32(n, ldq), ctypes.c_int(ldq), ctypes.c_int(nh), ctypes.c_int(nkv), f32(258), ctypes.c_int(0), f16(1), f16(1))
    with pytest.raises(RuntimeError): O.mod.q3p_mm_q4k                           # a kernel this library does not serve: the loader's error, not a silent skip


def test_q35own_and_gguf_wrappers(ref):
    n, N = 7, 5120
    O = ref.q35own.Ops('cpu')
    O.add_rms16(f32(n, N), f32(N), 1e-6, f16(n, N), n, N, d=f32(n, N), h=f32(n, N))
    T = ref.q35own.Ops('cpu', module=ref.q35own.MODULE_TCAP)
    T.emb_iq2s(u8(50 * 8 * 82), 8 * 82, 50, i32(n), f32(n, 2048), n, 2048)
    y = ref.gguf.quantize_q8_1(f32(1000))
    assert y.numel() == 32 * 36
    ref.gguf.silu_mul(f32(640), f32(640))
    assert entries() == ['q35p_add_rms16', 'q35t_emb_iq2s', 'gg_quantize_q8_1', 'gg_silu_mul']


@pytest.mark.parametrize('module,D', [('prefill_glue', 2560), ('prefill_glue_q35', 2048), ('prefill_glue_q35d', 5120)])
def test_glue_wrappers(ref, module, D):
    T, HC, E, k = 6, 4, 256, 10; R = T * HC
    G = ref.glue.Glue('cpu', module=module)
    assert G.D == D
    W = max(D, 2560)                                                               # (the reference sizes some checks by its default width: buffers at least that wide)
    G.rms_mul(f32(R, W), f32(HC, D), f32(R, W), R, 1e-6, ybf=bf(R, W), scale=f32(R))
    G.rms_mul(f32(R, W), f32(1, D), None, R, 1e-6, scale=f32(R))
    G.hc_post_rms(f32(T, W), f32(T, HC), f32(R, W), f32(HC, W), T, HC, 1e-6, xn=f32(R, W), xnbf=bf(R, W), scale=f32(R))
    G.hc_post(f32(T, W), f32(T, HC), f32(R, W), T, HC, D=D)
    G.hc_mean(f32(R, W), f32(R, W), f32(T, W), T, HC, D=D, scale=f32(R), w=f32(HC, W))
    G.router(f32(T, E), T, E, k, i32(T, k), f32(T, k), i32(1))
    G.add_sum(f32(T * D), f32(T * D), f32(T * D), T * D)
    G.silu_bf16(f32(T, 512), bf(ref.glue.tpad(T), 512), T, 512, 0.5)
    G.to_bf16(f32(T, 512), bf(ref.glue.tpad(T), 512), T, 512)
    assert entries() == ['pf_rms_mul', 'pf_rms_mul', 'pf_hc_post_rms', 'pf_hc_post', 'pf_hc_mean', 'pf_router', 'pf_add_sum', 'pf_silu_bf16', 'pf_to_bf16']
    e, a = Recorder.log[0]
    assert isinstance(a[-2], int) and a[-2] == D                                # the row width the reference bakes into the code object, before the stream
    assert Recorder.log[5][1][0] == T                                            # pf_router: the token count of the launch grid leads


def test_training_line_forwards(ref):
    """the forward launches of train/actq.py (through the autograd Functions, as the model calls them) and train/fuse.py"""
    M, K, F_, d = 9, 1024, 512, 896
    ref.actq.actq(bf(M, K), 4, 1.0)
    ref.actq.scales(f32(M, K), 4, 1.0)
    ref.actq.codes(f32(M, K), 4, 1.0)
    ref.actq.codes(bf(M, K), 4, 1.0, dequant=True)
    ref.actq.actq_codes(bf(M, K), 4, 1.0)
    ref.actq.silu_mul_actq(bf(M, 2 * F_), 4, 1.0)
    ref.actq.block_entry(f32(M, d), f32(d), bf(6, d), 1e-6, 4, 1.0)
    ref.actq.block_entry(f32(M, d), f32(d), None, 1e-6, 4, 1.0)
    assert entries() == ['actq_fwd_bf16', 'actq_fwd_f32', 'actq_fwd_codes_f32', 'actq_fwd_codes_bf16', 'actq_fwd_codes_bf16', 'silu_mul_actq_fwd',
                         'block_entry_fwd', 'block_entry_fwd']
    assert all(a[0] == M for _, a in Recorder.log)                               # the row count of every launch grid leads
    Recorder.log.clear()
    out = ref.fuse.ResidualSlices.apply(f32(M, d), bf(M, d), bf(M, d), bf(3, d), i32(M))
    ref.fuse.ResidualSlices.apply(f32(M, d), bf(M, d), bf(M, d), None, None)
    assert out.shape == (M, d) and entries() == ['residual_slices_fwd', 'residual_slices_fwd']
