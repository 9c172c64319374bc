"""CPU-side checks: the C-ABI library loads and exports every entry include/caminus_b200.h declares (no compute call is
made), the host logic of the wrappers refuses what the reference's wrappers refuse, and the sharding helpers partition."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_entries():
    text = open(os.path.join(ROOT, 'include', 'caminus_b200.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'^\s*(?:const\s+)?(?:int|char)\s*\*?\s*(\w+)\s*\(', text, flags=re.M)))


def test_library_exports_every_declared_entry():
    from caminus_b200 import build, lib
    build.build()
    L = ctypes.CDLL(lib.path())
    names = declared_entries()
    assert len(names) >= 16 and 'q3p_emb' in names and 'cam_error_string' in names
    for n in names: assert hasattr(L, n), f'{n} is declared but not exported'
    assert set(lib.SIGNATURES) | {'cam_abi_version', 'cam_error_string'} == set(names)      # the binding covers the header
    lib.load()
    assert lib.load().cam_abi_version() == lib.ABI_VERSION
    assert 'aligned' in lib.error_string(-2) and lib.error_string(0) == 'ok'
    with pytest.raises(ValueError): lib.check(-1, 'x')
    with pytest.raises(RuntimeError, match='CUDA error'): lib.check(700, 'x')


def test_missing_library_is_loud(monkeypatch, tmp_path):
    from caminus_b200 import lib
    monkeypatch.setattr(lib, '_lib', None)
    monkeypatch.setenv('CAMINUS_B200_LIB', str(tmp_path / 'nope.so'))
    with pytest.raises(FileNotFoundError, match='no CPU or PyTorch fallback'): lib.load()


def test_loader_module_names():
    from caminus_b200.device import cuda as hip
    with pytest.raises(FileNotFoundError): hip.Module('k3_q3m_lean')
    m = hip.Module('q3m_prefill_yarn')
    assert m.q3p_qk_rope.entry == 'q3p_qk_rope_yarn' and hip.Module('q3m_prefill').q3p_qk_rope.entry == 'q3p_qk_rope'
    assert m.q3p_emb.ngrid == 1 and m.q3p_swiglu.ngrid == 0
    with pytest.raises(RuntimeError): m.q3p_mm_q4k
    with pytest.raises(ValueError): m.q3p_emb((1,), (256,), __import__('torch').zeros(4))     # a CPU tensor is refused before any launch


def test_span_checks_match_the_reference_wrapper():
    """python/caminus/prefill/q3m_ops.py:109-120 and engine/k3.py:422-433: refused before any launch"""
    import torch
    from caminus_b200.engine import k3
    from caminus_b200.prefill.q3m_ops import Ops
    O = Ops.__new__(Ops); O.q8 = False; O.yarn = False
    nkv, ctx = 4, 100
    cache = torch.zeros(ctx * 2 * nkv * 128, dtype=torch.float16)
    O._span('qk_rope', cache, 0, 100, nkv, None)
    O._span('qk_rope', cache, 25, 75, nkv, None)
    for pos0, n, rows in ((-1, 5, None), (96, 5, None), (30, 7, 36), (1000.5, 1, None), (True, 1, None)):
        with pytest.raises(k3.ContextBoundsError): O._span('qk_rope', cache, pos0, n, nkv, rows)
    with pytest.raises(ValueError): O._span('qk_rope', cache, 0, 0, nkv, None)
    with pytest.raises(ValueError): O._span('qk_rope', cache.float(), 0, 1, nkv, None)
    with pytest.raises(ValueError): O._span('qk_rope', cache, 0, 1, nkv, ctx + 1)
    with pytest.raises(ValueError): O._span('qk_rope', cache[:-3], 0, 1, nkv, None)
    assert k3.kv_rows(cache, nkv * 128) == ctx


def test_shards_partition():
    from caminus_b200 import dist as D
    for T in (1, 7, 4096, 65536, 65537):
        for G in (1, 2, 4, 8):
            edges = [D.row_shard(T, r, G) for r in range(G)]
            assert edges[0][0] == 0 and edges[-1][1] == T and all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
            assert max(b - a for a, b in edges) - min(b - a for a, b in edges) <= 1
    assert [D.col_shard(5120, r, 8) for r in range(8)] == [(640 * r, 640 * (r + 1)) for r in range(8)]
    with pytest.raises(ValueError): D.col_shard(5120, 0, 3)
    with pytest.raises(ValueError): D.row_shard(10, 2, 2)


def test_synth_is_seeded():
    from caminus_b200 import synth
    a = synth.swiglu_inputs(3, 64, seed=4); b = synth.swiglu_inputs(3, 64, seed=4)
    assert all(np.array_equal(x, y) for x, y in zip(a, b)) and a[0].dtype == np.float16
    W = synth.q4k_table(5, 512, seed=1)
    assert W.shape == (5, 2, 144) and (W[:, :, 0:4].copy().view(np.float16) >= 0).all()
    par = synth.rope_par(yarn_table=synth.yarn_table())
    assert par.size == 258 + 65 and par[256] == np.float32(np.float32(1e6) ** np.float32(-2.0 / 128))


def test_flag_word_checks_raise_the_reference_errors():
    """the third error tier: sticky device flag words read on the host (no GPU needed: the words are plain tensors here)"""
    import torch
    from caminus_b200.engine import k3
    from caminus_b200.errors import InvalidKVEncoding, NumericalFailure
    from caminus_b200.prefill.q3m_ops import Ops
    O = Ops.__new__(Ops)                                       # (the checks use no device state)
    err = torch.tensor([3], dtype=torch.int32)
    with pytest.raises(k3.ContextBoundsError, match='0x3'): O.check_flags(err, 'chunk')
    assert int(err.item()) == 0
    O.check_flags(err); O.check_kv_code(err)
    err[0] = 2
    with pytest.raises(InvalidKVEncoding): O.check_kv_code(err)
    assert int(err.item()) == 2 and issubclass(InvalidKVEncoding, NumericalFailure) and issubclass(NumericalFailure, RuntimeError)


def test_mmq_buffer_arithmetic_matches_the_reference():
    """k_pad / y_bytes size the quantised activation buffer as python/caminus/prefill/mmq.py:102-108 does (K padded to 512, 144-byte
    blocks of 128 values, an 18432-byte tail)"""
    from caminus_b200.prefill import mmq
    assert [mmq.k_pad(k) for k in (1, 512, 513, 2048, 2560, 25600)] == [512, 512, 1024, 2048, 2560, 25600]
    assert mmq.y_bytes(2048, 10) == 2048 // 128 * 10 * 144 + 18432 and mmq.y_bytes(600, 3) == 1024 // 128 * 3 * 144 + 18432
    assert (mmq.D4, mmq.DS4) == (0, 1)


def test_iq2s_grid_packing():
    """the packed IQ2_S grid (the layout of the reference's kernels/iq2s_grid.h): the shim's packing == the oracle's, both input forms, refusals"""
    import oracle
    from caminus_b200.device import cuda as hip
    g = np.array([8, 25, 43], np.uint8)[np.random.default_rng(1).integers(0, 3, (1024, 8))]
    w = hip.pack_iq2s_grid(g)
    assert w.dtype == np.uint32 and w.shape == (512,) and np.array_equal(w, oracle.pack_iq2s_grid(g))
    e5 = (w[2] >> 16) & 0xffff                                            # entry 5 = word 2, high half
    assert [(int(e5) >> (2 * k)) & 3 for k in range(8)] == [{8: 0, 25: 1, 43: 2}[int(v)] for v in g[5]]
    assert np.array_equal(hip.pack_iq2s_grid(w), w) and np.array_equal(hip.pack_iq2s_grid(w.view(np.int32)), w)
    with pytest.raises(ValueError): hip.pack_iq2s_grid(np.zeros((1024, 8), np.uint8))
    with pytest.raises(ValueError): hip.pack_iq2s_grid(np.zeros(100, np.uint32))


def test_no_packed_product_feeds_a_packed_sum():
    """the assembler contracts mul.rn.f32x2 into a packed add / sub that consumes it (unlike the scalar forms), so a kernel that needs
    the rounded product writes prod2(..) or scalar products; the one place that nests them (the Q4_K gather) has an exact product"""
    csrc = os.path.join(ROOT, 'caminus_b200', 'csrc')
    hits = []
    for name in sorted(os.listdir(csrc)):
        if not name.endswith(('.cu', '.cuh')): continue
        for no, line in enumerate(open(os.path.join(csrc, name)), 1):
            code = line.split('//')[0]
            if re.search(r'\b(add2|sub2)\(\s*mul2\(', code) or re.search(r'\b(add2|sub2)\([^;]*,\s*mul2\(', code): hits.append((name, no))
    assert all(n == 'emb_q4k.cu' for n, _ in hits) and len(hits) == 4, hits
