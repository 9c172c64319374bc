"""The entry point that allocates nothing (cam_rms_norm_f16_static): for callers that may not allocate device memory,
the two-kernel RMSNorm keeps its per-row sums in a static array inside the library. Called here through the C ABI, twice
in a row on different batches, and compared byte for byte with the existing pair of entries (cam_rms_partial_f16 +
cam_rms_apply_f16) that takes the intermediate buffer from the caller. The file name sorts last on purpose: a run that
stops at the first failure has already run every other test."""
import numpy as np
import pytest

torch = pytest.importorskip('torch')
pytestmark = pytest.mark.gpu

DEV = 'cuda:0'


def _pair(lib, x, d, nw, eps, N):
    """the existing entries: the caller's own buffer carries the sums between the two launches"""
    n = x.shape[0]
    ss = torch.empty(n, dtype=torch.float32, device=DEV)
    h16 = torch.empty_like(x)
    s = torch.cuda.current_stream().cuda_stream
    lib.check(lib.load().cam_rms_partial_f16(n, x.data_ptr(), 0 if d is None else d.data_ptr(), ss.data_ptr(), N, s), 'partial')
    lib.check(lib.load().cam_rms_apply_f16(n, x.data_ptr(), 0 if d is None else d.data_ptr(), ss.data_ptr(), nw.data_ptr(), eps,
                                           h16.data_ptr(), N, N, s), 'apply')
    return h16


def test_static_scratch_entry_matches_the_pair_twice_in_a_row():
    from caminus_b200 import lib, synth
    L = lib.load()
    eps = 1e-6
    with torch.cuda.device(DEV):
        # two calls in a row; the second is smaller and has no addend, so rows of the static array keep stale sums beyond it
        for n, N, add, seed in ((3000, 5120, True, 1), (257, 2048, False, 2), (65536, 256, True, 3)):
            x0, r0, w = synth.add_rms_inputs(n, N, seed=seed, dtype=np.float16)
            nw = torch.from_numpy(w).to(DEV)
            d = torch.from_numpy(r0).to(DEV) if add else None
            xa = torch.from_numpy(x0).to(DEV); xb = xa.clone()
            want = _pair(lib, xa, d, nw, eps, N)
            got = torch.empty_like(xb)
            s = torch.cuda.current_stream().cuda_stream
            lib.check(L.cam_rms_norm_f16_static(n, xb.data_ptr(), 0 if d is None else d.data_ptr(), nw.data_ptr(), eps, got.data_ptr(), N, s),
                      'cam_rms_norm_f16_static')
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.int16), want.view(torch.int16))          # the normed rows: the same bytes
            assert torch.equal(xb.view(torch.int16), xa.view(torch.int16))              # and the same residual update
            assert bool(torch.isfinite(got.float()).all())
        # more rows than the static array holds: refused with a clear error, nothing launched
        big = torch.zeros(65537, 8, dtype=torch.float16, device=DEV); out = torch.ones_like(big)
        with pytest.raises(ValueError, match='fixed-size buffer'):
            lib.check(L.cam_rms_norm_f16_static(65537, big.data_ptr(), 0, torch.ones(8, device=DEV).data_ptr(), eps, out.data_ptr(), 8, 0), 'static')
        torch.cuda.synchronize()
        assert bool((out == 1).all())
