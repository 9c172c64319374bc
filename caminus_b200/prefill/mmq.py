"""The activation quantiser of the reference's MMQ glue (python/caminus/prefill/mmq.py:245-281, class Mmq: quantize and
quantize_scatter) over libcaminus_b200: fp32 rows -> block_q8_1_mmq columns [K_pad / 128][ncols] of 144 bytes, optionally
gathered by a row index or scattered to each token's compact columns. The quantised GEMMs of that class are outside this
library."""
import torch

from .. import lib as _lib

QK8_1_MMQ, Y_BLOCK, MATRIX_ROW_PADDING = 128, 144, 512
Y_TAIL = 18432                     # the reference's tail behind the blocks (its GEMM reads past the last column tile)
D4, DS4 = 0, 1                     # mmq_q8_1_ds_layout (D2S6 is not built by the reference either: mmq.py:83)


def k_pad(K):
    return (int(K) + MATRIX_ROW_PADDING - 1) // MATRIX_ROW_PADDING * MATRIX_ROW_PADDING


def y_bytes(K, ncols):
    """bytes of a quantised activation buffer for ncols columns of K values (K padded to 512, + Y_TAIL), as the reference sizes it"""
    return k_pad(K) // QK8_1_MMQ * int(ncols) * Y_BLOCK + Y_TAIL


def _view_bytes(t):
    return t.numel() * t.element_size()


class Mmq:
    """quantize / quantize_scatter with the reference's arguments, meanings and refusals (ValueError before any launch)"""

    def __init__(self, dev):
        self.dev = torch.device(dev)
        _lib.load()

    def _chk(self, t, what, dtype=None):
        if not isinstance(t, torch.Tensor) or t.device != self.dev or not t.is_contiguous(): raise ValueError(f'mmq: {what} must be a contiguous tensor on {self.dev}')
        if dtype is not None and t.dtype != dtype: raise ValueError(f'mmq: {what} must be {dtype}, not {t.dtype}')

    def quantize(self, x, K, ncols, y, layout, s01=None, ids=None, stream=None):
        """column c of y = x row (ids[c] if ids else c) (x fp32, row stride s01 floats, default K); y in ggml's
        [K_pad / 128][ncols] block_q8_1_mmq layout, the K padding zeros"""
        K, ncols = int(K), int(ncols); s01 = K if s01 is None else int(s01)
        self._chk(x, 'x', torch.float32); self._chk(y, 'y')
        if K % 4 or ncols < 1 or s01 < K: raise ValueError(f'mmq.quantize: K {K} (a multiple of 4), ncols {ncols}, s01 {s01}')
        if layout not in (D4, DS4): raise ValueError(f'mmq.quantize: layout {layout}')
        if _view_bytes(y) < y_bytes(K, ncols): raise ValueError(f'mmq.quantize: y holds {_view_bytes(y)} B < {y_bytes(K, ncols)}')
        xb = 4 * ((ncols - 1) * s01 + K)
        if _view_bytes(x) < xb: raise ValueError(f'mmq.quantize: x holds {_view_bytes(x)} B < {ncols} rows ({xb} B)')
        if ids is not None:
            self._chk(ids, 'ids', torch.int32)
            if ids.numel() < ncols: raise ValueError(f'mmq.quantize: ids holds {ids.numel()} < {ncols}')
        with torch.cuda.device(self.dev):
            s = torch.cuda.current_stream().cuda_stream if stream is None else int(stream)
            r = _lib.load().cam_quantize_mmq_q8_1_ids(x.data_ptr(), 0 if ids is None else ids.data_ptr(), y.data_ptr(), K, k_pad(K), s01, ncols, layout, s)
        _lib.check(r, 'mmq.quantize')

    def swiglu_quantize(self, g, u, K, ncols, y, layout, s01=None, ids=None, stream=None):
        """quantize() of silu(g) * u without storing the products: column c of y = the blocks of row (ids[c] if ids else c) of gate and
        up (both fp32 or both fp16, row stride s01 values). The bytes the reference's fused gate / up kernel writes for its down
        projection (kernels/prefill_moe.hip:339-396), here from stored gate and up rows"""
        K, ncols = int(K), int(ncols); s01 = K if s01 is None else int(s01)
        self._chk(g, 'gate'); self._chk(u, 'up', g.dtype); self._chk(y, 'y')
        if g.dtype not in (torch.float32, torch.float16): raise ValueError(f'mmq.swiglu_quantize: gate and up fp32 or fp16, not {g.dtype}')
        if K % 4 or ncols < 1 or s01 < K: raise ValueError(f'mmq.swiglu_quantize: K {K} (a multiple of 4), ncols {ncols}, s01 {s01}')
        if layout not in (D4, DS4): raise ValueError(f'mmq.swiglu_quantize: layout {layout}')
        if _view_bytes(y) < y_bytes(K, ncols): raise ValueError(f'mmq.swiglu_quantize: y holds {_view_bytes(y)} B < {y_bytes(K, ncols)}')
        need = g.element_size() * ((ncols - 1) * s01 + K)
        if _view_bytes(g) < need or _view_bytes(u) < need: raise ValueError(f'mmq.swiglu_quantize: gate / up hold fewer than {ncols} rows ({need} B)')
        if ids is not None:
            self._chk(ids, 'ids', torch.int32)
            if ids.numel() < ncols: raise ValueError(f'mmq.swiglu_quantize: ids holds {ids.numel()} < {ncols}')
        fn = _lib.load().cam_swiglu_mmq_q8_1_f16_ids if g.dtype == torch.float16 else _lib.load().cam_swiglu_mmq_q8_1_ids
        with torch.cuda.device(self.dev):
            s = torch.cuda.current_stream().cuda_stream if stream is None else int(stream)
            r = fn(g.data_ptr(), u.data_ptr(), 0 if ids is None else ids.data_ptr(), y.data_ptr(), K, k_pad(K), s01, ncols, layout, s)
        _lib.check(r, 'mmq.swiglu_quantize')

    def quantize_scatter(self, x, K, ntok, ids_inv, k, y, layout, s_tok=None, stream=None):
        """each token's row of x quantised once and written to its k compact columns ids_inv[t * k + slot] of y
        ([K_pad / 128][ntok * k])"""
        K, ntok, k = int(K), int(ntok), int(k); s_tok = K if s_tok is None else int(s_tok)
        self._chk(x, 'x', torch.float32); self._chk(y, 'y'); self._chk(ids_inv, 'ids_inv', torch.int32)
        if K % 4 or ntok < 1 or k < 1 or s_tok < K: raise ValueError(f'mmq.quantize_scatter: K {K}, ntok {ntok}, k {k}, s_tok {s_tok}')
        if layout not in (D4, DS4): raise ValueError(f'mmq.quantize_scatter: layout {layout}')
        if ids_inv.numel() < ntok * k: raise ValueError(f'mmq.quantize_scatter: ids_inv holds {ids_inv.numel()} < {ntok * k}')
        xb = 4 * ((ntok - 1) * s_tok + K)
        if _view_bytes(x) < xb: raise ValueError(f'mmq.quantize_scatter: x holds {_view_bytes(x)} B < {ntok} rows ({xb} B)')
        if _view_bytes(y) < y_bytes(K, ntok * k): raise ValueError(f'mmq.quantize_scatter: y holds {_view_bytes(y)} B < {y_bytes(K, ntok * k)}')
        with torch.cuda.device(self.dev):
            s = torch.cuda.current_stream().cuda_stream if stream is None else int(stream)
            r = _lib.load().cam_quantize_mmq_q8_1_scatter(x.data_ptr(), ids_inv.data_ptr(), y.data_ptr(), K, k_pad(K), s_tok, ntok, k, layout, s)
        _lib.check(r, 'mmq.quantize_scatter')
