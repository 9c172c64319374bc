"""ctypes binding of libcaminus_b200.so: the one place the shared library is loaded and its entry points are typed.

There is no fallback: if the library is missing, does not load, or lacks an entry of include/caminus_b200.h, importing
a kernel raises. CAMINUS_B200_LIB names another build of the library (as CAMINUS_KERNEL_DIR names another kernel
directory in the reference, python/caminus/device/kernels.py:64-72).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_PATH = os.path.join(_HERE, 'lib', 'libcaminus_b200.so')
ABI_VERSION = 1

P, I, L, F, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float, ctypes.c_uint

# entry -> argument types, in the order of include/caminus_b200.h (every entry returns int)
SIGNATURES = {
    'q3p_emb': [I, P, I, I, P, P, I, P],
    'q3p_add_rms16': [I, P, P, P, I, P, F, P, P, I, P],
    'q35p_add_rms16': [I, P, P, P, F, P, P, I, P],
    'cam_add_rms_f16': [I, P, P, P, F, P, I, P],
    'cam_ipc_open': [P, P],
    'cam_ipc_close': [P],
    'cam_tp_rms_words': [I, I],
    'cam_tp_rms_norm_f16': [I, P, P, P, F, P, I, I, P, I, I, I, U, P, P],
    'cam_rms_partial_f16': [I, P, P, P, I, P],
    'cam_rms_apply_f16': [I, P, P, P, P, F, P, I, I, P],
    'cam_rms_norm_f16_static': [I, P, P, P, F, P, I, P],
    'q3p_swiglu': [P, P, P, I, P],
    'gg_silu_mul': [P, P, P, I, P],
    'gg_quantize_q8_1': [P, P, I, P],
    'gg_swiglu_q8_1': [P, P, P, L, P],
    'gg_swiglu_q8_1_f16': [P, P, P, L, P],
    'gg_swiglu_q8_1_sums': [P, P, P, L, P],
    'gg_swiglu_q8_1_f16_sums': [P, P, P, L, P],
    'gg_swiglu_q8_1_strict': [P, P, P, L, P],
    'gg_swiglu_q8_1_f16_strict': [P, P, P, L, P],
    'gg_silu_scale_q8_1': [P, F, P, L, P],
    'cam_probe_silu_f16': [P, P, P, I, P],
    'gg_silu_scale_q8_1_sums': [P, F, P, L, P],
    'q3p_qk_rope': [I, P, I, I, I, P, I, P, P, P],
    'q3p_qk_rope_yarn': [I, P, I, I, I, P, I, P, P, P],
    'cam_qk_rope_f16': [I, P, P, I, I, P, I, P, P, I, P],
    'q3p_qk_rope_q8': [I, P, I, I, I, P, I, P, P, P, P],
    'q3p_qk_rope_q8_yarn': [I, P, I, I, I, P, I, P, P, P, P],
    'cam_quantize_mmq_q8_1': [P, P, I, I, L, I, I, P],
    'cam_swiglu_mmq_q8_1': [P, P, P, I, I, L, I, I, P],
    'cam_swiglu_mmq_q8_1_f16': [P, P, P, I, I, L, I, I, P],
    'cam_swiglu_mmq_q8_1_ids': [P, P, P, P, I, I, L, I, I, P],
    'cam_swiglu_mmq_q8_1_f16_ids': [P, P, P, P, I, I, L, I, I, P],
    'cam_quantize_mmq_q8_1_ids': [P, P, P, I, I, L, I, I, P],
    'cam_quantize_mmq_q8_1_scatter': [P, P, P, I, I, L, I, I, I, P],
    'actq_fwd_bf16': [I, P, P, P, I, F, I, P],
    'actq_fwd_f32': [I, P, P, P, I, F, I, P],
    'actq_fwd_codes_bf16': [I, P, P, P, P, I, F, I, P],
    'actq_fwd_codes_f32': [I, P, P, P, P, I, F, I, P],
    'silu_mul_actq_fwd': [I, P, I, I, P, P, P, F, I, P],
    'block_entry_fwd': [I, P, P, P, I, F, P, P, P, P, P, I, F, I, P],
    'embd_rows_iq4xs': [P, P, I, I, I, P, P, P],
    'ple_rows_iq4nl': [P, P, I, I, I, P, P, P],
    'cam_emb_rows_q6k': [I, P, I, I, P, P, I, P],
    'q35t_emb_iq2s': [I, P, I, I, P, P, I, P, P],
    'q3p_router': [I, P, P, I, I, P, P],
    'q3p_topk': [I, P, I, I, F, P, P, P, P],
    'q3p_group': [P, I, I, I, P, P, P, P, P, P],
    'pf_router': [I, P, I, I, F, P, P, P, P],
    'pf_rms_mul': [P, P, P, P, P, I, I, F, I, P],
    'cam_rms_mul_q8_1': [P, P, P, P, I, I, F, I, P],
    'pf_hc_post_rms': [P, P, P, P, P, P, P, I, I, F, F, I, P],
    'pf_hc_post': [P, P, P, I, I, I, F, P],
    'pf_hc_mean': [P, P, P, P, P, I, I, I, F, P],
    'pf_add_sum': [P, P, P, L, P],
    'pf_swiglu': [P, P, P, L, P],
    'pf_silu_bf16': [P, I, P, I, I, I, F, P],
    'pf_to_bf16': [P, I, P, I, I, I, P],
    'pf_qk_nr': [I, P, I, I, P, I, I, F, F, I, P, P],
    'embedding_f32': [I, P, P, P, I, P],
    'rmsnorm_f32': [I, P, P, P, I, F, P],
    'silu_mul_bf16': [P, P, I, L, P],
    'residual3': [P, P, P, P, L, P],
    'cast_bf16': [P, P, L, P],
    'residual_slices_fwd': [P, P, P, P, P, P, I, L, P],
}

_lib = None


def path():
    return os.environ.get('CAMINUS_B200_LIB', DEFAULT_PATH)


def missing_message(p):
    return (f'caminus_b200: the kernel library {p} is missing. Build it with `python -m caminus_b200.build` (nvcc, sm_100a) '
            f'or point CAMINUS_B200_LIB at a build. There is no CPU or PyTorch fallback.')


def load():
    """the loaded library (ctypes.CDLL), every entry typed; raises if it cannot be loaded whole"""
    global _lib
    if _lib is not None: return _lib
    p = path()
    if not os.path.isfile(p): raise FileNotFoundError(missing_message(p))
    lib = ctypes.CDLL(p)
    lib.cam_abi_version.restype = I; lib.cam_abi_version.argtypes = []
    lib.cam_error_string.restype = ctypes.c_char_p; lib.cam_error_string.argtypes = [I]
    for name, args in SIGNATURES.items():
        try: fn = getattr(lib, name)
        except AttributeError: raise RuntimeError(f'caminus_b200: {p} does not export {name}') from None
        fn.restype = I; fn.argtypes = args
    v = lib.cam_abi_version()
    if v != ABI_VERSION: raise RuntimeError(f'caminus_b200: {p} has ABI version {v}, this package binds version {ABI_VERSION}')
    _lib = lib
    return lib


def error_string(code):
    return load().cam_error_string(int(code)).decode()


def check(code, what=''):
    """0: nothing. Negative (an argument refusal): ValueError. Positive (a cudaError_t): RuntimeError('CUDA error ...')."""
    if code == 0: return
    if code < 0: raise ValueError(f'caminus_b200 {what}: {error_string(code)}')
    raise RuntimeError(f'CUDA error {code}: {error_string(code)}' + (f' ({what})' if what else ''))
