"""ctypes binding of libqtip_b200.so: one Python function per C-ABI entry point of include/qtip_b200.h.

The library is the product; there is no Python or CPU fallback. Loading fails loudly when the shared library is
missing, and every call raises QtipError with the library's message on a non-zero status.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("QTIP_B200_LIB", os.path.join(_HERE, "libqtip_b200.so"))  # override: a differently built library


class QtipError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("qtip_b200 status %d: %s" % (code, message))
        self.code = code


class QtipMatrix(C.Structure):
    """POD mirror of qtip_matrix (QtipMatrix of the reference runtime): device pointers + geometry."""
    _fields_ = [("trellis", C.c_void_p), ("su", C.c_void_p), ("sv", C.c_void_p), ("lut", C.c_void_p),
                ("n_in", C.c_int), ("n_out", C.c_int)]


class QtipTpExchange(C.Structure):
    """POD mirror of qtip_tp_exchange: every rank's exchange buffer as addressable from this process."""
    _fields_ = [("base", C.c_void_p * 8), ("bytes", C.c_size_t), ("rank", C.c_int), ("ranks", C.c_int)]


class QtipCheckpointLinear(C.Structure):
    """POD mirror of qtip_checkpoint_linear: host pointers of one linear's checkpoint tensors."""
    _fields_ = [("name", C.c_char_p), ("m", C.c_int), ("n", C.c_int), ("trellis_h", C.c_void_p),
                ("su_bf16_h", C.c_void_p), ("sv_h", C.c_void_p), ("tlut_h", C.c_void_p)]


class QtipGroupLinear(C.Structure):
    """POD mirror of qtip_group_linear: one linear of a Hessian group (inputs W_d, m, sv_d, trellis_d; the rest is output)."""
    _fields_ = [("W_d", C.c_void_p), ("m", C.c_long), ("sv_d", C.c_void_p), ("trellis_d", C.c_void_p),
                ("wscale", C.c_float), ("proxy", C.c_double), ("proxy_rot_reg", C.c_double)]


_P, _I, _L, _Z, _F = C.c_void_p, C.c_int, C.c_long, C.c_size_t, C.c_float
_X = C.POINTER(QtipTpExchange)

# name -> argument types; every function returns int except where noted in _RESTYPES
SIGNATURES = {
    "qtip_init": [],
    "qtip_encoder_lut": [_P, _P, C.POINTER(C.c_double), _P],
    "qtip_runtime_lut": [_P, _P, _P],
    "qtip_k_ldlq_prep": [_P, _P, _P, _P, _L, _L, _I, _I, _P, _P],
    "qtip_k_viterbi_fwd": [_P, _P, _I, _I, _P, _P, _P, _P],
    "qtip_k_viterbi_overlap": [_P, _P, _I, _P, _P],
    "qtip_k_viterbi_finish": [_P, _P, _I, _I, _P, _I, _I, _P, _L, _I, _P, _P],
    "qtip_k_decode_states": [_P, _I, _P, _P, _P],
    "qtip_k_hadamard_rows": [_P, _L, _I, _L, _I, _P],
    "qtip_k_transpose": [_P, _L, _L, _L, _P, _L, _P],
    "qtip_k_scale_rows_cols": [_P, _L, _L, _L, _P, _P, _P],
    "qtip_k_scale": [_P, _L, _L, _L, _F, _P],
    "qtip_k_sub": [_P, _P, _P, _L, _L, _L, _P],
    "qtip_k_sumsq": [_P, _L, _L, _L, _P, _P],
    "qtip_k_dot": [_P, _L, _P, _L, _L, _L, _P, _P],
    "qtip_k_add_diag": [_P, _L, _F, _P],
    "qtip_k_diag_sum": [_P, _L, _P, _P],
    "qtip_k_split_bf16": [_P, _L, _L, _L, _P, _P, _L, _P],
    "qtip_k_diff_split_bf16": [_P, _P, _L, _L, _L, _P, _P, _L, _P],
    "qtip_quantize_tiles": [_P, _I, _P, _P, _P, _P, _Z, _P],
    "qtip_quantize_tiles_scatter": [_P, _I, _I, _P, _P, _I, _I, _P, _L, _I, _P, _Z, _P],
    "qtip_quantize_tiles_noalloc": [_P, _I, _P, _P, _P, _P],
    "qtip_workspace_status": [_P, _P],
    "qtip_k_viterbi_fwd_words": [_P, _P, _I, _I, _P, _I, _P, _P, _P, _P],
    "qtip_k_viterbi_overlap_words": [_P, _P, _I, _P, _P],
    "qtip_k_viterbi_finish_words": [_P, _P, _I, _I, _P, _I, _I, _P, _P, _L, _I, _P, _P],
    "qtip_tiles_from_matrix": [_P, _L, _L, _L, _P, _P],
    "qtip_ldlq": [_P, _P, _L, _L, _L, _L, _P, _P, _P, _P, _Z, _P],
    "qtip_quantize_linear": [_P, _P, _L, _L, _P, _P, _P, C.c_double, C.c_double, _P, _P, _P, _P, C.POINTER(C.c_float), _P,
                             _Z, _P],
    "qtip_quantize_group": [C.POINTER(QtipGroupLinear), _I, _L, _P, _P, _P, C.c_double, _P, C.c_double, C.c_double, _P, _P,
                            _P, _P, _Z, _P],
    "qtip_rotate_hessian": [_P, _L, _P, C.c_double, _P, C.POINTER(C.c_double), _P, _P],
    "qtip_block_ldl": [_P, _L, _P, _P, _P, _Z, _P],
    "qtip_block_ldl_status": [_P, _P],
    "qtip_write_layer_file": [C.c_char_p, _I, C.POINTER(QtipCheckpointLinear), _I],
    "qtip_read_layer_linear": [C.c_char_p, _I, C.c_char_p, _I, _I, _P, _P, _P, _P],
    "qtip_pack_trellis": [_P, _L, _P, _P],
    "qtip_unpack_trellis": [_P, _L, _P, _P],
    "qtip_swizzle_for_kernel": [_P, _I, _I, _P, _P],
    "qtip_unswizzle_for_kernel": [_P, _I, _I, _P, _P],
    "qtip_prepare": [QtipMatrix, _P, _P, _P, _P, _I, _I],
    "qtip_multiply": [QtipMatrix, _P, _P, _I, _I, _P, _I],
    "qtip_finish": [QtipMatrix, _P, _P, _P, _I, _I, _P, _I, _I],
    "qtip_finish_b16": [QtipMatrix, _P, _P, _P, _I, _P, _I],
    "qtip_forward": [QtipMatrix, _P, _P, _P, _P, _P, _I, _P, _I],
    "qtip_multiply_batch": [QtipMatrix, _P, _P, _I, _I, _I, _P, _I],
    "qtip_input_transform": [_P, _L, _P, _F, _P, _I, _I, _P, _L, _P, _P],
    "qtip_output_residual": [_P, _I, _I, _I, _P, _I, _P, _P],
    "qtip_output_gateup": [_P, _I, _I, _P, _P, _I, _P, _P],
    "qtip_output_residual_input": [_P, _I, _I, _I, _P, _I, _P, _P, _F, _P, _P, _L, _P, _P],
    "qtip_decode_matrix": [QtipMatrix, _P, _P],
    "qtip_prefill_gemm": [_P, _P, _P, _I, _I, _I, _I, _P, _P],
    "qtip_prefill_gemm_splitk": [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "qtip_multiply_tc": [QtipMatrix, _P, _P, _I, _I, _I, _P, _P],
    "qtip_kernel_status": [_P],
    "qtip_debug_set_status": [_I, _I, _P],
    "qtip_decode_fp8_matrix": [_P, _P, _Z, _P],
    "qtip_fp8_forward": [_P, _P, _P, _P, _I, _I, _I, _P],
    "qtip_reduce_products": [_P, _Z, _I, _P],
    "qtip_reduce_to_b16": [_P, _P, _P, _Z, _I, _I, _P],
    "qtip_tp_alloc": [_Z, C.POINTER(C.c_void_p)],
    "qtip_tp_free": [_P],
    "qtip_tp_export": [_P, C.c_char_p],
    "qtip_tp_import": [C.c_char_p, C.POINTER(C.c_void_p)],
    "qtip_tp_close": [_P],
    "qtip_tp_reset": [_X, _P],
    "qtip_multiply_push": [QtipMatrix, _P, _X, _I, _I, _I, _I, _P, _I, _I],
    "qtip_gathered_products": [_X, _I, C.POINTER(C.c_void_p)],
    "qtip_gather_wait": [_X, _I, C.POINTER(C.c_void_p), _P],
    "qtip_tp_status": [_X, _P],
}
_RESTYPES = {
    "qtip_last_error": (C.c_char_p, []),
    "qtip_abi_version": (C.c_int, []),
    "qtip_quantize_workspace_bytes": (C.c_size_t, [_I]),
    "qtip_ldlq_workspace_bytes": (C.c_size_t, [_L, _L]),
    "qtip_block_ldl_workspace_bytes": (C.c_size_t, [_L]),
    "qtip_quantize_group_workspace_bytes": (C.c_size_t, [_L, _L, _L]),
    "qtip_quantize_linear_workspace_bytes": (C.c_size_t, [_L, _L]),
    "qtip_tp_exchange_bytes": (C.c_size_t, [_I, _I, _I]),
}


def exported_names():
    return sorted(list(SIGNATURES) + list(_RESTYPES))


class Library:
    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise ImportError("%s is missing: build it with `python behemoth-qtip_b200/build.py` (needs nvcc); "
                              "there is no CPU fallback" % path)
        self.cdll = C.CDLL(path)
        for name, args in SIGNATURES.items():
            fn = getattr(self.cdll, name)
            fn.restype = C.c_int
            fn.argtypes = args
        for name, (res, args) in _RESTYPES.items():
            fn = getattr(self.cdll, name)
            fn.restype = res
            fn.argtypes = args

    def last_error(self):
        return self.cdll.qtip_last_error().decode()

    def call(self, name, *args):
        rc = getattr(self.cdll, name)(*args)
        if rc != 0:
            raise QtipError(rc, self.last_error())

    def raw(self, name):
        return getattr(self.cdll, name)


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = Library()
    return _lib
