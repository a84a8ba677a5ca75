"""Host-side mirror of the quantizer's kernel interface (src/gpu.hpp:276-292 and src/quantizer.hpp:60-78 of the
reference): same names, argument order and meaning, with torch CUDA tensors in place of raw device pointers.
Every function launches on the current torch stream through the C ABI and returns without synchronising.
"""
import ctypes as C

import numpy as np
import torch

from ._lib import lib

kSeq, kSteps, kWordsPerTrellis = 256, 128, 32

_initialised = set()


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def init():
    """Per-device set-up (qtip_init) for the current device; idempotent."""
    dev = torch.cuda.current_device()
    if dev not in _initialised:
        lib().call("qtip_init")
        _initialised.add(dev)


def _p(t, dtype=None):
    if t is None:
        return None
    if isinstance(t, int):  # a raw device address (a slot of a tensor-parallel exchange buffer)
        return C.c_void_p(t)
    assert t.is_cuda and t.is_contiguous(), "device-resident contiguous tensor expected"
    if dtype is not None:
        assert t.dtype == dtype, "expected %s, got %s" % (dtype, t.dtype)
    return C.c_void_p(t.data_ptr())


def device_lut(tlut_f16):
    """Encoder table of a tlut ([512, 2] fp16 values or raw uint16 bits, host): returns (lut_h2 int32[65536] on the
    device, lut_rms). device_lut() / build_codebook() of the reference with the table as a parameter."""
    init()
    bits = tlut_bits(tlut_f16)
    out = torch.empty(65536, dtype=torch.int32, device="cuda")
    rms = C.c_double()
    lib().call("qtip_encoder_lut", bits.ctypes.data_as(C.c_void_p), _p(out), C.byref(rms), _stream())
    return out, rms.value


def tlut_bits(tlut):
    a = np.asarray(tlut.cpu() if isinstance(tlut, torch.Tensor) else tlut)
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    a = np.ascontiguousarray(a, dtype=np.uint16).reshape(-1)
    assert a.size == 1024, "tlut must be [512, 2]"
    return a


def k_ldlq_prep(WT, hatWT, prod, L, n, m, col0, bufend, X):
    init()
    lib().call("qtip_k_ldlq_prep", _p(WT, torch.float32), _p(hatWT, torch.float32), _p(prod, torch.float32),
               _p(L, torch.float32), n, m, col0, bufend, _p(X, torch.float32), _stream())


def k_viterbi_fwd(X, overlap, roll, B, A, final_state, lut_h2):
    init()
    lib().call("qtip_k_viterbi_fwd", _p(X, torch.float32), _p(overlap, torch.int32), int(roll), B, _p(A, torch.int16),
               _p(final_state, torch.int16), _p(lut_h2, torch.int32), _stream())


def k_viterbi_overlap(A, final_state, B, overlap):
    init()
    lib().call("qtip_k_viterbi_overlap", _p(A, torch.int16), _p(final_state, torch.int16), B, _p(overlap, torch.int32),
               _stream())


def k_viterbi_finish(A, final_state, B, b0, Q, nblk, blk, hatWT, m, col0, lut_h2):
    init()
    lib().call("qtip_k_viterbi_finish", _p(A, torch.int16), _p(final_state, torch.int16), B, b0, _p(Q, torch.int16),
               nblk, blk, _p(hatWT, torch.float32), m, col0, _p(lut_h2, torch.int32), _stream())


def k_decode_states(states, B, hat, lut_h2):
    init()
    lib().call("qtip_k_decode_states", _p(states, torch.int16), B, _p(hat, torch.float32), _p(lut_h2, torch.int32),
               _stream())


def k_hadamard_rows(X, rows, n, ld, transpose):
    init()
    lib().call("qtip_k_hadamard_rows", _p(X, torch.float32), rows, n, ld, int(bool(transpose)), _stream())


def k_transpose(src, rows, cols, ld_in, dst, ld_out):
    init()
    lib().call("qtip_k_transpose", _p(src, torch.float32), rows, cols, ld_in, _p(dst, torch.float32), ld_out, _stream())


def k_scale_rows_cols(X, rows, cols, ld, rs, cs):
    init()
    lib().call("qtip_k_scale_rows_cols", _p(X, torch.float32), rows, cols, ld, _p(rs, torch.float32),
               _p(cs, torch.float32), _stream())


def k_scale(X, rows, cols, ld, a):
    init()
    lib().call("qtip_k_scale", _p(X, torch.float32), rows, cols, ld, C.c_float(a), _stream())


def k_sub(A, B, D, rows, cols, ld):
    init()
    lib().call("qtip_k_sub", _p(A, torch.float32), _p(B, torch.float32), _p(D, torch.float32), rows, cols, ld, _stream())


def k_sumsq(X, rows, cols, ld, out):
    init()
    lib().call("qtip_k_sumsq", _p(X, torch.float32), rows, cols, ld, _p(out, torch.float64), _stream())


def k_dot(A, lda, B, ldb, rows, cols, out):
    init()
    lib().call("qtip_k_dot", _p(A, torch.float32), lda, _p(B, torch.float32), ldb, rows, cols, _p(out, torch.float64),
               _stream())


def k_add_diag(H, n, a):
    init()
    lib().call("qtip_k_add_diag", _p(H, torch.float32), n, C.c_float(a), _stream())


def k_diag_sum(H, n, out):
    init()
    lib().call("qtip_k_diag_sum", _p(H, torch.float32), n, _p(out, torch.float64), _stream())


def k_split_bf16(X, rows, cols, ld_in, hi, lo, ld_out):
    init()
    lib().call("qtip_k_split_bf16", _p(X, torch.float32), rows, cols, ld_in, _p(hi, torch.int16), _p(lo, torch.int16),
               ld_out, _stream())


def k_diff_split_bf16(A, B, rows, cols, ld, hi, lo, ld_out):
    init()
    lib().call("qtip_k_diff_split_bf16", _p(A, torch.float32), _p(B, torch.float32), rows, cols, ld,
               _p(hi, torch.int16), _p(lo, torch.int16), ld_out, _stream())


class Workspace:
    """Device scratch of the fused entry points, owned by the caller (the C ABI allocates nothing)."""

    def __init__(self, nbytes):
        self.buf = torch.empty(int(nbytes), dtype=torch.uint8, device="cuda")

    @property
    def ptr(self):
        return C.c_void_p(self.buf.data_ptr())

    @property
    def nbytes(self):
        return self.buf.numel()

    def check(self):
        """Synchronises the current stream and raises if a kernel reported a timed-out hand-shake."""
        lib().call("qtip_workspace_status", self.ptr, _stream())


def quantize_workspace(max_tiles):
    init()
    return Workspace(lib().raw("qtip_quantize_workspace_bytes")(int(max_tiles)))


def quantize_tiles(X, lut_h2, states=None, hat=None, workspace=None, want_hat=True):
    """Two-pass tail-biting quantisation of X [B, 256] f32 -> (states int16 [B, 128], hat f32 [B, 256]); with
    want_hat=False the decoded values are not written (the C ABI takes a null pointer) and None is returned for them."""
    init()
    B = X.shape[0]
    if states is None:
        states = torch.empty((B, 128), dtype=torch.int16, device=X.device)
    if hat is None and want_hat:
        hat = torch.empty((B, 256), dtype=torch.float32, device=X.device)
    if workspace is None:
        workspace = quantize_workspace(min(max(B, 8), 4608))
    lib().call("qtip_quantize_tiles", _p(X, torch.float32), B, _p(lut_h2, torch.int32), _p(states, torch.int16),
               _p(hat, torch.float32), workspace.ptr, workspace.nbytes, _stream())
    return states, hat


def quantize_tiles_scatter(X, b0, lut_h2, Q, nblk, blk, hatWT, m, col0, workspace):
    init()
    lib().call("qtip_quantize_tiles_scatter", _p(X, torch.float32), X.shape[0], b0, _p(lut_h2, torch.int32),
               _p(Q, torch.int16), nblk, blk, _p(hatWT, torch.float32), m, col0, workspace.ptr, workspace.nbytes,
               _stream())


def k_viterbi_fwd_words(X, overlap, roll, B, bp, first_block, final_state, lut_h2, status):
    init()
    lib().call("qtip_k_viterbi_fwd_words", _p(X, torch.float32), _p(overlap, torch.int32), int(roll), B,
               _p(bp, torch.int32), first_block, _p(final_state, torch.int16), _p(lut_h2, torch.int32),
               _p(status, torch.int32), _stream())


def k_viterbi_overlap_words(bp, final_state, B, overlap):
    init()
    lib().call("qtip_k_viterbi_overlap_words", _p(bp, torch.int32), _p(final_state, torch.int16), B,
               _p(overlap, torch.int32), _stream())


def k_viterbi_finish_words(bp, final_state, B, b0, Q, nblk, blk, hat, hatWT, m, col0, lut_h2):
    init()
    lib().call("qtip_k_viterbi_finish_words", _p(bp, torch.int32), _p(final_state, torch.int16), B, b0,
               _p(Q, torch.int16), nblk, blk, _p(hat, torch.float32), _p(hatWT, torch.float32), m, col0,
               _p(lut_h2, torch.int32), _stream())


def tiles_from_matrix(W, X=None):
    """[m, n] f32 row-major -> [tiles, 256] sequences of its 16x16 tiles (tile-row-major) on the device."""
    init()
    m, n = W.shape
    if X is None:
        X = torch.empty((m // 16) * (n // 16), 256, dtype=torch.float32, device=W.device)
    lib().call("qtip_tiles_from_matrix", _p(W, torch.float32), m, n, W.stride(0), _p(X, torch.float32), _stream())
    return X


def ldlq_workspace(n, m):
    init()
    return Workspace(lib().raw("qtip_ldlq_workspace_bytes")(int(n), int(m)))


def ldlq_gpu(WT, L, n, m, hatWT, Q, lut_h2, workspace=None, j0=0, mj=None):
    """ldlq_gpu of the reference (src/quantizer.cpp:30-89): WT [n, m] f32 scaled, L [n, n] f32 strictly block-lower;
    writes hatWT [n, m] and Q [(m/16)(n/16), 128]. [j0, j0+mj) restricts the call to a slice of W rows."""
    init()
    if workspace is None:
        workspace = ldlq_workspace(n, m)
    lib().call("qtip_ldlq", _p(WT, torch.float32), _p(L, torch.float32), n, m, j0, m if mj is None else mj,
               _p(hatWT, torch.float32), _p(Q, torch.int16), _p(lut_h2, torch.int32), workspace.ptr, workspace.nbytes,
               _stream())
    return workspace


def pack_trellis(states, packed=None):
    init()
    B = states.shape[0]
    if packed is None:
        packed = torch.empty((B, 32), dtype=torch.int16, device=states.device)
    lib().call("qtip_pack_trellis", _p(states, torch.int16), B, _p(packed, torch.int16), _stream())
    return packed


def unpack_trellis(packed, states=None):
    init()
    B = packed.shape[0]
    if states is None:
        states = torch.empty((B, 128), dtype=torch.int16, device=packed.device)
    lib().call("qtip_unpack_trellis", _p(packed, torch.int16), B, _p(states, torch.int16), _stream())
    return states


def swizzle_for_kernel(packed, m, n, out=None):
    init()
    if out is None:
        out = torch.empty_like(packed)
    lib().call("qtip_swizzle_for_kernel", _p(packed, torch.int16), m, n, _p(out, torch.int16), _stream())
    return out


def unswizzle_for_kernel(words, m, n, out=None):
    init()
    if out is None:
        out = torch.empty_like(words)
    lib().call("qtip_unswizzle_for_kernel", _p(words, torch.int16), m, n, _p(out, torch.int16), _stream())
    return out


# ---------------------------------------------------------------------------------------------------------------
# quantize_group of the reference (src/quantizer.cpp:124-346) assembled from the kernels above: Hessian rotation,
# weight rotation and scaling, LDLQ + Viterbi, proxy error, pack + kernel layout. The block LDL itself is an input
# (`L`, strictly block-lower fp32): the reference computes it on the CPU in fp64 (src/qtip_core.cpp:444-487).

def rotate_hessian(H, su, sigma_reg=1e-2):
    """HRr = hadUt(hadUt((H + creg I) scaled by SU on both sides)^T) for H [n, n] f32 on the device (modified in place
    and returned rotated); returns (HRr, creg). src/quantizer.cpp:124-152."""
    init()
    n = H.shape[0]
    acc = torch.zeros(1, dtype=torch.float64, device=H.device)
    k_diag_sum(H, n, acc)
    creg = sigma_reg * float(acc) / n
    k_add_diag(H, n, creg)
    k_scale_rows_cols(H, n, n, n, su, su)
    k_hadamard_rows(H, n, n, n, True)
    HR = torch.empty_like(H)
    k_transpose(H, n, n, n, HR, n)
    k_hadamard_rows(HR, n, n, n, True)
    return HR, creg


def rotate_weight(W, su, sv, lut_rms, scale_override=0.9):
    """WT [n, m] = (T_m^T diag(SV) W diag(SU) T_n)^T / Wscale with Wscale = rms / (float32(lut_rms) * scale_override).
    W [m, n] f32 on the device (scratch: overwritten). Returns (WT, wscale). src/quantizer.cpp:236-250."""
    init()
    m, n = W.shape
    k_scale_rows_cols(W, m, n, n, sv, su)
    k_hadamard_rows(W, m, n, n, True)
    WT = torch.empty((n, m), dtype=torch.float32, device=W.device)
    k_transpose(W, m, n, n, WT, m)
    k_hadamard_rows(WT, n, m, m, True)
    acc = torch.zeros(1, dtype=torch.float64, device=W.device)
    k_sumsq(WT, n, m, m, acc)
    rms = (float(acc) / (float(n) * m)) ** 0.5
    wscale = float(np.float32(rms / (float(np.float32(lut_rms)) * scale_override)))
    k_scale(WT, n, m, m, 1.0 / wscale)
    return WT, wscale


def proxy_error(WT, hatWT, HRr):
    """tr(D H D^T) / tr(W H W^T) in the rotated, scaled domain (D = W - hatW), fp32 GEMMs with fp64 reduction.
    src/quantizer.cpp:272-301 (the reference uses split-bf16 GEMMs for the same traces)."""
    D = WT - hatWT
    num = (D * (HRr @ D)).sum(dtype=torch.float64)
    den = (WT * (HRr @ WT)).sum(dtype=torch.float64)
    return float(num / den)


def quantize_linear(W, L, su, sv, lut_h2, lut_rms, workspace=None, scale_override=0.9):
    """One linear of a Hessian group: rotate, scale, LDLQ + Viterbi, pack, kernel layout.
    W [m, n] f32 (device, overwritten), L [n, n] f32 strictly block-lower. Returns a dict with the checkpoint tensors
    (trellis int16 [(m/16)(n/16), 32] in kernel layout, SU bf16, SV f32 = sign * Wscale) plus WT, hatWT, Q."""
    m, n = W.shape
    WT, wscale = rotate_weight(W, su, sv, lut_rms, scale_override)
    hatWT = torch.empty_like(WT)
    Q = torch.empty(((m // 16) * (n // 16), 128), dtype=torch.int16, device=W.device)
    ws = ldlq_gpu(WT, L, n, m, hatWT, Q, lut_h2, workspace=workspace)
    packed = pack_trellis(Q)
    trellis = swizzle_for_kernel(packed, m, n)
    return {"trellis": trellis, "SU": su.to(torch.bfloat16), "SV": sv * wscale, "wscale": wscale, "WT": WT,
            "hatWT": hatWT, "Q": Q, "workspace": ws}


def quantize_linear_fused(W, L, su, sv, lut_h2, lut_rms, workspace=None, scale_override=0.9):
    """quantize_linear as ONE C-ABI call (qtip_quantize_linear): same inputs, same outputs, bit for bit."""
    init()
    m, n = W.shape
    WT = torch.empty((n, m), dtype=torch.float32, device=W.device)
    hatWT = torch.empty_like(WT)
    Q = torch.empty(((m // 16) * (n // 16), 128), dtype=torch.int16, device=W.device)
    trellis = torch.empty(((m // 16) * (n // 16), 32), dtype=torch.int16, device=W.device)
    if workspace is None:
        workspace = Workspace(lib().raw("qtip_quantize_linear_workspace_bytes")(m, n))
    wscale = C.c_float()
    lib().call("qtip_quantize_linear", _p(W, torch.float32), _p(L, torch.float32), m, n, _p(su, torch.float32),
               _p(sv, torch.float32), _p(lut_h2, torch.int32), float(lut_rms), float(scale_override),
               _p(WT, torch.float32), _p(hatWT, torch.float32), _p(Q, torch.int16), _p(trellis, torch.int16),
               C.byref(wscale), workspace.ptr, workspace.nbytes, _stream())
    return {"trellis": trellis, "SU": su.to(torch.bfloat16), "SV": sv * wscale.value, "wscale": wscale.value, "WT": WT,
            "hatWT": hatWT, "Q": Q, "workspace": workspace}


def block_ldl(HR, want_f64=False, workspace=None):
    """ldl_hessian of the reference (src/quantizer.cpp:154-165) on the GPU: fp64 symmetrisation, blocked Cholesky and the
    16 x 16 block LDL of HR [n, n] f32 (the rotated, damped Hessian). Returns L [n, n] f32, strictly block-lower (with
    want_f64 also the values before rounding to fp32). Raises QtipError (code -6) when HR is not positive definite."""
    init()
    n = HR.shape[0]
    if workspace is None:
        workspace = Workspace(lib().raw("qtip_block_ldl_workspace_bytes")(int(n)))
    L = torch.empty((n, n), dtype=torch.float32, device=HR.device)
    L64 = torch.empty((n, n), dtype=torch.float64, device=HR.device) if want_f64 else None
    lib().call("qtip_block_ldl", _p(HR, torch.float32), n, _p(L, torch.float32), _p(L64, torch.float64), workspace.ptr,
               workspace.nbytes, _stream())
    lib().call("qtip_block_ldl_status", workspace.ptr, _stream())
    return (L, L64) if want_f64 else L


def quantize_group(weights, HR, L, su, svs, creg, lut_h2, lut_rms, scale_override=0.9, workspace=None):
    """quantize_group of the reference (src/quantizer.cpp:166-346) as ONE C-ABI call: `weights` [m_i, n] f32 device
    tensors (overwritten) that share the rotated Hessian HR, its block LDL factor L and SU; `svs` their sign vectors.
    Returns one dict per linear (trellis in kernel layout, SU bf16, SV = sign * Wscale, wscale, proxy, proxy_rot_reg)
    and the shared tensors (WT, hatWT, Q)."""
    from ._lib import QtipGroupLinear
    init()
    n = HR.shape[0]
    mt = sum(int(w.shape[0]) for w in weights)
    m_max = max(int(w.shape[0]) for w in weights)
    dev = HR.device
    WT = torch.empty((n, mt), dtype=torch.float32, device=dev)
    hatWT = torch.empty_like(WT)
    Q = torch.empty(((mt // 16) * (n // 16), 128), dtype=torch.int16, device=dev)
    trellis = [torch.empty(((w.shape[0] // 16) * (n // 16), 32), dtype=torch.int16, device=dev) for w in weights]
    lins = (QtipGroupLinear * len(weights))()
    for i, (w, sv) in enumerate(zip(weights, svs)):
        assert w.dtype == torch.float32 and w.is_contiguous() and w.shape[1] == n
        lins[i].W_d, lins[i].m, lins[i].sv_d, lins[i].trellis_d = w.data_ptr(), w.shape[0], sv.data_ptr(), trellis[i].data_ptr()
    if workspace is None:
        workspace = Workspace(lib().raw("qtip_quantize_group_workspace_bytes")(n, mt, m_max))
    lib().call("qtip_quantize_group", lins, len(weights), n, _p(HR, torch.float32), _p(L, torch.float32),
               _p(su, torch.float32), float(creg), _p(lut_h2, torch.int32), float(lut_rms), float(scale_override),
               _p(WT, torch.float32), _p(hatWT, torch.float32), _p(Q, torch.int16), workspace.ptr, workspace.nbytes,
               _stream())
    workspace.check()
    outs = [{"trellis": trellis[i], "SU": su.to(torch.bfloat16), "SV": svs[i] * lins[i].wscale, "wscale": lins[i].wscale,
             "proxy": lins[i].proxy, "proxy_rot_reg": lins[i].proxy_rot_reg} for i in range(len(weights))]
    return outs, {"WT": WT, "hatWT": hatWT, "Q": Q}


def rotate_hessian_fused(H, su, sigma_reg=1e-2):
    """rotate_hessian as ONE C-ABI call (qtip_rotate_hessian): same result, bit for bit."""
    init()
    n = H.shape[0]
    HR = torch.empty_like(H)
    scratch = torch.zeros(1, dtype=torch.float64, device=H.device)
    creg = C.c_double()
    lib().call("qtip_rotate_hessian", _p(H, torch.float32), n, _p(su, torch.float32), float(sigma_reg),
               _p(HR, torch.float32), C.byref(creg), _p(scratch, torch.float64), _stream())
    return HR, creg.value
