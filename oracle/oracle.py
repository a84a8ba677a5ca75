"""TEST INFRASTRUCTURE ONLY: numpy/ctypes front end of the CPU oracle (liboracle.so, built from qtip_oracle.c) and,
when present, of the reference's own CPU code compiled in place (_ref/libqtip_ref_{encode,decode}.so).

Only the test suite, the smoke check and the CPU-baseline leg of the benchmark may import this module. The
product package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")


def reference_root():
    """Root of the reference project's source tree: the QTIP_REFERENCE_ROOT environment variable, else the Makefile's
    default (REF). The tree is optional: without it only the prebuilt files under _ref/ are used."""
    root = os.environ.get("QTIP_REFERENCE_ROOT")
    if root:
        return root
    with open(os.path.join(_HERE, "Makefile")) as f:
        for line in f:
            if line.startswith("REF ?="):
                return line.split("=", 1)[1].strip()
    return ""


def build(ref=False):
    """Compile the oracle (and, with ref=True and the reference tree present, the reference's CPU code and, when nvcc is
    there, the reference's CUDA kernels for this path)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    root = reference_root()
    if ref and root and os.path.isdir(os.path.join(root, "src")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "REF=" + root], stderr=subprocess.DEVNULL)
        if os.path.exists(os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")):
            subprocess.check_call(["make", "-s", "-C", _HERE, "refgpu", "refquant", "REF=" + root],
                                  stderr=subprocess.DEVNULL)


def _load(path):
    return C.CDLL(path) if os.path.exists(path) else None


def _opt(a, ptr_type=None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Oracle:
    """The plain-C restatement."""

    def __init__(self):
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        L = self.lib = C.CDLL(path)
        L.qo_f16_to_f32.restype = C.c_float
        L.qo_f16_to_f32.argtypes = [C.c_uint16]
        L.qo_f32_to_f16.restype = C.c_uint16
        L.qo_f32_to_f16.argtypes = [C.c_float]
        L.qo_build_lut.argtypes = [_u16p, _u32p, C.POINTER(C.c_double)]
        L.qo_runtime_codebook.argtypes = [_u16p, _f32p, _f32p, _u32p]
        L.qo_perm.argtypes = [_i32p, _i32p]
        L.qo_viterbi_fwd.argtypes = [_f32p, C.c_void_p, C.c_int, C.c_int, _u16p, _u16p, _u32p]
        L.qo_viterbi_overlap.argtypes = [_u16p, _u16p, C.c_int, _i32p]
        L.qo_viterbi_finish.argtypes = [_u16p, _u16p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                        C.c_long, C.c_int, _u32p]
        L.qo_decode_states.argtypes = [_u16p, C.c_int, _f32p, _u32p]
        L.qo_quantize_tiles.argtypes = [_f32p, C.c_int, _u32p, C.c_void_p, C.c_void_p]
        L.qo_quantize_seq_ref.argtypes = [_f32p, C.c_int, _u32p, _u16p, C.c_void_p, C.c_void_p]
        L.qo_path_cost.restype = C.c_double
        L.qo_path_cost.argtypes = [_f32p, _u16p, _u32p]
        L.qo_pack_trellis.argtypes = [_u16p, C.c_long, _u16p]
        L.qo_unpack_trellis.argtypes = [_u16p, C.c_long, _u16p]
        L.qo_swizzle.argtypes = [_u16p, C.c_int, C.c_int, _u16p]
        L.qo_unswizzle.argtypes = [_u16p, C.c_int, C.c_int, _u16p]
        L.qo_had_table.argtypes = [C.c_int, _i8p]
        L.qo_had_K.argtypes = [C.c_int]
        L.qo_hadamard_rows_ref.argtypes = [_f64p, C.c_long, C.c_int, C.c_long, C.c_int]
        L.qo_ldlq_prep.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_long, C.c_long, C.c_int, C.c_int, _f32p]
        L.qo_ldlq_f32.argtypes = [_f32p, _f32p, C.c_long, C.c_long, _f32p, _u16p, _u32p]
        L.qo_ldlq_ref.argtypes = [_f32p, _f32p, C.c_int, C.c_int, _f32p, _u16p, _u32p]
        L.qo_block_ldl.argtypes = [_f64p, C.c_int, _f32p]
        L.qo_decode_rows.argtypes = [_u16p, C.c_int, C.c_int, _f32p, _f32p, C.c_int, C.c_int, _f32p]
        L.qo_rt_hadamard.argtypes = [_f64p, C.c_int, C.c_int]
        L.qo_reference_forward.argtypes = [_u16p, _f32p, _f32p, _u16p, C.c_int, C.c_int, _f32p, C.c_int, C.c_int,
                                           C.c_int, _f32p, C.c_void_p]
        L.qo_fp8_forward.argtypes = [_u8p, _f32p, C.c_int, C.c_int, _f32p, C.c_int, C.c_int, _f32p]

    # ---- codebook
    def build_lut(self, tlut_h):
        tlut_h = np.ascontiguousarray(tlut_h, np.uint16).reshape(-1)
        assert tlut_h.size == 1024
        lut = np.empty(65536, np.uint32)
        rms = C.c_double()
        self.lib.qo_build_lut(tlut_h, lut, C.byref(rms))
        return lut, rms.value

    def runtime_codebook(self, tlut_h):
        tlut_h = np.ascontiguousarray(tlut_h, np.uint16).reshape(-1)
        c0, c1, b2 = np.empty(1024, np.float32), np.empty(1024, np.float32), np.empty(1024, np.uint32)
        if self.lib.qo_runtime_codebook(tlut_h, c0, c1, b2):
            raise ValueError("non-finite tlut entry")
        return c0, c1, b2

    def perm(self):
        p, i = np.empty(256, np.int32), np.empty(256, np.int32)
        self.lib.qo_perm(p, i)
        return p, i

    # ---- exact Viterbi (kernel arithmetic)
    def viterbi_fwd(self, X, overlap, roll, lut):
        X = np.ascontiguousarray(X, np.float32).reshape(-1, 256)
        B = X.shape[0]
        A = np.empty((B, 127, 1024), np.uint16)
        fs = np.empty(B, np.uint16)
        ov = None if overlap is None else np.ascontiguousarray(overlap, np.int32)
        self.lib.qo_viterbi_fwd(X, _opt(ov), int(roll), B, A, fs, lut)
        return A, fs

    def viterbi_overlap(self, A, fs):
        B = fs.shape[0]
        ov = np.empty(B, np.int32)
        self.lib.qo_viterbi_overlap(A, fs, B, ov)
        return ov

    def viterbi_finish(self, A, fs, lut, b0=0, nblk=1, blk=0, Q=None, hatWT=None, m=0, col0=0):
        B = fs.shape[0]
        if Q is None:
            Q = np.zeros(((b0 + B) * nblk, 128), np.uint16)
        self.lib.qo_viterbi_finish(A, fs, B, b0, _opt(Q), nblk, blk, _opt(hatWT), m, col0, lut)
        return Q

    def decode_states(self, states, lut):
        states = np.ascontiguousarray(states, np.uint16).reshape(-1, 128)
        hat = np.empty((states.shape[0], 256), np.float32)
        self.lib.qo_decode_states(states, states.shape[0], hat, lut)
        return hat

    def quantize_tiles(self, X, lut):
        X = np.ascontiguousarray(X, np.float32).reshape(-1, 256)
        B = X.shape[0]
        st, hat = np.empty((B, 128), np.uint16), np.empty((B, 256), np.float32)
        self.lib.qo_quantize_tiles(X, B, lut, _opt(st), _opt(hat))
        return st, hat

    # ---- fp64 Viterbi
    def quantize_seq_ref(self, X, lut):
        X = np.ascontiguousarray(X, np.float32).reshape(-1, 256)
        B = X.shape[0]
        st, hat, cost = np.empty((B, 128), np.uint16), np.empty((B, 256), np.float32), np.empty(B, np.float64)
        self.lib.qo_quantize_seq_ref(X, B, lut, st, _opt(hat), _opt(cost))
        return st, hat, cost

    def path_cost(self, x, states, lut):
        return self.lib.qo_path_cost(np.ascontiguousarray(x, np.float32), np.ascontiguousarray(states, np.uint16), lut)

    # ---- packing
    def pack(self, states):
        states = np.ascontiguousarray(states, np.uint16).reshape(-1, 128)
        out = np.empty((states.shape[0], 32), np.uint16)
        self.lib.qo_pack_trellis(states, states.shape[0], out)
        return out

    def unpack(self, packed):
        packed = np.ascontiguousarray(packed, np.uint16).reshape(-1, 32)
        out = np.empty((packed.shape[0], 128), np.uint16)
        self.lib.qo_unpack_trellis(packed, packed.shape[0], out)
        return out

    def swizzle(self, packed, m, n):
        packed = np.ascontiguousarray(packed, np.uint16)
        out = np.empty_like(packed)
        if self.lib.qo_swizzle(packed, m, n, out):
            raise ValueError("kernel layout needs m, n multiples of 32")
        return out

    def unswizzle(self, words, m, n):
        words = np.ascontiguousarray(words, np.uint16)
        out = np.empty_like(words)
        if self.lib.qo_unswizzle(words, m, n, out):
            raise ValueError("kernel layout needs m, n multiples of 32")
        return out

    # ---- Hadamard
    def had_table(self, K):
        H = np.empty((K, K), np.int8)
        if self.lib.qo_had_table(K, H):
            raise ValueError("no table of order %d" % K)
        return H

    def had_K(self, n):
        return self.lib.qo_had_K(n)

    def hadamard_rows(self, X, transpose):
        X = np.array(X, np.float64, order="C")
        X2 = X.reshape(-1, X.shape[-1])
        if self.lib.qo_hadamard_rows_ref(X2, X2.shape[0], X2.shape[1], X2.shape[1], int(transpose)):
            raise ValueError("unsupported Hadamard size")
        return X

    # ---- LDLQ
    def ldlq_prep(self, WT, hatWT, prod, L, col0, bufend):
        n, m = WT.shape
        X = np.empty((m // 16, 256), np.float32)
        self.lib.qo_ldlq_prep(WT, hatWT, prod, L, n, m, col0, bufend, X)
        return X

    def ldlq_f32(self, WT, L, lut):
        WT = np.ascontiguousarray(WT, np.float32)
        L = np.ascontiguousarray(L, np.float32)
        n, m = WT.shape
        hat = np.empty((n, m), np.float32)
        Q = np.empty(((m // 16) * (n // 16), 128), np.uint16)
        if self.lib.qo_ldlq_f32(WT, L, n, m, hat, Q, lut):
            raise ValueError("LDLQ needs n % 128 == 0 and m % 16 == 0")
        return hat, Q

    def ldlq_ref(self, Wr, L, lut):
        Wr = np.ascontiguousarray(Wr, np.float32)
        L = np.ascontiguousarray(L, np.float32)
        m, n = Wr.shape
        hat = np.empty((m, n), np.float32)
        Q = np.empty(((m // 16) * (n // 16), 128), np.uint16)
        if self.lib.qo_ldlq_ref(Wr, L, m, n, hat, Q, lut):
            raise ValueError("LDLQ needs n % 128 == 0 and m % 16 == 0")
        return hat, Q

    def block_ldl(self, H):
        A = np.array(H, np.float64, order="C")
        n = A.shape[0]
        L = np.empty((n, n), np.float32)
        rc = self.lib.qo_block_ldl(A, n, L)
        if rc:
            raise ValueError("block LDL failed (%d)" % rc)
        return L

    # ---- decode side
    def decode_rows(self, trellis, n_in, n_out, tlut_h, row0, rows, bf16):
        c0, c1, b2 = self.runtime_codebook(tlut_h)
        if bf16:
            c0 = ((b2 & 0xFFFF) << 16).astype(np.uint32).view(np.float32)
            c1 = (b2 & 0xFFFF0000).astype(np.uint32).view(np.float32)
        w = np.empty((rows, n_in), np.float32)
        if self.lib.qo_decode_rows(np.ascontiguousarray(trellis, np.uint16).reshape(-1), n_in, n_out,
                                   np.ascontiguousarray(c0), np.ascontiguousarray(c1), row0, rows, w):
            raise ValueError("decode rows must be whole 16-row tiles")
        return w

    def rt_hadamard(self, x, transpose):
        x = np.array(x, np.float64, order="C")
        if self.lib.qo_rt_hadamard(x, x.size, int(transpose)):
            raise ValueError("unsupported Hadamard size")
        return x

    # ---- fused decode-step epilogues (runtime/src/qtip.hip:713-930 of the reference), restated in numpy around the
    # fp64 transform: where the device rounds to bf16, so does this; the transforms themselves are exact here.
    @staticmethod
    def _bf16(x):
        u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
        return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)

    def input_transform(self, x, norm, epsilon, su):
        """x [rows, n] (bf16 values as f32), norm [n] (bf16 values) or None -> (u, xn): input_transform_chunk."""
        x = np.asarray(x, np.float32)
        xn = x
        if norm is not None:
            factor = (1.0 / np.sqrt(np.mean(x.astype(np.float64) ** 2, axis=1) + epsilon)).astype(np.float32)
            xn = self._bf16(x * factor[:, None] * np.asarray(norm, np.float32)[None, :])
        u = np.stack([self.rt_hadamard(np.asarray(su, np.float64) * r, True) for r in xn.astype(np.float64)])
        return self._bf16(u.astype(np.float32)), xn

    def output_transform(self, z, sv, round_z=False):
        """bf16(SV (.) hadU(z)) per row: the operator's output stage."""
        z = np.asarray(z, np.float32)
        if round_z:
            z = self._bf16(z)
        y = np.stack([self.rt_hadamard(r, False) for r in z.astype(np.float64)]) * np.asarray(sv, np.float64)[None, :]
        return self._bf16(y.astype(np.float32))

    def output_residual(self, z, sv, state):
        return self._bf16(np.asarray(state, np.float32) + self.output_transform(z, sv))

    def output_gateup(self, z, sv_gate, sv_up):
        F = z.shape[1] // 2
        g = self.output_transform(z[:, :F], sv_gate, True).astype(np.float64)
        u = self.output_transform(z[:, F:], sv_up, True).astype(np.float64)
        return self._bf16((g / (1.0 + np.exp(-g)) * u).astype(np.float32))

    def reference_forward(self, trellis, su, sv, tlut_h, n_in, n_out, x, device_rounding=False, round_z=False,
                          want_z=False):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, n_in)
        rows = x.shape[0]
        y = np.empty((rows, n_out), np.float32)
        z = np.empty((rows, n_out), np.float32) if want_z else None
        rc = self.lib.qo_reference_forward(np.ascontiguousarray(trellis, np.uint16).reshape(-1),
                                           np.ascontiguousarray(su, np.float32), np.ascontiguousarray(sv, np.float32),
                                           np.ascontiguousarray(tlut_h, np.uint16).reshape(-1), n_in, n_out, x, rows,
                                           int(device_rounding), int(round_z), y, _opt(z))
        if rc:
            raise ValueError("reference_forward failed")
        return (y, z) if want_z else y

    def fp8_forward(self, w, scale, x, device_rounding=True):
        w = np.ascontiguousarray(w, np.uint8)
        n_out, n_in = w.shape
        x = np.ascontiguousarray(x, np.float32).reshape(-1, n_in)
        y = np.empty((x.shape[0], n_out), np.float32)
        self.lib.qo_fp8_forward(w, np.ascontiguousarray(scale, np.float32), n_in, n_out, x, x.shape[0],
                                int(device_rounding), y)
        return y


class Reference:
    """The reference's own CPU code compiled in place. `available` is False when the prebuilt files are absent."""

    def __init__(self):
        self.enc = _load(os.path.join(_HERE, "_ref", "libqtip_ref_encode.so"))
        self.dec = _load(os.path.join(_HERE, "_ref", "libqtip_ref_decode.so"))
        self.available = self.enc is not None and self.dec is not None
        if self.enc is not None:
            E = self.enc
            E.ref_codebook.argtypes = [_u16p, _u32p, C.POINTER(C.c_double)]
            E.ref_perm.argtypes = [_i32p, _i32p]
            E.ref_had_table.argtypes = [C.c_int, _i8p]
            E.ref_hadamard_rows.argtypes = [_f64p, C.c_long, C.c_int, C.c_long, C.c_int]
            E.ref_quantize_seqs.argtypes = [_f32p, C.c_int, _u16p, C.c_void_p, C.c_void_p]
            E.ref_path_cost.restype = C.c_double
            E.ref_path_cost.argtypes = [_f32p, _u16p]
            E.ref_pack_trellis.argtypes = [_u16p, C.c_long, _u16p]
            E.ref_unpack_trellis.argtypes = [_u16p, C.c_long, _u16p]
            E.ref_swizzle.argtypes = [_u16p, C.c_int, C.c_int, _u16p]
            E.ref_unswizzle.argtypes = [_u16p, C.c_int, C.c_int, _u16p]
            E.ref_block_ldl.argtypes = [_f64p, C.c_int, _f32p, C.c_int]
        if self.dec is not None:
            D = self.dec
            D.rref_codebook.argtypes = [_u16p, _f32p, _f32p, _u32p]
            D.rref_hadamard.argtypes = [_f64p, C.c_int, C.c_int]
            D.rref_decode_rows.argtypes = [_u16p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _f32p]
            D.rref_forward.argtypes = [_u16p, _f32p, _f32p, _u16p, C.c_int, C.c_int, _f32p, C.c_int, C.c_int, C.c_int,
                                       _f32p]

    def codebook(self):
        """(tlut fp16 bits [512,2], lut_h2 [65536], lut_rms) of the reference's committed HYB code."""
        t, l, r = np.empty(1024, np.uint16), np.empty(65536, np.uint32), C.c_double()
        self.enc.ref_codebook(t, l, C.byref(r))
        return t.reshape(512, 2), l, r.value

    def perm(self):
        p, i = np.empty(256, np.int32), np.empty(256, np.int32)
        self.enc.ref_perm(p, i)
        return p, i

    def had_table(self, K):
        H = np.empty((K, K), np.int8)
        return H if self.enc.ref_had_table(K, H) else None

    def hadamard_rows(self, X, transpose):
        X = np.array(X, np.float64, order="C")
        X2 = X.reshape(-1, X.shape[-1])
        self.enc.ref_hadamard_rows(X2, X2.shape[0], X2.shape[1], X2.shape[1], int(transpose))
        return X

    def quantize_seqs(self, X):
        X = np.ascontiguousarray(X, np.float32).reshape(-1, 256)
        B = X.shape[0]
        st, hat, cost = np.empty((B, 128), np.uint16), np.empty((B, 256), np.float32), np.empty(B, np.float64)
        self.enc.ref_quantize_seqs(X, B, st, _opt(hat), _opt(cost))
        return st, hat, cost

    def pack(self, states):
        states = np.ascontiguousarray(states, np.uint16).reshape(-1, 128)
        out = np.empty((states.shape[0], 32), np.uint16)
        self.enc.ref_pack_trellis(states, states.shape[0], out)
        return out

    def unpack(self, packed):
        packed = np.ascontiguousarray(packed, np.uint16).reshape(-1, 32)
        out = np.empty((packed.shape[0], 128), np.uint16)
        self.enc.ref_unpack_trellis(packed, packed.shape[0], out)
        return out

    def swizzle(self, packed, m, n):
        packed = np.ascontiguousarray(packed, np.uint16)
        out = np.empty_like(packed)
        self.enc.ref_swizzle(packed, m, n, out)
        return out

    def block_ldl(self, H, threads=4):
        A = np.array(H, np.float64, order="C")
        L = np.empty(A.shape, np.float32)
        if self.enc.ref_block_ldl(A, A.shape[0], L, threads):
            raise ValueError("block LDL failed")
        return L

    def runtime_codebook(self, tlut_h):
        c0, c1, b2 = np.empty(1024, np.float32), np.empty(1024, np.float32), np.empty(1024, np.uint32)
        if self.dec.rref_codebook(np.ascontiguousarray(tlut_h, np.uint16).reshape(-1), c0, c1, b2):
            raise ValueError("make_codebook failed")
        return c0, c1, b2

    def rt_hadamard(self, x, transpose):
        x = np.array(x, np.float64, order="C")
        if self.dec.rref_hadamard(x, x.size, int(transpose)):
            raise ValueError("unsupported Hadamard size")
        return x

    def decode_rows(self, trellis, n_in, n_out, tlut_h, row0, rows, bf16):
        w = np.empty((rows, n_in), np.float32)
        if self.dec.rref_decode_rows(np.ascontiguousarray(trellis, np.uint16).reshape(-1),
                                     np.ascontiguousarray(tlut_h, np.uint16).reshape(-1), n_in, n_out, row0, rows,
                                     int(bf16), w):
            raise ValueError("decode_rows failed")
        return w

    def reference_forward(self, trellis, su, sv, tlut_h, n_in, n_out, x, device_rounding=False, round_z=False):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, n_in)
        y = np.empty((x.shape[0], n_out), np.float32)
        if self.dec.rref_forward(np.ascontiguousarray(trellis, np.uint16).reshape(-1),
                                 np.ascontiguousarray(su, np.float32), np.ascontiguousarray(sv, np.float32),
                                 np.ascontiguousarray(tlut_h, np.uint16).reshape(-1), n_in, n_out, x, x.shape[0],
                                 int(device_rounding), int(round_z), y):
            raise ValueError("reference_forward failed")
        return y


    # ---- layer files (safetensors): the quantizer's container writer and the runtime's loader
    def write_layer_file(self, path, layer, linears, tlut_h):
        """SafeTensorsWriter of the reference with write_layer_file's tensor set. linears: {name: (m, n, trellis u16, su
        bf16 bits u16, sv f32)}."""
        count = len(linears)
        names = (C.c_char_p * count)(*[k.encode() for k in linears])
        vals = list(linears.values())
        m = (C.c_int * count)(*[v[0] for v in vals])
        n = (C.c_int * count)(*[v[1] for v in vals])
        keep = [[np.ascontiguousarray(v[2], np.uint16), np.ascontiguousarray(v[3], np.uint16),
                 np.ascontiguousarray(v[4], np.float32)] for v in vals]
        tr = (C.c_void_p * count)(*[k[0].ctypes.data for k in keep])
        su = (C.c_void_p * count)(*[k[1].ctypes.data for k in keep])
        sv = (C.c_void_p * count)(*[k[2].ctypes.data for k in keep])
        tl = np.ascontiguousarray(tlut_h, np.uint16).reshape(-1)
        self.enc.ref_write_layer_file.restype = None
        self.enc.ref_write_layer_file.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        self.enc.ref_write_layer_file(str(path).encode(), layer, count, names, m, n, tr, su, sv, tl.ctypes.data)

    def load_linear(self, path, layer, name, hidden, intermediate, kv_heads, dim, m, n):
        """load_linear of the reference runtime on a layer file; raises ValueError with its message on a failed check."""
        tr = np.empty(((m // 16) * (n // 16), 32), np.uint16)
        su, sv, tl = np.empty(n, np.float32), np.empty(m, np.float32), np.empty((512, 2), np.uint16)
        i_in, i_out = C.c_int(0), C.c_int(0)
        f = self.dec.rref_load_linear
        f.argtypes = [C.c_char_p, C.c_int, C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int),
                      C.POINTER(C.c_int), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        if f(str(path).encode(), layer, name.encode(), hidden, intermediate, kv_heads, dim, C.byref(i_in), C.byref(i_out),
             tr.ctypes.data, su.ctypes.data, sv.ctypes.data, tl.ctypes.data):
            self.dec.rref_last_error.restype = C.c_char_p
            raise ValueError(self.dec.rref_last_error().decode())
        assert (i_in.value, i_out.value) == (n, m)
        return {"trellis": tr, "SU": su, "SV": sv, "tlut": tl}


class ReferenceGpu:
    """The reference's own CUDA kernels for this path, compiled in place for sm_100a (Makefile target `refgpu`).

    Every pointer argument is a raw device address (an int, e.g. a torch tensor's data_ptr()); `stream` is a
    cudaStream_t as an int (0 = the default stream). Encode-side errors abort the process, as in the reference; the
    runtime-side wrappers raise RuntimeError with the reference's message. `available` is False when the prebuilt
    files are absent."""

    def __init__(self):
        self.enc = _load(os.path.join(_HERE, "_ref", "libqtip_ref_gpu_encode.so"))
        self.dec = _load(os.path.join(_HERE, "_ref", "libqtip_ref_gpu_decode.so"))
        self.available = self.enc is not None and self.dec is not None
        P, I, L = C.c_void_p, C.c_int, C.c_long
        if self.enc is not None:
            E = self.enc
            E.refgpu_ldlq_prep.argtypes = [P, P, P, P, L, L, I, I, P, P]
            E.refgpu_viterbi_fwd.argtypes = [P, P, I, I, P, P, P, P]
            E.refgpu_viterbi_overlap.argtypes = [P, P, I, P, P]
            E.refgpu_viterbi_finish.argtypes = [P, P, I, I, P, I, I, P, L, I, P, P]
            E.refgpu_decode_states.argtypes = [P, I, P, P, P]
            for f in (E.refgpu_ldlq_prep, E.refgpu_viterbi_fwd, E.refgpu_viterbi_overlap, E.refgpu_viterbi_finish,
                      E.refgpu_decode_states):
                f.restype = None
        if self.dec is not None:
            D = self.dec
            D.refgpu_last_error.restype = C.c_char_p
            M = [P, P, P, P, I, I]  # trellis, su, sv, lut, in, out
            D.refgpu_qtip_prepare.argtypes = M + [P, P, P, P, I, I]
            D.refgpu_qtip_multiply.argtypes = M + [P, P, I, I, P, I]
            D.refgpu_qtip_finish.argtypes = M + [P, P, P, I, I, P, I, I]
            D.refgpu_qtip_forward.argtypes = M + [P, P, P, P, P, I, P, I]
            D.refgpu_qtip_multiply_batch.argtypes = M + [P, P, I, I, I, P, I]
            D.refgpu_qtip_decode_matrix.argtypes = M + [P, P]
            D.refgpu_fp8_forward.argtypes = [P, P, P, P, I, I, P]

    def _rt(self, rc):
        if rc:
            raise RuntimeError(self.dec.refgpu_last_error().decode())

    # ---- encode side (src/gpu.hpp:276-292)
    def ldlq_prep(self, WT, hatWT, prod, L, n, m, col0, bufend, X, stream=0):
        self.enc.refgpu_ldlq_prep(WT, hatWT, prod, L, n, m, col0, bufend, X, stream)

    def viterbi_fwd(self, X, overlap, roll, B, A, final_state, lut_h2, stream=0):
        self.enc.refgpu_viterbi_fwd(X, overlap, roll, B, A, final_state, lut_h2, stream)

    def viterbi_overlap(self, A, final_state, B, overlap, stream=0):
        self.enc.refgpu_viterbi_overlap(A, final_state, B, overlap, stream)

    def viterbi_finish(self, A, final_state, B, b0, Q, nblk, blk, hatWT, m, col0, lut_h2, stream=0):
        self.enc.refgpu_viterbi_finish(A, final_state, B, b0, Q, nblk, blk, hatWT, m, col0, lut_h2, stream)

    def decode_states(self, states, B, hat, lut_h2, stream=0):
        self.enc.refgpu_decode_states(states, B, hat, lut_h2, stream)

    # ---- runtime side (runtime/cuda/kernels.hpp:5-24, runtime/cuda/batch_kernels.hpp:5-8); w = (trellis, su, sv, lut, in, out)
    def initialize_tables(self):
        self._rt(self.dec.refgpu_initialize_tables())

    def qtip_prepare(self, w, x, scratch, rotated, tokens=1, rank_major=False, stream=0):
        self._rt(self.dec.refgpu_qtip_prepare(*w, x, scratch, rotated, stream, tokens, int(rank_major)))

    def qtip_multiply(self, w, rotated, z, stride, splits, tokens=1, stream=0):
        self._rt(self.dec.refgpu_qtip_multiply(*w, rotated, z, stride, splits, stream, tokens))

    def qtip_finish(self, w, z, y, scratch, round_z, splits, tokens=1, rank_major=False, stream=0):
        self._rt(self.dec.refgpu_qtip_finish(*w, z, y, scratch, int(round_z), splits, stream, tokens, int(rank_major)))

    def qtip_forward(self, w, x, y, scratch, rotated, z, round_z, splits=1, stream=0):
        self._rt(self.dec.refgpu_qtip_forward(*w, x, y, scratch, rotated, z, int(round_z), stream, splits))

    def qtip_multiply_batch(self, w, rotated, z, stride, splits, tokens, implementation=-1, stream=0):
        self._rt(self.dec.refgpu_qtip_multiply_batch(*w, rotated, z, stride, splits, tokens, stream, implementation))

    def qtip_decode_matrix(self, w, dense, stream=0):
        self._rt(self.dec.refgpu_qtip_decode_matrix(*w, dense, stream))

    def fp8_forward(self, wq, scale, x, y, n_in, n_out, stream=0):
        self._rt(self.dec.refgpu_fp8_forward(wq, scale, x, y, n_in, n_out, stream))


class ReferenceQuant:
    """The reference's own GPU quantizer (src/quantizer.cpp: ldlq_gpu and quantize_group, with its kernels and its
    library-GEMM wrapper), compiled in place for sm_100a (Makefile target `refquant`). Its codebook is the one compiled
    into the reference. `available` is False when the prebuilt file is absent."""

    def __init__(self):
        self.lib = _load(os.path.join(_HERE, "_ref", "libqtip_ref_gpu_quant.so"))
        self.available = self.lib is not None
        if self.lib is None:
            return
        P, I, L, D = C.c_void_p, C.c_int, C.c_long, C.c_double
        self.lib.refq_ldlq_gpu.argtypes = [P, P, L, L, P, P, I, C.POINTER(D), P]
        self.lib.refq_ldlq_gpu.restype = None
        self.lib.refq_quantize_group.argtypes = [I, P, P, I, P, C.c_uint64, D, D, I, P, P, P, P, P, P, P, P]
        self.lib.refq_quantize_group.restype = None

    def ldlq_gpu(self, WT, L, n, m, hatWT, Q, vit_batch=1024, stream=0):
        """Device addresses (ints). Returns the seconds the reference spent in its Viterbi kernels (it synchronises
        around them to measure)."""
        vit = C.c_double(0.0)
        self.lib.refq_ldlq_gpu(WT, L, n, m, hatWT, Q, vit_batch, C.byref(vit), stream)
        return vit.value

    def quantize_group(self, weights, H, seed, sigma_reg=1e-2, scale_override=0.9, ldl_threads=8, stream=0):
        """weights: list of [m_i, n] fp32 host arrays sharing the Hessian H [n, n] (fp32 host). Returns one dict per
        linear (trellis, su_bf16, sv, wscale, proxy, proxy_rot_reg) and the GroupTiming fields."""
        n = H.shape[0]
        count = len(weights)
        W = [np.ascontiguousarray(w, np.float32) for w in weights]
        H = np.ascontiguousarray(H, np.float32)
        m = (C.c_int * count)(*[w.shape[0] for w in W])
        wp = (C.c_void_p * count)(*[w.ctypes.data for w in W])
        tr = [np.empty((w.shape[0] // 16) * (n // 16) * 32, np.uint16) for w in W]
        su = [np.empty(n, np.uint16) for _ in W]
        sv = [np.empty(w.shape[0], np.float32) for w in W]
        trp = (C.c_void_p * count)(*[a.ctypes.data for a in tr])
        sup = (C.c_void_p * count)(*[a.ctypes.data for a in su])
        svp = (C.c_void_p * count)(*[a.ctypes.data for a in sv])
        wscale = np.empty(count, np.float32)
        proxy, proxy_rr = np.empty(count, np.float64), np.empty(count, np.float64)
        timing = np.zeros(8, np.float64)
        self.lib.refq_quantize_group(count, m, wp, n, H.ctypes.data, seed, sigma_reg, scale_override, ldl_threads, trp, sup,
                                     svp, wscale.ctypes.data, proxy.ctypes.data, proxy_rr.ctypes.data,
                                     timing.ctypes.data, stream)
        names = ("load", "rht", "ldl_cpu", "ldlq", "viterbi", "proxy", "pack", "total")
        outs = [{"trellis": tr[i], "su_bf16": su[i], "sv": sv[i], "wscale": float(wscale[i]), "proxy": float(proxy[i]),
                 "proxy_rot_reg": float(proxy_rr[i])} for i in range(count)]
        return outs, dict(zip(names, timing.tolist()))
