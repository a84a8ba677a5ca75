"""Host-side mirror of the runtime's QTIP linear operator (runtime/cuda/kernels.hpp:5-24 and
runtime/cuda/batch_kernels.hpp:5-8,22-23 of the reference): QtipMatrix and the prepare / multiply / finish stages,
with torch CUDA tensors in place of raw device pointers. bf16 tensors are passed as torch.bfloat16.
"""
import ctypes as C

import torch

from ._lib import QtipMatrix, lib
from .codec import _p, _stream, init, tlut_bits


def runtime_lut(tlut_f16):
    """bf16x2 table (1,024 sign-folded entries) of a tlut on the current device: make_codebook of the reference."""
    init()
    bits = tlut_bits(tlut_f16)
    out = torch.empty(1024, dtype=torch.int32, device="cuda")
    lib().call("qtip_runtime_lut", bits.ctypes.data_as(C.c_void_p), _p(out), _stream())
    return out


class Matrix:
    """Owns the device tensors of one linear and exposes the POD QtipMatrix the C ABI takes by value."""

    def __init__(self, trellis, su, sv, lut, n_in, n_out):
        # trellis may be None for an object that is only handed to the transforms (qtip_prepare / qtip_finish)
        assert trellis is None or (trellis.dtype == torch.int16 and
                                   trellis.numel() == (n_out // 16) * (n_in // 16) * 32)
        assert su.dtype == torch.float32 and su.numel() == n_in and sv.dtype == torch.float32 and sv.numel() == n_out
        self.trellis, self.su, self.sv, self.lut, self.n_in, self.n_out = trellis, su, sv, lut, n_in, n_out

    @property
    def pod(self):
        return QtipMatrix(None if self.trellis is None else self.trellis.data_ptr(), self.su.data_ptr(),
                          self.sv.data_ptr(), None if self.lut is None else self.lut.data_ptr(), self.n_in, self.n_out)

    def rows(self, row0, rows):
        """Matrix of output rows [row0, row0 + rows) (whole 32-row block-rows): a contiguous run of the trellis, the
        sharding unit of rotated-row tensor parallelism. Use it for qtip_multiply only: the output transform runs on the
        gathered full-width z with the full matrix's SV."""
        assert row0 % 32 == 0 and rows % 32 == 0
        per = (self.n_in // 32) * 128
        t = self.trellis.view(-1)[(row0 // 32) * per:((row0 + rows) // 32) * per]
        return Matrix(t, self.su, self.sv[row0:row0 + rows].contiguous(), self.lut, self.n_in, rows)


def qtip_prepare(w, x, scratch, rotated, tokens=1, rank_major=0):
    init()
    lib().call("qtip_prepare", w.pod, _p(x, torch.bfloat16), _p(scratch), _p(rotated, torch.bfloat16), _stream(), tokens,
               int(rank_major))


def qtip_multiply(w, rotated, z, stride, splits, tokens=1):
    init()
    lib().call("qtip_multiply", w.pod, _p(rotated, torch.bfloat16), _p(z, torch.float32), stride, splits, _stream(),
               tokens)


def qtip_finish(w, z, y, scratch, round_z, splits, tokens=1, rank_major=0):
    init()
    lib().call("qtip_finish", w.pod, _p(z, torch.float32), _p(y, torch.bfloat16), _p(scratch), int(bool(round_z)),
               splits, _stream(), tokens, int(rank_major))


def qtip_finish_b16(w, z, y, scratch, tokens, rank_major=0):
    init()
    lib().call("qtip_finish_b16", w.pod, _p(z, torch.bfloat16), _p(y, torch.bfloat16), _p(scratch), tokens, _stream(),
               int(rank_major))


def qtip_forward(w, x, y, scratch, rotated, z, round_z, splits=1):
    init()
    lib().call("qtip_forward", w.pod, _p(x, torch.bfloat16), _p(y, torch.bfloat16), _p(scratch),
               _p(rotated, torch.bfloat16), _p(z, torch.float32), int(bool(round_z)), _stream(), splits)


def input_transform(x, norm, epsilon, su, n, rows, u, xn=None, ldx=None, ldu=None):
    """u = bf16(hadUt(SU (.) x')), x' = RMSNorm(x) with the runtime's rounding when `norm` (bf16 [n]) is given; xn
    (optional) receives x'. input_transform of the reference's ROCm operator (runtime/src/qtip.hip:713-786)."""
    init()
    lib().call("qtip_input_transform", _p(x, torch.bfloat16), n if ldx is None else ldx, _p(norm, torch.bfloat16),
               float(epsilon), _p(su, torch.float32), n, rows, _p(u, torch.bfloat16), n if ldu is None else ldu,
               _p(xn, torch.bfloat16), _stream())


def output_residual(z, splits, rows, sv, n, state, rank_major=0):
    """state = bf16(state + bf16(SV (.) hadU(sum of the K-split partials z))): output_residual of the reference."""
    init()
    lib().call("qtip_output_residual", _p(z, torch.float32), splits, rows, int(rank_major), _p(sv, torch.float32), n,
               _p(state, torch.bfloat16), _stream())


def output_gateup(z, splits, rows, sv_gate, sv_up, features, h):
    """h = bf16(silu(g) * u) from the stacked gate | up products z [splits, rows, 2 F]: output_gateup of the reference."""
    init()
    lib().call("qtip_output_gateup", _p(z, torch.float32), splits, rows, _p(sv_gate, torch.float32),
               _p(sv_up, torch.float32), features, _p(h, torch.bfloat16), _stream())


def output_residual_input(z, splits, rows, sv, n, state, norm, epsilon, su, u, xn=None, rank_major=0, ldu=None):
    """output_residual, then input_transform of the updated state (output_residual_input of the reference)."""
    init()
    lib().call("qtip_output_residual_input", _p(z, torch.float32), splits, rows, int(rank_major), _p(sv, torch.float32), n,
               _p(state, torch.bfloat16), _p(norm, torch.bfloat16), float(epsilon), _p(su, torch.float32),
               _p(u, torch.bfloat16), n if ldu is None else ldu, _p(xn, torch.bfloat16), _stream())


def qtip_multiply_batch(w, x, z, stride, splits, tokens, implementation=-1):
    init()
    lib().call("qtip_multiply_batch", w.pod, _p(x, torch.bfloat16), _p(z, torch.float32), stride, splits, tokens,
               _stream(), implementation)


def qtip_multiply_tc(w, x, z, stride, splits, tokens, status=None):
    """Decode fused into the tcgen05 product (17 .. a few hundred tokens); z [splits, tokens, stride] fp32."""
    init()
    lib().call("qtip_multiply_tc", w.pod, _p(x, torch.bfloat16), _p(z, torch.float32), stride, splits, tokens,
               _p(status, torch.int32), _stream())


def tc_splits(n_out, sm_count=148, max_splits=4):
    """K-splits for qtip_multiply_tc that waste the fewest SM rounds: the kernel runs out / 128 x splits CTAs of
    1 / splits of the K range each, one per SM at a time."""
    tiles = max(1, n_out // 128)
    return min(range(1, max_splits + 1), key=lambda sp: (-(-tiles * sp // sm_count) / sp, sp))


def batch_uses_tc(n_in, n_out, tokens):
    """The rule by which qtip_multiply_batch (implementation = -1) takes the fused tensor-core kernel."""
    return n_in % 64 == 0 and n_out % 128 == 0 and (tokens > 16 or (tokens > 8 and n_out <= 16384))


def kernel_status():
    """Synchronises; raises QtipError if a tensor-core kernel without a status word reported a time-out."""
    lib().call("qtip_kernel_status", _stream())


def qtip_decode_matrix(w, out):
    init()
    lib().call("qtip_decode_matrix", w.pod, _p(out, torch.bfloat16), _stream())


def reduce_products(x, elements, splits):
    init()
    lib().call("qtip_reduce_products", _p(x, torch.float32), elements, splits, _stream())


def reduce_to_b16(x, scale, y, elements, width, splits):
    init()
    lib().call("qtip_reduce_to_b16", _p(x, torch.float32), _p(scale, torch.float32), _p(y, torch.bfloat16), elements,
               width, splits, _stream())


def fp8_forward(w, scale, x, y, n_in, n_out, tokens=1):
    """FP8 e4m3 K/V projection: w uint8 [out, in], scale f32 [out], x bf16 [tokens, in] -> y bf16 [tokens, out]."""
    init()
    lib().call("qtip_fp8_forward", _p(w, torch.uint8), _p(scale, torch.float32), _p(x, torch.bfloat16),
               _p(y, torch.bfloat16), n_in, n_out, tokens, _stream())


def prefill_gemm(w_dense, x, z, stride, n_in, n_out, tokens, status=None):
    """z [tokens, stride] f32 = x [tokens, in] . w_dense [out, in]^T on the tcgen05 tensor cores."""
    init()
    lib().call("qtip_prefill_gemm", _p(w_dense, torch.bfloat16), _p(x, torch.bfloat16), _p(z, torch.float32), stride,
               n_in, n_out, tokens, _p(status, torch.int32), _stream())


def qtip_multiply_prefill(w, x, z, stride, tokens, dense_scratch, status=None):
    """The >= 128-token regime of the reference (Rank::multiply, runtime/cuda/tensor_model.cpp:210-222): dense bf16
    decode of the shard into `dense_scratch` [out, in], then the tensor-core product."""
    qtip_decode_matrix(w, dense_scratch)
    prefill_gemm(dense_scratch, x, z, stride, w.n_in, w.n_out, tokens, status)


def prefill_gemm_splitk(w_dense, x, z, stride, n_in, n_out, tokens, splits, status=None):
    """prefill_gemm with the K range split over the grid: z [splits, tokens, stride] f32 partial sums."""
    init()
    lib().call("qtip_prefill_gemm_splitk", _p(w_dense, torch.bfloat16), _p(x, torch.bfloat16), _p(z, torch.float32),
               stride, n_in, n_out, tokens, splits, _p(status, torch.int32), _stream())


def fp8_splits(n_in, n_out, tokens, sm_count=148):
    """K-splits that give the tensor-core product of a few-row weight about one CTA per SM."""
    tiles = -(-n_out // 256) * -(-tokens // 256)
    return max(1, min(n_in // 64 // 4, sm_count // tiles))


def fp8_forward_prefill(w, scale, x, y, n_in, n_out, tokens, dense_scratch, z, splits=None):
    """FP8 K/V projection for batches of tokens on the tensor cores: exact bf16 copy of the weights, tcgen05 product with
    the K range split over the SMs into z [splits, tokens, out] f32, then the sum of the partials, the per-row scale and
    the bf16 rounding (the reference's decode_fp8_matrix path)."""
    init()
    if splits is None:
        splits = fp8_splits(n_in, n_out, tokens)
    lib().call("qtip_decode_fp8_matrix", _p(w, torch.uint8), _p(dense_scratch, torch.bfloat16), n_in * n_out, _stream())
    prefill_gemm_splitk(dense_scratch, x, z, n_out, n_in, n_out, tokens, splits)
    reduce_to_b16(z, scale, y, tokens * n_out, n_out, splits)
