"""This repository's kernels against the reference's own CUDA kernels (src/viterbi.hip with QTIP_CUDA,
runtime/cuda/kernels.cu, runtime/cuda/batch_kernels.cu, compiled in place for sm_100a), both run on the same GPU on the
same seeded inputs. Encode side: bit-exact. Runtime side: the fp32 products differ only by summation order."""
import numpy as np
import pytest
import torch

from test_decode_gpu import bf16_dev, make_linear, rel_l2
from test_viterbi_gpu import dev, gpu_lut, u16

pytestmark = pytest.mark.gpu


def p(t):
    return None if t is None else t.data_ptr()


def reference_quantize(refgpu, Xd, lut_d, batch=1024):
    """fwd (rolled) -> overlap -> fwd (constrained) -> finish with the reference's kernels, `batch` sequences at a time
    (its back-pointer table is 260 KB per sequence). src/quantizer.cpp:54-62."""
    B = Xd.shape[0]
    Q = torch.zeros((B, 128), dtype=torch.int16, device="cuda")
    hatWT = torch.zeros((16, 16 * B), dtype=torch.float32, device="cuda")  # one 16-column block, m = 16 B
    A = torch.empty((batch, 127, 1024), dtype=torch.int16, device="cuda")
    fs = torch.empty(batch, dtype=torch.int16, device="cuda")
    ov = torch.empty(batch, dtype=torch.int32, device="cuda")
    for b0 in range(0, B, batch):
        nb = min(batch, B - b0)
        x = Xd[b0:b0 + nb]
        refgpu.viterbi_fwd(p(x), None, 1, nb, p(A), p(fs), p(lut_d))
        refgpu.viterbi_overlap(p(A), p(fs), nb, p(ov))
        refgpu.viterbi_fwd(p(x), p(ov), 0, nb, p(A), p(fs), p(lut_d))
        refgpu.viterbi_finish(p(A), p(fs), nb, b0, p(Q), 1, 0, p(hatWT), 16 * B, 0, p(lut_d))
    torch.cuda.synchronize()
    return Q, hatWT


def test_viterbi_codes_identical_to_reference_kernels(gpu, refgpu):
    """10,240 random tiles at three scales, seeded codebook: identical states and identical decoded values."""
    B = 10240
    rng = np.random.default_rng(2024)
    X = rng.standard_normal((B, 256)).astype(np.float32)
    X *= np.repeat(np.array([0.6, 1.0, 1.6, 1.0], np.float32), B // 4)[:, None]
    tl = gpu.synth.seeded_tlut(1).view(np.uint16)
    lut_d, _ = gpu_lut(gpu, tl)
    Xd = dev(X)
    states, hat = gpu.codec.quantize_tiles(Xd, lut_d)
    Qr, hatWT = reference_quantize(refgpu, Xd, lut_d)
    assert torch.equal(states, Qr)
    # the reference scatters decoded values to hatWT[c][16 b + r]; bring ours to the same layout
    perm = torch.from_numpy(gpu.synth.tile_perm().astype(np.int64)).cuda()  # sequence position -> 16 r + c
    tiles = torch.empty_like(hat)
    tiles[:, perm] = hat
    ours = tiles.view(B, 16, 16).permute(2, 0, 1).reshape(16, 16 * B)
    assert torch.equal(ours, hatWT)


def test_back_pointers_identical_to_reference_kernel(gpu, refgpu, hyb):
    """Kernel-level entry point (the reference's buffer layout): every back-pointer and final state of both passes."""
    tl, _, _ = hyb
    lut_d, _ = gpu_lut(gpu, tl)
    B = 96
    X = (np.random.default_rng(77).standard_normal((B, 256)) * 0.9).astype(np.float32)
    Xd = dev(X)
    c = gpu.codec
    A, Ar = (torch.empty((B, 127, 1024), dtype=torch.int16, device="cuda") for _ in range(2))
    fs, fsr = (torch.empty(B, dtype=torch.int16, device="cuda") for _ in range(2))
    ov, ovr = (torch.empty(B, dtype=torch.int32, device="cuda") for _ in range(2))
    c.k_viterbi_fwd(Xd, None, 1, B, A, fs, lut_d)
    refgpu.viterbi_fwd(p(Xd), None, 1, B, p(Ar), p(fsr), p(lut_d))
    assert torch.equal(A, Ar) and torch.equal(fs, fsr)
    c.k_viterbi_overlap(A, fs, B, ov)
    refgpu.viterbi_overlap(p(Ar), p(fsr), B, p(ovr))
    assert torch.equal(ov, ovr)
    c.k_viterbi_fwd(Xd, ov, 0, B, A, fs, lut_d)
    refgpu.viterbi_fwd(p(Xd), p(ovr), 0, B, p(Ar), p(fsr), p(lut_d))
    assert torch.equal(A, Ar) and torch.equal(fs, fsr)
    hs, hr = (torch.empty((B, 256), dtype=torch.float32, device="cuda") for _ in range(2))
    Q = torch.zeros((B, 128), dtype=torch.int16, device="cuda")
    c.k_viterbi_finish(A, fs, B, 0, Q, 1, 0, None, 0, 0, lut_d)
    c.k_decode_states(Q, B, hs, lut_d)
    refgpu.decode_states(p(Q), B, p(hr), p(lut_d))
    assert torch.equal(hs, hr)


def test_ldlq_prep_identical_to_reference_kernel(gpu, refgpu):
    n, m = 256, 528
    rng = np.random.default_rng(5)
    WT = dev(rng.standard_normal((n, m)).astype(np.float32))
    hatWT = dev(rng.standard_normal((n, m)).astype(np.float32))
    prod = dev((rng.standard_normal((n, m)) * 0.1).astype(np.float32))
    L = dev((np.tril(rng.standard_normal((n, n)), -1) * 0.05).astype(np.float32))
    for col0, bufend in ((240, 256), (128, 256), (176, 256), (0, 128)):
        X, Xr = (torch.zeros((m // 16, 256), dtype=torch.float32, device="cuda") for _ in range(2))
        gpu.codec.k_ldlq_prep(WT, hatWT, prod, L, n, m, col0, bufend, X)
        refgpu.ldlq_prep(p(WT), p(hatWT), p(prod), p(L), n, m, col0, bufend, p(Xr))
        torch.cuda.synchronize()
        assert torch.equal(X, Xr)


def ref_matrix(w):
    return (p(w.trellis), p(w.su), p(w.sv), p(w.lut), w.n_in, w.n_out)


def test_decode_matrix_identical_to_reference_kernel(gpu, refgpu):
    n_in, n_out = 1536, 640
    w, *_ = make_linear(gpu, n_in, n_out, 91)
    ours, ref = (torch.empty((n_out, n_in), dtype=torch.bfloat16, device="cuda") for _ in range(2))
    gpu.linear.qtip_decode_matrix(w, ours)
    refgpu.qtip_decode_matrix(ref_matrix(w), p(ref))
    torch.cuda.synchronize()
    assert torch.equal(ours.view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("n_in,n_out,splits", [(1536, 1024, 1), (12288, 3584, 1), (3584, 1536, 4), (12288, 7168, 2)])
def test_operator_against_reference_operator(gpu, refgpu, n_in, n_out, splits):
    """prepare / multiply / finish, stage by stage. Rotated activations (bf16): at most one value in a thousand differs,
    by one bf16 ulp (the transforms add in different orders). Products z on the SAME rotated input: rel-L2 <= 1e-5.
    Outputs y (bf16) of the whole operator: rel-L2 <= 5e-3."""
    w, *_ = make_linear(gpu, n_in, n_out, 70 + splits, sv_scale=0.01)
    xb = gpu.synth.f32_to_bf16_bits((np.random.default_rng(3).standard_normal(n_in) * 0.2).astype(np.float32))
    x = bf16_dev(xb)
    scratch, scratch_r = (torch.empty(max(n_in, n_out), dtype=torch.float32, device="cuda") for _ in range(2))
    rot, rot_r = (torch.empty(n_in, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    gpu.linear.qtip_prepare(w, x, scratch, rot)
    refgpu.qtip_prepare(ref_matrix(w), p(x), p(scratch_r), p(rot_r))
    torch.cuda.synchronize()
    assert rel_l2(rot.float().cpu().numpy(), rot_r.float().cpu().numpy().astype(np.float64)) < 2e-3
    z, z_r = (torch.zeros((splits, n_out), dtype=torch.float32, device="cuda") for _ in range(2))
    gpu.linear.qtip_multiply(w, rot_r, z, n_out, splits)
    refgpu.qtip_multiply(ref_matrix(w), p(rot_r), p(z_r), n_out, splits)
    torch.cuda.synchronize()
    assert rel_l2(z.sum(0).cpu().numpy(), z_r.sum(0).cpu().numpy().astype(np.float64)) < 1e-5
    for round_z in (False, True):
        y, y_r = (torch.empty(n_out, dtype=torch.bfloat16, device="cuda") for _ in range(2))
        gpu.linear.qtip_finish(w, z_r, y, scratch, round_z, splits)
        refgpu.qtip_finish(ref_matrix(w), p(z_r), p(y_r), p(scratch_r), round_z, splits)
        torch.cuda.synchronize()
        assert rel_l2(y.float().cpu().numpy(), y_r.float().cpu().numpy().astype(np.float64)) < 5e-3


@pytest.mark.parametrize("tokens", [3, 8, 16, 40])
def test_multiply_batch_against_reference_kernels(gpu, refgpu, tokens):
    n_in, n_out, splits = 2048, 768, 2
    w, *_ = make_linear(gpu, n_in, n_out, 80)
    xb = gpu.synth.f32_to_bf16_bits(np.random.default_rng(tokens).standard_normal((tokens, n_in)).astype(np.float32))
    x = bf16_dev(xb)
    z, z_r = (torch.zeros((splits, tokens, n_out), dtype=torch.float32, device="cuda") for _ in range(2))
    gpu.linear.qtip_multiply_batch(w, x, z, n_out, splits, tokens)
    refgpu.qtip_multiply_batch(ref_matrix(w), p(x), p(z_r), n_out, splits, tokens)
    torch.cuda.synchronize()
    assert rel_l2(z.sum(0).cpu().numpy(), z_r.sum(0).cpu().numpy().astype(np.float64)) < 1e-5


def test_fp8_forward_against_reference_kernel(gpu, refgpu):
    n_in, n_out = 12288, 1024
    rng = np.random.default_rng(8)
    wq = rng.integers(0, 256, (n_out, n_in), dtype=np.uint8)
    wq[(wq & 0x7F) == 0x7F] = 0x3C  # no NaN codes
    scale = (rng.random(n_out) * 0.01 + 0.001).astype(np.float32)
    x = bf16_dev(gpu.synth.f32_to_bf16_bits(rng.standard_normal(n_in).astype(np.float32)))
    wd, sd = torch.from_numpy(wq).cuda(), dev(scale)
    y, y_r = (torch.empty(n_out, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    gpu.linear.fp8_forward(wd, sd, x, y, n_in, n_out)
    refgpu.fp8_forward(p(wd), p(sd), p(x), p(y_r), n_in, n_out)
    torch.cuda.synchronize()
    assert rel_l2(y.float().cpu().numpy(), y_r.float().cpu().numpy().astype(np.float64)) < 4e-3
