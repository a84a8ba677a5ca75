"""Parity at the full sizes of the benchmark configurations (the other test files use sizes the CPU oracle finishes in
seconds): every tile of the 12288 x 12288 encode against the reference's own CUDA kernel, the batch-1 operator on the
57344 x 12288 matrix against the reference's CPU operator, and the products of the layer's q / gate / down linears at
16, 64, 256 and 2,048 tokens against the reference's kernels (or, where the reference itself calls a library GEMM, against
its dense decode followed by an fp32 matrix product)."""
import numpy as np
import pytest
import torch

from test_decode_gpu import bf16_dev, rel_l2
from test_reference_gpu import p, ref_matrix, reference_quantize
from test_viterbi_gpu import dev

pytestmark = pytest.mark.gpu


def device_linear(gpu, n_in, n_out, seed):
    """Random codes made on the device (as the benchmark does), seeded codebook, seeded +-1 sign vectors."""
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    tr = torch.randint(-32768, 32768, ((n_out // 16) * (n_in // 16) * 32,), generator=g, device="cuda", dtype=torch.int16)
    su, sv = dev(gpu.synth.signs(n_in, 7)), dev(gpu.synth.signs(n_out, 8))
    tl = gpu.synth.seeded_tlut(1).view(np.uint16)
    return gpu.linear.Matrix(tr, su, sv, gpu.linear.runtime_lut(tl), n_in, n_out), tl


def test_config2_every_tile_identical_to_the_reference_kernel(gpu, refgpu):
    """All 589,824 tiles of the seeded 12288 x 12288 N(0,1) matrix: states identical to the reference's CUDA Viterbi
    (forward, overlap, forward, finish in batches of 1,024 sequences, as its quantizer runs them)."""
    m = n = 12288
    g = torch.Generator(device="cuda")
    g.manual_seed(2)
    W = torch.randn(m, n, generator=g, device="cuda", dtype=torch.float32)
    X = gpu.codec.tiles_from_matrix(W)
    del W
    lut_d, _ = gpu.codec.device_lut(gpu.synth.seeded_tlut(1))
    ws = gpu.codec.quantize_workspace(2 * 4608)
    states, _ = gpu.codec.quantize_tiles(X, lut_d, workspace=ws, want_hat=False)
    ws.check()
    tiles = X.shape[0]
    assert tiles == 589824
    step = 73728  # an eighth of the matrix per comparison keeps the reference's scratch small
    for t0 in range(0, tiles, step):
        Qr, _ = reference_quantize(refgpu, X[t0:t0 + step], lut_d)
        assert torch.equal(states[t0:t0 + step], Qr), "states differ in tiles [%d, %d)" % (t0, t0 + step)
        del Qr


def test_config4_operator_at_full_size(gpu, oracle):
    """57344 x 12288, one token. z within 1e-3 (relative L2) of the reference's CPU operator with device rounding
    (bf16 rotated input, bf16 table values, double accumulation); bf16 outputs within a bf16 rounding of its outputs;
    the dense decode of a 2,048-row band bit-identical to decode_rows_bf16."""
    n_in, n_out = 12288, 57344
    w, tl = device_linear(gpu, n_in, n_out, 9)
    tr = w.trellis.cpu().numpy().view(np.uint16)
    su, sv = w.su.cpu().numpy(), w.sv.cpu().numpy()
    xb = gpu.synth.f32_to_bf16_bits(np.random.default_rng(10).standard_normal(n_in).astype(np.float32))
    x = bf16_dev(xb)
    y = torch.empty(n_out, dtype=torch.bfloat16, device="cuda")
    rot = torch.empty(n_in, dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(n_out, dtype=torch.float32, device="cuda")
    for splits in (1, 3):
        z = torch.empty((splits, n_out), dtype=torch.float32, device="cuda")
        gpu.linear.qtip_forward(w, x, y, scratch, rot, z, False, splits)
        y_ref, z_ref = oracle.reference_forward(tr, su, sv, tl, n_in, n_out, gpu.synth.bf16_bits_to_f32(xb), True, False,
                                                want_z=True)
        assert rel_l2(z.sum(0).cpu().numpy(), z_ref[0].astype(np.float64)) < 1e-3  # the stated tolerance, fp32 products
        y_ref_b = gpu.synth.bf16_bits_to_f32(gpu.synth.f32_to_bf16_bits(y_ref[0].astype(np.float32)))
        assert rel_l2(y.float().cpu().numpy(), y_ref_b.astype(np.float64)) < 4e-3  # one bf16 rounding = 2^-8
    band0, band = 30720, 2048
    ws = w.rows(band0, band)
    out = torch.empty((band, n_in), dtype=torch.bfloat16, device="cuda")
    gpu.linear.qtip_decode_matrix(ws, out)
    assert np.array_equal(out.float().cpu().numpy(), oracle.decode_rows(tr, n_in, n_out, tl, band0, band, True))


@pytest.mark.parametrize("name,n_in,n_out", [("q", 12288, 12288), ("gate", 12288, 28672), ("down", 28672, 12288)])
def test_config5_linears_at_full_size(gpu, refgpu, name, n_in, n_out):
    """Products of one full-size linear at 16, 64, 256 and 2,048 tokens on the same rotated input. Up to 64 tokens the
    yard-stick is the reference's own batch kernel; above that the reference decodes to dense bf16 and calls a library
    GEMM (runtime/cuda/tensor_model.cpp:210-222), so the yard-stick is its dense decode followed by an fp32 product.
    Tolerances (relative L2): 2e-5 against the reference's kernel (fp32 summation order only); 5e-5 against the fp32
    library product and against fp64 on one token row (two fp32 sums over 12,288 .. 28,672 terms, the tensor cores'
    among them, each sit about 1e-5 from the exact value)."""
    w, _ = device_linear(gpu, n_in, n_out, {"q": 9, "gate": 11, "down": 13}[name])
    dense_ref = torch.empty((n_out, n_in), dtype=torch.bfloat16, device="cuda")
    refgpu.qtip_decode_matrix(ref_matrix(w), p(dense_ref))
    dense = torch.empty((n_out, n_in), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda")
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for tokens in (16, 64, 256, 2048):
            g.manual_seed(100 + tokens)
            x = torch.randn(tokens, n_in, generator=g, device="cuda").to(torch.bfloat16)
            if tokens <= 512:
                splits = gpu.linear.tc_splits(n_out) if gpu.linear.batch_uses_tc(n_in, n_out, tokens) else 2
                z = torch.zeros((splits, tokens, n_out), dtype=torch.float32, device="cuda")
                gpu.linear.qtip_multiply_batch(w, x, z, n_out, splits, tokens)
                ours = z.sum(0)
            else:
                ours = torch.zeros((tokens, n_out), dtype=torch.float32, device="cuda")
                gpu.linear.qtip_multiply_prefill(w, x, ours, n_out, tokens, dense, status)
                assert torch.equal(dense.view(torch.int16), dense_ref.view(torch.int16))
            if tokens <= 64:
                z_r = torch.zeros((2, tokens, n_out), dtype=torch.float32, device="cuda")
                refgpu.qtip_multiply_batch(ref_matrix(w), p(x), p(z_r), n_out, 2, tokens)
                torch.cuda.synchronize()
                ref = z_r.sum(0)
            else:
                ref = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
                xf = x.float()
                for r0 in range(0, n_out, 4096):  # fp32 product in row bands: the fp32 copy of the weights stays small
                    ref[:, r0:r0 + 4096] = xf @ dense_ref[r0:r0 + 4096].float().T
            torch.cuda.synchronize()
            err = float((ours - ref).double().norm() / ref.double().norm())
            assert err < (2e-5 if tokens <= 64 else 5e-5), "%s at %d tokens: rel-L2 %.3g" % (name, tokens, err)
            row = tokens - 1
            exact = torch.empty(n_out, dtype=torch.float64, device="cuda")
            xd = x[row].double()
            for r0 in range(0, n_out, 4096):
                exact[r0:r0 + 4096] = dense_ref[r0:r0 + 4096].double() @ xd
            err64 = float((ours[row].double() - exact).norm() / exact.norm())
            assert err64 < 5e-5, "%s at %d tokens, last row vs fp64: rel-L2 %.3g" % (name, tokens, err64)
            del x, ours, ref
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    assert int(status) == 0
    gpu.linear.kernel_status()
