"""The trellis-decode linear operator against the oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import golden
from test_viterbi_gpu import dev, u16

pytestmark = pytest.mark.gpu


def make_linear(gpu, n_in, n_out, seed, tl=None, sv_scale=1.0):
    s = gpu.synth
    tl = s.seeded_tlut(1).view(np.uint16) if tl is None else tl
    tr = s.random_trellis(n_out, n_in, seed)
    su, sv = s.signs(n_in, seed + 1), s.signs(n_out, seed + 2) * np.float32(sv_scale)
    w = gpu.linear.Matrix(dev(tr), dev(su), dev(sv), gpu.linear.runtime_lut(tl), n_in, n_out)
    return w, tr, su, sv, tl


def bf16_dev(x):
    bits = np.ascontiguousarray(x)
    return torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / np.linalg.norm(b))


def test_runtime_lut_matches_reference_vectors(gpu, hyb):
    tl, _, _ = hyb
    g = golden("decode_ref.npz")
    assert np.array_equal(gpu.linear.runtime_lut(tl).cpu().numpy().view(np.uint32), g["bf16x2"])
    bad = tl.copy()
    bad[5, 1] = 0x7C00  # +inf
    with pytest.raises(gpu.QtipError):
        gpu.linear.runtime_lut(bad)


def test_decode_matrix_bit_exact(gpu, oracle, hyb):
    tl, _, _ = hyb
    g = golden("decode_ref.npz")
    n_in, n_out = int(g["n_in"]), int(g["n_out"])
    w = gpu.linear.Matrix(dev(g["trellis"]), dev(g["su"]), dev(g["sv"]), gpu.linear.runtime_lut(tl), n_in, n_out)
    out = torch.empty((n_out, n_in), dtype=torch.bfloat16, device="cuda")
    gpu.linear.qtip_decode_matrix(w, out)
    dense = out.float().cpu().numpy()
    assert np.array_equal(dense[32:96], g["rows_bf16"])  # the reference's decode_rows_bf16
    assert np.array_equal(dense, oracle.decode_rows(g["trellis"], n_in, n_out, tl, 0, n_out, True))
    # a wider matrix: more than one 256-column strip, and a ragged last strip
    w2, tr2, _, _, tl2 = make_linear(gpu, 1024 + 96, 64, 31)
    out2 = torch.empty((64, 1120), dtype=torch.bfloat16, device="cuda")
    gpu.linear.qtip_decode_matrix(w2, out2)
    assert np.array_equal(out2.float().cpu().numpy(), oracle.decode_rows(tr2, 1120, 64, tl2, 0, 64, True))


@pytest.mark.parametrize("n_in,n_out,splits", [(384, 256, 1), (384, 256, 3), (1024, 128, 4), (12288, 64, 1),
                                               (3584, 96, 2), (1024, 57344 // 16, 1)])
def test_multiply_against_decoded_weights(gpu, oracle, n_in, n_out, splits):
    """z = What . u with What the bit-exact decoded bf16 weights and u a bf16 vector: fp32 tensor-core accumulation vs
    float64, rel-L2 <= 1e-5 (only the summation order differs)."""
    w, tr, su, sv, tl = make_linear(gpu, n_in, n_out, 40 + splits)
    u_bits = gpu.synth.f32_to_bf16_bits(np.random.default_rng(6).standard_normal(n_in).astype(np.float32))
    z = torch.zeros((splits, n_out), dtype=torch.float32, device="cuda")
    gpu.linear.qtip_multiply(w, bf16_dev(u_bits), z, n_out, splits, 1)
    W = oracle.decode_rows(tr, n_in, n_out, tl, 0, n_out, True).astype(np.float64)
    ref = W @ gpu.synth.bf16_bits_to_f32(u_bits).astype(np.float64)
    assert rel_l2(z.sum(0).cpu().numpy(), ref) < 1e-5
    z2 = torch.zeros_like(z)
    gpu.linear.qtip_multiply(w, bf16_dev(u_bits), z2, n_out, splits, 1)
    assert torch.equal(z, z2)  # deterministic reduction order


@pytest.mark.parametrize("n_in,n_out", [(384, 256), (1024, 384), (12288, 1024), (3584, 12288 // 8)])
def test_forward_against_reference_linear(gpu, oracle, n_in, n_out):
    """prepare + multiply + finish vs reference_forward(device_rounding = true). bf16 outputs against the bf16-rounded
    reference: rel-L2 < 4e-3 (one bf16 rounding; 1e-2 when z is rounded to bf16 first); the fp32 products z against the
    oracle's z: rel-L2 <= 1e-3."""
    w, tr, su, sv, tl = make_linear(gpu, n_in, n_out, 50, sv_scale=0.003)
    x = (np.random.default_rng(9).standard_normal(n_in) * 0.1).astype(np.float32)
    xb = gpu.synth.f32_to_bf16_bits(x)
    y = torch.empty(n_out, dtype=torch.bfloat16, device="cuda")
    rot = torch.empty(n_in, dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(max(n_in, n_out), dtype=torch.float32, device="cuda")
    for splits, round_z in ((1, False), (4, False), (2, True)):
        z = torch.zeros((splits, n_out), dtype=torch.float32, device="cuda")
        gpu.linear.qtip_forward(w, bf16_dev(xb), y, scratch, rot, z, round_z, splits)
        yo, zo = oracle.reference_forward(tr, su, sv, tl, n_in, n_out, gpu.synth.bf16_bits_to_f32(xb), True, round_z,
                                          want_z=True)
        zz = z.sum(0).cpu().numpy()
        if not round_z:
            assert rel_l2(zz, zo[0]) < 1e-3
        yo_b = gpu.synth.bf16_bits_to_f32(gpu.synth.f32_to_bf16_bits(yo[0]))
        # one bf16 rounding of the output (2^-8); with round_z the bf16 rounding of z can also flip where the fp32 and
        # the double sums straddle a rounding boundary
        assert rel_l2(y.float().cpu().numpy(), yo_b) < (1e-2 if round_z else 4e-3)
        assert np.abs(y.float().cpu().numpy() - yo_b).max() < 0.03 * np.abs(yo_b).max()


def test_forward_against_reference_vectors(gpu, hyb):
    """The committed outputs of the reference's reference_forward (in = 384, out = 256, three tokens)."""
    tl, _, _ = hyb
    g = golden("decode_ref.npz")
    n_in, n_out = int(g["n_in"]), int(g["n_out"])
    w = gpu.linear.Matrix(dev(g["trellis"]), dev(g["su"]), dev(g["sv"]), gpu.linear.runtime_lut(tl), n_in, n_out)
    xb = gpu.synth.f32_to_bf16_bits(g["x"])
    tokens = xb.shape[0]
    rot = torch.empty((tokens, n_in), dtype=torch.bfloat16, device="cuda")
    z = torch.zeros((2, tokens, n_out), dtype=torch.float32, device="cuda")
    y = torch.empty((tokens, n_out), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(tokens * n_in, dtype=torch.float32, device="cuda")
    gpu.linear.qtip_prepare(w, bf16_dev(xb), scratch, rot, tokens)
    gpu.linear.qtip_multiply_batch(w, rot, z, n_out, 2, tokens)
    gpu.linear.qtip_finish(w, z, y, scratch, False, 2, tokens)
    # the fixture used fp32 x; the operator takes bf16 x: compare with tolerance of the input rounding (2^-9 relative)
    assert rel_l2(y.float().cpu().numpy(), g["y_10"]) < 2e-2


@pytest.mark.parametrize("tokens", [2, 8, 13, 16, 40])
def test_multiply_batch(gpu, oracle, tokens):
    n_in, n_out = 1024, 256
    w, tr, su, sv, tl = make_linear(gpu, n_in, n_out, 60)
    xb = gpu.synth.f32_to_bf16_bits(np.random.default_rng(tokens).standard_normal((tokens, n_in)).astype(np.float32))
    z = torch.zeros((3, tokens, n_out), dtype=torch.float32, device="cuda")
    gpu.linear.qtip_multiply_batch(w, bf16_dev(xb), z, n_out, 3, tokens)
    W = oracle.decode_rows(tr, n_in, n_out, tl, 0, n_out, True).astype(np.float64)
    ref = gpu.synth.bf16_bits_to_f32(xb).astype(np.float64) @ W.T
    assert rel_l2(z.sum(0).cpu().numpy(), ref) < 1e-5
    zr = z.clone()
    gpu.linear.reduce_products(zr, tokens * n_out, 3)
    assert torch.equal(zr[0], (z[0] + z[1]) + z[2])
    yb = torch.empty((tokens, n_out), dtype=torch.bfloat16, device="cuda")
    gpu.linear.reduce_to_b16(z, None, yb, tokens * n_out, n_out, 3)
    assert np.array_equal(u16(yb.view(torch.int16)), gpu.synth.f32_to_bf16_bits(zr[0].cpu().numpy()))


def test_row_sharded_multiply_equals_full(gpu):
    """Rotated-row tensor parallelism: contiguous block-row shards of the trellis give the same z slices."""
    n_in, n_out = 1024, 512
    w, *_ = make_linear(gpu, n_in, n_out, 70)
    ub = gpu.synth.f32_to_bf16_bits(np.random.default_rng(1).standard_normal(n_in).astype(np.float32))
    z = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    gpu.linear.qtip_multiply(w, bf16_dev(ub), z, n_out, 1, 1)
    for world in (2, 4):
        parts = []
        for r in range(world):
            row0, rows = gpu.sharding.block_row_range(n_out, r, world)
            zr = torch.zeros(rows, dtype=torch.float32, device="cuda")
            gpu.linear.qtip_multiply(w.rows(row0, rows), bf16_dev(ub), zr, rows, 1, 1)
            parts.append(zr)
        assert torch.equal(torch.cat(parts), z)


def test_geometry_errors(gpu):
    w, *_ = make_linear(gpu, 384, 256, 80)
    z = torch.zeros(256, dtype=torch.float32, device="cuda")
    u = torch.zeros(384, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(gpu.QtipError) as e:
        gpu.linear.qtip_multiply(w, u, z, 128, 1, 1)  # stride < out
    assert e.value.code == -2
    with pytest.raises(gpu.QtipError):
        gpu.linear.qtip_multiply(w, u, z, 256, 33, 1)  # more than 32 splits


@pytest.mark.parametrize("tokens", [1, 5, 19])
def test_fp8_kv_projection(gpu, oracle, tokens):
    """Random e4m3 bytes (NaN codes remapped to 0) with the reference test's per-row scales, against the oracle's
    restatement of the FP8 branch of reference_forward, rounded to bf16. Tolerance: one bf16 ulp."""
    rng = np.random.default_rng(11)
    n_in, n_out = 1536, 200
    w = rng.integers(0, 256, (n_out, n_in), dtype=np.uint8)
    w[(w & 127) == 127] = 0
    scale = ((1 + np.arange(n_out) % 7) / 4096.0).astype(np.float32)
    xb = gpu.synth.f32_to_bf16_bits(rng.standard_normal((tokens, n_in)).astype(np.float32))
    y = torch.empty((tokens, n_out), dtype=torch.bfloat16, device="cuda")
    gpu.linear.fp8_forward(torch.from_numpy(w).cuda(), dev(scale), bf16_dev(xb), y, n_in, n_out, tokens)
    ref = oracle.fp8_forward(w, scale, gpu.synth.bf16_bits_to_f32(xb), True)
    ref_b = gpu.synth.bf16_bits_to_f32(gpu.synth.f32_to_bf16_bits(ref))
    got = y.float().cpu().numpy()
    assert np.abs(got - ref_b).max() <= 2.0 ** -7 * np.abs(ref_b).max()
    assert rel_l2(got, ref_b) < 4e-3
    if tokens == 19 and n_out % 128 != 0:  # tensor-core variant needs out % 128 == 0: take the first 128 rows
        wd = torch.from_numpy(np.ascontiguousarray(w[:128])).cuda()
        dense = torch.empty((128, n_in), dtype=torch.bfloat16, device="cuda")
        y2 = torch.empty((tokens, 128), dtype=torch.bfloat16, device="cuda")
        for splits in (1, 5, None):  # None: the K range spread over the SMs (here 6 K-splits of 4 steps)
            sp = splits or gpu.linear.fp8_splits(n_in, 128, tokens)
            z = torch.full((sp, tokens, 128), float("nan"), dtype=torch.float32, device="cuda")
            y2.zero_()
            gpu.linear.fp8_forward_prefill(wd, dev(scale[:128]), bf16_dev(xb), y2, n_in, 128, tokens, dense, z, splits)
            assert rel_l2(y2.float().cpu().numpy(), ref_b[:, :128]) < 4e-3


@pytest.mark.parametrize("n_in,n_out,tokens", [(512, 256, 300), (1024, 128, 256), (12288, 384, 17), (1024, 1536, 520),
                                               (512, 4096, 2560), (1024, 4096, 2560)])
def test_prefill_gemm_tensor_cores(gpu, n_in, n_out, tokens):
    """tcgen05 product against float64 on the same bf16 operands: fp32 accumulation, rel-L2 <= 5e-5 (K up to 12,288
    terms per output); ragged token counts (rows past the end are not written). The shapes cover the tile-per-CTA launch
    (1 and 2 tiles), the persistent launch with tiles split 8 ways (2 tiles, one of them half a tile high) and 2 ways
    (18 tiles), with whole-tile rounds only (160 tiles, 8 K steps) and with whole-tile rounds plus 12 split tiles."""
    rng = np.random.default_rng(n_in + tokens)
    wb = gpu.synth.f32_to_bf16_bits(rng.standard_normal((n_out, n_in)).astype(np.float32))
    xb = gpu.synth.f32_to_bf16_bits(rng.standard_normal((tokens, n_in)).astype(np.float32))
    z = torch.full((tokens + 3, n_out), 7.0, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gpu.linear.prefill_gemm(bf16_dev(wb), bf16_dev(xb), z, n_out, n_in, n_out, tokens, status)
    torch.cuda.synchronize()
    assert int(status) == 0
    ref = gpu.synth.bf16_bits_to_f32(xb).astype(np.float64) @ gpu.synth.bf16_bits_to_f32(wb).astype(np.float64).T
    assert rel_l2(z[:tokens].cpu().numpy(), ref) < 5e-5
    assert bool((z[tokens:] == 7.0).all())


def test_prefill_gemm_split_tiles_are_reproducible(gpu):
    """A product whose tiles are split over several CTAs and summed in the output: 40 launches give the same bits (the
    order of the additions is fixed) and the library's ring of state blocks wraps around without being cleared."""
    n_in, n_out, tokens = 1024, 1536, 520
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    w = torch.randn(n_out, n_in, generator=g, device="cuda").to(torch.bfloat16)
    x = torch.randn(tokens, n_in, generator=g, device="cuda").to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    first = None
    for _ in range(40):
        z = torch.full((tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
        gpu.linear.prefill_gemm(w, x, z, n_out, n_in, n_out, tokens, status)
        if first is None:
            first = z
            ref = x.double() @ w.double().T
            assert float((z.double() - ref).norm() / ref.norm()) < 5e-5
        else:
            assert torch.equal(z, first)
    assert int(status) == 0


def test_prefill_gemm_replays_from_a_cuda_graph(gpu):
    """The persistent launch (cooperative, with its counters inside the library) captured once and replayed: every replay
    gives the bits of the eager call (the counters are versioned by an epoch the kernel itself advances)."""
    n_in, n_out, tokens = 1024, 1536, 520
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    w = torch.randn(n_out, n_in, generator=g, device="cuda").to(torch.bfloat16)
    x = torch.randn(tokens, n_in, generator=g, device="cuda").to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    eager = torch.zeros((tokens, n_out), dtype=torch.float32, device="cuda")
    gpu.linear.prefill_gemm(w, x, eager, n_out, n_in, n_out, tokens, status)
    z = torch.zeros((tokens, n_out), dtype=torch.float32, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            gpu.linear.prefill_gemm(w, x, z, n_out, n_in, n_out, tokens, status)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        z.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(z, eager)
    assert int(status) == 0


def test_multiply_prefill_matches_batch_path(gpu, oracle):
    n_in, n_out, tokens = 1024, 256, 200
    w, tr, su, sv, tl = make_linear(gpu, n_in, n_out, 90)
    xb = gpu.synth.f32_to_bf16_bits(np.random.default_rng(2).standard_normal((tokens, n_in)).astype(np.float32))
    dense = torch.empty((n_out, n_in), dtype=torch.bfloat16, device="cuda")
    z = torch.zeros((tokens, n_out), dtype=torch.float32, device="cuda")
    gpu.linear.qtip_multiply_prefill(w, bf16_dev(xb), z, n_out, tokens, dense)
    W = oracle.decode_rows(tr, n_in, n_out, tl, 0, n_out, True).astype(np.float64)
    ref = gpu.synth.bf16_bits_to_f32(xb).astype(np.float64) @ W.T
    assert rel_l2(z.cpu().numpy(), ref) < 1e-5


@pytest.mark.parametrize("n_in,n_out,tokens,splits", [(1024, 256, 17, 1), (1024, 256, 64, 2), (1024, 384, 100, 1),
                                                      (3584, 128, 128, 3), (2048, 256, 200, 1), (1024, 256, 256, 1),
                                                      (1024, 256, 300, 2), (12288, 512, 40, 1), (64, 128, 33, 4)])
def test_fused_decode_tensor_core_product(gpu, oracle, n_in, n_out, tokens, splits):
    """Decode fused into the tcgen05 product against float64 on the bit-exact decoded weights: only the fp32 summation
    order differs, rel-L2 <= 5e-5 (K up to 12,288). Token tiles of 64 / 128 / 256 incl. ragged ends, K-splits incl.
    more splits than K steps, and the deterministic repeat."""
    w, tr, su, sv, tl = make_linear(gpu, n_in, n_out, 700 + tokens)
    xb = gpu.synth.f32_to_bf16_bits(np.random.default_rng(tokens).standard_normal((tokens, n_in)).astype(np.float32))
    z = torch.full((splits, tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gpu.linear.qtip_multiply_tc(w, bf16_dev(xb), z, n_out, splits, tokens, status)
    assert int(status) == 0
    W = oracle.decode_rows(tr, n_in, n_out, tl, 0, n_out, True).astype(np.float64)
    ref = gpu.synth.bf16_bits_to_f32(xb).astype(np.float64) @ W.T
    got = z.sum(0).cpu().numpy()
    assert np.isfinite(got).all()
    assert rel_l2(got, ref) < 5e-5
    z2 = torch.zeros_like(z)
    if splits <= n_in // 32:  # the batch entry point keeps the reference's bound on K-splits
        gpu.linear.qtip_multiply_batch(w, bf16_dev(xb), z2, n_out, splits, tokens, 2)
        gpu.linear.kernel_status()
    else:
        gpu.linear.qtip_multiply_tc(w, bf16_dev(xb), z2, n_out, splits, tokens, status)
    assert torch.equal(z, z2)
