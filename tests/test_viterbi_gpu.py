"""Parity of the CUDA Viterbi with the CPU oracle, through the C ABI. Bit-exact: states, back-pointers, decoded values."""
import numpy as np
import pytest
import torch

from conftest import golden

pytestmark = pytest.mark.gpu


def dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    return torch.from_numpy(a).cuda()


def u16(t):
    return t.cpu().numpy().view(np.uint16)


def gpu_lut(gpu, tl):
    lut_d, rms = gpu.codec.device_lut(tl)
    return lut_d, rms


def staged(gpu, X, lut_d):
    """The four kernel-level calls in the order of the reference's ldlq_gpu."""
    c = gpu.codec
    B = X.shape[0]
    Xd = dev(X)
    A = torch.empty((B, 127, 1024), dtype=torch.int16, device="cuda")
    fs = torch.empty(B, dtype=torch.int16, device="cuda")
    ov = torch.empty(B, dtype=torch.int32, device="cuda")
    Q = torch.zeros((B, 128), dtype=torch.int16, device="cuda")
    c.k_viterbi_fwd(Xd, None, 1, B, A, fs, lut_d)
    A1, fs1 = u16(A).copy(), u16(fs).copy()
    c.k_viterbi_overlap(A, fs, B, ov)
    c.k_viterbi_fwd(Xd, ov, 0, B, A, fs, lut_d)
    c.k_viterbi_finish(A, fs, B, 0, Q, 1, 0, None, 0, 0, lut_d)
    return A1, fs1, ov.cpu().numpy(), u16(A), u16(fs), u16(Q)


def test_encoder_table_matches_oracle(gpu, oracle, hyb):
    tl, lut, rms = hyb
    lut_d, rms_d = gpu_lut(gpu, tl)
    assert np.array_equal(lut_d.cpu().numpy().view(np.uint32), lut)
    assert rms_d == rms


def test_kernel_level_calls_bit_exact(gpu, oracle, hyb):
    tl, lut, _ = hyb
    X = golden("viterbi_ref.npz")["X"][:12]
    lut_d, _ = gpu_lut(gpu, tl)
    A1, fs1, ov, A2, fs2, Q = staged(gpu, X, lut_d)
    oA1, ofs1 = oracle.viterbi_fwd(X, None, 1, lut)
    assert np.array_equal(fs1, ofs1)
    assert np.array_equal(A1, oA1)  # every back-pointer of the rolled pass
    oov = oracle.viterbi_overlap(oA1, ofs1)
    assert np.array_equal(ov, oov)
    oA2, ofs2 = oracle.viterbi_fwd(X, oov, 0, lut)
    assert np.array_equal(fs2, ofs2) and np.array_equal(A2, oA2)
    assert np.array_equal(Q, oracle.viterbi_finish(oA2, ofs2, lut))


def test_fused_matches_reference_vectors(gpu, hyb):
    """Golden vectors made by the reference's fp64 Viterbi: identical states on fp16-representable inputs."""
    tl, lut, _ = hyb
    g = golden("viterbi_ref.npz")
    lut_d, _ = gpu_lut(gpu, tl)
    ws = gpu.codec.quantize_workspace(64)
    st, hat = gpu.codec.quantize_tiles(dev(g["X"]), lut_d, workspace=ws)
    ws.check()
    same = (u16(st) == g["states"]).all(axis=1)
    assert same.sum() >= len(same) - 3
    assert np.array_equal(hat.cpu().numpy()[same], g["hat"][same])


@pytest.mark.parametrize("B", [1, 7, 8, 9, 24, 131])
def test_fused_bit_exact_ragged_batches(gpu, oracle, B):
    """Seeded codebook, unrounded N(0,1) inputs, batch sizes around the 8-sequence cluster batch."""
    tl = gpu.synth.seeded_tlut(1).view(np.uint16)
    lut, _ = oracle.build_lut(tl)
    lut_d, _ = gpu_lut(gpu, tl)
    X = np.random.default_rng(100 + B).standard_normal((B, 256), dtype=np.float32)
    ws = gpu.codec.quantize_workspace(B)
    st, hat = gpu.codec.quantize_tiles(dev(X), lut_d, workspace=ws)
    ws.check()
    ost, ohat = oracle.quantize_tiles(X, lut)
    assert np.array_equal(u16(st), ost)
    assert np.array_equal(hat.cpu().numpy(), ohat)


def test_fused_equals_kernel_level_and_is_deterministic(gpu, hyb):
    tl, _, _ = hyb
    lut_d, _ = gpu_lut(gpu, tl)
    X = (np.random.default_rng(5).standard_normal((40, 256)) * 1.3).astype(np.float32)
    *_, Q = staged(gpu, X, lut_d)
    ws = gpu.codec.quantize_workspace(16)  # smaller than the batch: exercises the chunk loop
    st1, _ = gpu.codec.quantize_tiles(dev(X), lut_d, workspace=ws)
    st2, _ = gpu.codec.quantize_tiles(dev(X), lut_d, workspace=ws)
    ws.check()
    assert np.array_equal(u16(st1), Q) and np.array_equal(u16(st1), u16(st2))


def test_edge_inputs(gpu, oracle, hyb):
    """All-zero, constant out-of-range, alternating-sign and large-magnitude sequences; empty batch."""
    tl, lut, _ = hyb
    lut_d, _ = gpu_lut(gpu, tl)
    X = np.zeros((6, 256), np.float32)
    X[1] = 3.5
    X[2, ::2], X[2, 1::2] = 2.0, -2.0
    X[3] = np.random.default_rng(1).standard_normal(256) * 40.0
    X[4] = np.random.default_rng(2).standard_normal(256) * 1e-4
    X[5] = -0.0
    ws = gpu.codec.quantize_workspace(8)
    st, hat = gpu.codec.quantize_tiles(dev(X), lut_d, workspace=ws)
    ws.check()
    ost, ohat = oracle.quantize_tiles(X, lut)
    assert np.array_equal(u16(st), ost) and np.array_equal(hat.cpu().numpy(), ohat)
    empty = torch.empty((0, 256), dtype=torch.float32, device="cuda")
    st0, hat0 = gpu.codec.quantize_tiles(empty, lut_d, workspace=ws)
    assert st0.shape == (0, 128) and hat0.shape == (0, 256)
    small = gpu.codec.Workspace(1024)
    with pytest.raises(gpu.QtipError) as e:
        gpu.codec.quantize_tiles(dev(X), lut_d, workspace=small)
    assert e.value.code == -3


def test_config1_plumbing(gpu, oracle):
    """256 x 256 N(0,1) matrix from seed 0, seeded codebook from seed 1, identity Hessian: encode, pack, kernel layout
    and back, decode; codes bit-exact against the oracle and per-tile MSE equal to the CPU path's."""
    s = gpu.synth
    tl = s.seeded_tlut(1).view(np.uint16)
    lut, _ = oracle.build_lut(tl)
    lut_d, _ = gpu_lut(gpu, tl)
    W = s.gaussian_matrix(256, 256, 0)
    X = s.tile_sequences(W)
    ws = gpu.codec.quantize_workspace(256)
    st, hat = gpu.codec.quantize_tiles(dev(X), lut_d, workspace=ws)
    ws.check()
    ost, ohat = oracle.quantize_tiles(X, lut)
    assert np.array_equal(u16(st), ost)
    packed = gpu.codec.pack_trellis(st)
    assert np.array_equal(u16(packed), oracle.pack(ost))
    words = gpu.codec.swizzle_for_kernel(packed, 256, 256)
    assert np.array_equal(u16(words).reshape(-1), oracle.swizzle(oracle.pack(ost), 256, 256).reshape(-1))
    back = gpu.codec.unpack_trellis(gpu.codec.unswizzle_for_kernel(words, 256, 256))
    assert np.array_equal(u16(back), ost)
    dec = torch.empty((256, 256), dtype=torch.float32, device="cuda")
    gpu.codec.k_decode_states(back, 256, dec, lut_d)
    assert np.array_equal(dec.cpu().numpy(), ohat)
    mse_gpu = ((dec.cpu().numpy() - X) ** 2).mean(axis=1)
    mse_cpu = ((ohat - X) ** 2).mean(axis=1)
    assert np.array_equal(mse_gpu, mse_cpu)
    # the fp64 reference Viterbi on the fp16-rounded matrix: same paths on nearly every tile, same distortion
    st64, hat64, _ = oracle.quantize_seq_ref(X.astype(np.float16).astype(np.float32), lut)
    assert (st64 == ost).all(axis=1).mean() > 0.9
    assert abs(((hat64 - X) ** 2).mean() - mse_cpu.mean()) < 1e-4


def test_invariants_at_scale(gpu):
    """4,608 sequences (more than one wave of clusters): trellis links, tail-biting, decode(encode) round trip,
    pack/unpack round trip, and distortion in the range of a 2-bit trellis code on N(0,1) data."""
    s = gpu.synth
    tl = s.seeded_tlut(1)
    lut_d, rms = gpu_lut(gpu, tl)
    X = s.gaussian_matrix(4608, 256, 2) * np.float32(rms / 0.9)  # the quantizer's scaling of a unit-variance matrix
    ws = gpu.codec.quantize_workspace(2304)
    st, hat = gpu.codec.quantize_tiles(dev(X), lut_d, workspace=ws)
    ws.check()
    sd = st.to(torch.int32) & 0xFFFF
    assert bool(((sd[:, 127] & 0xFFF) == (sd[:, 0] >> 4)).all())
    assert bool((((sd[:, :-1] << 4) & 0xFFFF) == (sd[:, 1:] & 0xFFF0)).all())
    dec = torch.empty_like(hat)
    gpu.codec.k_decode_states(st, 4608, dec, lut_d)
    assert torch.equal(dec, hat)
    assert torch.equal(gpu.codec.unpack_trellis(gpu.codec.pack_trellis(st)), st)
    mse = float(((hat - dev(X)) ** 2).mean()) / float((dev(X) ** 2).mean())
    assert 0.05 < mse < 0.2, mse  # a random Gaussian codebook is worse than the trained one (0.07) but well below 1 bit


@pytest.mark.parametrize("B", [1, 13, 64])
def test_kernel_level_forward_ragged_batches_bit_exact(gpu, oracle, hyb, B):
    """qtip_k_viterbi_fwd (cluster kernel writing the reference's back-pointer layout) against the oracle's restatement
    of the reference kernel: every back-pointer word and final state, both passes, batch sizes that leave the last
    cluster batch partly filled."""
    tl, lut, _ = hyb
    lut_d, _ = gpu_lut(gpu, tl)
    X = (np.random.default_rng(100 + B).standard_normal((B, 256)) * 1.1).astype(np.float32)
    A1, fs1, ov, A2, fs2, Q = staged(gpu, X, lut_d)
    oA1, ofs1 = oracle.viterbi_fwd(X, None, 1, lut)
    assert np.array_equal(A1, oA1) and np.array_equal(fs1, ofs1)
    oov = oracle.viterbi_overlap(oA1, ofs1)
    assert np.array_equal(ov, oov)
    oA2, ofs2 = oracle.viterbi_fwd(X, oov, 0, lut)
    assert np.array_equal(A2, oA2) and np.array_equal(fs2, ofs2)
    assert np.array_equal(Q, oracle.viterbi_finish(oA2, ofs2, lut))
    gpu.linear.kernel_status()


def test_two_chunks_in_flight_give_the_same_codes(gpu, hyb):
    """A workspace smaller than the batch makes the fused call alternate chunks between its stream and a side stream;
    the result must equal the single-chunk run bit for bit, and the status word must stay clean."""
    tl, _, _ = hyb
    lut_d, _ = gpu_lut(gpu, tl)
    B = 600
    X = dev((np.random.default_rng(9).standard_normal((B, 256)) * 0.8).astype(np.float32))
    c = gpu.codec
    big = c.quantize_workspace(2 * B)      # B <= half of the capacity: one chunk, one stream
    small = c.quantize_workspace(256)      # chunks of 128 sequences on two streams
    s1, h1 = c.quantize_tiles(X, lut_d, workspace=big)
    s2, h2 = c.quantize_tiles(X, lut_d, workspace=small)
    big.check()
    small.check()
    assert torch.equal(s1, s2) and torch.equal(h1, h2)
