"""Fused decode-step epilogues (qtip_input_transform, qtip_output_residual, qtip_output_gateup,
qtip_output_residual_input) against (1) the unfused stages of the operator composed by hand, bit for bit; (2) each other:
the chunk-per-CTA kernels (few rows) and the whole-row kernels (many rows) must give identical bits, which is the
reference's own acceptance test for its row-batched variants (runtime/tests/qtip_tests.cpp:570-696); (3) a numpy
restatement around the fp64 transform, within one bf16 rounding."""
import numpy as np
import pytest
import torch

from test_decode_gpu import rel_l2
from test_viterbi_gpu import dev

pytestmark = pytest.mark.gpu
EPS = 1e-5


def bf16_rows(rows, n, seed, scale=1.0):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return (torch.randn(rows, n, generator=g, device="cuda") * scale).to(torch.bfloat16)


def ulp_report(a, b):
    """(fraction of differing elements, largest difference in bf16 code steps) of two bf16 tensors."""
    ia, ib = a.view(torch.int16).int(), b.view(torch.int16).int()
    d = (ia - ib).abs()
    return float((d != 0).float().mean()), int(d.max())


@pytest.mark.parametrize("n", [12288, 28672, 1024])
def test_input_transform_without_norm_equals_prepare(gpu, n):
    lin = gpu.linear
    su = dev(gpu.synth.signs(n, 7))
    w = lin.Matrix(None, su, dev(gpu.synth.signs(32, 8)), None, n, 32)
    for rows in (1, 3, 40):  # K CTAs per row, and one CTA per row
        x = bf16_rows(rows, n, rows)
        u, rot = (torch.empty(rows, n, dtype=torch.bfloat16, device="cuda") for _ in range(2))
        lin.input_transform(x, None, 0.0, su, n, rows, u)
        lin.qtip_prepare(w, x, torch.empty(1, device="cuda"), rot, rows)
        assert torch.equal(u.view(torch.int16), rot.view(torch.int16))


@pytest.mark.parametrize("n", [12288, 28672, 8192])
def test_input_transform_with_norm(gpu, oracle, n):
    lin = gpu.linear
    su = dev(gpu.synth.signs(n, 7))
    norm = (1.0 + 0.1 * bf16_rows(1, n, 99).float()).to(torch.bfloat16).view(-1)
    big = bf16_rows(40, n, 5, 2.0)
    u_big, xn_big = (torch.empty(40, n, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    lin.input_transform(big, norm, EPS, su, n, 40, u_big, xn_big)  # one CTA per row
    small = big[:3].contiguous()
    u_s, xn_s = (torch.empty(3, n, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    lin.input_transform(small, norm, EPS, su, n, 3, u_s, xn_s)     # K CTAs per row
    assert torch.equal(u_s.view(torch.int16), u_big[:3].view(torch.int16))
    assert torch.equal(xn_s.view(torch.int16), xn_big[:3].view(torch.int16))
    # the transform of the normalised row is the operator's input stage, bit for bit
    w = lin.Matrix(None, su, dev(gpu.synth.signs(32, 8)), None, n, 32)
    rot = torch.empty(40, n, dtype=torch.bfloat16, device="cuda")
    lin.qtip_prepare(w, xn_big, torch.empty(1, device="cuda"), rot, 40)
    assert torch.equal(rot.view(torch.int16), u_big.view(torch.int16))
    # RMSNorm against fp64: the normalised row differs by at most one bf16 step, and rarely
    x64 = big.double()
    ref = (x64 * torch.rsqrt((x64 * x64).mean(dim=1, keepdim=True) + EPS)).float() * norm.float()[None, :]
    frac, steps = ulp_report(xn_big, ref.to(torch.bfloat16))
    assert steps <= 1 and frac < 2e-2
    # and the whole stage against the numpy restatement (first two rows)
    u_o, _ = oracle.input_transform(big[:2].float().cpu().numpy(), norm.float().cpu().numpy(), EPS, su.cpu().numpy())
    assert rel_l2(u_big[:2].float().cpu().numpy(), u_o.astype(np.float64)) < 4e-3


@pytest.mark.parametrize("n,splits", [(12288, 1), (12288, 3), (28672, 2), (1024, 1)])
def test_output_residual(gpu, oracle, n, splits):
    lin = gpu.linear
    sv = dev((gpu.synth.signs(n, 8) * np.float32(0.02)).astype(np.float32))
    w = lin.Matrix(None, dev(gpu.synth.signs(32, 7)), sv, None, 32, n)
    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    for rows in (2, 40):
        z = torch.randn(splits, rows, n, generator=g, device="cuda")
        state = bf16_rows(rows, n, 12)
        y = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
        lin.qtip_finish(w, z, y, torch.empty(1, device="cuda"), False, splits, rows)
        expect = (state.float() + y.float()).to(torch.bfloat16)
        st = state.clone()
        lin.output_residual(z, splits, rows, sv, n, st)
        assert torch.equal(st.view(torch.int16), expect.view(torch.int16))
    zs = z.sum(0)[:2].cpu().numpy()
    ref = oracle.output_residual(zs, sv.cpu().numpy(), state[:2].float().cpu().numpy())
    assert rel_l2(st[:2].float().cpu().numpy(), ref.astype(np.float64)) < 4e-3


@pytest.mark.parametrize("F,splits", [(28672, 1), (28672, 2), (12288, 1), (8192, 1)])
def test_output_gateup(gpu, oracle, F, splits):
    lin = gpu.linear
    svg = dev((gpu.synth.signs(F, 8) * np.float32(0.05)).astype(np.float32))
    svu = dev((gpu.synth.signs(F, 9) * np.float32(0.04)).astype(np.float32))
    wg = lin.Matrix(None, dev(gpu.synth.signs(32, 7)), svg, None, 32, F)
    wu = lin.Matrix(None, dev(gpu.synth.signs(32, 7)), svu, None, 32, F)
    g = torch.Generator(device="cuda")
    g.manual_seed(21)
    z40 = torch.randn(splits, 40, 2 * F, generator=g, device="cuda")
    outs = {}
    for rows, z in ((40, z40), (3, z40[:, :3].contiguous())):  # one CTA per row, and K CTAs per row
        h = torch.empty(rows, F, dtype=torch.bfloat16, device="cuda")
        lin.output_gateup(z, splits, rows, svg, svu, F, h)
        outs[rows] = h
    yg, yu = (torch.empty(40, F, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    scratch = torch.empty(1, device="cuda")
    lin.qtip_finish(wg, z40[:, :, :F].contiguous(), yg, scratch, True, splits, 40)
    lin.qtip_finish(wu, z40[:, :, F:].contiguous(), yu, scratch, True, splits, 40)
    gf, uf = yg.float(), yu.float()
    expect = (gf / (1.0 + torch.exp(-gf)) * uf).to(torch.bfloat16)
    frac, steps = ulp_report(outs[40], expect)
    assert steps <= 1 and frac < 1e-3  # exp() of two libraries
    assert torch.equal(outs[3].view(torch.int16), outs[40][:3].view(torch.int16))  # chunk kernels == row kernels
    ref = oracle.output_gateup(z40.sum(0)[:2].cpu().numpy(), svg.cpu().numpy(), svu.cpu().numpy())
    assert rel_l2(outs[40][:2].float().cpu().numpy(), ref.astype(np.float64)) < 6e-3


@pytest.mark.parametrize("n", [12288, 28672])
def test_output_residual_input_fused_equals_separate(gpu, n):
    lin = gpu.linear
    su = dev(gpu.synth.signs(n, 7))
    sv = dev((gpu.synth.signs(n, 8) * np.float32(0.02)).astype(np.float32))
    norm = (1.0 + 0.1 * bf16_rows(1, n, 98).float()).to(torch.bfloat16).view(-1)
    g = torch.Generator(device="cuda")
    g.manual_seed(31)
    z = torch.randn(2, 40, n, generator=g, device="cuda")
    state0 = bf16_rows(40, n, 32)
    # separate stages
    st_a = state0.clone()
    u_a, xn_a = (torch.empty(40, n, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    lin.output_residual(z, 2, 40, sv, n, st_a)
    lin.input_transform(st_a, norm, EPS, su, n, 40, u_a, xn_a)
    # one call, 40 rows: the fused whole-row kernel
    st_b = state0.clone()
    u_b, xn_b = (torch.empty(40, n, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    lin.output_residual_input(z, 2, 40, sv, n, st_b, norm, EPS, su, u_b, xn_b)
    for a, b in ((st_a, st_b), (u_a, u_b), (xn_a, xn_b)):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    # one call, 3 rows: two launches inside
    st_c = state0[:3].clone()
    u_c = torch.empty(3, n, dtype=torch.bfloat16, device="cuda")
    lin.output_residual_input(z[:, :3].contiguous(), 2, 3, sv, n, st_c, norm, EPS, su, u_c)
    assert torch.equal(st_c.view(torch.int16), st_a[:3].view(torch.int16))
    assert torch.equal(u_c.view(torch.int16), u_a[:3].view(torch.int16))


@pytest.mark.parametrize("n", [12288, 28672])
def test_large_batch_row_kernels_match_the_chunk_kernels(gpu, n):
    """Large batches (whole-row CTAs of 512 threads, several per SM) against the few-row chunk kernels on the same rows:
    identical bits for the input transform, the output transform from fp32 products (with and without the bf16 rounding
    of z) and the output transform from bf16 products."""
    rows = 333  # more rows than SMs, not a multiple of anything
    lin = gpu.linear
    su, sv = dev(gpu.synth.signs(n, 7)), dev(gpu.synth.signs(n, 8)) * 0.01
    w = lin.Matrix(None, su, sv, None, n, n)
    scratch = torch.empty(1, device="cuda")
    x = bf16_rows(rows, n, 3)
    u_big = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
    lin.qtip_prepare(w, x, scratch, u_big, rows)
    pick = [0, 147, 148, rows - 1]
    for r in pick:
        u_one = torch.empty(1, n, dtype=torch.bfloat16, device="cuda")
        lin.qtip_prepare(w, x[r:r + 1].contiguous(), scratch, u_one, 1)
        assert torch.equal(u_big[r].view(torch.int16), u_one[0].view(torch.int16)), "input transform, row %d" % r
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    z = torch.randn(1, rows, n, generator=g, device="cuda")
    for round_z in (False, True):
        y_big = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
        lin.qtip_finish(w, z, y_big, scratch, round_z, 1, rows)
        for r in pick:
            y_one = torch.empty(1, n, dtype=torch.bfloat16, device="cuda")
            lin.qtip_finish(w, z[:, r:r + 1].contiguous(), y_one, scratch, round_z, 1, 1)
            assert torch.equal(y_big[r].view(torch.int16), y_one[0].view(torch.int16)), "output transform, row %d" % r
    zb = z[0].to(torch.bfloat16)
    y_big = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
    lin.qtip_finish_b16(w, zb, y_big, scratch, rows)
    for r in pick:
        y_one = torch.empty(1, n, dtype=torch.bfloat16, device="cuda")
        lin.qtip_finish_b16(w, zb[r:r + 1].contiguous(), y_one, scratch, 1)
        assert torch.equal(y_big[r].view(torch.int16), y_one[0].view(torch.int16)), "bf16 output transform, row %d" % r
