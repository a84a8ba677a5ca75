"""Small fixed workloads for ncu captures (the commands in profiles/*.md run this file):

    python tests/profile_targets.py viterbi <sequences>     # 4 forward passes of the cluster Viterbi kernel
    python tests/profile_targets.py gemv <out rows>         # 3 x qtip_forward on an <out rows> x 12288 linear
    python tests/profile_targets.py fused <out rows> [tokens] [splits]   # 3 x qtip_multiply_tc, <out rows> x 12288
    python tests/profile_targets.py prefill <out rows> [tokens]          # 3 x qtip_prefill_gemm, <out rows> x 12288
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import __graft_entry__ as graft  # noqa: E402


def main():
    pkg = graft.load_package()
    codec, linear, synth = pkg.codec, pkg.linear, pkg.synth
    codec.init()
    what, size = sys.argv[1], int(sys.argv[2])
    gen = torch.Generator(device="cuda")
    gen.manual_seed(9)
    if what == "viterbi":
        lut_d, _ = codec.device_lut(synth.seeded_tlut(1))
        X = torch.randn(size, 256, generator=gen, device="cuda")
        bp = torch.empty((size, 16, 4096), dtype=torch.int32, device="cuda")
        fs = torch.empty(size, dtype=torch.int16, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        for _ in range(4):
            codec.k_viterbi_fwd_words(X, None, 1, size, bp, 0, fs, lut_d, status)
        torch.cuda.synchronize()
        assert int(status) == 0
    elif what == "prefill":
        n_in, n_out = 12288, size
        tokens = int(sys.argv[3]) if len(sys.argv) > 3 else 2048
        wd = torch.randn(n_out, n_in, generator=gen, device="cuda").to(torch.bfloat16)
        x = torch.randn(tokens, n_in, generator=gen, device="cuda").to(torch.bfloat16)
        z = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        for _ in range(3):
            linear.prefill_gemm(wd, x, z, n_out, n_in, n_out, tokens, status)
        torch.cuda.synchronize()
        assert int(status) == 0
    elif what == "fused":
        n_in, n_out = 12288, size
        tokens = int(sys.argv[3]) if len(sys.argv) > 3 else 64
        splits = int(sys.argv[4]) if len(sys.argv) > 4 else 1
        trellis = torch.randint(-32768, 32768, ((n_out // 16) * (n_in // 16) * 32,), generator=gen, device="cuda",
                                dtype=torch.int16)
        su = torch.from_numpy(synth.signs(n_in, 7)).cuda()
        sv = torch.from_numpy(synth.signs(n_out, 8)).cuda()
        w = linear.Matrix(trellis, su, sv, linear.runtime_lut(synth.seeded_tlut(1)), n_in, n_out)
        x = torch.randn(tokens, n_in, generator=gen, device="cuda").to(torch.bfloat16)
        z = torch.empty((splits, tokens, n_out), dtype=torch.float32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        for _ in range(3):
            linear.qtip_multiply_tc(w, x, z, n_out, splits, tokens, status)
        torch.cuda.synchronize()
        assert int(status) == 0
    else:
        n_in, n_out = 12288, size
        trellis = torch.randint(-32768, 32768, ((n_out // 16) * (n_in // 16) * 32,), generator=gen, device="cuda",
                                dtype=torch.int16)
        su = torch.from_numpy(synth.signs(n_in, 7)).cuda()
        sv = torch.from_numpy(synth.signs(n_out, 8)).cuda()
        w = linear.Matrix(trellis, su, sv, linear.runtime_lut(synth.seeded_tlut(1)), n_in, n_out)
        x = torch.randn(n_in, generator=gen, device="cuda").to(torch.bfloat16)
        y = torch.empty(n_out, dtype=torch.bfloat16, device="cuda")
        rot = torch.empty(n_in, dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(n_out, dtype=torch.float32, device="cuda")
        z = torch.empty(n_out, dtype=torch.float32, device="cuda")
        for _ in range(3):
            linear.qtip_forward(w, x, y, scratch, rot, z, False, 1)
        torch.cuda.synchronize()


if __name__ == "__main__":
    main()
