"""Worker of the two-process tensor-parallel test (launched by torch.distributed.run, one process per GPU)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    import __graft_entry__ as g
    pkg = g.load_package()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("gloo")
    pkg.codec.init()
    from test_decode_gpu import bf16_dev, make_linear
    n_in, n_out, tokens = 3584, 4096, 3
    w, *_ = make_linear(pkg, n_in, n_out, 500, sv_scale=0.02)
    row0, rows = pkg.sharding.block_row_range(n_out, rank, world)
    shard = w.rows(row0, rows)
    ex = pkg.tp.Exchange.from_process_group(n_out, max_tokens=tokens)
    rot = torch.empty((tokens, n_in), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(tokens * max(n_in, n_out), dtype=torch.float32, device="cuda")
    y = torch.empty((tokens, n_out), dtype=torch.bfloat16, device="cuda")
    want = torch.empty_like(y)
    z = torch.zeros((1, tokens, n_out), dtype=torch.float32, device="cuda")
    for step in range(6):
        xb = pkg.synth.f32_to_bf16_bits((np.random.default_rng(step).standard_normal((tokens, n_in)) * 0.3).astype(np.float32))
        x = bf16_dev(xb)
        pkg.tp.forward_tp(ex, w, shard, row0, x, y, scratch, rot, False, 1, tokens, wait_inside=step % 3 != 2)
        ex.check()
        pkg.linear.qtip_prepare(w, x, scratch, rot, tokens)
        pkg.linear.qtip_multiply_batch(w, rot, z, n_out, 1, tokens)
        pkg.linear.qtip_finish(w, z, want, scratch, False, 1, tokens)
        torch.cuda.synchronize()
        err = float((y.float() - want.float()).norm() / want.float().norm())
        assert err < 2e-3, (step, err)  # the unsharded launch adds the K pieces of some rows in another order
    dist.barrier()
    ex.close()
    dist.destroy_process_group()
    print("tp worker ok", flush=True)


if __name__ == "__main__":
    main()
