#!/usr/bin/env python
"""Benchmark of the QTIP trellis codec hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU implementation of the same path

Headline workload (N = 1): two-pass tail-biting Viterbi encode of a 12288 x 12288 fp32 matrix (i.i.d. N(0,1) from a
seed, seeded 2^9-entry codebook, identity Hessian, 589,824 independent 16x16 tiles). One step = the whole matrix. For
N > 1 the tile rows are split contiguously over the ranks (strong scaling, no collective on the data path).
One JSON line on stdout (rank 0).
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, N_COLS = 12288, 12288
LANE_OPS_PER_WEIGHT = 327680  # 2 passes x 128 steps x 65,536 states / 256 weights x 5 ops (add, 2 fma, tag, min)
METRIC = "viterbi_quantized_weights_per_second"
NCU_DRAM_BYTES_PER_TILE_PASS = 9104128 // 240  # DRAM read + write of one profiled 240-sequence launch


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "sm_max_mhz": 1965.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.out = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.out.flush()
        self.out.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.out.read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        self.out.close()
        os.unlink(self.out.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        # median over the upper half of the samples: the sampler also sees the idle gaps around the timed region
        load = sm[len(sm) // 2:]
        return {"sm_mhz": load[len(load) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_rate(seconds_target, X, tlut_bits):
    """weights/s of the reference's own fp64 tail-biting Viterbi (quantize_seq_ref, compiled in place, OpenMP over
    sequences) on a bounded sample; falls back to the oracle port when the reference build is absent."""
    from oracle.oracle import Oracle, Reference
    R = Reference()
    threads = len(os.sched_getaffinity(0))
    try:  # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core
        import ctypes
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(threads)
    except OSError:
        pass
    x16 = lambda a: a.astype(np.float16).astype(np.float32)  # noqa: E731  (the quantizer hands the CPU path fp16 values)
    if R.available and np.array_equal(R.codebook()[0].reshape(-1), tlut_bits.reshape(-1)):
        run, kind = (lambda a: R.quantize_seqs(a)), "reference"
    elif R.available:
        # the reference's codebook is compiled in; its speed does not depend on the table's values
        run, kind = (lambda a: R.quantize_seqs(a)), "reference"
    else:
        O = Oracle()
        lut, _ = O.build_lut(tlut_bits)
        run, kind = (lambda a: O.quantize_seq_ref(a, lut)), "port"
    probe = x16(X[:4 * threads])
    t0 = time.perf_counter()
    run(probe)
    dt = time.perf_counter() - t0
    n = int(max(4 * threads, min(len(X), len(probe) * seconds_target / max(dt, 1e-3))))
    n = n // threads * threads
    sample = x16(X[:n])
    t0 = time.perf_counter()
    run(sample)
    dt = time.perf_counter() - t0
    return {"value": n * 256 / dt, "unit": "weights/s", "cores": threads, "kind": kind,
            "sample": "%d tiles of the workload's distribution (i.i.d. N(0,1), same codebook), %.1f s" % (n, dt)}


def reference_gpu_rates(pkg, torch):
    """The reference's own CUDA kernels (compiled in place for sm_100a, test infrastructure under oracle/_ref) timed on
    this GPU beside ours, as a second reported baseline: its two-pass Viterbi on 4,096 tiles (the size of its own
    --bench run) and its batch-1 operator on the 57344 x 12288 matrix. CUDA events, launches queued back to back."""
    from oracle.oracle import ReferenceGpu
    R = ReferenceGpu()
    if not R.available:
        return {"unavailable": "oracle/_ref holds no build of the reference's CUDA kernels"}
    synth, codec, linear = pkg.synth, pkg.codec, pkg.linear
    p = lambda t: None if t is None else t.data_ptr()  # noqa: E731

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    tiles, batch = 4096, 1024
    X = torch.from_numpy(synth.tile_sequences(synth.gaussian_matrix(256, tiles, 2))).cuda()  # 16 x (tiles / 16) tiles
    lut_d, _ = codec.device_lut(synth.seeded_tlut(1))
    A = torch.empty((batch, 127, 1024), dtype=torch.int16, device="cuda")
    fs = torch.empty(batch, dtype=torch.int16, device="cuda")
    ov = torch.empty(batch, dtype=torch.int32, device="cuda")
    Q = torch.empty((tiles, 128), dtype=torch.int16, device="cuda")
    hat = torch.empty((16, 16 * tiles), dtype=torch.float32, device="cuda")

    def ref_quantize():
        for b0 in range(0, tiles, batch):
            x = X[b0:b0 + batch]
            R.viterbi_fwd(p(x), None, 1, batch, p(A), p(fs), p(lut_d))
            R.viterbi_overlap(p(A), p(fs), batch, p(ov))
            R.viterbi_fwd(p(x), p(ov), 0, batch, p(A), p(fs), p(lut_d))
            R.viterbi_finish(p(A), p(fs), batch, b0, p(Q), 1, 0, p(hat), 16 * tiles, 0, p(lut_d))

    vit_ms = timed(ref_quantize, 2)
    ours_states, _ = codec.quantize_tiles(X, lut_d)
    same = bool(torch.equal(ours_states, Q))
    del A, hat
    res = {"viterbi_weights_per_s": tiles * 256 / (vit_ms * 1e-3), "viterbi_sample": "%d tiles, batches of %d" % (tiles, batch),
           "viterbi_codes_identical_to_ours": same}

    n_in, n_out = 12288, 57344
    R.initialize_tables()
    trellis = torch.from_numpy(synth.random_trellis(n_out, n_in, 4).view(np.int16)).cuda()
    su, sv = (torch.from_numpy(synth.signs(n, 5 + i)).cuda() for i, n in enumerate((n_in, n_out)))
    w = linear.Matrix(trellis, su, sv, linear.runtime_lut(synth.seeded_tlut(1)), n_in, n_out)
    wr = (p(w.trellis), p(w.su), p(w.sv), p(w.lut), n_in, n_out)
    x = torch.randn(n_in, device="cuda").to(torch.bfloat16)
    rot = torch.empty(n_in, dtype=torch.bfloat16, device="cuda")
    y = torch.empty(n_out, dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(n_out, dtype=torch.float32, device="cuda")
    z = torch.empty((32, n_out), dtype=torch.float32, device="cuda")
    R.qtip_prepare(wr, p(x), p(scratch), p(rot))
    best = None
    for splits in (1, 2, 4, 8, 16, 32):
        mus = timed(lambda: R.qtip_multiply(wr, p(rot), p(z), n_out, splits), 20) * 1e3
        fus = timed(lambda: R.qtip_forward(wr, p(x), p(y), p(scratch), p(rot), p(z), False, splits), 20) * 1e3
        if best is None or fus < best["gemv_forward_us"]:
            best = {"gemv_splits": splits, "gemv_multiply_us": mus, "gemv_forward_us": fus}
    res.update(best)
    res["kind"] = "the reference's CUDA kernels recompiled for sm_100a, same GPU, same inputs"
    try:
        res["gemv_cpu"] = cpu_gemv(pkg, torch, w, x, y)
    except Exception as ex:
        res["gemv_cpu"] = {"error": repr(ex)}
    return res


def cpu_gemv(pkg, torch, w, x, y_ref_gpu):
    """Reported CPU baseline of the decode operator: the reference's own reference_forward (runtime/src/qtip.cpp:129-192,
    compiled in place, OpenMP, double accumulation, device rounding) on the full 57344 x 12288 matrix, one token, beside
    the outputs the reference's GPU operator just produced for the same input. Test infrastructure."""
    from oracle.oracle import Oracle, Reference
    R, synth = Reference(), pkg.synth
    fwd, kind = (R.reference_forward, "reference") if R.available else (Oracle().reference_forward, "port")
    tr = w.trellis.cpu().numpy().view(np.uint16)
    su, sv = w.su.cpu().numpy(), w.sv.cpu().numpy()
    xf = x.float().cpu().numpy()
    tl = synth.seeded_tlut(1).view(np.uint16)
    t0 = time.perf_counter()
    out = fwd(tr, su, sv, tl, w.n_in, w.n_out, xf, True, False)
    dt = time.perf_counter() - t0
    yc = np.asarray(out[0] if isinstance(out, tuple) else out, dtype=np.float64).reshape(-1)
    yg = y_ref_gpu.float().cpu().numpy().astype(np.float64)
    return {"kind": kind, "cores": len(os.sched_getaffinity(0)), "seconds": dt, "sample": "the whole matrix, one token",
            "gbs_on_algorithmic_bytes": (w.n_in * w.n_out / 4 + 2 * w.n_in + 4 * w.n_out + 4096) / dt / 1e9,
            "rel_l2_of_the_gpu_operator_output": float(np.linalg.norm(yg - yc) / np.linalg.norm(yc))}


def reference_arm(args):
    """The reference's CPU implementation of the path on the host cores, same config and metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import __graft_entry__ as graft
    pkg = graft.load_package()
    s = pkg.synth
    tiles = 4096
    X = s.tile_sequences(s.gaussian_matrix(256, tiles * 16, 2))  # 4,096 tiles of the same distribution
    tl = s.seeded_tlut(1).view(np.uint16)
    rates, last = [], None
    per_step = max(3.0, min(20.0, 90.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        last = cpu_reference_rate(per_step, X, tl)
        if i >= args.warmup:
            rates.append(last["value"])
    v = float(np.mean(rates))
    last["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "weights/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * M * N_COLS / v, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": "viterbi_encode_12288x12288_identityH", "tiles": M * N_COLS // 256,
                       "note": "CPU path timed on a bounded sample; ms_per_step extrapolates to the full matrix"},
            "cpu_baseline": last,
            "e2e": {"value": v, "unit": "weights/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


class Ctx:
    pass


def setup(args):
    """One process per GPU: device, process group (NCCL) when launched under torchrun, library set-up."""
    import torch
    import torch.distributed as dist
    import __graft_entry__ as graft
    ctx = Ctx()
    ctx.torch, ctx.dist, ctx.pkg = torch, dist, graft.load_package()
    ctx.rank = int(os.environ.get("RANK", "0"))
    ctx.world = int(os.environ.get("WORLD_SIZE", "1"))
    ctx.local = int(os.environ.get("LOCAL_RANK", "0"))
    assert ctx.world == args.gpus, "launch with torchrun --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus)
    torch.cuda.set_device(ctx.local)
    if ctx.world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", ctx.local))
    ctx.pkg.codec.init()
    return ctx


def finish(ctx):
    if ctx.world > 1:
        ctx.dist.barrier()
        ctx.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=M, help="rows of the matrix (default: the full 12288)")
    ap.add_argument("--no-extras", action="store_true", help="skip the GEMV section and the CPU baseline")
    ap.add_argument("--workload", default="viterbi", choices=["viterbi", "ldlq", "layer", "kernel"],
                    help="viterbi: the headline identity-Hessian encode; ldlq: LDLQ + Viterbi on a 12288 x 28672 matrix "
                         "with a synthetic correlated Hessian (secondary line); layer: the products of one layer; "
                         "kernel: a few launches of one kernel on a small case (for profiler captures)")
    ap.add_argument("--ldlq-shape", default="12288x28672", help="m x n of the ldlq workload")
    ap.add_argument("--kernel", default="gemv", choices=["viterbi", "gemv", "fused", "prefill", "epilogue"],
                    help="--workload kernel: which kernel")
    ap.add_argument("--size", type=int, default=16384, help="--workload kernel: sequences (viterbi) or output rows")
    ap.add_argument("--tokens", type=int, default=0, help="--workload kernel: token count (fused: 64, prefill: 2048)")
    ap.add_argument("--splits", type=int, default=1, help="--workload kernel: K-splits (fused, gemv)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload == "kernel":
        return kernel_workload(args)
    ctx = setup(args)
    if args.workload == "ldlq":
        res = ldlq_section(ctx, args.ldlq_shape, args.steps, args.warmup)
        if ctx.rank == 0:
            print(json.dumps(res))
        return finish(ctx)
    if args.workload == "layer":
        res = layer_section(ctx)
        if ctx.rank == 0:
            print(json.dumps(res))
        return finish(ctx)
    torch, dist, pkg = ctx.torch, ctx.dist, ctx.pkg
    codec, synth = pkg.codec, pkg.synth
    rank, world, local = ctx.rank, ctx.world, ctx.local
    peaks, peak_src = measured_peaks()

    # ---- this rank's tile rows of the matrix (generated per rank from the same seed: row r comes from seed 2 + r)
    m_rows = args.rows
    b, e = pkg.sharding.tile_row_range(m_rows // 16, rank, world)
    tiles_local = (e - b) * (N_COLS // 16)
    tl = synth.seeded_tlut(1)
    lut_d, lut_rms = codec.device_lut(tl)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2 + 1000003 * b)
    W = torch.randn((e - b) * 16, N_COLS, generator=gen, device="cuda", dtype=torch.float32)
    X = codec.tiles_from_matrix(W)
    chunk = 4608  # sequences per forward launch; the workspace holds two chunks, which alternate between two streams
    ws = codec.quantize_workspace(2 * chunk)
    states = torch.empty((tiles_local, 128), dtype=torch.int16, device="cuda")
    torch.cuda.synchronize()

    # hat output is optional in the C ABI; the encode bench needs the codes only
    def step_codes():
        pkg.lib().call("qtip_quantize_tiles", X.data_ptr(), tiles_local, lut_d.data_ptr(), states.data_ptr(), None,
                       ws.ptr, ws.nbytes, torch.cuda.current_stream().cuda_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Inputs smaller than twice the 126 MB L2 (many ranks): overwrite a 256 MB buffer between steps so that no step
    # starts with its sequences cached (0.04 ms per flush inside a step of hundreds of ms).
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if tiles_local * 1024 < (252 << 20) else None
    for _ in range(args.warmup):
        step_codes()
    ws.check()
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        if flush is not None:
            flush.zero_()
        step_codes()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if sampler else None
    ws.check()
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t) / args.steps
    total_weights = m_rows * N_COLS
    value = total_weights / (ms_step * 1e-3)

    # ---- the dominant kernel alone: forward passes over one chunk, CUDA events on the launching stream
    nb = min(chunk, tiles_local)
    bp = torch.empty((nb, 16, 4096), dtype=torch.int32, device="cuda")
    fs = torch.empty(nb, dtype=torch.int16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    reps = 4
    codec.k_viterbi_fwd_words(X, None, 1, nb, bp, 0, fs, lut_d, status)
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(reps):
        codec.k_viterbi_fwd_words(X, None, 1, nb, bp, 0, fs, lut_d, status)
    k1.record()
    torch.cuda.synchronize()
    kern_ms = k0.elapsed_time(k1) / reps
    lane_ops = nb * 256 * LANE_OPS_PER_WEIGHT / 2  # one pass
    sm_count = torch.cuda.get_device_properties(local).multi_processor_count
    peak_ops = sm_count * 128 * peaks.get("sm_max_mhz", 1965.0) * 1e6
    achieved = lane_ops / (kern_ms * 1e-3)
    launches_per_step = 4 * ((tiles_local + chunk - 1) // chunk)

    # ---- end to end through the C ABI with host buffers: H2D of the fp32 matrix, tile gather, two-pass Viterbi, pack,
    # kernel-layout swizzle, D2H of the trellis words. Rank 0's share at N > 1 (every rank does the same on its rows).
    rows_local = (e - b) * 16
    e2e = None
    if rank == 0:
        W_h = torch.empty((rows_local, N_COLS), dtype=torch.float32).pin_memory()
        W_h.copy_(W.cpu())
        out_h = torch.empty((tiles_local, 32), dtype=torch.int16).pin_memory()
        packed = torch.empty((tiles_local, 32), dtype=torch.int16, device="cuda")
        words = torch.empty_like(packed)

        def step_e2e():
            W.copy_(W_h, non_blocking=True)
            codec.tiles_from_matrix(W, X)
            step_codes()
            codec.pack_trellis(states, packed)
            if rows_local % 32 == 0:
                codec.swizzle_for_kernel(packed, rows_local, N_COLS, words)
                out_h.copy_(words, non_blocking=True)
            else:
                out_h.copy_(packed, non_blocking=True)
            torch.cuda.synchronize()

        step_e2e()
        t0 = time.perf_counter()
        e2e_steps = max(1, min(2, args.steps))
        for _ in range(e2e_steps):
            step_e2e()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        e2e = {"value": rows_local * N_COLS * world / e2e_s, "unit": "weights/s",
               "h2d_bytes_per_step": rows_local * N_COLS * 4, "d2h_bytes_per_step": tiles_local * 64}
        del W_h, out_h, packed, words
    del W, X, states, ws, bp, fs
    torch.cuda.empty_cache()

    # ---- the other configurations of the path, as extra objects of the same line: batch-1 GEMV (config 4), LDLQ +
    # Viterbi (config 3), the products of one layer (config 5). Every rank takes part; a failure of one of them on one
    # GPU must not lose the headline.
    extras = {}
    if not args.no_extras:
        sections = [("gemv", lambda: gemv_section(pkg, peaks, peak_src, rank, world))]
        if m_rows == M:  # reduced-size runs (profiler captures) skip the long sections
            sections += [("ldlq", lambda: ldlq_section(ctx, "12288x28672", 1, 1)), ("layer", lambda: layer_section(ctx))]
        for name, fn in sections:
            try:
                extras[name] = fn()
            except Exception as ex:
                if world > 1:
                    raise
                extras[name] = {"error": repr(ex)}
            torch.cuda.empty_cache()
    if rank != 0:
        return finish(ctx)

    line = {"metric": METRIC, "value": value, "unit": "weights/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "viterbi_encode_%dx%d_identityH" % (m_rows, N_COLS), "tiles": total_weights // 256,
                       "L": 16, "K": 2, "V": 2, "codebook": "seeded N(0,1) 2^9 x 2, unit rms, fp16",
                       "l2": ("inputs (%.0f MB per rank) exceed the 126 MB L2" % (tiles_local * 1024 / 1e6)) if flush is None
                       else ("inputs are %.0f MB per rank: a 256 MB buffer is overwritten between steps to flush the L2"
                             % (tiles_local * 1024 / 1e6)),
                       "sharding": "contiguous tile rows per rank, no collective", "chunk_tiles": chunk,
                       "chunks_in_flight": 2 if tiles_local > chunk else 1},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "fp32_issue", "kernel": "vit_fwd_cluster_kernel", "achieved": achieved / 1e12,
                         "peak": peak_ops / 1e12, "unit": "Tlane-op/s", "frac": achieved / peak_ops,
                         "peak_source": "%d SMs x 128 lanes x sm_max_mhz of MEASURED_PEAKS.json (%s)" % (sm_count, peak_src),
                         "ms_per_launch": kern_ms, "tiles_per_launch": nb,
                         "traffic": nb * NCU_DRAM_BYTES_PER_TILE_PASS,
                         "traffic_note": "DRAM bytes of a 240-sequence ncu capture scaled by sequences (lower bound)",
                         "frac_at_sampled_clock": (achieved / (sm_count * 128 * clocks["sm_mhz"] * 1e6)
                                                   if clocks and clocks.get("sm_mhz") else None)}}
    line.update(extras)
    if not args.no_extras and world == 1:
        Xs = synth.tile_sequences(synth.gaussian_matrix(256, 4096 * 16, 2))
        line["cpu_baseline"] = cpu_reference_rate(12.0, Xs, tl.view(np.uint16))
        try:
            line["reference_gpu"] = reference_gpu_rates(pkg, torch)
        except Exception as ex:
            line["reference_gpu"] = {"error": repr(ex)}
    print(json.dumps(line))
    finish(ctx)


def synthetic_block_ldl(n, torch, tokens=65536, rank_r=64, chunk=8192):
    """Strictly block-lower fp32 L of the rotated, damped Hessian of synthetic activations: X = Z + Zr C (Z, Zr N(0,1),
    C = N(0,1)/8, rank 64) in bf16, H = X^T X / tokens with fp32 accumulation, + 1e-2 mean(diag) I, two-sided
    hadUt with seeded SU signs (qtip_rotate_hessian), fp64 block LDL on the GPU (qtip_block_ldl; the reference does this
    step on the host in fp64). Returns (L, su, seconds per stage)."""
    import __graft_entry__ as graft
    pkg = graft.load_package()
    codec, synth = pkg.codec, pkg.synth
    t0 = time.perf_counter()
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    C = torch.randn(rank_r, n, generator=g, device="cuda") / 8.0
    H = torch.zeros((n, n), dtype=torch.float32, device="cuda")
    for _ in range(0, tokens, chunk):
        Xc = (torch.randn(chunk, n, generator=g, device="cuda") +
              torch.randn(chunk, rank_r, generator=g, device="cuda") @ C).to(torch.bfloat16).float()
        H.addmm_(Xc.T, Xc)
        del Xc
    H /= tokens
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    su = torch.from_numpy(synth.signs(n, 7)).cuda()
    HR, creg = codec.rotate_hessian_fused(H, su)
    del H
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    L = codec.block_ldl(HR)
    torch.cuda.synchronize()
    t3 = time.perf_counter()
    del HR
    return L, su, {"synthetic_hessian_s": t1 - t0, "rotate_hessian_s": t2 - t1, "block_ldl_s": t3 - t2}


def ldlq_section(ctx, shape, steps, warmup, reference_leg=True):
    """LDLQ + Viterbi of a down_proj-shaped matrix: weights N(0, 0.02), synthetic correlated Hessian, random-Hadamard
    rotation, 128-column buffers. Timed region: qtip_ldlq only (Hessian, rotation and block LDL reported beside it). Rows
    of W are split over the ranks (no collective); every rank builds the same L. On one GPU the reference's own GPU
    ldlq_gpu (compiled in place, test infrastructure) is timed on a row slice of the same problem beside ours."""
    torch, dist, pkg = ctx.torch, ctx.dist, ctx.pkg
    codec, synth = pkg.codec, pkg.synth
    rank, world, local = ctx.rank, ctx.world, ctx.local
    m, n = (int(v) for v in shape.split("x"))
    L, su, stages = synthetic_block_ldl(n, torch)
    lut_d, lut_rms = codec.device_lut(synth.seeded_tlut(1))
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    W = torch.randn(m, n, generator=g, device="cuda") * 0.02
    sv = torch.from_numpy(synth.signs(m, 8)).cuda()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    WT_full, wscale = codec.rotate_weight(W, su, sv, lut_rms)
    e1.record()
    torch.cuda.synchronize()
    t_rht = e0.elapsed_time(e1)
    del W
    b, e = pkg.sharding.tile_row_range(m // 16, rank, world)
    mj = (e - b) * 16
    WT = WT_full[:, 16 * b:16 * e].contiguous()
    hatWT = torch.empty_like(WT)
    Q = torch.empty(((mj // 16) * (n // 16), 128), dtype=torch.int16, device="cuda")
    ws = codec.ldlq_workspace(n, mj)
    times = []
    for i in range(warmup + steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        codec.ldlq_gpu(WT, L, n, mj, hatWT, Q, lut_d, workspace=ws)
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    ws.check()
    t = torch.tensor([sum(times) / len(times)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t)
    # invariants on this rank's codes: trellis links, tail-biting, decode(states) == hatWT tile by tile
    sd = Q.to(torch.int32) & 0xFFFF
    links = bool((((sd[:, :-1] << 4) & 0xFFFF) == (sd[:, 1:] & 0xFFF0)).all()) and \
        bool(((sd[:, 127] & 0xFFF) == (sd[:, 0] >> 4)).all())
    del sd
    nt = min(Q.shape[0], 4096)
    dec = torch.empty((nt, 256), dtype=torch.float32, device="cuda")
    codec.k_decode_states(Q[:nt].contiguous(), nt, dec, lut_d)
    perm = torch.from_numpy(synth.tile_perm()).cuda()
    nbk = n // 16
    tiles = hatWT.T.reshape(mj // 16, 16, nbk, 16).permute(0, 2, 1, 3).reshape(-1, 256)[:nt][:, perm]
    decode_ok = bool(torch.equal(dec, tiles))
    D = WT - hatWT
    rel_mse = float((D * D).sum(dtype=torch.float64) / (WT * WT).sum(dtype=torch.float64))
    del D, dec, tiles
    res = {"metric": "ldlq_viterbi_quantized_weights_per_second", "value": m * n / (ms * 1e-3),
           "unit": "weights/s", "n_gpus": world, "steps": steps, "warmup": warmup,
           "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic",
           "config": {"workload": "ldlq_viterbi_%dx%d" % (m, n), "column_steps": n // 16,
                      "sequences_per_step_per_rank": mj // 16, "buffers": n // 128},
           "roofline": ldlq_roofline(m, n, ms, world, torch, local),
           "stages_ms": dict(stages, weight_rht_ms=t_rht, ldlq_ms=ms),
           "checks": {"trellis_links_and_tail_biting": links, "decode_equals_hatW": decode_ok,
                      "relative_mse": rel_mse, "wscale": wscale}}
    if reference_leg and world == 1:
        try:
            res["reference_gpu"] = reference_ldlq(ctx, WT_full, L, n, m)
        except Exception as ex:
            res["reference_gpu"] = {"error": repr(ex)}
        try:
            res["cpu_baseline"] = cpu_ldlq(ctx, WT_full, L, lut_d)
        except Exception as ex:
            res["cpu_baseline"] = {"error": repr(ex)}
    return res


def cpu_ldlq(ctx, WT_full, L, lut_d, rows=256, cols=1024):
    """Reported CPU baseline of the LDLQ workload: the fp64 LDLQ of the reference's tests (tests/test_gpu.cpp:181-225,
    restated in the oracle: fp64 Viterbi per tile, OpenMP over the sequences of a column step) on the leading
    rows x cols corner of the same rotated matrix with the matching corner of L (the factor of the leading block of
    the Hessian), beside this library on the same corner. Test infrastructure, timed after the GPU numbers."""
    from oracle.oracle import Oracle
    torch, codec = ctx.torch, ctx.pkg.codec
    O = Oracle()
    WTc = WT_full[:cols, :rows].contiguous()
    Lc = L[:cols, :cols].contiguous()
    lut_h = lut_d.cpu().numpy().view(np.uint32)
    t0 = time.perf_counter()
    hat_c, _ = O.ldlq_ref(WTc.T.contiguous().cpu().numpy(), Lc.cpu().numpy(), lut_h)
    cpu_s = time.perf_counter() - t0
    hat = torch.empty_like(WTc)
    Q = torch.empty(((rows // 16) * (cols // 16), 128), dtype=torch.int16, device="cuda")
    ws = codec.ldlq_workspace(cols, rows)
    codec.ldlq_gpu(WTc, Lc, cols, rows, hat, Q, lut_d, workspace=ws)
    torch.cuda.synchronize()
    ws.check()
    den = float((WTc * WTc).sum(dtype=torch.float64))
    err_cpu = float(((WTc.T.cpu().double() - torch.from_numpy(hat_c).double()) ** 2).sum()) / den
    return {"kind": "port", "what": "fp64 LDLQ of the reference's tests, restated", "sample": "%d x %d corner" % (rows, cols),
            "cores": os.cpu_count(), "seconds": cpu_s, "value": rows * cols / cpu_s, "unit": "weights/s",
            "relative_mse_cpu": err_cpu, "relative_mse_ours_same_corner": float(((WTc - hat) ** 2).sum(dtype=torch.float64)) / den}


def reference_ldlq(ctx, WT_full, L, n, m, rows=1536):
    """The reference's own GPU ldlq_gpu (src/quantizer.cpp:30-89, compiled in place for sm_100a, test infrastructure) on
    the first `rows` rows of the same rotated matrix and the same L, beside this library's qtip_ldlq on that slice, both
    with the codebook compiled into the reference: seconds, proxy-style relative error, fraction of identical
    trellises. A row slice keeps the reference's run short; rows are independent, so the slice is a valid sub-problem."""
    from oracle.oracle import Reference, ReferenceQuant
    torch, pkg = ctx.torch, ctx.pkg
    codec = pkg.codec
    RQ, R = ReferenceQuant(), Reference()
    if not (RQ.available and R.available):
        return {"unavailable": "oracle/_ref holds no build of the reference's GPU quantizer"}
    rows = min(rows, m)
    lut_d, _ = codec.device_lut(R.codebook()[0])
    WT = WT_full[:, :rows].contiguous()
    hat, hat_r = torch.empty_like(WT), torch.empty_like(WT)
    Q, Q_r = (torch.empty(((rows // 16) * (n // 16), 128), dtype=torch.int16, device="cuda") for _ in range(2))
    ws = codec.ldlq_workspace(n, rows)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    codec.ldlq_gpu(WT, L, n, rows, hat, Q, lut_d, workspace=ws)  # warm-up
    torch.cuda.synchronize()
    e0.record()
    codec.ldlq_gpu(WT, L, n, rows, hat, Q, lut_d, workspace=ws)
    e1.record()
    torch.cuda.synchronize()
    ours_s = e0.elapsed_time(e1) * 1e-3
    ws.check()
    t0 = time.perf_counter()
    vit_s = RQ.ldlq_gpu(WT.data_ptr(), L.data_ptr(), n, rows, hat_r.data_ptr(), Q_r.data_ptr())
    torch.cuda.synchronize()
    ref_s = time.perf_counter() - t0
    den = float((WT * WT).sum(dtype=torch.float64))
    return {"kind": "the reference's ldlq_gpu recompiled for sm_100a, same GPU, same WT and L, its own codebook",
            "rows": rows, "n": n, "reference_s": ref_s, "reference_viterbi_s": vit_s, "ours_s": ours_s,
            "reference_weights_per_s": rows * n / ref_s, "ours_weights_per_s": rows * n / ours_s,
            "identical_trellis_fraction": float((Q == Q_r).all(dim=1).double().mean()),
            "relative_mse_ours": float(((WT - hat) ** 2).sum(dtype=torch.float64)) / den,
            "relative_mse_reference": float(((WT - hat_r) ** 2).sum(dtype=torch.float64)) / den}


def layer_section_tp(ctx):
    """The layer workload on N GPUs: every linear sharded by output rows (rotated-row tensor parallelism, contiguous
    32-row block-rows per rank), input transform on every rank, products of the shard, gather, output transform on every
    rank. <= 16 tokens: products pushed into every rank's gathered buffer by the product kernel (no collective call);
    64 / 256 tokens: fused decode + tcgen05 product of the shard, K-split partials summed, NCCL all-gather; 2048 tokens:
    dense decode + tcgen05 GEMM of the shard, NCCL all-gather. K/V (FP8): rows sharded, NCCL all-gather of the outputs.
    Time per layer = max over ranks, CUDA events (graph replay up to 256 tokens)."""
    torch, dist, pkg = ctx.torch, ctx.dist, ctx.pkg
    linear, synth, tp = pkg.linear, pkg.synth, pkg.tp
    rank, world = ctx.rank, ctx.world
    peaks, peak_src = measured_peaks()
    hidden, inter, kv = 12288, 28672, 1024
    shapes = {"q": (hidden, hidden), "o": (hidden, hidden), "gate": (hidden, inter), "up": (hidden, inter),
              "down": (inter, hidden)}
    lut = linear.runtime_lut(synth.seeded_tlut(1))
    g = torch.Generator(device="cuda")
    full, shard, row0 = {}, {}, {}
    for i, (name, (n_in, n_out)) in enumerate(shapes.items()):
        r0, rows = pkg.sharding.block_row_range(n_out, rank, world)
        su = torch.from_numpy(synth.signs(n_in, 7)).cuda()
        sv = torch.from_numpy(synth.signs(n_out, 8)).cuda()
        if name == "q":  # every rank makes the whole matrix: the sharded result is checked against the unsharded operator
            g.manual_seed(9)
            tr_full = torch.randint(-32768, 32768, ((n_out // 16) * (n_in // 16) * 32,), generator=g, device="cuda",
                                    dtype=torch.int16)
            q_full = linear.Matrix(tr_full, su, sv, lut, n_in, n_out)
            full[name], shard[name] = linear.Matrix(None, su, sv, None, n_in, n_out), q_full.rows(r0, rows)
        else:
            g.manual_seed(9 + i + 100 * rank)
            tr = torch.randint(-32768, 32768, ((rows // 16) * (n_in // 16) * 32,), generator=g, device="cuda",
                               dtype=torch.int16)
            full[name] = linear.Matrix(None, su, sv, None, n_in, n_out)
            shard[name] = linear.Matrix(tr, su, sv[r0:r0 + rows].contiguous(), lut, n_in, rows)
        row0[name] = r0
    kv_rows = kv // world
    g.manual_seed(11 + rank)
    w8 = [torch.randint(0, 255, (kv_rows, hidden), generator=g, device="cuda", dtype=torch.uint8) for _ in range(2)]
    for w in w8:
        w[(w & 127) == 127] = 0
    s8 = ((1 + torch.arange(kv_rows, device="cuda") % 7) / 4096.0).float()
    code_bytes = sum(a * b // 4 for a, b in shapes.values()) + 2 * kv * hidden
    weights = sum(a * b for a, b in shapes.values()) + 2 * kv * hidden
    dense = torch.empty((inter // world) * hidden, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ex = {n_out: tp.Exchange.from_process_group(n_out, max_tokens=16, max_splits=4) for n_out in (hidden, inter)}
    out = {}
    for T in (1, 16, 64, 256, 2048):
        g.manual_seed(10)
        xs = {n: torch.randn(T, n, generator=g, device="cuda").to(torch.bfloat16) for n in (hidden, inter)}
        rot = {n: torch.empty(T, n, dtype=torch.bfloat16, device="cuda") for n in (hidden, inter)}
        ys = {n: torch.empty(T, n, dtype=torch.bfloat16, device="cuda") for n in (hidden, inter)}
        y_q = torch.empty(T, hidden, dtype=torch.bfloat16, device="cuda")
        ykv_l = torch.empty(T, kv_rows, dtype=torch.bfloat16, device="cuda")
        ykv = torch.empty(world, T, kv_rows, dtype=torch.bfloat16, device="cuda")
        rows_max = inter // world
        z_l = torch.empty(4 * T * rows_max, dtype=torch.float32, device="cuda")
        z_g = torch.empty(world * T * rows_max, dtype=torch.float32, device="cuda")
        scratch = torch.empty(1, dtype=torch.float32, device="cuda")
        if 16 < T <= 512:
            splits = {name: max(1, min(4, -(-2 * 148 // (shard[name].n_out // 128)))) for name in shapes}
        else:
            splits = {name: (2 if T <= 16 else 1) for name in shapes}

        def layer():
            for name, (n_in, n_out) in shapes.items():
                w, ws, sp = full[name], shard[name], splits[name]
                rows = ws.n_out
                yo = y_q if name == "q" else ys[n_out]
                if T <= 16:
                    tp.forward_tp(ex[n_out], w, ws, row0[name], xs[n_in], yo, scratch, rot[n_in],
                                  name in ("gate", "up"), sp, T)
                    continue
                linear.qtip_prepare(ws, xs[n_in], scratch, rot[n_in], T)
                zl = z_l[:sp * T * rows]
                if T > 512:
                    linear.qtip_multiply_prefill(ws, rot[n_in], zl, rows, T, dense[:rows * n_in].view(rows, n_in), status)
                else:
                    linear.qtip_multiply_batch(ws, rot[n_in], zl, rows, sp, T)
                    linear.reduce_products(zl, T * rows, sp)
                zg = z_g[:world * T * rows]
                dist.all_gather_into_tensor(zg, zl[:T * rows])
                linear.qtip_finish(w, zg, yo, scratch, name in ("gate", "up"), 1, T, world)
            for w in w8:
                if T >= 8:
                    linear.fp8_forward_prefill(w, s8, xs[hidden], ykv_l, hidden, kv_rows, T, dense[:kv_rows * hidden], z_l)
                else:
                    linear.fp8_forward(w, s8, xs[hidden], ykv_l, hidden, kv_rows, T)
                dist.all_gather_into_tensor(ykv.view(-1), ykv_l.view(-1))

        # before timing: the sharded q projection against the unsharded operator on the same input (bf16 outputs)
        layer()
        torch.cuda.synchronize()
        check = _unsharded_reference(linear, q_full, xs[hidden], T, torch)
        q_err = float((y_q.float() - check.float()).norm() / check.float().norm())
        del check
        dist.barrier()
        us = _graph_us(layer, 2, torch) if T <= 512 else _time_us(layer, 3, torch)
        t = torch.tensor([us], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t)
        flops = 2.0 * T * weights
        out["T%d" % T] = {"layer_us": us, "code_gbs": code_bytes / us / 1e3, "tflops": flops / us / 1e6,
                          "frac_of_hbm_peak": code_bytes / us / 1e3 / (world * peaks["hbm_gbs"]),
                          "frac_of_bf16_peak": flops / us / 1e6 / (world * peaks["bf16_tflops"]),
                          "q_rel_l2_vs_unsharded_operator": q_err}
        del xs, rot, ys, z_l, z_g
    for e in ex.values():
        e.check()
    assert int(status) == 0
    linear.kernel_status()
    dist.barrier()
    for e in ex.values():
        e.close()
    return {"metric": "qtip_layer_products", "unit": "us per layer", "n_gpus": world, "data": "synthetic",
            "config": {"workload": "mistral_large_layer_products", "hidden": hidden, "intermediate": inter,
                       "code_bytes": code_bytes, "weights": weights, "peaks": peak_src,
                       "parallelism": "rotated-row tensor parallel x%d" % world}, "tokens": out}


def _unsharded_reference(linear, w, x, T, torch):
    """y = operator(w, x) for T tokens through the unsharded entry points with one K-split (the yard-stick the sharded
    and the batched paths of the layer workload are compared with before they are timed)."""
    n_in, n_out = w.n_in, w.n_out
    rot = torch.empty(T, n_in, dtype=torch.bfloat16, device="cuda")
    z = torch.empty(T, n_out, dtype=torch.float32, device="cuda")
    y = torch.empty(T, n_out, dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(1, dtype=torch.float32, device="cuda")
    linear.qtip_prepare(w, x, scratch, rot, T)
    for t0 in range(0, T, 16):  # the 16-tokens-per-pass register kernel: the simplest product path
        t1 = min(T, t0 + 16)
        linear.qtip_multiply_batch(w, rot[t0:t1], z[t0:t1], n_out, 1, t1 - t0, implementation=0)
    linear.qtip_finish(w, z, y, scratch, False, 1, T)
    return y


def ldlq_roofline(m, n, ms, world, torch, local):
    """The whole LDLQ + Viterbi section against the FP32-issue peak of the GPUs used (327,680 lane-ops per weight)."""
    peaks, peak_src = measured_peaks()
    sm_count = torch.cuda.get_device_properties(local).multi_processor_count
    peak = world * sm_count * 128 * peaks.get("sm_max_mhz", 1965.0) * 1e6
    achieved = m * n * LANE_OPS_PER_WEIGHT / (ms * 1e-3)
    return {"bound": "fp32_issue", "achieved": achieved / 1e12, "peak": peak / 1e12, "unit": "Tlane-op/s",
            "frac": achieved / peak, "peak_source": "%d GPU(s) x %d SMs x 128 lanes x sm_max_mhz (%s)" % (world, sm_count, peak_src)}


def layer_section(ctx):
    """Decode/prefill products of one Mistral-Large-shaped layer (hidden 12288, intermediate 28672, 96 Q / 8 KV heads of
    128): q, o, gate, up, down as 2-bit QTIP linears with random codes, k, v as FP8 e4m3, bf16 activations N(0,1), token
    batches 1, 16, 64, 256 and 2048. Each linear runs input transform, product, output transform. <= 16 tokens:
    MMA-fragment kernel; 64 and 256 tokens: decode fused into the tcgen05 product (HBM-side metric: code bytes per
    second); 2048 tokens: dense decode + tcgen05 GEMM (TFLOP/s). One GPU."""
    if ctx.world > 1:
        return layer_section_tp(ctx)
    torch, pkg = ctx.torch, ctx.pkg
    linear, synth = pkg.linear, pkg.synth
    peaks, peak_src = measured_peaks()
    hidden, inter, kv = 12288, 28672, 1024
    shapes = {"q": (hidden, hidden), "o": (hidden, hidden), "gate": (hidden, inter), "up": (hidden, inter),
              "down": (inter, hidden)}
    lut = linear.runtime_lut(synth.seeded_tlut(1))
    g = torch.Generator(device="cuda")
    mats = {}
    for i, (name, (n_in, n_out)) in enumerate(shapes.items()):
        g.manual_seed(9 + i)
        tr = torch.randint(-32768, 32768, ((n_out // 16) * (n_in // 16) * 32,), generator=g, device="cuda", dtype=torch.int16)
        mats[name] = linear.Matrix(tr, torch.from_numpy(synth.signs(n_in, 7)).cuda(),
                                   torch.from_numpy(synth.signs(n_out, 8)).cuda(), lut, n_in, n_out)
    g.manual_seed(11)
    w8 = [torch.randint(0, 255, (kv, hidden), generator=g, device="cuda", dtype=torch.uint8) for _ in range(2)]
    for w in w8:
        w[(w & 127) == 127] = 0
    s8 = ((1 + torch.arange(kv, device="cuda") % 7) / 4096.0).float()
    code_bytes = sum(a * b // 4 for a, b in shapes.values()) + 2 * kv * hidden
    weights = sum(a * b for a, b in shapes.values()) + 2 * kv * hidden
    dense = torch.empty(inter * hidden, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = {}
    for T in (1, 16, 64, 256, 2048):
        g.manual_seed(10)
        xs = {n: torch.randn(T, n, generator=g, device="cuda").to(torch.bfloat16) for n in (hidden, inter)}
        rot = {n: torch.empty(T, n, dtype=torch.bfloat16, device="cuda") for n in (hidden, inter)}
        ys = {n: torch.empty(T, n, dtype=torch.bfloat16, device="cuda") for n in (hidden, inter, kv)}
        splits = {}
        for name, (n_in, n_out) in shapes.items():
            if T <= 512 and linear.batch_uses_tc(n_in, n_out, T):
                splits[name] = linear.tc_splits(n_out)
            else:
                splits[name] = 2 if (T <= 16 and n_out == hidden) else 1
        z = torch.empty(4 * T * inter if T <= 512 else T * inter, dtype=torch.float32, device="cuda")
        scratch = torch.empty(1, dtype=torch.float32, device="cuda")

        def layer():
            for name, (n_in, n_out) in shapes.items():
                w, sp = mats[name], splits[name]
                linear.qtip_prepare(w, xs[n_in], scratch, rot[n_in], T)
                if T > 512:
                    linear.qtip_multiply_prefill(w, rot[n_in], z, n_out, T, dense[:n_out * n_in].view(n_out, n_in), status)
                elif T == 1:
                    linear.qtip_multiply(w, rot[n_in], z, n_out, sp, 1)
                else:
                    linear.qtip_multiply_batch(w, rot[n_in], z, n_out, sp, T)
                linear.qtip_finish(w, z, ys[n_out], scratch, name in ("gate", "up"), sp, T)
            for w in w8:
                if T >= 8:  # tensor cores with the K range split over the SMs; below that the streaming SIMT kernel
                    linear.fp8_forward_prefill(w, s8, xs[hidden], ys[kv], hidden, kv, T, dense[:kv * hidden], z)
                else:
                    linear.fp8_forward(w, s8, xs[hidden], ys[kv], hidden, kv, T)

        # before timing: the q projection of this batch size against the simplest product path on the same input
        w, sp = mats["q"], splits["q"]
        linear.qtip_prepare(w, xs[hidden], scratch, rot[hidden], T)
        if T > 512:
            linear.qtip_multiply_prefill(w, rot[hidden], z, hidden, T, dense[:hidden * hidden].view(hidden, hidden), status)
        elif T == 1:
            linear.qtip_multiply(w, rot[hidden], z, hidden, sp, 1)
        else:
            linear.qtip_multiply_batch(w, rot[hidden], z, hidden, sp, T)
        linear.qtip_finish(w, z, ys[hidden], scratch, False, sp, T)
        check = _unsharded_reference(linear, w, xs[hidden], T, torch)
        q_err = float((ys[hidden].float() - check.float()).norm() / check.float().norm())
        del check
        # Prefill-sized batches run at the power cap and the clock sags over the first seconds of load: both schedules
        # are timed twice, alternating, and the faster pass of each is kept, so that the two numbers see the same clocks.
        timed = (lambda: _graph_us(layer, 2, torch)) if T <= 512 else (lambda: _time_us(layer, 3, torch))
        saved, us, lin_us = w8[:], float("inf"), float("inf")
        if T > 512:
            timed()  # discarded: brings the GPU to the clocks it holds under this load
        for _ in range(1 if T <= 512 else 2):
            us = min(us, timed())
            del w8[:]  # the same schedule without the FP8 K/V projections: the number the reference leg is compared with
            lin_us = min(lin_us, timed())
            w8.extend(saved)
        flops = 2.0 * T * weights
        out["T%d" % T] = {"layer_us": us, "linears_us": lin_us, "code_gbs": code_bytes / us / 1e3,
                          "tflops": flops / us / 1e6,
                          "frac_of_hbm_peak": code_bytes / us / 1e3 / peaks["hbm_gbs"],
                          "frac_of_bf16_peak": flops / us / 1e6 / peaks["bf16_tflops"],
                          "q_rel_l2_vs_register_kernel": q_err}
        del xs, rot, ys, z
    assert int(status) == 0
    linear.kernel_status()
    res = {"metric": "qtip_layer_products", "unit": "us per layer", "n_gpus": 1, "data": "synthetic",
           "config": {"workload": "mistral_large_layer_products", "hidden": hidden, "intermediate": inter,
                      "code_bytes": code_bytes, "weights": weights, "peaks": peak_src}, "tokens": out}
    try:
        res["decode_step_fused"] = decode_step_fused(ctx, mats, w8, s8)
    except Exception as ex:
        res["decode_step_fused"] = {"error": repr(ex)}
    try:
        res["reference_gpu"] = reference_layer(ctx, mats, w8, s8)
    except Exception as ex:
        res["reference_gpu"] = {"error": repr(ex)}
    return res


def decode_step_fused(ctx, mats, w8, s8):
    """The same layer as a decode step with the fused epilogues, at 1 and 16 tokens: RMSNorm + input transform (the
    normalised row also feeds the FP8 K/V projections), q; o with the residual add and the next RMSNorm + input transform
    in its epilogue; gate and up as ONE product over the stacked 57,344-row matrix with SiLU(gate) * up in its epilogue;
    down with the residual add. Besides the products of `layer_us` this does both norms, both residual adds and the
    activation (the attention between q/k/v and o is outside the path: o reads a stand-in input). CUDA-graph replay."""
    torch, pkg = ctx.torch, ctx.pkg
    linear = pkg.linear
    hidden, inter, kv, eps = 12288, 28672, 1024, 1e-5
    q, o, gate, up, down = (mats[k] for k in ("q", "o", "gate", "up", "down"))
    gu = linear.Matrix(torch.cat([gate.trellis, up.trellis]), gate.su, torch.cat([gate.sv, up.sv]), gate.lut, hidden, 2 * inter)
    g = torch.Generator(device="cuda")
    g.manual_seed(21)
    out = {}
    for T in (1, 16):
        bf = lambda *shape: (0.05 * torch.randn(*shape, generator=g, device="cuda")).to(torch.bfloat16)  # noqa: E731
        state, attn = bf(T, hidden), bf(T, hidden)
        norm1, norm2 = ((1.0 + bf(hidden).float()).to(torch.bfloat16) for _ in range(2))
        u_h, xn, u_o, y_q = (torch.empty(T, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(4))
        h, u_d = (torch.empty(T, inter, dtype=torch.bfloat16, device="cuda") for _ in range(2))
        y_kv = torch.empty(T, kv, dtype=torch.bfloat16, device="cuda")
        # K-splits as in the unfused schedule: the tensor-core kernel's own choice where the batch takes it, else two for
        # the 12,288-row products and one for the wide one
        sp = {w: (linear.tc_splits(w.n_out) if T > 1 and linear.batch_uses_tc(w.n_in, w.n_out, T) else
                  (2 if w.n_out == hidden else 1)) for w in (q, o, gu, down)}
        z_h = torch.empty(max(sp[q], sp[o], sp[down]) * T * hidden, dtype=torch.float32, device="cuda")
        z_gu = torch.empty(sp[gu] * T * 2 * inter, dtype=torch.float32, device="cuda")
        scratch = torch.empty(1, dtype=torch.float32, device="cuda")
        sv_h_scaled = (q.sv * 1e-3).contiguous()  # keeps the residual stream finite over the replays

        def product(w, x, z):
            if T == 1:
                linear.qtip_multiply(w, x, z, w.n_out, sp[w], 1)
            else:
                linear.qtip_multiply_batch(w, x, z, w.n_out, sp[w], T)

        def step():
            linear.input_transform(state, norm1, eps, q.su, hidden, T, u_h, xn)
            product(q, u_h, z_h)
            linear.qtip_finish(q, z_h, y_q, scratch, False, sp[q], T)
            for w in w8:
                linear.fp8_forward(w, s8, xn, y_kv, hidden, kv, T)
            linear.qtip_prepare(o, attn, scratch, u_o, T)
            product(o, u_o, z_h)
            linear.output_residual_input(z_h, sp[o], T, sv_h_scaled, hidden, state, norm2, eps, gate.su, u_h)
            product(gu, u_h, z_gu)
            linear.output_gateup(z_gu, sp[gu], T, gate.sv, up.sv, inter, h)
            linear.qtip_prepare(down, h, scratch, u_d, T)
            product(down, u_d, z_h)
            linear.output_residual(z_h, sp[down], T, sv_h_scaled, hidden, state)

        # the same step from the unfused operator stages, with the element-wise work as library kernels (one RMSNorm
        # kernel, one add, SiLU and multiply), gate and up as two products: what a runtime without the epilogues launches
        F = torch.nn.functional
        y_h, y_g, y_u = y_q, torch.empty_like(h), torch.empty_like(h)
        z_g = torch.empty(max(sp[gu], 1) * T * inter, dtype=torch.float32, device="cuda")
        spl = {w: (linear.tc_splits(w.n_out) if T > 1 and linear.batch_uses_tc(w.n_in, w.n_out, T) else 1) for w in (gate, up)}

        def product2(w, x, z):
            if T == 1:
                linear.qtip_multiply(w, x, z, w.n_out, spl[w], 1)
            else:
                linear.qtip_multiply_batch(w, x, z, w.n_out, spl[w], T)

        def step_unfused():
            xn.copy_(F.rms_norm(state, (hidden,), norm1, eps))
            linear.qtip_prepare(q, xn, scratch, u_h, T)
            product(q, u_h, z_h)
            linear.qtip_finish(q, z_h, y_q, scratch, False, sp[q], T)
            for w in w8:
                linear.fp8_forward(w, s8, xn, y_kv, hidden, kv, T)
            linear.qtip_prepare(o, attn, scratch, u_o, T)
            product(o, u_o, z_h)
            linear.qtip_finish(o, z_h, y_h, scratch, False, sp[o], T)
            state.add_(y_h, alpha=1e-3)
            xn.copy_(F.rms_norm(state, (hidden,), norm2, eps))
            linear.qtip_prepare(gate, xn, scratch, u_h, T)
            product2(gate, u_h, z_g)
            linear.qtip_finish(gate, z_g, y_g, scratch, True, spl[gate], T)
            product2(up, u_h, z_g)
            linear.qtip_finish(up, z_g, y_u, scratch, True, spl[up], T)
            torch.mul(F.silu(y_g), y_u, out=h)
            linear.qtip_prepare(down, h, scratch, u_d, T)
            product(down, u_d, z_h)
            linear.qtip_finish(down, z_h, y_h, scratch, False, sp[down], T)
            state.add_(y_h, alpha=1e-3)

        fused_us = _graph_us(step, 2, torch)
        ok = bool(torch.isfinite(state.float()).all()) and bool(torch.isfinite(h.float()).all())
        out["T%d" % T] = {"step_us": fused_us, "unfused_step_us": _graph_us(step_unfused, 2, torch), "finite": ok}
        del y_g, y_u, z_g
        del state, attn, u_h, xn, u_o, y_q, h, u_d, z_h, z_gu
    out["what"] = ("RMSNorm + input transform, q, FP8 k / v, o + residual + next norm and input transform, stacked "
                   "gate|up + SiLU * up, down + residual; unfused_step_us: the same work from the operator's three stages with "
                   "library kernels for norm, add and activation; layer_us above times the bare products")
    return out



def reference_layer(ctx, mats, w8, s8):
    """The reference's own CUDA kernels (runtime/cuda/kernels.cu, batch_kernels.cu, recompiled for sm_100a; test
    infrastructure) on the five QTIP linears of the same layer, same codes and inputs: input transform + products +
    output transform per linear at 1, 16, 64 and 2,048 tokens. 1 token: qtip_forward, best of its K-splits; 16 / 64:
    qtip_multiply_batch; 2,048: its >= 128-token path, qtip_decode_matrix followed by the library GEMM it calls
    (bf16 x bf16 -> fp32, here through torch.mm). CUDA-graph replays on the current stream."""
    from oracle.oracle import ReferenceGpu
    torch, pkg = ctx.torch, ctx.pkg
    R = ReferenceGpu()
    if not R.available:
        return {"unavailable": "oracle/_ref holds no build of the reference's CUDA kernels"}
    R.initialize_tables()
    p = lambda t: t.data_ptr()  # noqa: E731
    st = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    hidden, inter = 12288, 28672
    g = torch.Generator(device="cuda")
    dense = torch.empty(inter * hidden, dtype=torch.bfloat16, device="cuda")
    out = {}
    for T in (1, 16, 64, 2048):
        g.manual_seed(10)
        xs = {n: torch.randn(T, n, generator=g, device="cuda").to(torch.bfloat16) for n in (hidden, inter)}
        rot = {n: torch.empty(T, n, dtype=torch.bfloat16, device="cuda") for n in (hidden, inter)}
        ys = {n: torch.empty(T, n, dtype=torch.bfloat16, device="cuda") for n in (hidden, inter)}
        scratch = torch.empty(T * inter, dtype=torch.float32, device="cuda")
        z = torch.empty(8 * T * inter if T <= 64 else T * inter, dtype=torch.float32, device="cuda")

        def one(name, splits):
            w = mats[name]
            wr = (p(w.trellis), p(w.su), p(w.sv), p(w.lut), w.n_in, w.n_out)
            x, r, y = xs[w.n_in], rot[w.n_in], ys[w.n_out]
            rz = name in ("gate", "up")
            if T == 1:
                R.qtip_forward(wr, p(x), p(y), p(scratch), p(r), p(z), rz, splits, stream=st())
                return
            R.qtip_prepare(wr, p(x), p(scratch), p(r), T, stream=st())
            if T <= 64:
                R.qtip_multiply_batch(wr, p(r), p(z), w.n_out, splits, T, stream=st())
            else:
                d = dense[:w.n_out * w.n_in].view(w.n_out, w.n_in)
                R.qtip_decode_matrix(wr, p(d), stream=st())
                zz = torch.mm(r, d.T, out_dtype=torch.float32)  # the library GEMM of the reference's >= 128-token path
                R.qtip_finish(wr, p(zz), p(y), p(scratch), rz, 1, T, stream=st())
                return
            R.qtip_finish(wr, p(z), p(y), p(scratch), rz, splits, T, stream=st())

        total, per = 0.0, {}
        for name in mats:
            best = None
            for splits in ((1, 2, 4, 8) if T <= 64 else (1,)):
                us = _graph_us(lambda: one(name, splits), 2, torch) if T <= 64 else _time_us(lambda: one(name, splits), 3, torch)
                if best is None or us < best[0]:
                    best = (us, splits)
            per[name] = {"us": best[0], "splits": best[1]}
            total += best[0]
        out["T%d" % T] = {"linears_us": total, "per_linear": per}
        del xs, rot, ys, scratch, z
    out["kind"] = "the reference's CUDA kernels recompiled for sm_100a, same GPU, same codes; QTIP linears only (no FP8 K/V)"
    try:
        out["cpu_q_proj_16_tokens"] = cpu_q_proj(ctx, mats["q"])
    except Exception as ex:
        out["cpu_q_proj_16_tokens"] = {"error": repr(ex)}
    return out


def cpu_q_proj(ctx, w, tokens=16):
    """Reported CPU baseline of the batched products: the reference's CPU reference_forward (runtime/src/qtip.cpp:129-192,
    compiled in place, OpenMP, double accumulation, device rounding) on the q projection at 16 tokens, beside this
    library's operator on the same input. Test infrastructure."""
    from oracle.oracle import Oracle, Reference
    torch, pkg = ctx.torch, ctx.pkg
    linear, synth = pkg.linear, pkg.synth
    R = Reference()
    fwd, kind = (R.reference_forward, "reference") if R.available else (Oracle().reference_forward, "port")
    g = torch.Generator(device="cuda")
    g.manual_seed(16)
    x = torch.randn(tokens, w.n_in, generator=g, device="cuda").to(torch.bfloat16)
    t0 = time.perf_counter()
    out = fwd(w.trellis.cpu().numpy().view(np.uint16), w.su.cpu().numpy(), w.sv.cpu().numpy(),
              synth.seeded_tlut(1).view(np.uint16), w.n_in, w.n_out, x.float().cpu().numpy(), True, False)
    dt = time.perf_counter() - t0
    yc = np.asarray(out[0] if isinstance(out, tuple) else out, dtype=np.float64).reshape(tokens, w.n_out)
    ours = _unsharded_reference(linear, w, x, tokens, torch).float().cpu().numpy().astype(np.float64)
    return {"kind": kind, "cores": len(os.sched_getaffinity(0)), "seconds": dt, "tokens": tokens,
            "rel_l2_of_this_library": float(np.linalg.norm(ours - yc) / np.linalg.norm(yc))}


def kernel_workload(args):
    """A few launches of one kernel of the path on a small fixed case, timed with CUDA events: the command a profiler
    capture wraps (one kernel, few launches before it, a few hundred MB on the device at most).
        --kernel viterbi --size <sequences>                          forward pass of the cluster Viterbi kernel
        --kernel gemv    --size <out rows> [--splits s]              qtip_multiply, one token, <out rows> x 12288
        --kernel fused   --size <out rows> [--tokens t] [--splits s] qtip_multiply_tc
        --kernel prefill --size <out rows> [--tokens t]              qtip_prefill_gemm on a dense bf16 matrix"""
    import torch
    import __graft_entry__ as graft
    pkg = graft.load_package()
    codec, linear, synth = pkg.codec, pkg.linear, pkg.synth
    torch.cuda.set_device(0)
    codec.init()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(9)
    size, n_in = args.size, 12288
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def qtip_linear(n_out):
        trellis = torch.randint(-32768, 32768, ((n_out // 16) * (n_in // 16) * 32,), generator=gen, device="cuda",
                                dtype=torch.int16)
        su, sv = torch.from_numpy(synth.signs(n_in, 7)).cuda(), torch.from_numpy(synth.signs(n_out, 8)).cuda()
        return linear.Matrix(trellis, su, sv, linear.runtime_lut(synth.seeded_tlut(1)), n_in, n_out)

    if args.kernel == "epilogue":
        return print(json.dumps(epilogue_timings(torch, pkg, args.tokens or 64)))
    if args.kernel == "viterbi":
        lut_d, _ = codec.device_lut(synth.seeded_tlut(1))
        X = torch.randn(size, 256, generator=gen, device="cuda")
        bp = torch.empty((size, 16, 4096), dtype=torch.int32, device="cuda")
        fs = torch.empty(size, dtype=torch.int16, device="cuda")
        fn = lambda: codec.k_viterbi_fwd_words(X, None, 1, size, bp, 0, fs, lut_d, status)  # noqa: E731
    elif args.kernel == "prefill":
        tokens = args.tokens or 2048
        wd = torch.randn(size, n_in, generator=gen, device="cuda").to(torch.bfloat16)
        x = torch.randn(tokens, n_in, generator=gen, device="cuda").to(torch.bfloat16)
        z = torch.empty((tokens, size), dtype=torch.float32, device="cuda")
        fn = lambda: linear.prefill_gemm(wd, x, z, size, n_in, size, tokens, status)  # noqa: E731
    elif args.kernel == "fused":
        tokens = args.tokens or 64
        w = qtip_linear(size)
        x = torch.randn(tokens, n_in, generator=gen, device="cuda").to(torch.bfloat16)
        z = torch.empty((args.splits, tokens, size), dtype=torch.float32, device="cuda")
        fn = lambda: linear.qtip_multiply_tc(w, x, z, size, args.splits, tokens, status)  # noqa: E731
    else:
        w = qtip_linear(size)
        rot = torch.randn(n_in, generator=gen, device="cuda").to(torch.bfloat16)
        z = torch.empty((args.splits, size), dtype=torch.float32, device="cuda")
        fn = lambda: linear.qtip_multiply(w, rot, z, size, args.splits, 1)  # noqa: E731
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        fn()
    e1.record()
    torch.cuda.synchronize()
    assert int(status) == 0, "a bounded wait ran out"
    linear.kernel_status()
    print(json.dumps({"workload": "kernel", "kernel": args.kernel, "size": size, "tokens": args.tokens,
                      "splits": args.splits, "us_per_launch": e0.elapsed_time(e1) * 1e3 / 3}))


def epilogue_timings(torch, pkg, rows):
    """GPU time (CUDA-graph replay) of the fused decode-step epilogues beside the unfused stages they replace, at the
    layer's widths (hidden 12288, intermediate 28672) for `rows` tokens."""
    linear, synth = pkg.linear, pkg.synth
    hidden, inter = 12288, 28672
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    bf = lambda *shape: torch.randn(*shape, generator=g, device="cuda").to(torch.bfloat16)  # noqa: E731
    su_h, su_i = (torch.from_numpy(synth.signs(n, 7)).cuda() for n in (hidden, inter))
    sv_h, sv_i = (torch.from_numpy(synth.signs(n, 8)).cuda() * 0.02 for n in (hidden, inter))
    norm = (1.0 + 0.1 * bf(hidden).float()).to(torch.bfloat16)
    x, state = bf(rows, hidden), bf(rows, hidden)
    u, xn, y = (torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(3))
    z_h = torch.randn(1, rows, hidden, generator=g, device="cuda")
    z_gu = torch.randn(1, rows, 2 * inter, generator=g, device="cuda")
    z_g, z_u = z_gu[0, :, :inter].contiguous(), z_gu[0, :, inter:].contiguous()
    h, yg, yu = (torch.empty(rows, inter, dtype=torch.bfloat16, device="cuda") for _ in range(3))
    scratch = torch.empty(1, device="cuda")
    w_h = linear.Matrix(None, su_h, sv_h, None, hidden, hidden)
    w_i = linear.Matrix(None, su_i, sv_i, None, inter, inter)

    def unfused_gateup():
        linear.qtip_finish(w_i, z_g, yg, scratch, True, 1, rows)
        linear.qtip_finish(w_i, z_u, yu, scratch, True, 1, rows)
        gf = yg.float()
        torch.mul(gf / (1.0 + torch.exp(-gf)), yu.float(), out=gf)
        h.copy_(gf)

    def unfused_residual_input():
        linear.qtip_finish(w_h, z_h, y, scratch, False, 1, rows)
        state.add_(y)
        xf = state.float()
        xn.copy_(xf * torch.rsqrt((xf * xf).mean(dim=1, keepdim=True) + 1e-5) * norm.float())
        linear.qtip_prepare(w_h, xn, scratch, u, rows)

    t = lambda fn: _graph_us(fn, 4, torch)  # noqa: E731
    return {"workload": "kernel", "kernel": "epilogue", "rows": rows,
            "input_transform_with_norm_us": t(lambda: linear.input_transform(x, norm, 1e-5, su_h, hidden, rows, u, xn)),
            "prepare_alone_us": t(lambda: linear.qtip_prepare(w_h, x, scratch, u, rows)),
            "output_residual_us": t(lambda: linear.output_residual(z_h, 1, rows, sv_h, hidden, state)),
            "finish_alone_us": t(lambda: linear.qtip_finish(w_h, z_h, y, scratch, False, 1, rows)),
            "output_residual_input_us": t(lambda: linear.output_residual_input(z_h, 1, rows, sv_h, hidden, state, norm,
                                                                                1e-5, su_h, u, xn)),
            "finish_add_norm_prepare_unfused_us": t(unfused_residual_input),
            "output_gateup_us": t(lambda: linear.output_gateup(z_gu, 1, rows, sv_i, sv_i, inter, h)),
            "two_finishes_and_silu_unfused_us": t(unfused_gateup)}


def _time_us(fn, iters, torch):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def _graph_us(fn, reps, torch):
    """GPU time of one fn() with the launches replayed from a CUDA graph (no host launch overhead in the number)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    return _time_us(g.replay, 5, torch) / reps


def gemv_section(pkg, peaks, peak_src, rank, world):
    """Batch-1 trellis-decode GEMV y = W x for a 57344 x 12288 2-bit weight. One GPU: the multiply kernel alone and the
    whole operator (input transform + multiply + output transform), as achieved HBM GB/s on the algorithmic bytes.
    N GPUs: rotated-row tensor parallelism, each rank multiplies its contiguous block-rows, NCCL all-gather of z,
    output transform on every rank; time = max over ranks."""
    import torch
    import torch.distributed as dist
    linear, synth = pkg.linear, pkg.synth
    n_in, n_out = 12288, 57344
    row0, rows = pkg.sharding.block_row_range(n_out, rank, world)
    g = torch.Generator(device="cuda")
    g.manual_seed(9 + rank)
    trellis = torch.randint(-32768, 32768, ((rows // 16) * (n_in // 16) * 32,), generator=g, device="cuda",
                            dtype=torch.int16)
    su = torch.from_numpy(synth.signs(n_in, 7)).cuda()
    sv = torch.from_numpy(synth.signs(n_out, 8)).cuda()
    lut = linear.runtime_lut(synth.seeded_tlut(1))
    shard = linear.Matrix(trellis, su, sv[row0:row0 + rows].contiguous(), lut, n_in, rows)
    g.manual_seed(10)
    x = torch.randn(n_in, generator=g, device="cuda").to(torch.bfloat16)
    y = torch.empty(n_out, dtype=torch.bfloat16, device="cuda")
    rot = torch.empty(n_in, dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(n_out, dtype=torch.float32, device="cuda")
    algo_bytes = n_out * n_in // 4 + 2 * n_in + 4 * n_out + 4096
    res = {"algorithmic_bytes": algo_bytes, "peak_gbs": peaks["hbm_gbs"], "peak_source": peak_src, "n_gpus": world,
           "timing": "CUDA events; 176 MB of codes per call exceed the L2, so no flush between calls"}
    if world == 1:
        best = None
        for splits in (1, 2, 3, 4):
            z = torch.empty((splits, n_out), dtype=torch.float32, device="cuda")
            linear.qtip_prepare(shard, x, scratch, rot)
            us = _time_us(lambda: linear.qtip_multiply(shard, rot, z, n_out, splits), 20, torch)
            fus = _graph_us(lambda: linear.qtip_forward(shard, x, y, scratch, rot, z, False, splits), 10, torch)
            res["splits_%d" % splits] = {"multiply_us": us, "forward_us": fus}
            if best is None or fus < best[2]:
                best = (splits, us, fus)
        res.update({"best_splits": best[0], "multiply_us": best[1], "forward_us": best[2],
                    "multiply_gbs": algo_bytes / best[1] / 1e3, "forward_gbs": algo_bytes / best[2] / 1e3,
                    "multiply_frac_of_peak": algo_bytes / best[1] / 1e3 / peaks["hbm_gbs"],
                    "forward_frac_of_peak": algo_bytes / best[2] / 1e3 / peaks["hbm_gbs"],
                    "forward_timing": "CUDA graph replay of prepare + multiply + finish"})
        return res
    full = linear.Matrix(None, su, sv, None, n_in, n_out)  # the output transform needs the geometry and SV only
    z_local = torch.empty(rows, dtype=torch.float32, device="cuda")
    z_full = torch.empty(n_out, dtype=torch.float32, device="cuda")
    # A rank's shard (176 MB / N) fits the 126 MB L2 from N = 2 on, so a replay of ONE shard would time the L2, not HBM.
    # The timed loops therefore walk over `copies` identical copies of the shard (together more than twice the L2), one
    # per projection: every projection streams its codes from HBM ("cold"). The single-copy replay is reported beside it
    # ("warm") because a decode step that re-reads a resident shard is a real case too.
    shard_bytes = trellis.numel() * 2
    copies = max(2, -(-(2 * 126 << 20) // shard_bytes) + 1)
    shards = [shard] + [linear.Matrix(trellis.clone(), su, shard.sv, lut, n_in, rows) for _ in range(copies - 1)]
    reps = 2 * copies if (2 * copies) % 2 == 0 else 2 * copies + 1
    turn = [0]

    def next_shard(cold):
        if not cold:
            return shard
        turn[0] = (turn[0] + 1) % copies
        return shards[turn[0]]

    def forward_tp(cold=True):
        sh = next_shard(cold)
        linear.qtip_prepare(sh, x, scratch, rot)
        linear.qtip_multiply(sh, rot, z_local, rows, 1)
        dist.all_gather_into_tensor(z_full, z_local)
        linear.qtip_finish(full, z_full, y, scratch, False, 1)

    # The same projection with the gather fused into the product kernel: every rank's kernel stores its products into
    # every rank's gathered buffer over NVLink (plain peer stores), the last CTA waits for the peers' flags.
    ex = pkg.tp.Exchange.from_process_group(n_out, max_tokens=1, max_splits=4)
    y_nccl = torch.empty_like(y)
    fused_splits = [1]

    def forward_fused(cold=True):
        pkg.tp.forward_tp(ex, full, next_shard(cold), row0, x, y, scratch, rot, False, fused_splits[0])

    forward_tp()
    y_nccl.copy_(y)
    forward_fused()
    ex.check()
    same = bool(torch.equal(y.view(torch.int16), y_nccl.view(torch.int16)))
    # Both variants are replayed from CUDA graphs of `reps` projections (an even count: the fused exchange alternates its
    # two slots), so that the numbers hold GPU time and not the host's launch rate.

    def timed(fn, cold):
        dist.barrier()
        v = torch.tensor([_graph_us(lambda: fn(cold), reps, torch)], device="cuda", dtype=torch.float64)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v[0])

    try:
        fus = timed(forward_tp, True)
        fus_warm = timed(forward_tp, False)
        nccl_timing = "CUDA graph replay"
    except Exception:  # a library that refuses capture: fall back to eager launches
        torch.cuda.synchronize()
        dist.barrier()
        fus = _time_us(lambda: forward_tp(True), 50, torch)
        fus_warm = _time_us(lambda: forward_tp(False), 50, torch)
        nccl_timing = "eager launches"
    sweep, sweep_warm = {}, {}
    for sp in (1, 2, 3, 4):  # K-splits give a small shard more work items than SMs; the output transform adds the partials
        fused_splits[0] = sp
        sweep["splits_%d" % sp] = timed(forward_fused, True)
        sweep_warm["splits_%d" % sp] = timed(forward_fused, False)
    ex.check()
    dist.barrier()

    def multiply_only(cold):
        linear.qtip_multiply(next_shard(cold), rot, z_local, rows, 1)

    mus = _graph_us(lambda: multiply_only(True), reps, torch)
    mus_warm = _graph_us(lambda: multiply_only(False), reps, torch)
    t = torch.tensor([mus, mus_warm, 0.0 if same else 1.0], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    mus, mus_warm, differ = float(t[0]), float(t[1]), float(t[2])
    dist.barrier()
    ex.close()
    best = min(sweep, key=sweep.get)
    pus = sweep[best]
    res.update({"forward_us": pus, "forward_splits": int(best.split("_")[1]), "forward_nccl_us": fus, "multiply_us": mus,
                "forward_warm_us": min(sweep_warm.values()), "forward_nccl_warm_us": fus_warm, "multiply_warm_us": mus_warm,
                "forward_gbs": algo_bytes / pus / 1e3,
                "forward_nccl_gbs": algo_bytes / fus / 1e3, "multiply_gbs": algo_bytes / mus / 1e3,
                "collective": "all-gather of z fused into the product kernel: peer stores over NVLink (fp32, %d B per "
                              "rank and destination) + flag wait; forward_nccl_us is the same projection with "
                              "ncclAllGather" % (rows * 4),
                "fused_equals_nccl_bitwise": differ == 0.0, "forward_us_by_splits": sweep,
                "forward_warm_us_by_splits": sweep_warm,
                "forward_timing": "CUDA graph replay of %d projections" % reps,
                "forward_nccl_timing": nccl_timing,
                "timing": "cold: the timed loop walks over %d identical copies of the rank's %.0f MB shard (more than twice "
                          "the 126 MB L2), so every projection reads its codes from HBM; *_warm_us: one copy replayed, "
                          "L2-resident from N = 2 on" % (copies, shard_bytes / 1e6)})
    return res


if __name__ == "__main__":
    # Libraries (NCCL's version banner, for one) write to file descriptor 1. Point it at stderr while the bench runs and
    # keep the real stdout for the JSON line alone.
    sys.stdout.flush()
    _real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    sys.stdout = _real_stdout
    main()
    sys.stdout.flush()
