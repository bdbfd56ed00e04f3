#!/usr/bin/env python3
"""Benchmark of the EOQ hot path on B200: fused rANS-decode + INT4 dequantise + GEMV at batch 1.

Workload (the one the headline metric is quoted on): a Llama-7B-shape MLP pair --
an 11008 x 4096 weight times x ~ N(0,1) of length 4096, and the transposed 4096 x 11008
down-projection times a vector of length 11008; weights N(0, 0.02), INT4 symmetric absmax,
group 128, fp16 scales, entropy-coded; activations and outputs fp16.  A step is one pass
over both products.  All data is synthetic and seeded.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

value   = algorithmic bytes per step / device time per step (CUDA events, max over ranks),
          with every input already resident in HBM; "algorithmic bytes" are the bytes the
          reference's own wire format needs for the same tensors (rANS blocks of 4096 symbols at
          12-bit precision + block offsets + fp16 scales + x + y), not this library's tile bytes.
e2e     = the same metric through the C ABI with HOST buffers (eoq_b200_gemv_host): x copied in
          from pinned memory and y copied out inside the timed region, every step.
N > 1   : each layer is sharded by output rows over the ranks (strong scaling); a step is the
          two local products plus the gather of the output slices, fused into the GEMV kernels
          (peer stores over NVLink; --gather nccl: an NCCL all-gather per layer instead).
extras  : unless --no-extras, the line also carries `llama7b_step` (a Llama-7B-shape decode step,
          row-sharded like the headline) and `prefill_tp` (the Llama-70B gate/up projection at
          M = 16 ... 2048 tokens, row-sharded, with the all-gather of the output slices).
--workload wire_decode | decode_dequant | polar_q5 | llama7b_step | prefill_gemm | model_load | packed_gemv :
          the other configurations, one JSON line each (single GPU).
--impl reference : the reference's CPU path for the same step -- eoq_parallel_decode
          (compiled from the reference's C sources when available, else the C restatement)
          followed by torch dequantise + F.linear -- on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_UP, K_UP = 11008, 4096          # gate/up projection
N_DN, K_DN = 4096, 11008          # down projection
GROUP = 128
REPLICAS = 8                       # weight copies cycled through so that the working set exceeds L2
WORKLOAD = "llama7b_mlp_pair_int4_g128_rans_b1"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the fused kernel, from the ncu capture
# summarised under profiles/
NCU_TRAFFIC_BYTES_PER_LAUNCH = 22170880    # 11008 x 4096 launch
NCU_TRAFFIC_SOURCE = "profiles/gemv_pairs_kernel__llama7b_mlp_pair.md"
SM_COUNT, SM_CLOCK_MHZ = 148, 1965
# what one rANS step of a warp (32 lanes x 3 weights) costs inside the column loop of the fused kernel, from the ncu
# capture in NCU_TRAFFIC_SOURCE: shared-memory wavefronts (the four sub-partitions of an SM share one pipe) and issue slots
SMEM_WAVEFRONTS_PER_WARP_STEP, ISSUE_SLOTS_PER_WARP_STEP = 5.7, 19.5


def issue_bound(n, k, alg_bytes):
    """The floor the SM itself puts under one launch: every weight costs a third of a rANS step of its lane, and a step
    of a warp cannot go faster than the shared-memory pipe and the issue slots allow, whatever the memory system does."""
    warp_steps_per_subpartition = n * k / 96.0 / (SM_COUNT * 4)
    cycles = warp_steps_per_subpartition * max(SMEM_WAVEFRONTS_PER_WARP_STEP * 4, ISSUE_SLOTS_PER_WARP_STEP)
    us = cycles / SM_CLOCK_MHZ
    return {"us": us, "gbs": alg_bytes / us / 1e3, "binding": "shared-memory pipe",
            "cycles_per_warp_step": max(SMEM_WAVEFRONTS_PER_WARP_STEP * 4, ISSUE_SLOTS_PER_WARP_STEP)}


def make_layer(n, k, seed):
    """Seeded synthetic layer: symbols (uint8 code+7), fp16 scales."""
    import torch
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.02
    blocks = w.view(-1, GROUP)
    scale = (blocks.abs().amax(dim=1) / 7).clamp(min=1e-10)
    codes = (blocks / scale[:, None]).round().clamp(-7, 7).to(torch.int8).view(n, k)
    return (codes + 7).to(torch.uint8).numpy(), scale.half().numpy()


def wire_bytes(sym, scales, n, k, batch=1, impl="b200"):
    """Bytes the reference's wire format needs for this tensor and one GEMV: stream + offsets + scales + x + y.
    The two arms use their own encoder (the library's, or the CPU checker's in the reference arm, which must not
    load the library); the encoders are byte-identical, so the count is the same."""
    if impl == "reference":
        from oracle import oracle as O
        data = O.encode_blocked(sym.ravel().astype(np.int64), 15, 4096, 12)
    else:
        from eoq_quantization_b200.core import rans_blocked as RB
        data = RB.BlockedRANSEncoder(block_size=4096, precision_bits=12).encode(sym.ravel().astype(np.int64), 15)
    return len(data.compressed_blocks) + 4 * data.num_blocks + scales.size * 2 + batch * (k + n) * 2, data


def workload_config(world):
    """The part of the JSON line that names the workload: the same object in both arms."""
    return {"workload": WORKLOAD, "batch": 1, "group": GROUP, "shapes": [[N_UP, K_UP], [N_DN, K_DN]],
            "l2": f"{REPLICAS} weight copies cycled so that the working set exceeds L2",
            "parallelism": f"row-sharded tp{world}"}


class ClockSampler:
    """nvidia-smi clock / throttle sampling during the timed region."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True).start()
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            p = [s.strip() for s in l.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for nm, v in zip(names, p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def shutdown_distributed(world):
    """Leave the process group without blocking the job for ever: captured CUDA graphs that contain NCCL kernels can
    make communicator teardown hang, so the graphs are dropped first and the teardown gets a deadline; a rank that
    misses it says so and exits with a failure code."""
    if world <= 1:
        return
    import gc
    import torch
    import torch.distributed as dist
    sys.stdout.flush()
    gc.collect()
    torch.cuda.synchronize()
    def give_up():
        sys.stderr.write("bench.py: process-group teardown did not finish within 30 s\n")
        sys.stderr.flush()
        os._exit(17)
    timer = threading.Timer(30.0, give_up)
    timer.daemon = True
    timer.start()
    try:
        dist.barrier()
        dist.destroy_process_group()
    finally:
        timer.cancel()


def measured_peak():
    try:
        d = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(d["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# --------------------------------------------------------------------------- CPU reference arm
class CpuReference:
    """The reference's CPU path for one step: eoq_parallel_decode over row-chunk tasks, then torch
    dequantise ((sym - 7) * scale) and F.linear (core/quantized_linear.py:189-228)."""

    def __init__(self, layers, rows_per_task=64):
        import torch
        from oracle import oracle as O
        self.torch, self.O = torch, O
        self.kind = "reference" if O.RefC.available() else "port"
        self.ref = O.RefC() if self.kind == "reference" else None
        self.cores = self.ref.threads() if self.ref else 1
        torch.set_num_threads(max(1, os.cpu_count() or 1))
        self.layers = []
        for sym, scales, n, k in layers:
            items = []
            for lo in range(0, n, rows_per_task):
                chunk = sym[lo:lo + rows_per_task].ravel().astype(np.int64)
                items.append(O.make_c_payload(O.encode_blocked(chunk, 15, 4096, 12)))
            self.layers.append((items, torch.from_numpy(scales.astype(np.float32)), n, k))

    def step(self, xs):
        torch = self.torch
        outs = []
        for (items, scales, n, k), x in zip(self.layers, xs):
            if self.ref:
                rc, decoded, _ = self.ref.parallel_decode(items, 0)
                assert rc == 0
            else:
                decoded = [self.O.decode_c_payload(h, b)[1] for h, b in items]
            sym = torch.from_numpy(np.concatenate(decoded)).view(n, k)
            w = ((sym.float() - 7.0).view(-1, GROUP) * scales[:, None]).view(n, k)
            outs.append(torch.nn.functional.linear(x, w))
        return outs


def run_reference_arm(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    layers = [(*make_layer(N_UP, K_UP, 1), N_UP, K_UP), (*make_layer(N_DN, K_DN, 2), N_DN, K_DN)]
    alg = sum(wire_bytes(s, sc, n, k, impl="reference")[0] for s, sc, n, k in layers)
    cpu = CpuReference(layers)
    xs = [torch.randn(1, K_UP), torch.randn(1, K_DN)]
    for _ in range(args.warmup):
        cpu.step(xs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu.step(xs)
    dt = (time.perf_counter() - t0) / args.steps
    gbs = alg / dt / 1e9
    sample = "whole step: both 11008x4096 and 4096x11008 layers, 64-row decode tasks, fp32 activations"
    line = {"impl": "reference", "metric": "fused decode+INT4 GEMV effective HBM GB/s", "value": gbs, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u32 rANS state, fp32 accumulate",
            "data": "synthetic", "config": workload_config(args.gpus),
            "tokens_per_s": 1.0 / dt,
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cpu.cores, "kind": cpu.kind, "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from eoq_quantization_b200 import _lib
    from eoq_quantization_b200.fused import EOQWeight
    from eoq_quantization_b200.tp import gather_rows, shard_rows

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product has no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = _lib.lib()

    layers = [(*make_layer(N_UP, K_UP, 1), N_UP, K_UP), (*make_layer(N_DN, K_DN, 2), N_DN, K_DN)]
    alg_bytes = [wire_bytes(s, sc, n, k)[0] for s, sc, n, k in layers]
    alg_step = sum(alg_bytes)

    # this rank's row shard of each layer, REPLICAS copies each
    shards = []
    for sym, scales, n, k in layers:
        lo, hi = shard_rows(n, world, rank)
        per_row = k // GROUP
        shards.append(EOQWeight.replicas(REPLICAS, sym[lo:hi], scales[lo * per_row:hi * per_row]))
    g = torch.Generator(device="cuda").manual_seed(1234)
    xs = [torch.randn(1, K_UP, device="cuda", generator=g).half(), torch.randn(1, K_DN, device="cuda", generator=g).half()]

    # N > 1: the all-gather of the output slices is fused into the GEMV kernel (value+epoch words stored into the
    # peers' memory over NVLink, unpacked by a small kernel behind it);
    # --gather nccl, or a failure to set the shared buffers up, falls back to a library all-gather per layer
    pg, gather_mode = None, "none"
    if world > 1:
        gather_mode = "nccl all-gather per layer"
        if args.gather == "peer":
            try:
                from eoq_quantization_b200.tp import PeerGather
                pg = PeerGather(slot_bytes=max(N_UP, N_DN) * 2, slots=2)
                gather_mode = "all-gather fused into the kernel (8-byte value+epoch stores into peer memory)"
            except Exception as exc:                                 # pragma: no cover - depends on the box
                gather_mode += f" (peer set-up failed: {type(exc).__name__})"
    n_total = [N_UP, N_DN]

    def step(i):
        r = i % REPLICAS
        outs = []
        for li in range(2):
            if pg is not None:
                y = pg.gemv(shards[li][r], xs[li], n_total[li], slot=li)
            else:
                y = shards[li][r].gemv(xs[li])
                if world > 1:
                    y = gather_rows(y)
            outs.append(y)
        return outs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if world > 1:
        # the fused gather must give every rank exactly what a library all-gather of the slices gives; if it does not
        # (or could not be set up) on any rank, every rank falls back to the library all-gather
        ok = 1 if pg is not None else 0
        agree = torch.tensor([ok], device="cuda")
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) == 0:
            pg = None
        if pg is not None:
            try:
                for li in range(2):
                    fused = pg.gemv(shards[li][0], xs[li], n_total[li], slot=li).clone()
                    plain = gather_rows(shards[li][0].gemv(xs[li]))
                    ok = ok and bool(torch.equal(fused, plain))
                pg.check()
            except Exception:                                        # a bounded wait gave up
                ok = 0
            agree = torch.tensor([int(ok)], device="cuda")
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
            if int(agree.item()) == 0:
                pg, gather_mode = None, "nccl all-gather per layer (fused gather failed its check)"
        barrier()

    # Warm up eagerly, then capture the steps into CUDA graphs (REPLICAS steps per graph, plus single steps for the
    # remainder) so that the timed region measures the device, not the Python launch path.
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(max(args.warmup, REPLICAS)):
            step(i)
    torch.cuda.current_stream().wait_stream(side)
    barrier()
    launch_mode = "cuda-graph"
    try:
        if args.eager:
            raise RuntimeError("eager launches requested")
        g_full = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_full):
            for i in range(REPLICAS):
                step(i)
        g_one = []
        for r in range(args.steps % REPLICAS):
            g1 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1):
                step(r)
            g_one.append(g1)
    except Exception as exc:                                     # pragma: no cover - depends on the driver stack
        launch_mode = f"eager ({type(exc).__name__})"
        g_full, g_one = None, []

    def run_steps(nsteps):
        if g_full is None:
            for i in range(nsteps):
                step(i)
            return
        for _ in range(nsteps // REPLICAS):
            g_full.replay()
        for g1 in g_one[:nsteps % REPLICAS]:
            g1.replay()

    for _ in range(3):
        run_steps(args.steps)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev0.record()
        run_steps(args.steps)
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1) / args.steps
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        # keep the same load running for at least half a second so that the clock record is meaningful; the number of
        # repetitions comes from the all-reduced time, so every rank runs the same number of exchanges
        for _ in range(int(0.6 / max(ms * 1e-3 * args.steps, 1e-6)) + 1):
            run_steps(args.steps)
        torch.cuda.synchronize()
    launches_timed = (4 if pg is not None else 2) * args.steps          # per rank: two GEMVs (+ two flag waits)
    value = alg_step / (ms * 1e-3) / 1e9

    # per-kernel device time, for the roofline of the dominant kernel (the fused GEMV; the larger share is the
    # 11008 x 4096 launch, the other launch is the same kernel on the transposed shape)
    barrier()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    y_up = torch.empty(1, N_UP // world, device="cuda", dtype=torch.float16)
    cur = torch.cuda.current_stream().cuda_stream

    def up_only():
        for r in range(REPLICAS):
            _lib.check(lib.eoq_b200_gemv(shards[0][r]._h, xs[0].data_ptr(), _lib.F16, 1, y_up.data_ptr(), _lib.F16, None,
                                         torch.cuda.current_stream().cuda_stream), "eoq_b200_gemv")
    g_up = None
    if g_full is not None:
        try:
            g_up = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_up):
                up_only()
        except Exception:
            g_up = None
    reps = max(1, args.steps // REPLICAS)
    for _ in range(2):
        g_up.replay() if g_up is not None else up_only()
    torch.cuda.synchronize()
    k0.record()
    for _ in range(reps):
        g_up.replay() if g_up is not None else up_only()
    k1.record()
    torch.cuda.synchronize()
    up_ms = k0.elapsed_time(k1) / (reps * REPLICAS)
    peak, peak_src = measured_peak()
    up_alg = alg_bytes[0] / world
    roof = {"bound": "hbm", "kernel": "gemv_pairs_kernel<3,1,512>", "achieved": up_alg / (up_ms * 1e-3) / 1e9, "peak": peak,
            "unit": "GB/s", "frac": up_alg / (up_ms * 1e-3) / 1e9 / peak, "peak_source": peak_src,
            "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None,
            "traffic_source": "ncu capture of this kernel on this workload, summarised in " + NCU_TRAFFIC_SOURCE + " (not measured in this run)",
            "launch_us": up_ms * 1e3, "algorithmic_bytes_per_launch": up_alg,
            "fp16_gemv_bytes": N_UP * K_UP * 2 // world, "issue_bound": issue_bound(N_UP // world, K_UP, up_alg)}

    # end to end through the C ABI with host buffers (pinned x in, y out, every step)
    hx = [torch.randn(1, K_UP).half().pin_memory(), torch.randn(1, K_DN).half().pin_memory()]
    hy = [torch.empty(1, (N_UP // world)).half().pin_memory(), torch.empty(1, (N_DN // world)).half().pin_memory()]
    stream = torch.cuda.current_stream().cuda_stream
    e2e_streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()

    def e2e_step(i):
        # each layer is queued on its own stream (x in, kernel, y out, from and to pinned host buffers), so one layer's
        # copies overlap the other's kernel; then both streams are synchronised through their status words
        r = i % REPLICAS
        for li in range(2):
            _lib.check(lib.eoq_b200_gemv_host_async(shards[li][r]._h, hx[li].data_ptr(), _lib.F16, 1, hy[li].data_ptr(), _lib.F16,
                                                    None, e2e_streams[li].cuda_stream), "eoq_b200_gemv_host_async")
        for li in range(2):
            _lib.check(lib.eoq_b200_weight_status(shards[li][r]._h, e2e_streams[li].cuda_stream), "eoq_b200_weight_status")
    for i in range(args.warmup):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    barrier()
    e2e_s = (time.perf_counter() - t0) / args.steps
    # what landed in the host buffers is what the device-resident call computes from the same x
    for li in range(2):
        want = shards[li][(args.steps - 1) % REPLICAS].gemv(hx[li].cuda()).float().cpu()
        err = float((hy[li].float() - want).norm() / want.norm())
        if not err < 1e-3:
            raise SystemExit(f"end-to-end result of layer {li} differs from the device-resident one: rel-L2 {err:.3e}")
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": alg_step / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": (K_UP + K_DN) * 2,
           "d2h_bytes_per_step": (N_UP + N_DN) * 2 // world, "ms_per_step": e2e_s * 1e3,
           "note": ("y is pinned: the kernel stores its results into host memory itself, x goes in by a copy" +
                    ("; per-rank output slices are read back, no gather on the host path" if world > 1 else ""))}

    extras = {}
    if not args.no_extras:
        # the other multi-GPU configurations, appended to the headline line (each guarded: a failure here must not lose the headline)
        del shards
        torch.cuda.empty_cache()
        for key, fn in (("llama7b_step", lambda: measure_llama_step(world, rank, 10, args.gather, world == 1)),
                        ("prefill_tp", lambda: measure_prefill_tp(world, rank, 5))):
            try:
                extras[key] = fn()
            except Exception as exc:                               # pragma: no cover
                extras[key] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            torch.cuda.empty_cache()
        lo_, hi_ = shard_rows(N_UP, world, rank)
        shards = [EOQWeight.replicas(1, layers[0][0][lo_:hi_], layers[0][1][lo_ * (K_UP // GROUP):hi_ * (K_UP // GROUP)]),
                  EOQWeight.replicas(1, layers[1][0][shard_rows(N_DN, world, rank)[0]:shard_rows(N_DN, world, rank)[1]],
                                     layers[1][1][shard_rows(N_DN, world, rank)[0] * (K_DN // GROUP):shard_rows(N_DN, world, rank)[1] * (K_DN // GROUP)])]
    if rank == 0:
        cpu_line = None
        if world == 1 and not args.no_cpu_baseline:
            cpu = CpuReference(layers)
            cx = [x.float().cpu() for x in xs]
            outs = cpu.step(cx)                                   # also a last parity check of the timed kernels
            got = step(0)
            for a, b in zip(got, outs):
                err = float((a.float().cpu() - b).norm() / b.norm())
                assert err < 1e-3, f"bench parity check failed: rel-L2 {err}"
            reps = 3
            t0 = time.perf_counter()
            for _ in range(reps):
                cpu.step(cx)
            cdt = (time.perf_counter() - t0) / reps
            cpu_line = {"value": alg_step / cdt / 1e9, "unit": "GB/s", "cores": cpu.cores, "kind": cpu.kind,
                        "sample": f"whole step ({reps} repetitions): eoq_parallel_decode over 64-row tasks + torch dequantise + F.linear, fp32 activations",
                        "ms_per_step": cdt * 1e3}
        info = shards[0][0].info
        line = {"metric": "fused decode+INT4 GEMV effective HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "u32 rANS state, fp32 accumulate, fp16 in/out",
                "data": "synthetic",
                "config": workload_config(world),
                "setup": {"working_set_mib_per_rank": REPLICAS * sum(s[0].info.stream_bytes for s in shards) >> 20,
                          "gather": gather_mode, "launch": launch_mode, "symbols_per_step": int(info.symbols_per_step),
                          "precision_bits": int(info.precision_bits)},
                "tokens_per_s": 1e3 / ms, "pct_of_hbm_peak": 100.0 * value / (peak * world),
                "algorithmic_bytes_per_step": alg_step,
                "tile_bytes_per_step": int(sum(s[0].info.stream_bytes + s[0].info.scale_bytes for s in shards)) * world,
                "clocks": clocks.summary(), "roofline": roof, "e2e": e2e, "gpu_launches": int(launches_timed) * world}
        if cpu_line:
            line["cpu_baseline"] = cpu_line
        line.update(extras)
        print(json.dumps(line), flush=True)
    g_full = g_one = g_up = None                                 # drop the captured graphs before the communicator goes
    shutdown_distributed(world)


# --------------------------------------------------------------------------- secondary workloads
def run_aux(args):
    """Single-GPU timings of the other benchmark configurations (one JSON line each):
    decode_dequant -- 4096 x 4096 INT4 g128: decode the tiles to packed INT4 and to the fp16 dequantised matrix;
    polar_q5       -- 14336 x 4096 PolarQuant Q5 (per-64 norms), fused decode+GEMV at batch 1, 4, 8."""
    import torch
    from eoq_quantization_b200 import _lib
    from eoq_quantization_b200.fused import EOQWeight
    torch.cuda.set_device(0)
    lib = _lib.lib()
    peak, peak_src = measured_peak()

    def timed(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    if args.workload == "decode_dequant":
        n = k = 4096
        sym, scales = make_layer(n, k, 3)
        alg, _ = wire_bytes(sym, scales, n, k, batch=0)
        ws = EOQWeight.replicas(16, sym, scales)                        # 16 x ~8 MB of tiles + 16 x 32 MB of output > L2
        outs = [torch.empty(n, k, dtype=torch.float16, device="cuda") for _ in ws]
        packs = [torch.empty(n, k // 2, dtype=torch.uint8, device="cuda") for _ in ws]
        st = torch.cuda.current_stream().cuda_stream
        it = {"i": 0}

        def deq():
            i = it["i"] % len(ws); it["i"] += 1
            _lib.check(lib.eoq_b200_weight_decode(ws[i]._h, None, 0, outs[i].data_ptr(), _lib.F16, st))

        def pack():
            i = it["i"] % len(ws); it["i"] += 1
            _lib.check(lib.eoq_b200_weight_decode(ws[i]._h, packs[i].data_ptr(), 1, None, 0, st))
        ms_d, ms_p = timed(deq, args.steps), timed(pack, args.steps)
        ref = (torch.from_numpy(sym.astype(np.float32)).cuda() - 7).view(-1, GROUP) * torch.from_numpy(scales.astype(np.float32)).cuda()[:, None]
        assert torch.equal(outs[0], ref.view(n, k).half()), "decode+dequantise mismatch"
        line = {"metric": "decode+dequantise effective HBM GB/s (compressed bytes read)", "unit": "GB/s", "n_gpus": 1,
                "steps": args.steps, "data": "synthetic", "config": {"workload": "decode_dequant_4096x4096_int4_g128"},
                "value": alg / (ms_d * 1e-3) / 1e9, "ms_per_step": ms_d, "fp16_out_gbs": n * k * 2 / (ms_d * 1e-3) / 1e9,
                "packed_ms": ms_p, "packed_compressed_gbs": alg / (ms_p * 1e-3) / 1e9,
                "symbols_per_s_fp16": n * k / (ms_d * 1e-3), "symbols_per_s_packed": n * k / (ms_p * 1e-3),
                "peak": peak, "peak_source": peak_src, "algorithmic_bytes": alg}
        print(json.dumps(line), flush=True)
        return

    if args.workload == "prefill_gemm":
        return run_prefill_gemm(args, torch, _lib, lib, EOQWeight)

    if args.workload == "packed_gemv":
        # QuantizedLinear's forward for up to 32 rows of fp16 activations: one pass over the packed codes the module keeps
        # in HBM (no entropy coding) with warp-level tensor-core products, beside the entropy-coded fused GEMV and a dense fp16 GEMV of the same layers; graph replay over 8
        # copies of each layer (> L2), both layers of the MLP pair per step
        from eoq_quantization_b200.fused import gemv_packed
        shapes = [(11008, 4096), (4096, 11008)]
        res = {}
        copies = 8
        for bits in (4, 8, 2):
            layers = []
            for li, (n, k) in enumerate(shapes):
                g = torch.Generator().manual_seed(10 + li)
                w = torch.randn(n, k, generator=g) * 0.02
                qmax = (1 << (bits - 1)) - 1
                blocks = w.view(-1, GROUP)
                scale = (blocks.abs().amax(dim=1) / qmax).clamp(min=1e-10)
                codes = (blocks / scale[:, None]).round().clamp(-qmax, qmax).to(torch.int16).view(n, k)
                if bits == 4:
                    u = (codes + qmax).to(torch.uint8); pk = u[:, 0::2] | (u[:, 1::2] << 4)
                elif bits == 2:
                    u = (codes + qmax).to(torch.uint8); pk = u[:, 0::4] | (u[:, 1::4] << 2) | (u[:, 2::4] << 4) | (u[:, 3::4] << 6)
                else:
                    pk = codes.to(torch.int8).view(torch.uint8)
                dense = (codes.float().view(-1, GROUP) * scale.half().float()[:, None]).view(n, k)
                layers.append((n, k, [pk.contiguous().cuda().clone() for _ in range(copies)], scale.half().cuda(), dense))
            per_b = {}
            for batch, xdt in ([(b, torch.float16) for b in (1, 4, 8, 16, 32)] + ([(1, torch.bfloat16)] if bits == 8 else []) +
                               ([(1, torch.float32), (8, torch.float32)] if bits == 4 else [])):
                xs = [torch.randn(batch, k, device="cuda").to(xdt) for (_, k) in shapes]
                y = gemv_packed(layers[0][2][0], layers[0][3], shapes[0][0], shapes[0][1], bits, GROUP, xs[0], out_dtype=torch.float32)
                want = xs[0].float().cpu().double() @ layers[0][4].double().T
                err = float((y.cpu().double() - want).norm() / want.norm())
                assert err < 1e-4, f"packed GEMV check failed: {err}"
                i = [0]

                def step():
                    c = i[0] % copies
                    i[0] += 1
                    for (n, k, pks, sc, _), x in zip(layers, xs):
                        gemv_packed(pks[c], sc, n, k, bits, GROUP, x)
                for _ in range(3):
                    step()
                torch.cuda.synchronize()
                gph = torch.cuda.CUDAGraph()
                side = torch.cuda.Stream()
                with torch.cuda.stream(side):
                    i[0] = 0
                    with torch.cuda.graph(gph):
                        for _ in range(copies):
                            step()
                torch.cuda.synchronize()
                ms = timed(gph.replay, max(3, args.steps // copies)) / copies
                nbytes = sum(p[2][0].numel() + p[3].numel() * 2 + (p[0] + p[1]) * batch * 2 for p in layers)
                per_b[f"batch{batch}" + {torch.float16: "", torch.bfloat16: "_bf16", torch.float32: "_fp32"}[xdt]] = {"us_per_step": ms * 1e3, "gbs": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / peak,
                                          "bytes_per_step": nbytes, "rel_l2_vs_dequantise_then_matmul": err}
            res[f"int{bits}"] = per_b
        # beyond 32 rows the modules dequantise the packed codes to a 16-bit matrix and call a library GEMM: the
        # dequantisation alone (4-bit, both layers, fp16 out) and the pair at 64 and 256 rows
        from eoq_quantization_b200.fused import dequant_packed
        lay4 = []
        for li, (n, k) in enumerate(shapes):
            pk = torch.randint(0, 255, (n, k // 2), dtype=torch.uint8, device="cuda")
            lay4.append((n, k, [pk.clone() for _ in range(copies)], (torch.rand(n * k // GROUP, device="cuda") * 0.01).half()))
        deq = {}
        for rows in (0, 64, 256):
            xs = [torch.randn(max(rows, 1), k, device="cuda").half() for (_, k) in shapes]
            i = [0]

            def dstep():
                c = i[0] % copies
                i[0] += 1
                for (n, k, pks, sc), x in zip(lay4, xs):
                    wd = dequant_packed(pks[c], sc, n, k, 4, GROUP, dtype=torch.float16)
                    if rows:
                        torch.nn.functional.linear(x, wd)
            for _ in range(3):
                dstep()
            torch.cuda.synchronize()
            gq = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                i[0] = 0
                with torch.cuda.graph(gq):
                    for _ in range(copies):
                        dstep()
            torch.cuda.synchronize()
            deq["dequantise_only_us" if rows == 0 else f"dequantise_then_gemm_{rows}_rows_us"] = timed(gq.replay, max(3, args.steps // copies)) / copies * 1e3
        deq["dequantised_bytes_written"] = sum(n * k * 2 for (n, k) in shapes)
        lib.eoq_b200_tune(b"dequant_vec", 0)                           # the general (any shape) kernel on the same layers
        xs, i[0] = [torch.randn(1, k, device="cuda").half() for (_, k) in shapes], 0
        rows = 0
        for _ in range(3):
            dstep()
        torch.cuda.synchronize()
        deq["dequantise_only_general_kernel_us"] = timed(dstep, 16) * 1e3
        lib.eoq_b200_tune(b"dequant_vec", 1)
        del lay4
        # comparators on the 4-bit layers: dense fp16 GEMV (torch) and the entropy-coded fused GEMV
        xs = [torch.randn(1, k, device="cuda").half() for (_, k) in shapes]
        dense16 = [[torch.randn(n, k, device="cuda", dtype=torch.float16) for _ in range(4)] for (n, k) in shapes]
        j = [0]

        def dense_step():
            c = j[0] % 4
            j[0] += 1
            for ws_, x in zip(dense16, xs):
                torch.nn.functional.linear(x, ws_[c])
        for _ in range(3):
            dense_step()
        torch.cuda.synchronize()
        gd = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            j[0] = 0
            with torch.cuda.graph(gd):
                for _ in range(4):
                    dense_step()
        torch.cuda.synchronize()
        dense_us = timed(gd.replay, max(3, args.steps // 4)) / 4 * 1e3
        line = {"metric": "packed-code GEMV (QuantizedLinear forward, few rows) effective HBM GB/s", "unit": "GB/s", "n_gpus": 1,
                "steps": args.steps, "data": "synthetic", "higher_is_better": True, "dtype": "packed integer codes, fp32 accumulate, fp16 in/out",
                "config": {"workload": "llama7b_mlp_pair_packed_g128", "shapes": shapes, "l2": f"{copies} copies of each layer cycled (> L2)",
                           "launch": "cuda-graph"},
                "value": res["int4"]["batch1"]["gbs"], "ms_per_step": res["int4"]["batch1"]["us_per_step"] / 1e3,
                "roofline": {"bound": "hbm", "kernel": "gemv_packed_mma_kernel<4,fp16,1>", "achieved": res["int4"]["batch1"]["gbs"], "peak": peak,
                             "unit": "GB/s", "frac": res["int4"]["batch1"]["frac_of_hbm_peak"], "peak_source": peak_src, "traffic": None},
                "per_width": res, "beyond_32_rows_int4": deq, "fp16_dense_us_per_step": dense_us}
        print(json.dumps(line), flush=True)
        return

    # polar_q5
    n, k, d = 14336, 4096, 64
    z = np.load(os.path.join(ROOT, "tests", "golden", "ref_polar.npz"))
    cent = torch.from_numpy(z["centroids5"]).cuda()
    H = torch.from_numpy(z["hadamard64"]).cuda()
    g = torch.Generator(device="cuda").manual_seed(3)
    w = torch.randn(n, k, device="cuda", generator=g) * 0.015
    outl = torch.rand(n, k, device="cuda", generator=g) < 1e-3
    sign = torch.where(torch.rand(n, k, device="cuda", generator=g) < 0.5, -1.0, 1.0)
    w = torch.where(outl, sign * 8 * 0.015, w)
    codes = torch.empty(n, k, dtype=torch.uint8, device="cuda")
    norms = torch.empty(n * k // d, dtype=torch.float16, device="cuda")
    for lo in range(0, n, 512):                                          # core/polar_quant.py:138-213, chunked by rows
        blk = w[lo:lo + 512].reshape(-1, d)
        nr = blk.norm(dim=1, keepdim=True).clamp(min=1e-10)
        c = (((blk / nr) @ H * (d ** 0.5)).unsqueeze(-1) - cent).abs().argmin(dim=-1)
        codes[lo:lo + 512] = c.reshape(512, k).to(torch.uint8)
        norms[lo * k // d:(lo + 512) * k // d] = nr.squeeze(1).half()
    from eoq_quantization_b200.core import rans_blocked as RB
    sym = codes.cpu().numpy()
    wire = RB.BlockedRANSEncoder(block_size=4096, precision_bits=12).encode(sym.ravel().astype(np.int64), 32)
    ws = EOQWeight.replicas(4, sym, norms, kind=_lib.KIND_Q5_POLAR, group=64, centroids=z["centroids5"])
    res = {}
    for batch in (1, 4, 8):
        x = torch.randn(batch, k, device="cuda", generator=g).half()
        y = torch.empty(batch, n, device="cuda", dtype=torch.float16)
        st = torch.cuda.current_stream().cuda_stream
        it = {"i": 0}

        def run():
            i = it["i"] % len(ws); it["i"] += 1
            _lib.check(lib.eoq_b200_gemv(ws[i]._h, x.data_ptr(), _lib.F16, batch, y.data_ptr(), _lib.F16, None, st))
        ms = timed(run, args.steps)
        alg = len(wire.compressed_blocks) + 4 * wire.num_blocks + norms.numel() * 2 + batch * (n + k) * 2
        res[f"batch{batch}"] = {"ms": ms, "gbs": alg / (ms * 1e-3) / 1e9, "pct_of_peak": 100 * alg / (ms * 1e-3) / 1e9 / peak}
    # the same layer from the byte codes PolarLinear keeps resident (8 bit/weight, no entropy coding): rotation of x
    # (torch) + one pass over the codes per step; 4 copies cycled like the tiles above
    from eoq_quantization_b200.fused import gemv_polar_codes
    cds = [codes.clone() for _ in range(4)]
    byte_codes = {"tensor_cores": {}, "cuda_cores": {}}
    for form, tc in (("tensor_cores", True), ("cuda_cores", False)):
        for batch in (1, 4, 8, 16, 32) if tc else (1, 4, 8):
            x = torch.randn(batch, k, device="cuda", generator=g).half()
            want = torch.cat([ws[0].gemv(x[lo:lo + 8], out_dtype=torch.float32) for lo in range(0, batch, 8)])
            got = gemv_polar_codes(cds[0], norms, cent, n, k, 5, d, x, tensor_cores=tc)
            err = float((got - want).norm() / want.norm())
            assert err < 1e-4, f"byte-code polar GEMV differs from the entropy-coded one: {err}"
            it = {"i": 0}

            def run_codes():
                i = it["i"] % len(cds); it["i"] += 1
                gemv_polar_codes(cds[i], norms, cent, n, k, 5, d, x, out_dtype=torch.float16, tensor_cores=tc)
            for _ in range(3):
                run_codes()
            torch.cuda.synchronize()
            gph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()        # rotation (torch) + kernel, one replayed graph over the 4 copies
            with torch.cuda.stream(side):
                it["i"] = 0
                with torch.cuda.graph(gph):
                    for _ in range(len(cds)):
                        run_codes()
            torch.cuda.synchronize()
            ms = timed(gph.replay, max(3, args.steps // len(cds))) / len(cds)
            nbytes = n * k + norms.numel() * 2 + batch * (n * 2 + k * 6)
            byte_codes[form][f"batch{batch}"] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "pct_of_peak": 100 * nbytes / (ms * 1e-3) / 1e9 / peak,
                                                 "rel_l2_vs_entropy_coded": err}
    line = {"metric": "fused decode+Q5 polar GEMV effective HBM GB/s", "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "data": "synthetic", "config": {"workload": "polar_q5_14336x4096_g64", "l2": "4 weight copies cycled"},
            "value": res["batch1"]["gbs"], "ms_per_step": res["batch1"]["ms"], "batches": res, "peak": peak,
            "peak_source": peak_src, "wire_bits_per_weight": len(wire.compressed_blocks) * 8 / (n * k),
            "tile_bits_per_weight": ws[0].info.bits_per_weight, "from_byte_codes": byte_codes}
    print(json.dumps(line), flush=True)


def run_llama_step(args):
    """Llama-7B-shape decode step, random init (configuration 4 of the benchmark set): 32 layers, hidden 4096, 32 heads, SwiGLU 11008,
    vocabulary 32000, KV length 1024, batch 1.  Every linear is INT4 g128 entropy-coded and runs through the fused
    kernel; norms, rotary embedding, attention (torch SDPA) and the activation are torch ops.  All 32 layers hold
    their own copy of the tiles in HBM (one set of values, 32 uploads), so every byte of weight is read from DRAM.
    With N ranks every linear is row-sharded and followed by an all-gather of the output slices.  The same step
    with dense fp16 weights (torch matmul) is timed beside it."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    line = measure_llama_step(world, rank, min(args.steps, 50), args.gather, world == 1 and not args.no_cpu_baseline)
    if rank == 0:
        print(json.dumps(line), flush=True)
    shutdown_distributed(world)


def measure_llama_step(world, rank, steps, gather, with_fp16):
    """One measurement of the Llama-7B-shape decode step on an initialised process group; returns the JSON object."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from eoq_quantization_b200.fused import EOQWeight
    from eoq_quantization_b200.tp import gather_rows, shard_rows
    H, NH, HD, FF, V, L, KV = 4096, 32, 128, 11008, 32000, 32, 1024
    shapes = {"qkv": (3 * H, H), "o": (H, H), "gate_up": (2 * FF, H), "down": (H, FF)}
    layers, alg_layer = {}, 0
    for i, (name, (n, k)) in enumerate(shapes.items()):
        sym, scales = make_layer(n, k, 10 + i)
        alg_layer += wire_bytes(sym, scales, n, k)[0]
        lo, hi = shard_rows(n, world, rank)
        layers[name] = EOQWeight.replicas(L, sym[lo:hi], scales[lo * (k // GROUP):hi * (k // GROUP)])
    sym, scales = make_layer(V, H, 20)
    alg_head = wire_bytes(sym, scales, V, H)[0]
    lo, hi = shard_rows(V, world, rank)
    head = EOQWeight.from_symbols(sym[lo:hi], scales[lo * (H // GROUP):hi * (H // GROUP)])
    alg_step = L * alg_layer + alg_head

    g = torch.Generator(device="cuda").manual_seed(5)
    kc = [torch.randn(1, NH // world, KV, HD, device="cuda", generator=g).half() for _ in range(L)]
    vc = [torch.randn(1, NH // world, KV, HD, device="cuda", generator=g).half() for _ in range(L)]
    nw = torch.ones(H, device="cuda", dtype=torch.float16)
    x0 = torch.randn(1, H, device="cuda", generator=g).half()

    def norm(x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).half() * nw

    # N > 1: the output slices of every linear meet through the gather fused into the GEMV kernel (three slots in
    # rotation: 129 gathers per step, so consecutive gathers never share a slot, also across steps); the attention
    # output, which no GEMV produces, goes through a library all-gather
    pg, call_no = None, [0]
    if world > 1 and gather == "peer":
        from eoq_quantization_b200.tp import PeerGather
        pg = PeerGather(slot_bytes=V * 2, slots=3)

    def linear(w, x, n_total):
        if pg is not None:
            slot = call_no[0] % 3
            call_no[0] += 1
            return pg.gemv(w, x, n_total, slot=slot)
        y = w.gemv(x)
        return gather_rows(y) if world > 1 else y

    def step(x, lin):
        call_no[0] = 0
        for i in range(L):
            h = norm(x)
            qkv = lin("qkv", i, h)
            q, k, v = qkv.view(1, 3, NH, HD).unbind(1)
            hs = NH // world                                       # attention is sharded by heads
            qs = q[:, rank * hs:(rank + 1) * hs].transpose(0, 1).reshape(1, hs, 1, HD)
            att = F.scaled_dot_product_attention(qs, kc[i], vc[i])  # new k/v of this token would be appended here
            att = att.reshape(1, hs * HD)
            if world > 1:
                att = gather_rows(att)
            x = x + lin("o", i, att)
            h = norm(x)
            gu = lin("gate_up", i, h)
            x = x + lin("down", i, F.silu(gu[:, :FF]) * gu[:, FF:])
        return lin("head", 0, norm(x))

    def lin_eoq(name, i, x):
        return linear(head if name == "head" else layers[name][i], x, V if name == "head" else shapes[name][0])

    def timed(fn, steps):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph, mode = torch.cuda.CUDAGraph(), "cuda-graph"
        try:
            with torch.cuda.graph(graph):
                fn()
            run = graph.replay
        except Exception as exc:                               # pragma: no cover
            run, mode = fn, f"eager ({type(exc).__name__})"
        for _ in range(3):
            run()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, mode

    ms, mode = timed(lambda: step(x0, lin_eoq), steps)
    if pg is not None:
        pg.check()                                               # no gather may have given up waiting for a peer
    line = {"metric": "Llama-7B-shape decode step, tokens/s at batch 1", "unit": "tokens/s", "value": 1e3 / ms,
            "ms_per_step": ms, "n_gpus": world, "steps": steps, "data": "synthetic", "scaling": "strong",
            "config": {"workload": "llama7b_decode_step_int4_g128_rans", "layers": L, "hidden": H, "kv_len": KV,
                       "launch": mode, "parallelism": f"row-sharded tp{world}" + ("" if world == 1 else
                                                   " + gather fused into the GEMVs" if pg is not None else " + nccl all-gather")},
            "gathers_per_step": 0 if world == 1 else 4 * L + 1 + L,
            "algorithmic_weight_bytes_per_step": alg_step, "weight_gbs": alg_step / (ms * 1e-3) / 1e9}
    if with_fp16:
        # the same step on the codes as QuantizedLinear keeps them (packed INT4 + fp16 scales, no entropy coding: 4.125
        # bit/weight resident instead of ~3.7), multiplied straight from the packed form; one copy per layer
        from eoq_quantization_b200.fused import gemv_packed
        packed = {}
        for i, (name, (n, k)) in enumerate(list(shapes.items()) + [("head", (V, H))]):
            sym, scales = make_layer(n, k, 20 if name == "head" else 10 + i)
            u = torch.from_numpy(sym).cuda()
            pk = (u[:, 0::2] | (u[:, 1::2] << 4)).contiguous()
            sc = torch.from_numpy(scales).cuda()
            packed[name] = ([pk.clone() for _ in range(1 if name == "head" else L)], sc, n, k)
            del u, pk

        def lin_packed(name, i, x):
            pks, sc, n, k = packed[name]
            return gemv_packed(pks[i], sc, n, k, 4, GROUP, x)
        y_eoq, y_pk = step(x0, lin_eoq), step(x0, lin_packed)
        err = float((y_eoq.float() - y_pk.float()).norm() / y_eoq.float().norm())
        assert err < 2e-2, f"packed and entropy-coded steps disagree: {err}"      # same weights, fp16 hand-offs between 129 linears
        msp, _ = timed(lambda: step(x0, lin_packed), steps)
        line["packed_int4_ms_per_step"] = msp
        line["packed_int4_tokens_per_s"] = 1e3 / msp
        line["packed_vs_entropy_coded_rel_l2"] = err
        del packed
        # dense fp16 comparator: same step, weights as fp16 matrices (one copy per layer)
        del layers
        torch.cuda.empty_cache()
        dense = {n_: [torch.randn(s_[0], s_[1], device="cuda", dtype=torch.float16) * 0.02 for _ in range(L)] for n_, s_ in shapes.items()}
        dhead = torch.randn(V, H, device="cuda", dtype=torch.float16) * 0.02

        def lin_f16(name, i, x):
            return x @ (dhead if name == "head" else dense[name][i]).T
        ms16, _ = timed(lambda: step(x0, lin_f16), steps)
        line["fp16_dense_ms_per_step"] = ms16
        line["fp16_dense_tokens_per_s"] = 1e3 / ms16
        line["speedup_vs_fp16_dense"] = ms16 / ms
        line["packed_int4_speedup_vs_fp16_dense"] = ms16 / line["packed_int4_ms_per_step"]
        del dense, dhead
    if pg is not None:
        pg.close()
    return line


def measure_prefill_tp(world, rank, steps):
    """Llama-70B-shape gate/up projection (28672 x 8192, INT4 g128 rANS-coded, N(0, 0.015)) row-sharded over the ranks:
    per M, EOQWeight.linear on this rank's rows (the fused decode + tensor-core GEMM up to 128 rows of activations, decode
    to bf16 + library GEMM beyond) followed by the all-gather of the output slices (NCCL); device time, max over ranks.  Every rank's shard is drawn from the same distribution (its own seed)."""
    import torch
    import torch.distributed as dist
    from eoq_quantization_b200 import _lib
    from eoq_quantization_b200.fused import EOQWeight
    lib = _lib.lib()
    n_total, k = 28672, 8192
    n = n_total // world
    rng = np.random.default_rng(100 + rank)
    res = {}
    chunk = 3584                                                    # encode in shards of the 8-rank size to bound host memory
    ws = []
    for lo in range(0, n, chunk):
        w = (rng.standard_normal((min(chunk, n - lo), k)) * 0.015).astype(np.float32)
        sc = np.maximum(np.abs(w.reshape(-1, GROUP)).max(axis=1) / 7.0, 1e-10).astype(np.float32)
        sym = (np.clip(np.round(w.reshape(-1, GROUP) / sc[:, None]), -7, 7) + 7).astype(np.uint8).reshape(w.shape)
        ws.append(EOQWeight.from_symbols(sym, sc.astype(np.float16)))
        del w, sym
    from eoq_quantization_b200.fused import GEMM_MAX_ROWS
    for m in (16, 64, 128, 256, 2048):
        x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        full = torch.empty(world, m, n, device="cuda", dtype=torch.bfloat16) if world > 1 else None

        def run():
            # EOQWeight.linear is the call a module makes: fused decode + tensor-core MMA up to GEMM_MAX_ROWS rows,
            # one fused decode + dequantise to 16 bits and a library GEMM beyond
            ys = [wi.linear(x) for wi in ws]
            if world > 1:
                local = ys[0] if len(ys) == 1 else torch.cat(ys, dim=1)
                dist.all_gather_into_tensor(full, local.contiguous())
        for _ in range(3):
            run()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        # one replayed graph per M (compute kernels + the collective), so that the device time is not the host's launch rate;
        # plain launches if the capture is refused
        launch = "cuda-graph"
        graph = torch.cuda.CUDAGraph()
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                run()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph):
                run()
            replay = graph.replay
        except Exception as exc:                                    # noqa: BLE001 -- any capture failure means eager timing
            launch = f"eager ({type(exc).__name__})"
            replay = run
        ok = torch.tensor([1.0 if launch == "cuda-graph" else 0.0], device="cuda")
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)                 # every rank must take the same route
        if float(ok.item()) == 0.0:
            replay, launch = run, launch if launch != "cuda-graph" else "eager (another rank could not capture)"
        for _ in range(2):
            replay()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(3, min(steps, 10))
        e0.record()
        for _ in range(reps):
            replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / reps * 1e3
        if world > 1:
            t = torch.tensor([us], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t.item())
        res[f"M{m}"] = {"us": us, "tflops": 2.0 * m * n_total * k / us / 1e6,
                        "path": "fused decode + tcgen05 MMA" if m <= GEMM_MAX_ROWS else "fused decode to bf16, then library GEMM",
                        "launch": launch}
    return {"workload": "llama70b_gate_up_28672x8192_int4_g128_rans, bf16 x", "parallelism": f"row-sharded tp{world}" +
            (" + nccl all-gather of [M, rows / ranks] slices" if world > 1 else ""), "rows_per_rank": n, "per_m": res}


def run_prefill_gemm(args, torch, _lib, lib, EOQWeight):
    """Batched prefill on Llama-70B-shape layers (hidden 8192, intermediate 28672), one GPU's row shard at tp8:
    bf16 activations N(0,1), INT4 g128 rANS-coded N(0,0.015) weights, M tokens.  For M <= 128 (and 256, two passes)
    the fused path decodes tiles straight into tcgen05 MMAs; the line also times decode-to-fp16 + library GEMM,
    which is what larger M uses, and the library GEMM alone on a resident fp16 matrix (4.4x the weight bytes)."""
    tf_peak = None
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            tf_peak = json.load(f).get("bf16_tflops")
    tf_peak, tf_src = (tf_peak, "measured") if tf_peak else (1590.0, "fallback")
    st_capture = torch.cuda.Stream()

    def graph_us(fn, reps, warm=1):
        for _ in range(warm):            # the first call on a weight allocates its scratch: not inside a capture
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(st_capture):
            fn()
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=st_capture):
                for _ in range(reps):
                    fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * reps) * 1e3

    shapes = {"gate_up_shard": (3584, 8192), "down_shard": (1024, 28672), "qo_shard": (1024, 8192)}
    if args.eager:                      # plain launches of one case, for profilers
        shapes = {"gate_up_shard": shapes["gate_up_shard"]}
    out = {}
    for name, (n, k) in shapes.items():
        rng = np.random.default_rng(11)
        w = (rng.standard_normal((n, k)) * 0.015).astype(np.float32)
        sc = np.maximum(np.abs(w.reshape(-1, GROUP)).max(axis=1) / 7.0, 1e-10).astype(np.float32)
        sym = (np.clip(np.round(w.reshape(-1, GROUP) / sc[:, None]), -7, 7) + 7).astype(np.uint8).reshape(n, k)
        del w
        copies = max(2, int(160e6 // (n * k * 0.46)) + 1)                 # compressed copies cycled: working set > L2
        ws = EOQWeight.replicas(copies, sym, sc.astype(np.float16))
        info = ws[0].info
        dense = ws[0].dequantize(torch.float16)
        res = {}
        for m in ((64,) if args.eager else (16, 64, 256, 2048)):
            x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
            y = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
            xh = x.half()
            it = {"i": 0}

            def fused():
                i = it["i"] % len(ws); it["i"] += 1
                _lib.check(lib.eoq_b200_gemm(ws[i]._h, x.data_ptr(), _lib.BF16, m, y.data_ptr(), _lib.BF16, None,
                                             torch.cuda.current_stream().cuda_stream), "gemm")

            def decode_then_library():
                i = it["i"] % len(ws); it["i"] += 1
                _lib.check(lib.eoq_b200_weight_decode(ws[i]._h, None, 0, dense.data_ptr(), _lib.F16,
                                                      torch.cuda.current_stream().cuda_stream), "decode")
                torch.matmul(xh, dense.t())

            def library_only():
                torch.matmul(xh, dense.t())
            flop = 2.0 * m * n * k
            r = {}
            if args.eager:
                for _ in range(max(args.steps, 1)):
                    fused()
                torch.cuda.synchronize()
                print(json.dumps({"workload": "prefill_gemm eager", "shape": [n, k], "M": m, "launches": max(args.steps, 1)}), flush=True)
                return
            if True:                                                       # every M runs fused: 512 rows share one pass
                us = graph_us(fused, 12 if m <= 256 else 4, warm=len(ws))
                want = (xh.float() @ dense.float().t())
                err = float((y.float() - want).norm() / want.norm())
                assert err < 8e-3, f"fused GEMM mismatch {err}"            # bf16 output rounding ~ 4e-3
                r["fused_us"], r["fused_tflops"], r["fused_rel_l2_vs_fp16_matmul"] = us, flop / us / 1e6, err
            r["decode_then_library_us"] = graph_us(decode_then_library, 6)
            r["library_fp16_resident_us"] = graph_us(library_only, 12)
            best = min(r.get("fused_us", 1e30), r["decode_then_library_us"])
            r["path"] = "fused-tcgen05" if best == r.get("fused_us") else "decode+library-gemm"
            r["tflops"] = flop / best / 1e6
            r["compressed_gbs"] = info.stream_bytes / best / 1e3
            res[f"M{m}"] = r
        out[name] = {"shape": [n, k], "bits_per_weight": info.bits_per_weight, "precision_bits": int(info.precision_bits), **res}
        del ws, dense
        torch.cuda.empty_cache()
    top = out["gate_up_shard"]["M64"]
    line = {"metric": "fused decode+INT4 prefill GEMM TFLOP/s", "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "data": "synthetic",
            "dtype": "u32 rANS state, fp16 operands, fp32 accumulate (TMEM), bf16 in/out",
            "config": {"workload": "llama70b_prefill_gemm_tp8_shard_int4_g128_rans", "l2": "compressed copies cycled (> L2)",
                       "launch": "cuda-graph"},
            "value": top["tflops"], "ms_per_step": top["fused_us"] / 1e3, "shapes": out,
            "roofline": {"bound": "tensor", "achieved": top["tflops"], "peak": tf_peak, "unit": "TFLOP/s",
                         "frac": top["tflops"] / tf_peak, "peak_source": tf_src, "traffic": None,
                         "note": "decode-bound: the MMAs use a few percent of the tensor pipe; see profiles/"}}
    print(json.dumps(line), flush=True)


def run_wire_decode(args):
    """Decode of the reference's wire format (independent rANS blocks, byte renormalisation), one JSON line per case:
    configuration 1 of the benchmark set (4096 x 4096 INT4 symbols, blocks of 4096, 12-bit table), the .eoq default (blocks of
    256, 14-bit table) and an EOQ-GGUF-style payload (byte alphabet, 16-bit table, blocks of 256).
    value  = symbols per second of the decode kernel on device-resident inputs (eoq_cuda_decode_tensor_device),
             eight copies of the tensor cycled so that streams and outputs come from DRAM;
    e2e    = the same through eoq_parallel_decode with host buffers (64-row tasks; payloads copied in and symbols
             copied out inside the timed region);
    beside them: the reference's own CUDA kernel (compiled from its source into oracle/_ref) on the same device
    buffers, and its C decoder (eoq_parallel_decode.c) on the host cores."""
    import ctypes as C
    import torch
    from eoq_quantization_b200 import _lib
    from eoq_quantization_b200.core import rans_blocked as RB
    from eoq_quantization_b200.core.rans import _normalize_frequencies
    torch.cuda.set_device(0)
    lib = _lib.lib()
    peak, peak_src = measured_peak()
    n = k = 4096
    sym4, _ = make_layer(n, k, 3)
    cases = [("config1_4096x4096_int4_block4096_p12", sym4.ravel(), 15, 4096, 12),
             ("eoq_default_4096x4096_int4_block256_p14", sym4.ravel(), 15, 256, 14),
             ("gguf_bytes_8Mi_block256_p16", (sym4[:, 0::2] | (sym4[:, 1::2] << 4)).ravel(), 256, 256, 16)]
    ref_cuda = ref_c = None
    if not args.no_cpu_baseline:
        try:
            from oracle import oracle as O
            ref_cuda = O.RefCuda() if O.RefCuda.available() else None
            ref_c = O.RefC() if O.RefC.available() else None
        except Exception:
            pass
    copies = 8
    for name, sym, alphabet, block, p in cases:
        sym = np.ascontiguousarray(sym)
        total = sym.size
        data = RB.BlockedRANSEncoder(block_size=block, precision_bits=p).encode(sym.astype(np.int64), alphabet)
        freq, cdf = _normalize_frequencies(np.asarray(data.freq_table, np.int64), p)
        offs = np.asarray(data.block_offsets, np.uint32)
        sizes = np.diff(np.append(offs.astype(np.int64), len(data.compressed_blocks))).astype(np.uint32)
        info = np.zeros((1 << p, 4), np.uint16)                       # {symbol, freq, cum, pad} per slot
        for s_ in range(alphabet):
            info[cdf[s_]:cdf[s_ + 1]] = (s_, freq[s_] & 0xFFFF, cdf[s_], 0)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1).copy()).cuda()
        d_streams = [dev(np.frombuffer(data.compressed_blocks, np.uint8)) for _ in range(copies)]
        d_outs = [torch.empty(total, dtype=torch.uint8, device="cuda") for _ in range(copies)]
        d_offs, d_sizes, d_info = dev(offs), dev(sizes), dev(info)
        st = torch.cuda.current_stream().cuda_stream
        it = {"i": 0}

        def ours():
            i = it["i"] % copies; it["i"] += 1
            rc = lib.eoq_cuda_decode_tensor_device(d_streams[i].data_ptr(), d_offs.data_ptr(), d_sizes.data_ptr(), d_info.data_ptr(),
                                                   d_outs[i].data_ptr(), data.num_blocks, block, total, p, st)
            assert rc == 0

        def theirs():
            i = it["i"] % copies; it["i"] += 1
            assert ref_cuda.decode_device(d_streams[i].data_ptr(), d_offs.data_ptr(), d_sizes.data_ptr(), d_info.data_ptr(),
                                          d_outs[i].data_ptr(), data.num_blocks, block, total, p, st) == 0

        def timed(fn, reps):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps
        reps = max(copies, min(args.steps, 50))                       # every copy is decoded at least once
        ms = timed(ours, reps)
        want = torch.from_numpy(sym.astype(np.uint8)).cuda()
        assert all(torch.equal(o, want) for o in d_outs), "decoded symbols differ from the encoder's input"
        line = {"metric": "wire-format rANS decode, symbols/s", "unit": "Gsym/s", "n_gpus": 1, "steps": reps, "warmup": 3,
                "higher_is_better": True, "data": "synthetic", "dtype": "u32 rANS state, byte renormalisation, u8 symbols",
                "config": {"workload": name, "symbols": int(total), "alphabet": alphabet, "block": block, "precision_bits": p,
                           "l2": f"{copies} copies of stream and output cycled (> L2)"},
                "value": total / (ms * 1e-3) / 1e9, "ms_per_step": ms, "compressed_bytes": len(data.compressed_blocks),
                "bits_per_symbol": len(data.compressed_blocks) * 8 / total, "gpu_launches": reps}
        traffic = len(data.compressed_blocks) + total + 8 * data.num_blocks
        line["roofline"] = {"bound": "hbm", "kernel": "decode_v1_lanes_kernel", "achieved": traffic / (ms * 1e-3) / 1e9, "peak": peak,
                            "unit": "GB/s", "frac": traffic / (ms * 1e-3) / 1e9 / peak, "peak_source": peak_src, "traffic": None,
                            "algorithmic_bytes_per_launch": traffic, "note": "stream + block offsets and sizes read, one byte per symbol written"}
        if ref_cuda is not None:
            for o in d_outs:
                o.zero_()
            ms_ref = timed(theirs, max(3, reps // 4))
            assert all(torch.equal(o, want) for o in d_outs), "the reference kernel's symbols differ"
            line["reference_cuda_kernel"] = {"kernel": "eoq_rans_decode_blocks_kernel (llamacpp_integration/eoq_cuda_decompress.cu:235-302)",
                                             "ms": ms_ref, "gsym_per_s": total / (ms_ref * 1e-3) / 1e9, "speedup": ms_ref / ms}
        # end to end: host payloads -> eoq_parallel_decode -> host symbols, 64-row tasks
        rows_per_task = 64
        per = rows_per_task * (total // n)
        tasks_n = total // per
        tasks = (_lib.DecodeTask * tasks_n)()
        keep = []
        for i in range(tasks_n):
            d = RB.BlockedRANSEncoder(block_size=block, precision_bits=p).encode(sym[i * per:(i + 1) * per].astype(np.int64), alphabet)
            f_, _c = _normalize_frequencies(np.asarray(d.freq_table, np.int64), p)
            body = f_.astype("<u2").tobytes() + np.asarray(d.block_offsets, "<u4").tobytes() + bytes(d.compressed_blocks)
            h = _lib.TensorHeader(0, d.num_blocks, alphabet, p, block, len(body), per)
            buf = (C.c_ubyte * len(body)).from_buffer_copy(body)
            out = np.zeros(per, np.uint8)
            keep.append((h, buf, out))
            tasks[i].header = C.pointer(h); tasks[i].compressed_data = C.cast(buf, C.c_void_p)
            tasks[i].compressed_size = len(body); tasks[i].output = out.ctypes.data; tasks[i].output_capacity = per
        h2d = sum(len(b) for _, b, _ in keep)
        popts = _lib.ParallelOpts(8, _lib.PARALLEL_PROGRESS_FN(), None)
        for _ in range(2):
            assert lib.eoq_parallel_decode(tasks, tasks_n, C.byref(popts)) == 0
        t0 = time.perf_counter()
        e2e_reps = 5
        for _ in range(e2e_reps):
            assert lib.eoq_parallel_decode(tasks, tasks_n, C.byref(popts)) == 0
        e2e_s = (time.perf_counter() - t0) / e2e_reps
        assert all(np.array_equal(o, sym[i * per:(i + 1) * per].astype(np.uint8)) for i, (_, _, o) in enumerate(keep))
        line["e2e"] = {"value": total / e2e_s / 1e9, "unit": "Gsym/s", "ms_per_step": e2e_s * 1e3, "h2d_bytes_per_step": h2d,
                       "d2h_bytes_per_step": int(total), "tasks": tasks_n, "note": "eoq_parallel_decode, pageable host buffers"}
        if ref_c is not None:
            items = [(np.array([getattr(h, f) for f, _ in _lib.TensorHeader._fields_], np.uint32), bytes(b)) for h, b, _ in keep]
            rc, outs, dt = ref_c.parallel_decode(items, 0)
            rc, outs, dt = ref_c.parallel_decode(items, 0)
            assert rc == 0 and all(np.array_equal(o, sym[i * per:(i + 1) * per].astype(np.uint8)) for i, o in enumerate(outs))
            line["cpu_baseline"] = {"value": total / dt / 1e9, "unit": "Gsym/s", "cores": ref_c.threads(), "kind": "reference",
                                    "sample": f"the whole tensor once: eoq_parallel_decode.c over {tasks_n} tasks", "ms": dt * 1e3}
        print(json.dumps(line), flush=True)
        del d_streams, d_outs


def run_model_load(args):
    """Load time of one Llama-7B-shape transformer block (wq, wk, wv, wo 4096 x 4096; gate, up 11008 x 4096; down
    4096 x 11008: 202 M INT4 weights) from the reference's wire format (`RANS` containers, 256-symbol blocks, p = 14,
    as an `.eoq` file holds them) to resident entropy-coded tiles, by phase:
      wire decode   -- BlockedRANSDecoder.decode_all: payload to the device, lane kernel, symbols back to the host;
      tile encode   -- EOQWeight.from_symbols: symbols to the device, tile encoder kernels, scales and tables uploaded;
      from_rans     -- EOQWeight.from_rans: wire decode and tile encode on the device in one call (the symbols never
                       visit the host), what `EOQLinear` and `load_eoq_to_device` use.
    One JSON line; a 32-block model is 32 times this plus embeddings (not coded)."""
    import torch
    from eoq_quantization_b200.core import rans_blocked as RB
    from eoq_quantization_b200.fused import EOQWeight
    torch.cuda.set_device(0)
    shapes = [("wq", 4096, 4096), ("wk", 4096, 4096), ("wv", 4096, 4096), ("wo", 4096, 4096),
              ("gate", 11008, 4096), ("up", 11008, 4096), ("down", 4096, 11008)]
    layers = []
    for i, (name, n, k) in enumerate(shapes):
        sym, scales = make_layer(n, k, 40 + i)
        t0 = time.perf_counter()
        data = RB.BlockedRANSEncoder(256, 14).encode(sym.reshape(-1), 15)
        enc_s = time.perf_counter() - t0
        layers.append((name, n, k, sym, scales, data, RB.serialize_blocked_rans(data), enc_s))
    # context, kernels and the library's device arenas warm (the arenas grow to the largest matrix once per process)
    t0 = time.perf_counter()
    big = max(layers, key=lambda L: L[1] * L[2])
    EOQWeight.from_rans(big[6], big[4], (big[1], big[2]))
    torch.cuda.synchronize()
    first_call_s = time.perf_counter() - t0
    EOQWeight.from_symbols(big[3], big[4])
    RB.BlockedRANSDecoder().decode_all(layers[0][5])
    tot = {"wire_decode_s": 0.0, "tile_encode_s": 0.0, "from_rans_s": 0.0, "wire_encode_s": 0.0}
    per_layer, weights, wire, keep = {}, 0, 0, []
    for name, n, k, sym, scales, data, raw, enc_s in layers:
        t0 = time.perf_counter()
        got = RB.BlockedRANSDecoder().decode_all(data)
        t1 = time.perf_counter()
        w1 = EOQWeight.from_symbols(sym, scales)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        w2 = EOQWeight.from_rans(raw, scales, (n, k))
        torch.cuda.synchronize()
        t3 = time.perf_counter()
        assert np.array_equal(np.asarray(got, dtype=np.uint8), sym.reshape(-1))
        assert torch.equal(w2.decode_symbols(), w1.decode_symbols())
        per_layer[name] = {"shape": [n, k], "wire_decode_ms": (t1 - t0) * 1e3, "tile_encode_ms": (t2 - t1) * 1e3,
                           "from_rans_ms": (t3 - t2) * 1e3, "wire_encode_ms": enc_s * 1e3}
        tot["wire_decode_s"] += t1 - t0; tot["tile_encode_s"] += t2 - t1; tot["from_rans_s"] += t3 - t2; tot["wire_encode_s"] += enc_s
        weights += n * k
        wire += len(raw)
        keep = [w1, w2]
    line = {"metric": "model load: reference wire format to resident tiles, symbols/s", "unit": "Gsym/s", "n_gpus": 1,
            "higher_is_better": True, "data": "synthetic", "dtype": "u32 rANS state",
            "config": {"workload": "llama7b_block_load_int4_g128_block256_p14", "weights_per_block": weights,
                       "wire_bytes_per_block": wire, "host_threads": os.cpu_count()},
            "value": weights / tot["from_rans_s"] / 1e9, "block_load_s": tot["from_rans_s"],
            "model_32_blocks_s": 32 * tot["from_rans_s"], "first_call_s": first_call_s, "phases_s": tot, "per_layer": per_layer,
            "note": "from_rans = payload to the device + wire decode + tile encoder kernels, symbols never on the host; "
                    "wire_decode = BlockedRANSDecoder.decode_all to a host array; tile_encode = from_symbols from a host array; "
                    "wire_encode is the host encoder behind BlockedRANSEncoder.encode (conversion time, not load time)"}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline line only: skip the Llama-7B step and the prefill GEMM")
    ap.add_argument("--eager", action="store_true", help="plain launches instead of CUDA graphs (for profilers)")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"], help="N > 1: how output slices are exchanged")
    ap.add_argument("--no-pdl", action="store_true", help="plain launches instead of programmatic dependent launches")
    ap.add_argument("--workload", default="mlp_pair",
                    choices=["mlp_pair", "decode_dequant", "polar_q5", "llama7b_step", "prefill_gemm", "wire_decode", "model_load", "packed_gemv"])
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="pass a knob to eoq_b200_tune (e.g. gemv_pairs=0: the one-tile-per-warp ring kernel)")
    args = ap.parse_args()
    if args.tune and args.impl != "reference":
        from eoq_quantization_b200 import _lib
        for kv in args.tune:
            key, _, val = kv.partition("=")
            if _lib.lib().eoq_b200_tune(key.encode(), int(val)) != 0:
                raise SystemExit(f"unknown tuning knob {key!r}")
    if args.no_pdl and args.impl != "reference":
        from eoq_quantization_b200 import _lib
        _lib.lib().eoq_b200_tune(b"pdl", 0)
    if args.workload == "llama7b_step":
        return run_llama_step(args)
    if args.workload == "wire_decode":
        return run_wire_decode(args)
    if args.workload == "model_load":
        return run_model_load(args)
    if args.workload != "mlp_pair":
        args.steps = min(args.steps, 50)
        return run_aux(args)
    args.warmup = max(args.warmup, 3)                       # the same warm-up rule in both arms
    if args.impl == "reference":
        args.steps = min(args.steps, 200)                   # ~0.13 s per step on 16 cores: the run stays within a minute
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
