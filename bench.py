#!/usr/bin/env python
"""Benchmark of the rotation/flip-invariant SOM hot path on B200.

Headline workload (the large hexagonal SOM the scaling target is quoted on): hexagonal
SOM of radius 30 (2,791 neurons), 128x128 single-channel images, 90x90 neurons, 64x64
distance region, 720 rotations + flip (1,440 transforms), uint8 distance, Gaussian
neighbourhood sigma 3.0 / damping 0.05, random-uniform SOM, synthetic Gaussian-blob
images.  One step = sequential training on one batch of images (image i+1 sees the SOM
updated by image i).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B]
  python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
  python bench.py --impl reference ...     # the reference's CPU path on the host cores

Prints ONE JSON line (rank 0).  `value` is training images/s with the image batches
resident in HBM; `e2e` is the same metric through the host-buffer entry point (pinned host
images copied in, BMU hit counters copied out, every step).  With N > 1 the neurons are
sharded over the ranks (strong scaling): every rank sees every image, computes distances
for its shard, the shards' best matching units are exchanged, and each rank updates its
own neurons.  Extra blocks of the line: `check` (checksums of a fixed untimed training
prefix, identical for every N), `roofline` / `kernels` / `timeline` (per-phase device
times of a profiled pass), `map` (mapping images/s, images sharded over the ranks),
`other_configs` (the smaller training configurations, one GPU), `cpu_baseline`.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FLOAT, UINT16, UINT8 = 0, 1, 2
WORKLOADS = {
    "C4": dict(name="hex-r30 SOM (2791 neurons) train, 128x128 images, 90x90 neurons, 64x64 ED, 720 rot + flip, uint8",
               som_layout=1, som_dim=61, channels=1, image_dim=128, neuron_dim=90, ed_dim=64,
               rotations=720, flip=True, sigma=3.0, damping=0.05, mode=UINT8, seed=1004),
    "C1": dict(name="10x10 SOM train, 64x64 images, 44x44 neurons, 31x31 ED, 360 rot + flip, uint8",
               som_layout=0, som_dim=10, channels=1, image_dim=64, neuron_dim=44, ed_dim=31,
               rotations=360, flip=True, sigma=1.1, damping=0.2, mode=UINT8, seed=1001),
    "C2": dict(name="20x20 SOM map, 128x128 images, 90x90 neurons, 64x64 ED, 360 rot + flip, float32",
               som_layout=0, som_dim=20, channels=1, image_dim=128, neuron_dim=90, ed_dim=64,
               rotations=360, flip=True, sigma=1.1, damping=0.2, mode=FLOAT, seed=1002),
    "C3": dict(name="40x40 SOM train, 2x150x150 images, 2x106x106 neurons, 75x75 ED, 360 rot + flip, uint16",
               som_layout=0, som_dim=40, channels=2, image_dim=150, neuron_dim=106, ed_dim=75,
               rotations=360, flip=True, sigma=2.0, damping=0.1, mode=UINT16, seed=1003),
}
WORKLOAD = WORKLOADS["C4"]
POOL_IMAGES = 2048          # distinct synthetic images; steps take consecutive, wrapping slices of the pool
CHECK_IMAGES = 64           # untimed prefix whose results are checksummed


def som_size(w):
    """Neurons of the SOM grid: dim x dim (cartesian) or the hexagon of side dim (3 r (r + 1) + 1, r = (dim - 1) / 2)."""
    if w["som_layout"] == 0:
        return w["som_dim"] ** 2
    r = (w["som_dim"] - 1) // 2
    return 3 * r * (r + 1) + 1


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def tracked_figure(name, key):
    """A figure quoted from a tracked summary under profiles/ (lines `key = value`), or None."""
    path = os.path.join(ROOT, "profiles", name)
    if not os.path.exists(path):
        return None
    with open(path) as f:
        for line in f:
            parts = line.split("=")
            if len(parts) == 2 and parts[0].strip() == key:
                try:
                    return float(parts[1].split()[0])
                except ValueError:
                    return None
    return None


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.proc = index, [], None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                self.samples.append([x.strip() for x in line.split(",")])
        except Exception:
            pass

    def stop(self):
        if self.proc:
            self.proc.terminate()
        self.join(timeout=2)
        sm = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples if len(s) >= 6 for i in range(4) if s[2 + i] == "Active"})
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(sm))


def make_inputs(w, n_images=POOL_IMAGES):
    """Seeded inputs of a workload: (N, SOM [N][P], images [n][C*id*id]).  Pure numpy: loads no compiled library."""
    from pink_b200.synthetic import blob_images, mt19937_uniform
    N = som_size(w)
    P = w["channels"] * w["neuron_dim"] ** 2
    som = mt19937_uniform(N * P, 1234).reshape(N, P)
    pool = blob_images(n_images, w["image_dim"], w["channels"], seed=w["seed"]).reshape(n_images, -1)
    return N, som, pool


# ---------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own CPU Trainer on the host cores
# ---------------------------------------------------------------------------------------------

def reference_stepper(w, N, som, pool):
    """Returns (step(i), kind, cores).  All host threads are used whatever the launcher exported."""
    threads = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(threads)          # torch.distributed.run exports 1
    import oracle as O
    if O.have_ref():
        O.ref().ref_set_num_threads(threads)
        sess = O.RefSession(som.reshape(N, w["channels"], w["neuron_dim"], w["neuron_dim"]), w["som_layout"],
                            w["som_dim"], w["som_dim"], 0 if w["channels"] == 1 else w["channels"], w["image_dim"],
                            w["neuron_dim"], w["ed_dim"], w["rotations"], w["flip"], O.FUNC_GAUSSIAN, w["sigma"],
                            w["damping"])
        n = len(pool)
        return (lambda i: sess.train(pool[i % n:i % n + 1])), "reference", int(O.ref().ref_num_threads())
    F = O.update_factors(w["som_layout"], w["som_dim"], w["som_dim"], O.FUNC_GAUSSIAN, w["sigma"], w["damping"])
    s = som.reshape(N, w["channels"], w["neuron_dim"], w["neuron_dim"]).copy()
    shape = (w["channels"], w["image_dim"], w["image_dim"])
    n = len(pool)
    return (lambda i: O.train_step(s, pool[i % n].reshape(shape), F, w["ed_dim"], w["rotations"], w["flip"], 0)), "port", 1


def cpu_baseline(w, N, som, pool, budget_s=12.0, max_images=4):
    """Times the reference's CPU training step (float32, its only CPU mode) on the first images of the workload."""
    step, kind, cores = reference_stepper(w, N, som, pool)
    t0 = time.perf_counter()
    n = 0
    while n < max_images and (n == 0 or time.perf_counter() - t0 < budget_s):
        step(n)
        n += 1
    dt = time.perf_counter() - t0
    return dict(value=n / dt, unit="images/s", cores=cores, kind=kind, host_cpus=os.cpu_count() or 1,
                sample="first %d images of the workload, float32 distance (the reference has no integer CPU mode), "
                       "%.1f s wall" % (n, dt))


def run_reference(args, w):
    """The reference's own CPU implementation on the host cores; one step = one image."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    N, som, pool = make_inputs(w, 64)
    step, kind, cores = reference_stepper(w, N, som, pool)
    for i in range(args.warmup):
        step(i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(args.warmup + i)
    dt = time.perf_counter() - t0
    v = args.steps / dt
    sample = "1 image per step, float32 distance (the reference's CPU path has no integer mode), %d threads" % cores
    print(json.dumps({
        "impl": "reference", "metric": "train_images_per_sec", "value": v, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["name"], "images_per_step": 1},
        "cpu_baseline": {"value": v, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------

def crc(a):
    return "%08x" % (zlib.crc32(np.ascontiguousarray(a).tobytes()) & 0xFFFFFFFF)


def training_check(eng, som, pool, n_images, reduce=None):
    """Trains the first n_images of the pool on the seeded SOM and returns checksums of the BMU sequence, the hit
    counters and the trained SOM.  uint8 training is bit-exact, so the values do not depend on the number of
    ranks.  reduce(array, op): combines the ranks' partial results ("min" / "sum"); None for a single rank."""
    eng.set_som(som)
    counts0 = eng.update_counts().astype(np.int64)       # the counters run over the context's whole life
    eng.train(pool[:n_images])
    eng.synchronize()
    bmus = eng.bmu_log(n_images).astype(np.int64)        # 0xFFFFFFFF where another rank owns the unit
    counts = eng.update_counts().astype(np.int64) - counts0
    part = eng.get_som(np.zeros_like(som))
    if reduce is not None:
        bmus, counts, part = reduce(bmus, "min"), reduce(counts, "sum"), reduce(part, "sum")
    return {"images": n_images, "bmu_crc32": crc(bmus.astype(np.uint32)), "counts_crc32": crc(counts.astype(np.uint32)),
            "som_crc32": crc(part.astype(np.float32)), "bmu_first8": [int(b) for b in bmus[:8]]}


def make_engine(w, N, device, rank=0, world=1, max_batch=0, options=None):
    from pink_b200 import engine
    return engine.Engine(N, w["channels"], w["image_dim"], w["neuron_dim"], w["ed_dim"], w["rotations"], w["flip"],
                         w["mode"], device=device, rank=rank, world_size=world, max_batch=max_batch, options=options)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=512, help="images per step")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the map / other-configuration / reference-GPU blocks")
    ap.add_argument("--option", action="append", default=[], help="context switch name=value (see pink_b200_set_option)")
    ap.add_argument("--only", default=None, help="profiling aid: run one small pass of map-C4, map-C2, train-C1 or train-C3 "
                                                 "(few images, no timing contract) and print its figures")
    ap.add_argument("--images", type=int, default=64, help="images of an --only pass")
    args = ap.parse_args()
    w = WORKLOAD
    if args.impl == "reference":
        return run_reference(args, w)
    if args.only:
        return run_only(args)
    if args.warmup < 3:
        args.warmup = 3
    options = {k: int(v) for k, v in (o.split("=") for o in args.option)}

    import torch
    import torch.distributed as dist
    from pink_b200 import capi, engine

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        sys.exit("bench.py --gpus %d must be launched with torch.distributed.run (one rank per GPU)" % args.gpus)
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def reduce(a, op):
        if world == 1:
            return a
        t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MIN if op == "min" else dist.ReduceOp.SUM)
        return t.cpu().numpy()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    N, som, pool = make_inputs(w)
    F = engine.update_factors(w["som_layout"], w["som_dim"], w["som_dim"], capi.FUNC_GAUSSIAN, w["sigma"], w["damping"])
    B = args.batch
    isz = pool.shape[1]
    eng = make_engine(w, N, local, rank, world, B, options)
    if world > 1:
        uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(engine.Engine.unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        eng.comm_init(bytes(uid.cpu().numpy()))
    # one factor per distance class of the grid; F (the N x N table of the same factors) only serves the accounting below
    eng.set_update_function(w["som_layout"], w["som_dim"], w["som_dim"], capi.FUNC_GAUSSIAN, w["sigma"], w["damping"])

    # ---- untimed: a fixed training prefix whose results must not depend on the number of ranks -----------
    check = training_check(eng, som, pool, CHECK_IMAGES, reduce if world > 1 else None)

    d_pool = torch.from_numpy(pool).cuda()
    h_pool = torch.from_numpy(pool).pin_memory()
    stream = torch.cuda.ExternalStream(eng.stream)
    n_slices = POOL_IMAGES // B

    def slice_ptr(t, step):
        return t.data_ptr() + (step % n_slices) * B * isz * 4

    def timed(fn, steps, sync, ev_stream):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ev_stream)
        for s in range(steps):
            fn(s)
        e1.record(ev_stream)
        sync()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- device-resident training throughput ---------------------------------------------------------------
    step_dev = lambda s: eng.train_device(slice_ptr(d_pool, s), B)
    for s in range(args.warmup):
        step_dev(s)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    exchange_kind = eng.exchange_kind()
    launches0 = eng.launch_count()
    ms = timed(lambda s: step_dev(args.warmup + s), args.steps, eng.synchronize, stream)
    launches = eng.launch_count() - launches0          # kernels of this library launched inside the timed region
    clocks = sampler.stop() if rank == 0 else None
    value = args.steps * B / (ms * 1e-3)

    # ---- end to end: pinned host images in, BMU hit counters out, every step -------------------------------
    counts = np.empty(N, np.uint32)

    def step_e2e(s):
        capi.check(capi.lib.pink_b200_train(eng._h, slice_ptr(h_pool, s), B))
        capi.check(capi.lib.pink_b200_get_update_counts(eng._h, counts.ctypes.data))
    for s in range(3):
        step_e2e(s)
    ms_e2e = timed(step_e2e, args.steps, eng.synchronize, stream)
    e2e = args.steps * B / (ms_e2e * 1e-3)

    # ---- per-phase device time (separate profiled pass of the same workload) -------------------------------
    prof_steps = min(B, 256)
    stats0 = eng.update_stats()
    eng.profile_begin(prof_steps)
    eng.train_device(slice_ptr(d_pool, 1), prof_steps)
    phase_ms, covered = eng.profile_end()
    detail = eng.profile_detail()
    stats1 = eng.update_stats()

    peaks = measured_peaks()
    T = w["rotations"] * (2 if w["flip"] else 1)
    K = w["channels"] * w["ed_dim"] ** 2
    P = w["channels"] * w["neuron_dim"] ** 2
    nl = eng.count
    # Update traffic.  Algorithmic (what the reference's kernel moves): every neuron of this shard with a non-zero
    # factor for the image's best matching unit is read and written once, 8 * N_upd * P.  Moved: the kernel leaves
    # out neurons that provably cannot change and does not write back neurons in which no value changed (both
    # counted on the device), with bit-identical maps: 4 P per neuron read + (4 P + K) per neuron written.
    bmus = reduce(eng.bmu_log(prof_steps).astype(np.int64), "min")
    nz_rows = (F[:, eng.neurons] != 0).sum(1)
    n_upd = float(nz_rows[bmus[bmus < N]].mean())
    n_read = (stats1[0] - stats0[0]) / prof_steps
    n_written = (stats1[1] - stats0[1]) / prof_steps
    t_dist = phase_ms["distance"] / covered * 1e-3
    t_bmu = phase_ms["bmu"] / covered * 1e-3
    t_upd = phase_ms["update"] / covered * 1e-3
    t_rot = phase_ms["rotate"] / covered * 1e-3
    dist_ops = 2.0 * nl * T * K
    upd_bytes = 8.0 * n_upd * P
    moved_bytes = 4.0 * P * n_read + (4.0 * P + K) * n_written
    int8_peak = 2.0 * peaks["bf16_tflops"]
    mma_peak = None                                  # tcgen05.mma kind::i8 alone on resident operands, measured now
    if world == 1:
        import ctypes
        tops = ctypes.c_double(0.0)
        pair_opt = dict(o.split("=") for o in args.option).get("mma_pairs", "1") != "0"
        capi.check(capi.lib.pink_b200_mma_i8_peak(local, 240, 1 if pair_opt else 0, ctypes.byref(tops)))
        mma_peak = tops.value
    fused = detail["launch_us"] > 0                  # the persistent kernel ran: phases come from device-timer stamps
    timing = ("device-timer stamps of block 0 inside the persistent kernel, each phase up to and including its grid "
              "barrier, %d steps" % covered) if fused else \
             ("CUDA events around every launch in a separate profiled pass of %d steps" % covered)
    kernels = {
        "update": {"bound": "hbm", "achieved": moved_bytes / t_upd / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                   "frac": moved_bytes / t_upd / 1e9 / peaks["hbm_gbs"], "us_per_image": t_upd * 1e6,
                   "moved_bytes": moved_bytes, "neurons_read": n_read, "neurons_written": n_written,
                   "effective_bytes": upd_bytes, "effective_frac": upd_bytes / t_upd / 1e9 / peaks["hbm_gbs"],
                   "neurons_with_nonzero_factor": n_upd,
                   "note": "achieved / frac use the bytes the kernel moves; effective_* the 8 * N_upd * P the "
                           "reference's kernel would move for the same step"},
        "distance": {"bound": "tensor", "achieved": dist_ops / t_dist / 1e12, "peak": int8_peak, "unit": "TOP/s",
                     "frac": dist_ops / t_dist / 1e12 / int8_peak, "us_per_image": t_dist * 1e6,
                     "algorithmic_ops": dist_ops,
                     "peak_note": "int8 peak taken as 2 x the %s bf16 cuBLAS figure" % peaks["source"],
                     "frac_of_mma_only_peak": (dist_ops / t_dist / 1e12 / mma_peak) if mma_peak else None,
                     "mma_only_peak_tops": mma_peak,
                     "mma_only_peak_note": "pink_b200_mma_i8_peak: the same instruction shape back to back on operands "
                                           "resident in shared memory, one CTA pair per SM, no loads and no epilogue"},
        "bmu+exchange+list": {"us_per_image": t_bmu * 1e6},
        "rotate": {"us_per_image": t_rot * 1e6},
    }
    roof = dict(kernels["update"] if t_upd >= t_dist else kernels["distance"])
    roof["kernel"] = ("train_steps_kernel, " if fused else "") + ("update phase" if t_upd >= t_dist else "distance phase")
    roof["peak_source"] = peaks["source"]
    roof["timing"] = timing
    # DRAM bytes of one image's share of a launch, from the tracked ncu summary, scaled by the bytes the live pass moved
    cap_traffic = tracked_figure("train_steps_kernel_u8_c4.txt", "dram_bytes_per_image")
    cap_moved = tracked_figure("train_steps_kernel_u8_c4.txt", "moved_bytes_per_image")
    roof["traffic"] = cap_traffic * moved_bytes / cap_moved if (cap_traffic and cap_moved and world == 1) else None
    roof["traffic_note"] = ("profiles/train_steps_kernel_u8_c4.txt (dram__bytes_read + write per image of a captured "
                            "launch), scaled by moved_bytes live / captured") if roof["traffic"] else None
    timeline = None
    if fused:
        sol_us = dist_ops / (int8_peak * 1e12) * 1e6 + moved_bytes / (peaks["hbm_gbs"] * 1e9) * 1e6
        per_image = detail["launch_us"] / max(detail["images_per_launch"], 1.0)
        timeline = dict(detail)
        timeline.update({"us_per_image_in_kernel": per_image, "rotate_us_per_image": t_rot * 1e6,
                         "step_us_per_image_measured": ms / args.steps * 1e3 / B,
                         "speed_of_light_us_per_image": sol_us, "frac_of_speed_of_light": sol_us / per_image,
                         "note": "launch_us: CUDA events around one launch of the persistent kernel; speed of light = "
                                 "distance ops / int8 peak + moved update bytes / HBM peak (the phases depend on each "
                                 "other and cannot overlap)"})

    # ---- mapping throughput: images sharded over the ranks, one whole-SOM context per rank -----------------
    extras = {}
    if not args.no_extras:
        eng.close()
        eng = None
        extras["map"] = bench_map(torch, dist, barrier, rank, world, local, som, pool)
        if world == 1:
            extras["other_configs"] = bench_other_configs(torch, local)
            extras["distance_sweep"] = bench_distance_sweep(torch)
            extras["cli"] = bench_cli(w, pool)
            extras["python_api"] = bench_python_api(w, som, pool)
            extras["reference_gpu"] = bench_reference_gpu(w, som, pool)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cpu = cpu_baseline(w, N, som, pool)
        except Exception as ex:          # the checker is optional equipment of the benchmark
            cpu = {"unavailable": repr(ex)}

    if rank == 0:
        line = {
            "metric": "train_images_per_sec", "value": value, "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": w["name"], "images_per_step": B, "parallelism": "neuron-shard x%d" % world,
                       "exchange": {0: "none", 1: "nccl all-gather", 2: "peer-memory records",
                                    3: "peer-memory records + shared rotation work"}[exchange_kind],
                       "options": options,
                       "l2": "every step trains on a different slice of a 134 MB image pool; SOM (90 MB) + operand "
                             "(11 MB) + batch (34 MB) exceed the 126 MB L2"},
            "e2e": {"value": e2e, "unit": "images/s", "h2d_bytes_per_step": B * isz * 4, "d2h_bytes_per_step": N * 4,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "check": check,
            "roofline": roof,
            "kernels": kernels,
            "timeline": timeline,
            "cpu_baseline": cpu,
        }
        line.update(extras)
        print(json.dumps(line))
    if eng is not None:
        eng.close()
    if world > 1:
        dist.destroy_process_group()


def run_only(args):
    """One small pass of one configuration's path (for profilers: few launches, little memory)."""
    import torch
    from pink_b200 import capi
    torch.cuda.set_device(0)
    kind, key = args.only.split("-")
    w = WORKLOADS[key]
    N, som, pool = make_inputs(w, args.images)
    eng = make_engine(w, N, 0, options={k: int(v) for k, v in (o.split("=") for o in args.option)})
    eng.set_som(som)
    d_img = torch.from_numpy(pool).cuda()
    out = {"only": args.only, "workload": w["name"], "images": args.images}
    if kind == "map":
        d_dist = torch.empty((args.images, N), dtype=torch.float32, device="cuda")
        d_rot = torch.empty((args.images, N), dtype=torch.int32, device="cuda")
        for rep in range(2):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            eng.map_device(d_img.data_ptr(), args.images, d_dist.data_ptr(), d_rot.data_ptr())
            eng.synchronize()
            out["images_per_s"] = args.images / (time.perf_counter() - t0)
        if w["mode"] == 0:
            out["filter"] = eng.map_filter_stats()
    else:
        eng.set_update_function(w["som_layout"], w["som_dim"], w["som_dim"], capi.FUNC_GAUSSIAN, w["sigma"], w["damping"])
        for rep in range(2):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            eng.train_device(d_img.data_ptr(), args.images)
            eng.synchronize()
            out["images_per_s"] = args.images / (time.perf_counter() - t0)
        out["update_stats"] = eng.update_stats()
    eng.close()
    print(json.dumps(out))


def bench_map(torch, dist, barrier, rank, world, local, som4, pool4):
    """Mapping images/s of C4 (uint8) and C2 (float32): every rank holds the whole SOM and maps its share of the
    images (round robin); device-resident and through host buffers (pinned images in, results out)."""
    out = {}
    for key, n_img in (("C4", 2048), ("C2", 2048)):
        w = WORKLOADS[key]
        if key == "C4":
            N, som, pool = som_size(w), som4, pool4
        else:
            N, som, pool = make_inputs(w, n_img)
        mine = np.ascontiguousarray(pool[rank::world])
        n = len(mine)
        eng = make_engine(w, N, local)
        eng.set_som(som)
        d_img = torch.from_numpy(mine).cuda()
        d_dist = torch.empty((n, N), dtype=torch.float32, device="cuda")
        d_rot = torch.empty((n, N), dtype=torch.int32, device="cuda")
        h_img = torch.from_numpy(mine).pin_memory()
        h_dist = torch.empty((n, N), dtype=torch.float32).pin_memory()
        h_rot = torch.empty((n, N), dtype=torch.int32).pin_memory()
        from pink_b200 import capi
        dev = lambda: eng.map_device(d_img.data_ptr(), n, d_dist.data_ptr(), d_rot.data_ptr())
        host = lambda: capi.check(capi.lib.pink_b200_map(eng._h, h_img.data_ptr(), n, h_dist.data_ptr(), h_rot.data_ptr()))
        res = {}
        for name, fn in (("value", dev), ("e2e", host)):
            fn()
            eng.synchronize()
            reps = 3
            barrier()
            t0 = time.perf_counter()
            for _ in range(reps):
                fn()
            eng.synchronize()
            barrier()
            dt = torch.tensor([time.perf_counter() - t0], device="cuda")
            if world > 1:
                dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            res[name] = reps * len(pool) / float(dt.item())
        T = w["rotations"] * (2 if w["flip"] else 1)
        K = w["channels"] * w["ed_dim"] ** 2
        res.update({"unit": "images/s", "workload": w["name"], "images": len(pool), "sharding": "images round robin x%d" % world,
                    "distance_ops_per_image": 2.0 * N * T * K,
                    "timing": "host clock around %d whole passes, synchronised on both sides, max over ranks" % reps})
        if w["mode"] == 0:
            st = eng.map_filter_stats()              # float32: tensor-core estimate + exact pass
            res["filter"] = {"exact_sums_per_neuron_and_image": st["pairs_exact"] * w["rotations"] * (2 if w["flip"] else 1)
                             / max(st["pairs_estimated"], 1.0), "worst_estimate_error": st["worst_estimate_error"],
                             "error_bound": st["error_bound"]}
        out[key] = res
        eng.close()
    return out


def bench_cli(w, pool, n_images=2048, epochs=8):
    """The command line program on a data file (the reference's `Pink --train`): images/s of its training loop,
    file reading included (reader thread, pinned double buffer), from the program's own progress clock."""
    import re, subprocess, tempfile
    from pink_b200 import build as B, files
    if not os.path.exists(B.CLI):
        return {"unavailable": "pink_b200/Pink is not built"}
    n_images = min(n_images, len(pool))
    with tempfile.TemporaryDirectory() as tmp:
        data, som_path = os.path.join(tmp, "data.bin"), os.path.join(tmp, "som.bin")
        files.write_data_file(data, pool[:n_images].reshape(n_images, w["image_dim"], w["image_dim"]))
        cmd = [B.CLI, "--layout", "hexagonal" if w["som_layout"] == 1 else "cartesian", "--som-width", str(w["som_dim"]),
               "--som-height", str(w["som_dim"]), "--numrot", str(w["rotations"]), "--neuron-dimension", str(w["neuron_dim"]),
               "--euclidean-distance-dimension", str(w["ed_dim"]), "--euclidean-distance-type", "uint8", "--seed", "1234",
               "--init", "random", "--num-iter", str(epochs), "--dist-func", "gaussian", str(w["sigma"]), str(w["damping"]),
               "--input-shuffle-off", "--progress", "4", "--train", data, som_path]
        t0 = time.perf_counter()
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        wall = time.perf_counter() - t0
    if r.returncode != 0:
        return {"unavailable": (r.stdout + r.stderr)[-300:]}
    marks = re.findall(r"\] 100 % ([0-9.]+) s", r.stdout)
    if not marks:
        return {"unavailable": "no progress line in the program's output"}
    loop_s = float(marks[-1])
    return {"value": n_images * epochs / loop_s, "unit": "images/s", "images": n_images, "epochs": epochs,
            "loop_seconds": loop_s, "process_seconds": wall,
            "note": "Pink --train on a data file of the bench workload, all visible GPUs of the process (here one); "
                    "loop time from the program's progress output, process time includes start-up and writing the map"}


def bench_python_api(w, som, pool, n_images=2048):
    """The reference's Python usage (python/pink/train.py): one Trainer call per image from a Python loop, then
    update_som(); through the compiled module pink_b200._pink."""
    try:
        from pink_b200 import _pink as pink
    except ImportError as ex:
        return {"unavailable": "pink_b200._pink is not built: %s" % ex}
    N = som_size(w)
    n_images = min(n_images, len(pool))
    images = pool[:n_images].reshape(n_images, w["image_dim"], w["image_dim"])
    hexa = w["som_layout"] == 1
    shape = (N, w["neuron_dim"], w["neuron_dim"]) if hexa else (w["som_dim"], w["som_dim"], w["neuron_dim"], w["neuron_dim"])
    som_obj = pink.SOM(np.ascontiguousarray(som.reshape(shape)), som_layout="hexagonal-2d" if hexa else "cartesian-2d")
    trainer = pink.Trainer(som_obj, pink.GaussianFunctor(w["sigma"], w["damping"]), number_of_rotations=w["rotations"],
                           use_flip=bool(w["flip"]), euclidean_distance_dim=w["ed_dim"],
                           euclidean_distance_type=pink.DataType.UINT8)
    for i in range(32):                              # context creation and warm-up
        trainer(pink.Data(images[i]))
    trainer.update_som()
    t0 = time.perf_counter()
    for i in range(n_images):
        trainer(pink.Data(images[i]))
    trainer.update_som()
    dt = time.perf_counter() - t0
    return {"value": n_images / dt, "unit": "images/s", "images": n_images,
            "note": "for i: trainer(pink.Data(image[i])); then trainer.update_som() -- wall clock of the Python loop"}


def bench_distance_sweep(torch):
    """Distance kernel alone over the grid of shapes BASELINE.json names (neurons x region size x rotations, all three
    distance types): 2 * N * T * K multiply-adds per image and second, operands resident, 8 images per launch."""
    import ctypes
    from pink_b200 import capi
    out = {"unit": "Tera multiply-add operations/s (2 * N * T * K per image)", "images_per_launch": 8,
           "timing": "CUDA events around 3 launches after one warm-up launch", "shapes": []}
    n_img = 8
    ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    gen = torch.Generator(device="cuda").manual_seed(5)
    for mode, name in ((2, "uint8"), (1, "uint16"), (0, "float32")):
        rates = []
        for N in (400, 1600, 2791):
            for K in (44 * 44, 64 * 64, 90 * 90):
                for R in (90, 360, 720):
                    T = 2 * R
                    Kp = capi.lib.pink_b200_operand_stride(K, mode)

                    def planes(rows):
                        if mode == 0:
                            x = torch.rand((rows, Kp), device="cuda", generator=gen)
                            x[:, K:] = 0
                            return x, None, None
                        hi = torch.randint(0, 256, (rows, Kp), dtype=torch.uint8, device="cuda", generator=gen)
                        hi[:, K:] = 0
                        if mode == 2:
                            return hi, None, (hi.to(torch.int64) ** 2).sum(1).to(torch.int32)
                        lo = torch.randint(0, 256, (rows, Kp), dtype=torch.uint8, device="cuda", generator=gen)
                        lo[:, K:] = 0
                        v = hi.to(torch.int64) * 256 + lo.to(torch.int64)
                        return hi, lo, (v * v).sum(1)
                    a0, a1, an = planes(N)
                    b0, b1, bn = planes(n_img * T)
                    keys = torch.full((n_img, N), -1, dtype=torch.int64, device="cuda")
                    call = lambda: capi.check(capi.lib.pink_b200_op_distance(mode, N, T, K, ptr(a0), ptr(a1), ptr(an), ptr(b0),
                                                                             ptr(b1), ptr(bn), n_img, ptr(keys), None, None))
                    call()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(3):
                        call()
                    e1.record()
                    torch.cuda.synchronize()
                    capi.check(capi.lib.pink_b200_op_status())
                    rate = 3 * n_img * 2.0 * N * T * K / (e0.elapsed_time(e1) * 1e-3) / 1e12
                    rates.append(rate)
                    out["shapes"].append([name, N, K, R, round(rate, 1)])
        rates.sort()
        out[name] = {"min": rates[0], "median": rates[len(rates) // 2], "max": rates[-1]}
    return out


def bench_reference_gpu(w, som, pool, n_images=24):
    """The reference's own CUDA path (unmodified, compiled for sm_100a) on the same GPU and workload: images/s of its
    Trainer and Mapper, uint8 distances, on the first images of the pool.  Runs in a child process."""
    import oracle as O
    if not O.have_ref_cuda():
        return {"unavailable": "the reference's CUDA path was not built (its source tree was absent at build time)"}
    N = som_size(w)
    out = {"workload": w["name"], "images": n_images, "unit": "images/s",
           "note": "reference Trainer / Mapper with UseGPU = true, one visible GPU, wall clock of its own loop after one warm-up step"}
    args = (som.reshape(N, w["neuron_dim"], w["neuron_dim"]), pool[:n_images].reshape(n_images, w["image_dim"], w["image_dim"]),
            w["som_layout"], w["som_dim"], w["som_dim"], w["image_dim"], w["neuron_dim"], w["ed_dim"], w["rotations"], w["flip"], w["mode"])
    for task in ("train", "map"):
        try:
            r = O.ref_cuda_run(task, *args, sigma=w["sigma"], damping=w["damping"], timeout=240)
            out[task] = n_images / float(r["seconds"])
        except Exception as ex:
            out[task] = None
            out[task + "_error"] = str(ex)[:300]
    if out.get("train") is None and out.get("map") is None:
        return out                        # its uint8 run failed: the float run is not tried
    for task in ("train", "map"):         # the same geometry with float distances (the reference's default type)
        try:
            r = O.ref_cuda_run(task, *(args[:-1] + (0,)), sigma=w["sigma"], damping=w["damping"], timeout=240)
            out[task + "_float"] = n_images / float(r["seconds"])
        except Exception as ex:
            out[task + "_float"] = None
            out[task + "_float_error"] = str(ex)[:300]
    return out


def bench_other_configs(torch, local):
    """Training images/s of the smaller configurations (one GPU, device-resident images)."""
    from pink_b200 import capi, engine
    out = {}
    for key, n_img in (("C1", 2000), ("C3", 256)):
        w = WORKLOADS[key]
        N, som, pool = make_inputs(w, n_img)
        eng = make_engine(w, N, local)
        eng.set_som(som)
        eng.set_update_function(w["som_layout"], w["som_dim"], w["som_dim"], capi.FUNC_GAUSSIAN, w["sigma"], w["damping"])
        d_pool = torch.from_numpy(pool).cuda()
        eng.train_device(d_pool.data_ptr(), n_img)
        eng.synchronize()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.train_device(d_pool.data_ptr(), n_img)
        eng.synchronize()
        dt = time.perf_counter() - t0
        eng.profile_begin(min(n_img, 128))
        eng.train_device(d_pool.data_ptr(), min(n_img, 128))
        phase_ms, covered = eng.profile_end()
        out[key] = {"value": n_img / dt, "unit": "images/s", "workload": w["name"], "images": n_img,
                    "phase_us_per_image": {k: v / covered * 1e3 for k, v in phase_ms.items()},
                    "persistent_kernel": eng.profile_detail()["launch_us"] > 0}
        eng.close()
    return out


if __name__ == "__main__":
    main()
