#!/usr/bin/env python3
"""MobileNetV1-224 inference throughput on the cuda backend (and the CPU reference arm).

    python bench.py --gpus N --steps K --warmup W            # this backend
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU path

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE for N > 1).  The workload is
BASELINE config 5: MobileNetV1-1.0-224 with every filter stored as uint8 affine-quantised
bytes, one global batch of 1024 synthetic images sharded by batch over the N GPUs (strong
scaling, no collective on the data path; torch.distributed is used only for the barrier and
the max-over-ranks of the timings).  `--workload cfg4` runs config 4 instead (float32 weights,
batch 64 per GPU).

A step is one forward pass over the rank's shard: 26 kernel launches (30 with --forward
layerwise) replayed from a CUDA graph.  `value` is images/s with the images resident in device memory; `e2e` repeats the
measurement through the public API with the shard in pinned host memory, copying it to the
device and reading the probabilities back inside every timed step.
"""
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

METRIC = "MobileNetV1-224 images/s"
UNIT = "img/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--workload", default="cfg5", choices=["cfg5", "cfg4"])
    ap.add_argument("--math", default="tf32", choices=["tf32", "3xtf32"])
    ap.add_argument("--dequant", default="cached", choices=["cached", "in-loop"],
                    help="uint8 weights of the GEMM layers: expanded once into cached tf32 planes, or "
                         "kept uint8 and dequantised in shared memory inside the GEMM main loop")
    ap.add_argument("--forward", default="separable", choices=["separable", "layerwise"],
                    help="separable: each depthwise + pointwise pair is one fusedSeparableConv2d call (the "
                         "first five pairs then run as single kernels that keep the depthwise result on "
                         "chip); layerwise: one kernel per layer (30 launches)")
    ap.add_argument("--global-batch", type=int, default=0, help="override the workload's batch")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a graph")
    ap.add_argument("--pdl", action="store_true", help="programmatic dependent launch instead of plain stream order")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-sample", type=int, default=12, help="images in the cpu_baseline sample")
    ap.add_argument("--ref-threads", type=int, default=0, help="host threads of --impl reference (0 = all)")
    return ap.parse_args()


def workload_config(args, world):
    if args.workload == "cfg5":
        gb = args.global_batch or 1024
        assert gb % world == 0, "the global batch must divide evenly over the GPUs"
        return dict(name="cfg5: MobileNetV1-1.0-224, uint8 affine-quantised filters dequantised on "
                         "device, global batch %d sharded by batch" % gb,
                    global_batch=gb, per_gpu=gb // world, quantized=True, seed=4, gain=1.0,
                    scaling="strong")
    per = args.global_batch or 64
    return dict(name="cfg4: MobileNetV1-1.0-224, float32 filters, batch %d per GPU" % per,
                global_batch=per * world, per_gpu=per, quantized=False, seed=3, gain=1.5, scaling="weak")


# ---- clocks ------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU while a region runs: NVML reads
    every 2 ms from a thread (read-only queries), or `nvidia-smi -lms` when pynvml is missing."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.rows, self.proc = device, [], None
        self.samples, self.stop_flag, self.thread, self.nvml = [], False, None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            index = device
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            if visible:
                entry = visible.split(",")[device].strip()
                index = int(entry) if entry.isdigit() else None
            self.handle = (pynvml.nvmlDeviceGetHandleByIndex(index) if index is not None
                           else pynvml.nvmlDeviceGetHandleByUUID(entry))
            self.nvml = pynvml
        except Exception:
            self.nvml = None

    def _read_nvml(self):
        n = self.nvml
        reasons = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
        names = []
        for name, bit in (("hw_slowdown", n.nvmlClocksEventReasonHwSlowdown),
                          ("hw_thermal_slowdown", n.nvmlClocksEventReasonHwThermalSlowdown),
                          ("sw_thermal_slowdown", n.nvmlClocksEventReasonSwThermalSlowdown),
                          ("sw_power_cap", n.nvmlClocksEventReasonSwPowerCap)):
            if reasons & bit:
                names.append(name)
        return (float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)),
                float(n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)),
                n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0, names)

    def _loop(self):
        while not self.stop_flag:
            try:
                self.samples.append(self._read_nvml())
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nvml is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device), f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        sm, mx, reasons, power = [], [], set(), []
        if self.thread is not None:
            try:  # one more read before the load goes away, so that short regions have a sample
                self.samples.append(self._read_nvml())
            except Exception:
                pass
            self.stop_flag = True
            self.thread.join(timeout=1)
            for s_, m_, p_, names in self.samples:
                sm.append(s_)
                mx.append(m_)
                power.append(p_)
                reasons.update(names)
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                power.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm)}


# ---- distributed plumbing -----------------------------------------------------------------------
class Dist:
    def __init__(self, backend):
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.torch = None
        if self.world > 1:
            import torch
            import torch.distributed as dist
            self.torch, self.dist = torch, dist
            if backend == "nccl":
                torch.cuda.set_device(self.local_rank)
            dist.init_process_group(backend=backend)
            self.device = torch.device("cuda", self.local_rank) if backend == "nccl" else torch.device("cpu")

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()

    def max(self, value):
        if self.world == 1:
            return value
        t = self.torch.tensor([value], dtype=self.torch.float64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


# ---- reference arm ------------------------------------------------------------------------------
def cpu_forward_images_per_second(params, images, threads):
    """Times the CPU oracle (restated MathBackendCPU) over `images`, one image per call, spread
    over `threads` host threads (ctypes releases the GIL)."""
    from oracle import mobilenet as oracle_net
    chunks = [images[i::threads] for i in range(threads)]

    def work(chunk):
        for i in range(chunk.shape[0]):
            oracle_net.forward(chunk[i:i + 1], params)

    t0 = time.perf_counter()
    ts = [threading.Thread(target=work, args=(c,)) for c in chunks if c.shape[0]]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    dt = time.perf_counter() - t0
    return images.shape[0] / dt, dt


def run_reference(args):
    """--impl reference: the reference's own CPU implementation of the path.  tfjs-core's
    MathBackendCPU is TypeScript and no JavaScript runtime exists on the box, so this times its
    C restatement (oracle/) on the host cores.  Each step is a bounded sample of the workload:
    one image per host thread."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from tfjs_core_b200 import mobilenet
    oracle.build()
    cfg = workload_config(args, max(world, 1))
    threads = args.ref_threads or os.cpu_count() or 1
    params = mobilenet.make_weights(cfg["seed"], quantized=cfg["quantized"], gain=cfg["gain"])
    images = mobilenet.make_input(cfg["seed"], threads)
    for _ in range(args.warmup):
        cpu_forward_images_per_second(params, images[:threads], threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_forward_images_per_second(params, images, threads)
    dt = time.perf_counter() - t0
    value = args.steps * threads / dt
    sample = f"{threads} images per step (one per host thread) of the {cfg['global_batch']}-image batch"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": cfg["scaling"], "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": cfg["name"], "global_batch": cfg["global_batch"],
                                        "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "restated MathBackendCPU (C, -O2, unfused passes); the JavaScript original cannot run here",
    }
    print(json.dumps(line), flush=True)


# ---- this backend -------------------------------------------------------------------------------
KERNEL_FAMILY = {"separableConv2d (fused dw3x3 s1 + pw, TF32)": "separable_fused",
                 "separableConv2d (fused dw3x3 s2 + pw, TF32)": "separable_fused",
                 "gemm_tcgen05 (TF32)": "gemm_tcgen05", "gemm_tcgen05 (3xTF32)": "gemm_tcgen05",
                 "gemm_tcgen05 (TF32, uint8 weights)": "gemm_tcgen05",
                 "gemm_tcgen05 (3xTF32, uint8 weights)": "gemm_tcgen05",
                 "conv2d_tcgen05 (TF32)": "conv2d_tcgen05", "conv2d_tcgen05 (3xTF32)": "conv2d_tcgen05",
                 "conv2d_tcgen05 (3-channel 3x3, window TMA, TF32)": "conv2d_tcgen05",
                 "conv2d_tcgen05 (shifted-patch TMA, TF32)": "conv2d_tcgen05",
                 "depthwiseConv2D (3x3 strip)": "depthwise3x3", "depthwiseConv2D (3x3 image window, TMA)": "depthwise3x3",
                 "conv2d (stem)": "conv2d_stem",
                 "avgPool (global)": "global_avgpool", "softmax_last": "softmax"}


def run_cuda(args):
    from tfjs_core_b200 import BackendCuda, ENGINE, mobilenet, ops

    d = Dist("nccl")
    cfg = workload_config(args, d.world)
    per = cfg["per_gpu"]
    bk = BackendCuda(d.local_rank, args.math)
    ENGINE.registerBackend("bench-cuda", lambda: bk, 10)
    assert ENGINE.setBackend("bench-cuda")
    bk.setOption("dequant_in_gemm", 1 if args.dequant == "in-loop" else 0)
    bk.setOption("pdl", 1 if args.pdl else 0)

    params = mobilenet.make_weights(cfg["seed"], quantized=cfg["quantized"], gain=cfg["gain"])
    net = mobilenet.MobileNetV1(params, bk)
    forward = net.forward_separable if args.forward == "separable" else net.forward_fused
    x_host = mobilenet.make_input(cfg["seed"], per, offset=0 if d.world == 1 else 0)
    # every rank draws its own slice of the global batch: different seeds per rank keep the
    # generation cheap (skipping d.rank * per images of one stream would cost minutes)
    if d.world > 1:
        rng = np.random.Generator(np.random.PCG64([cfg["seed"], 12345, d.rank]))
        x_host = (rng.random(size=x_host.shape, dtype=np.float32) * 2.0 - 1.0).astype(np.float32)
    x = ops.tensor(x_host)

    # eager pass: fills the weight-repack cache and the allocator's free lists
    logits, probs = forward(x)
    first = probs.dataSync()
    assert np.isfinite(first).all()
    logits.dispose()
    probs.dispose()

    graph = None
    if not args.no_graph:
        bk.graphBegin()
        logits, probs = forward(x)
        graph = bk.graphEnd()

    def step():
        if graph is not None:
            bk.graphLaunch(graph)
            return None
        lg, pr = forward(x)
        lg.dispose()
        return pr

    def run_steps(n):
        outs = []
        for _ in range(n):
            o = step()
            if o is not None:
                outs.append(o)
                if len(outs) > 2:
                    outs.pop(0).dispose()
        for o in outs:
            o.dispose()

    # ---- device-resident throughput ----
    run_steps(args.warmup)
    bk.sync()
    d.barrier()
    sampler = ClockSampler(d.local_rank)
    sampler.start()
    launches_before = bk.launchCount()
    t = bk.time(lambda: run_steps(args.steps))
    clocks = sampler.stop()
    gpu_launches = bk.launchCount() - launches_before
    d.barrier()
    ms_total = d.max(t["kernelMs"])
    ms_per_step = ms_total / args.steps
    value = cfg["global_batch"] / (ms_per_step * 1e-3)

    # ---- per-kernel device times (eager, events between launches, same stream) ----
    prof_steps = min(args.steps, 5)
    # one untimed eager pass first: the graph keeps its own buffers, so the eager path has to
    # fill the allocator's free lists again (cudaMalloc must not land inside a measured launch)
    before = bk.launchCount()
    lg, pr = forward(x)
    launches_per_step = bk.launchCount() - before
    lg.dispose()
    pr.dispose()
    bk.sync()
    bk.profileBegin(launches_per_step * prof_steps + 8)
    for _ in range(prof_steps):
        lg, pr = forward(x)
        lg.dispose()
        pr.dispose()
    rows = bk.profileEnd()
    layer_bytes = mobilenet.launch_algorithmic_bytes(per, cfg["quantized"],
                                                     [name for name, _ in rows[:launches_per_step]])
    fam = {}
    for i, (name, ms) in enumerate(rows):
        f = KERNEL_FAMILY.get(name, name)
        e = fam.setdefault(f, {"ms": 0.0, "launches": 0, "bytes": 0})
        e["ms"] += ms
        e["launches"] += 1
        e["bytes"] += layer_bytes[i % launches_per_step]
    total_ms = sum(e["ms"] for e in fam.values())
    top = max(fam, key=lambda k: fam[k]["ms"])
    peaks = {}
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peaks = json.load(open(peaks_path))
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured" if peaks else "fallback"
    achieved = fam[top]["bytes"] / (fam[top]["ms"] * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                "frac": achieved / hbm_peak, "peak_source": peak_kind,
                "launches_per_step": fam[top]["launches"] // prof_steps,
                "avg_launch_ms": fam[top]["ms"] / fam[top]["launches"],
                "share_of_step": fam[top]["ms"] / total_ms,
                "traffic": (TRAFFIC_MB_PER_IMAGE_AND_LAUNCH[top] * 1e6 * per
                            if top in TRAFFIC_MB_PER_IMAGE_AND_LAUNCH else None)}
    kernels = {k: {"ms_per_step": v["ms"] / prof_steps, "share": v["ms"] / total_ms,
                   "launches_per_step": v["launches"] // prof_steps,
                   "achieved_gbs": v["bytes"] / (v["ms"] * 1e-3) / 1e9} for k, v in fam.items()}
    step_bytes = sum(layer_bytes)
    net_gbs = step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the public API: pinned host -> device -> forward -> host ----
    # Every step uploads its own input from pinned host memory and reads its probabilities back.
    # Two input tensors (each with its own captured graph) alternate, and the upload of step
    # i + 1 is issued with writeAsync before step i is launched, so it overlaps step i's kernels;
    # the blocking read of step i's result closes the step.
    import ctypes as C
    lib = bk._lib
    nbytes = x_host.nbytes
    pinned = C.c_void_p()
    assert lib.tfjs_cuda_host_alloc(C.byref(pinned), nbytes) == 0
    C.memmove(pinned, x_host.ctypes.data, nbytes)
    out_bytes = per * 1000 * 4
    xs = [x, ops.tensor(x_host)]
    graphs, outs = [graph], [probs if graph is not None else None]
    if graph is not None:
        bk.graphBegin()
        lg2, pr2 = forward(xs[1])
        graphs.append(bk.graphEnd())
        outs.append(pr2)

    def e2e_run(n):
        res = None
        bk.writeAsync(xs[0].dataId, pinned, nbytes)
        for i in range(n):
            cur = i % 2
            if i + 1 < n:
                bk.writeAsync(xs[1 - cur].dataId, pinned, nbytes)
            if graph is not None:
                bk.graphLaunch(graphs[cur], inputs=[xs[cur]])
                res = outs[cur].dataSync()
            else:
                lg, pr = forward(xs[cur])
                res = pr.dataSync()
                lg.dispose()
                pr.dispose()
        return res

    e2e_run(max(2, min(args.warmup, 3)))
    bk.sync()
    d.barrier()
    t0 = time.perf_counter()
    res = e2e_run(args.steps)
    bk.sync()
    e2e_s = d.max(time.perf_counter() - t0)
    d.barrier()
    assert np.isfinite(res).all() and np.allclose(res, first, rtol=0, atol=1e-6)
    e2e_value = cfg["global_batch"] * args.steps / e2e_s
    lib.tfjs_cuda_host_free(pinned)
    if len(graphs) > 1:
        bk.graphDestroy(graphs[1])

    # ---- CPU baseline beside it (rank 0, N = 1 only) ----
    cpu_baseline = None
    if d.rank == 0 and d.world == 1 and not args.no_cpu_baseline:
        import oracle
        oracle.build()
        n = args.cpu_sample
        ips, secs = cpu_forward_images_per_second(params, x_host[:n], 1)
        cpu_baseline = {"value": ips, "unit": UNIT, "cores": 1, "kind": "port",
                        "sample": f"first {n} images of the batch, {secs:.1f} s, restated MathBackendCPU "
                                  "(C, unfused passes), 1 thread as the JavaScript original is single-threaded"}

    if d.rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": d.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": cfg["scaling"], "vs_baseline": None, "dtype": "tf32" if args.math == "tf32" else "3xtf32",
            "data": "synthetic",
            "config": {"workload": cfg["name"], "global_batch": cfg["global_batch"], "per_gpu_batch": per,
                       "math_mode": args.math, "dequant": args.dequant, "forward": args.forward,
                       "launches_per_step": int(launches_per_step), "launch": "eager" if graph is None else "cuda-graph replay",
                       "l2": "every step streams %.1f GB of activations per GPU (> 126 MB L2) between reuses"
                             % (step_bytes / 1e9)},
            "roofline": roofline, "net_hbm": {"algorithmic_gb_per_step": step_bytes / 1e9,
                                              "achieved_gbs": net_gbs, "frac": net_gbs / hbm_peak},
            "kernels": kernels, "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": out_bytes},
            "gpu_launches": int(gpu_launches), "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if graph is not None:
        bk.graphDestroy(graph)
    d.close()


# dram__bytes_read.sum + dram__bytes_write.sum per launch of each kernel family, averaged over
# the family's launches of one forward pass, from the batch-256 (fused blocks: batch-128) ncu
# captures summarised under profiles/; it grows in proportion to the batch.
TRAFFIC_MB_PER_IMAGE_AND_LAUNCH = {"separable_fused": 1934.3 / 5 / 128,
                                   "gemm_tcgen05": 4062.4 / 14 / 256,
                                   "depthwise3x3": 4638.7 / 13 / 256,
                                   "conv2d_tcgen05": 502.7 / 256}


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
