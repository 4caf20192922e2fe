#!/usr/bin/env python3
"""MobileNetV1-224 inference throughput on the cuda backend (and the CPU reference arm).

    python bench.py --gpus N --steps K --warmup W            # this backend
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU path

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE for N > 1).  The workload is
BASELINE config 5: MobileNetV1-1.0-224 with every filter stored as uint8 affine-quantised
bytes, one global batch of 1024 synthetic images sharded by batch over the N GPUs (strong
scaling, no collective on the data path; torch.distributed over gloo serves only the barrier and
the max-over-ranks of the timings).  `--workload cfg4` runs config 4 instead (float32 weights,
batch 64 per GPU).

A step is one forward pass over the rank's shard: 25 kernel launches (30 with --forward
layerwise, 77 with --forward reference-api) replayed from a CUDA graph.  Before anything is timed
the same code path is checked against the CPU oracle on a few images (`parity_check`).  `value`
is images/s with the images resident in device memory; `e2e` repeats the measurement through the
public API with the shard in pinned host memory, copying it to the device and reading the
probabilities back inside every timed step, and states the host-to-device copy rate of the same
buffers without any kernel as its ceiling.  With N > 1 rank 0 afterwards also times the library's
own in-process runner (one context and one host thread per device, host-side gather) over the
same global batch (`e2e_in_process`).
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
    ap.add_argument("--forward", default="separable", choices=["separable", "layerwise", "reference-api"],
                    help="separable: each depthwise + pointwise pair is one fusedSeparableConv2d call (the "
                         "first five pairs then run as single kernels that keep the depthwise result on "
                         "chip); layerwise: one kernel per layer (30 launches); reference-api: the network "
                         "as unmodified tf.* code expresses it (77 backend calls: conv -> add -> clipByValue, "
                         "the 8-kernel softmax chain)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the extra measurements (in-loop dequantisation, in-process sharded runner)")
    ap.add_argument("--activations", default="f32", choices=["f32", "f16"],
                    help="f16: activations are stored as IEEE half between the layers (the reference's 16-bit "
                         "precision class); a SEPARATE configuration with its own algorithmic-bytes figure, "
                         "never the headline")
    ap.add_argument("--input", default="float32", choices=["float32", "uint8"],
                    help="uint8: the images are pixel bytes (tf.browser.fromPixels) registered as a quantised "
                         "tensor x = q / 127.5 - 1 and decoded by the stem kernel on chip: 4x fewer host-to-device "
                         "bytes; a SEPARATE configuration, never the headline")
    ap.add_argument("--global-batch", type=int, default=0, help="override the workload's batch")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a graph")
    ap.add_argument("--pdl", action="store_true", help="programmatic dependent launch instead of plain stream order")
    ap.add_argument("--streams", type=int, default=0, choices=[0, 1, 2, 3, 4],
                    help="contexts (streams, each with its own activation buffers and captured graph) of the "
                         "GPU that the steps take in turn, so that the CTAs of one step's kernels take the SMs "
                         "that the tail of another step's kernel has left; 0 (default): 4 up to 128 images per "
                         "GPU, else 2; 1: one context, one stream")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-sample", type=int, default=12, help="images in the cpu_baseline sample")
    ap.add_argument("--ref-threads", type=int, default=0, help="host threads of --impl reference (0 = all)")
    return ap.parse_args()


def workload_config(args, world):
    if args.workload == "cfg5":
        gb = args.global_batch or 1024
        assert gb % world == 0, "the global batch must divide evenly over the GPUs"
        how = ("inside the GEMM main loop" if args.dequant == "in-loop"
               else "once on device into cached tf32 planes")
        half = ", float16 activation storage (16-bit precision class: separate configuration)" \
            if getattr(args, "activations", "f32") == "f16" else ""
        if getattr(args, "input", "float32") == "uint8":
            half += ", images as uint8 pixels decoded in the stem (separate configuration)"
        return dict(name="cfg5: MobileNetV1-1.0-224, uint8 affine-quantised filters dequantised %s, "
                         "global batch %d sharded by batch%s" % (how, gb, half),
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
KERNEL_FAMILY = {"separableConv2d (fused dw3x3 s1 + pw, TF32, float16)": "separable_fused",
                 "separableConv2d (fused dw3x3 s2 + pw, TF32, float16)": "separable_fused",
                 "gemm_tcgen05 (F16)": "gemm_tcgen05",
                 "conv2d_tcgen05 (3-channel 3x3, window TMA, TF32, float16 out)": "conv2d_tcgen05",
                 "conv2d_tcgen05 (3-channel 3x3, window TMA, TF32, uint8 in)": "conv2d_tcgen05",
                 "conv2d_tcgen05 (3-channel 3x3, window TMA, TF32, uint8 in, float16 out)": "conv2d_tcgen05",
                 "depthwiseConv2D (3x3 image window, TMA, float16)": "depthwise3x3",
                 "avgPool (global, float16 in)": "global_avgpool",
                 "separableConv2d (fused dw3x3 s1 + pw, TF32)": "separable_fused",
                 "separableConv2d (fused dw3x3 s2 + pw, TF32)": "separable_fused",
                 "gemm_tcgen05 (TF32)": "gemm_tcgen05", "gemm_tcgen05 (3xTF32)": "gemm_tcgen05",
                 "gemm_tcgen05 (TF32, CTA pairs)": "gemm_tcgen05",
                 "gemm_tcgen05 (3xTF32, CTA pairs)": "gemm_tcgen05",
                 "gemm_tcgen05 (TF32, uint8 weights, CTA pairs)": "gemm_tcgen05",
                 "conv2d_tcgen05 (3-channel 3x3, window TMA, 3xTF32)": "conv2d_tcgen05",
                 "conv2d_tcgen05 (shifted-patch TMA, 3xTF32)": "conv2d_tcgen05",
                 "gemm_tcgen05 (TF32, uint8 weights)": "gemm_tcgen05",
                 "gemm_tcgen05 (3xTF32, uint8 weights)": "gemm_tcgen05",
                 "conv2d_tcgen05 (TF32)": "conv2d_tcgen05", "conv2d_tcgen05 (3xTF32)": "conv2d_tcgen05",
                 "conv2d_tcgen05 (3-channel 3x3, window TMA, TF32)": "conv2d_tcgen05",
                 "conv2d_tcgen05 (shifted-patch TMA, TF32)": "conv2d_tcgen05",
                 "depthwiseConv2D (3x3 strip)": "depthwise3x3", "depthwiseConv2D (3x3 image window, TMA)": "depthwise3x3",
                 "conv2d (stem)": "conv2d_stem", "binary (vectorised)": "binary", "binary (general)": "binary",
                 "unary": "unary", "reduce_last": "reduce_last", "pool2d": "pool2d", "pool2d (128-bit)": "pool2d",
                 "avgPool (global)": "global_avgpool", "softmax_last": "softmax"}


def load_measured_traffic():
    """DRAM bytes per image and launch of each kernel family, from the table of ncu captures in
    profiles/dram_traffic_per_launch.md (rows `| family | MB per image per launch | batch | ... |`)."""
    path = os.path.join(ROOT, "profiles", "dram_traffic_per_launch.md")
    table = {}
    if os.path.exists(path):
        for line in open(path):
            cells = [c.strip() for c in line.strip().strip("|").split("|")]
            if len(cells) >= 3 and cells[0] in set(KERNEL_FAMILY.values()):
                try:
                    table[cells[0]] = (float(cells[1]), int(cells[2]))
                except ValueError:
                    continue
    return table


def pick_forward(net, args):
    return {"separable": net.forward_separable, "layerwise": net.forward_fused,
            "reference-api": net.forward_reference_api}[args.forward]


def parity_check(bk, args, images=4):
    """The timed code path (same forward, math mode and uint8 weight handling) on a network whose
    logits mean something -- Glorot weights, stored uint8 when the workload is quantised -- against
    the CPU oracle, before anything is timed.  BASELINE config 5's own weights make a chaotic
    network (the oracle itself is 1e-2 away from exact arithmetic on it), so they cannot serve."""
    import oracle
    from oracle import mobilenet as oracle_net
    from tfjs_core_b200 import mobilenet, ops
    oracle.build()
    params = mobilenet.make_weights(3, gain=1.5)
    if args.workload == "cfg5":
        params = mobilenet.quantize_params(params)
    x = mobilenet.make_input(3, images)
    net = mobilenet.MobileNetV1(params, bk)
    # At the timed batch the deep pointwise layers run on CTA pairs, which the dispatcher would not
    # pick for a handful of images: force them here wherever the shape allows (512-channel layers).
    bk.setOption("gemm_pair", 2)
    try:
        logits, probs = pick_forward(net, args)(ops.tensor(x))
        got = logits.dataSync().reshape(images, -1)
        logits.dispose()
        probs.dispose()
    finally:
        bk.setOption("gemm_pair", 1)
        net.dispose()
    want = np.concatenate([oracle_net.forward(x[i:i + 1], params)[0] for i in range(images)], 0)
    err = float(np.abs(got - want).max() / np.abs(want).max())
    tol = 1e-3 if args.math == "tf32" else 1e-4
    if args.activations == "f16":
        tol = 5e-3   # 16-bit precision class (the reference's own tolerance there is 1e-1)
    same = bool((got.argmax(1) == want.argmax(1)).all())
    assert err <= tol, f"parity check failed: logits differ from the oracle by {err:.2e} (> {tol})"
    assert same, "parity check failed: argmax differs from the oracle"
    return {"images": images,
            "weights": "Glorot (gain 1.5), stored %s" % ("uint8" if args.workload == "cfg5" else "float32"),
            "against": "CPU oracle (restated MathBackendCPU)", "max_rel_err_logits": err, "tolerance": tol,
            "argmax_identical": same}


def run_cuda(args):
    from tfjs_core_b200 import BackendCuda, ENGINE, mobilenet, ops

    d = Dist("gloo")
    cfg = workload_config(args, d.world)
    per = cfg["per_gpu"]
    bk = BackendCuda(d.local_rank, args.math)
    ENGINE.registerBackend("bench-cuda", lambda: bk, 10)
    assert ENGINE.setBackend("bench-cuda")
    bk.setOption("dequant_in_gemm", 1 if args.dequant == "in-loop" else 0)
    bk.setOption("pdl", 1 if args.pdl else 0)
    half = args.activations == "f16"
    if half:
        assert args.math == "tf32" and args.forward != "reference-api", \
            "float16 activation storage goes with --math tf32 and the fused forwards"
        bk.setActivationStorage("float16")

    parity = parity_check(bk, args) if d.rank == 0 else None

    params = mobilenet.make_weights(cfg["seed"], quantized=cfg["quantized"], gain=cfg["gain"])
    net = mobilenet.MobileNetV1(params, bk)
    forward = pick_forward(net, args)
    x_host = mobilenet.make_input(cfg["seed"], per)
    # every rank draws its own slice of the global batch: different seeds per rank keep the
    # generation cheap (skipping d.rank * per images of one stream would cost minutes)
    if d.world > 1:
        rng = np.random.Generator(np.random.PCG64([cfg["seed"], 12345, d.rank]))
        x_host = (rng.random(size=x_host.shape, dtype=np.float32) * 2.0 - 1.0).astype(np.float32)
    pixels = args.input == "uint8"
    if pixels:
        assert args.forward != "reference-api", "pixel input goes with the fused forwards"
        # the same images as bytes: q = round((x + 1) * 127.5), x' = q / 127.5 - 1
        q_host = np.clip(np.rint((x_host + 1.0) * 127.5), 0, 255).astype(np.uint8)
        x_float = (q_host.astype(np.float64) / 127.5 - 1.0).astype(np.float32)   # what the device decodes
        x_host = q_host
        x = bk.registerQuantized(list(q_host.shape), q_host, 1.0 / 127.5, -1.0)
    else:
        x_float = x_host
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

    # ---- more streams: further contexts on the same device, each with its own network, input and
    # captured graph; the steps take them in turn, so that the CTAs of one step's kernels take the
    # SMs that the tail of another step's kernel has already left ----
    n_streams = args.streams if args.streams > 0 else (4 if per <= 128 else 2)
    others = []   # (backend, graph) of the additional contexts
    if n_streams > 1 and graph is not None:
        for k in range(1, n_streams):
            bk_k = BackendCuda(d.local_rank, args.math)
            name = "bench-cuda-%d" % (k + 1)
            ENGINE.registerBackend(name, lambda b=bk_k: b, 9)
            assert ENGINE.setBackend(name)
            try:
                bk_k.setOption("dequant_in_gemm", 1 if args.dequant == "in-loop" else 0)
                bk_k.setOption("pdl", 1 if args.pdl else 0)
                if half:
                    bk_k.setActivationStorage("float16")
                net_k = mobilenet.MobileNetV1(params, bk_k)
                x_k = (bk_k.registerQuantized(list(x_host.shape), x_host, 1.0 / 127.5, -1.0) if pixels
                       else ops.tensor(x_host))
                lg_k, pr_k = pick_forward(net_k, args)(x_k)
                assert np.array_equal(pr_k.dataSync(), first)     # every context computes the same bits
                lg_k.dispose()
                pr_k.dispose()
                bk_k.graphBegin()
                pick_forward(net_k, args)(x_k)
                others.append((bk_k, bk_k.graphEnd()))
            finally:
                assert ENGINE.setBackend("bench-cuda")
        plain_step = step

        def step(counter=[0]):  # noqa: B006 -- the counter is the point
            turn = counter[0] % (len(others) + 1)
            counter[0] += 1
            if turn == 0:
                return plain_step()
            bk_k, graph_k = others[turn - 1]
            bk_k.graphLaunch(graph_k)
            return None

    def timed(fn):
        """Device time of fn's launches: CUDA events on the launching stream; with several streams
        all are bracketed (their start events are recorded back to back on idle streams) and the
        longest span counts."""
        spans = []

        def nest(k):
            if k == len(others):
                return fn()
            spans.append(others[k][0].time(lambda: nest(k + 1))["kernelMs"])
        spans.append(bk.time(lambda: nest(0))["kernelMs"])
        return max(spans)

    def all_launches():
        return bk.launchCount() + sum(b.launchCount() for b, _ in others)

    # ---- device-resident throughput ----
    run_steps(args.warmup)
    bk.sync()
    for bk_k, _ in others:
        bk_k.sync()
    d.barrier()
    sampler = ClockSampler(d.local_rank)
    sampler.start()
    launches_before = all_launches()
    t = {"kernelMs": timed(lambda: run_steps(args.steps))}
    clocks = sampler.stop()
    gpu_launches = all_launches() - launches_before
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
    names = [name for name, _ in rows[:launches_per_step]]
    if args.forward == "reference-api":
        layer_bytes = mobilenet.reference_api_launch_bytes(per, cfg["quantized"], names)
    else:
        layer_bytes = mobilenet.launch_algorithmic_bytes(per, cfg["quantized"], names, half)
        if pixels:
            layer_bytes[0] -= 3 * per * 224 * 224 * 3   # the stem reads one byte per value instead of four
    # per launch of the forward pass: the median over the profile passes (one slow pass, e.g. the
    # first after the graph replays, must not skew a kernel's figure); every pass then counts with it
    import statistics
    typical = [statistics.median(rows[i + k * launches_per_step][1] for k in range(prof_steps))
               for i in range(launches_per_step)]
    rows = [(rows[i][0], typical[i % launches_per_step]) for i in range(launches_per_step * prof_steps)]
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
    measured_traffic = load_measured_traffic()
    traffic, traffic_from = None, None
    if top in measured_traffic:
        mb, at_batch = measured_traffic[top]
        traffic = mb * 1e6 * per
        traffic_from = (f"ncu capture of full-size launches at batch {at_batch}" if at_batch == per else
                        f"ncu capture at batch {at_batch}, scaled to batch {per} (traffic grows with the batch)")
    roofline = {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                "frac": achieved / hbm_peak, "peak_source": peak_kind,
                "launches_per_step": fam[top]["launches"] // prof_steps,
                "avg_launch_ms": fam[top]["ms"] / fam[top]["launches"],
                "share_of_step": fam[top]["ms"] / total_ms,
                "traffic": traffic, "traffic_source": traffic_from}
    kernels = {k: {"ms_per_step": v["ms"] / prof_steps, "share": v["ms"] / total_ms,
                   "launches_per_step": v["launches"] // prof_steps,
                   "achieved_gbs": v["bytes"] / (v["ms"] * 1e-3) / 1e9,
                   "frac_of_hbm_peak": v["bytes"] / (v["ms"] * 1e-3) / 1e9 / hbm_peak} for k, v in fam.items()}
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
    xs = [x, bk.registerQuantized(list(x_host.shape), x_host, 1.0 / 127.5, -1.0) if pixels else ops.tensor(x_host)]
    graphs, outs = [graph], [probs if graph is not None else None]
    if graph is not None:
        bk.graphBegin()
        lg2, pr2 = forward(xs[1])
        graphs.append(bk.graphEnd())
        outs.append(pr2)

    def e2e_run(n, kernels_too=True):
        res = None
        bk.writeAsync(xs[0].dataId, pinned, nbytes)
        for i in range(n):
            cur = i % 2
            if i + 1 < n:
                bk.writeAsync(xs[1 - cur].dataId, pinned, nbytes)
            if not kernels_too:
                continue
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
    # the ceiling of that number: the same uploads from the same pinned buffer with no kernel and
    # no read in between (all ranks at once, as in the run above: GPUs share host uplinks)

    def wait_uploads():
        for t_in in xs:
            lib.tfjs_cuda_tensor_wait(bk._ctx, bk._rec(t_in.dataId)["id"])
        bk.sync()

    e2e_run(2, kernels_too=False)
    wait_uploads()
    d.barrier()
    t0 = time.perf_counter()
    e2e_run(args.steps, kernels_too=False)
    wait_uploads()
    copy_s = d.max(time.perf_counter() - t0)
    d.barrier()
    h2d_gbs_per_gpu = nbytes * args.steps / copy_s / 1e9
    h2d_ceiling_value = cfg["global_batch"] * args.steps / copy_s
    lib.tfjs_cuda_host_free(pinned)
    if len(graphs) > 1:
        bk.graphDestroy(graphs[1])

    # ---- extra: the same step with the uint8 weights dequantised inside the GEMM main loop ----
    extras = {}
    if cfg["quantized"] and args.dequant == "cached" and graph is not None and not args.no_extras and not half \
            and not pixels:
        bk.setOption("dequant_in_gemm", 1)
        lg, pr = forward(x)          # prepares the K-major uint8 layouts
        lg.dispose()
        pr.dispose()
        bk.graphBegin()
        lg_q, pr_q = forward(x)
        g_q = bk.graphEnd()
        for _ in range(3):
            bk.graphLaunch(g_q)
        bk.sync()
        d.barrier()
        n_q = max(3, args.steps // 2)
        tq = bk.time(lambda: [bk.graphLaunch(g_q) for _ in range(n_q)])
        ms_q = d.max(tq["kernelMs"]) / n_q
        same_q = bool(np.array_equal(pr_q.dataSync(), first))
        bk.graphDestroy(g_q)
        lg_q.dispose()
        pr_q.dispose()
        bk.setOption("dequant_in_gemm", 0)
        extras["dequant_in_gemm_main_loop"] = {
            "value": cfg["global_batch"] / (ms_q * 1e-3), "unit": UNIT, "ms_per_step": ms_q,
            "bit_identical_to_cached_planes": same_q,
            "note": "uint8 filters of the GEMM layers stay uint8 in device memory and are dequantised in "
                    "shared memory inside the main loop"}

    # ---- CPU baseline beside it (rank 0, N = 1 only) ----
    cpu_baseline = None
    if d.rank == 0 and d.world == 1 and not args.no_cpu_baseline:
        import oracle
        oracle.build()
        n = args.cpu_sample
        ips, secs = cpu_forward_images_per_second(params, x_float[:n], 1)
        cpu_baseline = {"value": ips, "unit": UNIT, "cores": 1, "kind": "port",
                        "sample": f"first {n} images of the batch, {secs:.1f} s, restated MathBackendCPU "
                                  "(C, unfused passes), 1 thread as the JavaScript original is single-threaded"}

    # ---- extra: the library's in-process runner over all N devices (rank 0, the other ranks idle) ----
    d.barrier()
    if d.rank == 0 and d.world > 1 and not args.no_extras and not args.no_graph and not half and not pixels:
        try:
            extras["e2e_in_process"] = in_process_e2e(args, cfg, params, d.world)
        except Exception as err:  # an extra must never cost the bench line
            extras["e2e_in_process"] = {"error": f"{type(err).__name__}: {err}"}
    d.barrier()

    if d.rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": d.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": cfg["scaling"], "vs_baseline": None,
            "dtype": ("tf32 (float16 activation storage)" if half else "tf32") if args.math == "tf32" else "3xtf32",
            "data": "synthetic",
            "config": {"workload": cfg["name"], "global_batch": cfg["global_batch"], "per_gpu_batch": per,
                       "math_mode": args.math, "dequant": args.dequant, "forward": args.forward,
                       "activation_storage": "float16" if half else "float32", "input": args.input,
                       "launches_per_step": int(launches_per_step),
                       "launch": "eager" if graph is None else "cuda-graph replay",
                       "streams": len(others) + 1,
                       "l2": "every step streams %.1f GB of activations per GPU (> 126 MB L2) between reuses"
                             % (step_bytes / 1e9)},
            "parity_check": parity,
            "roofline": roofline, "net_hbm": {"algorithmic_gb_per_step": step_bytes / 1e9,
                                              "achieved_gbs": net_gbs, "frac": net_gbs / hbm_peak},
            "kernels": kernels, "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": out_bytes,
                    "h2d_ceiling_gbs_per_gpu": h2d_gbs_per_gpu, "h2d_ceiling_value": h2d_ceiling_value,
                    "frac_of_h2d_ceiling": e2e_value / h2d_ceiling_value,
                    "note": ("uint8 pixels, 150 KB per image" if pixels else "float32 images, 602 KB each") +
                            "; the ceiling is the measured rate of the same uploads with no kernel in between"},
            "extras": extras,
            "gpu_launches": int(gpu_launches), "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if graph is not None:
        bk.graphDestroy(graph)
    d.close()


def in_process_e2e(args, cfg, params, n_devices):
    """End to end through the library's own multi-device entry point: one process, one context and
    one host thread per device, uploads from one pinned buffer, host-side gather of the
    [batch, 1000] probabilities into one pinned buffer."""
    from tfjs_core_b200 import ShardedRunner, mobilenet
    batch = cfg["global_batch"]
    options = {"dequant_in_gemm": 1 if args.dequant == "in-loop" else 0}
    runner = ShardedRunner(lambda backend: mobilenet.MobileNetV1(params, backend),
                           lambda net, x: pick_forward(net, args)(x), batch, (224, 224, 3),
                           devices=list(range(n_devices)), math_mode=args.math, options=options)
    try:
        rng = np.random.Generator(np.random.PCG64([cfg["seed"], 777]))
        for slot in runner.input_slots:
            slot[...] = rng.random(size=slot.shape, dtype=np.float32) * 2.0 - 1.0
        runner.run_pipelined(2)
        seen = []
        t0 = time.perf_counter()
        runner.run_pipelined(args.steps, consume=lambda k, res: seen.append(float(res[0].sum())))
        dt = time.perf_counter() - t0
        assert len(seen) == args.steps and all(abs(v - 1.0) < 1e-3 for v in seen), "gathered probabilities are off"
        return {"value": batch * args.steps / dt, "unit": UNIT, "devices": n_devices,
                "host_threads": n_devices, "h2d_bytes_per_step": int(batch * 224 * 224 * 3 * 4),
                "d2h_bytes_per_step": int(batch * 1000 * 4),
                "note": "ShardedRunner.run_pipelined: wall clock of this one process over all devices"}
    finally:
        runner.dispose()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
