"""Benchmark of the activation compress / decompress hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

One STEP = one pass of the adaptive (per-sample bit width, the default level L3) codec over
one batch of synthetic activations: a bfloat16 activation of shape [512, 256, 28, 28]
(102.8 M elements, 256-element groups) whose samples have LogNormal(0, 1) sensitivities is
compressed at a 2.0-bit average budget with ONE native call (per-group min/max ->
per-sample sensitivity -> greedy bit allocation -> stochastic rounding and mixed-precision
pack) and a compressed activation is decompressed again.  Metric: algorithmic GB/s of
compress + decompress.  Per element (s = 2 bytes, b = 2 bits average, two 2-byte
statistics per 256-element group):
    compress    2 s + b/8 + 2*2/256   (the activation is necessarily read twice: the widths
                                       depend on the ranges of all samples)    = 438.3 MB
    decompress  b/8 + 2*2/256 + s                                              = 232.8 MB

The printed JSON line carries
  value       device-resident throughput (inputs in HBM, raw C-ABI calls, the K steps replayed
              from one CUDA graph, CUDA events; median over the replays, min / max reported);
  e2e         the same work through the public Python API from pinned HOST buffers:
              H2D copy -> quantize_activation(scheme) -> dequantize_activation -> D2H copy,
              three steps in flight on three streams;
  roofline    the kernel of the step that is furthest below the measured HBM copy peak;
  kernels     per-kernel GB/s and fraction of the peak for every kernel of the path, the
              uniform-width fused pair on the float16 [256, 256, 28, 28] and the float32
              [64, 64, 56, 56] activations included;
  resnet50_l3 images/s of a ResNet-50 training step (batch 256 per GPU, float16 autocast):
              stock torch ("exact"), this library without compression (L0) and at level L3;
              DDP + synchronised batch norm when N > 1;
  cpu_baseline  the CPU oracle (a restatement of the reference's simulate path) timed on the
              host cores over a bounded sample of the same workload (rank 0, N = 1 only).
`--impl reference` times only that CPU implementation and prints the reference arm's line.

Inputs rotate through a pool whose total size is several times the 126 MB L2, and a packed
buffer is decoded only after half the pool has been re-written, so neither the activation
reads nor the packed reads are served from L2 (the second read of an activation inside one
compress call may be: that is the library's doing, not the benchmark's).
With N > 1 every rank processes its own batch on its own GPU (the codec is independent per
sample: no data-path collective); value = all ranks' bytes / max-over-ranks time.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = {"name": "cfg3-l3-mixed-codec", "shape": [512, 256, 28, 28], "dtype": "bfloat16", "avg_bits": 2.0,
            "initial_bits": 8, "group_size": 256}
POOL = 6                                    # rotating buffers: 6 x 205.5 MB in, 6 x 27.3 MB packed
REPLAYS = 50                                # timed replays of the K-step graph


def algorithmic_bytes(elements: int, elem_size: int, bits: float, stat_size: int = 2, gs: int = 256,
                      reads: int = 1) -> float:
    """Bytes one direction of the codec must move: the activation (`reads` times), the
    packed codes and the two per-group statistics."""
    return elements * (reads * elem_size + bits / 8.0 + 2.0 * stat_size / gs)


def synthetic_activation(torch, n, c, h, w, dtype, device, seed):
    """ReLU(N(0,1)) samples scaled so that their sensitivities (proportional to the squared
    ranges) are LogNormal(0, 1): sample n is multiplied by exp(z_n / 2)."""
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.relu(torch.randn(n, c * h * w, device=device, generator=g))
    z = torch.randn(n, 1, device=device, generator=g)
    return (x * torch.exp(0.5 * z)).to(dtype).view(n, c * h * w // 256, 256)


# ---------------------------------------------------------------------------------------
# multi-rank bookkeeping (one process per GPU; the codec itself needs no collective)
# ---------------------------------------------------------------------------------------
def init_nccl(dist, torch, dev):
    """Join the NCCL group.  The library prints its version banner on stdout when its first
    communicator is created; stdout carries exactly one JSON line, so file descriptor 1 points at
    stderr until that has happened."""
    sys.stdout.flush()
    saved = os.dup(1)
    try:
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=dev)
        warm = torch.zeros(1, device=dev)
        dist.all_reduce(warm)
        torch.cuda.synchronize()
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


def max_over_ranks(local_ms: float, device=None) -> float:
    """The slowest rank's time: the whole job is as slow as its slowest replica."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(local_ms)
    t = torch.tensor([float(local_ms)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def whole_job_gbs(bytes_per_rank_step: float, world: int, ms_per_step: float) -> float:
    """Aggregate throughput of `world` replicas that each move `bytes_per_rank_step` per step."""
    return world * bytes_per_rank_step / (ms_per_step * 1e-3) / 1e9


# ---------------------------------------------------------------------------------------
# clocks: sampled with NVML from a side thread while the GPU is under load
# ---------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            if visible:
                index = int(visible.split(",")[index]) if visible.split(",")[index].isdigit() else index
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _run(self):
        n = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM))
                mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nvml:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "window": "unavailable"}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s), "window": "pre-heat + timed region"}


# ---------------------------------------------------------------------------------------
# the CPU arm: the oracle (restated reference simulate path) on the host cores
# ---------------------------------------------------------------------------------------
def step_bytes_of(n: int) -> float:
    """Algorithmic bytes of one compress + decompress of `n` samples of the workload."""
    _, c, h, w = WORKLOAD["shape"]
    e = n * c * h * w
    return algorithmic_bytes(e, 2, WORKLOAD["avg_bits"], reads=2) + algorithmic_bytes(e, 2, WORKLOAD["avg_bits"])


def cpu_round_trip_gbs(sample_n: int, repeats: int, warmup: int = 1):
    """GB/s of the adaptive compress + decompress of `sample_n` samples of the workload with
    the CPU oracle, all host threads.  Returns (gbs, seconds_per_pass, cores)."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import actnn_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    _, c, h, w = WORKLOAD["shape"]
    x = synthetic_activation(torch, sample_n, c, h, w, torch.bfloat16, "cpu", 0).view(sample_n, c, h, w)
    g = torch.Generator().manual_seed(0)
    shape = tuple(x.shape)
    one = torch.ones(1)

    def one_pass():
        q = O.quantize_activation(x, WORKLOAD["avg_bits"], lambda gr: O.torch_noise(gr.shape, gr.dtype, g),
                                  coeff=(9 / 4, one), scheme=True, initial_bits=WORKLOAD["initial_bits"])
        return O.dequantize_activation(q, shape, dtype=x.dtype)

    for _ in range(warmup):
        one_pass()
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return step_bytes_of(sample_n) / sec / 1e9, sec, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_n = 64
    warm = max(args.warmup, 1)
    import torch  # noqa: F401
    gbs, sec, cores = cpu_round_trip_gbs(sample_n, min(args.steps, 40), warmup=min(warm, 3))
    line = {
        "impl": "reference", "metric": "pack+unpack HBM GB/s", "value": round(gbs, 4), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], "shape": WORKLOAD["shape"], "avg_bits": WORKLOAD["avg_bits"],
                   "group_size": 256, "step": "adaptive compress + decompress of %d of the 512 samples "
                   "(at most 40 timed passes)" % sample_n},
        "cpu_baseline": {"value": round(gbs, 4), "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "%d of 512 samples of the bfloat16 [512,256,28,28] activation per step; the "
                                   "reference's simulate path (min/max, sensitivities, greedy heap, quantize, "
                                   "dequantize) restated for CPU tensors (oracle/actnn_oracle.py), torch threads "
                                   "= cores" % sample_n},
        "e2e": {"value": round(gbs, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------
def kernel_table(torch, lib, _lib, quantization, dev, args, xs, packed, scales, mins, bits_t, offs_t, outs, c_out,
                 ws, ws_bytes, peak, graph_of, timed_replays, median):
    """GB/s and fraction of the copy peak of every kernel of the path, each alone in a CUDA graph
    over the rotating pool.  Returns (table, roofline entry of the step's slowest kernel)."""
    N, C, H, W = WORKLOAD["shape"]
    gs, avg_bits = 256, WORKLOAD["avg_bits"]
    elements, G = N * C * H * W, C * H * W // gs
    DT = _lib.dtype_id(torch.bfloat16)
    count = max(4, min(args.steps, 24))
    stream = lambda: torch.cuda.current_stream().cuda_stream     # noqa: E731
    table = {}

    def timed(name, fn, nbytes, note=None):
        g = graph_of(fn, count)
        g.replay()
        ms = median(timed_replays(g, 9)) / count
        entry = {"ms": round(ms, 5)}
        if nbytes:
            gbs = nbytes / ms / 1e6
            entry.update({"gbs": round(gbs, 1), "frac": round(gbs / peak, 4), "bytes": nbytes})
        if note:
            entry["note"] = note
        table[name] = entry
        return entry

    stat_b = 2.0 * 2 / gs
    mn = [torch.empty(N * G, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    timed("minimax_bf16", lambda r: lib.actnn_minimax(xs[r % POOL].data_ptr(), mn[0].data_ptr(), mn[1].data_ptr(),
                                                     N * G, gs, DT, stream()), elements * (2 + stat_b))
    # per-buffer min / max for the pack-only entry (the bits and offsets are those of the timed step)
    mnx = [tuple(torch.empty(N * G, dtype=torch.bfloat16, device=dev) for _ in range(2)) for _ in range(POOL)]
    for i in range(POOL):
        lib.actnn_minimax(xs[i].data_ptr(), mnx[i][0].data_ptr(), mnx[i][1].data_ptr(), N * G, gs, DT, stream())
    e_pack = timed("pack_mixed_bf16_2b_avg", lambda r: lib.actnn_pack_mixed(
        xs[r % POOL].data_ptr(), mnx[r % POOL][0].data_ptr(), mnx[r % POOL][1].data_ptr(), bits_t[r % POOL].data_ptr(),
        offs_t[r % POOL].data_ptr(), packed[r % POOL].data_ptr(), scales[r % POOL].data_ptr(), None, N, G, gs, DT, DT,
        1, None, 7, 4 * r, stream()), algorithmic_bytes(elements, 2, avg_bits) + elements * stat_b)
    e_unpack = timed("unpack_mixed_bf16_2b_avg", lambda r: lib.actnn_unpack_mixed(
        packed[(r + 3) % POOL].data_ptr(), bits_t[(r + 3) % POOL].data_ptr(), offs_t[(r + 3) % POOL].data_ptr(),
        scales[(r + 3) % POOL].data_ptr(), mnx[(r + 3) % POOL][0].data_ptr(), outs[r % 2].data_ptr(), N, G, gs, DT, DT,
        stream()), algorithmic_bytes(elements, 2, avg_bits))
    timed("compress_mixed_bf16_2b_avg_one_call", lambda r: lib.actnn_compress_mixed(
        xs[r % POOL].data_ptr(), packed[r % POOL].data_ptr(), scales[r % POOL].data_ptr(), mins[r % POOL].data_ptr(),
        bits_t[r % POOL].data_ptr(), offs_t[r % POOL].data_ptr(), c_out.data_ptr(), ws.data_ptr(), ws_bytes, N, G, gs,
        DT, DT, gs / float(H * W), 9 / 4, None, 8, float(int(avg_bits * N)), 1, None, 7, 4 * r, stream()),
        algorithmic_bytes(elements, 2, avg_bits, reads=2),
        "minimax + sensitivity + greedy + pack; algorithmic bytes count the two reads of the activation")
    timed("calc_precision_n512", lambda r: lib.actnn_calc_precision(
        c_out.data_ptr(), None, N, 8, float(int(avg_bits * N)), bits_t[0].data_ptr(), offs_t[0].data_ptr(), G, gs,
        None, 0, stream()), 0)
    del mnx, mn

    # ---- uniform-width fused pair: float16 [256,256,28,28] and float32 [64,64,56,56], 2 bits
    for tag, shape, dt in (("f16_256x256x28x28", (256, 256, 28, 28), torch.float16),
                           ("f32_64x64x56x56", (64, 64, 56, 56), torch.float32)):
        n, c, h, w = shape
        e, g = n * c * h * w, c * h * w // gs
        pool = 4 if dt == torch.float16 else 6
        id_ = _lib.dtype_id(dt)
        sdt = torch.bfloat16 if dt == torch.float32 else dt
        sid = _lib.dtype_id(sdt)
        gen = torch.Generator(device=dev).manual_seed(5)
        xin = [torch.relu(torch.randn(n, g, gs, device=dev, generator=gen)).to(dt) for _ in range(pool)]
        pk = [torch.empty(quantization.single_precision_bytes(2, n, g, gs), dtype=torch.int8, device=dev)
              for _ in range(pool)]
        sc = [torch.empty(n, g, 1, dtype=sdt, device=dev) for _ in range(pool)]
        mi = [torch.empty(n, g, 1, dtype=sdt, device=dev) for _ in range(pool)]
        out = [torch.empty(n, g, gs, dtype=dt, device=dev) for _ in range(2)]
        one_way = algorithmic_bytes(e, xin[0].element_size(), 2)
        for i in range(pool):
            lib.actnn_compress_single(xin[i].data_ptr(), 2, pk[i].data_ptr(), sc[i].data_ptr(), mi[i].data_ptr(), None,
                                      n, g, gs, id_, sid, 1, None, 3, 0, stream())
        timed("compress_single_2b_fused_" + tag, lambda r: lib.actnn_compress_single(
            xin[r % pool].data_ptr(), 2, pk[r % pool].data_ptr(), sc[r % pool].data_ptr(), mi[r % pool].data_ptr(),
            None, n, g, gs, id_, sid, 1, None, 3, 4 * r, stream()), one_way)
        timed("unpack_single_2b_" + tag, lambda r: lib.actnn_unpack_single(
            pk[(r + pool // 2) % pool].data_ptr(), 2, sc[(r + pool // 2) % pool].data_ptr(),
            mi[(r + pool // 2) % pool].data_ptr(), out[r % 2].data_ptr(), n, g, gs, id_, sid, stream()), one_way)
        if dt == torch.float16:
            masks = [torch.empty((e + 31) // 32, dtype=torch.int32, device=dev) for _ in range(pool)]
            for i in range(pool):
                lib.actnn_relu_forward(xin[i].data_ptr(), out[0].data_ptr(), masks[i].data_ptr(), e, id_, stream())
            timed("relu_forward_" + tag, lambda r: lib.actnn_relu_forward(
                xin[r % pool].data_ptr(), out[r % 2].data_ptr(), masks[r % pool].data_ptr(), e, id_, stream()),
                e * (4 + 1 / 8))
            timed("relu_backward_" + tag, lambda r: lib.actnn_relu_backward(
                xin[r % pool].data_ptr(), masks[(r + 2) % pool].data_ptr(), out[r % 2].data_ptr(), e, id_, stream()),
                e * (4 + 1 / 8))
            del masks
        del xin, pk, sc, mi, out
    torch.cuda.empty_cache()

    # ---- roofline: the kernel of the timed step that sits furthest below the copy peak
    name, ent = min((("pack_mixed_flat_kernel<bfloat16> (inside actnn_compress_mixed)", e_pack),
                     ("unpack_mixed_flat_kernel<bfloat16> (actnn_unpack_mixed)", e_unpack)), key=lambda t: t[1]["frac"])
    traffic, traffic_src = None, None
    tpath = os.path.join(ROOT, "profiles", "roofline_traffic.json")
    if os.path.exists(tpath):
        key = ("pack" if name.startswith("pack") else "unpack") + "_mixed_bf16_bytes_per_launch"
        traffic = json.load(open(tpath)).get(key)
        traffic_src = "static figure from an ncu capture (profiles/roofline_traffic.json), not measured in this run"
    roof = {"kernel": name, "bound": "hbm", "achieved": ent["gbs"], "unit": "GB/s", "frac": ent["frac"],
            "traffic": traffic, "traffic_source": traffic_src, "algorithmic_bytes_per_launch": ent["bytes"],
            "ms_per_launch": ent["ms"]}
    return table, roof


def e2e_leg(torch, actnn, dev, world, args, barrier, step_bytes):
    """The same work through the public API, host buffers in, host buffers out.  Three steps are
    in flight at once, each on its own stream with its own buffers, so that the upload of one
    step overlaps the download of the previous one (PCIe is full duplex) and the kernels of the
    one in between.  Every step still uploads its input and downloads its result."""
    N, C, H, W = WORKLOAD["shape"]
    dt = torch.bfloat16
    shape = (N, C, H, W)
    actnn.set_optimization_level("L3")
    conv = actnn.QConv2d(C, C, 3, padding=1).to(dev)          # the layer whose input is compressed
    scheme = conv.scheme
    LANES = 3
    base = synthetic_activation(torch, N, C, H, W, dt, "cpu", 99).view(shape)
    host_in = [base.clone().pin_memory() for _ in range(LANES)]
    host_out = [torch.empty(shape, dtype=dt).pin_memory() for _ in range(LANES)]
    dev_in = [torch.empty(shape, dtype=dt, device=dev) for _ in range(LANES)]
    lanes = [torch.cuda.Stream(dev) for _ in range(LANES)]

    def e2e_step(k):
        lane = k % LANES
        with torch.cuda.stream(lanes[lane]):
            dev_in[lane].copy_(host_in[lane], non_blocking=True)
            q = actnn.ops.quantize_activation(dev_in[lane], scheme)
            y = actnn.ops.dequantize_activation(q, shape, dt)
            host_out[lane].copy_(y, non_blocking=True)
            y.record_stream(lanes[lane])
            for t in q:
                if isinstance(t, torch.Tensor):
                    t.record_stream(lanes[lane])

    def e2e_run(count):
        cur = torch.cuda.current_stream(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(cur)
        for lane in lanes:
            lane.wait_event(a)
        for k in range(count):
            e2e_step(k)
        for lane in lanes:
            done = torch.cuda.Event()
            done.record(lane)
            cur.wait_event(done)
        b.record(cur)
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b)

    e2e_run(2 * LANES)
    e2e_steps = max(2 * LANES, min(args.steps, 18))
    barrier()
    e2e_total_ms = e2e_run(e2e_steps)
    barrier()
    # the last download must have delivered the decoded activation: finite, and (stochastic
    # rounding is unbiased) with the mean of what went up
    got, ref = host_out[(e2e_steps - 1) % LANES].double(), host_in[(e2e_steps - 1) % LANES].double()
    assert bool(torch.isfinite(got).all())
    assert abs(float(got.mean() - ref.mean())) < 0.02 * float(ref.abs().mean())
    e2e_ms = max_over_ranks(e2e_total_ms / e2e_steps, dev)
    elements = N * C * H * W
    del host_in, host_out, dev_in
    return {"value": round(whole_job_gbs(step_bytes, world, e2e_ms), 2), "unit": "GB/s",
            "h2d_bytes_per_step": elements * 2, "d2h_bytes_per_step": elements * 2, "ms_per_step": round(e2e_ms, 4),
            "steps": e2e_steps,
            "path": "pinned host -> H2D -> ops.quantize_activation(x, QConv2d.scheme) at level L3 -> "
                    "ops.dequantize_activation -> D2H, three steps in flight on three streams"}


def resnet_leg(torch, dev, world, rank, args):
    """ResNet-50 training throughput next to the codec numbers: stock torch, this library
    without compression (L0) and level L3; DDP + synchronised batch norm when world > 1."""
    import torch.distributed as dist
    if args.no_resnet:
        return None
    steps, warm = 8, 4
    res = {}
    for level in ("exact", "L0", "L3"):
        res[level] = resnet_throughput(level, 256, steps, warm, dev, world, "resnet50", "float16",
                                       check_sync_bn=world > 1)
        if world > 1:
            t = torch.tensor([res[level]["ms_per_step"]], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[level]["ms_per_step"] = round(float(t.item()), 2)
            res[level]["images_per_s_per_gpu"] = round(256 / float(t.item()) * 1e3, 1)
    if rank != 0:
        return None
    out = {"batch_per_gpu": 256, "amp": "float16", "optimizer": "SGD momentum 0.9", "steps": steps, "warmup": warm,
           "parallelism": "ddp x%d, synchronised batch norm" % world if world > 1 else "single GPU",
           "timing": "median step, CUDA events, max over ranks"}
    for level in ("exact", "L0", "L3"):
        r = res[level]
        out[level] = {"images_per_s": round(r["images_per_s_per_gpu"] * world, 1), "ms_per_step": r["ms_per_step"],
                      "activation_bytes": r["activation_bytes"], "peak_bytes": r["peak_bytes"]}
        if "sync_bn_stats_identical_across_ranks" in r:
            out[level]["sync_bn_stats_identical_across_ranks"] = r["sync_bn_stats_identical_across_ranks"]
    out["L3_over_L0"] = round(out["L3"]["images_per_s"] / out["L0"]["images_per_s"], 4)
    out["L3_over_exact"] = round(out["L3"]["images_per_s"] / out["exact"]["images_per_s"], 4)
    out["activation_reduction_vs_float16_autocast"] = round(
        out["exact"]["activation_bytes"] / max(out["L3"]["activation_bytes"], 1), 2)
    return out


def load_peak():
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        return float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy kernel)"
    return 6650.0, "fallback (no MEASURED_PEAKS.json beside bench.py)"


def run_ours(args):
    import torch
    import torch.distributed as dist

    import actnn_b200 as actnn
    from actnn_b200 import _lib
    from actnn_b200.cpp_extension import quantization

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        init_nccl(dist, torch, dev)

    N, C, H, W = WORKLOAD["shape"]
    gs, avg_bits, init_bits = 256, WORKLOAD["avg_bits"], WORKLOAD["initial_bits"]
    elements = N * C * H * W
    G = C * H * W // gs
    dt = torch.bfloat16
    DT = _lib.dtype_id(dt)
    lib = _lib.load()
    peak, peak_src = load_peak()
    compress_bytes = algorithmic_bytes(elements, 2, avg_bits, reads=2)
    pack_bytes = algorithmic_bytes(elements, 2, avg_bits) + elements * 2.0 * 2 / gs     # reads min and max too
    unpack_bytes = algorithmic_bytes(elements, 2, avg_bits)
    step_bytes = compress_bytes + unpack_bytes
    target_bits = int(avg_bits * N)
    words = target_bits * G * gs // 32

    xs = [synthetic_activation(torch, N, C, H, W, dt, dev, 1234 + 97 * rank + i) for i in range(POOL)]
    packed = [torch.empty(words, dtype=torch.int32, device=dev) for _ in range(POOL)]
    scales = [torch.empty(N, G, 1, dtype=dt, device=dev) for _ in range(POOL)]
    mins = [torch.empty(N, G, 1, dtype=dt, device=dev) for _ in range(POOL)]
    bits_t = [torch.empty(N, dtype=torch.int32, device=dev) for _ in range(POOL)]
    offs_t = [torch.empty(N + 1, dtype=torch.int64, device=dev) for _ in range(POOL)]
    c_out = torch.empty(N, dtype=torch.float32, device=dev)
    ws_bytes = lib.actnn_compress_mixed_workspace(N, G, DT)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    outs = [torch.empty(N, G, gs, dtype=dt, device=dev) for _ in range(2)]
    range_factor = gs / float(H * W)

    def cur_stream():
        return torch.cuda.current_stream().cuda_stream

    def compress(i, step_no):
        _lib.check(lib.actnn_compress_mixed(
            xs[i].data_ptr(), packed[i].data_ptr(), scales[i].data_ptr(), mins[i].data_ptr(), bits_t[i].data_ptr(),
            offs_t[i].data_ptr(), c_out.data_ptr(), ws.data_ptr(), ws_bytes, N, G, gs, DT, DT, range_factor, 9 / 4,
            None, init_bits, float(target_bits), 1, None, 1234 + rank, 4 * step_no, cur_stream()),
            "actnn_compress_mixed")

    def decompress(i, o):
        _lib.check(lib.actnn_unpack_mixed(packed[i].data_ptr(), bits_t[i].data_ptr(), offs_t[i].data_ptr(),
                                          scales[i].data_ptr(), mins[i].data_ptr(), outs[o].data_ptr(), N, G, gs,
                                          DT, DT, cur_stream()), "actnn_unpack_mixed")

    def step(k):
        compress(k % POOL, k)
        decompress((k + POOL // 2) % POOL, k % 2)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def graph_of(fn, count):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for k in range(count):
                fn(k)
        return g

    def timed_replays(g, replays, sync_ranks=False):
        """Milliseconds of each of `replays` replays, CUDA events on the launching stream."""
        out = []
        for _ in range(replays):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if sync_ranks:
                barrier()
            else:
                torch.cuda.synchronize()
            a.record()
            g.replay()
            b.record()
            if sync_ranks:
                barrier()
            else:
                torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return out

    def median(v):
        v = sorted(v)
        return v[len(v) // 2]

    sampler = ClockSampler(local)
    with sampler:
        for i in range(POOL):                               # fill the pool so every decode has input
            compress(i, i)
        for k in range(max(args.warmup, 3)):
            step(k)
        torch.cuda.synchronize()
        # ---- timed region: exactly K steps, captured once into a CUDA graph (launch gaps of a few
        # microseconds would otherwise be a visible part of kernels this short); the graph is
        # replayed REPLAYS times, every replay bracketed by a barrier + synchronize and by CUDA
        # events on the launching stream.
        g_steps = graph_of(step, args.steps)
        for _ in range(3):                                  # pre-heat: clocks seen are clocks under load
            g_steps.replay()
        replay_ms = timed_replays(g_steps, REPLAYS, sync_ranks=True)
    replay_ms = [max_over_ranks(t, dev) for t in replay_ms] if world > 1 else replay_ms
    total_ms = median(replay_ms)
    ms_per_step = total_ms / args.steps
    value = whole_job_gbs(step_bytes, world, ms_per_step)

    # ---- every kernel of the path alone, same rotation, graph-replayed (rank 0)
    kernels = {}
    roof = None
    if rank == 0:
        kernels, roof = kernel_table(torch, lib, _lib, quantization, dev, args, xs, packed, scales, mins, bits_t,
                                     offs_t, outs, c_out, ws, ws_bytes, peak, graph_of, timed_replays, median)
    e2e = e2e_leg(torch, actnn, dev, world, args, barrier, step_bytes)
    resnet = resnet_leg(torch, dev, world, rank, args)

    if rank == 0:
        line = {
            "metric": "pack+unpack HBM GB/s", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD["name"], "shape": WORKLOAD["shape"], "avg_bits": avg_bits,
                       "initial_bits": init_bits, "group_size": gs,
                       "step": "adaptive (L3) compress in one call + decompress of one [512,256,28,28] bfloat16 "
                               "activation, LogNormal(0,1) sensitivities",
                       "bytes_per_step": step_bytes, "l2": "inputs rotate over a pool of %d buffers (%.0f MB), "
                       "larger than L2; packed buffers are decoded %d steps after they were written"
                       % (POOL, POOL * elements * 2 / 1e6, POOL // 2), "parallelism": "replicas x%d" % world},
            "timing": {"replays": len(replay_ms), "ms_per_replay_median": round(total_ms, 4),
                       "ms_per_replay_min": round(min(replay_ms), 4), "ms_per_replay_max": round(max(replay_ms), 4),
                       "value_from": "median replay of the K-step CUDA graph, max over ranks per replay"},
            "e2e": e2e,
            "gpu_launches": 4 * args.steps,
            "launch_mode": "the K steps replayed from one CUDA graph; 3 kernels per compress (group min / max, width allocation, pack), 1 per decompress",
            "roofline": dict(roof, peak=peak, peak_source=peak_src) if roof else None,
            "kernels": kernels,
            "resnet50_l3": resnet,
            "clocks": sampler.summary(),
        }
        if world == 1:
            gbs, sec, cores = cpu_round_trip_gbs(128, repeats=30)
            line["cpu_baseline"] = {"value": round(gbs, 4), "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": "128 of the 512 samples, 30 passes (%.2f s each), CPU oracle = the "
                                              "reference's simulate path restated for CPU tensors, torch threads "
                                              "= cores" % sec}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------
# the callers of the path: ResNet-50 training step with compressed activations
# ---------------------------------------------------------------------------------------
def resnet_throughput(level: str, batch: int, steps: int, warmup: int, dev, world: int, arch: str = "resnet50",
                      amp_dtype="float16", check_sync_bn: bool = False):
    """images/s per GPU (median step, CUDA events) and activation bytes of one training step of a
    torchvision ResNet (random init, synthetic 224x224 images) under ``actnn`` level `level`.
    Protocols follow the reference's mem_speed_benchmark/train.py:363-438."""
    import torch
    import torch.nn as nn
    import torchvision

    import actnn_b200 as actnn
    from actnn_b200.conf import QuantizationConfig

    torch.cuda.reset_peak_memory_stats(dev)
    actnn.config.__dict__.update(QuantizationConfig().__dict__)
    actnn.QScheme.layers.clear()
    actnn.QBNScheme.layers.clear()
    actnn.QScheme.num_layers = 0
    if level != "exact":
        actnn.set_optimization_level(level)
    torch.manual_seed(0)
    model = getattr(torchvision.models, arch)()
    if world > 1:
        model = nn.SyncBatchNorm.convert_sync_batchnorm(model)
    if level != "exact":
        model = actnn.QModule(model)
    model = model.to(dev).train()
    if world > 1:
        model = nn.parallel.DistributedDataParallel(model, device_ids=[dev.index])
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    dt = getattr(torch, amp_dtype)
    scaler = torch.amp.GradScaler("cuda", enabled=dt == torch.float16)
    crit = nn.CrossEntropyLoss()
    g = torch.Generator(device=dev).manual_seed(dev.index or 0)
    images = torch.randn(batch, 3, 224, 224, device=dev, generator=g)
    target = torch.randint(0, 1000, (batch,), device=dev, generator=g)
    times, act_bytes = [], None
    for it in range(warmup + steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        before = torch.cuda.memory_allocated(dev)
        with torch.autocast("cuda", dtype=dt, enabled=dt != torch.float32):
            out = model(images)
            loss = crit(out, target)
        if it == warmup - 1:
            act_bytes = torch.cuda.memory_allocated(dev) - before - out.numel() * out.element_size() - 4
        opt.zero_grad(set_to_none=True)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        b.record()
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(a.elapsed_time(b))
        if it == 0 and check_sync_bn and world > 1:
            # after one step every rank must hold the same running statistics in every
            # (synchronised) batch norm: first and last layer are compared bit for bit
            import torch.distributed as dist
            stats = [m_ for m_ in model.modules() if hasattr(m_, "running_mean") and m_.running_mean is not None]
            same = True
            for bn in (stats[0], stats[-1]):
                mine = torch.cat([bn.running_mean.float(), bn.running_var.float()])
                gathered = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(gathered, mine)
                same = same and all(torch.equal(gathered[0], t_) for t_ in gathered[1:])
            sync_same = bool(same)
            assert sync_same, "running statistics differ across ranks after one synchronised step"
    times.sort()
    med = times[len(times) // 2]
    peak = torch.cuda.max_memory_allocated(dev)
    del model, opt, images, out, loss
    torch.cuda.empty_cache()
    out = {"images_per_s_per_gpu": round(batch / med * 1e3, 1), "ms_per_step": round(med, 2),
           "activation_bytes": int(act_bytes), "peak_bytes": int(peak)}
    if check_sync_bn and world > 1:
        out["sync_bn_stats_identical_across_ranks"] = sync_same
    return out


def resnet_kernel_table(args):
    """`--workload resnet --kernel-table`: GPU time of three training steps by kernel (torch
    profiler, CUPTI), printed as a table.  A diagnostic, not a bench value."""
    import torch
    import torch.nn as nn
    import torchvision
    from torch.profiler import ProfilerActivity, profile

    import actnn_b200 as actnn
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if args.level != "exact":
        actnn.set_optimization_level(args.level)
    model = getattr(torchvision.models, args.arch)()
    if args.level != "exact":
        model = actnn.QModule(model)
    model = model.to(dev).train()
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    dt = getattr(torch, args.amp)
    scaler = torch.amp.GradScaler("cuda", enabled=dt == torch.float16)
    crit = nn.CrossEntropyLoss()
    images = torch.randn(args.batch, 3, 224, 224, device=dev)
    target = torch.randint(0, 1000, (args.batch,), device=dev)

    def step():
        with torch.autocast("cuda", dtype=dt):
            loss = crit(model(images), target)
        opt.zero_grad(set_to_none=True)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()

    for _ in range(4):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    rows = sorted(prof.key_averages(), key=lambda e: -e.self_device_time_total)
    total = sum(e.self_device_time_total for e in rows)
    print("GPU time of 3 steps: %.1f ms (%.1f ms per step)" % (total / 1e3, total / 3e3))
    print("| kernel | launches | total ms | avg us | share |\n|---|---|---|---|---|")
    for e in rows[:30]:
        print("| `%s` | %d | %.2f | %.1f | %.1f%% |" % (e.key[:90], e.count, e.self_device_time_total / 1e3,
                                                     e.self_device_time_total / max(e.count, 1),
                                                     100.0 * e.self_device_time_total / max(total, 1)))


def run_resnet(args):
    """`--workload resnet50`: whole-job images/s of L3 training next to exact training."""
    import torch
    import torch.distributed as dist

    if args.kernel_table:
        return resnet_kernel_table(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        init_nccl(dist, torch, dev)
    steps, warm = max(3, min(args.steps, 30)), max(3, min(args.warmup, 5))
    if args.level in ("L4", "L5", "swap"):
        warm = max(warm, 8)          # the pinned pool of the host swap fills while the per-layer widths settle
    res = {}
    for level in ("exact", args.level):
        res[level] = resnet_throughput(level, args.batch, steps, warm, dev, world, args.arch, args.amp)
        if world > 1:
            t = torch.tensor([res[level]["ms_per_step"]], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[level]["ms_per_step"] = float(t.item())
            res[level]["images_per_s_per_gpu"] = round(args.batch / float(t.item()) * 1e3, 1)
    # the reference's memory tables compare with float32 training: one float32 exact step for its bytes
    fp32_act = None
    if world == 1 and args.amp != "float32":
        fp32_act = resnet_throughput("exact", args.batch, 1, 1, dev, world, args.arch, "float32")["activation_bytes"]
    if rank == 0:
        q, e = res[args.level], res["exact"]
        print(json.dumps({
            "metric": "%s %s images/s" % (args.arch, args.level), "value": round(q["images_per_s_per_gpu"] * world, 1),
            "unit": "images/s", "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": q["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.amp, "data": "synthetic",
            "config": {"workload": "%s-%s-training" % (args.arch, args.level), "batch_per_gpu": args.batch,
                       "image": [3, 224, 224], "optimizer": "SGD momentum 0.9", "parallelism": "ddp x%d" % world,
                       "sync_bn": world > 1},
            "exact_images_per_s": round(e["images_per_s_per_gpu"] * world, 1),
            "ratio_to_exact": round(q["images_per_s_per_gpu"] / e["images_per_s_per_gpu"], 4),
            "activation_bytes": q["activation_bytes"], "exact_activation_bytes": e["activation_bytes"],
            "peak_bytes": q["peak_bytes"], "exact_peak_bytes": e["peak_bytes"],
            "activation_reduction_vs_%s_autocast" % args.amp: round(e["activation_bytes"] / max(q["activation_bytes"], 1), 2),
            "exact_float32_activation_bytes": fp32_act,
            "activation_reduction_vs_float32": None if not fp32_act else round(fp32_act / max(q["activation_bytes"], 1), 2),
        }))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------
# profiling helper: a few launches of ONE kernel on a case that is larger than L2 but small
# enough for a multi-pass ncu capture (float16 [512, 256, 28, 28] = 205 MB)
# ---------------------------------------------------------------------------------------
def run_profile(args):
    import torch

    from actnn_b200 import _lib
    from actnn_b200.cpp_extension import calc_precision, minimax, quantization

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    N, G, gs, bits = 512, 784, 256, 2
    dt = getattr(torch, args.profile_dtype)
    F16 = _lib.dtype_id(dt)                    # id of the chosen dtype (float16 unless --profile-dtype says otherwise)
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(0)
    x = torch.randn(N, G, gs, device=dev, dtype=dt)
    out = torch.empty_like(x)
    scale = torch.empty(N, G, 1, dtype=dt, device=dev)
    mn = torch.empty(N, G, 1, dtype=dt, device=dev)
    mx = torch.empty(N, G, 1, dtype=dt, device=dev)
    packed = torch.empty(quantization.single_precision_bytes(bits, N, G, gs), dtype=torch.int8, device=dev)
    Cs = torch.exp(torch.randn(N, device=dev))
    bt, offs = calc_precision.allocate_bits(Cs, 8, 2 * N, None, G, gs, with_offsets=True)
    pm = torch.empty(2 * N * G * gs // 32, dtype=torch.int32, device=dev)
    mask = torch.empty((x.numel() + 31) // 32, dtype=torch.int32, device=dev)
    lib.actnn_minimax(x.data_ptr(), mn.data_ptr(), mx.data_ptr(), N * G, gs, F16, st)
    lib.actnn_compress_single(x.data_ptr(), bits, packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), None, N, G,
                              gs, F16, F16, 1, None, 1, 0, st)
    lib.actnn_pack_mixed(x.data_ptr(), mn.data_ptr(), mx.data_ptr(), bt.data_ptr(), offs.data_ptr(), pm.data_ptr(),
                         scale.data_ptr(), None, N, G, gs, F16, F16, 1, None, 1, 0, st)
    lib.actnn_relu_forward(x.data_ptr(), out.data_ptr(), mask.data_ptr(), x.numel(), F16, st)
    ws_cm_bytes = lib.actnn_compress_mixed_workspace(N, G, F16)
    ws_cm = torch.empty(ws_cm_bytes, dtype=torch.uint8, device=dev)
    c_out = torch.empty(N, dtype=torch.float32, device=dev)
    bt2, offs2 = torch.empty_like(bt), torch.empty_like(offs)
    calls = {
        "compress_mixed": lambda: lib.actnn_compress_mixed(
            x.data_ptr(), pm.data_ptr(), scale.data_ptr(), mn.data_ptr(), bt2.data_ptr(), offs2.data_ptr(),
            c_out.data_ptr(), ws_cm.data_ptr(), ws_cm_bytes, N, G, gs, F16, F16, gs / 784.0, 9 / 4, None, 8,
            float(2 * N), 1, None, 1, 0, st),
        "compress_single": lambda: lib.actnn_compress_single(
            x.data_ptr(), bits, packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), None, N, G, gs, F16, F16, 1,
            None, 1, 0, st),
        "unpack_single": lambda: lib.actnn_unpack_single(
            packed.data_ptr(), bits, scale.data_ptr(), mn.data_ptr(), out.data_ptr(), N, G, gs, F16, F16, st),
        "minimax": lambda: lib.actnn_minimax(x.data_ptr(), mn.data_ptr(), mx.data_ptr(), N * G, gs, F16, st),
        "pack_mixed": lambda: lib.actnn_pack_mixed(
            x.data_ptr(), mn.data_ptr(), mx.data_ptr(), bt.data_ptr(), offs.data_ptr(), pm.data_ptr(),
            scale.data_ptr(), None, N, G, gs, F16, F16, 1, None, 1, 0, st),
        "unpack_mixed": lambda: lib.actnn_unpack_mixed(
            pm.data_ptr(), bt.data_ptr(), offs.data_ptr(), scale.data_ptr(), mn.data_ptr(), out.data_ptr(), N, G,
            gs, F16, F16, st),
        "relu_forward": lambda: lib.actnn_relu_forward(x.data_ptr(), out.data_ptr(), mask.data_ptr(), x.numel(),
                                                       F16, st),
        "relu_backward": lambda: lib.actnn_relu_backward(x.data_ptr(), mask.data_ptr(), out.data_ptr(), x.numel(),
                                                        F16, st),
    }
    # batch norm over the same bytes viewed as NCHW [512, 256, 28, 28]
    bn_c, bn_hw = 256, 784
    w = torch.ones(bn_c, device=dev)
    bvec = torch.zeros(bn_c, device=dev)
    rm, rv = torch.zeros(bn_c, device=dev), torch.ones(bn_c, device=dev)
    sm, si = torch.empty(bn_c, device=dev), torch.empty(bn_c, device=dev)
    gw, gb = torch.empty(bn_c, device=dev), torch.empty(bn_c, device=dev)
    dy = torch.randn_like(x)
    ws_bytes = lib.actnn_batch_norm_workspace(N, bn_c, bn_hw)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    calls["batch_norm_forward"] = lambda: lib.actnn_batch_norm_forward(
        x.data_ptr(), w.data_ptr(), bvec.data_ptr(), rm.data_ptr(), rv.data_ptr(), out.data_ptr(), sm.data_ptr(),
        si.data_ptr(), N, bn_c, bn_hw, 0.1, 1e-5, F16, ws.data_ptr(), ws_bytes, st)
    calls["batch_norm_backward"] = lambda: lib.actnn_batch_norm_backward(
        x.data_ptr(), dy.data_ptr(), w.data_ptr(), sm.data_ptr(), si.data_ptr(), out.data_ptr(), gw.data_ptr(),
        gb.data_ptr(), N, bn_c, bn_hw, F16, ws.data_ptr(), ws_bytes, st)
    sm_bytes = lib.actnn_batch_norm_stats_minimax_workspace(N, bn_c, bn_hw)
    sm_ws = torch.empty(max(sm_bytes, 16), dtype=torch.uint8, device=dev)
    calls["batch_norm_stats_minimax"] = lambda: lib.actnn_batch_norm_stats_minimax(
        x.data_ptr(), mn.data_ptr(), mx.data_ptr(), w.data_ptr(), bvec.data_ptr(), rm.data_ptr(), rv.data_ptr(),
        sm.data_ptr(), si.data_ptr(), N, bn_c, bn_hw, 0.1, 1e-5, F16, sm_ws.data_ptr(), sm_bytes, st)
    # max pooling 3x3 / stride 2 / padding 1 (the ResNet stem) over the same bytes viewed as [128, 64, 112, 112]
    pn, pc, ph, pw = 128, 64, 112, 112
    py = torch.empty(pn, pc, ph // 2, pw // 2, dtype=dt, device=dev)
    pidx = torch.empty(pn, pc, ph // 2, pw // 2, dtype=torch.int8, device=dev)
    calls["max_pool_forward"] = lambda: lib.actnn_max_pool2d_forward(
        x.data_ptr(), py.data_ptr(), pidx.data_ptr(), pn, pc, ph, pw, 3, 3, 2, 2, 1, 1, 1, 1, F16, st)
    calls["max_pool_backward"] = lambda: lib.actnn_max_pool2d_backward(
        py.data_ptr(), pidx.data_ptr(), out.data_ptr(), pn, pc, ph, pw, 3, 3, 2, 2, 1, 1, 1, 1, F16, st)
    calls["max_pool_forward"]()
    calls["batch_norm_forward"]()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    names = list(calls) if args.profile == "all" else [args.profile]
    for name in names:
        calls[name]()
        a.record()
        for _ in range(args.launches):
            _lib.check(calls[name](), name)
        b.record()
        torch.cuda.synchronize()
        print(json.dumps({"profile": name, "shape": [N, G, gs], "dtype": args.profile_dtype, "launches": args.launches,
                          "ms_per_launch": round(a.elapsed_time(b) / args.launches, 5)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="codec", choices=["codec", "resnet"],
                    help="codec (default, the headline metric) or a ResNet training step through the Q-layers")
    ap.add_argument("--arch", default="resnet50")
    ap.add_argument("--level", default="L3")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--amp", default="float16", choices=["float16", "bfloat16"])
    ap.add_argument("--kernel-table", action="store_true",
                    help="with --workload resnet: print GPU time by kernel for three steps (torch profiler)")
    ap.add_argument("--profile", default=None, help="run a few launches of one kernel (for ncu); 'all' = each")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--profile-dtype", default="float16", choices=["float16", "bfloat16", "float32"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-resnet", action="store_true", help="codec workload: skip the ResNet-50 object")
    args = ap.parse_args()
    if args.profile:
        run_profile(args)
    elif args.workload == "resnet":
        run_resnet(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
