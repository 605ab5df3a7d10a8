"""Benchmark of the activation compress / decompress hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

One STEP = one pass of the codec over one batch of synthetic activations of the headline
workload: a float16 activation of shape [256, 256, 28, 28] (51.4 M elements, 256-element
groups), compressed to 2 bits with the fused single-pass kernel (min/max + stochastic
rounding + pack) and decompressed again.  Metric: algorithmic GB/s of compress +
decompress, i.e. per element  s + b/8 + 2*s_stat/gs  bytes each way (s = 2 bytes, b = 2
bits, two 2-byte statistics per 256-element group) = 232.8 MB per step.

The printed JSON line carries
  value       device-resident throughput (inputs in HBM, raw C-ABI calls, CUDA-event timed);
  e2e         the same work through the public Python API from pinned HOST buffers:
              H2D copy -> quantize_activation -> dequantize_activation -> D2H copy, three steps in
              flight on three streams so that uploads, kernels and downloads overlap;
  roofline    the dominant kernel (fused compress) against the measured HBM copy peak;
  kernels     per-kernel GB/s for the other kernels of the path (informational);
  cpu_baseline  the CPU oracle (a restatement of the reference's simulate path) timed on the
              host cores over a bounded sample of the same workload (rank 0, N = 1 only).
`--impl reference` times only that CPU implementation and prints the reference arm's line.

Inputs rotate through a pool whose total size is several times the 126 MB L2, and a packed
buffer is decoded only after half the pool has been re-written, so neither the activation
reads nor the packed reads are served from L2.
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

WORKLOAD = {"name": "cfg2-activation-codec", "shape": [256, 256, 28, 28], "dtype": "float16", "bits": 2,
            "group_size": 256}
POOL = 8                                    # rotating buffers: 8 x 102.8 MB in, 8 x 13.6 MB packed


def algorithmic_bytes(elements: int, elem_size: int, bits: float, stat_size: int = 2, gs: int = 256) -> float:
    """Bytes one direction of the codec must move: the activation, the packed codes and the
    two per-group statistics."""
    return elements * (elem_size + bits / 8.0 + 2.0 * stat_size / gs)


# ---------------------------------------------------------------------------------------
# multi-rank bookkeeping (one process per GPU; the codec itself needs no collective)
# ---------------------------------------------------------------------------------------
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
def cpu_round_trip_gbs(sample_n: int, repeats: int, warmup: int = 1):
    """GB/s of compress + decompress of the first `sample_n` samples of the workload with the
    CPU oracle, all host threads.  Returns (gbs, seconds_per_pass, cores)."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import actnn_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    _, c, h, w = WORKLOAD["shape"]
    g = torch.Generator().manual_seed(0)
    x = torch.randn(sample_n, c, h, w, generator=g).to(torch.float16)
    shape = tuple(x.shape)

    def one_pass():
        q = O.quantize_activation(x, WORKLOAD["bits"], lambda gr: O.torch_noise(gr.shape, gr.dtype, g), scheme=False)
        return O.dequantize_activation(q, shape, dtype=x.dtype)

    for _ in range(warmup):
        one_pass()
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    nbytes = 2 * algorithmic_bytes(x.numel(), 2, WORKLOAD["bits"])
    return nbytes / sec / 1e9, sec, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_n = 64
    warm = max(args.warmup, 1)
    import torch  # noqa: F401
    gbs, sec, cores = cpu_round_trip_gbs(sample_n, args.steps, warmup=min(warm, 3))
    line = {
        "impl": "reference", "metric": "pack+unpack HBM GB/s", "value": round(gbs, 4), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], "shape": WORKLOAD["shape"], "bits": WORKLOAD["bits"],
                   "group_size": 256, "step": "compress + decompress of %d of the 256 samples" % sample_n},
        "cpu_baseline": {"value": round(gbs, 4), "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "%d of 256 samples of the cfg2 activation per step; the reference's simulate "
                                   "path restated for CPU tensors (oracle/actnn_oracle.py), torch threads = cores"
                                   % sample_n},
        "e2e": {"value": round(gbs, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    import actnn_b200 as actnn
    from actnn_b200 import _lib
    from actnn_b200.cpp_extension import minimax, quantization
    from actnn_b200.cpp_extension import calc_precision

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    N, C, H, W = WORKLOAD["shape"]
    bits, gs = WORKLOAD["bits"], 256
    elements = N * C * H * W
    G = C * H * W // gs
    dt = torch.float16
    F16 = _lib.dtype_id(dt)
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    one_way = algorithmic_bytes(elements, 2, bits)
    step_bytes = 2 * one_way

    torch.manual_seed(1234 + rank)
    xs = [torch.randn(N, G, gs, device=dev, dtype=dt) for _ in range(POOL)]
    packed = [torch.empty(quantization.single_precision_bytes(bits, N, G, gs), dtype=torch.int8, device=dev)
              for _ in range(POOL)]
    scales = [torch.empty(N, G, 1, dtype=dt, device=dev) for _ in range(POOL)]
    mins = [torch.empty(N, G, 1, dtype=dt, device=dev) for _ in range(POOL)]
    outs = [torch.empty(N, G, gs, dtype=dt, device=dev) for _ in range(2)]

    def cur_stream():
        return torch.cuda.current_stream().cuda_stream

    def compress(i, step_no):
        _lib.check(lib.actnn_compress_single(xs[i].data_ptr(), bits, packed[i].data_ptr(), scales[i].data_ptr(),
                                             mins[i].data_ptr(), None, N, G, gs, F16, F16, 1, None, 1234 + rank,
                                             4 * step_no, cur_stream()), "actnn_compress_single")

    def decompress(i, o):
        _lib.check(lib.actnn_unpack_single(packed[i].data_ptr(), bits, scales[i].data_ptr(), mins[i].data_ptr(),
                                           outs[o].data_ptr(), N, G, gs, F16, F16, cur_stream()),
                   "actnn_unpack_single")

    def step(k):
        compress(k % POOL, k)
        decompress((k + POOL // 2) % POOL, k % 2)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local)
    with sampler:
        for i in range(POOL):                               # fill the pool so every decode has input
            compress(i, i)
        for k in range(max(args.warmup, 3)):
            step(k)
        # pre-heat ~0.2 s so that the clocks seen are clocks under load
        t_end = time.perf_counter() + 0.2
        k = 0
        while time.perf_counter() < t_end:
            for _ in range(50):
                step(k)
                k += 1
            torch.cuda.synchronize()

        # ---- timed region: exactly K steps.  The K steps are captured once into a CUDA graph
        # (launch gaps of a few microseconds would otherwise be a tenth of a 25-microsecond
        # kernel) and the replay is bracketed by CUDA events on the launching stream.
        def graph_of(fn, count):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for k in range(count):
                    fn(k)
            return g

        def timed_replay(g):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            a.record()
            g.replay()
            b.record()
            barrier()
            return a.elapsed_time(b)

        g_steps = graph_of(step, args.steps)
        g_steps.replay()
        total_ms = timed_replay(g_steps)
        # the two kernels of the step, each alone, same rotation (for the roofline figure)
        g_pack = graph_of(lambda k: compress(k % POOL, k), args.steps)
        g_unpack = graph_of(lambda k: decompress((k + POOL // 2) % POOL, k % 2), args.steps)
        g_pack.replay()
        pack_ms = timed_replay(g_pack) / args.steps
        g_unpack.replay()
        unpack_ms = timed_replay(g_unpack) / args.steps
    total_ms = max_over_ranks(total_ms, dev)
    ms_per_step = total_ms / args.steps
    value = whole_job_gbs(step_bytes, world, ms_per_step)

    # ---- other kernels of the path, each timed alone over the rotating pool (informational)
    def time_kernel(fn, reps=16):
        for r in range(3):
            fn(r)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for r in range(reps):
            fn(r)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    kernels = {}
    if rank == 0:
        stat_b = 2.0 * 2 / gs
        kernels["compress_single_2b_fused"] = {"ms": round(pack_ms, 5), "gbs": round(one_way / pack_ms / 1e6, 1)}
        kernels["unpack_single_2b"] = {"ms": round(unpack_ms, 5), "gbs": round(one_way / unpack_ms / 1e6, 1)}
        mn = [torch.empty(N * G, dtype=dt, device=dev) for _ in range(2)]
        ms = time_kernel(lambda r: lib.actnn_minimax(xs[r % POOL].data_ptr(), mn[0].data_ptr(), mn[1].data_ptr(),
                                                    N * G, gs, F16, stream))
        kernels["minimax"] = {"ms": round(ms, 5), "gbs": round(elements * (2 + stat_b) / ms / 1e6, 1)}
        # adaptive (L3) path: 2.0-bit average, per-sample widths from LogNormal sensitivities
        Cs = torch.exp(torch.randn(N, device=dev))
        bt, offs = calc_precision.allocate_bits(Cs, 8, 2 * N, None, G, gs, with_offsets=True)
        words = 2 * N * G * gs // 32
        pm = [torch.empty(words, dtype=torch.int32, device=dev) for _ in range(POOL)]
        mnx = []
        for i in range(POOL):
            a, b = minimax.minimax(xs[i].view(-1, gs))
            mnx.append((a, b))
        ms = time_kernel(lambda r: lib.actnn_pack_mixed(
            xs[r % POOL].data_ptr(), mnx[r % POOL][0].data_ptr(), mnx[r % POOL][1].data_ptr(), bt.data_ptr(),
            offs.data_ptr(), pm[r % POOL].data_ptr(), scales[r % POOL].data_ptr(), None, N, G, gs, F16, F16, 1,
            None, 7, 4 * r, stream))
        kernels["pack_mixed_2b_avg"] = {"ms": round(ms, 5), "gbs": round((one_way + elements * stat_b) / ms / 1e6, 1)}
        ms = time_kernel(lambda r: lib.actnn_unpack_mixed(
            pm[(r + 4) % POOL].data_ptr(), bt.data_ptr(), offs.data_ptr(), scales[(r + 4) % POOL].data_ptr(),
            mnx[(r + 4) % POOL][0].data_ptr(), outs[r % 2].data_ptr(), N, G, gs, F16, F16, stream))
        kernels["unpack_mixed_2b_avg"] = {"ms": round(ms, 5), "gbs": round(one_way / ms / 1e6, 1)}
        # the whole adaptive compress in one call: min/max, sensitivities, greedy, pack (X is read twice)
        ws_bytes = lib.actnn_compress_mixed_workspace(N, G, F16)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        c_out = torch.empty(N, dtype=torch.float32, device=dev)
        bt2, offs2 = torch.empty_like(bt), torch.empty_like(offs)
        mn_o = torch.empty(N * G, dtype=dt, device=dev)
        ms = time_kernel(lambda r: lib.actnn_compress_mixed(
            xs[r % POOL].data_ptr(), pm[r % POOL].data_ptr(), scales[r % POOL].data_ptr(), mn_o.data_ptr(),
            bt2.data_ptr(), offs2.data_ptr(), c_out.data_ptr(), ws.data_ptr(), ws_bytes, N, G, gs, F16, F16,
            gs / float(H * W), 1.0, None, 8, float(2 * N), 1, None, 7, 4 * r, stream))
        kernels["compress_mixed_2b_avg_one_call"] = {
            "ms": round(ms, 5), "gbs": round((one_way + elements * 2.0) / ms / 1e6, 1),
            "note": "minimax + sensitivity + greedy + pack; algorithmic bytes count the two reads of X"}
        ms = time_kernel(lambda r: lib.actnn_calc_precision(Cs.data_ptr(), None, N, 8, float(2 * N), bt.data_ptr(),
                                                           offs.data_ptr(), G, gs, None, 0, stream))
        kernels["calc_precision_n256"] = {"ms": round(ms, 5)}
        del pm, mnx
        masks = [torch.empty((elements + 31) // 32, dtype=torch.int32, device=dev) for _ in range(POOL)]
        ms = time_kernel(lambda r: lib.actnn_relu_forward(xs[r % POOL].data_ptr(), outs[r % 2].data_ptr(),
                                                         masks[r % POOL].data_ptr(), elements, F16, stream))
        kernels["relu_forward"] = {"ms": round(ms, 5), "gbs": round(elements * (4 + 1 / 8) / ms / 1e6, 1)}
        ms = time_kernel(lambda r: lib.actnn_relu_backward(xs[r % POOL].data_ptr(), masks[(r + 4) % POOL].data_ptr(),
                                                          outs[r % 2].data_ptr(), elements, F16, stream))
        kernels["relu_backward"] = {"ms": round(ms, 5), "gbs": round(elements * (4 + 1 / 8) / ms / 1e6, 1)}
        del masks

    # ---- end to end through the public API, host buffers in, host buffers out
    actnn.set_optimization_level("L2")                      # uniform width, no adaptive scheme
    actnn.config.activation_compression_bits = [bits]
    shape = (N, C, H, W)
    # Three steps are in flight at once, each on its own stream with its own buffers, so that the
    # upload of one step overlaps the download of the previous one (PCIe is full duplex) and the
    # kernels of the one in between.  Every step still uploads its input and downloads its result.
    LANES = 3
    host_in = [torch.randn(shape, dtype=dt).pin_memory() for _ in range(LANES)]
    host_out = [torch.empty(shape, dtype=dt).pin_memory() for _ in range(LANES)]
    dev_in = [torch.empty(shape, dtype=dt, device=dev) for _ in range(LANES)]
    lanes = [torch.cuda.Stream(dev) for _ in range(LANES)]

    def e2e_step(k):
        lane = k % LANES
        with torch.cuda.stream(lanes[lane]):
            dev_in[lane].copy_(host_in[lane], non_blocking=True)
            q = actnn.ops.quantize_activation(dev_in[lane], None)
            y = actnn.ops.dequantize_activation(q, shape, dt)
            host_out[lane].copy_(y, non_blocking=True)
            y.record_stream(lanes[lane])

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
    e2e_steps = max(2 * LANES, min(args.steps, 24))
    barrier()
    e2e_total_ms = e2e_run(e2e_steps)
    barrier()
    # the last download must have delivered the decoded activation
    assert bool(torch.isfinite(host_out[(e2e_steps - 1) % LANES].float()).all())
    e2e_ms = e2e_total_ms / e2e_steps
    e2e_ms = max_over_ranks(e2e_ms, dev)
    e2e_value = whole_job_gbs(step_bytes, world, e2e_ms)

    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(peaks_path):
            peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy kernel)"
        else:
            peak, peak_src = 6650.0, "fallback (earlier measurement on this pool)"
        achieved = one_way / (pack_ms * 1e-3) / 1e9
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "roofline_traffic.json")
        if os.path.exists(tpath):
            traffic = json.load(open(tpath)).get("compress_single_2b_fused_bytes_per_launch")
        line = {
            "metric": "pack+unpack HBM GB/s", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD["name"], "shape": WORKLOAD["shape"], "bits": bits, "group_size": gs,
                       "step": "fused 2-bit compress + decompress of one [256,256,28,28] float16 activation",
                       "bytes_per_step": step_bytes, "l2": "inputs rotate over a pool of %d buffers (%.0f MB), "
                       "larger than L2; packed buffers are decoded %d steps after they were written"
                       % (POOL, POOL * elements * 2 / 1e6, POOL // 2), "parallelism": "replicas x%d" % world},
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": elements * 2,
                    "d2h_bytes_per_step": elements * 2, "ms_per_step": round(e2e_ms, 4),
                    "path": "pinned host -> H2D -> ops.quantize_activation -> ops.dequantize_activation -> D2H, "
                            "three steps in flight on three streams"},
            "gpu_launches": 2 * args.steps, "launch_mode": "the K steps replayed from one CUDA graph",
            "roofline": {"kernel": "pack_single_kernel<half, 2 bit, fused> (actnn_compress_single)", "bound": "hbm",
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "traffic": traffic, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": one_way},
            "kernels": kernels,
            "clocks": sampler.summary(),
        }
        if world == 1:
            gbs, sec, cores = cpu_round_trip_gbs(256, repeats=30)
            line["cpu_baseline"] = {"value": round(gbs, 4), "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": "the whole [256,256,28,28] activation, 30 passes (%.2f s each), CPU "
                                              "oracle = the reference's simulate path restated for CPU tensors, "
                                              "torch threads = cores" % sec}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------
# the callers of the path: ResNet-50 training step with compressed activations
# ---------------------------------------------------------------------------------------
def resnet_throughput(level: str, batch: int, steps: int, warmup: int, dev, world: int, arch: str = "resnet50",
                      amp_dtype="float16"):
    """images/s per GPU (median step, CUDA events) and activation bytes of one training step of a
    torchvision ResNet (random init, synthetic 224x224 images) under ``actnn`` level `level`.
    Protocols follow the reference's mem_speed_benchmark/train.py:363-438."""
    import torch
    import torch.nn as nn
    import torchvision

    import actnn_b200 as actnn
    from actnn_b200.conf import QuantizationConfig

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
    times.sort()
    med = times[len(times) // 2]
    peak = torch.cuda.max_memory_allocated(dev)
    del model, opt, images, out, loss
    torch.cuda.empty_cache()
    return {"images_per_s_per_gpu": round(batch / med * 1e3, 1), "ms_per_step": round(med, 2),
            "activation_bytes": int(act_bytes), "peak_bytes": int(peak)}


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
        dist.init_process_group("nccl", device_id=dev)
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
    dt = torch.float16
    F16 = _lib.dtype_id(dt)
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
    calls = {
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
        print(json.dumps({"profile": name, "shape": [N, G, gs], "dtype": "f16", "launches": args.launches,
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
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
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
