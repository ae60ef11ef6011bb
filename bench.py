"""Benchmark of the differentiable-rasterisation hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg3|cfg1|cfg2|cfg4|cfg5|sort]

Workload (default): configuration 3 of the reference's benchmark plan - 200 000 seeded random triangles, 1920x1080, 16x16 tiles, fp32,
forward + backward of mean((image - target)^2).  One step = a batch of views of the mesh (default 8 per GPU, each with its
own target image) through the whole path, gradients summed.  With N > 1 GPUs (one process per GPU under
torchrun) every rank renders its own views and the summed vertex/colour/opacity gradients are combined
with one NCCL all-reduce per step (weak scaling: per-GPU work is fixed).

Prints ONE JSON line (rank 0).  `value` is fwd+bwd Mpix/s with inputs resident in HBM through
``trigrad_b200.views.l2_view_step`` (forward, then the backward with the loss gradient formed inside the kernel), the
views of a step spread over CUDA streams, timed with CUDA events per step with an L2 flush between steps; `e2e` is the
same call from pinned HOST buffers (inputs copied in, loss and gradients copied out, every step); `single_view` is ONE
view on ONE stream, both through ``trigrad_b200.render`` + torch autograd (the reference's signature) and through
``l2_view_step``; `other_configs` gives milliseconds per view of the other configurations; `cfg4_sharded` is the
64-camera ring split over the ranks with its all-reduce (the multi-GPU configuration); `roofline` describes the
dominant kernel; `cpu_baseline` is the CPU oracle timed on this machine's host cores.

`--impl reference` times the reference algorithm on the host cores (the reference has no CPU path and
only exists as CUDA; the CPU restatement under ``oracle/`` stands in), with all host threads.
`--workload sort --pairs N` times the device-wide radix sort alone and prints its algorithmic GB/s.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fwd+bwd Mpix/s"
UNIT = "Mpix/s"


# ----------------------------------------------------------------------------------------------------
def make_scene(name: str):
    from trigrad_b200 import scenes as S

    if name == "cfg3":
        return S.config3_random200k(), "cfg3_random200k_1920x1080"
    if name == "cfg2":
        return S.config2_random10k(), "cfg2_random10k_512x512"
    if name == "cfg1":
        return S.config1_icosphere(), "cfg1_icosphere1280_256x256"
    if name == "cfg5":
        return S.config5_overlap(), "cfg5_overlap2M_3840x2160"
    if name == "cfg4":
        mesh = S.displaced_sphere(8)
        pvs = S.camera_ring(64)
        sc = S.config4_view(mesh, pvs[0], name="cfg4_sphere1M_view0")
        sc.meta["mesh"], sc.meta["pvs"] = mesh, pvs
        return sc, "cfg4_displaced_sphere_1.3M_tris_64_cameras_1920x1080"
    raise SystemExit(f"unknown workload {name}")


def S_project(scene, pv: np.ndarray) -> np.ndarray:
    from trigrad_b200 import scenes as S

    return S.project_numpy(scene.meta["mesh"].points, pv)


def view_vertices(vertices: np.ndarray, k: int) -> np.ndarray:
    """View k of the scene: the NDC xy plane rotated by 0.01*k rad (view 0 is the scene itself)."""
    if k == 0:
        return vertices
    a = 0.01 * k
    out = vertices.copy()
    out[:, 0] = np.cos(a) * vertices[:, 0] - np.sin(a) * vertices[:, 1]
    out[:, 1] = np.sin(a) * vertices[:, 0] + np.cos(a) * vertices[:, 1]
    return out


# ----------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while a region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.period = period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self) -> dict:
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------------
def cpu_step_factory(scene, tile_stride: int = 1):
    """The CPU oracle's fwd+bwd step on prepared float32 arrays (lists, matrices, forward, loss, backward)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as O

    v, i, c, o = scene.vertices, scene.indices, scene.colors, scene.opacities
    target = scene.target()
    W, H, tw, th = scene.width, scene.height, scene.tile_width, scene.tile_height
    scale = np.float32(2.0 / (W * H * 4))
    gd = np.zeros((H, W), np.float32)

    def step():
        f = O.forward(v, i, c, o, W, H, tw, th, tile_stride=tile_stride)
        gi = (f.image - target) * scale
        return O.backward(v, i, c, o, W, H, f, gi, gd, tw, th, tile_stride=tile_stride)

    return step, O


def time_cpu(scene, steps: int, warmup: int, limit_s: float):
    """Times `steps` CPU steps after `warmup`; picks a tile stride so that the run fits the time limit."""
    step, O = cpu_step_factory(scene, 1)
    # all host threads, also under a launcher that sets OMP_NUM_THREADS=1 for its workers
    try:
        O.set_num_threads(len(os.sched_getaffinity(0)))
    except AttributeError:
        O.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    step()
    first = time.perf_counter() - t0
    stride = 1
    total_steps = steps + max(warmup - 1, 0)
    if first * total_steps > limit_s:
        stride = int(np.ceil(first * total_steps / limit_s))
        step, O = cpu_step_factory(scene, stride)
    for _ in range(max(warmup - 1, 0) if stride == 1 else warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    px = O.sampled_pixels(scene, stride)
    sample = (f"{steps} full steps" if stride == 1 else
              f"{steps} steps compositing every {stride}th tile ({px} of {scene.width * scene.height} pixels); "
              "binning and sorting in full")
    return px / dt / 1e6, dt, O.num_threads(), sample


def run_reference_arm(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    scene, wname = make_scene(args.workload)
    value, dt, cores, sample = time_cpu(scene, args.steps, args.warmup, limit_s=150.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wname, "triangles": scene.num_triangles, "width": scene.width, "height": scene.height,
                   "tile": [scene.tile_width, scene.tile_height], "per_pixel_sort": True, "max_layers": 32,
                   "note": "reference algorithm on host cores: the reference ships no CPU path, its CPU restatement (oracle/) is timed"},
        "triangles_per_s": scene.num_triangles / dt * (1.0 if "full" in sample else float("nan")),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line, allow_nan=True).replace("NaN", "null"))


# ----------------------------------------------------------------------------------------------------
def bind_host_to_gpu_numa_node(index: int):
    """Run the calling thread on the CPUs of the NUMA node the GPU hangs off, so that pinned host buffers allocated
    next land in that node's memory (first touch).  Returns the previous affinity to restore, or None when the
    topology cannot be read.  Reads sysfs and NVML only; changes nothing on the GPU."""
    try:
        import pynvml

        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(index)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:
            bus = bus[4:]
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        old = os.sched_getaffinity(0)
        cpus &= old
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return old
    except Exception:
        return None


class ViewBatch:
    """A batch of views of one mesh on one GPU: the views are spread round-robin over CUDA streams (they are
    independent, so view b+1's binning overlaps with view b's compositing) and their gradients are summed.

    Random-triangle scenes (a view = the NDC vertex array rotated in the image plane): all views, on all streams,
    add into ONE packed accumulator, cleared and unpacked once per batch.  Camera-ring scene (a view = a 4x4
    projection*view matrix passed by value to the projection kernel): every stream has a packed accumulator of its
    own that one kernel per view carries through the projection's VJP into the shared world-space buffer with
    atomic additions.  Either way the summed gradients and the loss end up in ``self.grads`` (one contiguous fp32
    buffer, the object of the all-reduce)."""

    def __init__(self, torch, Vw, scene, dev, n_streams, one_kernel=False, host_threads=1):
        self.torch, self.Vw, self.scene, self.dev, self.one_kernel = torch, Vw, scene, dev, one_kernel
        # Every view makes the issuing host thread wait once (for the number of list entries, before the compositing
        # kernels can be launched).  With several host threads, each feeding its own streams, one thread's wait no
        # longer holds back the launches of the other streams (ctypes calls and the wait release the GIL).
        self.host_threads = max(1, host_threads)
        self.pool = None
        if self.host_threads > 1:
            from concurrent.futures import ThreadPoolExecutor

            self.pool = ThreadPoolExecutor(max_workers=self.host_threads)
        self.camera_ring = "mesh" in scene.meta
        self.W, self.H = scene.width, scene.height
        self.V = scene.num_vertices
        self.i = torch.from_numpy(scene.indices).to(dev)
        self.c = torch.from_numpy(scene.colors).to(dev)
        self.o = torch.from_numpy(scene.opacities).to(dev)
        self.points = torch.from_numpy(scene.meta["mesh"].points).to(dev) if self.camera_ring else None
        self.pos_comp = 3 if self.camera_ring else 4
        self.grads = Vw.GradBuffer.allocate(self.V, dev, position_components=self.pos_comp)
        self.n_streams = max(1, n_streams)
        self.side_streams = [torch.cuda.Stream(device=dev) for _ in range(self.n_streams - 1)]
        n_packed = self.n_streams if self.camera_ring else 1
        self.packed = [Vw.PackedGradients(self.V, dev) for _ in range(n_packed)]

    def render_view(self, v, target, si):
        """fwd + bwd of one view on the current stream (stream slot `si`)."""
        sc, Vw, g = self.scene, self.Vw, self.grads
        if self.camera_ring:
            Vw.l2_world_view_step(self.points, v, self.i, self.c, self.o, target, self.W, self.H, g.points, g.colors,
                                  g.opacities, g.loss, sc.tile_width, sc.tile_height, one_kernel=self.one_kernel,
                                  packed=self.packed[si])
        else:
            Vw.l2_view_step(v, self.i, self.c, self.o, target, self.W, self.H, None, None, None, None, sc.tile_width,
                            sc.tile_height, one_kernel=self.one_kernel, packed=self.packed[0])

    def run(self, items):
        """Render (vertices or matrix, target, ready_event) items; returns the summed loss (a view into ``grads``)."""
        torch = self.torch
        main = torch.cuda.current_stream(self.dev)
        if self.camera_ring:
            self.grads.zero_()          # the packed accumulators are left zero by every view
        else:
            self.packed[0].zero_()
        start = torch.cuda.Event()
        start.record(main)
        for st in self.side_streams:
            st.wait_event(start)
        def issue(si_set):
            torch.cuda.set_device(self.dev)          # the current device is a per-thread setting
            for b, (v, t, ready) in enumerate(items):
                si = b % self.n_streams
                if si not in si_set:
                    continue
                stream = main if si == 0 else self.side_streams[si - 1]
                with torch.cuda.stream(stream):
                    if ready is not None:
                        stream.wait_event(ready)
                        if isinstance(v, torch.Tensor):
                            v.record_stream(stream)
                        t.record_stream(stream)
                    self.render_view(v, t, si)

        if self.pool is None:
            issue(set(range(self.n_streams)))
        else:
            sets = [set(range(k, self.n_streams, self.host_threads)) for k in range(self.host_threads)]
            for f in [self.pool.submit(issue, ss) for ss in sets if ss]:
                f.result()
        for st in self.side_streams:
            done = torch.cuda.Event()
            done.record(st)
            main.wait_event(done)
        if not self.camera_ring:
            g = self.grads
            self.packed[0].unpack(self.W, self.H, g.points, g.colors, g.opacities, g.loss, accumulate=False)
        return self.grads.loss


def median_ms(torch, fn, flush, reps: int, warmup: int = 3):
    """Median device time of fn() over `reps` runs, L2 flushed before each, CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    ms = []
    for _ in range(reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ms.append(a.elapsed_time(b))
    return statistics.median(ms)


def single_view_times(torch, Vw, scene, verts_np, dev, flush, reps: int) -> dict:
    """ONE view on ONE stream: (a) through ``trigrad_b200.render`` + torch autograd of mean((image - target)^2), the
    reference's own signature and caller pattern; (b) through ``views.l2_view_step`` (loss fused into the backward)."""
    import trigrad_b200

    W, H = scene.width, scene.height
    v = torch.from_numpy(verts_np).to(dev)
    i = torch.from_numpy(scene.indices).to(dev)
    c = torch.from_numpy(scene.colors).to(dev)
    o = torch.from_numpy(scene.opacities).to(dev)
    target = torch.from_numpy(scene.target()).to(dev)
    V = scene.num_vertices

    def autograd_step():
        vv, cc, oo = v.detach().requires_grad_(), c.detach().requires_grad_(), o.detach().requires_grad_()
        image, _ = trigrad_b200.render(vv, i, cc, oo, W, H, scene.tile_width, scene.tile_height)
        torch.mean((image - target) ** 2).backward()

    gV = torch.zeros((V, 4), device=dev)
    gC = torch.zeros((V, 3), device=dev)
    gO = torch.zeros((V,), device=dev)
    loss = torch.zeros((), device=dev)

    def fused_step():
        Vw.l2_view_step(v, i, c, o, target, W, H, gV, gC, gO, loss, scene.tile_width, scene.tile_height)

    out = {}
    for key, fn in (("render_autograd", autograd_step), ("l2_view_step", fused_step)):
        ms = median_ms(torch, fn, flush, reps)
        out[key] = {"ms": ms, "mpix_s": W * H / (ms * 1e-3) / 1e6}
    out["note"] = ("one view, one stream, median of %d, L2 flushed before each; render_autograd = trigrad_b200.render + "
                   "torch autograd of mean((image-target)^2), gradients of vertices, colours and opacities") % reps
    return out


def other_config_times(torch, Vw, dev, flush, skip: str, reps: int = 5) -> dict:
    """fwd+bwd milliseconds per view of the other benchmark configurations (one view, one stream, fused loss)."""
    out = {}
    for name in ("cfg1", "cfg2", "cfg4", "cfg5"):
        if name == skip:
            continue
        scene, wname = make_scene(name)
        batch = ViewBatch(torch, Vw, scene, dev, 1)
        W, H = scene.width, scene.height
        if batch.camera_ring:
            view = scene.meta["pvs"][0]
        else:
            view = torch.from_numpy(scene.vertices).to(dev)
        target = torch.from_numpy(scene.target()).to(dev)
        ms = median_ms(torch, lambda: batch.run([(view, target, None)]), flush, reps, warmup=2)
        out[name] = {"workload": wname, "triangles": scene.num_triangles, "width": W, "height": H, "ms_per_view": ms,
                     "mpix_s": W * H / (ms * 1e-3) / 1e6}
        del batch, scene, view, target
        torch.cuda.empty_cache()
    return out


def cfg4_sharded_block(torch, dist, Vw, dev, rank: int, world: int, n_streams: int, flush, batches: int = 3) -> dict:
    """The multi-GPU configuration: the 64 cameras of the ring split in contiguous blocks over the ranks (strong
    scaling), world-space gradients through the projection VJP into one buffer, ONE in-place all-reduce of it."""
    scene, wname = make_scene("cfg4")
    pvs = scene.meta["pvs"]
    mine = list(Vw.shard_views(len(pvs), rank, world))
    n_s = min(n_streams, max(1, len(mine)))
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    batch = ViewBatch(torch, Vw, scene, dev, n_s, host_threads=max(1, min(n_s, cores // max(1, world))))
    W, H = scene.width, scene.height
    rng = np.random.default_rng(100 + rank)
    # a handful of distinct targets reused round-robin (64 full-size fp32 targets would be 2 GB of nothing new)
    targets = [torch.from_numpy(rng.random((H, W, 4), dtype=np.float32)).to(dev) for _ in range(min(4, len(mine)))]
    items = [(pvs[k], targets[n % len(targets)], None) for n, k in enumerate(mine)]

    def one_batch(ev=None):
        batch.run(items)
        if ev is not None:
            ev[1].record()
        if world > 1:
            Vw.allreduce_gradients(batch.grads)
        if ev is not None:
            ev[2].record()

    one_batch()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    tot, red = [], []
    for _ in range(batches):
        flush.zero_()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        if world > 1:
            dist.barrier()
        ev[0].record()
        one_batch(ev)
        ev[2].synchronize()
        tot.append(ev[0].elapsed_time(ev[2]))
        red.append(ev[1].elapsed_time(ev[2]))
    t = torch.tensor([statistics.median(tot), statistics.median(red)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_batch, ms_red = float(t[0]), float(t[1])
    V = scene.num_vertices
    return {"workload": wname, "cameras": len(pvs), "views_per_rank": len(mine), "scaling": "strong",
            "triangles": scene.num_triangles, "vertices": V, "streams": batch.n_streams,
            "ms_per_batch": ms_batch, "mpix_s": W * H * len(pvs) / (ms_batch * 1e-3) / 1e6,
            "triangles_per_s": scene.num_triangles * len(pvs) / (ms_batch * 1e-3),
            "ms_allreduce": ms_red if world > 1 else 0.0,
            "allreduce_share": (ms_red / ms_batch) if world > 1 else 0.0,
            "allreduce_bytes": (7 * V + 1) * 4 if world > 1 else 0,
            "note": "max over ranks of the median of %d batches; all-reduce timed with CUDA events around it "
                    "(includes waiting for the slowest rank)" % batches}


def run_sort_workload(args) -> None:
    """``--workload sort --pairs N``: the device-wide onesweep radix sort (``tg_sort_pairs``) on N random
    (uint64 key, uint32 value) pairs, 45 significant key bits (6 passes, as tile << 32 | depth keys of a 1080p frame).
    Prints algorithmic GB/s = (8 + 24 * passes) * N bytes / time against the measured HBM peak."""
    import torch

    from trigrad_b200 import _native as N
    from trigrad_b200 import stages as St

    torch.cuda.set_device(0)
    n = int(args.pairs)
    bits = 45
    passes = (bits + 7) // 8
    g = torch.Generator(device="cuda").manual_seed(0)
    keys = torch.randint(0, 1 << bits, (n,), dtype=torch.int64, device="cuda", generator=g)
    vals = torch.arange(n, dtype=torch.int32, device="cuda")
    buf = St.SortBuffers(n)
    ms = []
    launches0 = N.lib().tg_launch_count()
    with ClockSampler(0) as clk:
        for it in range(max(args.warmup, 3) + args.steps):
            buf.load(keys, vals)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            sk, sv = buf.sort(0, bits)
            b.record()
            b.synchronize()
            if it >= max(args.warmup, 3):
                ms.append(a.elapsed_time(b))
    assert int(buf.status[0]) == 0
    check = min(n, 1 << 20)
    assert bool((sk[1:check] >= sk[:check - 1]).all()), "not sorted"
    t = statistics.median(ms)
    peaks = load_peaks()
    nbytes = (8 + 24 * passes) * n
    gbs = nbytes / (t * 1e-3) / 1e9
    print(json.dumps({
        "metric": "onesweep radix sort, algorithmic GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": t, "higher_is_better": True, "dtype": "u64+u32", "data": "synthetic",
        "config": {"workload": "sort", "pairs": n, "key_bits": bits, "passes": passes,
                   "l2": "inputs of %d MB per buffer (larger than L2 from 2^24 pairs on)" % (12 * n >> 20)},
        "pairs_per_s": n / (t * 1e-3),
        "roofline": {"kernel": "sort_histogram_kernel + %d x onesweep_pass_kernel" % passes, "bound": "hbm", "achieved": gbs,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                     "peak_source": peaks["source"], "algorithmic_bytes_per_launch": nbytes, "ms_per_launch": t},
        "gpu_launches": int(N.lib().tg_launch_count() - launches0), "clocks": clk.summary()}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3", help="cfg1..cfg5, or `sort` (radix sort alone, see --pairs)")
    ap.add_argument("--pairs", type=float, default=float(1 << 25), help="--workload sort: number of pairs")
    ap.add_argument("--streams", type=int, default=4,
                    help="CUDA streams the views of a step are spread over (independent views overlap on the GPU)")
    ap.add_argument("--host-threads", type=int, default=0,
                    help="host threads that issue the views of a step, each feeding its own subset of the streams "
                         "(0 = one per stream)")
    ap.add_argument("--views-per-gpu", type=int, default=8,
                    help="views of the mesh rendered per GPU per step (a batch of views; gradients are summed)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the single-view, other-configuration and sharded camera-ring blocks of the line")
    ap.add_argument("--one-kernel", action="store_true",
                    help="forward and backward of a view in one compositing kernel (tg_render_step_l2)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if args.workload == "sort":
        if rank == 0:
            run_sort_workload(args)
        return

    import torch
    import torch.distributed as dist

    import trigrad_b200  # noqa: F401
    from trigrad_b200 import _native as N
    from trigrad_b200 import stages as St
    from trigrad_b200 import views as Vw

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    scene, wname = make_scene(args.workload)
    W, H = scene.width, scene.height
    T, V = scene.num_triangles, scene.num_vertices
    B = max(1, args.views_per_gpu)
    # rank r renders views [r*B, (r+1)*B) of the same mesh; every view has its own target image.
    camera_ring = "mesh" in scene.meta
    if camera_ring:
        views_np = [scene.meta["pvs"][(rank * B + b) % 64] for b in range(B)]
    else:
        views_np = [view_vertices(scene.vertices, rank * B + b) for b in range(B)]
    rng = np.random.default_rng(3 + rank)
    targets_np = [scene.target() if b == 0 else rng.random((H, W, 4), dtype=np.float32) for b in range(B)]
    verts_np = S_project(scene, views_np[0]) if camera_ring else views_np[0]

    n_streams = max(1, min(args.streams, B))
    # one issuing thread per stream, but no more threads than this rank's share of the host cores
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    host_threads = args.host_threads if args.host_threads > 0 else max(1, min(n_streams, cores // max(1, world)))
    batch = ViewBatch(torch, Vw, scene, dev, n_streams, one_kernel=args.one_kernel, host_threads=host_threads)
    grads = batch.grads
    pos_comp = batch.pos_comp
    dv = list(views_np) if camera_ring else [torch.from_numpy(x).to(dev) for x in views_np]
    dt = [torch.from_numpy(x).to(dev) for x in targets_np]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)    # > L2 (126 MB)
    lib = N.lib()

    def step(vs, ts):
        """One step: B views, then (N > 1) one all-reduce of the summed gradients."""
        loss = batch.run([(v, t, None) for v, t in zip(vs, ts)])
        if world > 1:
            Vw.allreduce_gradients(grads)
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if world > 1:
        # the first collectives on a communicator set up channels and buffers: keep that out of the steps
        for _ in range(5):
            Vw.allreduce_gradients(grads)
        barrier()
    for _ in range(max(args.warmup, 3)):
        step(dv, dt)
    barrier()

    # ---- timed region: K steps, CUDA events per step, L2 flushed between steps -----------------------
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    n_launch0 = lib.tg_launch_count()
    with ClockSampler(local_rank) as clk:
        barrier()
        t_wall0 = time.perf_counter()
        for k in range(args.steps):
            flush.zero_()
            starts[k].record()
            step(dv, dt)
            stops[k].record()
        barrier()
        t_wall = time.perf_counter() - t_wall0
    n_launch = lib.tg_launch_count() - n_launch0
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(total_ms.item()) / args.steps
    value = W * H * B * world / (ms_per_step * 1e-3) / 1e6

    # ---- end to end from host buffers through the public API -----------------------------------------
    # Every step copies all of its inputs from pinned host memory (shared mesh attributes once, per-view
    # vertices and target for each view) and copies the loss and the summed gradients back.  The copies of
    # view b+1 run on a second stream while view b renders; the loop is measured both with and without overlap
    # between consecutive steps (see e2e_loop).  Targets travel as 8-bit RGBA (what an image on
    # the host is; the loss reads value / 255): a quarter of the bytes of a float32 target.  The pinned buffers
    # are allocated from the NUMA node the GPU hangs off.
    old_affinity = bind_host_to_gpu_numa_node(local_rank)
    hi, hc, ho = (torch.from_numpy(x).pin_memory() for x in (scene.indices, scene.colors, scene.opacities))
    hp = torch.from_numpy(scene.meta["mesh"].points).pin_memory() if camera_ring else None
    hv = [] if camera_ring else [torch.from_numpy(x).pin_memory() for x in views_np]   # camera matrices stay on the host
    ht = [torch.from_numpy(np.round(x * 255).astype(np.uint8)).pin_memory() for x in targets_np]
    out_g = [torch.empty_like(grads.flat, device="cpu").pin_memory() for _ in range(2)]   # gradients and, last, the loss
    if old_affinity is not None:
        os.sched_setaffinity(0, old_affinity)
    h2d = sum(t.numel() * t.element_size() for t in [hi, hc, ho] + hv + ht + ([hp] if camera_ring else []))
    d2h = out_g[0].numel() * 4
    copy_stream = torch.cuda.Stream(device=dev)
    d2h_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    snapshot = [torch.empty_like(grads.flat) for _ in range(2)]

    class InputSet:
        """Device-side buffers for one step's inputs, allocated once: nothing is allocated or freed inside the loop."""

        def __init__(self):
            like = lambda h: torch.empty(h.shape, dtype=h.dtype, device=dev)
            self.shared = [like(h) for h in [hi, hc, ho] + ([hp] if camera_ring else [])]
            self.views = [like(h) for h in hv]
            self.targets = [like(h) for h in ht]
            self.free = None        # event: the step that last read this set has finished rendering

    input_sets = [InputSet(), InputSet()]

    def stage_inputs(s):
        """Queue one step's host->device copies into input set `s` on the copy stream (after the step that last read
        the set): the shared mesh attributes, then per view its vertices (or nothing: camera matrices are passed by
        value) and its target, each view with an event."""
        staged = []
        if s.free is not None:
            copy_stream.wait_event(s.free)
        with torch.cuda.stream(copy_stream):
            for d, h in zip(s.shared, [hi, hc, ho] + ([hp] if camera_ring else [])):
                d.copy_(h, non_blocking=True)
            for b in range(B):
                if not camera_ring:
                    s.views[b].copy_(hv[b], non_blocking=True)
                s.targets[b].copy_(ht[b], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
                staged.append((views_np[b] if camera_ring else s.views[b], s.targets[b], ev))
        return staged

    def e2e_loop(n: int, pipelined: bool) -> float:
        """n steps from host buffers; seconds per step by the host clock, everything delivered at the end.

        Not pipelined: a step's copies start once the step before has delivered its result to the host.
        Pipelined (two sets of buffers, the loop a trainer with a prefetching loader runs): the copies of step k+1
        are queued before step k is launched, and step k's result is copied to the host on a stream of its own while
        step k+1 renders; the host reads it one step late.  Either way every step copies all of its inputs and
        returns all of its gradients inside the timed region."""
        barrier()
        t0 = time.perf_counter()
        delivered = [None, None]
        pending = stage_inputs(input_sets[0]) if pipelined else None
        for k in range(n):
            s = input_sets[k % 2] if pipelined else input_sets[0]
            staged = pending if pipelined else stage_inputs(s)
            pending = stage_inputs(input_sets[(k + 1) % 2]) if pipelined and k + 1 < n else None
            batch.i, batch.c, batch.o = s.shared[:3]
            if camera_ring:
                batch.points = s.shared[3]
            batch.run(staged)        # each view waits for its own copies (queued after the shared ones)
            s.free = torch.cuda.Event()
            s.free.record(main_stream)      # run() has joined the side streams into this one
            if world > 1:
                Vw.allreduce_gradients(grads)
            if not pipelined:
                out_g[0].copy_(grads.flat, non_blocking=True)
                main_stream.synchronize()
                continue
            slot = k % 2
            if delivered[slot] is not None:
                delivered[slot].synchronize()           # the host has read step k-2 before its buffers are reused
            snapshot[slot].copy_(grads.flat)
            ready = torch.cuda.Event()
            ready.record(main_stream)
            d2h_stream.wait_event(ready)
            with torch.cuda.stream(d2h_stream):
                out_g[slot].copy_(snapshot[slot], non_blocking=True)
                delivered[slot] = torch.cuda.Event()
                delivered[slot].record(d2h_stream)
            if delivered[1 - slot] is not None:
                delivered[1 - slot].synchronize()       # result of the step before, read while this one renders
        for ev in delivered:
            if ev is not None:
                ev.synchronize()
        barrier()
        dt = torch.tensor([(time.perf_counter() - t0) / n], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        return float(dt.item())

    def copies_alone_gbs() -> float:
        """Host->device rate of one step's input copies with nothing else running (what bounds the pipelined loop
        when the step's rendering takes less time than its copies)."""
        best = float("inf")
        for _ in range(4):
            barrier()
            t0 = time.perf_counter()
            stage_inputs(input_sets[0])
            copy_stream.synchronize()
            best = min(best, time.perf_counter() - t0)
        return h2d / best / 1e9

    e2e_steps = max(3, min(args.steps, 20))
    h2d_gbs = copies_alone_gbs()
    # three rounds of e2e_steps steps each way, the median round reported (a single round on a freshly started box
    # was once several times slower than every other)
    e2e_loop(2, False)
    e2e_serial_s = sorted(e2e_loop(e2e_steps, False) for _ in range(3))[1]
    e2e_loop(3, True)
    e2e_s = sorted(e2e_loop(e2e_steps, True) for _ in range(3))[1]
    e2e_value = W * H * B * world / e2e_s / 1e6
    e2e_serial_value = W * H * B * world / e2e_serial_s / 1e6

    # ---- per-kernel timing for the roofline (stage entry points, CUDA events, L2 flushed) ------------
    stages = measure_stages(torch, St, scene, verts_np, flush, reps=max(5, min(20, args.steps)))
    peaks = load_peaks()
    dominant = max((s for s in stages.values() if isinstance(s, dict) and s.get("kernel")), key=lambda s: s["ms"])
    captured = NCU_DRAM_BYTES.get((dominant["kernel"], args.workload))
    roofline = {
        "kernel": dominant["kernel"], "bound": "hbm", "achieved": dominant["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
        "frac": dominant["gbs"] / peaks["hbm_gbs"], "traffic": captured[0] if captured else None,
        "traffic_source": captured[1] if captured else None,
        "peak_source": peaks["source"],
        "algorithmic_bytes_per_launch": dominant["bytes"], "ms_per_launch": dominant["ms"],
    }

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": wname, "triangles": T, "vertices": V, "width": W, "height": H,
                   "tile": [scene.tile_width, scene.tile_height], "per_pixel_sort": True, "max_layers": 32,
                   "views_per_gpu_per_step": B, "streams": n_streams, "host_threads": batch.host_threads, "one_kernel_step": bool(args.one_kernel), "K_pairs": stages["_K"], "l2": "256 MB buffer rewritten between timed steps",
                   "e2e_target_dtype": "u8 rgba (value / 255)",
                   "exchange": "none" if world == 1 else f"one NCCL all_reduce of {pos_comp + 4}V fp32 gradients per step"},
        "triangles_per_s": T * B * world / (ms_per_step * 1e-3),
        "ms_per_view": ms_per_step / B,
        "wall_s_timed_region": t_wall,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_s * 1e3, "steps": e2e_steps, "rounds": "median of 3", "h2d_gbs_copies_alone": h2d_gbs,
                "pipeline": "two buffer sets: step k+1's inputs are copied while step k renders, step k's gradients "
                            "are read back while step k+1 renders; every step's copies are inside the timed region",
                "unpipelined": {"value": e2e_serial_value, "ms_per_step": e2e_serial_s * 1e3,
                                "note": "a step's copies start after the step before has delivered its result"}},
        "gpu_launches": int(n_launch),
        "clocks": clk.summary(),
        "roofline": roofline,
        "stages": {k: s for k, s in stages.items() if not k.startswith("_")},
    }
    if not args.no_extras:
        if rank == 0:
            line["single_view"] = single_view_times(torch, Vw, scene, verts_np, dev, flush, reps=20)
            if world == 1:
                line["other_configs"] = other_config_times(torch, Vw, dev, flush, skip=args.workload)
        del batch, dv, dt
        torch.cuda.empty_cache()
        sharded = cfg4_sharded_block(torch, dist, Vw, dev, rank, world, args.streams, flush)
        line["cfg4_sharded"] = sharded
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cv, cdt, cores, sample = time_cpu(scene, steps=3, warmup=1, limit_s=25.0)
        line["cpu_baseline"] = {"value": cv, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                "ms_per_step": cdt * 1e3}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (read + write) of one launch of the dominant kernel from an ncu capture of the same kernel on the same
# workload, with the summary the figure was read from; the kernels may have changed since that capture.
NCU_DRAM_BYTES = {
    ("blend_backward_queued_kernel (+ memset, unpack_gradients_kernel)", "cfg3"):
        (183.2e6 + 11.5e6 + 13.0e6 + 38.4e6, "profiles/blend_kernels_cfg3.md"),
    ("blend_forward_kernel", "cfg3"): (53.1e6 + 45.5e6, "profiles/blend_kernels_cfg3.md"),
    ("blend_forward_kernel", "cfg4"): (256.4e6 + 73.5e6, "profiles/blend_forward_cfg4_view.md"),
}


def load_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


def measure_stages(torch, St, scene, verts_np, flush, reps: int) -> dict:
    """Average device time of each kernel of the path on the bench workload and its algorithmic bytes."""
    import copy

    sc = copy.copy(scene)
    sc.vertices = verts_np
    tens = St.scene_tensors(sc)
    T, V, W, H = sc.num_triangles, sc.num_vertices, sc.width, sc.height
    tiles = St.num_tiles(sc)

    def timed(fn, setup=None):
        ms = []
        out = None
        for _ in range(reps):
            if setup is not None:
                setup()
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = fn()
            b.record()
            b.synchronize()
            ms.append(a.elapsed_time(b))
        return statistics.median(ms), out

    from trigrad_b200 import wrapper as Wr

    # forward: the stage times come from events recorded inside the one forward call (L2 flushed before it)
    acc = {k: [] for k in Wr.TIMING_KEYS}
    out = None
    for _ in range(reps):
        flush.zero_()
        out = Wr.forward_native(*tens, W, H,
                                sc.tile_width, sc.tile_height, 1 / 256, True, True, 32, cull_tiles=True)
        for k in acc:
            acc[k].append(out[9][k] * 1e3)
    med = {k: statistics.median(v) for k, v in acc.items()}
    image, depth, fw, sids, offsets, geo, attr, ends, sel, _ = out
    K = int(sids.numel())
    fwd = (image, depth, fw, ends, sel)
    res = {}
    res["init"] = {"kernel": "memset", "ms": med["init"], "bytes": 4 * tiles + 8 * ((T + 255) // 256)}
    res["binning"] = {"kernel": "preprocess_count_kernel", "ms": med["bary_transforms"],
                      "bytes": 12 * T + 32 * V + 164 * T + 8 * tiles}
    res["emit_entries"] = {"kernel": "emit_keys_kernel<direct> (with the read-back of K)", "ms": med["per_tile_lists"],
                           "bytes": 16 * T + 16 * V + 8 * K + 8 * tiles}
    res["tile_sort"] = {"kernel": "tile_sort_kernel (+ tile_sort_mid_kernel, tile_sort_long_kernel when needed)", "ms": med["sorting"],
                        "bytes": 12 * K + 8 * tiles}
    res["blend_forward"] = {"kernel": "blend_forward_kernel", "ms": med["rasterization"], "bytes": 100 * K + 28 * W * H}
    gi = torch.randn((H, W, 4), device="cuda")
    gd = torch.zeros((H, W), device="cuda")
    ms, _ = timed(lambda: St.blend_backward(sc, geo, attr, sids, offsets, fwd, gi, gd))
    res["blend_backward"] = {"kernel": "blend_backward_queued_kernel (+ memset, unpack_gradients_kernel)", "ms": ms, "bytes": 100 * K + 48 * W * H + 32 * V}
    for s in res.values():
        s["gbs"] = s["bytes"] / (s["ms"] * 1e-3) / 1e9 if s["ms"] > 0 else 0.0
    res["_K"] = K
    return res


if __name__ == "__main__":
    main()
