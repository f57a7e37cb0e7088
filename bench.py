"""Benchmark of the submanifold sparse-convolution inference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (benchmark configuration 3): 3-D submanifold U-Net inference, m=32, reps=2,
planes 32..224, 4096^3 field, batch of 8 synthetic rooms of ~200 k voxels each per GPU.
One step = one forward over the batch with a FRESH Metadata: input-layer hash build, every
rulebook, every layer, the 20-class linear head and (N > 1) the NCCL gather of the per-voxel
scores to rank 0.  `value` = voxels/s with inputs resident in HBM; `e2e` = the same through the
public API from pinned host buffers (host->device copy of coordinates and features,
device->host copy of the scores inside the timed region).  `scaling` "weak": every rank runs its
own 8 rooms; with N > 1 the line also carries `strong_scaling` (the same 8 rooms split over the
ranks by batch index) and `gather_check` (what the gather delivered, checked untimed).

Also on the line: `roofline` of the convolution kernel with the largest share of the step and
`breakdown_ms_per_step` (CUDA events around every operator call), `configs` (voxels/s of
configurations 1, 2, 4 and 5 with the reference's CPU figure beside each), `submanifold_conv`
(configuration 1 cold / warm / rulebook only), `variants_voxels_per_sec`, `training_step`,
`cpu_baseline` (the reference's own Python package and CPU extension on this box's host cores, the
same batch) and `clocks`.

`--impl reference` times that reference CPU path on the same 8-room batch per step; it imports
neither this package nor its library.  `--probe-mma` prints the measured cost of tcgen05.mma.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIG = 3
ROOMS_PER_GPU = 8
METRIC = "unet3d_voxels_per_sec"
UNIT = "voxels/s"
# DRAM bytes per launch of a convolution kernel as a multiple of the algorithmic bytes of that
# launch, from ncu captures of a 4-room case (dram__bytes_read + dram__bytes_write of consecutive
# launches against their algorithmic bytes).  The traffic grows with the rows, like the
# algorithmic bytes: DRAM sees input, rulebook and output about once, the gather's re-reads
# (which the algorithmic figure counts per rule) hit L2.
TRAFFIC_RATIO = {"k_conv_tma": 0.22, "k_conv_pipe_mma": 0.22, "k_conv_rows": 0.24, "k_conv_simt": 0.25,
                 "k_conv_wide": 0.17}
# (bound reported for the kernel, what the ncu captures show as its limiter)
LIMITS = {
    "k_conv_tma": ("hbm", "shared-memory data pipe 77 % busy, tensor pipe 40-46 % (ncu, 4-room case)"),
    "k_conv_pipe_mma": ("hbm", "instruction issue and the shared-memory data pipe of small (offset, 128-row) steps"),
    "k_conv_rows": ("hbm", "no saturated pipe (ncu, 4-room case): warp-level tensor pipe 41-53 % active, LSU wavefronts "
                           "39-47 % of peak, issue slots 42-57 %; the warp's dependent chain rulebook entry -> gather -> "
                           "fragment loads -> bf16 split -> tensor instruction with 13-19 warps per SM; DRAM sees 0.19-0.24 "
                           "of the algorithmic bytes, the gather's re-reads hit L2"),
    "k_conv_wide": ("hbm", "shared-memory bandwidth: a 32-plane step writes 45 KB of tiles and slabs and the tensor core reads "
                           "72 KB of operands, against 128 B per cycle; tensor pipe 47.5 % active (ncu, 4-room case)"),
    "k_conv_tc": ("hbm", "latency: few 256-row tiles per level (tensor pipe 13-16 %)"),
}
# what `dtype` says for each arithmetic mode: the type the path computes in, kernel by kernel
DTYPE_LABEL = {
    "fp32": "f32 (fp32 FMA in every convolution)",
    "tf32x3": "f32-class split arithmetic, fp32 accumulate: every operand as two bf16 parts, three bf16 products "
              "per term -- warp-level mma.sync.m16n8k16 for 32/64 output planes, tcgen05 kind::f16 with TMEM "
              "accumulators for wider layers",
    "tf32": "tf32 (single pass, fp32 accumulate)",
    "bf16": "bf16 (single pass, fp32 accumulate)",
}
CONFIG_NAMES = {
    1: "config1: SubmanifoldConvolution 3D f3 32->32, 256^3 shells and planes, batch 1, fresh Metadata per step",
    2: "config2: 2D stroke classifier (VGG stack -> SparseToDense 10x10x32), batch 100, field 87x87",
    4: "config4: 3D SparseResNet on 127^3, batch 16 superquadric surfaces, 50-class head",
    5: "config5: 4D stack 4 x (SubmanifoldConvolution 64->64 f3 = 81 offsets + BatchNormReLU), 4 sequences x 8 frames",
}


def workload_name(rooms=ROOMS_PER_GPU):
    return ("config3: 3D submanifold U-Net m=32 reps=2 planes[32..224] 4096^3, %d rooms x ~200k voxels "
            "per GPU, fp32, fresh Metadata per step" % rooms)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peak_tflops():
    """Dense tf32 peak used for the tensor-pipe utilisation figure: half of the measured sustained
    bf16 cuBLAS figure (there is no tf32 entry in MEASURED_PEAKS.json), else half of the
    fallback 1400."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return 0.5 * float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 1400.0))), "0.5 x measured bf16 sustained"
    return 700.0, "0.5 x fallback bf16 sustained"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while a timed region runs
    (read-only queries).  NVML is initialised in the constructor, on the calling thread and before
    anything is timed: the library's first initialisation in a process holds up kernel launches of the
    same process for tens to hundreds of milliseconds (measured: one 707 ms step among 13.7 ms ones when
    it ran beside the timed loop); the queries themselves do not disturb it."""

    def __init__(self, index, period=0.02):
        threading.Thread.__init__(self, daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop_flag = threading.Event()
        self._nv = self._handle = None
        try:
            import pynvml as nv
            nv.nvmlInit()
            self._handle = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self._handle, nv.NVML_CLOCK_SM)
            nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)  # first query of each kind: here, not in the loop
            self._get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons
            self._get_reasons(self._handle)
            self._nv = nv
        except Exception as e:  # clocks are evidence, not a dependency
            self.reasons.add("unavailable: %s" % type(e).__name__)

    def run(self):
        nv, h = self._nv, self._handle
        if nv is None:
            return
        try:
            names = {
                getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            }
            while not self._stop_flag.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = self._get_reasons(h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
                time.sleep(self.period)
        except Exception as e:
            self.reasons.add("unavailable: %s" % type(e).__name__)

    def stop(self):
        self._stop_flag.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def conv_bytes(r):
    """Algorithmic bytes of one convolution call: one gathered input row and one 8-byte rule
    per rule, every output row written once, the weights once."""
    groups = r["groups"]
    cin, cout = r["cin"] * groups, r["cout"] * groups
    rules = r["macs"] / max(r["cin"] * r["cout"] * groups, 1)
    return rules * (cin * 4 + 8) + r["n_out"] * cout * 4 + r["offsets"] * r["cin"] * r["cout"] * groups * 4


def op_bytes(r):
    k = r["kind"]
    if k == "conv":
        return conv_bytes(r)
    if k == "batchnorm":
        return 2.0 * r["rows"] * r["planes"] * 4
    if k == "rules_submanifold":
        # coords in, one slot written at insert time is accounted to input_hash; here: one key
        # read per site, one 16-byte slot per probe, one 4-byte table entry per (site, offset)
        return r["sites"] * 8 + r["sites"] * r["offsets"] * (16 + 4)
    if k == "rules_strided":
        return r["sites"] * (8 + 16 + 16) + r.get("sites_out", 0) * (16 + 8 + 4 * r["offsets"])
    if k == "input_hash":
        return r["rows"] * r["cols"] * 8 + r["rows"] * 16 + r.get("sites", 0) * 8
    if k == "rows_affine":
        return r["rows"] * (r["nin"] + r["nout"]) * 4
    if k == "input_features":
        return (r["rows"] + r["sites"]) * r["planes"] * 4
    return 0.0


def summarize_profile(rows):
    """Per kernel class: time, calls, algorithmic bytes and FLOPs of one step.  Convolution calls
    are split by the kernel that ran them.  A rulebook lookup that was served from the Metadata's
    cache is counted as a call but gets no bytes: only the call that built the rulebook moved them."""
    agg = {}
    for r in rows:
        name = r.get("kernel", r["kind"]) if r["kind"] == "conv" else r["kind"]
        a = agg.setdefault(name, {"ms": 0.0, "calls": 0, "bytes": 0.0, "flops": 0.0})
        if r["kind"].startswith("rules_"):
            a["built"] = a.get("built", 0) + (1 if r.get("built", True) else 0)
            if r.get("overlapped") and r.get("built", True):
                # built on the side stream beside other operators: the call only took the result over
                a["overlapped_builds"] = a.get("overlapped_builds", 0) + 1
            if not r.get("built", True) or r.get("overlapped"):
                a["calls"] += 1
                a["cached_ms"] = a.get("cached_ms", 0.0) + r["ms"]
                continue
        a["ms"] += r["ms"]
        a["calls"] += 1
        a["bytes"] += op_bytes(r)
        if r["kind"] == "conv":
            a["flops"] += 2.0 * r["macs"]
    return agg


def load_workloads():
    """The workload generators, loaded by path: importing the package would load the CUDA library,
    which the reference arm must not do."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("scn_workloads", os.path.join(ROOT, "sparseconvnet_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class ReferenceCpu(object):
    """The reference's own stock path on the host cores: its unmodified Python package
    (scn.InputLayer, scn.UNet, scn.SparseResNet ... from sparseconvnet/*.py) on its own CPU
    extension, both staged under oracle/_ref by oracle/build_ref.py.  Falls back to the numpy
    restatement only where that build is absent (kind "port")."""

    def __init__(self, workloads):
        import torch
        from oracle import refpkg
        self.workloads, self.torch = workloads, torch
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        self.kind = "reference" if refpkg.available("cpu") else "port"
        self.scn = refpkg.load("cpu") if self.kind == "reference" else None

    def prepare(self, config, samples):
        """Returns (step function, voxels per step); one step = one forward over the whole batch with a
        fresh Metadata, as in the GPU arm."""
        torch, wl = self.torch, self.workloads
        coords, feats = wl.make_batch(config, samples)
        if self.kind == "reference":
            inp, net, head = wl.build_config(config, scn=self.scn)
            c, f = torch.from_numpy(coords), torch.from_numpy(feats)

            def step():
                with torch.no_grad():
                    y = net(inp([c, f]))
                    return head(y.features) if head is not None else y
        else:
            from oracle import runner
            inp, net, head = wl.build_config(config)
            be = runner.PortBackend()

            def step():
                y = runner.run_module(net, runner.run_module(inp, [coords, feats], be), be)
                return runner.run_module(head, y, be) if head is not None else y
        return step, coords.shape[0]

    def time(self, config, samples, warmup, steps):
        step, n = self.prepare(config, samples)
        for _ in range(warmup):
            step()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        dt = time.perf_counter() - t0
        return n * steps / dt, dt / steps, n


def run_reference(args, rank):
    """The reference's CPU implementation on the host cores, on the same batch as rank 0 of the GPU
    arm: K steps of all 8 rooms each."""
    if rank != 0:
        return
    cpu = ReferenceCpu(load_workloads())
    samples = list(range(args.rooms)) if cpu.kind == "reference" else [0]
    v, sec, n = cpu.time(CONFIG, samples, args.warmup, args.steps)
    sample = "the whole batch of rank 0 (%d rooms, %d voxels) per step, %d steps" % (len(samples), n, args.steps)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sec,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(len(samples)), "voxels_per_step": n, "sample": sample,
                   "path": "the reference's own Python package and CPU extension" if cpu.kind == "reference"
                   else "numpy restatement (the compiled reference is absent)"},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cpu.cores, "kind": cpu.kind, "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def cpu_baseline_sample(workloads, rooms):
    """Bounded CPU sample for the default run: the reference on the same batch as the GPU arm,
    1 warm-up + 2 timed forwards."""
    cpu = ReferenceCpu(workloads)
    samples = list(range(rooms)) if cpu.kind == "reference" else [0]
    v, sec, n = cpu.time(CONFIG, samples, 1, 2)
    return cpu, {"value": v, "unit": UNIT, "cores": cpu.cores, "kind": cpu.kind, "ms_per_step": 1e3 * sec,
                 "sample": "%d rooms, %d voxels per forward, mean of 2 forwards after 1 warm-up" % (len(samples), n)}


def run_probe_mma(args):
    """Cycles per tcgen05.mma for every legal (M, N, kind) the kernels could issue, measured by the
    library's own probe entry point: one CTA (clock64 figures) and one CTA per SM (CUDA-event
    figure), 2048 instructions each."""
    import ctypes as C
    import torch
    from sparseconvnet_b200 import SCN
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    sampler = ClockSampler(0)
    sampler.start()
    rows = []
    n_mma = 2048
    n_sm = torch.cuda.get_device_properties(0).multi_processor_count
    for a_tmem in (0, 1):
        for m in (128, 64):
            if a_tmem and m != 128:
                continue
            for bf16 in (0, 1):
                for n in (8, 16, 32, 48, 64, 96, 128, 192, 256):
                    if n < (16 if m == 128 else 8):
                        continue
                    rec = {"M": m, "N": n, "kind": "bf16 k16" if bf16 else "tf32 k8", "A": "tmem" if a_tmem else "smem"}
                    for ctas, tag in ((1, "one_cta"), (n_sm, "all_sms")):
                        ci, ct, ms = C.c_double(), C.c_double(), C.c_double()
                        SCN.check(SCN.lib.scn_tc_probe_mma(m, n, bf16, a_tmem, n_mma, ctas, SCN._stream(),
                                                           C.byref(ci), C.byref(ct), C.byref(ms)))
                        rec[tag] = {"cycles_issue": round(ci.value, 1), "cycles_complete": round(ct.value, 1),
                                    "event_us": round(1e3 * ms.value, 1)}
                    rows.append(rec)
    clocks = sampler.stop()
    print(json.dumps({"probe": "tcgen05.mma cycles per instruction", "instructions_per_cta": n_mma,
                      "clocks": clocks, "rows": rows}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--probe-mma", action="store_true",
                    help="print the measured cost of one tcgen05.mma per shape and exit (1 GPU)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="tf32x3", choices=["fp32", "tf32x3", "tf32", "bf16"],
                    help="convolution arithmetic of the headline number (tf32x3 and fp32 meet the fp32 parity bar)")
    ap.add_argument("--no-variants", action="store_true", help="skip timing the other arithmetic modes")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--data-parallel-training", action="store_true",
                    help="with --gpus N > 1: also time a training step of two rooms per rank with BatchNorm statistics "
                         "and gradients exchanged between the ranks (`training_step_data_parallel` on the line)")
    ap.add_argument("--no-config1", action="store_true", help="skip the single-convolution (configuration 1) numbers")
    ap.add_argument("--rooms", type=int, default=ROOMS_PER_GPU,
                    help="rooms per GPU; the benchmark is 8, smaller values are for profiler captures of a small case")
    ap.add_argument("--profile-out", default=None, help="write the per-operator breakdown to this file")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank)
    if args.probe_mma:
        return run_probe_mma(args)

    import numpy as np
    import torch
    import torch.distributed as dist
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import SCN, shard, workloads

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    count_group = None
    if world > 1:  # row counts travel on the host, not through the stream
        try:
            count_group = shard.host_group()
        except Exception as e:  # no host group: the counts go through NCCL and are read back from the device
            sys.stderr.write("host group for the row counts unavailable (%s); using the device path\n" % e)

    inp, net, head = workloads.build_config(CONFIG)
    net.to(dev)
    head.to(dev)
    head_wt = head.weight.detach().t().contiguous()
    head_b = head.bias.detach()

    def scores(x, out=None):
        """The 20-class head on the library's rows-times-small-matrix kernel (one read of the rows, one
        write of the scores; torch.nn.Linear's weight transposed)."""
        return SCN.rows_affine(x, head_wt, head_b, out=out)

    class Job(object):
        """One rank's share of a batch: resident and pinned copies of its inputs, the gather buffers."""

        def __init__(self, samples):
            self.samples = list(samples)
            if self.samples:
                c, f = workloads.make_batch(CONFIG, self.samples)
            else:  # more ranks than rooms: an empty shard still takes part in the collectives
                c, f = np.zeros((0, 4), np.int64), np.zeros((0, 3), np.float32)
            self.coords_host = torch.from_numpy(c).pin_memory()
            self.feats_host = torch.from_numpy(f).pin_memory()
            self.coords_dev, self.feats_dev = self.coords_host.to(dev), self.feats_host.to(dev)
            self.n_vox = c.shape[0]
            self.total_vox = self.n_vox
            self.gather = None
            if world > 1:
                t = torch.tensor([self.n_vox, self.n_vox], device=dev, dtype=torch.int64)
                tmax = t.clone()
                dist.all_reduce(t)
                dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
                self.total_vox = int(t[0].item())
                # rank 0 receives every rank's scores; the head writes them into the gather buffer
                self.gather = shard.RowGather(20, int(tmax[0].item()), dev, count_group=count_group, dst=0)
            self.pending = []

        def forward(self, c, f):
            """This rank's per-voxel scores.  With N > 1 the head writes them into this rank's block of
            the gather buffer and one NCCL gather (to rank 0) is enqueued; it runs beside the kernels of
            the next step and is taken one step later (after the last step: drain, inside the timed region)."""
            with torch.no_grad():
                x = net(inp([c, f])).features
                if self.gather is None:
                    return scores(x)
                y = scores(x, out=self.gather.block(x.shape[0]))
                self.pending.append(self.gather.start(x.shape[0]))
                if len(self.pending) > 1:
                    self.pending.pop(0).wait()
            return y

        def drain(self):
            while self.pending:
                self.pending.pop(0).wait()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, begin=None, end=None, drain=None):
        # a cyclic-GC pass of the interpreter in the middle of a step stalls the launch thread for
        # tens of ms (seen as one 70 ms step among 31 ms ones): collect before, not during
        import gc
        gc.collect()
        gc.disable()
        try:
            return _timed(fn, steps, begin, end, drain)
        finally:
            gc.enable()

    def _timed(fn, steps, begin, end, drain):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = SCN.launch_count()
        w0 = SCN.host_wait_count()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps - 1)]
        a.record()
        if begin:
            begin(steps)
        for i in range(steps):
            fn()
            if i < steps - 1:
                marks[i].record()
        if end:
            end()
        if drain:
            drain()
        b.record()
        barrier()
        ms = a.elapsed_time(b)
        edges = [a] + marks + [b]
        timed.per_step = [round(edges[i].elapsed_time(edges[i + 1]), 3) for i in range(steps)]
        launches = SCN.launch_count() - l0
        timed.host_waits = SCN.host_wait_count() - w0
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, launches

    class E2E(object):
        """End to end: every step copies its inputs from pinned host memory and its scores back to pinned
        host memory.  As in a serving loop, the copies run on two copy streams and overlap the
        neighbouring steps' kernels: the inputs of step i+1 travel while step i computes (two device
        input buffers), the scores of step i travel while step i+1 computes (two host output buffers)."""

        def __init__(self, job):
            self.job = job
            self.main = torch.cuda.current_stream()
            self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
            self.c_buf = [torch.empty_like(job.coords_dev) for _ in range(2)]
            self.f_buf = [torch.empty_like(job.feats_dev) for _ in range(2)]
            self.out_buf = [torch.empty(job.n_vox, 20, dtype=torch.float32).pin_memory() for _ in range(2)]
            self.in_ready = [torch.cuda.Event() for _ in range(2)]
            self.in_free = [torch.cuda.Event() for _ in range(2)]
            self.out_free = [torch.cuda.Event() for _ in range(2)]

        def fetch_inputs(self, b):
            with torch.cuda.stream(self.s_in):
                self.s_in.wait_event(self.in_free[b])      # the step that last read this buffer has finished
                self.c_buf[b].copy_(self.job.coords_host, non_blocking=True)
                self.f_buf[b].copy_(self.job.feats_host, non_blocking=True)
                self.in_ready[b].record(self.s_in)

        def begin(self, steps):
            self.i, self.steps = 0, steps
            for b in range(2):
                self.in_free[b].record(self.main)
                self.out_free[b].record(self.main)
            self.fetch_inputs(0)

        def step(self):
            b = self.i & 1
            if self.i + 1 < self.steps:
                self.fetch_inputs(b ^ 1)
            self.main.wait_event(self.in_ready[b])
            self.main.wait_event(self.out_free[b])     # the scores of two steps ago have left their buffer
            y = self.job.forward(self.c_buf[b], self.f_buf[b])
            self.in_free[b].record(self.main)
            done = torch.cuda.Event()
            done.record(self.main)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                self.out_buf[b].copy_(y, non_blocking=True)
                self.out_free[b].record(self.s_out)
            y.record_stream(self.s_out)
            self.i += 1
            return y

        def end(self):
            self.main.wait_stream(self.s_out)          # the last scores have reached the host inside the timed region

    def measure(job, steps, warmup):
        """(ms resident, launches, per-step ms, clocks, ms end to end) of `steps` forwards of `job`."""
        sampler = ClockSampler(local)  # NVML comes up here, before the warm-up
        for _ in range(warmup):
            job.forward(job.coords_dev, job.feats_dev)
        job.drain()
        # Still untimed: the warm-up goes on until two steps in a row are within 3 % of the fastest step seen, eight
        # more steps at most (clocks that are still rising after the idle seconds of the set-up, memory pools that
        # are still growing: seen once as 25 and 32 ms for the first two of ten timed steps of 13.1 ms).  Every rank
        # takes the same decision (the largest step time over the ranks).
        best, calm, extra, seen = None, 0, 0, []
        while extra < 8 and calm < 2:
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            job.forward(job.coords_dev, job.feats_dev)
            job.drain()
            t1.record()
            t1.synchronize()
            step_ms = torch.tensor([t0.elapsed_time(t1)], device=dev)
            if world > 1:
                dist.all_reduce(step_ms, op=dist.ReduceOp.MAX)
            step_ms = float(step_ms.item())
            extra += 1
            seen.append(round(step_ms, 3))
            best = step_ms if best is None else min(best, step_ms)
            calm = calm + 1 if step_ms <= 1.03 * best and extra > 1 else 0
        measure.settle_steps = seen
        sampler.start()
        ms, launches = timed(lambda: job.forward(job.coords_dev, job.feats_dev), steps, drain=job.drain)
        per_step = timed.per_step
        measure.host_waits_per_step = timed.host_waits / float(steps)
        clocks = sampler.stop()
        loop = E2E(job)
        for _ in range(2):
            loop.begin(1)
            loop.step()
            loop.end()
        job.drain()
        ms_e2e, _ = timed(loop.step, steps, loop.begin, loop.end, drain=job.drain)
        measure.per_step_e2e = timed.per_step
        return ms, launches, per_step, clocks, ms_e2e

    scn.set_precision(args.precision)
    job = Job(range(rank * args.rooms, (rank + 1) * args.rooms))
    ms, launches, per_step, clocks, ms_e2e = measure(job, args.steps, args.warmup)
    settle_steps = measure.settle_steps
    total_vox, n_vox = job.total_vox, job.n_vox
    value = total_vox * args.steps / (ms / 1e3)
    e2e = total_vox * args.steps / (ms_e2e / 1e3)

    # ---- N > 1: what the gather delivered, checked outside the timed region ------------------------------
    gather_check = None
    strong = None
    if world > 1:
        with torch.no_grad():
            y_ref = scores(net(inp([job.coords_dev, job.feats_dev])).features)     # the plain path, own rows
            check = shard.RowGather(20, job.gather.capacity, dev, count_group=count_group, dst=None, depth=1)
            scores(net(inp([job.coords_dev, job.feats_dev])).features, out=check.block(y_ref.shape[0]))
            views, counts = check.start(y_ref.shape[0]).blocks()
            torch.cuda.synchronize()
        # every rank: its own block of the gathered buffer holds exactly the bits of its plain result;
        # rank 0: every block's checksum equals the checksum its sender computed from its own result
        own_equal = bool(torch.equal(views[rank], y_ref))
        sums = torch.stack([v.double().sum() for v in views])
        mine = torch.zeros(world, dtype=torch.float64, device=dev)
        mine[rank] = y_ref.double().sum()
        dist.all_reduce(mine)
        flags = torch.tensor([1 if own_equal else 0, 1 if torch.equal(sums, mine) else 0], device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        gather_check = {"own_block_bit_equal_on_every_rank": bool(flags[0].item()),
                        "block_checksums_match_senders": bool(flags[1].item()),
                        "counts": counts, "counts_add_up": sum(counts) == total_vox}
        del check, views, y_ref
        # strong scaling of the batch the metric names: the same 8 rooms split over the ranks by batch index
        lo, hi = shard.shard_range(ROOMS_PER_GPU, rank, world)
        sjob = Job(range(lo, hi))
        s_ms, _, s_per_step, _, s_ms_e2e = measure(sjob, args.steps, args.warmup)
        strong = {"workload": workload_name(ROOMS_PER_GPU).replace("per GPU", "in all, split over %d GPUs" % world),
                  "voxels_per_step": sjob.total_vox, "rooms_per_rank": [len(range(*shard.shard_range(ROOMS_PER_GPU, r, world)))
                                                                         for r in range(world)],
                  "value": sjob.total_vox * args.steps / (s_ms / 1e3), "unit": UNIT, "ms_per_step": s_ms / args.steps,
                  "e2e_value": sjob.total_vox * args.steps / (s_ms_e2e / 1e3), "e2e_ms_per_step": s_ms_e2e / args.steps,
                  "scaling": "strong"}
        del sjob

    # ---- per-operator breakdown (CUDA events around every operator call, four extra steps) -------
    # An operator's pair of events also sees the GPU idle when the host is late with the launch in between (seen:
    # one call of 4 ms among its 0.6 ms peers).  So the step is profiled four times with the cyclic GC held off as
    # in the timed regions; the first pass, which creates the events' pool, is dropped and every call is given
    # the median of its three times.
    import gc
    gc.collect()
    gc.disable()
    profiled = []
    try:
        for i in range(4):
            torch.cuda.synchronize()
            with SCN.Profile() as prof:
                job.forward(job.coords_dev, job.feats_dev)
            job.drain()
            if i:
                profiled.append(prof.rows())
    finally:
        gc.enable()
    prof_rows = profiled[-1]
    if all(len(r) == len(prof_rows) and all(x["kind"] == y["kind"] for x, y in zip(r, prof_rows)) for r in profiled):
        for j, row in enumerate(prof_rows):
            row["ms"] = sorted(r[j]["ms"] for r in profiled)[len(profiled) // 2]
    agg = summarize_profile(prof_rows)
    peak, peak_src = peaks()
    tpeak, tsrc = tensor_peak_tflops()
    conv_classes = [k for k in agg if agg[k]["flops"]]
    top = max(conv_classes or agg, key=lambda k: agg[k]["ms"])
    a = agg[top]
    achieved = a["bytes"] / (a["ms"] / 1e3) / 1e9
    roofline = {"kernel": top, "bound": LIMITS.get(top, ("hbm", None))[0], "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                "frac_of_nominal_7700": achieved / 7700.0,
                "traffic": (TRAFFIC_RATIO[top] * a["bytes"] / a["calls"]) if top in TRAFFIC_RATIO else None,
                "algorithmic_bytes_per_launch": a["bytes"] / a["calls"], "launches_per_step": a["calls"],
                "ms_per_step": a["ms"], "tflops": a["flops"] / (a["ms"] / 1e3) / 1e12 if a["flops"] else None,
                "limiter": LIMITS.get(top, (None, None))[1]}
    if a["flops"]:
        # the same kernel against the tensor pipe: algorithmic FLOPs (2 x rules x Cin x Cout; the
        # split mode issues three products per FLOP counted) over the dense tf32 peak
        roofline["tensor"] = {"achieved": roofline["tflops"], "peak": tpeak, "unit": "TFLOP/s",
                              "frac": roofline["tflops"] / tpeak, "peak_source": tsrc}
    breakdown = {}
    for k, v in sorted(agg.items(), key=lambda kv: -kv[1]["ms"]):
        gbps = v["bytes"] / (v["ms"] / 1e3) / 1e9 if v["ms"] > 0 else None
        breakdown[k] = {"ms": round(v["ms"], 4), "calls": v["calls"], "GBps": round(gbps, 1) if gbps else None,
                        "frac_of_hbm_peak": round(gbps / peak, 3) if gbps else None}
        if v["flops"]:
            tf = v["flops"] / (v["ms"] / 1e3) / 1e12
            breakdown[k]["TFLOPs"] = round(tf, 1)
            breakdown[k]["frac_of_tf32_peak"] = round(tf / tpeak, 3)
        if "built" in v:
            breakdown[k]["built"] = v["built"]
        if "overlapped_builds" in v:
            breakdown[k]["built_on_side_stream"] = v["overlapped_builds"]

    # ---- the other configurations (rank 0, one GPU): voxels/s and the reference CPU beside each -----------
    configs = None
    sub = None
    cpu_ref = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_ref, cpu = cpu_baseline_sample(workloads, args.rooms)
    else:
        cpu = None
    if rank == 0 and world == 1 and not args.no_config1:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # larger than the 126 MB L2

        def ev_each(fn, reps):
            """Mean CUDA-event time of `reps` calls, L2 flushed (a 256 MB write) before each."""
            tot = 0.0
            for _ in range(reps):
                flush.fill_(1)
                a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a_.record()
                fn()
                b_.record()
                torch.cuda.synchronize()
                tot += a_.elapsed_time(b_)
            return tot / reps

        configs = {}
        table = [(1, [0], ("fp32", "tf32x3")), (2, list(range(100)), ("fp32", "tf32x3")),
                 (4, list(range(16)), ("fp32", "tf32x3")), (5, list(range(4)), ("bf16", "tf32x3"))]
        for cfg, samples, modes in table:
            inp_c, net_c, head_c = workloads.build_config(cfg)
            net_c.to(dev)
            if head_c is not None:
                head_c.to(dev)
            c_np, f_np = workloads.make_batch(cfg, samples)
            c_d, f_d = torch.from_numpy(c_np).to(dev), torch.from_numpy(f_np).to(dev)

            def fwd():
                with torch.no_grad():
                    y = net_c(inp_c([c_d, f_d]))
                    return head_c(y.features) if head_c is not None else y

            rec = {"workload": CONFIG_NAMES[cfg], "voxels_per_step": int(c_np.shape[0]),
                   "l2": "flushed before every timed forward"}
            for mode in modes:
                scn.set_precision(mode)
                for _ in range(3):
                    fwd()
                t = ev_each(fwd, max(3, args.steps // 2))
                rec[mode] = {"ms_per_step": round(t, 4), "voxels_per_sec": c_np.shape[0] / (t / 1e3)}
            scn.set_precision(args.precision)
            if cfg == 1:
                # cold = hash + rulebook + convolution (fresh Metadata); warm = cached rulebook; rules only
                with torch.no_grad():
                    x1 = inp_c([c_d, f_d])
                    net_c(x1)
                    t_warm = ev_each(lambda: net_c(x1), 10)

                    def rules_only():
                        x = inp_c([c_d, f_d])
                        SCN.lib.scn_md_submanifold_rulebook(x.metadata._h, SCN.sizes([256] * 3), SCN.sizes([3] * 3),
                                                            SCN._stream(), None)
                    t_rules = ev_each(rules_only, 10)
                n1 = c_np.shape[0]
                t_cold = rec[args.precision if args.precision in rec else "tf32x3"]["ms_per_step"]
                sub = {"workload": CONFIG_NAMES[1], "sites": n1, "precision": args.precision,
                       "cold_sites_per_sec": n1 / (t_cold / 1e3), "warm_sites_per_sec": n1 / (t_warm / 1e3),
                       "hash_and_rulebook_sites_per_sec": n1 / (t_rules / 1e3),
                       "ms": {"cold": t_cold, "warm": t_warm, "hash_and_rulebook": t_rules}}
            if cpu_ref is not None:
                v_cpu, sec_cpu, _ = cpu_ref.time(cfg, samples, 0 if cfg == 5 else 1, 1 if cfg == 5 else 2)
                rec["reference_cpu"] = {"voxels_per_sec": v_cpu, "ms_per_step": 1e3 * sec_cpu, "cores": cpu_ref.cores,
                                        "kind": cpu_ref.kind}
            configs["config%d" % cfg] = rec
            del net_c, c_d, f_d
        del flush

    # ---- the other arithmetic modes on the same workload (resident inputs, fewer steps) ---------
    variants = {args.precision: value}
    if not args.no_variants:
        for mode in ("fp32", "tf32x3", "tf32", "bf16"):
            if mode == args.precision:
                continue
            scn.set_precision(mode)
            for _ in range(3):  # the mode's first steps grow the allocator's pool for its scratch buffers
                job.forward(job.coords_dev, job.feats_dev)
            job.drain()
            ms_v, _ = timed(lambda: job.forward(job.coords_dev, job.feats_dev), max(2, args.steps // 2), drain=job.drain)
            variants[mode] = total_vox * max(2, args.steps // 2) / (ms_v / 1e3)
        scn.set_precision(args.precision)

    # ---- training step of the same network (forward + backward + SGD), two rooms -----------------
    training = None
    if rank == 0 and world == 1 and not args.no_variants:
        inp_t, net_t, head_t = workloads.build_config(CONFIG)
        net_t.to(dev).train()
        head_t.to(dev).train()
        ct_np, ft_np = workloads.make_batch(CONFIG, [0, 1])
        ct, ft = torch.from_numpy(ct_np), torch.from_numpy(ft_np).to(dev)
        params = list(net_t.parameters()) + list(head_t.parameters())
        opt = torch.optim.SGD(params, lr=1e-3)
        labels = torch.randint(0, 20, (ct_np.shape[0],), device=dev, generator=torch.Generator(dev).manual_seed(1))

        def train_step():
            logits = head_t(net_t(inp_t([ct, ft])).features)
            loss = torch.nn.functional.cross_entropy(logits, labels[:logits.size(0)])
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
            return loss

        scn.set_backward_precision(args.precision)  # input gradients on the forward's kernels
        try:
            train_step()
            ms_t, _ = timed(train_step, 3)
        finally:
            scn.set_backward_precision("fp32")
        training = {"workload": workload_name(2), "voxels_per_step": int(ct_np.shape[0]), "ms_per_step": ms_t / 3,
                    "voxels_per_sec": ct_np.shape[0] * 3 / (ms_t / 1e3), "forward": scn.get_precision(),
                    "backward": "input gradients %s, weight gradients fp32" % args.precision, "optimizer": "SGD"}
        del net_t, head_t, params, opt

    # ---- the same training step data-parallel: two rooms per rank, BatchNorm statistics over all ranks, gradients
    # summed over the ranks before the optimizer step (asked for with --data-parallel-training) -------------------
    training_dp = None
    if world > 1 and args.data_parallel_training:
        inp_t, net_t, head_t = workloads.build_config(CONFIG)
        net_t.to(dev).train()
        head_t.to(dev).train()
        shard.share_batchnorm_statistics(net_t)
        ct_np, ft_np = workloads.make_batch(CONFIG, [2 * rank, 2 * rank + 1])
        ct, ft = torch.from_numpy(ct_np), torch.from_numpy(ft_np).to(dev)
        params = list(net_t.parameters()) + list(head_t.parameters())
        opt = torch.optim.SGD(params, lr=1e-3)
        labels = torch.randint(0, 20, (ct_np.shape[0],), device=dev, generator=torch.Generator(dev).manual_seed(1))
        count = torch.tensor([float(ct_np.shape[0])], device=dev)
        dist.all_reduce(count)
        vox_all = int(count.item())
        reduces = [0]

        def train_step_dp():
            logits = head_t(net_t(inp_t([ct, ft])).features)
            loss = torch.nn.functional.cross_entropy(logits, labels[:logits.size(0)], reduction="sum") / vox_all
            opt.zero_grad(set_to_none=True)
            loss.backward()
            reduces[0] = shard.sum_gradients(params)
            opt.step()
            return loss

        scn.set_backward_precision(args.precision)
        try:
            train_step_dp()
            ms_t, _ = timed(train_step_dp, 3)
        finally:
            scn.set_backward_precision("fp32")
        n_bn = sum(1 for m in net_t.modules() if isinstance(m, scn.BatchNormalization))
        training_dp = {"workload": workload_name(2), "voxels_per_step": vox_all, "ms_per_step": ms_t / 3,
                       "voxels_per_sec": vox_all * 3 / (ms_t / 1e3), "scaling": "weak",
                       "exchanges_per_step": "%d all-reduces of BatchNorm sums (forward + backward of %d layers), "
                                             "%d of gradient buckets" % (2 * n_bn, n_bn, reduces[0])}
        del net_t, head_t, params, opt

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": DTYPE_LABEL[args.precision], "data": "synthetic",
            "config": {"workload": workload_name(args.rooms), "voxels_per_step": total_vox,
                       "l2": "inputs and activations (>200 MB per tensor) exceed the 126 MB L2",
                       "precision": scn.get_precision(), "parallelism": "dp%d by batch index" % world,
                       "untimed_steps_after_warmup": len(settle_steps), "their_ms": settle_steps},
            "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(job.coords_host.numel() * 8 + job.feats_host.numel() * 4),
                    "d2h_bytes_per_step": int(n_vox * 20 * 4)},
            "gpu_launches": int(launches), "host_waits_per_step": measure.host_waits_per_step,
            "ms_each_step": per_step, "ms_each_step_e2e": measure.per_step_e2e,
            "roofline": roofline, "breakdown_ms_per_step": breakdown, "submanifold_conv": sub, "configs": configs,
            "variants_voxels_per_sec": variants, "training_step": training,
            "training_step_data_parallel": training_dp,
            "cpu_baseline": cpu, "clocks": clocks,
        }
        if world > 1:
            line["gather_check"] = gather_check
            line["strong_scaling"] = strong
        print(json.dumps(line))
        if args.profile_out:
            with open(args.profile_out, "w") as f:
                json.dump({"breakdown": breakdown, "rows": prof_rows}, f, indent=1)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
