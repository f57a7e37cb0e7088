"""Benchmark of the submanifold sparse-convolution inference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (BASELINE configuration 3): 3-D submanifold U-Net inference, m=32, reps=2,
planes 32..224, 4096^3 field, batch of 8 synthetic rooms of ~200 k voxels each per GPU, fp32.
One step = one forward over the batch with a FRESH Metadata: input-layer hash build, every
rulebook, every layer, the 20-class linear head and (N > 1) the NCCL gather of the per-voxel
outputs.  `value` = voxels/s with inputs resident in HBM; `e2e` = the same through the public
API from pinned host buffers (host->device copy of coordinates and features, device->host
copy of the scores inside the timed region).  Weak scaling: every rank runs its own 8 rooms.

Also reported on the same line: `submanifold_conv` (BASELINE configuration 1: one 32->32
3-D submanifold convolution, active sites/s cold / warm / rulebook only), `roofline` of the
dominant kernel from CUDA-event timing of every operator call, `cpu_baseline` (the reference's
CPU implementation timed on this box's host cores on a bounded sample) and `clocks`.

`--impl reference` times the reference's own CPU implementation (oracle/_ref, compiled from
the reference sources; the numpy restatement if that is absent) on one room per step.
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
# DRAM bytes per launch of the dominant kernel as a multiple of the algorithmic bytes of that
# launch, from the committed ncu captures (profiles/): k_conv_tma 75 MB against 343 MB per launch
# (4-room case, 18 launches); k_conv_pipe 553 MB against 2.18 GB (32->32) and 768 MB against
# 4.03 GB (64->32) at 8 rooms; k_conv_rows 263 MB against 1.08 GB (32->32, 4 rooms).  The traffic
# grows with the rows, like the algorithmic bytes.
TRAFFIC_RATIO = {"k_conv_tma": 0.22, "k_conv_pipe_mma": 0.22, "k_conv_rows": 0.24, "k_conv_simt": 0.25}


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
    (read-only queries)."""

    def __init__(self, index, period=0.02):
        threading.Thread.__init__(self, daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop_flag = threading.Event()

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            }
            get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self._stop_flag.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = get_reasons(h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
                time.sleep(self.period)
        except Exception as e:  # clocks are evidence, not a dependency
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
    if k == "input_features":
        return (r["rows"] + r["sites"]) * r["planes"] * 4
    return 0.0


def summarize_profile(rows):
    """Per kernel class: time, calls, algorithmic bytes and FLOPs of one step.  Convolution calls
    are split by the kernel that ran them."""
    agg = {}
    for r in rows:
        name = r.get("kernel", r["kind"]) if r["kind"] == "conv" else r["kind"]
        a = agg.setdefault(name, {"ms": 0.0, "calls": 0, "bytes": 0.0, "flops": 0.0})
        a["ms"] += r["ms"]
        a["calls"] += 1
        a["bytes"] += op_bytes(r)
        if r["kind"] == "conv":
            a["flops"] += 2.0 * r["macs"]
    return agg


def run_reference(args, rank):
    """The reference's CPU implementation on the host cores: K steps of one room each."""
    if rank != 0:
        return
    import numpy as np
    import torch
    from oracle import runner
    from sparseconvnet_b200 import workloads
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    be, kind = (runner.RefBackend(), "reference") if runner.reference_available() else (runner.PortBackend(), "port")
    inp, net, head = workloads.build_config(CONFIG)
    rooms = [workloads.batch_config3([s]) for s in range(max(1, min(args.steps + args.warmup, 4)))]

    def step(i):
        c, f = rooms[i % len(rooms)]
        y = runner.run_module(net, runner.run_module(inp, [c, f], be), be)
        runner.run_module(head, y, be)
        return c.shape[0]

    for i in range(args.warmup):
        step(i)
    t0 = time.perf_counter()
    vox = 0
    for i in range(args.steps):
        vox += step(args.warmup + i)
    dt = time.perf_counter() - t0
    v = vox / dt
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(), "sample": "one room (~200k voxels) per step"},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": "one room (~200k voxels) per step, %d steps" % args.steps},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def cpu_baseline_sample():
    """Bounded CPU sample for the default run: the reference CPU build on one room, 1 warm-up +
    3 timed forwards (about 10 s of CPU work)."""
    import torch
    from oracle import runner
    from sparseconvnet_b200 import workloads
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ref = runner.reference_available()
    be, kind = (runner.RefBackend(), "reference") if ref else (runner.PortBackend(), "port")
    inp, net, head = workloads.build_config(CONFIG)
    c, f = workloads.batch_config3([0], target_voxels=200000 if ref else 20000)
    times = []
    for i in range(4 if ref else 2):
        t0 = time.perf_counter()
        y = runner.run_module(net, runner.run_module(inp, [c, f], be), be)
        runner.run_module(head, y, be)
        times.append(time.perf_counter() - t0)
    t = sorted(times[1:])[len(times[1:]) // 2]
    return {"value": c.shape[0] / t, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": "one room of %d voxels, median of %d forwards after 1 warm-up" % (c.shape[0], len(times) - 1)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="tf32x3", choices=["fp32", "tf32x3", "tf32", "bf16"],
                    help="convolution arithmetic of the headline number (tf32x3 and fp32 meet the fp32 parity bar)")
    ap.add_argument("--no-variants", action="store_true", help="skip timing the other arithmetic modes")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    samples = list(range(rank * args.rooms, (rank + 1) * args.rooms))
    coords_np, feats_np = workloads.make_batch(CONFIG, samples)
    coords_host = torch.from_numpy(coords_np).pin_memory()
    feats_host = torch.from_numpy(feats_np).pin_memory()
    coords_dev, feats_dev = coords_host.to(dev), feats_host.to(dev)
    n_vox = coords_np.shape[0]
    out_host = torch.empty(n_vox, 20, dtype=torch.float32).pin_memory()

    def forward(c, f):
        """Returns this rank's per-voxel scores; with N > 1 every rank also receives all ranks'
        rows (one padded all_gather over NCCL)."""
        with torch.no_grad():
            y = head(net(inp([c, f])).features)
            if world > 1:
                # the gather of step i runs beside the kernels of step i+1; its result is taken one
                # step later (and after the last step, inside the timed region: drain_gather)
                pending.append(shard.gather_rows(y, count_group=count_group, async_op=True))
                if len(pending) > 1:
                    pending.pop(0).result()
        return y

    pending = []

    def drain_gather():
        while pending:
            pending.pop(0).result()

    def step_resident():
        return forward(coords_dev, feats_dev)

    # End to end: every step copies its inputs from pinned host memory and its scores back to pinned
    # host memory.  As in a serving loop, the copies run on two copy streams and overlap the
    # neighbouring steps' kernels: the inputs of step i+1 travel while step i computes (two device
    # input buffers), the scores of step i travel while step i+1 computes (two host output buffers).
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    c_buf = [torch.empty_like(coords_dev) for _ in range(2)]
    f_buf = [torch.empty_like(feats_dev) for _ in range(2)]
    out_buf = [out_host, torch.empty_like(out_host).pin_memory()]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_free = [torch.cuda.Event() for _ in range(2)]

    def fetch_inputs(b):
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[b])      # the step that last read this buffer has finished
            c_buf[b].copy_(coords_host, non_blocking=True)
            f_buf[b].copy_(feats_host, non_blocking=True)
            in_ready[b].record(s_in)

    class E2E:
        def begin(self, steps):
            self.i, self.steps = 0, steps
            for b in range(2):
                in_free[b].record(main)
                out_free[b].record(main)
            fetch_inputs(0)

        def step(self):
            b = self.i & 1
            if self.i + 1 < self.steps:
                fetch_inputs(b ^ 1)
            main.wait_event(in_ready[b])
            y = forward(c_buf[b], f_buf[b])
            in_free[b].record(main)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                s_out.wait_event(out_free[b])
                out_buf[b].copy_(y, non_blocking=True)
                out_free[b].record(s_out)
            y.record_stream(s_out)
            self.i += 1
            return y

        def end(self):
            main.wait_stream(s_out)          # the last scores have reached the host inside the timed region

    e2e_loop = E2E()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, begin=None, end=None):
        # a cyclic-GC pass of the interpreter in the middle of a step stalls the launch thread for
        # tens of ms (seen as one 70 ms step among 31 ms ones): collect before, not during
        import gc
        gc.collect()
        gc.disable()
        try:
            return _timed(fn, steps, begin, end)
        finally:
            gc.enable()

    def _timed(fn, steps, begin, end):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = SCN.launch_count()
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
        drain_gather()
        b.record()
        barrier()
        ms = a.elapsed_time(b)
        edges = [a] + marks + [b]
        timed.per_step = [round(edges[i].elapsed_time(edges[i + 1]), 3) for i in range(steps)]
        launches = SCN.launch_count() - l0
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, launches

    scn.set_precision(args.precision)
    for _ in range(args.warmup):
        step_resident()
    sampler = ClockSampler(local)
    sampler.start()
    ms, launches = timed(step_resident, args.steps)
    per_step = timed.per_step
    clocks = sampler.stop()
    for _ in range(2):
        e2e_loop.begin(1)
        e2e_loop.step()
        e2e_loop.end()
    ms_e2e, _ = timed(e2e_loop.step, args.steps, e2e_loop.begin, e2e_loop.end)

    total_vox = n_vox
    if world > 1:
        t = torch.tensor([n_vox], device=dev, dtype=torch.int64)
        dist.all_reduce(t)
        total_vox = int(t.item())
    value = total_vox * args.steps / (ms / 1e3)
    e2e = total_vox * args.steps / (ms_e2e / 1e3)

    # ---- per-operator breakdown (CUDA events around every operator call, one extra step) -------
    with SCN.Profile() as prof:
        step_resident()
    agg = summarize_profile(prof.rows())
    peak, peak_src = peaks()
    top = max(agg, key=lambda k: agg[k]["ms"])
    a = agg[top]
    achieved = a["bytes"] / (a["ms"] / 1e3) / 1e9
    roofline = {"kernel": {"batchnorm": "k_bn_apply", "rules_submanifold": "k_submanifold_rules",
                           "rules_strided": "k_strided_*", "input_hash": "k_insert_input"}.get(top, top),
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": peak_src, "frac_of_nominal_7700": achieved / 7700.0,
                "traffic": (TRAFFIC_RATIO[top] * a["bytes"] / a["calls"]) if top in TRAFFIC_RATIO else None,
                "algorithmic_bytes_per_step": a["bytes"], "launches_per_step": a["calls"], "ms_per_step": a["ms"],
                "tflops": a["flops"] / (a["ms"] / 1e3) / 1e12 if a["flops"] else None}
    if a["flops"]:
        # the same kernel against the tensor pipe: algorithmic FLOPs (2 x rules x Cin x Cout; the
        # three-pass mode issues three times as many) over the dense tf32 peak
        tpeak, tsrc = tensor_peak_tflops()
        roofline["tensor"] = {"achieved": roofline["tflops"], "peak": tpeak, "unit": "TFLOP/s",
                              "frac": roofline["tflops"] / tpeak, "peak_source": tsrc}
    roofline["limiter"] = {
        "k_conv_tma": "shared-memory data pipe (ncu: 77 % busy, tensor pipe 40-46 %), see "
                      "profiles/k_conv_tma_tf32x3_unet3d_4rooms.md",
        "k_conv_pipe_mma": "instruction issue and shared-memory data pipe of small (offset, 128-row) steps, see "
                           "profiles/k_conv_pipe_mma_unet3d_4and8rooms.md",
        "k_conv_rows": "LSU data pipe 75 % busy (fragment loads, weight fragments from L2), warp-level tensor pipe "
                       "43-50 %, see profiles/k_conv_rows_unet3d_4rooms.md"}.get(top)
    breakdown = {k: {"ms": round(v["ms"], 4), "calls": v["calls"],
                     "GBps": round(v["bytes"] / (v["ms"] / 1e3) / 1e9, 1) if v["ms"] > 0 else None}
                 for k, v in sorted(agg.items(), key=lambda kv: -kv[1]["ms"])}

    # ---- configuration 1: one 3-D submanifold convolution 32->32 ------------------------------
    sub = None
    if rank == 0 and not args.no_config1:
        inp1, net1, _ = workloads.build_config(1)
        net1.to(dev)
        c1, f1 = workloads.make_batch(1, [0])
        c1d, f1d = torch.from_numpy(c1).to(dev), torch.from_numpy(f1).to(dev)

        def ev_time(fn, reps):
            torch.cuda.synchronize()
            a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a_.record()
            for _ in range(reps):
                fn()
            b_.record()
            torch.cuda.synchronize()
            return a_.elapsed_time(b_) / reps

        with torch.no_grad():
            def cold():
                return net1(inp1([c1d, f1d]))

            for _ in range(3):
                x1 = inp1([c1d, f1d])
                net1(x1)
            t_cold = ev_time(cold, 10)
            t_warm = ev_time(lambda: net1(x1), 20)

            def rules_only():
                x = inp1([c1d, f1d])
                SCN.lib.scn_md_submanifold_rulebook(x.metadata._h, SCN.sizes([256] * 3), SCN.sizes([3] * 3),
                                                    SCN._stream(), None)
            t_rules = ev_time(rules_only, 10)
        n1 = c1.shape[0]
        sub = {"workload": "config1: SubmanifoldConvolution 3D f3 32->32 fp32, 256^3, batch 1", "sites": n1,
               "cold_sites_per_sec": n1 / (t_cold / 1e3), "warm_sites_per_sec": n1 / (t_warm / 1e3),
               "hash_and_rulebook_sites_per_sec": n1 / (t_rules / 1e3),
               "ms": {"cold": t_cold, "warm": t_warm, "hash_and_rulebook": t_rules}}

    # ---- the other arithmetic modes on the same workload (resident inputs, fewer steps) ---------
    variants = {args.precision: value}
    if not args.no_variants:
        for mode in ("fp32", "tf32x3", "tf32", "bf16"):
            if mode == args.precision:
                continue
            scn.set_precision(mode)
            for _ in range(3):  # the mode's first steps grow the allocator's pool for its scratch buffers
                step_resident()
            ms_v, _ = timed(step_resident, max(2, args.steps // 2))
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

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_sample()

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": {"fp32": "f32", "tf32x3": "f32 (3-pass tf32 split on tcgen05, fp32 accumulate)",
                      "tf32": "tf32", "bf16": "bf16"}[args.precision], "data": "synthetic",
            "config": {"workload": workload_name(args.rooms), "voxels_per_step": total_vox,
                       "l2": "inputs and activations (>200 MB per tensor) exceed the 126 MB L2",
                       "precision": scn.get_precision(), "parallelism": "dp%d by batch index" % world},
            "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(coords_host.numel() * 8 + feats_host.numel() * 4),
                    "d2h_bytes_per_step": int(out_host.numel() * 4)},
            "gpu_launches": int(launches), "ms_each_step": per_step,
            "roofline": roofline, "breakdown_ms_per_step": breakdown, "submanifold_conv": sub,
            "variants_voxels_per_sec": variants, "training_step": training,
            "cpu_baseline": cpu, "clocks": clocks,
        }
        print(json.dumps(line))
        if args.profile_out:
            with open(args.profile_out, "w") as f:
                json.dump({"breakdown": breakdown, "rows": prof.rows()}, f, indent=1)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
