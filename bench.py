#!/usr/bin/env python3
"""Benchmark of the deformable-kernel layer: forward + backward images/s and achieved HBM
bandwidth on the MobileNetV2-style depthwise layer sweep (batch 128 per GPU, fp16 storage,
fp32 arithmetic; five layer shapes x stride 1 and 2, scope 4x4, kernel 3, pad 1).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one forward + backward of all ten layers on one batch, issued through the
public autograd API; it is captured once as a CUDA graph and replayed (--eager launches it
call by call).  Rank 0 prints ONE JSON line.  `value` is device-timed with inputs resident
in HBM; `e2e` is the same step
through the public autograd API with every input copied from pinned host memory and every
result copied back inside the timed region.  The batch is sharded by replication of the
per-GPU batch (weak scaling, no collective: nothing on this path is exchanged between
samples except the bank gradient, which op-level runs do not all-reduce).

--impl reference times the CPU oracle (oracle/dk_oracle.c, OpenMP over all host cores): the
reference project has no CPU implementation of this path, so its restatement stands in.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "deformable-kernels_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

LAYERS = [(c, hw, s) for (c, hw) in [(96, 112), (144, 56), (192, 28), (384, 14), (960, 7)] for s in (1, 2)]
SCOPE, K, PAD = 4, 3, 1
METRIC = "DK layer fwd+bwd images/sec (MobileNetV2 depthwise sweep, batch 128 fp16)"
HBM_NOMINAL_GBS = 8000.0


_RESULT_FD = None


def quiet_stdout():
    """Everything libraries print on stdout while the benchmark runs (NCCL's version banner, for one) goes to stderr, so
    that stdout carries the one JSON line and nothing else."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    sys.stdout.flush()
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        os.write(1, data)
    else:
        os.write(_RESULT_FD, data)


def out_hw(hw, s):
    return (hw + 2 * PAD - K) // s + 1


def layer_bytes(n, c, hw, s, e=2):
    """Algorithmic bytes of one layer, every tensor touched once per pass."""
    ho = out_hw(hw, s)
    x, y, rot, w = n * c * hw * hw, n * c * ho * ho, n * 2 * K * K * ho * ho, c * SCOPE * SCOPE
    fwd = e * (x + rot + y + w)
    bwd = e * (y + x + rot + x + rot + 2 * w)
    return fwd, bwd


def kernel_bytes(name, n, c, hw, s, e=2):
    ho = out_hw(hw, s)
    x, y, rot, w = n * c * hw * hw, n * c * ho * ho, n * 2 * K * K * ho * ho, c * SCOPE * SCOPE
    return e * {"forward": x + rot + y + w, "backward_data": y + rot + w + x, "backward_rotation": y + x + rot + w + rot,
                "backward_filter": y + x + rot + w, "backward_rotation_filter": y + x + rot + w + rot + w}[name]


def measured_traffic(n):
    """DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch of the kernels of the largest layer, from the
    ncu capture summarised under profiles/ (taken at a smaller batch; the traffic of these streaming kernels grows in
    proportion to the batch, so it is scaled to n images).  None when the summary is missing."""
    try:
        rec = json.load(open(os.path.join(ROOT, "profiles", "local_dk_ring_kernels_traffic.json")))
        return {k: v * n / rec["batch"] for k, v in rec["dram_bytes_per_launch"].items()}, rec.get("source")
    except Exception:
        return None, None


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines, self.begin = index, None, [], 0

    def start(self):
        """Starts nvidia-smi looping every 10 ms and waits for its first line, so that it is already sampling when the
        timed region begins (the region of the default run lasts 30 ms)."""
        for period_ms in ("10", "50"):  # a driver that refuses the short period gets the longer one
            try:
                self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                                              "--format=csv,noheader,nounits", "-lms", period_ms], stdout=subprocess.PIPE,
                                             stderr=subprocess.DEVNULL, text=True)
            except OSError:
                self.proc = None
                break
            threading.Thread(target=self._read, args=(self.proc,), daemon=True).start()
            t0 = time.time()
            while not self.lines and time.time() - t0 < 3.0 and self.proc.poll() is None:
                time.sleep(0.005)
            if self.lines:
                break
        self.mark()

    def mark(self):
        """The timed region begins here: earlier samples are only used if the region turns out shorter than a sample."""
        self.begin = len(self.lines)

    def _read(self, proc):
        for line in proc.stdout:
            self.lines.append(line)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.03)
        self.proc.terminate()
        lines, window = self.lines[self.begin:], "timed region"
        if len(lines) < 2:  # shorter than the sampling period: take the samples of the warm-up steps (same load) as well
            lines, window = self.lines[max(0, self.begin - 8):], "warm-up + timed region"
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in lines:
            f = [v.strip() for v in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])), mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


def cpu_sweep(n_img, threads=None):
    """Forward + backward of the ten layers on n_img images with the CPU oracle (fp32 math on
    fp16-rounded inputs).  Returns seconds."""
    from deformable_kernels import synthetic as dk_cases
    from oracle import dk_oracle as O
    if threads:
        O.set_threads(threads)
    total = 0.0
    for (c, hw, s) in LAYERS:
        case = dk_cases.cfg3(c, hw, s, n=n_img, seed=7)
        x, r, w, dy = (case[k].half().float() for k in ("input", "rotation", "weight", "grad_output"))
        t0 = time.perf_counter()
        O.sample_depthwise_forward(x, r, w, **case["args"])
        O.sample_depthwise_backward(dy, x, r, w, **case["args"])
        total += time.perf_counter() - t0
    return total


def other_configs(dev, time_call):
    """BASELINE.json configs 1, 2 and 4 (parity-test cases, not the headline): device-timed forward + backward."""
    from deformable_kernels import synthetic as dk_cases
    from deformable_kernels.modules import GlobalDeformKernel2d
    from deformable_kernels.ops.deform_kernel.functions import deform_sample_depthwise, nd_linear_sample, sample_depthwise
    out = {}

    def fb(fn, ins, dy):
        def run():
            y = fn(*ins)
            torch.autograd.grad(y, ins, dy)
        return run

    def graph_us(run):
        """The same forward + backward captured once into a CUDA graph and replayed: what the launches cost on the device
        when the host's per-call work (Python, autograd bookkeeping) is out of the way.  None if capture fails."""
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(3):
                    run()
            torch.cuda.current_stream(dev).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                run()
            return round(time_call(graph.replay, 50) * 1e3, 1)
        except Exception:
            torch.cuda.synchronize(dev)
            return None

    c1 = dk_cases.cfg1()
    ins = [c1[k].to(dev).requires_grad_(True) for k in ("input", "rotation", "weight")]
    run1 = fb(lambda x, r, w: sample_depthwise(x, r, w, **c1["args"]), ins, c1["grad_output"].to(dev))
    t = time_call(run1, 20)
    out["cfg1 local DK N=2 C=64 28x28 fp32"] = {"fwd_bwd_us": round(t * 1e3, 1), "fwd_bwd_cuda_graph_us": graph_us(run1),
                                                  "algorithmic_MB": 2.36}

    c2 = dk_cases.cfg2()
    ins = [c2[k].to(dev).requires_grad_(True) for k in ("data", "coord")]
    run2 = fb(nd_linear_sample, ins, c2["grad_output"].to(dev))
    t = time_call(run2, 20)
    out["cfg2 nd_linear_sample C=256 2x2, 32 samples fp32"] = {"fwd_bwd_us": round(t * 1e3, 1),
                                                                 "fwd_bwd_cuda_graph_us": graph_us(run2), "algorithmic_MB": 0.079}
    m = GlobalDeformKernel2d((2, 2), 256, 256, kernel_size=1, groups=256).to(dev)
    x2 = c2["input"].to(dev).requires_grad_(True)

    def mod():
        y = m(x2)
        torch.autograd.grad(y.sum(), [x2, m.weight, m.fc.weight])
    t = time_call(mod, 10)
    out["cfg2 GlobalDeformKernel2d module N=32 C=256 14x14 fp32"] = {"fwd_bwd_us": round(t * 1e3, 1),
                                                                       "fwd_bwd_cuda_graph_us": graph_us(mod), "algorithmic_MB": 32.3}

    n4 = 64
    g = torch.Generator(device=dev).manual_seed(4)
    w = (torch.randn(256, 1, 4, 4, device=dev, generator=g) * 0.354).half().requires_grad_(True)
    x = torch.randn(n4, 256, 56, 56, device=dev, generator=g).half().requires_grad_(True)
    rot = (torch.randn(n4, 18, 56, 56, device=dev, generator=g) * 0.5).half().requires_grad_(True)
    off = (torch.randn(n4, 18, 56, 56, device=dev, generator=g) * 2.0).half().requires_grad_(True)
    dy = torch.randn(n4, 256, 56, 56, device=dev, generator=g).half()
    t = time_call(fb(lambda a, o, r, b: deform_sample_depthwise(a, o, r, b), [x, off, rot, w], dy), 3)
    out["cfg4 DK+DCN N=64 C=256 56x56 fp16"] = {"fwd_bwd_ms": round(t, 3), "images_per_s": round(n4 / (t * 1e-3), 1),
                                                  "GBps": round(557.2e6 / (t * 1e-3) / 1e9, 1), "algorithmic_MB": 557.2}
    return out


def build_mobilenet_dk():
    """torchvision's MobileNetV2-1.0 skeleton (random init; the reference ships no model) with each of its 17
    depthwise 3x3 convolutions replaced by DeformKernel2d((4, 4), C, C, 3, stride, 1, groups=C)."""
    import torchvision
    from deformable_kernels.modules import DeformKernel2d
    model = torchvision.models.mobilenet_v2(weights=None)
    replaced = 0
    for mod in model.modules():
        for name, child in list(mod.named_children()):
            if isinstance(child, torch.nn.Conv2d) and child.kernel_size == (3, 3) and child.groups == child.in_channels \
                    and child.groups > 1:
                dk = DeformKernel2d((4, 4), child.in_channels, child.out_channels, 3, child.stride[0], 1, groups=child.groups)
                torch.nn.init.normal_(dk.rotation_conv.weight, std=0.01)
                torch.nn.init.zeros_(dk.rotation_conv.bias)
                setattr(mod, name, dk)
                replaced += 1
    return model, replaced


def run_training_step(args, rank, world, local, dev):
    """BASELINE.json config 5: forward + backward + SGD step of MobileNetV2-DK on synthetic 224x224 images, fp16
    autocast, global batch sharded over the ranks, gradients all-reduced by NCCL through DDP."""
    import torch.distributed as dist
    torch.manual_seed(0)
    model, replaced = build_mobilenet_dk()
    model = model.to(dev).to(memory_format=torch.contiguous_format)
    if world > 1:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local])
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    per_gpu = args.global_batch // world
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(per_gpu, 3, 224, 224, device=dev, generator=gen)
    labels = torch.randint(0, 1000, (per_gpu,), device=dev, generator=gen)
    loss_fn = torch.nn.CrossEntropyLoss()
    scaler = torch.amp.GradScaler("cuda", init_scale=1024.0)
    graphed = bool(args.cuda_graph) and world == 1
    if graphed:
        # forward and backward of the whole network as two CUDA graphs (the operators capture: they enqueue on the
        # current stream, never synchronise and take their scratch from the caller); loss, scaler and optimizer stay eager
        with torch.autocast("cuda", dtype=torch.float16, cache_enabled=False):
            model = torch.cuda.make_graphed_callables(model, (x.clone(),))

    def step():
        opt.zero_grad(set_to_none=not graphed)
        with torch.autocast("cuda", dtype=torch.float16, cache_enabled=not graphed):
            loss = loss_fn(model(x), labels)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        return loss

    for _ in range(max(args.warmup, 3)):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    tms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms_step = float(tms.item()) / args.steps
    share = None
    if not graphed:
        # one more step with CUDA-event ranges around the 17 deformable-kernel operators (the SampleDepthwise modules
        # inside DeformKernel2d): forward range by forward hooks, backward range by the full-backward hooks.  EVERY rank
        # runs this step (its gradient all-reduce is a collective); only rank 0 reports.
        from deformable_kernels.ops.deform_kernel.modules import SampleDepthwise
        ranges, handles = {"fwd": [], "bwd": []}, []

        def opener(kind):
            def hook(*_a):
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                ranges[kind].append([ev, None])
            return hook

        def closer(kind):
            def hook(*_a):
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                for r in reversed(ranges[kind]):
                    if r[1] is None:
                        r[1] = ev
                        break
            return hook
        for mod in model.modules():
            if isinstance(mod, SampleDepthwise):
                handles += [mod.register_forward_pre_hook(opener("fwd")), mod.register_forward_hook(closer("fwd")),
                            mod.register_full_backward_pre_hook(opener("bwd")), mod.register_full_backward_hook(closer("bwd"))]
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        step()
        s1.record()
        torch.cuda.synchronize()
        for h in handles:
            h.remove()
        f_ms = sum(a.elapsed_time(b) for a, b in ranges["fwd"] if b is not None)
        b_ms = sum(a.elapsed_time(b) for a, b in ranges["bwd"] if b is not None)
        share = {"operators": len(ranges["fwd"]), "forward_ms": round(f_ms, 3), "backward_ms": round(b_ms, 3),
                 "step_ms": round(s0.elapsed_time(s1), 3), "share_of_step": round((f_ms + b_ms) / s0.elapsed_time(s1), 4)}
        if world > 1:
            dist.barrier()
    if rank == 0:
        emit(({
            "dk_operator_share": share,
            "metric": "MobileNetV2-DK training step images/sec (global batch %d, fp16 autocast)" % args.global_batch,
            "value": args.global_batch / (ms_step * 1e-3), "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 autocast, f32 master weights", "data": "synthetic",
            "config": {"workload": "cfg5: MobileNetV2-1.0 with %d DeformKernel2d layers (scope 4x4), 224x224, SGD step, "
                                   "DDP/NCCL gradient all-reduce" % replaced, "per_gpu_batch": per_gpu,
                       "cuda_graph": graphed},
            "loss": float(loss.item()), "clocks": clocks, "peak_mem_GB": round(torch.cuda.max_memory_allocated() / 1e9, 1)}))


def run_dcn_layer(args, rank, world, local, dev):
    """BASELINE.json config 4: one DK + DCN layer (C=256, 56x56, 3x3, scope 4x4, fp16), forward + backward through the
    autograd API, each rank on its own batch shard (weak scaling, no collective)."""
    import torch.distributed as dist
    from deformable_kernels.ops.deform_kernel.functions import deform_sample_depthwise
    n = args.dcn_batch
    g = torch.Generator(device=dev).manual_seed(4 + rank)
    w = (torch.randn(256, 1, 4, 4, device=dev, generator=g) * 0.354).half().requires_grad_(True)
    x = torch.randn(n, 256, 56, 56, device=dev, generator=g).half().requires_grad_(True)
    rot = (torch.randn(n, 18, 56, 56, device=dev, generator=g) * 0.5).half().requires_grad_(True)
    off = (torch.randn(n, 18, 56, 56, device=dev, generator=g) * 2.0).half().requires_grad_(True)
    dy = torch.randn(n, 256, 56, 56, device=dev, generator=g).half()
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2

    def step():
        y = deform_sample_depthwise(x, off, rot, w)
        return torch.autograd.grad(y, [x, off, rot, w], dy)

    for _ in range(max(args.warmup, 3)):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    total = 0.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(args.steps):
        flush.zero_()
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    tms = torch.tensor([total], device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms_step = float(tms.item()) / args.steps
    bytes_step = 557.2e6 * n / 64
    peak, peak_kind = measured_peak()
    if rank == 0:
        emit(({
            "metric": "DK+DCN layer fwd+bwd images/sec (C=256, 56x56, fp16)", "value": world * n / (ms_step * 1e-3),
            "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 sums", "data": "synthetic",
            "config": {"workload": "cfg4: DeformableSampleDepthwise C=256 56x56 k3 scope 4x4, batch %d per GPU, offsets "
                                   "~N(0,2^2), kernel offsets ~N(0,0.5^2)" % n,
                       "l2": "a 160 MB buffer is written between timed iterations"},
            "roofline": {"bound": "hbm", "achieved": round(bytes_step / (ms_step * 1e-3) / 1e9, 1), "peak": peak,
                         "peak_source": peak_kind, "unit": "GB/s",
                         "frac": round(bytes_step / (ms_step * 1e-3) / 1e9 / peak, 4), "traffic": None,
                         "algorithmic_bytes": bytes_step, "kernel": "whole layer, forward + backward (6 kernels)"},
            "gpu_launches": 10 * args.steps, "clocks": clocks}))


def time_reference_gpu(layers, n, time_call):
    """The reference's own CUDA kernels (unmodified extension from oracle/_ref/) on the same
    tensors: forward and the three backward launches per layer, device-timed.  A side
    measurement; never part of `value`."""
    try:
        from oracle import build_ref
        fs = build_ref.load_module("filter_sample_depthwise_cuda")
    except Exception as e:
        return {"unavailable": str(e)[:200]}
    out, tot = [], 0.0
    for t in layers:
        tail = (K, K, t["s"], t["s"], PAD, PAD, 1, 1, SCOPE, SCOPE, 1)
        x, rot, dy, w = t["x"].detach().float(), t["rot"].detach().float(), t["dy"].float(), t["w"].detach().float()
        y, gx, gr, gw = torch.empty_like(dy), torch.zeros_like(x), torch.zeros_like(rot), torch.zeros_like(w)
        tf = time_call(lambda: fs.sample_depthwise_forward_cuda(x, rot, w, y, *tail), 3)
        tb = (time_call(lambda: fs.sample_depthwise_backward_data_cuda(dy, x, rot, w, gx, *tail), 3) +
              time_call(lambda: fs.sample_depthwise_backward_rotation_cuda(dy, x, rot, w, gr, *tail), 3) +
              time_call(lambda: fs.sample_depthwise_backward_filter_cuda(dy, x, rot, w, gw, *tail), 3))
        out.append({"C": t["c"], "HW": t["hw"], "stride": t["s"], "fwd_ms": round(tf, 3), "bwd_ms": round(tb, 3)})
        tot += tf + tb
    return {"images_per_s": n / (tot * 1e-3), "ms_per_step": tot, "dtype": "f32 tensors, which is how the reference runs "
            "under Apex (amp.float_function)", "per_layer": out}


def run_reference(args, rank):
    if rank != 0:
        return
    from oracle import dk_oracle as O
    O.set_threads(os.cpu_count() or 1)  # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every host core
    cores = O.max_threads()
    n_img = 16  # about 2 s per step on 16 cores
    for _ in range(args.warmup):
        cpu_sweep(n_img)
    t = [cpu_sweep(n_img) for _ in range(args.steps)]
    sec = sum(t) / len(t)
    val = n_img / sec
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "images/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg3 layer sweep (10 DeformKernel2d layers), %d images per step on host cores" % n_img},
        "cpu_baseline": {"value": val, "unit": "images/s", "cores": cores, "kind": "port",
                         "sample": "%d images through all ten layers per step, OpenMP C restatement of the "
                                   "reference kernels (the reference has no CPU path)" % n_img},
        "e2e": {"value": val, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def bind_host_to_gpu(index):
    """Run this process on the CPUs NVML lists as local to GPU `index`, so that its pinned buffers (placed by first touch)
    and its copies stay on the GPU's side of the host.  Returns the number of CPUs kept, or None when NVML has no answer."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = ((os.cpu_count() or 64) + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (int(w) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=128, help="images per GPU")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true")
    ap.add_argument("--workload", default="sweep", choices=["sweep", "train", "dcn"],
                    help="sweep: the DK layer sweep (headline); train: MobileNetV2-DK training step, global batch 1024; "
                         "dcn: one DK + DCN layer (BASELINE config 4)")
    ap.add_argument("--global-batch", type=int, default=1024)
    ap.add_argument("--cuda-graph", action="store_true",
                    help="train workload, one GPU: run the network's forward and backward as captured CUDA graphs (the sweep replays "
                         "its step as a CUDA graph by default, see --eager)")
    ap.add_argument("--eager", action="store_true",
                    help="sweep: launch every step through the autograd API instead of replaying it as a CUDA graph")
    ap.add_argument("--dcn-batch", type=int, default=64, help="images per GPU of the dcn workload")
    ap.add_argument("--layers", default="", help="comma-separated indices into the ten-layer sweep (default: all)")
    ap.add_argument("--no-ref-gpu", action="store_true",
                    help="do not time the reference's own CUDA kernels (oracle/_ref build, when present) on this GPU")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: --batch images per GPU; strong: --batch images in total, split over the GPUs, the bank "
                         "gradients all-reduced by NCCL once per step")
    ap.add_argument("--sustained-s", type=float, default=3.0,
                    help="seconds of the back-to-back sustained-clock run reported beside the headline (0 = skip)")
    args = ap.parse_args()
    quiet_stdout()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist
    from deformable_kernels.ops.deform_kernel.functions import sample_depthwise
    from deformable_kernels.ops.deform_kernel import filter_sample_depthwise_cuda as fs

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    all_cpus = os.sched_getaffinity(0)
    host_cpus = None if os.environ.get("DK_BENCH_NO_BIND") else bind_host_to_gpu(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # stdout carries the one JSON line only
        dist.init_process_group("nccl", device_id=dev)
    if args.workload in ("train", "dcn"):
        (run_training_step if args.workload == "train" else run_dcn_layer)(args, rank, world, local, dev)
        if world > 1:
            dist.destroy_process_group()
        return

    from deformable_kernels import _cabi as C
    from deformable_kernels.sharding import shard_bounds
    strong = args.scaling == "strong"
    if strong:  # one global batch split into contiguous shards, the bank gradients all-reduced once per step
        lo, hi = shard_bounds(args.batch, rank, world)
        n = hi - lo
        images_per_step = args.batch
    else:
        n = args.batch
        images_per_step = world * n
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    layers = []
    chosen = [LAYERS[int(i)] for i in args.layers.split(",")] if args.layers else LAYERS
    for (c, hw, s) in chosen:
        ho = out_hw(hw, s)
        t = dict(c=c, hw=hw, s=s, ho=ho)
        t["w"] = (torch.randn(c, 1, SCOPE, SCOPE, device=dev, generator=gen) * (2.0 / 16) ** 0.5).half()
        t["x"] = torch.randn(n, c, hw, hw, device=dev, generator=gen).half()
        t["rot"] = torch.randn(n, 2 * K * K, ho, ho, device=dev, generator=gen).half()
        t["dy"] = torch.randn(n, c, ho, ho, device=dev, generator=gen).half()
        layers.append(t)
    if strong and world > 1:  # every rank starts from the same banks
        for t in layers:
            dist.broadcast(t["w"], 0)

    def fwd_bwd(t, x, rot, dy):
        x.requires_grad_(True), rot.requires_grad_(True), t["w"].requires_grad_(True)
        y = sample_depthwise(x, rot, t["w"], (K, K), (t["s"], t["s"]), (PAD, PAD), (1, 1), 1)
        gx, gr, gw = torch.autograd.grad(y, [x, rot, t["w"]], dy)
        return y, gx, gr, gw

    def compute():
        gws = []
        for t in layers:
            gws.append(fwd_bwd(t, t["x"], t["rot"], t["dy"])[3])
        return torch.cat([g.float().flatten() for g in gws]) if strong and world > 1 else None

    graph = None
    if not args.eager:
        # the ten layers' forward + backward captured once (the operators enqueue on the current stream, never synchronise
        # and take their scratch from the caller) and replayed: one host call per step instead of fifty launches through
        # the autograd API, which is what a step of a few hundred microseconds per layer shard is otherwise bound by
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(3):
                compute()
        torch.cuda.current_stream(dev).wait_stream(side)
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                flat_static = compute()
        except Exception as exc:  # no capture on this stack: the step runs eagerly (config.cuda_graph says which)
            sys.stderr.write("CUDA graph capture failed (%s): eager step\n" % exc)
            graph = None
            torch.cuda.synchronize()

    def step():
        if graph is not None:
            graph.replay()
            flat = flat_static
        else:
            flat = compute()
        if flat is not None:  # the only exchange of the path: 0.46 MB of bank gradients, one NCCL all-reduce
            dist.all_reduce(flat)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    tms = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms_step = float(tms.item()) / args.steps
    value = images_per_step / (ms_step * 1e-3)

    # The same step back to back for a few seconds: these kernels are bound by instruction issue, so their time follows the
    # SM clock, and a timed region of a few dozen milliseconds runs at boost clock.  This is the figure at the clock the GPU
    # holds under sustained load, with its own clock record.
    sustained = None
    if args.sustained_s > 0:
        reps = max(args.steps, int(args.sustained_s * 1e3 / max(ms_step, 1e-3)) + 1)
        s2 = ClockSampler(local)
        barrier()
        if rank == 0:
            s2.start()
        e0.record()
        for _ in range(reps):
            step()
        e1.record()
        barrier()
        tms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms_sus = float(tms.item()) / reps
        sustained = {"steps": reps, "ms_per_step": ms_sus, "value": images_per_step / (ms_sus * 1e-3),
                     "clocks": s2.stop() if rank == 0 else None}

    # per-layer forward / backward split and per-kernel times (device events on the launch stream)
    def time_call(fn, iters=5):
        fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters

    def fused_backward(t, dy, x, rot, w, gx, gr, gw):
        """dk_sample_depthwise_backward through the C ABI, as the autograd function calls it (gx = None: the two
        gradients that share the products dy * x only)."""
        geom = C.geom(x.shape, (K, K), (t["s"], t["s"]), (PAD, PAD), (1, 1), (SCOPE, SCOPE), 1)
        nb = C.lib.dk_sample_depthwise_backward_workspace_bytes(geom, C.DK_F16)
        ws = torch.empty(max(nb, 1), dtype=torch.uint8, device=dev)
        stream = C.stream_ptr(dev)

        def run():
            C.check(C.lib.dk_sample_depthwise_backward(C.ptr(dy), C.ptr(x), C.ptr(rot), C.ptr(w), C.ptr(gx), C.ptr(gr),
                                                       C.ptr(gw), geom, C.DK_F16, C.ptr(ws), nb, stream), "backward")
        return run

    per_layer, kern_tot = [], {}
    big = None
    for t in layers:
        tail = (K, K, t["s"], t["s"], PAD, PAD, 1, 1, SCOPE, SCOPE, 1)
        x, rot, dy, w = t["x"].detach(), t["rot"].detach(), t["dy"], t["w"].detach()
        y, gx, gr, gw = torch.empty_like(dy), torch.empty_like(x), torch.empty_like(rot), torch.empty_like(w)
        kt = {
            "forward": time_call(lambda: fs.sample_depthwise_forward_cuda(x, rot, w, y, *tail)),
            "backward_data": time_call(lambda: fs.sample_depthwise_backward_data_cuda(dy, x, rot, w, gx, *tail)),
            "backward_rotation_filter": time_call(fused_backward(t, dy, x, rot, w, None, gr, gw)),
        }
        t_bwd = time_call(fused_backward(t, dy, x, rot, w, gx, gr, gw))  # the call the autograd function makes
        fb, bb = layer_bytes(n, t["c"], t["hw"], t["s"])
        tf = kt["forward"]
        per_layer.append({"C": t["c"], "HW": t["hw"], "stride": t["s"], "fwd_ms": round(tf, 4), "bwd_ms": round(t_bwd, 4),
                          "GBps": round((fb + bb) / ((tf + t_bwd) * 1e-3) / 1e9, 1),
                          "frac": round((fb + bb) / ((tf + t_bwd) * 1e-3) / 1e9 / measured_peak()[0], 4),
                          "bwd_data_ms": round(kt["backward_data"], 4),
                          "bwd_offsets_and_bank_ms": round(kt["backward_rotation_filter"], 4)})
        for k, v in kt.items():
            kern_tot[k] = kern_tot.get(k, 0.0) + v
        if big is None:
            big = (t, kt, t_bwd)
    peak, peak_kind = measured_peak()
    dom = max(kern_tot, key=kern_tot.get)
    bt, bkt, b_bwd = big
    fb, bb = layer_bytes(n, bt["c"], bt["hw"], bt["s"])
    layer_ms = bkt["forward"] + b_bwd
    layer_gbs = (fb + bb) / (layer_ms * 1e-3) / 1e9
    tot_bytes = sum(sum(layer_bytes(n, c, hw, s)) for (c, hw, s) in chosen)
    sweep_gbs = tot_bytes / (ms_step * 1e-3) / 1e9
    traffic, traffic_src = (measured_traffic(n) if (bt["c"], bt["hw"], bt["s"]) == (96, 112, 1) else (None, None))
    per_kernel = {}
    for k, v in bkt.items():
        kb = kernel_bytes(k, n, bt["c"], bt["hw"], bt["s"])
        per_kernel[k] = {"kernel_ms": round(v, 4), "algorithmic_bytes": kb, "achieved": round(kb / (v * 1e-3) / 1e9, 1),
                         "frac": round(kb / (v * 1e-3) / 1e9 / peak, 4),
                         "traffic": traffic.get(k) if traffic else None}
    # `frac` is the whole layer (forward + backward algorithmic bytes over forward + backward time), which is what the
    # 70 % target is defined on; the kernel with the largest time summed over the sweep is reported beside it
    roofline = {"bound": "hbm",
                "kernel": "local DK layer, forward + backward = 3 kernels + the bank-gradient reduction (C=%d, %dx%d, stride %d, "
                          "batch %d)" % (bt["c"], bt["hw"], bt["hw"], bt["s"], n),
                "achieved": round(layer_gbs, 1), "peak": peak, "peak_source": peak_kind, "unit": "GB/s",
                "frac": round(layer_gbs / peak, 4), "frac_of_nominal_8TBs": round(layer_gbs / HBM_NOMINAL_GBS, 4),
                "algorithmic_bytes": fb + bb, "layer_ms": round(layer_ms, 4),
                "traffic": sum(traffic.values()) if traffic else None,
                "traffic_over_algorithmic": round(sum(traffic.values()) / (fb + bb), 3) if traffic else None,
                "traffic_source": traffic_src,
                "dominant_kernel": dict(per_kernel[dom], name=dom),
                "all_kernels_largest_layer": per_kernel,
                "sweep_fwd_bwd_GBps": round(sweep_gbs, 1), "sweep_frac": round(sweep_gbs / peak, 4)}

    # end to end: pinned host inputs -> device, forward + backward, all results -> pinned host
    host = []
    for t in layers:
        h = {k: torch.empty(t[k].shape, dtype=t[k].dtype, pin_memory=True).copy_(t[k]) for k in ("x", "rot", "dy")}
        ho = t["ho"]
        h["y"] = torch.empty(n, t["c"], ho, ho, dtype=torch.float16, pin_memory=True)
        h["gx"] = torch.empty(t["x"].shape, dtype=torch.float16, pin_memory=True)
        h["gr"] = torch.empty(t["rot"].shape, dtype=torch.float16, pin_memory=True)
        h["gw"] = torch.empty(t["w"].shape, dtype=torch.float16, pin_memory=True)
        host.append(h)
    h2d = sum(h[k].numel() * 2 for h in host for k in ("x", "rot", "dy"))
    d2h = sum(h[k].numel() * 2 for h in host for k in ("y", "gx", "gr", "gw"))

    # Three streams so that PCIe carries inputs and results at the same time as the kernels run: copy-in of
    # layer k+1, compute of layer k and copy-out of layer k-1 overlap; everything still happens inside the timed step.
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_cmp = torch.cuda.current_stream(dev)
    dev_in = [{k: torch.empty_like(t[k]) for k in ("x", "rot", "dy")} for t in layers]

    # Schedule of the end-to-end step.  Samples are independent (the bank gradient is a sum over them), so the host
    # feeds each layer in batch chunks of about 64 MB of inputs: results of chunk k flow back while chunk k+1 is on its
    # way in and both PCIe directions stay busy for almost the whole step.  Small layers go first and last so that
    # little of the step has only one direction in use.  The bank gradients of a layer's chunks are summed on the device.
    by_size = sorted(range(len(layers)), key=lambda i: layers[i]["x"].numel())
    order = by_size[0::2] + by_size[1::2][::-1]
    jobs = []
    for i in order:
        t = layers[i]
        per_image = sum(t[k][0].numel() * 2 for k in ("x", "rot", "dy"))
        step_n = max(1, min(n, (64 << 20) // per_image))
        bounds = list(range(0, n, step_n)) + [n]
        gw32 = torch.zeros(t["w"].shape, dtype=torch.float32, device=dev)
        for a0, a1 in zip(bounds[:-1], bounds[1:]):
            jobs.append((t, host[i], dev_in[i], a0, a1, gw32, a0 == 0, a1 == n))

    def e2e_step():
        ready = []
        for t, h, d, a0, a1, _, _, _ in jobs:
            with torch.cuda.stream(s_in):
                for k in ("x", "rot", "dy"):
                    d[k][a0:a1].copy_(h[k][a0:a1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
            ready.append(ev)
        for (t, h, d, a0, a1, gw32, first, last), ev in zip(jobs, ready):
            s_cmp.wait_event(ev)
            y, gx, gr, gw = fwd_bwd(t, d["x"][a0:a1].detach(), d["rot"][a0:a1].detach(), d["dy"][a0:a1])
            if first:
                gw32.copy_(gw)
            else:
                gw32.add_(gw)
            out = [(y.detach(), h["y"][a0:a1]), (gx, h["gx"][a0:a1]), (gr, h["gr"][a0:a1])]
            if last:
                out.append((gw32.half(), h["gw"]))
            done = torch.cuda.Event()
            done.record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for src, dst in out:
                    src.record_stream(s_out)
                    dst.copy_(src, non_blocking=True)
        s_cmp.wait_stream(s_out)
        s_in.wait_stream(s_cmp)
        torch.cuda.synchronize()

    e2e_val = None
    e2e_check = None
    if not args.no_e2e:
        e2e_step()
        # the chunked, streamed step must deliver what the resident step computes (largest layer, every output)
        t, h = layers[0], host[0]
        y, gx, gr, gw = fwd_bwd(t, t["x"], t["rot"], t["dy"])
        torch.cuda.synchronize()
        rel = lambda got, want: float((got.float() - want.float().cpu()).abs().max() / want.float().abs().max())
        e2e_check = {"y": rel(h["y"], y.detach()), "grad_input": rel(h["gx"], gx), "grad_offsets": rel(h["gr"], gr),
                     "grad_bank": rel(h["gw"], gw)}
        if not max(e2e_check.values()) < 2e-3:
            raise SystemExit("end-to-end step disagrees with the resident step: %r" % (e2e_check,))
        del y, gx, gr, gw
        barrier()
        t0 = time.perf_counter()
        e0.record()
        for _ in range(args.e2e_steps):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3)
        tms = torch.tensor([e2e_ms], device=dev)
        if world > 1:
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        e2e_val = images_per_step / (float(tms.item()) / args.e2e_steps * 1e-3)

    ref_gpu = None
    if rank == 0 and world == 1 and not args.no_ref_gpu:
        ref_gpu = time_reference_gpu(layers, n, time_call)
        if "per_layer" in ref_gpu:  # ours / theirs per layer, forward + backward
            for mine, theirs in zip(per_layer, ref_gpu["per_layer"]):
                theirs["speedup"] = round((theirs["fwd_ms"] + theirs["bwd_ms"]) / (mine["fwd_ms"] + mine["bwd_ms"]), 1)
            ref_gpu["speedup"] = round(ref_gpu["ms_per_step"] / sum(m["fwd_ms"] + m["bwd_ms"] for m in per_layer), 1)

    others = None
    if rank == 0 and world == 1 and not args.no_other_configs:
        others = other_configs(dev, time_call)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import dk_oracle as O
        os.sched_setaffinity(0, all_cpus)  # the CPU baseline gets every host core again
        O.set_threads(os.cpu_count() or 1)
        n_img = 96  # about 11 s on 16 cores
        cpu_sweep(1)
        sec = cpu_sweep(n_img)
        cpu = {"value": n_img / sec, "unit": "images/s", "cores": O.max_threads(), "kind": "port",
               "sample": "%d images through all ten layers once (%.1f s), OpenMP C restatement of the reference "
                         "kernels; the reference has no CPU path" % (n_img, sec)}

    if rank == 0:
        # launches of this library per step: ring layers (rows of 112 or 56, rows of 28 at stride 1) run forward,
        # grad-input, the fused offsets + bank pass (+ the reduction of its partial offset gradients when more than 144
        # channels are split into groups) and the bank reduction (or forward, the one-pass backward and the reduction); planes of
        # 14 x 14 outputs and below forward, grad-input, the fused band pass, the reduction of its partial offset
        # gradients when the channels are split into groups (more than 96 channels) and the bank reduction; the others
        # forward, grad-input, grad-offsets (+ the reduction of its partial sums when split), grad-bank + reduction
        def layer_launches(t):
            if t["hw"] in (112, 56) or (t["hw"] == 28 and t["s"] == 1):
                if t["hw"] == 56 and t["s"] == 2 and t["c"] <= 144:
                    return 3
                return 5 if t["c"] > 144 else 4
            if t["ho"] * t["ho"] <= 196:
                return 5 if t["c"] > 96 else 4
            q = (ctypes.c_longlong * 8)()
            geom = C.geom((n, t["c"], t["hw"], t["hw"]), (K, K), (t["s"], t["s"]), (PAD, PAD), (1, 1), (SCOPE, SCOPE), 1)
            split = C.lib.dk_local_plan_query(geom, C.DK_F16, 2, q) == 0 and q[2] > 1
            return 6 if split else 5
        launches = sum(layer_launches(t) for t in layers)
        mhz = clocks.get("sm_mhz") if clocks else None
        line = {
            "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "f16 operands, f32 sums", "data": "synthetic",
            "config": {"workload": "cfg3 layer sweep: DeformKernel2d (C,HW) in (96,112),(144,56),(192,28),(384,14),(960,7)"
                                   " x stride 1,2; scope 4x4, kernel 3, pad 1; offsets ~N(0,1); batch %s" %
                                   (("%d in total, split over the GPUs" % args.batch) if strong else ("%d per GPU" % n)),
                       "cuda_graph": graph is not None,
                       "storage": "f16 tensors; forward and grad-input: resampled kernel rounded to f16 (tensor-core output), "
                                  "exact f16 x f16 products summed in fp32; "
                                  "grad-offsets and grad-bank: products dy * x rounded to f16 (tensor-core operands), "
                                  "fp32 accumulation",
                       "l2": "the sweep touches %.1f GB per step, far above the 126 MB L2, so every layer's tensors "
                             "are evicted between steps" % (tot_bytes / 1e9)},
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "rel_err_vs_resident_step": e2e_check, "host_cpus_local_to_gpu": host_cpus},
            "gpu_launches": args.steps * launches, "clocks": clocks,
            "ms_per_step_x_sm_mhz": round(ms_step * mhz, 1) if mhz else None,
            "sustained": sustained, "per_layer": per_layer,
            "reference_cuda_on_this_gpu": ref_gpu, "other_configs": others,
            "kernel_ms_sum_over_layers": {k: round(v, 4) for k, v in kern_tot.items()},
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
