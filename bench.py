#!/usr/bin/env python
"""Benchmark of the batch-norm + ReLU hot path: forward + backward elements/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one fused forward and one fused backward over one batch of synthetic input.
Default workload: the sync-BN configuration of the reference benchmark definition
(global x f32 [2048, 256, 56, 56], sharded by batch over the N GPUs; fixed global batch, so
scaling is "strong").  Prints ONE JSON line on rank 0.  For N > 1 launch under torchrun.

Fields beyond the common contract:
  roofline      dominant kernel (backward, 12 algorithmic bytes/element) against the measured
                HBM copy peak of MEASURED_PEAKS.json (fallback 6650 GB/s)
  roofline_fwd, roofline_step   same for the forward kernel (8 B/el) and the whole step (20 B/el)
  e2e           same metric with inputs in pinned HOST memory: H2D of x, dy and D2H of y, dx inside
                the timed region, through the public host-buffer call of anode_b200.ops
  cpu_baseline  the CPU restatement of the reference's kernel chain (oracle/, OpenMP, all host
                cores) timed on a bounded channel subset of the same workload
  other_workloads  (N=1 only) the remaining single-GPU shapes of the benchmark definition
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BYTES_FWD, BYTES_BWD = 8.0, 12.0     # read x, write y | read x, read dy, write dx

WORKLOADS = {
    # name: global shape, distribution, loc, scale, sharded axis
    "cfg2_stem": dict(shape=(256, 64, 112, 112), dist="normal", loc=0.5, scale=2.0, axis=0),
    "cfg3_syncbn": dict(shape=(2048, 256, 56, 56), dist="normal", loc=0.0, scale=1.0, axis=0),
    "cfg4_unet3d": dict(shape=(4, 32, 128, 128, 128), dist="normal", loc=0.0, scale=1.0, axis=2),
    "cfg5_wide": dict(shape=(1024, 2048, 7, 7), dist="student3", loc=0.0, scale=4.0, axis=0),
}
DEFAULT = "cfg3_syncbn"
# DRAM bytes per element of the default workload's kernels come from the ncu summary under profiles/
# (row "traffic per element" of its counter table: dram__bytes_read.sum + dram__bytes_write.sum per launch
# / elements, captured on a 16-channel case of the same per-channel geometry; the kernels work channel by
# channel, so traffic is proportional to the channel count and is scaled by elements here).
TRAFFIC_SOURCE = "profiles/bn_ring_kernels_cfg3_syncbn.md"


def measured_traffic():
    """{'fwd': bytes/element, 'bwd': bytes/element} of the default workload on one GPU, or {}."""
    import re
    try:
        text = open(os.path.join(ROOT, TRAFFIC_SOURCE)).read()
    except OSError:
        return {}
    m = re.search(r"^\|\s*traffic per element[^|]*\|\s*([0-9.]+)\s*B[^|]*\|\s*([0-9.]+)\s*B", text, flags=re.M)
    return {"fwd": float(m.group(1)), "bwd": float(m.group(2))} if m else {}


SEED = 20240607
BLOCKS = 8        # the global tensor is generated in 8 blocks along the sharded axis, whatever N is


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def local_shape(w, rank, world):
    shape = list(w["shape"])
    assert shape[w["axis"]] % BLOCKS == 0 and BLOCKS % world == 0, "sharded extent must be a multiple of %d" % BLOCKS
    shape[w["axis"]] //= world
    return tuple(shape)


def gen_local(w, rank, world, device):
    """This rank's shard of the seeded global tensor (identical global data for every N)."""
    import torch
    ax = w["axis"]
    bshape = list(w["shape"]); bshape[ax] //= BLOCKS
    per = BLOCKS // world
    xs, dys = [], []
    for b in range(rank * per, (rank + 1) * per):
        g = torch.Generator(device=device); g.manual_seed(SEED + 1000 * b)
        if w["dist"] == "normal":
            x = torch.randn(bshape, device=device, generator=g) * w["scale"] + w["loc"]
        else:   # scale * Student-t(3) = Z / sqrt(chi2_3 / 3)
            z = torch.randn(bshape, device=device, generator=g)
            chi = torch.zeros(bshape, device=device)
            for _ in range(3):
                chi += torch.randn(bshape, device=device, generator=g) ** 2
            x = z * torch.rsqrt(chi / 3.0) * w["scale"]
            del z, chi
        xs.append(x)
        dys.append(torch.randn(bshape, device=device, generator=g))
    x = torch.cat(xs, dim=ax).contiguous() if len(xs) > 1 else xs[0]
    dy = torch.cat(dys, dim=ax).contiguous() if len(dys) > 1 else dys[0]
    c = w["shape"][1]
    g = torch.Generator(device=device); g.manual_seed(SEED - 1)
    gamma = torch.rand(c, device=device, generator=g) + 0.5
    beta = torch.rand(c, device=device, generator=g) * 0.2 - 0.1
    return x, dy, gamma, beta


class ClockSampler:
    """nvidia-smi in the background.  It is started before the warm-up (it needs a few hundred ms to
    produce its first line) and its time-stamped samples are filtered to the timed region."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.p, self.t0, self.t1 = index, None, None, None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "20"],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.p = None

    def begin(self):
        self.t0 = time.time()

    def end(self):
        self.t1 = time.time()

    def stop(self):
        import datetime
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except Exception:
            self.p.kill(); out = ""
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[1]), float(f[2]), [n for n, v in zip(names, f[5:9]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if self.t0 is not None and self.t0 <= r[0] <= self.t1]
        window = "timed region"
        if not inside and rows and self.t0 is not None:
            # region shorter than the sampling period: take the samples closest to it
            mid = 0.5 * (self.t0 + self.t1)
            inside = sorted(rows, key=lambda r: abs(r[0] - mid))[:3]
            window = "3 samples nearest to the timed region (region shorter than the 20 ms sampling period)"
        sm = [r[1] for r in inside]; mx = [r[2] for r in inside]
        reasons = sorted({n for r in inside for n in r[3]})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "window": window, "reasons": reasons}


def cpu_baseline(w, steps=3, warmup=0, seconds_hint=20.0):
    """Times the CPU restatement of the reference's kernel chain on a channel subset, with every
    host core (torchrun pins OMP_NUM_THREADS to 1; undo that before the OpenMP runtime loads)."""
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    import numpy as np
    from oracle import bn_oracle as o
    shape = list(w["shape"])
    c_sub = 16 if shape[1] >= 16 else shape[1]
    per_channel = 1
    for i, s in enumerate(shape):
        if i != 1:
            per_channel *= s
    while c_sub > 1 and c_sub * per_channel > 120e6:
        c_sub //= 2
    shape[1] = c_sub
    rng = np.random.default_rng(SEED)
    x = rng.standard_normal(shape, dtype=np.float32) * np.float32(w["scale"]) + np.float32(w["loc"])
    dy = rng.standard_normal(shape, dtype=np.float32)
    g = rng.uniform(0.5, 1.5, c_sub).astype(np.float32); b = rng.uniform(-0.1, 0.1, c_sub).astype(np.float32)
    rm, rv = np.zeros(c_sub, np.float32), np.ones(c_sub, np.float32)
    times = []
    t_all = time.perf_counter()
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        o.bn_relu_fwd_bwd_f32(x, dy, 1e-5, 0.1, rm, rv, g, b, block_sz=0)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_all > seconds_hint and times:
            break
    mean = sum(times) / len(times)
    return {"value": x.size / mean, "unit": "elements/s", "cores": o.num_threads(), "kind": "port",
            "sample": "%d of %d channels of %s, %d elements per step, mean of %d steps, f32, the 11 passes of the "
                      "reference's kernel chain" % (c_sub, w["shape"][1], "x".join(map(str, w["shape"])), x.size, len(times)),
            "seconds": mean}, times


def run_reference(args, rank):
    """--impl reference: the reference has no CPU batch-norm; its kernel chain restated in C
    (oracle/, OpenMP over all host cores) is timed.  When a GPU is visible the reference's own
    CUDA kernels (oracle/_ref, compiled unmodified) are timed beside it as extra information."""
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    base, times = cpu_baseline(w, steps=args.steps, warmup=args.warmup, seconds_hint=120.0)
    line = {
        "impl": "reference", "metric": "bn_relu_fwd_bwd_elements_per_s", "value": base["value"], "unit": "elements/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup, "ms_per_step": 1e3 * base["seconds"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload + " (CPU: bounded channel subset)", "global_shape": list(w["shape"])},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    try:
        import torch
        from oracle import ref_gpu
        if torch.cuda.is_available() and ref_gpu.available():
            torch.cuda.set_device(0)
            x, dy, _, _ = gen_local(w, 0, 1, torch.device("cuda", 0))
            c = x.shape[1]
            rm = torch.zeros(c, device="cuda"); rv = torch.ones(c, device="cuda")
            ts = []
            for i in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ref_gpu.bn_relu_fwd_bwd(x, dy, 1e-5, 0.1, rm, rv, timing=(e0, e1))
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            ms = min(ts[1:])
            line["ref_gpu_kernels"] = {
                "what": "the reference's own 11 CUDA kernels (oracle/_ref, built for sm_100, block_sz=1024, "
                        "max_block_ct=32*SMs) on this GPU, whole workload on one GPU",
                "ms_per_step": ms, "value": x.numel() / (ms * 1e-3), "unit": "elements/s"}
    except Exception as e:     # extra information only
        line["ref_gpu_kernels"] = {"unavailable": repr(e)[:200]}
    print(json.dumps(line), flush=True)


def time_layer(layer, x, dy, y, dx, steps, warmup, dist, sampler=None):
    """W warm-up steps, then K timed steps bracketed by barrier + synchronize; device time by CUDA
    events on the launching stream; per-kernel events inside.  Returns (total_ms, fwd_ms, bwd_ms)."""
    import torch
    if sampler:
        sampler.start()
    for _ in range(warmup):
        layer.forward(x, out=y); layer.backward(dy, out=dx)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    if sampler:
        sampler.begin()
    for i in range(steps):
        ev[i][0].record()
        layer.forward(x, out=y)
        ev[i][1].record()
        layer.backward(dy, out=dx)
        ev[i][2].record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    if sampler:
        sampler.end()
    clocks = sampler.stop() if sampler else None
    total = ev[0][0].elapsed_time(ev[-1][2])
    fwd = sum(e[0].elapsed_time(e[1]) for e in ev) / steps
    bwd = sum(e[1].elapsed_time(e[2]) for e in ev) / steps
    return total, fwd, bwd, clocks


def parity_check(layer, x, dy, y, dx, dist, device, eps=1e-5):
    """Numerical check of the last timed step against a float64 computation on the same data, over
    all ranks: per-channel sums are taken in float64 on every shard and all-reduced (the G-way result
    must equal the single-device result on the concatenated batch), mean / var / dgamma / dbeta are
    compared on every channel, y and dx element by element on four channels with the closed form
    dx = gamma*r*(dz - sum(dz)/M - xhat*sum(dz*xhat)/M), dz = dy where the forward output is positive.  Tolerance 1e-5 + 1e-4*|want| (channel sums:
    + 1e-4*rms).  Elements whose pre-activation is within 1e-5 of zero are skipped (mask undecidable
    in f32).  Also checks that the statistics are bit-identical on every rank."""
    import torch
    C = x.shape[1]
    ax = [0] + list(range(2, x.dim()))
    bs = [1, -1] + [1] * (x.dim() - 2)
    step = max(1, min(C, int(64e6 // max(1, x.numel() // C))))
    s = torch.zeros(2, C, dtype=torch.float64, device=device)
    for c0 in range(0, C, step):
        xs = x[:, c0:c0 + step].double()
        s[0, c0:c0 + step] = xs.sum(dim=ax); s[1, c0:c0 + step] = (xs * xs).sum(dim=ax)
        del xs
    cnt = torch.tensor([float(x.numel() // C)], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(s); dist.all_reduce(cnt)
    M = float(cnt.item())
    mean = s[0] / M
    # second pass about the global mean (float64 sums of squares of N(0,1) data would do, but this is exact for any input)
    v = torch.zeros(C, dtype=torch.float64, device=device)
    for c0 in range(0, C, step):
        d = x[:, c0:c0 + step].double() - mean[c0:c0 + step].view(bs)
        v[c0:c0 + step] = (d * d).sum(dim=ax)
        del d
    if dist is not None:
        dist.all_reduce(v)
    var = v / M + eps
    r = var.rsqrt()
    g = layer.gamma.double(); b = layer.beta.double()
    t = torch.zeros(2, C, dtype=torch.float64, device=device)
    for c0 in range(0, C, step):
        sl = slice(c0, c0 + step)
        xh = (x[:, sl].double() - mean[sl].view(bs)) * r[sl].view(bs)
        # the mask as the forward pass decided it (y > 0): with millions of elements per channel a few
        # pre-activations are within float32 rounding of zero, and each such element moves the channel
        # sums by |dy|; the forward / backward kernels derive bit-identical masks by construction
        dz = dy[:, sl].double() * (y[:, sl] > 0)
        t[0, sl] = dz.sum(dim=ax); t[1, sl] = (dz * xh).sum(dim=ax)
        del xh, dz
    if dist is not None:
        dist.all_reduce(t)
    worst = {"excess": 0.0, "rel": 0.0, "abs": 0.0}

    def cmp(got, want, extra_atol=0.0, skip=None):
        diff = (got.double() - want).abs()
        if skip is not None:
            diff = diff.masked_fill(skip, 0.0)
        worst["abs"] = max(worst["abs"], float(diff.max()))
        worst["rel"] = max(worst["rel"], float((diff / (want.abs() + 1e-3)).max()))
        worst["excess"] = max(worst["excess"], float((diff - 1e-4 * want.abs() - extra_atol).max()))

    cmp(layer.mean, mean); cmp(layer.var, var)
    cmp(layer.dbeta, t[0], 1e-4 * float(t[0].pow(2).mean().sqrt()))
    cmp(layer.dgamma, t[1], 1e-4 * float(t[1].pow(2).mean().sqrt()))
    chans = sorted({0, C // 3, (2 * C) // 3, C - 1})
    xs = x[:, chans].double(); m4 = mean[chans].view(bs); r4 = r[chans].view(bs); g4 = g[chans].view(bs)
    xh = (xs - m4) * r4
    ybn = xh * g4 + b[chans].view(bs)
    skip = ybn.abs() < 1e-5
    cmp(y[:, chans], ybn.clamp_min(0.0), skip=skip)
    dz = dy[:, chans].double() * (y[:, chans] > 0)
    want_dx = g4 * r4 * (dz - t[0][chans].view(bs) / M - xh * t[1][chans].view(bs) / M)
    cmp(dx[:, chans], want_dx, skip=skip)
    del xs, xh, ybn, dz, want_dx
    e = torch.tensor([worst["excess"], worst["rel"], worst["abs"]], dtype=torch.float64, device=device)
    same = True
    if dist is not None:
        dist.all_reduce(e, op=dist.ReduceOp.MAX)
        world = dist.get_world_size()
        mine = torch.stack([layer.mean, layer.var, layer.dgamma, layer.dbeta]).contiguous()
        allv = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allv, mine)
        same = all(bool((a.view(torch.int32) == allv[0].view(torch.int32)).all()) for a in allv[1:])
    excess, rel, ab = [float(q) for q in e.tolist()]
    return {"ok": bool(excess <= 1e-5 and same), "max_rel": rel, "max_abs": ab, "max_excess_over_1e-4_rel": excess,
            "stats_bit_identical_across_ranks": same, "channels_checked_elementwise": chans,
            "against": "float64 torch computation on the concatenated batch (sums all-reduced over ranks)",
            "tolerance": "1e-5 abs + 1e-4 rel (dgamma/dbeta: + 1e-4 rms)"}


def make_layer(ops, channels, world, gamma, beta):
    if world == 1:
        layer = ops.FusedBatchNormRelu(channels, epsilon=1e-5, avg_rate=0.1, affine=True, relu=True)
    else:
        layer = ops.SyncBatchNormRelu(channels, epsilon=1e-5, avg_rate=0.1, affine=True, relu=True,
                                      exchange=os.environ.get("ANODE_BENCH_NCCL_EXCHANGE", "0") != "1")
    layer.gamma.copy_(gamma); layer.beta.copy_(beta)
    return layer


def bench_workload(ops, name, rank, world, steps, warmup, dist, device, sample_clocks, with_e2e, check_parity=True):
    import torch
    w = WORKLOADS[name]
    x, dy, gamma, beta = gen_local(w, rank, world, device)
    y = torch.empty_like(x); dx = torch.empty_like(x)
    layer = make_layer(ops, x.shape[1], world, gamma, beta)
    sampler = ClockSampler(device.index) if (sample_clocks and rank == 0) else None
    total, fwd, bwd, clocks = time_layer(layer, x, dy, y, dx, steps, warmup, dist, sampler)
    status = layer.status()
    t = torch.tensor([total, fwd, bwd, float(status)], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total, fwd, bwd, status = [float(v) for v in t.tolist()]
    if status != 0:
        raise RuntimeError("device status word %d after the timed region" % int(status))
    parity = parity_check(layer, x, dy, y, dx, dist, device) if check_parity else None
    n_local = x.numel()
    n_global = n_local * world
    ms = total / steps
    res = {"ms_per_step": ms, "fwd_ms": fwd, "bwd_ms": bwd, "elements_local": n_local, "elements_global": n_global,
           "value": n_global / (ms * 1e-3), "clocks": clocks, "launches_per_step": layer.launches_per_step, "parity": parity}
    if with_e2e:
        res["e2e"] = bench_e2e(ops, layer, x, dy, y, dx, dist, device, min(steps, 3))     # first: it compares with y, dx of the timed steps
        res["infer"] = bench_infer(layer, x, y, steps, warmup)
        if world == 1:
            res["residual_block"] = bench_residual(ops, layer, x, dy, y, dx, steps, warmup)
    return res


def bench_residual(ops, layer, x, dy, y, dx, steps, warmup):
    """Residual-block epilogue y = relu(bn(x) + shortcut), forward + backward:
    12 + 20 algorithmic bytes per element (x, shortcut -> y; x, dy, y -> dx, dshortcut)."""
    import torch
    res = torch.randn_like(x)
    dres = torch.empty_like(x)
    axes = list(range(x.dim() - 2))
    ws = ops.Workspace(*ops.dims_of(x), x.device)

    def step():
        ops.BatchNormalize2dAddActFusedOp.apply(axes, layer.epsilon, layer.avg_rate, x, res, y, layer.mean, layer.var,
                                                layer.avg_mean, layer.avg_var, layer.gamma, layer.beta, 0.0, ws)
        ops.BatchNormalize2dAddActFusedOp.adjoint(axes, dy, x, y, layer.mean, layer.var, dx, dres, layer.gamma, layer.beta,
                                                  layer.dgamma, layer.dbeta, 0.0, workspace=ws)
    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    k = max(5, steps // 3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(k):
        step()
    e1.record()
    torch.cuda.synchronize()
    assert ws.status() == 0
    ms = e0.elapsed_time(e1) / k
    peak, kind = hbm_peak()
    gbs = 32.0 * x.numel() / (ms * 1e-3) / 1e9
    del res, dres
    from anode_b200 import _lib
    names = {1: "bn_ring_kernel", 2: "bn_segres_kernel", 3: "bn_resident_kernel", 4: "bn_pipeline_kernel"}
    d0, c, n = ops.dims_of(x)
    kk = [names.get(_lib.load().anode_gpu_batch_norm_add_act_fused_kernel_kind(d0, c, n, d), "?") for d in (0, 1)]
    return {"kernel": "%s (forward), %s (backward), residual epilogue" % tuple(kk), "ms_per_step": ms,
            "elements_per_s": x.numel() / (ms * 1e-3), "achieved_gbs": gbs, "frac_of_hbm_peak": gbs / peak, "peak_kind": kind}


def bench_infer(layer, x, y, steps, warmup):
    """Evaluation-mode pass (running statistics + ReLU in one kernel): 8 bytes per element."""
    import torch
    for _ in range(max(warmup, 3)):
        layer.infer(x, out=y)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        layer.infer(x, out=y)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    peak, kind = hbm_peak()
    gbs = 8.0 * x.numel() / (ms * 1e-3) / 1e9
    return {"kernel": "bn_infer_kernel", "ms": ms, "elements_per_s": x.numel() / (ms * 1e-3), "achieved_gbs": gbs,
            "frac_of_hbm_peak": gbs / peak, "peak_kind": kind}


class near_gpu:
    """Runs the enclosed allocations on the CPUs of the GPU's own NUMA node, so that page-locked host
    buffers land in the memory next to the GPU's PCIe root (first touch); the previous CPU affinity is
    restored afterwards.  Does nothing where the topology cannot be read."""

    def __init__(self, device_index):
        self.index, self.saved, self.node = device_index, None, None

    def __enter__(self):
        try:
            out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                                 capture_output=True, text=True, timeout=20).stdout.strip()
            bus = out.lower()
            if bus.startswith("00000000:"):
                bus = bus[4:]                        # sysfs uses a 4-digit domain
            node = int(open("/sys/bus/pci/devices/%s/numa_node" % bus).read().strip())
            if node < 0:
                return self
            cpus = set()
            for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            allowed = os.sched_getaffinity(0)
            if cpus & allowed:
                self.saved = allowed
                os.sched_setaffinity(0, cpus & allowed)
                self.node = node
        except Exception:
            pass
        return self

    def __exit__(self, *exc):
        if self.saved is not None:
            os.sched_setaffinity(0, self.saved)
        return False


def bench_e2e(ops, layer, x, dy, y, dx, dist, device, steps):
    """Same metric through the host-buffer call: pinned host x, dy in; y, dx back out."""
    import torch
    with near_gpu(device.index) as place:
        hx = torch.empty(x.shape, dtype=torch.float32, pin_memory=True); hx.copy_(x)
        hdy = torch.empty(x.shape, dtype=torch.float32, pin_memory=True); hdy.copy_(dy)
        hy = torch.empty(x.shape, dtype=torch.float32, pin_memory=True); hy.zero_()
        hdx = torch.empty(x.shape, dtype=torch.float32, pin_memory=True); hdx.zero_()
    chunk = int(os.environ.get("ANODE_BENCH_E2E_CHUNK", "0"))      # channels per block; 0: the library's choice
    blocks = layer.step_from_host(hx, hdy, hy, hdx, chunk)      # warm-up
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        layer.step_from_host(hx, hdy, hy, hdx, chunk)
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    if layer.host_step_status() != 0:
        raise RuntimeError("device status word %d after the host-buffer steps" % layer.host_step_status())
    # the host-buffer call must give what the device-resident call gave (same data, same layer)
    same = float(((hy.to(device) - y).abs() - 1e-4 * y.abs()).max()) <= 1e-5 and float(((hdx.to(device) - dx).abs() - 1e-4 * dx.abs()).max()) <= 1e-5
    ms = torch.tensor([e0.elapsed_time(e1) / steps, 0.0 if same else 1.0], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms, differs = [float(v) for v in ms.tolist()]
    if differs:
        raise RuntimeError("the host-buffer step and the device-resident step disagree")
    world = dist.get_world_size() if dist is not None else 1
    nbytes = x.numel() * 4
    return {"value": x.numel() * world / (ms * 1e-3), "unit": "elements/s", "ms_per_step": ms, "steps": steps,
            "h2d_bytes_per_step": 2 * nbytes, "d2h_bytes_per_step": 2 * nbytes,
            "channel_blocks": blocks, "gpu_launches_per_step": 2 * blocks, "matches_device_result": True,
            "host_buffers": "page-locked, allocated on the GPU's NUMA node %s" % place.node if place.node is not None else "page-locked",
            "how": ("one C-ABI call per step on pinned host tensors; channel blocks, copies in both directions "
                    "overlapped with the kernels") if world == 1 else
                   ("one C-ABI call per rank and step on pinned host tensors (anode_gpu_sync_batch_norm_relu_step_host_3d1_packed_f32): "
                    "channel blocks, copies in both directions overlapped with the synchronized kernels")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--shape", default=None, help="custom global shape N,C,spatial... (N(0,1) data, sharded on axis 0); "
                    "used for small profiler captures")
    ap.add_argument("--no-extras", action="store_true", help="skip cpu_baseline, e2e and other_workloads")
    ap.add_argument("--kernel", default="auto", choices=["auto", "tiled", "cluster", "resident", "plain"],
                    help="kernel preference of the fused calls (anode_gpu_batch_norm_fused_set_kernel); for profiler captures")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.shape:
        WORKLOADS["custom"] = dict(shape=tuple(int(v) for v in args.shape.split(",")), dist="normal", loc=0.0, scale=1.0, axis=0)
        args.workload = "custom"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as tdist
    from anode_b200 import ops            # raises if the CUDA library is not built
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch with torchrun --nproc-per-node %d" % (args.gpus, world, args.gpus))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        tdist.init_process_group("nccl", device_id=device)
        dist = tdist

    ops.set_kernel(args.kernel)
    main_res = bench_workload(ops, args.workload, rank, world, args.steps, args.warmup, dist, device,
                              sample_clocks=True, with_e2e=not args.no_extras)
    peak, peak_kind = hbm_peak()

    def roof(bytes_per_el, ms):
        ach = bytes_per_el * main_res["elements_local"] / (ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                "peak_kind": peak_kind, "traffic": None}

    w = WORKLOADS[args.workload]
    def kernel_name(direction):
        if main_res["launches_per_step"] != 2:
            return "reduce kernel + all-gather + merge kernel + apply kernel (%s)" % direction
        from anode_b200 import _lib
        shp = local_shape(w, rank, world)
        d0 = 1
        for v in shp[2:]:
            d0 *= int(v)
        c, n = int(shp[1]), int(shp[0])
        kind = _lib.load().anode_gpu_batch_norm_fused_kernel_kind(d0, c, n, 0 if direction == "fwd" else 1)
        return {3: "bn_resident_kernel<%s> (fused reduce+apply, slices resident in shared memory)",
                1: "bn_ring_kernel<%s> (fused reduce+apply, tiled)", 2: "bn_segres_kernel<%s> (fused reduce+apply, clusters)",
                4: "bn_pipeline_kernel<%s> (fused reduce+apply, plain)"}.get(kind, "?%s") % direction
    line = {
        "metric": "bn_relu_fwd_bwd_elements_per_s", "value": main_res["value"], "unit": "elements/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_res["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "global_shape": list(w["shape"]), "local_shape": list(local_shape(w, rank, world)),
                   "sharded_axis": w["axis"], "layout": "NCHW f32, eps=1e-5, avg_rate=0.1, gamma/beta, ReLU",
                   "l2": "inputs larger than L2 (no flush needed)" if main_res["elements_local"] * 4 > 512e6 else "inputs near L2 size",
                   "parallelism": "syncbn_dp%d" % world,
                   "exchange": "none" if world == 1 else ("in-kernel peer stores" if main_res["launches_per_step"] == 2 else "nccl all-gather")},
        "per_gpu_value": main_res["value"] / world,
        "fwd_ms": main_res["fwd_ms"], "bwd_ms": main_res["bwd_ms"],
        "roofline": dict(roof(BYTES_BWD, main_res["bwd_ms"]), kernel=kernel_name("bwd")),
        "roofline_fwd": dict(roof(BYTES_FWD, main_res["fwd_ms"]), kernel=kernel_name("fwd")),
        "roofline_step": roof(BYTES_FWD + BYTES_BWD, main_res["ms_per_step"]),
        "clocks": main_res["clocks"],
        "gpu_launches": main_res["launches_per_step"] * args.steps,
    }
    line["parity"] = main_res["parity"]
    if "e2e" in main_res:
        line["e2e"] = main_res["e2e"]
    if "infer" in main_res:
        line["infer"] = main_res["infer"]
    if "residual_block" in main_res:
        line["residual_block"] = main_res["residual_block"]
    tr = measured_traffic() if (world == 1 and args.workload == DEFAULT and args.kernel == "auto") else {}
    for key, rk in (("bwd", "roofline"), ("fwd", "roofline_fwd")):
        if key in tr:
            line[rk]["traffic"] = tr[key] * main_res["elements_local"]
            line[rk]["traffic_source"] = TRAFFIC_SOURCE + " (16-channel capture, scaled by elements)"

    if world == 1 and not args.no_extras:
        others = {}
        for name in sorted(WORKLOADS):
            if name == args.workload:
                continue
            torch.cuda.empty_cache()
            r = bench_workload(ops, name, 0, 1, max(5, args.steps // 2), 3, None, device, False, False)
            others[name] = {"value": r["value"], "ms_per_step": r["ms_per_step"], "fwd_ms": r["fwd_ms"], "bwd_ms": r["bwd_ms"],
                            "step_frac_of_hbm_peak": 20.0 * r["elements_local"] / (r["ms_per_step"] * 1e-3) / 1e9 / peak,
                            "parity_ok": r["parity"]["ok"], "parity_max_rel": r["parity"]["max_rel"]}
        line["other_workloads"] = others
        if rank == 0:
            torch.cuda.empty_cache()
            line["cpu_baseline"], _ = cpu_baseline(w)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    bad = [n for n, p in [(args.workload, line["parity"])] + [(n, {"ok": o["parity_ok"]}) for n, o in line.get("other_workloads", {}).items()]
           if p is not None and not p["ok"]]
    if bad:
        raise SystemExit("parity check failed on: %s" % ", ".join(bad))


if __name__ == "__main__":
    main()
