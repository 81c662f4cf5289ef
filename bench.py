#!/usr/bin/env python
"""KDA forward+backward throughput on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1|c2|c3]

One "step" = one forward + backward of ``chunk_kda`` over one batch of seeded synthetic
input (default: B=16, T=2048, H=6, d=128, BF16 operands, FP32 state, final state returned,
upstream gradient do ~ N(0,1)).  With N > 1 (torchrun, one rank per GPU) every rank runs the
same per-GPU batch on its own data -- sequences are independent, so there is no collective
on the kernel path -- and the reported value is all ranks' tokens / the slowest rank's time
(``scaling: weak``).  The same line also carries, as extra legs timed after the headline one:
``strong`` (N > 1): the ONE batch of the workload split over the ranks by sequence
(``openkimi_b200.partition.shard_batch``), and ``sublayer``: the whole KimiDeltaAttention
sublayer with its global batch of 64 split over the ranks.

The CPU arm (``--impl reference`` and the ``cpu_baseline`` object) times the oracle port on the
host cores on one head of one full-length sequence of the workload per step.

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, T, H, d, x_mean, a_lo, a_hi, beta_mean, n_docs)
    "c1": dict(B=16, T=2048, H=6, d=128, x_mean=0.0, a_lo=1.0, a_hi=16.0, beta_mean=0.0, docs=0,
               label="kda_fwd_bwd B=16 T=2048 H=6 d=128 bf16 chunk=64 (primary profile)"),
    "c2": dict(B=4, T=4096, H=6, d=128, x_mean=3.0, a_lo=8.0, a_hi=64.0, beta_mean=2.0, docs=0,
               label="kda_fwd_bwd B=4 T=4096 H=6 d=128 bf16 adversarial gate span"),
    "c3": dict(B=1, T=65536, H=6, d=128, x_mean=0.0, a_lo=1.0, a_hi=16.0, beta_mean=0.0, docs=16,
               label="kda_fwd_bwd packed T=65536 16 docs H=6 d=128 bf16 cu_seqlens"),
    # whole KimiDeltaAttention sublayer (projections, short conv, KDA, gated norm, o-proj), width 768;
    # the global batch of 64 is split over the ranks (strong scaling)
    "c4": dict(B=64, T=2048, H=6, d=128, x_mean=0.0, a_lo=1.0, a_hi=16.0, beta_mean=0.0, docs=0, sublayer=True,
               label="kda_sublayer_fwd_bwd global B=64 T=2048 width=768 H=6 d=128 bf16"),
}
METRIC = "kda_fwd_bwd_throughput"
UNIT = "Mtok/s"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback")


def stage_model(name, d, C=64, es=2):
    """Algorithmic FLOPs and HBM bytes of one (chunk, head) unit of each kernel (dense tiles,
    every tensor touched once; es = bytes per element of the BF16 records)."""
    t = C * d * es          # one [64, d] tile
    a = C * C * es          # one [64, 64] tile
    s = d * d * es          # one state
    f4 = C * d * 4          # one FP32 [64, d] tile
    a4 = C * C * 4          # one FP32 [64, 64] tile
    m = {
        # reads q, k, v, g, beta; writes W, U, Qt, Kh, Aqk, T, gamC and the kept prologue (G, q^, k^, norms, beta)
        "fwd_intra": (8 * C * C * d + 2 * C ** 3 // 3, (4 * t + C * es) + (4 * t + 2 * a + 4 * d) + (f4 + 2 * t + 3 * C * 4)),
        # reads W, U, Qt, Kh, Aqk, gamC; writes V', o, the chunk-entry state
        "fwd_state": (6 * C * d * d + 2 * C * C * d, (4 * t + a + 4 * d) + (2 * t + s)),
        # reads W, Qt, Kh, Aqk, gamC, dO; writes dV', the chunk-entry dS
        "bwd_state": (6 * C * d * d + 2 * C * C * d, (4 * t + a + 4 * d) + (t + s)),
        # fused FP32-math backward (validation mode only)
        "bwd_chunk": (6 * C * d * d + 16 * C * C * d + 4 * C ** 3, (5 * t + C * es) + 2 * t + 2 * s + a + (4 * t + C * es)),
        # dAqk, dWn, dQt, dKh (K=d), dVb, dKb, Z, dMn; reads dO, v, V', dV', S0, dS, T, W; writes dv and the
        # hand-over (dAqk, dM as three BF16 operand tiles each + the diagonal of dAqk; dQt, dKh, dKb in BF16)
        "bwd_wy": (10 * C * d * d + 8 * C * C * d, (2 * t) + 3 * t + 2 * s + a + (t + 6 * a + C * 4 + 3 * t)),
        # three pairwise products over the lower triangle (dense-tile count 6 C^2 d; the six BF16 passes of the
        # split operands are not counted); reads the kept prologue and the hand-over; writes dq, dk, dg, dbeta
        "bwd_intra": (6 * C * C * d, (f4 + 2 * t + 3 * C * 4) + (6 * a + C * 4) + 3 * t + (3 * t + C * es)),
        "param_reduce": (0, 4 * d + 4),
    }
    return m[name]


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.gpu)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = [r.split(",") for r in open(self.path).read().strip().splitlines() if r.count(",") >= 8]
        os.unlink(self.path)
        if not rows:
            return out
        clk = [float(r[1]) for r in rows]
        out["sm_mhz"] = statistics.median(clk)
        out["sm_max_mhz"] = float(rows[0][2])
        out["power_w_max"] = max(float(r[3]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        out["reasons"] = [n for i, n in enumerate(names) if any(r[5 + i].strip() == "Active" for r in rows)]
        out["samples"] = len(rows)
        return out


def make_workload(w, seed, device=None, pin=False):
    from openkimi_b200.synthetic import make_inputs, random_cu_seqlens
    inp = make_inputs(w["B"], w["T"], w["H"], w["d"], seed=seed, dtype=torch.bfloat16, x_mean=w["x_mean"],
                      a_lo=w["a_lo"], a_hi=w["a_hi"], beta_mean=w["beta_mean"])
    cu = h0 = None
    if w["docs"]:
        cu = random_cu_seqlens(w["T"], w["docs"], seed=seed)
        h0 = torch.randn(w["docs"], w["H"], w["d"], w["d"], generator=torch.Generator().manual_seed(seed + 1)) * 0.02
    host = dict(inp, cu=cu, h0=h0)
    if pin:
        host = {k: (v.pin_memory() if isinstance(v, torch.Tensor) else v) for k, v in host.items()}
    return host


def step_device(dev_in, w):
    """One forward + backward through the public op with inputs already on the device."""
    from openkimi_b200 import chunk_kda
    leaves = [dev_in[n].requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "a_log", "dt_bias")]
    for t in leaves:
        t.grad = None
    h0 = dev_in.get("h0")
    if h0 is not None:
        h0.requires_grad_(True)
        h0.grad = None
    o, ht = chunk_kda(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], A_log=leaves[5], dt_bias=leaves[6],
                      scale=w["d"] ** -0.5, initial_state=h0, output_final_state=True, use_qk_l2norm_in_kernel=True,
                      use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True, cu_seqlens=dev_in.get("cu"),
                      cu_seqlens_cpu=dev_in.get("cu_cpu"), state_v_first=True, disable_recompute=True)
    o.backward(dev_in["do"])
    return o, ht, leaves, h0


def make_sublayer(w, device, seed=0):
    """KimiDeltaAttention (k3mini/model.py:132-227) with random-init weights N(0, 0.02), A_log and
    dt_bias as the reference initialises them, norm weight 1."""
    from openkimi_b200 import KimiDeltaAttention
    torch.manual_seed(seed)
    m = KimiDeltaAttention(w["H"] * w["d"], w["H"], w["d"], conv_kernel=4, disable_recompute=True)
    with torch.no_grad():
        for name, prm in m.named_parameters():
            if name.endswith("proj.weight") or "out_gate" in name or name.endswith("conv.weight"):
                prm.normal_(0.0, 0.02)
    return m.to(device)


def step_sublayer(model, x, dout):
    for prm in model.parameters():
        prm.grad = None
    x.grad = None
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = model(x)
    out.backward(dout)
    return out


def to_device(host, device):
    dev = {k: v.to(device, non_blocking=True) for k, v in host.items() if isinstance(v, torch.Tensor)}
    if host.get("cu") is not None:
        dev["cu_cpu"] = host["cu"]
    return dev


def cpu_slice_inputs(w, seed=0):
    """One head of one full-length sequence of the workload ([1, T, 1, d], capped at 2048 tokens)."""
    from oracle.kda_oracle import make_inputs
    T = min(w["T"], 2048)
    inp = make_inputs(1, T, 1, w["d"], seed=seed, dtype=torch.bfloat16, x_mean=w["x_mean"], a_lo=w["a_lo"],
                      a_hi=w["a_hi"], beta_mean=w["beta_mean"])
    return inp, T


def cpu_slice_seconds(w, inp):
    """Seconds of the CPU oracle (PyTorch port of k3mini/model.py:101-129 + prologue :217-223), forward +
    autograd backward, on the prepared slice."""
    from oracle.kda_oracle import kda_oracle_fwd_bwd
    t0 = time.perf_counter()
    kda_oracle_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["do"], a_log=inp["a_log"],
                       dt_bias=inp["dt_bias"], scale=w["d"] ** -0.5)
    return time.perf_counter() - t0


def cpu_sample_text(w, T):
    return (f"each step = oracle fwd+bwd of one head of one full-length sequence, a [1,{T},1,{w['d']}] slice "
            f"(1/{w['H']} of the per-token work, counted as {T}/{w['H']} tokens); sequences and heads are independent")


def run_reference(args, w, rank, world):
    """The reference's CPU implementation of the path (the oracle port; the reference is Python
    and cannot travel to the GPU box) on the host cores."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    inp, T = cpu_slice_inputs(w)
    for _ in range(args.warmup):
        cpu_slice_seconds(w, inp)
    secs = sum(cpu_slice_seconds(w, inp) for _ in range(args.steps))
    val = args.steps * (T / w["H"]) / secs / 1e6
    sample = cpu_sample_text(w, T)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["label"], "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def bind_to_gpu_numa_node(gpu_index):
    """Pin this process to the CPUs NVML lists as local to the GPU (read-only query), so that the pinned
    host buffers allocated afterwards are first touched on that NUMA node.  Returns the CPU list or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = [64 * i + b for i, wd in enumerate(mask) for b in range(64) if (wd >> b) & 1]
        cpus = [c for c in cpus if c in os.sched_getaffinity(0)]
        if cpus:
            os.sched_setaffinity(0, cpus)
        return cpus or None
    except Exception:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra-legs", action="store_true", help="skip the strong-scaling and sublayer legs")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch size (profiling cases)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="profiling case: device-resident steps only (no end-to-end leg, no CPU baseline)")
    args = ap.parse_args()
    if args.impl == "ours" and not args.kernel_only:
        args.warmup = max(args.warmup, 3)
    w = dict(WORKLOADS[args.workload])
    if args.batch:
        w["B"] = args.batch
        w["label"] += f" [batch overridden to {args.batch}]"

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return

    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback")
    numa_cpus = bind_to_gpu_numa_node(local)  # before any pinned allocation: first touch on the GPU's node
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    from openkimi_b200 import _lib
    lib = _lib.load()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sub = bool(w.get("sublayer"))
    if sub:  # strong scaling: the global batch is split over the ranks
        w["B"] = max(1, w["B"] // world)
        gen = torch.Generator().manual_seed(100 + rank)
        width = w["H"] * w["d"]
        host = {"x": torch.randn(w["B"], w["T"], width, generator=gen).bfloat16().pin_memory(),
                "dout": torch.randn(w["B"], w["T"], width, generator=gen).bfloat16().pin_memory()}
        model = make_sublayer(w, device)
        dev_x = {k: v.to(device) for k, v in host.items()}
        dev_x["x"].requires_grad_(True)
        step_device_any = lambda: step_sublayer(model, dev_x["x"], dev_x["dout"])
    else:
        host = make_workload(w, seed=rank, pin=True)
        dev_in = to_device(host, device)
        step_device_any = lambda: step_device(dev_in, w)
    tokens = w["B"] * w["T"]
    units = None

    # ---- device-resident timing -------------------------------------------------------
    for _ in range(args.warmup):
        step_device_any()
    barrier()
    n_calls = 2 * args.steps
    lib.kda_profile_begin(n_calls)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # keep the GPU under the same load while the sampler comes up, so that its samples (20 ms
    # apart) cover loaded clocks even when the timed region itself lasts only tens of ms
    t_end = time.perf_counter() + 0.4
    while time.perf_counter() < t_end:
        step_device_any()
        torch.cuda.synchronize()
    lib.kda_profile_begin(n_calls)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step_device_any()
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1)
    # per-kernel durations from the events recorded inside the timed region
    names = {0: ["fwd_intra", "fwd_state"], 1: ["bwd_state", "bwd_chunk", "param_reduce"]}
    names_split = ["bwd_state", "bwd_wy", "bwd_intra", "param_reduce"]
    stage_ms, launches = {}, 0
    buf, kind = (C.c_float * 8)(), C.c_int()
    for call in range(n_calls):
        n = lib.kda_profile_read(call, C.byref(kind), buf, 8)
        for i in range(max(n, 0)):
            lst = names_split if (kind.value == 1 and n == 4) else names[kind.value]
            nm = lst[i] if i < len(lst) else f"stage{i}"
            stage_ms.setdefault(nm, []).append(buf[i])
            launches += 1
    lib.kda_profile_begin(0)
    t = torch.tensor([ms], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())

    if args.kernel_only:
        if rank == 0:
            avg = {k: sum(v) / len(v) for k, v in stage_ms.items()}
            print(json.dumps({"metric": METRIC, "value": world * tokens * args.steps / (ms / 1e3) / 1e6, "unit": UNIT,
                              "kernel_only": True, "ms_per_step": ms / args.steps, "kernels_ms": avg,
                              "config": {"workload": w["label"]}}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end: pinned host inputs -> device -> op -> pinned host results ---------
    # Every step copies its inputs host->device, runs the public op, and copies every output
    # and gradient device->host.  Three streams (H2D, compute, D2H) with two buffer sets let
    # step s+1's upload and step s-1's download run under step s's kernels, the way a caller
    # that streams batches through the op would drive it; each step still moves all its bytes.
    streams = (torch.cuda.Stream(device), torch.cuda.Stream(device), torch.cuda.Stream(device))  # H2D, compute, D2H
    names = [k for k, v in host.items() if isinstance(v, torch.Tensor)]
    dev_buf = [{k: torch.empty_like(host[k], device=device) for k in names} for _ in range(2)]
    pinned_out = [None, None]
    ev_up = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_down = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(sidx, overlap=True):
        # overlap=False puts the three parts of a step on ONE stream: no copy runs under another copy or under the
        # kernels.  Some hosts deliver far less than the sum when both copy directions run at once; the leg times a
        # few steps both ways first and keeps the faster schedule (reported in e2e.how).
        b = sidx & 1
        st_h2d, st_cmp, st_d2h = streams if overlap else (streams[1],) * 3
        with torch.cuda.stream(st_h2d):
            st_h2d.wait_event(ev_cmp[b])          # the compute that last read this buffer set is done
            for k in names:
                dev_buf[b][k].copy_(host[k], non_blocking=True)
            ev_up[b].record(st_h2d)
        with torch.cuda.stream(st_cmp):
            st_cmp.wait_event(ev_up[b])
            if sub:
                xd = dev_buf[b]["x"].detach().requires_grad_(True)
                out = step_sublayer(model, xd, dev_buf[b]["dout"])
                outs = [out.detach(), xd.grad]
            else:
                d = {k: dev_buf[b][k].detach() for k in names}
                if host.get("cu") is not None:
                    d["cu_cpu"] = host["cu"]
                o, ht, leaves, h0 = step_device(d, w)
                outs = [o.detach(), ht] + [x.grad for x in leaves] + ([h0.grad] if h0 is not None else [])
            ev_cmp[b].record(st_cmp)
        with torch.cuda.stream(st_d2h):
            st_d2h.wait_event(ev_cmp[b])
            if pinned_out[b] is None:
                pinned_out[b] = [torch.empty(x.shape, dtype=x.dtype, pin_memory=True) for x in outs]
            for dst, src in zip(pinned_out[b], outs):
                src.record_stream(st_d2h)
                dst.copy_(src, non_blocking=True)
            ev_down[b].record(st_d2h)
        return pinned_out[b]

    h2d = sum(host[k].numel() * host[k].element_size() for k in names)
    for sidx in range(2):
        res = e2e_step(sidx)
    torch.cuda.synchronize()
    d2h = sum(x.numel() * x.element_size() for x in res)

    def e2e_time(nsteps, overlap):
        """ms per step of nsteps end-to-end steps (device events around the whole pipelined region, max over ranks)."""
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        barrier()
        f0.record(streams[0] if overlap else streams[1])
        for sidx in range(nsteps):
            e2e_step(sidx, overlap)
        last = streams[2] if overlap else streams[1]
        last.wait_stream(streams[1])
        last.wait_stream(streams[0])
        f1.record(last)
        torch.cuda.synchronize()
        barrier()
        t2 = torch.tensor([f0.elapsed_time(f1)], device=device)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        return float(t2.item()) / nsteps

    e2e_steps = max(4, min(args.steps, 10))
    trial = {True: e2e_time(3, True), False: e2e_time(3, False)}   # (same decision on every rank: the times are maxima over ranks)
    e2e_overlap = trial[True] <= trial[False]
    e2e_ms = e2e_time(e2e_steps, e2e_overlap)
    # what the copy engines deliver on their own (one direction at a time, this rank's buffers, all ranks
    # at once): shows whether the end-to-end leg is limited by the host side of the copies
    def copy_rate(pairs, nbytes):
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        g0.record()
        for _ in range(3):
            for dst, src in pairs:
                dst.copy_(src, non_blocking=True)
        g1.record()
        barrier()
        r = torch.tensor([3 * nbytes / (g0.elapsed_time(g1) / 1e3) / 1e9], device=device)
        lo = r.clone()
        if world > 1:
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(r, op=dist.ReduceOp.SUM)
        return {"per_rank_min": float(lo.item()), "all_ranks": float(r.item())}
    h2d_rate = copy_rate([(dev_buf[0][k], host[k]) for k in names], h2d)
    d2h_rate = copy_rate(list(zip(pinned_out[0], [torch.empty_like(x, device=device) for x in pinned_out[0]])), d2h)

    # ---- extra legs (same JSON line): strong scaling of the workload's one batch, and the sublayer -----
    def timed(fn, steps, warm):
        for _ in range(warm):
            fn()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a0.record()
        for _ in range(steps):
            fn()
        a1.record()
        barrier()
        tt = torch.tensor([a0.elapsed_time(a1)], device=device)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item()) / steps

    strong = sublayer = None
    if not args.no_extra_legs and not sub:
        from openkimi_b200.partition import shard_batch
        if world > 1 and not w["docs"]:
            # the ONE batch of the workload (rank 0's data of the weak leg), sequences dealt to the ranks
            mine = shard_batch(w["B"], world, rank)
            full = make_workload(w, seed=0)
            part = {k: (v[mine.start:mine.stop].contiguous() if isinstance(v, torch.Tensor) and v.dim() >= 3 else v)
                    for k, v in full.items()}
            dev_part = to_device(part, device) if len(mine) else None
            ws = dict(w, B=len(mine))
            ms_s = timed((lambda: step_device(dev_part, ws)) if dev_part is not None else (lambda: None), args.steps, 3)
            strong = {"value": w["B"] * w["T"] / (ms_s / 1e3) / 1e6, "unit": UNIT, "ms_per_step": ms_s,
                      "global_batch": w["B"], "sequences_per_rank": len(mine),
                      "speedup_vs_one_gpu": (ms / args.steps) / ms_s, "efficiency": (ms / args.steps) / ms_s / world,
                      "how": "config batch split by sequence with partition.shard_batch; one-GPU time = this run's "
                             "weak-scaling step (every rank runs the whole batch there); no collective"}
            del dev_part
        w4 = dict(WORKLOADS["c4"])
        w4["B"] = max(1, w4["B"] // world)
        gen4 = torch.Generator().manual_seed(100 + rank)
        width = w4["H"] * w4["d"]
        x4 = torch.randn(w4["B"], w4["T"], width, generator=gen4).bfloat16().to(device).requires_grad_(True)
        dy4 = torch.randn(w4["B"], w4["T"], width, generator=gen4).bfloat16().to(device)
        model4 = make_sublayer(w4, device)
        ms4 = timed(lambda: step_sublayer(model4, x4, dy4), max(3, min(args.steps, 5)), 3)
        sublayer = {"value": world * w4["B"] * w4["T"] / (ms4 / 1e3) / 1e6, "unit": UNIT, "ms_per_step": ms4,
                    "workload": w4["label"], "batch_per_rank": w4["B"], "scaling": "strong",
                    "how": "KimiDeltaAttention fwd+bwd under BF16 autocast, conv fused into the KDA load stage, "
                           "projections by cuBLAS; global batch 64 split over the ranks"}
        del model4, x4, dy4

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = _peaks()
    from openkimi_b200.partition import aggregate_throughput
    value = aggregate_throughput(ms, tokens, args.steps, world) / 1e6   # ms is already the max over ranks
    nt_h = (w["B"] * math.ceil(w["T"] / 64) if not w["docs"] else None)
    if nt_h is None:
        cu = host["cu"].tolist()
        nt_h = sum(math.ceil((cu[i + 1] - cu[i]) / 64) for i in range(len(cu) - 1))
    units = nt_h * w["H"]
    avg = {k: sum(v) / len(v) for k, v in stage_ms.items()}
    dom = max(avg, key=avg.get)
    flops, byts = stage_model(dom, w["d"])
    intensity = flops / byts
    ridge = peaks["tflops"] * 1e12 / (peaks["hbm_gbs"] * 1e9)
    if intensity < ridge:
        ach = byts * units / (avg[dom] / 1e3) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"]}
    else:
        ach = flops * units / (avg[dom] / 1e3) / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": ach / peaks["tflops"]}
    # DRAM bytes per (chunk, head) unit: measured figures of one ncu capture of a small case, kept in a data
    # file next to the capture's summary together with the commit they were taken at; traffic grows in
    # proportion to the units, so a full launch is the per-unit figure times its units
    traffic = traffic_src = None
    tpath = os.path.join(ROOT, "profiles", "kda_bf16_kernels_c1_batch4.traffic.json")
    if os.path.exists(tpath) and w["d"] == 128 and not sub:
        tf = json.load(open(tpath))
        kt = tf.get("kernels", {}).get(dom)
        if kt:
            traffic = (kt["dram_bytes_read"] + kt["dram_bytes_write"]) / tf["units"] * units
            traffic_src = f"ncu capture of {tf['units']} units at commit {tf['commit']}, scaled by units"
    roof.update({"kernel": dom, "kernel_ms": avg[dom], "peak_source": peaks["source"], "traffic": traffic,
                 "traffic_source": traffic_src,
                 "units_per_launch": units, "algorithmic_bytes_per_unit": byts, "algorithmic_flops_per_unit": flops})
    # whole-op fractions: dense-tile FLOPs 3*(10*C*d + 6*d^2) per (token, head); minimal HBM bytes
    d = w["d"]
    op_flops = 3 * (10 * 64 * d + 6 * d * d) * w["H"] * tokens
    op_bytes = (4 * 2 * d + 2 + 2 * d + 4 * 2 * d + 2 + 2 * d + 4 * 2 * d + 2) * w["H"] * tokens
    step_s = ms / 1e3 / args.steps
    whole = {"dense_mma_frac": op_flops / step_s / (peaks["tflops"] * 1e12),
             "min_hbm_frac": op_bytes / step_s / (peaks["hbm_gbs"] * 1e9),
             "tflops": op_flops / step_s / 1e12, "flops_per_token": op_flops / tokens}

    line = {
        "metric": "kda_sublayer_fwd_bwd_throughput" if sub else METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if sub else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["label"], "per_gpu_tokens": tokens, "state": "fp32", "chunk": 64,
                   "l2": "inputs + per-chunk records of one step ~1 GB > 126 MB L2, no explicit flush",
                   "partition": f"{world} x independent batches (sequence-parallel, no collective)"},
        "clocks": clocks,
        "e2e": {"value": world * tokens / (e2e_ms / 1e3) / 1e6, "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "how": ("3 streams (H2D / compute / D2H), 2 buffer sets" if e2e_overlap else
                        "one stream (upload, kernels, download in turn), 2 buffer sets") + "; every step moves all its bytes",
                "schedule_trial_ms": {"overlapped": trial[True], "in_turn": trial[False]},
                "copy_only_gbs": {"h2d": h2d_rate, "d2h": d2h_rate}, "cpu_affinity": numa_cpus and len(numa_cpus)},
        "gpu_launches": launches,
        "kernels_ms": avg,
        "roofline": roof,
        "whole_op": whole,
    }
    if strong:
        line["strong"] = strong
    if sublayer:
        line["sublayer"] = sublayer
    if not args.no_cpu_baseline:
        try:
            os.sched_setaffinity(0, range(os.cpu_count()))  # the CPU arm may use every host core again
        except Exception:
            pass
        torch.set_num_threads(os.cpu_count() or 1)
        inp_c, T_c = cpu_slice_inputs(w)
        cpu_slice_seconds(w, inp_c)  # warm-up (thread pool, allocator)
        reps = 3
        secs = sum(cpu_slice_seconds(w, inp_c) for _ in range(reps)) / reps
        line["cpu_baseline"] = {"value": (T_c / w["H"]) / secs / 1e6, "unit": UNIT, "cores": torch.get_num_threads(),
                                "kind": "port", "sample": cpu_sample_text(w, T_c) + f"; {secs:.1f} s per slice, mean of {reps}"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
