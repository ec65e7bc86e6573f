#!/usr/bin/env python
"""Benchmark of the FLARE mixer forward+backward (Mtokens/s), one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

ours      : libflare_b200.so through the public API (flare_multihead_mixer, or its
            context-parallel form when N > 1: the token axis is sharded over the ranks,
            total work fixed -> "scaling": "strong").
reference : the reference project's CPU implementation of the same path (two SDPA
            calls + autograd, README.md:37-53), timed on the host cores of the box on a
            bounded sample of the same workload.

Workload: B=1, H=8, N=1,048,576, M=256, D=32, bf16, q,k,v ~ N(0, D^-1/2), dy ~ N(0,1),
seeded synthetic tensors (no dataset is involved).  K, V, dY, Y, dK, dV are 512 MiB each, so
every pass streams far more than the 126 MB L2; no explicit flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD = dict(B=1, H=8, N=1 << 20, M=256, D=32)
DTYPE = torch.bfloat16
METRIC = "FLARE mixer fwd+bwd Mtokens/s"
CPU_SAMPLE_TOKENS = 131072


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ----------------------------------------------------------------------------------
# clocks sampled while the timed region runs
# ----------------------------------------------------------------------------------
class ClockSampler:
    """SM clock and throttle reasons of one GPU, polled through NVML every ~2 ms from a thread while the timed
    region runs (the timed region is tens of milliseconds: nvidia-smi's own loop is too coarse for it).
    Reading only; nothing is set."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, index: int):
        self.index, self.sm, self.mask, self.max_mhz = index, [], 0, None
        self._stop = threading.Event()
        self._thread = None
        self._nv = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None
            return
        self._thread = threading.Thread(target=self._poll, daemon=True)
        self._thread.start()

    def _poll(self):
        nv = self._nv
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                if get_reasons:
                    self.mask |= int(get_reasons(self._h))
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self):
        if not self._thread:
            return None
        self._stop.set()
        self._thread.join(timeout=2)
        if not self.sm:
            return None
        reasons = sorted(n for bit, n in self.REASONS.items() if self.mask & bit)
        return dict(sm_mhz=statistics.median(self.sm), sm_max_mhz=self.max_mhz, reasons=reasons, samples=len(self.sm))


# ----------------------------------------------------------------------------------
# reference arm / CPU baseline: the two-SDPA path on the host cores
# ----------------------------------------------------------------------------------
def cpu_reference_step(q, k, v, dy):
    from oracle import flare_oracle as O
    q = q.detach().requires_grad_(True)
    k = k.detach().requires_grad_(True)
    v = v.detach().requires_grad_(True)
    y = O.mixer_sdpa(q, k, v, 1.0)
    y.backward(dy)
    return y, q.grad, k.grad, v.grad


def cpu_inputs(n_tokens):
    from oracle import flare_oracle as O
    w = WORKLOAD
    return O.make_inputs(w["B"], w["H"], n_tokens, w["M"], w["D"], dtype=DTYPE, seed=0)


def time_cpu(n_tokens, steps, warmup):
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, dy = cpu_inputs(n_tokens)
    for _ in range(warmup):
        cpu_reference_step(q, k, v, dy)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_reference_step(q, k, v, dy)
    dt = (time.perf_counter() - t0) / steps
    return dt, torch.get_num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOAD
    dt, cores = time_cpu(CPU_SAMPLE_TOKENS, args.steps, args.warmup)
    val = w["B"] * CPU_SAMPLE_TOKENS / dt / 1e6
    sample = (f"{CPU_SAMPLE_TOKENS} of {w['N']} tokens per step (same H, M, D, bf16), two SDPA calls + autograd "
              f"on the host CPU, torch {torch.__version__}")
    line = dict(
        impl="reference", metric=METRIC, value=val, unit="Mtokens/s", n_gpus=args.gpus, steps=args.steps,
        warmup=args.warmup, ms_per_step=dt * 1e3, higher_is_better=True, scaling="strong", vs_baseline=None,
        dtype="bf16", data="synthetic",
        config=dict(workload="mixer_1M: B=1 H=8 N=1048576 M=256 D=32 bf16 fwd+bwd", sample_tokens=CPU_SAMPLE_TOKENS),
        cpu_baseline=dict(value=val, unit="Mtokens/s", cores=cores, kind="port", sample=sample),
        e2e=dict(value=val, unit="Mtokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
        gpu_launches=0,
    )
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------
def pass_table(B, H, N, M, D, e):
    """Algorithmic work of each launch: FLOPs, exponentials, HBM bytes (W = B*H*M*N, T = B*H*N*D*e)."""
    W, T, r = B * H * M * N, B * H * N * D * e, B * H * N * 4
    return {
        "gather_partial": dict(flops=4 * W * D, exps=W, bytes=2 * T),
        "scatter":        dict(flops=4 * W * D, exps=W, bytes=2 * T + r),
        "bwd_dz_partial": dict(flops=4 * W * D, exps=W, bytes=2 * T + r),
        "bwd_main":       dict(flops=12 * W * D, exps=W, bytes=6 * T + r),
    }


def time_passes(fb, q, k, v, dy, iters=3):
    """CUDA-event time of every kernel of one fwd+bwd, launched one by one through the C ABI."""
    from flare_b200 import _cabi
    from flare_b200.mixer import make_problem
    lib, ptr = _cabi.lib, _cabi.ptr
    B, H, N, D = k.shape
    M = q.shape[-2]
    dev = k.device
    y, dk, dv = torch.empty_like(k), torch.empty_like(k), torch.empty_like(v)
    p = make_problem(q, k, 1.0, v=v, y=y, dy=dy, dk=dk, dv=dv)
    p.n_splits = lib.flare_pick_splits(C.byref(p))
    S = p.n_splits
    rec = torch.empty(S, B, H, M, D + 2, dtype=torch.float32, device=dev)
    part = torch.empty(S, B, H, M, D, dtype=torch.float32, device=dev)
    z32 = torch.empty(B, H, M, D, dtype=torch.float32, device=dev)
    dz32 = torch.empty_like(z32)
    lse_m = torch.empty(B, H, M, dtype=torch.float32, device=dev)
    lse_n = torch.empty(B, H, N, dtype=torch.float32, device=dev)
    delta = torch.empty_like(lse_n)
    dq = torch.empty(H, M, D, dtype=torch.float32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    P = C.byref(p)
    calls = [
        ("gather_partial", lambda: lib.flare_gather_partial(P, ptr(q), ptr(k), ptr(v), None, ptr(rec), st)),
        ("combine", lambda: lib.flare_combine(P, ptr(rec), S, ptr(z32), None, ptr(lse_m), None, st)),
        ("scatter", lambda: lib.flare_scatter(P, ptr(q), ptr(k), ptr(z32), None, ptr(y), ptr(lse_n), st)),
        ("bwd_dz_partial", lambda: lib.flare_bwd_dz_partial(P, ptr(q), ptr(k), ptr(dy), None, ptr(lse_n), ptr(part), st)),
        ("reduce_dz", lambda: lib.flare_reduce_sum(ptr(part), S, B * H * M, D, ptr(dz32), st)),
        ("bwd_main", lambda: lib.flare_bwd_main(P, 3, ptr(q), ptr(k), ptr(v), ptr(dy), ptr(y), None, ptr(z32), ptr(dz32),
                                               ptr(lse_m), ptr(lse_n), ptr(dk), ptr(dv), ptr(delta), ptr(part), st)),
        ("reduce_dq", lambda: lib.flare_reduce_sum(ptr(part), S * B, H * M, D, ptr(dq), st)),
    ]
    times = {n: [] for n, _ in calls}
    for it in range(iters + 1):
        for name, fn in calls:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            # the GPU is kept busy for ~0.25 ms while the host enqueues the events and the call, so that the
            # interval between the events is device time only (a call's host side -- tensor maps, several
            # launches -- takes tens of microseconds, more than the small kernels run)
            torch.cuda._sleep(500_000)
            e0.record()
            _cabi.check(fn(), name)
            e1.record()
            e1.synchronize()
            if it > 0:
                times[name].append(e0.elapsed_time(e1))
    return {n: sum(v_) / len(v_) for n, v_ in times.items()}, S


def measure_ex2_peak(dev):
    """Gexp/s of the exponential unit, from the library's probe kernel (148 SMs x 8 blocks)."""
    from flare_b200 import _cabi
    out = torch.zeros(1, device=dev)
    blocks, iters = 148 * 8, 4096
    st = torch.cuda.current_stream().cuda_stream
    best = 0.0
    for i in range(4):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _cabi.check(_cabi.lib.flare_probe_ex2(blocks, iters, out.data_ptr(), st), "probe")
        e1.record()
        e1.synchronize()
        if i:
            best = max(best, blocks * 256 * 8 * iters / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    return best


def run_ours(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import __graft_entry__
    if rank == 0:
        __graft_entry__.build()
    if world > 1:
        dist.barrier()
    import flare_b200 as fb
    from flare_b200.parallel import flare_mixer_context_parallel, shard_bounds

    w = dict(WORKLOAD)
    if args.tokens:
        w["N"] = args.tokens
    B, H, N, M, D = (w[x] for x in "BHNMD")
    n0, n1 = shard_bounds(N, world, rank, multiple=128)
    Nl = n1 - n0
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    sd = D ** -0.25
    # host (pinned) copies feed the end-to-end measurement; device copies feed the resident one
    hq = (torch.randn(H, M, D, generator=torch.Generator().manual_seed(7)) * sd).to(DTYPE).pin_memory()
    hk = (torch.randn(B, H, Nl, D, generator=g) * sd).to(DTYPE).pin_memory()
    hv = (torch.randn(B, H, Nl, D, generator=g) * sd).to(DTYPE).pin_memory()
    hdy = torch.randn(B, H, Nl, D, generator=g).to(DTYPE).pin_memory()
    q = hq.to(dev).requires_grad_(True)
    k = hk.to(dev).requires_grad_(True)
    v = hv.to(dev).requires_grad_(True)
    dy = hdy.to(dev)

    # N > 1: the exchanges go through symmetric memory and peer loads (FLARE_CP_EXCHANGE=nccl selects the
    # torch.distributed collectives instead)
    cp_ex, cp_kind = None, None
    if world > 1:
        from flare_b200.parallel import PeerExchange, RecordExchange
        cp_kind = os.environ.get("FLARE_CP_EXCHANGE", "peer")
        if cp_kind == "peer":
            try:
                cp_ex = PeerExchange()
                cp_ex.prepare_mixer(B, H, M, D, dev)            # the symmetric-memory rendezvous happens here
            except Exception as e:                              # no symmetric memory on this box: NCCL collectives
                print(f"[bench] peer-memory exchange unavailable ({e!r}); using NCCL", file=sys.stderr, flush=True)
                cp_kind, cp_ex = "nccl", None
        ok = torch.tensor([1 if cp_kind == "peer" else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)               # all ranks must agree
        if ok.item() == 0:
            cp_kind, cp_ex = "nccl", RecordExchange()

    def mixer(q_, k_, v_):
        if world > 1:
            return flare_mixer_context_parallel(q_, k_, v_, 1.0, exchange=cp_ex)
        return fb.flare_multihead_mixer(q_, k_, v_, scale=1.0)

    def step():
        q.grad = k.grad = v.grad = None
        y = mixer(q, k, v)
        y.backward(dy)
        return y

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # N > 1: the step recorded in a CUDA graph.  A rank's share of the step shrinks with N while the host's
    # cost to enqueue it does not; the recorded sequence (two steps, see GraphedStep) is replayed instead.
    # It has an exchange object of its own, so eager steps may run between replays.
    graphed = None
    if world > 1 and cp_kind == "peer" and not args.no_graph:
        from flare_b200.parallel import GraphedStep
        try:
            g_ex = PeerExchange()
            g_ex.prepare_mixer(B, H, M, D, dev)

            def graph_step():
                q.grad = k.grad = v.grad = None
                y = flare_mixer_context_parallel(q, k, v, 1.0, exchange=g_ex)
                y.backward(dy)
                return y

            graphed = GraphedStep(graph_step)
        except Exception as e:
            print(f"[bench] CUDA-graph capture of the step failed ({e!r}); eager launches", file=sys.stderr, flush=True)
            graphed = None
        ok = torch.tensor([1 if graphed is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)               # all ranks must agree
        if ok.item() == 0:
            graphed = None

    def run_steps(n):
        if graphed is not None:
            for _ in range(n // 2):
                graphed.replay()
            n = n % 2
        for _ in range(n):
            step()

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if fn is step:
            run_steps(steps)
        else:
            for _ in range(steps):
                fn()
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    total_ms = timed(step, args.steps)
    clocks = sampler.stop() if sampler else None
    ms_step = total_ms / args.steps
    value = B * N / (ms_step * 1e-3) / 1e6

    # host time per step (Python, ctypes, allocator): the launches are asynchronous, so the time the loop
    # takes to enqueue a step without waiting for the device is what the host side costs
    sync_all()
    t0 = time.perf_counter()
    run_steps(args.steps)
    host_ms = (time.perf_counter() - t0) / args.steps * 1e3
    sync_all()

    # the same step back to back for at least two seconds: the clock settles under sustained load
    sustained = None
    if not args.no_sustained:
        n_sus = max(args.steps, int(2000.0 / ms_step) + 1)
        s2 = ClockSampler(local) if rank == 0 else None
        if s2:
            s2.start()
        sus_ms = timed(step, n_sus) / n_sus
        c2 = s2.stop() if s2 else None
        if rank == 0:
            sustained = dict(steps=n_sus, ms_per_step=sus_ms, value=B * N / (sus_ms * 1e-3) / 1e6,
                             sm_mhz=c2["sm_mhz"] if c2 else None, reasons=c2["reasons"] if c2 else None,
                             ms_x_mhz=sus_ms * c2["sm_mhz"] if c2 else None)

    # N > 1: the context-parallel result against the single-GPU one on a small seeded problem
    cp_parity = None
    if world > 1:
        Np = 16384
        gp = torch.Generator(device="cpu").manual_seed(4321)
        pq = (torch.randn(H, M, D, generator=gp) * sd).to(DTYPE).to(dev)
        pk = (torch.randn(B, H, Np, D, generator=gp) * sd).to(DTYPE).to(dev)
        pv = (torch.randn(B, H, Np, D, generator=gp) * sd).to(DTYPE).to(dev)
        pdy = torch.randn(B, H, Np, D, generator=gp).to(DTYPE).to(dev)
        a0, a1 = shard_bounds(Np, world, rank, multiple=128)
        q1, k1, v1 = (t.clone().requires_grad_(True) for t in (pq, pk, pv))
        y1 = fb.flare_multihead_mixer(q1, k1, v1, scale=1.0)
        y1.backward(pdy)
        q2 = pq.clone().requires_grad_(True)
        k2 = pk[:, :, a0:a1].contiguous().requires_grad_(True)
        v2 = pv[:, :, a0:a1].contiguous().requires_grad_(True)
        y2 = flare_mixer_context_parallel(q2, k2, v2, 1.0, exchange=cp_ex)
        y2.backward(pdy[:, :, a0:a1].contiguous())

        def rel(a, b):
            a, b = a.float(), b.float()
            return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()

        errs = torch.tensor([rel(y2, y1[:, :, a0:a1]), rel(q2.grad, q1.grad), rel(k2.grad, k1.grad[:, :, a0:a1]),
                             rel(v2.grad, v1.grad[:, :, a0:a1])], device=dev)
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
        cp_parity = dict(zip(("y", "dq", "dk", "dv"), errs.tolist()), tokens=Np,
                         against="single-GPU mixer on the same tensors, max over ranks of the shard's relative L2")
        if not all(e <= 2e-2 for e in errs.tolist()):
            raise SystemExit(f"context-parallel parity failed: {cp_parity}")

    # end to end: pinned host inputs -> device, fwd+bwd, results back to pinned host memory.
    # The step a user of the library runs with host-resident data.  The two PCIe directions are used at
    # the same time where the data dependences allow it: dY goes up while the forward runs and y comes
    # down (side streams), everything else is ordered on the lane's stream.  On one GPU three such lanes
    # take turns, each with its own streams and host buffers, so that step i+1's inputs go up while step
    # i's gradients come down (measured: 50.9 ms per step with one lane, 39.2 with two, 35.8 with three, 35.1
    # with four: both PCIe directions busy) (what a prefetching loader does; every step still moves all of its bytes
    # inside the timed region).  Context-parallel runs keep one lane: two lanes would interleave two
    # sequences of exchanges on each GPU.
    class Lane:
        def __init__(self):
            self.main = torch.cuda.Stream(device=dev)
            self.s_in, self.s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
            self.hy = torch.empty_like(hk).pin_memory()
            self.hdk = torch.empty_like(hk).pin_memory()
            self.hdv = torch.empty_like(hk).pin_memory()
            self.hdq = torch.empty(H, M, D, dtype=DTYPE).pin_memory()

    lanes = [Lane() for _ in range(3 if world == 1 else 1)]
    hy, hdk, hdv, hdq = lanes[0].hy, lanes[0].hdk, lanes[0].hdv, lanes[0].hdq

    def e2e_step(lane):
        cur = lane.main
        with torch.cuda.stream(cur):
            q_ = hq.to(dev, non_blocking=True).requires_grad_(True)
            k_ = hk.to(dev, non_blocking=True).requires_grad_(True)
            v_ = hv.to(dev, non_blocking=True).requires_grad_(True)
            up = torch.cuda.Event()
            up.record(cur)
            with torch.cuda.stream(lane.s_in):
                lane.s_in.wait_event(up)                  # after k, v: the link is busy until then anyway
                dy_ = hdy.to(dev, non_blocking=True)
                dy_.record_stream(cur)
            y_ = mixer(q_, k_, v_)
            fwd = torch.cuda.Event()
            fwd.record(cur)
            with torch.cuda.stream(lane.s_out):
                lane.s_out.wait_event(fwd)
                yd = y_.detach()
                yd.record_stream(lane.s_out)
                lane.hy.copy_(yd, non_blocking=True)
            cur.wait_stream(lane.s_in)
            y_.backward(dy_)
            cur.wait_stream(lane.s_out)                   # device-to-host copies share one direction: keep them in order
            lane.hdk.copy_(k_.grad, non_blocking=True)
            lane.hdv.copy_(v_.grad, non_blocking=True)
            lane.hdq.copy_(q_.grad, non_blocking=True)

    def e2e_run(n):
        sync_all()
        cur0 = torch.cuda.current_stream(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(cur0)
        for lane in lanes:
            lane.main.wait_event(e0)
        for i in range(n):
            e2e_step(lanes[i % len(lanes)])
        for lane in lanes:
            cur0.wait_stream(lane.main)
        e1.record(cur0)
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    e2e_steps = max(4, min(args.steps, 10))
    e2e_run(2 * len(lanes))
    e2e_ms = e2e_run(e2e_steps) / e2e_steps
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdy))
    d2h = sum(t.numel() * t.element_size() for t in (hy, hdk, hdv, hdq))

    # per-kernel times and the roofline of the dominant one (rank 0's shard)
    pk = peaks()
    roof = None
    passes = {}
    if rank == 0:
        with torch.no_grad():
            passes, S = time_passes(fb, q.detach(), k.detach(), v.detach(), dy)
        tab = pass_table(B, H, Nl, M, D, 2)
        ex2 = measure_ex2_peak(dev)
        top = max(tab, key=lambda n: passes.get(n, 0.0))
        t_s = passes[top] * 1e-3
        work = tab[top]
        terms = dict(hbm_ms=work["bytes"] / (pk["hbm_gbs"] * 1e9) * 1e3,
                     tensor_ms=work["flops"] / (pk["bf16_tflops"] * 1e12) * 1e3,
                     mufu_ms=work["exps"] / (ex2 * 1e9) * 1e3)
        bound = max(("hbm", terms["hbm_ms"]), ("tensor", terms["tensor_ms"]), ("mufu", terms["mufu_ms"]), key=lambda x: x[1])[0]
        ach = {"hbm": work["bytes"] / t_s / 1e9, "tensor": work["flops"] / t_s / 1e12, "mufu": work["exps"] / t_s / 1e9}
        peak = {"hbm": pk["hbm_gbs"], "tensor": pk["bf16_tflops"], "mufu": ex2}
        unit = {"hbm": "GB/s", "tensor": "TFLOP/s", "mufu": "Gexp/s"}
        traffic = None
        tf = ROOT / "profiles" / "dram_traffic.json"
        if tf.exists():
            per = json.loads(tf.read_text()).get(top)
            if per:
                traffic = per["bytes_per_token_head"] * B * H * Nl
        all_tab = {n: tab[n] for n in tab}
        whole_bound_ms = max(sum(x["bytes"] for x in all_tab.values()) / (pk["hbm_gbs"] * 1e9),
                             sum(x["flops"] for x in all_tab.values()) / (pk["bf16_tflops"] * 1e12),
                             sum(x["exps"] for x in all_tab.values()) / (ex2 * 1e9)) * 1e3
        roof = dict(kernel=top, bound=bound, achieved=ach[bound], peak=peak[bound], unit=unit[bound],
                    frac=ach[bound] / peak[bound], traffic=traffic, peaks_source=pk["source"],
                    hbm_frac=ach["hbm"] / peak["hbm"], tensor_frac=ach["tensor"] / peak["tensor"],
                    mufu_frac=ach["mufu"] / peak["mufu"], ex2_peak_gexps=ex2, bound_terms_ms=terms,
                    kernel_ms=passes, path_bound_ms=whole_bound_ms,
                    path_frac=whole_bound_ms / (sum(passes.values())))

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        dt, cores = time_cpu(CPU_SAMPLE_TOKENS, 3, 1)
        cpu = dict(value=B * CPU_SAMPLE_TOKENS / dt / 1e6, unit="Mtokens/s", cores=cores, kind="port",
                   sample=f"{CPU_SAMPLE_TOKENS} of {N} tokens (same H, M, D, bf16), two SDPA calls + autograd, "
                          f"1 warm-up + 3 runs, mean")

    if rank == 0:
        # forward: gather, combine, scatter; backward: dZ partial, reduce, range check (2 kernels),
        # one-exponential main kernel, flag-gated exact kernel, dQ reduce.  Context parallel over peer memory:
        # each of the three exchanges adds the barrier kernel and the kernel that reads all ranks' buffers
        launches_per_step = 10 if world == 1 else (16 if cp_kind == "peer" else 11)
        line = dict(
            metric=METRIC, value=value, unit="Mtokens/s", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
            ms_per_step=ms_step, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16",
            data="synthetic",
            config=dict(workload=f"mixer_1M: B={B} H={H} N={N} M={M} D={D} bf16 fwd+bwd",
                        parallelism=("single GPU" if world == 1 else
                                     f"context parallel, N sharded over {world} ranks, exchange={cp_kind}"
                                     + (", step replayed from a CUDA graph" if graphed is not None else "")),
                        tokens_per_rank=Nl, l2="inputs larger than L2 (K,V,dY,Y,dK,dV 64 B x tokens x heads each); no flush",
                        kernel_path="tcgen05 (decoupled gather/scatter/dZ, pipelined one-exponential backward behind an on-device range check); fp32 reductions"),
            clocks=clocks,
            e2e=dict(value=B * N / (e2e_ms * 1e-3) / 1e6, unit="Mtokens/s", h2d_bytes_per_step=h2d * world,
                     d2h_bytes_per_step=d2h * world, ms_per_step=e2e_ms),
            gpu_launches=launches_per_step * args.steps,
            roofline=roof, cpu_baseline=cpu, sustained=sustained, host_ms_per_step=host_ms, cp_parity=cp_parity,
        )
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_causal(args):
    """Secondary workload (not the headline line): causal FLARE prefill and one decode step at the serving
    shape B=4, H=16, N=8192, D=64, M=128 bf16, device-resident inputs, CUDA events."""
    import flare_b200 as fb
    dev = torch.device("cuda:0")
    B, H, N, D, M = 4, 16, 8192, 64, 128
    g = torch.Generator().manual_seed(0)
    q = (torch.randn(H, M, D, generator=g) * D ** -0.25).bfloat16().to(dev)
    k = (torch.randn(B, H, N, D, generator=g) * D ** -0.25).bfloat16().to(dev)
    v = torch.randn(B, H, N, D, generator=g).bfloat16().to(dev)

    def timed(fn, steps, lead_cycles=0):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if lead_cycles:                              # the host enqueues ahead of the device: device time per call
            torch.cuda._sleep(lead_cycles)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    for _ in range(max(args.warmup, 1)):
        _, st = fb.flare_causal_prefill(q, k, v, 1.0)
    # four launches and three allocations per call cost the host about as much as the device needs for them
    ms = timed(lambda: fb.flare_causal_prefill(q, k, v, 1.0), args.steps, lead_cycles=400_000 * args.steps)
    k1, v1 = k[:, :, :1].contiguous(), v[:, :, :1].contiguous()
    fb.flare_causal_decode(q, k1, v1, st, 1.0)
    us = timed(lambda: fb.flare_causal_decode(q, k1, v1, st, 1.0), max(args.steps, 20)) * 1e3
    # the serving loop as it would run: 16 decode steps recorded once in a CUDA graph over static buffers and the
    # in-place state, replayed; device time per step without the host's launch cost
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        fb.flare_causal_decode(q, k1, v1, st, 1.0)
    torch.cuda.current_stream(dev).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(16):
            fb.flare_causal_decode(q, k1, v1, st, 1.0)
    graph.replay()
    us_graph = timed(graph.replay, max(args.steps, 20)) * 1e3 / 16
    # training step of the same layer: forward + backward through flare_causal_mixer
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    dy = torch.randn(B, H, N, D, generator=g).bfloat16().to(dev)

    def train_step():
        qg.grad = kg.grad = vg.grad = None
        fb.flare_causal_mixer(qg, kg, vg, 1.0).backward(dy)

    train_step()
    train_ms = timed(train_step, max(2, min(args.steps, 5)))
    # the prefill against its bounds: k, v read and y written once (2 bytes each), the three contractions of the
    # chunked form (scores, state update, read-out: 2 M D flops per token each); the walk of every 128-token chunk
    # runs on the tensor cores (five products per chunk), its softmax, running sum and mask on the fp32 pipes
    pk = peaks()
    tok_bytes = B * H * N * D * 2
    alg_bytes, alg_flops = 3 * tok_bytes, 3 * 2 * B * H * N * M * D
    roof = dict(bound="hbm", achieved=alg_bytes / (ms * 1e-3) / 1e9, peak=pk["hbm_gbs"], unit="GB/s",
                frac=alg_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], traffic=None, peaks_source=pk["source"],
                tensor_frac=alg_flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], kernel="k_causal_tc_walk (tcgen05)")
    print(json.dumps(dict(metric="causal FLARE prefill Mtokens/s", value=B * N / ms / 1e3, unit="Mtokens/s", n_gpus=1,
                          steps=args.steps, warmup=max(args.warmup, 1), ms_per_step=ms, higher_is_better=True,
                          dtype="bf16", data="synthetic", decode_step_us=us, decode_step_graph_us=us_graph, fwd_bwd_ms=train_ms,
                          roofline=roof,
                          config=dict(workload=f"causal_prefill: B={B} H={H} N={N} M={M} D={D} bf16, one layer's mixer"))),
          flush=True)


def run_triple(args):
    """Secondary workload (not the headline line): triple attention forward and forward + backward at the
    reference benchmark's shape (lra/models/triton/triple.py:936-1060: B=1, H=8, D=32, fp16), device-resident."""
    import flare_b200 as fb
    dev = torch.device("cuda:0")
    B, H, D = 1, 8, 32
    N = args.tokens or 500_000
    g = torch.Generator().manual_seed(0)
    mk = lambda s: (torch.randn(B, H, N, D, generator=g) * s).half().to(dev).requires_grad_(True)
    q1, q2, k1, k2 = (mk(D ** -0.5) for _ in range(4))
    v = mk(1.0)
    do = torch.randn(B, H, N, D, generator=g).half().to(dev)

    def timed(fn, steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def fwd():
        with torch.no_grad():
            return fb.triple_attention(q1, q2, k1, k2, v)

    def fwd_bwd():
        for t in (q1, q2, k1, k2, v):
            t.grad = None
        fb.triple_attention(q1, q2, k1, k2, v)[1].backward(do)

    for _ in range(max(args.warmup, 2)):
        fwd_bwd()
    ms_f, ms_fb = timed(fwd, args.steps), timed(fwd_bwd, args.steps)
    # every launch is one product over the 1024-long pair axis: 2 * 1024 * D flops per token and head;
    # forward = 2 launches (STATE, O), backward = 6 (dSTATE, dQ1, dQ2, dK1, dK2, dV)
    pk = peaks()
    per_launch = 2.0 * D * D * D * N * B * H
    roof = dict(bound="tensor", achieved=8 * per_launch / (ms_fb * 1e-3) / 1e12, peak=pk["bf16_tflops"], unit="TFLOP/s",
                frac=8 * per_launch / (ms_fb * 1e-3) / 1e12 / pk["bf16_tflops"], traffic=None, peaks_source=pk["source"],
                kernel="k_triple_tc_outer / k_triple_tc_contract")
    print(json.dumps(dict(metric="triple attention fwd+bwd Mtokens/s", value=B * N / ms_fb / 1e3, unit="Mtokens/s",
                          n_gpus=1, steps=args.steps, warmup=max(args.warmup, 2), ms_per_step=ms_fb, fwd_ms=ms_f,
                          higher_is_better=True, dtype="f16", data="synthetic", roofline=roof,
                          config=dict(workload=f"triple: B={B} H={H} N={N} D={D} fp16"))), flush=True)


def run_causal_linear(args):
    """Secondary workload (not the headline line): causal linear attention forward at the shape of the reference's
    benchmark (lra/models/triton/causal_linear.py:589-650: B=8, H=8, N=2048, Dk=128, Dv=32), bf16, device-resident."""
    import flare_b200 as fb
    dev = torch.device("cuda:0")
    B, H, Dk, Dv = 8, 8, 128, 32
    N = args.tokens or 2048
    g = torch.Generator().manual_seed(0)
    # one call's tensors (84 MB at the default N) fit in L2: the calls rotate over enough input sets to exceed it
    n_sets = max(2, -(-3 * 126_000_000 // (2 * B * H * N * (2 * Dk + 2 * Dv))))
    sets = [((torch.randn(B, H, N, Dk, generator=g) * Dk ** -0.5).bfloat16().to(dev),
             torch.randn(B, H, N, Dk, generator=g).bfloat16().to(dev),
             torch.randn(B, H, N, Dv, generator=g).bfloat16().to(dev)) for _ in range(n_sets)]
    for i in range(max(args.warmup, 3)):
        fb.causal_linear(*sets[i % n_sets])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(200_000 * args.steps)          # the host enqueues ahead of the device: device time per call
    e0.record()
    for i in range(args.steps):
        fb.causal_linear(*sets[i % n_sets])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    # q, k, v read and y written once (2 bytes each): the bound; the passes read k and v twice
    pk = peaks()
    alg_bytes = 2 * B * H * N * (2 * Dk + 2 * Dv)
    alg_flops = 2.0 * B * H * N * (128 * Dk + 128 * Dv + 2 * Dk * Dv)      # per token: S row, S V, K^T V and Q P
    roof = dict(bound="hbm", achieved=alg_bytes / (ms * 1e-3) / 1e9, peak=pk["hbm_gbs"], unit="GB/s",
                frac=alg_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], traffic=None, peaks_source=pk["source"],
                tensor_frac=alg_flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], kernel="k_cl_tc_sums / k_cl_tc_walk (tcgen05)")
    print(json.dumps(dict(metric="causal linear attention fwd Mtokens/s", value=B * N / ms / 1e3, unit="Mtokens/s",
                          n_gpus=1, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=ms, higher_is_better=True,
                          dtype="bf16", data="synthetic", roofline=roof,
                          config=dict(workload=f"causal_linear: B={B} H={H} N={N} Dk={Dk} Dv={Dv} bf16",
                                      l2=f"calls rotate over {n_sets} input sets, more than L2 together"))), flush=True)


def run_sdpa_gpu(args):
    """Secondary line (not the headline): the kernels the reference dispatches for this path on this GPU, i.e.
    its two F.scaled_dot_product_attention calls (README.md:49-50) and their autograd in bf16 through the
    installed torch, on the benchmark's tensors, next to this library's time for the same problem."""
    import torch.nn.functional as F
    import flare_b200 as fb
    dev = torch.device("cuda:0")
    w = dict(WORKLOAD)
    if args.tokens:
        w["N"] = args.tokens
    B, H, N, M, D = (w[x] for x in "BHNMD")
    g = torch.Generator().manual_seed(1234)
    sd = D ** -0.25
    q = (torch.randn(H, M, D, generator=g) * sd).to(DTYPE).to(dev).requires_grad_(True)
    k = (torch.randn(B, H, N, D, generator=g) * sd).to(DTYPE).to(dev).requires_grad_(True)
    v = (torch.randn(B, H, N, D, generator=g) * sd).to(DTYPE).to(dev).requires_grad_(True)
    dy = torch.randn(B, H, N, D, generator=g).to(DTYPE).to(dev)

    def sdpa_step():
        q.grad = k.grad = v.grad = None
        qe = q.unsqueeze(0).expand(B, -1, -1, -1)
        z = F.scaled_dot_product_attention(qe, k, v, scale=1.0)
        y = F.scaled_dot_product_attention(k, qe, z, scale=1.0)
        y.backward(dy)
        return y

    def ours_step():
        q.grad = k.grad = v.grad = None
        y = fb.flare_multihead_mixer(q, k, v, scale=1.0)
        y.backward(dy)
        return y

    def timed(fn, steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    out = {}
    for name, fn in (("sdpa", sdpa_step), ("ours", ours_step)):
        for _ in range(max(args.warmup, 3)):
            y = fn()
        out[name] = timed(fn, args.steps)
        out[name + "_y"] = y.detach().float()
        out[name + "_dk"] = k.grad.detach().float()
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()
    print(json.dumps(dict(
        metric="reference GPU path: two SDPA calls + autograd, Mtokens/s", value=B * N / out["sdpa"] / 1e3, unit="Mtokens/s",
        n_gpus=1, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=out["sdpa"], higher_is_better=True,
        dtype="bf16", data="synthetic", torch=torch.__version__,
        ours_ms_per_step=out["ours"], ours_over_sdpa=out["sdpa"] / out["ours"],
        agreement=dict(y=rel(out["ours_y"], out["sdpa_y"]), dk=rel(out["ours_dk"], out["sdpa_dk"])),
        config=dict(workload=f"sdpa_gpu: B={B} H={H} N={N} M={M} D={D} bf16 fwd+bwd"))), flush=True)


def run_cp_encoder(args):
    """Secondary line: the context-parallel FLARE encoder as a training step -- 3-D point cloud (3 coordinates
    + 4 channels), hidden 256, 8 heads (D = 32), 512 latents, 4 blocks, bf16 autocast, MSE, per-block activation
    checkpointing, the points sharded over the ranks.  16,777,216 points on 8 GPUs; with fewer ranks the same
    2,097,152 points per rank unless --tokens says otherwise."""
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import __graft_entry__
    if rank == 0:
        __graft_entry__.build()
    dist.barrier()
    import flare_b200 as fb
    n_points = args.tokens or (2_097_152 * world)
    torch.manual_seed(0)
    model = fb.FLAREModel(in_dim=7, out_dim=1, channel_dim=256, num_blocks=4, num_heads=8, num_latents=512).to(dev)
    kind = os.environ.get("FLARE_CP_EXCHANGE", "peer" if world > 1 else "collective")
    cp = fb.ContextParallel(exchange=kind)
    fb.enable_context_parallel(model, cp, checkpoint_blocks=True)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4)
    data = fb.ShardedPointCloud(n_points, 4, 1, rank, world, seed=0, device=dev)
    x, t = data.sample(0)

    def step():
        return fb.cp_train_step(model, opt, x, t, cp, autocast_dtype=torch.bfloat16, clip_grad_norm=1.0)

    for _ in range(max(args.warmup, 1)):
        loss = step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    peak = torch.tensor([torch.cuda.max_memory_allocated(dev) / 2 ** 30], device=dev)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps(dict(
            metric="context-parallel FLARE encoder training step, Mpoints/s", value=n_points / ms.item() / 1e3,
            unit="Mpoints/s", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 1), ms_per_step=ms.item(),
            higher_is_better=True, scaling="weak" if not args.tokens else "strong", dtype="bf16", data="synthetic",
            loss=loss.item(), peak_memory_gib=peak.item(), status=fb.device_status(),
            config=dict(workload=f"cp_encoder: N={n_points} points, C=256 H=8 D=32 M=512, 4 blocks, bf16 autocast, "
                                 f"AdamW, per-block checkpointing", points_per_rank=data.n1 - data.n0, exchange=kind))),
              flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="override N (profiling on a smaller case)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second sustained leg")
    ap.add_argument("--no-graph", action="store_true", help="N > 1: launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--workload", default="mixer", choices=["mixer", "causal", "triple", "causal_linear", "sdpa_gpu", "cp_encoder"],
                    help="mixer: the headline line; causal: a secondary line for causal prefill/decode/training; triple: a "
                         "secondary line for triple attention; causal_linear: a secondary line for causal linear attention; sdpa_gpu: "
                         "a secondary line timing the reference's own two SDPA calls + autograd on this GPU")
    args = ap.parse_args()
    if args.workload == "causal":
        run_causal(args)
    elif args.workload == "triple":
        run_triple(args)
    elif args.workload == "causal_linear":
        run_causal_linear(args)
    elif args.workload == "sdpa_gpu":
        run_sdpa_gpu(args)
    elif args.workload == "cp_encoder":
        run_cp_encoder(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
