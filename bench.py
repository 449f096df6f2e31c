#!/usr/bin/env python
"""Benchmark of the hot path: forward + backward + optimizer step, samples/s.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c1|c2|c4|c5] [--impl ours|reference]

N > 1 is launched by `python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...`
(one rank per GPU; RANK / LOCAL_RANK / WORLD_SIZE from the environment).  Rank 0 prints ONE JSON
line.  Weak scaling: every rank processes the same per-GPU batch on its own shard of synthetic data
and the ranks exchange gradients with one NCCL all-reduce per step.

The default workload is the CNN training step (conv-relu-pool x2, two linear layers, log-softmax
NLL, Adam) at 256 samples per GPU; inputs are seeded synthetic tensors with MNIST's shapes and value
range, weights are Kaiming-uniform from a seed.

--impl reference times the CPU restatement of the reference's CPU backend (oracle/, single thread,
as the reference's ndarray/matrixmultiply build is) on the same workload.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (config id, dims, samples per step per GPU, description)
    "c3": (3, [256, 28, 32, 64, 128, 10], 256, "C3 CNN train step, 256x1x28x28 per GPU, Adam"),
    "c1": (1, [64, 784, 128, 10], 64, "C1 MLP train step, batch 64, Adam"),
    "c2": (2, [4096, 4096], 4096, "C2 elementwise/reduction forward+backward on X [4096,4096], b [4096] (no optimizer; a sample is a row)"),
    "c4": (4, [128, 64, 56, 128], 128, "C4 conv/conv-transpose train step, 128x64x56x56, MomentumSGD"),
    "c5": (5, [65, 512, 128, 64], 64, "C5 char-LSTM train step, T=128, batch 64 per GPU, Adam"),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for s in self.samples:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_step_time(config, dims, seed, steps):
    """Times `steps` training steps of the CPU oracle (single thread). Returns seconds per step."""
    import oracle
    from rusttensor_b200.workloads import setup_trainer, workload_data

    e = oracle.engine()
    params, inputs = workload_data(config, dims, seed)
    tr = setup_trainer(e, config, dims, params)
    ins = [e.tensor(a, requires_grad=(config == 4 and i == 0)) for i, a in enumerate(inputs)]
    tr.step(ins)  # warm-up (page faults, allocator)
    t0 = time.perf_counter()
    for _ in range(steps):
        loss = tr.step(ins)
    float(loss.numpy())
    return (time.perf_counter() - t0) / steps


def _cpu_worker(a):
    config, dims, steps = a
    return cpu_step_time(config, dims, 0, steps)


def cpu_all_cores(config, dims, per_gpu, steps):
    """Throughput of the host with every core busy: one independent single-thread replica of the CPU path per core, each
    running full-batch steps (the most generous reading of 'all cores': no exchange between the replicas is counted).
    NOT reference behaviour: the reference's ndarray / matrixmultiply build runs one thread."""
    import multiprocessing as mp

    procs = max(1, os.cpu_count() or 1)
    t0 = time.perf_counter()
    with mp.get_context("fork").Pool(procs) as pool:
        secs = pool.map(_cpu_worker, [(config, dims, steps)] * procs)
    wall = time.perf_counter() - t0
    return {"value": procs * per_gpu / max(secs), "unit": "samples/s", "cores": procs, "kind": "port",
            "sample": f"{procs} independent single-thread replicas x {steps} full-batch steps, slowest replica {max(secs) * 1e3:.0f} ms per step "
                      f"(wall {wall:.1f} s incl. start-up); not reference behaviour (the reference runs one thread)"}


# How the timed steps treat the L2 (part of `config`, identical in both arms so that the two lines describe one configuration)
L2_POLICY = {
    "c3": "no explicit flush: one step touches about 230 MB of device tensors (L2 is 126 MB) and steps run back to back",
    "c4": "no explicit flush: one step touches about 2 GB of device tensors (L2 is 126 MB) and steps run back to back",
    "c2": "no explicit flush: one pass touches about 1.5 GB of device tensors (L2 is 126 MB) and passes run back to back",
    "c5": "no explicit flush: one step touches several hundred MB of device tensors (L2 is 126 MB) and steps run back to back",
    "c1": "no explicit flush: the model and a batch fit the L2 (a launch-bound workload); steps run back to back",
}


def workload_config(desc, per_gpu, world, workload=None):
    cfg = {"workload": desc, "per_gpu_batch": per_gpu, "global_batch": per_gpu * world, "parallelism": f"dp{world}"}
    if workload is not None:
        cfg["l2"] = L2_POLICY[workload]
    return cfg


def run_reference(args, rank, world):
    """The reference arm: the reference's own CPU algorithm (oracle port) on the host cores."""
    if rank != 0:
        return
    config, dims, per_gpu, desc = WORKLOADS[args.workload]
    n_timed = max(1, min(args.steps, 20 if args.workload in ("c3", "c1") else 1))  # bounded: about 10-15 s of CPU work
    sec = cpu_step_time(config, dims, 0, n_timed)
    value = per_gpu / sec
    cpu = {"value": value, "unit": "samples/s", "cores": 1, "kind": "port",
           "sample": f"{n_timed} timed full-batch steps ({per_gpu} samples each) of the C++ restatement of the reference "
                     f"CPU backend; the Rust reference cannot be built here (no cargo/rustc); host has {os.cpu_count()} cores, "
                     "the reference's ndarray/matrixmultiply build is single-threaded"}
    line = {
        "impl": "reference", "metric": "train_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(desc, per_gpu, max(1, args.gpus), args.workload),
        "note": "CPU path of the reference, single host thread (as the reference is built); one process whatever --gpus says",
        "cpu_baseline": cpu,
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if args.workload in ("c3", "c1"):
        line["cpu_all_cores"] = cpu_all_cores(config, dims, per_gpu, max(2, n_timed // 4))
    print(json.dumps(line))


def _recorded_traffic(key):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of a kernel at a given shape, from the ncu
    captures summarised under profiles/ (profiles/roofline_traffic.json); None when no capture matches."""
    path = os.path.join(ROOT, "profiles", "roofline_traffic.json")
    try:
        return json.load(open(path)).get(key, {}).get("dram_bytes_per_launch")
    except (OSError, ValueError):
        return None


def _time_call(capi, call, flush, reps=20):
    """Mean CUDA-event time (seconds) of the kernels of `call` on the library's stream with a 256 MB L2 flush before every
    launch.  The call is captured once into a CUDA graph and the graph is replayed between the events, as the training step
    replays it: the host-side part of the call (argument checks, tensor-map encoding, workspace bookkeeping) is then
    outside the timed region and the events bracket device work only."""
    ms = C.c_float(0)
    for _ in range(3):
        call()
    graph = C.c_void_p()
    capi.call("graph_begin")
    call()
    capi.call("graph_end", C.byref(graph))
    for _ in range(2):
        capi.call("graph_launch", graph)
    times = []
    for _ in range(reps):
        capi.call("fill", flush.ptr, C.c_float(1.0), C.c_int64(flush.size))
        capi.call("timer_start")
        capi.call("graph_launch", graph)
        capi.call("timer_stop", C.byref(ms))
        times.append(ms.value)
    capi.call("graph_destroy", graph)
    return float(np.mean(times)) * 1e-3


def measure_dominant_kernel(rt, capi, config, dims, pk):
    """Times the convolution-gradient contractions of the step in isolation (CUDA events on the library's stream, L2
    flushed between launches) and reports each against the 3xTF32 tensor-core roofline: flops = 2*M*N*K of real
    multiply-adds, peak = measured bf16 burst / 6 (TF32 runs at half the bf16 rate, three MMAs per fp32 product).
    `roofline` is the dominant one (C3: the conv2 input+weight gradient pair, one rt_conv2d_backward call); `kernels`
    lists every contraction on its own."""
    i64, i32 = C.c_int64, C.c_int
    peak = pk["bf16"] / 6.0
    src = f"{pk['source']} bf16 burst {pk['bf16']} TFLOP/s / 6 (TF32 = bf16/2, three TF32 MMAs per fp32 product)"
    r = np.random.default_rng(0)
    dev = lambda *shape: capi.to_device(r.standard_normal(shape).astype(np.float32))
    flush = capi.empty((64 * 1024 * 1024,))  # 256 MB > 126 MB L2

    def conv_case(tag, n, cin, hw, cout):
        x, w, g = dev(n, cin, hw, hw), dev(cout, cin, 3, 3), dev(n, cout, hw, hw)
        dx, dw = capi.empty((n, cin, hw, hw)), capi.empty((cout, cin, 3, 3))
        mk = lambda pdx, pdw: (lambda: capi.call("conv2d_backward", x.ptr, w.ptr, g.ptr, i64(n), i64(cin), i64(hw), i64(hw), i64(cout),
                                                 i32(3), i32(3), i32(1), i32(1), i32(1), i32(1), pdx, pdw, None))
        fl = 2.0 * n * hw * hw * cout * cin * 9
        shape = f"n{n}_c{cin}_hw{hw}_k{cout}"
        byt_dx = 4.0 * (n * cout * hw * hw + cout * cin * 9 + n * cin * hw * hw)
        byt_dw = 4.0 * (n * cout * hw * hw + n * cin * hw * hw + cout * cin * 9)
        return [(f"{tag} input gradient", f"conv3x3_dx_{shape}", fl, byt_dx, mk(dx.ptr, None)),
                (f"{tag} weight gradient", f"conv3x3_dw_{shape}", fl, byt_dw, mk(None, dw.ptr)),
                (f"{tag} input+weight gradient (one call)", f"conv3x3_dxdw_{shape}", 2 * fl, byt_dx + byt_dw - 4.0 * n * cout * hw * hw,
                 mk(dx.ptr, dw.ptr))]

    def convt_case(tag, n, cin, hw, cout):  # k4 s2 p1: x [n,cin,hw,hw], w [cin,cout,4,4], g [n,cout,2hw,2hw]
        x, w, g = dev(n, cin, hw, hw), dev(cin, cout, 4, 4), dev(n, cout, 2 * hw, 2 * hw)
        dx, dw = capi.empty((n, cin, hw, hw)), capi.empty((cin, cout, 4, 4))
        mk = lambda pdx, pdw: (lambda: capi.call("conv2d_transpose_backward", x.ptr, w.ptr, g.ptr, i64(n), i64(cin), i64(hw), i64(hw),
                                                 i64(cout), i32(4), i32(4), i32(2), i32(2), i32(1), i32(1), pdx, pdw, None))
        fl = 2.0 * n * hw * hw * cin * cout * 16
        shape = f"n{n}_c{cin}_hw{hw}_k{cout}"
        byt = 4.0 * (n * cout * 4 * hw * hw + cin * cout * 16 + n * cin * hw * hw)
        return [(f"{tag} input gradient", f"convT4x4s2_dx_{shape}", fl, byt, mk(dx.ptr, None)),
                (f"{tag} weight gradient", f"convT4x4s2_dw_{shape}", fl, byt, mk(None, dw.ptr))]

    if config == 3:
        n, hw, c1, c2 = dims[0], dims[1] // 2, dims[2], dims[3]
        cases = conv_case("conv2", n, c1, hw, c2)
        dominant = 2
    elif config == 4:
        n, cin, hw, cout = dims
        cases = conv_case("conv", n, cin, hw, cout)[:2] + convt_case("conv-transpose", n, cout, hw // 2, cin)
        dominant = None  # the slowest of the four
    else:
        return None
    kernels = []
    for name, key, flops, nbytes, call in cases:
        t = _time_call(capi, call, flush)
        achieved = flops / t / 1e12
        kernels.append({"bound": "tensor", "kernel": name, "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                        "traffic": _recorded_traffic(key), "traffic_unit": "bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum, ncu)",
                        "algorithmic_bytes": nbytes, "gflop": flops / 1e9, "avg_launch_ms": t * 1e3, "peak_source": src})
    if dominant is None:
        dominant = int(np.argmax([k["avg_launch_ms"] for k in kernels]))
    roof = dict(kernels[dominant])
    roof["kernels"] = [k for i, k in enumerate(kernels) if i != dominant]
    return roof


def mma_rate_table(capi, iters=512):
    """Cycles one tcgen05.mma.kind::tf32 (K = 8) occupies the tensor pipe, by M, N and source of the A operand
    (shared memory or tensor memory), with the fraction of the full rate (2048 multiply-adds per cycle per SM)."""
    out = []
    for m in (128, 64):
        for a_in_tmem in (0, 1):
            for n in (32, 64, 96, 128, 160, 192, 224, 256):
                issue, done = C.c_double(0), C.c_double(0)
                capi.call("tc_issue_rate", C.c_int(m), C.c_int(n), C.c_int(a_in_tmem), C.c_int(iters), C.byref(issue), C.byref(done))
                out.append({"M": m, "N": n, "A": "tmem" if a_in_tmem else "smem", "issue_cycles": round(issue.value, 1),
                            "cycles_per_mma": round(done.value, 1), "frac_of_full_rate": round(m * n * 8 / 2048.0 / done.value, 3)})
    return out


def data_parallel_check(rt, dist, config, dims, rank, world, local_rank, nccl_id, trainer_config, trained):
    """Correctness evidence for the multi-GPU step, run after the timed region on every rank:
    (1) the replicas trained by the benchmark hold bit-identical parameters (compared as 32-bit patterns: an all-reduce
        MAX must equal an all-reduce MIN);
    (2) a fresh data-parallel trainer, three steps on per-rank shards, ends within 1e-4 (the parity tolerance, with the
        5e-4 * lr floor the tests use after an Adam step) of one GPU trained on the concatenated batch.
    Returns a dict for the `dp_check` key; `ok` is true only if both hold."""
    import torch

    from rusttensor_b200.workloads import workload_data

    flat = np.concatenate([t.numpy().ravel() for t in trained.params]).view(np.int32)
    hi = torch.from_numpy(flat.copy()).to("cuda" if dist.get_backend() == "nccl" else "cpu")
    lo = hi.clone()
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    identical = bool(torch.equal(hi, lo))
    if config not in (1, 3):
        # C5 clips every rank's gradient before the exchange (clip, all-reduce, Adam), which one GPU on the joint batch
        # does not reproduce; C2 / C4 are single-GPU workloads
        return {"ok": identical, "replicas_bit_identical": identical, "joint_batch_within_tolerance": None,
                "what": "params after the benchmark compared across ranks as bit patterns; the joint-batch comparison only exists for C1 / C3"}
    # (2) one step of a fresh data-parallel trainer against one GPU on the joint batch.  Compared: Adam's first and second
    # moments after the step - (1 - beta) * g and (1 - beta) * g^2, i.e. the exchanged gradient itself - within the parity
    # tolerance, and the parameters within one Adam step (Adam divides by sqrt(v) + eps, so an element whose gradient is a
    # near-zero sum may move by up to lr in either direction for any summation order; the moments are the sharp test).
    small = list(dims)
    small[0] = max(4, small[0] // 8)
    dp = rt.DataParallelTrainer(trainer_config, small, rank=rank, world=world, nccl_id=nccl_id, device=local_rank)
    if os.environ.get("RT_B200_DP_FUSED", "0") == "1":
        if not dp.connect_peers(dist):
            dp = rt.DataParallelTrainer(trainer_config, small, rank=rank, world=world, nccl_id=nccl_id, device=local_rank)
    params, _ = workload_data(config, small, seed=0)
    for t, p in zip(dp.params, params):
        t.update_from_host(p)
    dp.step(workload_data(config, small, seed=100, rank=rank)[1])
    dp.last_loss()
    n = len(dp.params)
    got = {"m": [dp.state(0, i).numpy() for i in range(n)], "v": [dp.state(1, i).numpy() for i in range(n)], "p": [t.numpy() for t in dp.params]}
    worst, ok2 = 0.0, True
    if rank == 0:
        joint = list(small)
        joint[0] *= world
        one = rt.DataParallelTrainer(trainer_config, joint, device=local_rank)
        for t, p in zip(one.params, params):
            t.update_from_host(p)
        shards = [workload_data(config, small, seed=100, rank=r)[1] for r in range(world)]
        one.step([np.concatenate([sh[i] for sh in shards], axis=0) for i in range(len(shards[0]))])
        one.last_loss()
        ref = {"m": [one.state(0, i).numpy() for i in range(n)], "v": [one.state(1, i).numpy() for i in range(n)], "p": [t.numpy() for t in one.params]}
        lr = 1e-3
        for key in ("m", "v", "p"):
            for a, b in zip(got[key], ref[key]):
                a64, b64 = a.astype(np.float64), b.astype(np.float64)
                scale = float(np.max(np.abs(b64))) if b64.size else 0.0
                bound = 1e-4 * np.maximum(np.abs(a64), np.abs(b64)) + (2e-6 if key != "p" else 0.0) * scale + (2.1 * lr if key == "p" else 0.0)
                err = np.abs(a64 - b64)
                ok2 = ok2 and bool(np.all(err <= bound))
                if key != "p" and err.size:
                    worst = max(worst, float(np.max(err / np.maximum(bound, 1e-30))))
    flag = torch.tensor([1 if ok2 else 0], dtype=torch.int32, device="cuda" if dist.get_backend() == "nccl" else "cpu")
    dist.broadcast(flag, 0)
    return {"ok": bool(identical and flag.item() == 1), "replicas_bit_identical": identical, "joint_batch_within_tolerance": bool(flag.item() == 1),
            "worst_moment_error_over_bound": worst, "per_gpu_batch_of_check": small[0],
            "what": "params after the benchmark compared across ranks as bit patterns; one step of a fresh data-parallel run compared with one "
                    "GPU on the concatenated batch: Adam moments (= the exchanged gradient) within 1e-4 relative + 2e-6 of the tensor scale, "
                    "parameters within one Adam step"}


def kernel_bandwidth_table(capi, pk, rows=4096, cols=4096):
    """Times the HBM-bound kernels of the path one by one at the shapes of the element-wise / reduction
    micro-benchmark (X [rows,cols], b [cols]).  Bytes are the algorithmic ones: 4 x (elements of each distinct operand
    read at its un-broadcast size + elements written).

    `ms`: every kernel is given `sets` distinct sets of operands (together several times the 126 MB L2, so each launch
    finds its inputs in HBM only); one launch per set is captured into a CUDA graph - the way the training step issues
    its kernels - and the graph is replayed three times between two CUDA events on the library's stream; the time is divided
    by the number of launches.  `ms_single_launch`: one eager launch between two events after a 256 MB L2 flush; this
    includes the event pair's own cost, which the row "tiny launch" shows (a one-element fill measured the same two ways)."""
    from rusttensor_b200.capi import BINARY, REDUCE, UNARY

    r = np.random.default_rng(0)
    n = rows * cols
    sets = 8 if n <= 4096 * 4096 else 4
    host = lambda *shape: r.standard_normal(shape).astype(np.float32)
    hx, hg, ha = host(rows, cols), host(rows, cols), host(rows, cols)
    S = []
    for _ in range(sets):
        S.append(dict(X=capi.to_device(hx), G=capi.to_device(hg), A=capi.to_device(ha), D1=capi.empty((rows, cols)), D2=capi.empty((rows, cols)),
                      m=capi.to_device(np.zeros((rows, cols), np.float32)), v=capi.to_device(np.zeros((rows, cols), np.float32))))
    bvec = capi.to_device(host(cols))
    grow = capi.to_device(host(rows))
    dcol, drow = capi.empty((cols,)), capi.empty((rows,))
    pn, pc, ph = 256, 32, 28
    hpg, hpi = host(pn, pc, ph // 2, ph // 2), r.integers(0, 4, (pn, pc, ph // 2, ph // 2)).astype(np.float32)
    P = [dict(g=capi.to_device(hpg), idx=capi.to_device(hpi), dx=capi.empty((pn, pc, ph, ph))) for _ in range(sets)]
    one = capi.empty((4,))
    i64, f32, i32 = C.c_int64, C.c_float, C.c_int
    sh2, sh1 = capi.i64([rows, cols]), capi.i64([cols])
    cases = [
        ("tiny launch (fill of one element)", 0.0, lambda b: capi.call("fill", one.ptr, f32(1.0), i64(1))),
        ("unary_backward tanh", 12.0 * n,
         lambda b: capi.call("unary_backward", i32(UNARY["tanh"]), S[b]["X"].ptr, S[b]["G"].ptr, S[b]["D1"].ptr, i64(n), f32(0), f32(0))),
        ("unary exp (forward)", 8.0 * n, lambda b: capi.call("unary", i32(UNARY["exp"]), S[b]["X"].ptr, S[b]["D1"].ptr, i64(n), f32(0), f32(0))),
        ("binary_backward mul [R,C]*[C] (fused column sum)", 4.0 * (3 * n + 2 * cols),
         lambda b: capi.call("binary_backward", i32(BINARY["mul"]), S[b]["X"].ptr, sh2, i32(2), bvec.ptr, sh1, i32(1), S[b]["G"].ptr, S[b]["D1"].ptr,
                             dcol.ptr)),
        ("binary_backward mul same shape", 20.0 * n,
         lambda b: capi.call("binary_backward", i32(BINARY["mul"]), S[b]["X"].ptr, sh2, i32(2), S[b]["A"].ptr, sh2, i32(2), S[b]["G"].ptr,
                             S[b]["D1"].ptr, S[b]["D2"].ptr)),
        ("reduce sum along rows' axis 1", 4.0 * (n + rows),
         lambda b: capi.call("reduce", i32(REDUCE["sum"]), S[b]["X"].ptr, i64(rows), i64(cols), i64(1), drow.ptr)),
        ("reduce sum along axis 0", 4.0 * (n + cols),
         lambda b: capi.call("reduce", i32(REDUCE["sum"]), S[b]["X"].ptr, i64(1), i64(rows), i64(cols), dcol.ptr)),
        ("logsumexp axis 1 (forward)", 4.0 * (n + rows),
         lambda b: capi.call("reduce", i32(REDUCE["logsumexp"]), S[b]["X"].ptr, i64(rows), i64(cols), i64(1), drow.ptr)),
        ("logsumexp backward", 4.0 * (2 * n + rows),
         lambda b: capi.call("reduce_backward", i32(REDUCE["logsumexp"]), S[b]["X"].ptr, grow.ptr, i64(rows), i64(cols), i64(1), S[b]["D1"].ptr)),
        ("log_softmax backward", 12.0 * n,
         lambda b: capi.call("log_softmax_backward", S[b]["X"].ptr, S[b]["G"].ptr, i64(rows), i64(cols), i64(1), S[b]["D1"].ptr)),
        ("max_pool2d backward 2x2 [256,32,28,28]", 4.0 * (2 * hpg.size + pn * pc * ph * ph),
         lambda b: capi.call("max_pool2d_backward", P[b]["g"].ptr, P[b]["idx"].ptr, i64(pn), i64(pc), i64(ph), i64(ph), i32(2), i32(2), i32(2),
                             i32(2), i32(0), i32(0), P[b]["dx"].ptr)),
        ("adam step, %.1f M parameters" % (n / 1e6), 28.0 * n,
         lambda b: capi.call("adam_step", S[b]["A"].ptr, S[b]["G"].ptr, S[b]["m"].ptr, S[b]["v"].ptr, i64(n), f32(1e-3), f32(0.9), f32(0.999),
                             f32(1e-8), i64(1))),
    ]
    flush = capi.empty((64 * 1024 * 1024,))
    flush_sum = capi.empty((1,))
    ms = C.c_float(0)
    replays = 3
    out = []
    for name, nbytes, call in cases:
        for b in range(sets):
            call(b)
        graph = C.c_void_p()
        capi.call("graph_begin")
        for b in range(sets):
            call(b)
        capi.call("graph_end", C.byref(graph))
        capi.call("graph_launch", graph)
        rounds = []
        for _ in range(5):
            capi.call("timer_start")
            for _ in range(replays):
                capi.call("graph_launch", graph)
            capi.call("timer_stop", C.byref(ms))
            rounds.append(ms.value / (replays * sets))
        capi.call("graph_destroy", graph)
        singles = []
        for i in range(10):
            # L2 flush: write 256 MB, then read it back so that the dirty lines are written out before the timed
            # launch instead of during it
            capi.call("fill", flush.ptr, C.c_float(1.0), C.c_int64(flush.size))
            capi.call("reduce", i32(REDUCE["sum"]), flush.ptr, i64(1), i64(flush.size), i64(1), flush_sum.ptr)
            capi.call("timer_start")
            call(i % sets)
            capi.call("timer_stop", C.byref(ms))
            singles.append(ms.value)
        t = float(np.median(rounds)) * 1e-3
        gbs = nbytes / t / 1e9
        out.append({"kernel": name, "ms": t * 1e3, "ms_single_launch": float(np.mean(singles)), "algorithmic_MB": nbytes / 1e6, "GB/s": gbs,
                    "frac_of_measured_hbm": gbs / pk["hbm"], "frac_of_8TBs": gbs / 8000.0, "operand_sets": sets})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--fused-forward", action="store_true",
                    help="build the network from the fused forward ops (relu + max_pool2d in one kernel, the LSTM cell in two, the classification loss "
                         "in one kernel) instead of the reference's op sequence; same mathematics")
    ap.add_argument("--kernels-size", type=int, default=4096, help="rows = cols of the matrices of --kernels")
    ap.add_argument("--kernels", action="store_true",
                    help="print the bandwidth table of the HBM-bound kernels (one GPU) instead of the training-step line")
    ap.add_argument("--repeats", type=int, default=5,
                    help="how many times the --steps-long timed region is measured; the line reports the median region and the spread")
    ap.add_argument("--conv-kernels", default=None, metavar="N,CIN,HW,COUT",
                    help="run rt_conv2d_backward (3x3, stride 1, padding 1; dx, dw and db) a few times on this shape and exit: the small, "
                         "self-contained command the ncu captures of the convolution-gradient kernels are taken on")
    ap.add_argument("--steps-only", type=int, default=0, metavar="N",
                    help="run N captured training steps of --workload (with --fused-forward: its fused variant) and exit: the small command "
                         "the per-step kernel listing is captured on")
    ap.add_argument("--mma-rate", action="store_true",
                    help="print the issue-rate table of tcgen05.mma.kind::tf32 (cycles per MMA by shape and A-operand source)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.warmup < 3:
        args.warmup = 3

    import rusttensor_b200 as rt
    from rusttensor_b200.workloads import workload_data

    if args.conv_kernels:
        if rank == 0:
            rt.init(local_rank)
            capi = rt.CApi(ctx=rt.context_handle())
            n, cin, hw, cout = [int(v) for v in args.conv_kernels.split(",")]
            r = np.random.default_rng(1)
            x = capi.to_device(r.standard_normal((n, cin, hw, hw)).astype(np.float32))
            w = capi.to_device(r.standard_normal((cout, cin, 3, 3)).astype(np.float32))
            g = capi.to_device(r.standard_normal((n, cout, hw, hw)).astype(np.float32))
            dx, dw, db = capi.empty((n, cin, hw, hw)), capi.empty((cout, cin, 3, 3)), capi.empty((cout,))
            for _ in range(3):
                capi.call("conv2d_backward", x.ptr, w.ptr, g.ptr, C.c_int64(n), C.c_int64(cin), C.c_int64(hw), C.c_int64(hw), C.c_int64(cout),
                          C.c_int(3), C.c_int(3), C.c_int(1), C.c_int(1), C.c_int(1), C.c_int(1), dx.ptr, dw.ptr, db.ptr)
            capi.sync()
            print(json.dumps({"conv_kernels": args.conv_kernels, "calls": 3, "checksum_dw": float(np.abs(dw.numpy()).sum())}))
        return
    if args.steps_only:
        # a few captured training steps and nothing else: the command the per-step kernel listing (ncu launch list with
        # --cache-control none) is taken on; the last `nodes` launches of the capture are one whole step in order
        if rank == 0:
            config, dims, per_gpu, desc = WORKLOADS[args.workload]
            tr = rt.DataParallelTrainer(config + (100 if args.fused_forward else 0), dims, device=local_rank)
            params, inputs = workload_data(config, dims, seed=0)
            for t, p in zip(tr.params, params):
                t.update_from_host(p)
            for _ in range(2):
                tr.step(inputs)
            tr.last_loss()
            for _ in range(args.steps_only):
                tr.step(None)
            print(json.dumps({"steps_only": args.steps_only, "workload": desc, "loss": tr.last_loss(), "kernels_per_step": tr.graph_nodes()}))
        return
    if args.mma_rate:
        if rank == 0:
            rt.init(local_rank)
            print(json.dumps({"mma_rate": mma_rate_table(rt.CApi(ctx=rt.context_handle()))}))
        return
    if args.kernels:
        if rank == 0:
            rt.init(local_rank)
            pk = peaks()
            table = kernel_bandwidth_table(rt.CApi(ctx=rt.context_handle()), pk, args.kernels_size, args.kernels_size)
            print(json.dumps({"kernel_bandwidth": table, "hbm_peak_GBs": pk["hbm"], "peak_source": pk["source"],
                              "l2": "ms: launches cycle over distinct operand sets several times the L2 in total; ms_single_launch: 256 MB fill, then a "
                                    "read of the same 256 MB, before every timed launch",
                              "rows": args.kernels_size, "cols": args.kernels_size}))
        return
    config, dims, per_gpu, desc = WORKLOADS[args.workload]
    dist = None
    nccl_id = None
    if world > 1 or os.environ.get("RT_BENCH_FORCE_DIST") == "1":  # the second: a diagnostic (one rank with a process group)
        import torch
        import torch.distributed as dist

        from rusttensor_b200 import dp_setup

        # The process group only carries the set-up (communicator id, peer-memory handles, agreement checks), the barriers
        # around the timed regions and the max over the ranks: gloo by default.  Measured on B200s: after a few NCCL barriers of
        # torch's own communicator every later training step of the process ran 15 us slower (0.249 -> 0.264 ms, one rank, no
        # exchange at all); gloo barriers leave the step alone.  The gradient exchange itself never goes through this group: it
        # is the library's peer-memory kernels or its own NCCL communicator.  RT_BENCH_PG=nccl selects torch's NCCL group.
        pg_backend = os.environ.get("RT_BENCH_PG", "gloo")
        torch.cuda.set_device(local_rank)
        if pg_backend == "nccl":
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        else:
            dist.init_process_group(pg_backend)
        ddev = "cuda" if pg_backend == "nccl" else "cpu"
        nccl_id = dp_setup.share_unique_id(dist, rt.DataParallelTrainer.unique_id, rank, device=ddev)

    trainer_config = config + (100 if args.fused_forward else 0)
    if args.fused_forward:
        desc += " [fused forward ops]"
    uncoupled = world > 1 and os.environ.get("RT_BENCH_UNCOUPLED") == "1"
    if uncoupled:
        # diagnostic: the N processes train independent replicas (no gradient exchange); shows what the exchange costs
        tr = rt.DataParallelTrainer(trainer_config, dims, rank=0, world=1, device=local_rank)
    else:
        tr = rt.DataParallelTrainer(trainer_config, dims, rank=rank, world=world, nccl_id=nccl_id, device=local_rank)
    capi = rt.CApi(ctx=rt.context_handle())
    exchange = "one NCCL all-reduce of the flat gradients (N>1)"
    if uncoupled:
        exchange = "NONE (RT_BENCH_UNCOUPLED=1: independent replicas, a diagnostic and not a data-parallel run)"
    elif world > 1 and os.environ.get("RT_B200_DP_FUSED", "0") == "1":
        # RT_B200_DP_FUSED=1: the gradients are read from the peers' buffers inside the optimizer kernel and the whole step -
        # exchange included - is one CUDA-graph launch.  Default: one NCCL all-reduce between the graph and an eager optimizer
        # launch, which measured faster on this model's 1.7 MB of gradients (eight B200s: 0.288 against 0.297 ms per step;
        # two: 0.270 against 0.273).  Every rank must agree on the mode, so a set-up failure on any rank sends all of them to NCCL
        if tr.connect_peers(dist):
            exchange = "gradient exchange over peer memory fused into the optimizer kernel (N>1)"
        else:
            print(f"[rank {rank}] peer-memory exchange unavailable ({getattr(tr, 'peer_error', 'another rank failed')}); using NCCL",
                  file=sys.stderr)
            tr = rt.DataParallelTrainer(trainer_config, dims, rank=rank, world=world, nccl_id=nccl_id, device=local_rank)
    if world > 1 and not uncoupled:
        # every rank must have built the same model before the first exchange: raises on all ranks otherwise
        dp_setup.agree(dist, "the model (flat gradient length, number of parameter tensors)", [tr.flat_len, len(tr.params)], device=ddev)
    params, inputs = workload_data(config, dims, seed=0, rank=rank)  # same weights on every rank, different data
    for t, p in zip(tr.params, params):
        t.update_from_host(p)
    for i, a in enumerate(inputs):
        tr.pinned_input(i)[...] = a
    h2d = int(sum(a.nbytes for a in inputs))

    def barrier():
        capi.sync()
        if dist is not None:
            dist.barrier()
        capi.sync()

    # warm-up: the first step runs eagerly inside capture(); then replays
    l0 = capi.launches()
    tr.step(inputs)
    tr.last_loss()
    # kernels recorded in the graph; with the NCCL exchange the optimizer launch of that first step was eager (the all-reduce is
    # NCCL's kernel, not counted)
    eager_update = (world > 1 and not uncoupled and "peer memory" not in exchange and os.environ.get("RT_B200_DP_NCCL_GRAPH") != "1")
    launches_per_replay = capi.launches() - l0 - (1 if eager_update else 0)
    for _ in range(args.warmup):
        tr.step(None)
    barrier()

    def timed(fn, k, repeats=1):
        """`repeats` timed regions of k calls each, every region bracketed by barrier + synchronize on both sides and
        timed with CUDA events on the library's stream; per region the maximum over the ranks.  Returns the list."""
        out = []
        for _ in range(repeats):
            ms = C.c_float(0)
            barrier()
            capi.call("timer_start")
            for _ in range(k):
                fn()
            capi.call("timer_stop", C.byref(ms))
            barrier()
            v = ms.value
            if dist is not None:
                import torch

                tt = torch.tensor([v], device=ddev)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                v = float(tt.item())
            out.append(v)
        return out

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    lb = capi.launches()
    fused_exchange = world > 1 and exchange.startswith("gradient exchange over peer memory")
    wait0 = tr.peer_wait_ns if fused_exchange else 0
    regions = timed(lambda: tr.step(None), args.steps, repeats=args.repeats)  # each region is exactly --steps steps
    trace = None
    if os.environ.get("RT_B200_DP_TRACE") == "1":
        ts = tr.trace()
        names = ["begin->forward", "forward->backward", "backward->packed", "packed->peers complete", "peers complete->optimizer done"]
        idx = [(0, 1), (1, 2), (2, 3), (3, 4), (4, 6)] if fused_exchange else [(0, 1), (1, 2), None, None, (2, 6)]
        trace = {n: round((ts[b] - ts[a]) / 1e3, 2) for n, ab in zip(names, idx) if ab for a, b in [ab]}
        trace["note"] = "last step of this rank, GPU nanosecond timer, microseconds; each stamp is a one-thread kernel of its own"
    peer_wait = None
    if fused_exchange:
        # diagnostic: how long each rank's one-block wait kernel polled for its peers per step (device clock), all ranks
        import torch

        mine = torch.tensor([(tr.peer_wait_ns - wait0) / (args.steps * args.repeats) / 1e3], device=ddev)
        allw = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allw, mine)
        peer_wait = {"us_per_step_by_rank": [round(float(t.item()), 2) for t in allw],
                     "what": "time the wait kernel of each rank polled for the peers' flags, per step"}
    gpu_launches = (capi.launches() - lb) // args.repeats + launches_per_replay * args.steps  # per region
    clocks = sampler.stop() if rank == 0 else None
    ms_resident = float(np.median(regions))

    # End to end through the trainer's public API: every step uploads its inputs from pinned host memory and the
    # host reads every step's loss.  The trainer pipelines: while step i runs on the device the host already hands
    # over the buffers of step i+1 (their upload overlaps step i) and reads the loss of step i-1; the last loss is
    # read by pipeline_flush() inside the timed region.
    # Every step gets its own batch: eight distinct batches (this rank's shard) are cycled through, each copied into
    # the pinned buffer the trainer hands out before the step is submitted, as a data loader would.
    # (Workloads whose batch exceeds 16 MB keep one batch: copying 200 MB per step on the host would measure memcpy.)
    many = bool(inputs) and h2d <= (16 << 20)
    host_batches = [inputs] + ([workload_data(config, dims, seed=1000 + k, rank=rank)[1] for k in range(7)] if many else [])
    for k in range(2):  # fill both pinned buffer pairs, untimed
        for i, a in enumerate(host_batches[k % len(host_batches)]):
            tr.pipeline_buffer(i)[...] = a
        tr.step_pipelined()
    tr.pipeline_flush()
    losses = []
    e2e_count = [0]

    def e2e_step():
        batch = host_batches[e2e_count[0] % len(host_batches)]
        e2e_count[0] += 1
        for i, a in enumerate(batch):
            buf = tr.pipeline_buffer(i)           # the pinned buffer of this step
            if many:
                np.copyto(buf, a)                 # filled with this step's batch
        losses.append(tr.step_pipelined())  # H2D, graph, all-reduce, optimizer, D2H of the loss; returns the previous loss

    def e2e_all(k):
        for _ in range(k):
            e2e_step()
        losses.append(tr.pipeline_flush())

    ms_e2e = float(np.median(timed(lambda: e2e_all(args.steps), 1, repeats=min(3, args.repeats))))
    loss = losses[-1]
    code = C.c_int(0)
    capi.call("device_status", C.byref(code))  # raises if a bounded device-side wait (MMA pipeline, peer flags) expired

    # The data set resident on the device (data::get_random_batch without its host round trip): per step the host draws
    # the batch's row numbers and uploads those (4 bytes per sample); the rows are gathered on the device.
    dataset_line = None
    if config in (1, 3) and os.environ.get("RT_BENCH_SKIP_DATASET") != "1":
        try:
            n_rows = 16 * per_gpu
            parts = [workload_data(config, dims, seed=2000 + k, rank=rank)[1] for k in range(16)]
            tr.attach_dataset([np.concatenate([p_[i] for p_ in parts], axis=0) for i in range(len(inputs))])
            r_idx = np.random.default_rng(rank)
            tr.step_dataset(r_idx.choice(n_rows, per_gpu, replace=False))
            tr.pipeline_flush()

            def ds_all(k):
                for _ in range(k):
                    tr.step_dataset(r_idx.choice(n_rows, per_gpu, replace=False))
                tr.pipeline_flush()

            ms_ds = float(np.median(timed(lambda: ds_all(args.steps), 1, repeats=min(3, args.repeats))))
            dataset_line = {"value": per_gpu * world * args.steps / (ms_ds * 1e-3), "unit": "samples/s", "ms_per_step": ms_ds / args.steps,
                            "h2d_bytes_per_step": 4 * per_gpu * world, "d2h_bytes_per_step": 4 * world, "dataset_rows_per_gpu": n_rows,
                            "note": "data set resident on the device; the host samples the batch's rows without replacement and uploads the row "
                                    "numbers, the batch is gathered on the device (rt_gather_rows); every loss read on the host"}
        except Exception as e:  # noqa: BLE001  (the headline does not depend on this extra measurement)
            dataset_line = {"unavailable": str(e)}

    # The same network built from the fused forward ops (relu + max_pool2d and the classification loss as single
    # kernels), timed the same way on device-resident inputs; reported beside the headline, which keeps the reference's
    # own op sequence.
    fused_line = None
    if not args.fused_forward and config in (1, 3, 4, 5) and os.environ.get("RT_BENCH_SKIP_FUSED") != "1":
        try:
            tr2 = rt.DataParallelTrainer(config + 100, dims, rank=rank, world=world, nccl_id=nccl_id, device=local_rank)
            for t, p in zip(tr2.params, params):
                t.update_from_host(p)
            tr2.step(inputs)
            tr2.last_loss()
            for _ in range(args.warmup):
                tr2.step(None)
            ms2 = float(np.median(timed(lambda: tr2.step(None), args.steps, repeats=min(3, args.repeats))))
            fused_line = {"value": per_gpu * world * args.steps / (ms2 * 1e-3), "unit": "samples/s", "ms_per_step": ms2 / args.steps,
                          "note": "same network from the fused forward ops (ops::fused_conv2d_relu_max_pool2d, ops::fused_relu_max_pool2d, ops::fused_softmax_nll, ops::fused_lstm_cell_c/_h)"}
            del tr2
        except Exception as e:  # noqa: BLE001  (the headline above does not depend on this extra measurement)
            fused_line = {"unavailable": str(e)}

    if world == 1:
        step_text = "one CUDA-graph launch per step: forward, backward and the fused optimizer step (step count read on the device)"
    elif "peer memory" in exchange:
        step_text = ("one CUDA-graph launch per step: forward, backward, pack of the gradients, signal to / bounded wait for the peers, "
                     "optimizer kernel that reads every rank's gradients over NVLink (no all-reduce call)")
    elif os.environ.get("RT_B200_DP_NCCL_GRAPH") == "1":
        step_text = ("one CUDA-graph launch per step: forward, backward, pack of the gradients, NCCL all-reduce and the fused optimizer step "
                     "(step count read on the device) all recorded in the graph")
    else:
        step_text = f"CUDA-graph replay of forward+backward, {exchange}, one fused optimizer launch"
    dp_check = data_parallel_check(rt, dist, config, dims, rank, world, local_rank, nccl_id, trainer_config, tr) if world > 1 and not uncoupled else None

    if rank == 0:
        pk = peaks()
        res, in_use, nalloc = C.c_int64(0), C.c_int64(0), C.c_int64(0)
        capi.call("mem_stats", C.byref(res), C.byref(in_use), C.byref(nalloc))
        roof = measure_dominant_kernel(rt, capi, config, dims, pk)
        cpu = None
        if not args.no_cpu_baseline and world == 1:  # reported on the single-GPU run only
            steps_cpu = 15 if args.workload in ("c3", "c1") else 1
            sec = cpu_step_time(config, dims, 0, steps_cpu)
            cpu = {"value": per_gpu / sec, "unit": "samples/s", "cores": 1, "kind": "port",
                   "sample": f"{steps_cpu} full-batch steps ({per_gpu} samples each) of the C++ restatement of the reference CPU "
                             f"backend, single thread (as the reference builds ndarray/matrixmultiply); host has {os.cpu_count()} cores"}
        total = per_gpu * world
        line = {
            "metric": "train_samples_per_s", "value": total * args.steps / (ms_resident * 1e-3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_resident / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(desc, per_gpu, world, args.workload),
            "step_structure": step_text, "device_bytes_in_use": int(in_use.value),
            "e2e": {"value": total * args.steps / (ms_e2e * 1e-3), "unit": "samples/s", "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": 4 * world,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": int(gpu_launches), "final_loss": loss, "clocks": clocks,
            "peer_wait": peer_wait, "step_trace": trace,
            "timed_regions": {"n": len(regions), "steps_each": args.steps, "ms_per_step_median": ms_resident / args.steps,
                              "ms_per_step_min": min(regions) / args.steps, "ms_per_step_max": max(regions) / args.steps},
        }
        if dp_check:
            line["dp_check"] = dp_check
        if fused_line:
            line["fused_forward"] = fused_line
        if dataset_line:
            line["e2e_device_dataset"] = dataset_line
        if roof:
            line["roofline"] = roof
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
