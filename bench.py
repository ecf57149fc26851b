#!/usr/bin/env python
"""Benchmark of the NF4 quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (the configuration the headline metric is quoted on): the QLoRA decode GEMV
y = x W^T + s (x A^T) B^T with x bf16 [M, 4096] for M in {1, 4, 16}, W NF4 [11008, 4096]
(block 64, f32 absmax, N(0, 0.02^2)), LoRA rank 16 (A, B ~ N(0, 0.01^2)), s = 2.0.
One step = the three M passes.  Inputs are seeded synthetic data of those shapes.

`value` is the effective HBM bandwidth: algorithmic bytes of the three passes (packed
nibbles + absmax + A + B + x + y) divided by device time, with everything resident in HBM;
eight distinct weight copies (207 MB, larger than the 126 MB L2) are rotated per PASS, so every
pass streams its weight from HBM (a copy comes round again after seven other copies, 181 MB).  `e2e` is the same metric through the host-pointer C ABI
(pinned host x in, host y out, copies inside the timed region).

With N > 1 (torchrun) every rank owns one [11008, 4096] column shard of an N-times wider
layer and the ranks all-gather the step's outputs over NCCL, one collective per step on its
own stream beside the next step's passes (weak scaling).  The line then also carries the two
configurations that are sharded by definition, driven through ShardedNf4Linear and checked
against the unsharded forward on every rank: `prefill_sharded` (W [14336, 4096] split by output
columns, all-gather of y) and `qwen2_7b_block_sharded` (the seven projections of the block).

`--impl reference` times the reference's CPU algorithm for the same step on the host cores:
dequantize the packed weight to f32 (single-threaded scalar loop, as the reference's
PackedNf4Tensor::dequantize), then f32 matmuls on all cores (torch stands in for
burn-ndarray's matrixmultiply), as Nf4Linear::forward / QloraLinear::forward do.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

K, N, RANK, SCALE = 4096, 11008, 16, 2.0
MS = (1, 4, 16)
N_COPIES = 8
METRIC = "nf4_qlora_decode_effective_hbm_bandwidth"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0


def algorithmic_bytes(m: int) -> int:
    """Bytes one decode pass must move: packed codes, absmax, A, B, x, y (bf16 in/out)."""
    return N * K // 2 + N * K // 64 * 4 + RANK * K * 2 + N * RANK * 2 + m * K * 2 + m * N * 2


STEP_BYTES = sum(algorithmic_bytes(m) for m in MS)
WORKLOAD = ("QLoRA decode GEMV: x bf16 [M in {1,4,16}, 4096], W NF4 [11008, 4096] block 64 "
            "f32 absmax, LoRA rank 16, scale 2.0; one step = the three M passes")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def usable_cores() -> int:
    """Host cores this process may really use: the affinity mask, capped by a cgroup CPU quota."""
    try:
        n = len(os.sched_getaffinity(0))
    except Exception:
        n = os.cpu_count() or 1
    for path in ("/sys/fs/cgroup/cpu.max", "/sys/fs/cgroup/cpu/cpu.cfs_quota_us"):
        try:
            with open(path) as f:
                parts = f.read().split()
            if path.endswith("cpu.max"):
                if parts[0] != "max":
                    n = min(n, max(1, int(float(parts[0]) / float(parts[1]) + 0.5)))
            else:
                quota = int(parts[0])
                if quota > 0:
                    with open("/sys/fs/cgroup/cpu/cpu.cfs_period_us") as f:
                        n = min(n, max(1, int(quota / int(f.read().split()[0]) + 0.5)))
            break
        except Exception:
            continue
    return max(1, n)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the bench runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        mhz, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                mhz.append(float(r[0]))
                mx = float(r[1])
                for name, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        if not mhz:
            return {"sm_mhz": None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": 0}
        busy = [m for m in mhz if m >= 0.5 * max(mhz)]
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


# --------------------------------------------------------------------------- reference arm
def cpu_reference_setup(seed: int = 2):
    """Seeded config-2 inputs on the host, quantized by the CPU oracle."""
    import torch
    from oracle import nf4_oracle as o

    o.build()
    torch.set_num_threads(min(usable_cores(), 64))
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(N * K) * 0.02).astype(np.float32)
    packed, absmax = o.quantize_packed(w)
    rng = np.random.default_rng(3)
    a = o.round_bf16(rng.standard_normal((K, RANK)) * 0.01)   # reference shape A [d_in, r]
    b = o.round_bf16(rng.standard_normal((RANK, N)) * 0.01)   # B [r, d_out]
    rng = np.random.default_rng(4)
    xs = {m: torch.from_numpy(o.round_bf16(rng.standard_normal((m, K)))) for m in MS}
    return dict(packed=packed, absmax=absmax, a=torch.from_numpy(a), b=torch.from_numpy(b), xs=xs)


def cpu_reference_step(st, rows: int = N) -> None:
    """One step of the reference's CPU algorithm over the first `rows` output columns: per pass,
    rebuild the f32 weight (src/qwennet.rs:230-236 -> src/quantize.rs:355-366), linear
    (src/qwennet.rs:240), then the adapter's three ops (src/quantize.rs:620-624) and the sum
    (src/qwennet.rs:343)."""
    import torch
    from oracle import nf4_oracle as o

    for m in MS:
        w = torch.from_numpy(o.dequantize_packed(st["packed"][: rows * K // 2], rows * K,
                                                 st["absmax"][: rows * K // 64])).view(rows, K)
        x = st["xs"][m]
        y = x @ w.t()
        y = y + ((x @ st["a"]) @ st["b"][:, :rows]) * np.float32(SCALE)
        st["sink"] = float(y[0, 0])


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    st = cpu_reference_setup()
    t0 = time.perf_counter()
    cpu_reference_step(st)  # sizing probe (also the first warm-up step)
    t_full = time.perf_counter() - t0
    budget_s = 150.0
    rows = N
    total_steps = args.steps + args.warmup
    if t_full * total_steps > budget_s:
        rows = max(64, int(N * budget_s / (t_full * total_steps)) // 64 * 64)
    for _ in range(max(args.warmup - 1, 0)):
        cpu_reference_step(st, rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(st, rows)
    dt = time.perf_counter() - t0
    step_bytes = STEP_BYTES * rows / N
    value = step_bytes * args.steps / dt / 1e9
    cores = torch.get_num_threads()
    sample = (f"each step = the three M passes over the first {rows} of {N} weight rows "
              f"(scalar single-thread dequantize + torch f32 matmul on {cores} threads)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "host": "cpu"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------- own arm
def log(msg: str) -> None:
    """Progress line on stderr (rank-tagged) so a stuck multi-GPU run shows where it stopped."""
    sys.stderr.write(f"[bench rank {os.environ.get('RANK', '0')} +{time.perf_counter() - _T0:.1f}s] {msg}\n")
    sys.stderr.flush()


_T0 = time.perf_counter()


def run_own(args) -> None:
    import datetime

    import torch
    import torch.distributed as dist

    from unifur_b200 import _lib
    from unifur_b200.quantize import PackedNf4Tensor

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the NF4 library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        log("init_process_group(nccl)")
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
        log("process group up")
    lib = _lib.load()
    hbm_peak, _tf_peak, peak_kind = measured_peaks()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    # ---- resident data: eight weight copies, adapter, activations --------------------
    weights = []
    for c in range(N_COPIES):
        g = torch.Generator(device=dev).manual_seed(2 + c + 1000 * rank)
        w = torch.randn(N * K, device=dev, generator=g) * 0.02
        weights.append(PackedNf4Tensor.quantize(w))
        del w
    g = torch.Generator(device=dev).manual_seed(3)
    lora_a = (torch.randn(RANK, K, device=dev, generator=g) * 0.01).bfloat16()
    lora_b = (torch.randn(N, RANK, device=dev, generator=g) * 0.01).bfloat16()
    g = torch.Generator(device=dev).manual_seed(4)
    xs = {m: torch.randn(m, K, device=dev, generator=g).bfloat16() for m in MS}
    # the three passes write consecutive row ranges of one buffer, so that the sharded runs can
    # gather a step's outputs with a single collective
    # (two such buffers, used by alternate steps: the gather of one step runs on its own stream
    # beside the passes of the next)
    y_all = [torch.zeros(sum(MS), N, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    ys, row0 = {}, 0
    for m in MS:
        for par in range(2):
            ys[(m, par)] = y_all[par][row0:row0 + m]
        row0 += m
    # Sharded runs: every rank's kernel stores its columns straight into every rank's output
    # [rows, world * N] (peer stores over NVLink through IPC-mapped buffers), and a step ends with a
    # bounded wait for all ranks' CTAs on this rank's arrival counter: no collective, no copy.
    # Two outputs and counters, used by alternate steps (a rank may be one step ahead of another).
    y_full = arrivals = peer_y = peer_arr = None
    peer_stores = world > 1
    if world > 1:
        from unifur_b200.sharded import map_peer_tensors

        y_full = [torch.zeros(sum(MS), world * N, device=dev, dtype=torch.bfloat16) for _ in range(2)]
        arrivals = torch.zeros(64, device=dev, dtype=torch.int32)
        try:
            peer_y = [map_peer_tensors(y_full[par]) for par in range(2)]
            peer_arr = map_peer_tensors(arrivals)
            mapped = 1
        except Exception as e:  # no peer mapping on this machine (IPC closed, no peer access)
            log(f"peer mapping failed ({type(e).__name__}: {e}); the ranks exchange with an all-gather instead")
            mapped = 0
        flag = torch.tensor([mapped], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)  # every rank takes the same path
        peer_stores = bool(int(flag.item()))
        gathered_flat = None if peer_stores else torch.zeros(world, sum(MS), N, device=dev, dtype=torch.bfloat16)
    ws_bytes = max(int(lib.nf4_linear_workspace_bytes(m, K, N, RANK)) for m in MS)
    workspaces = {m: torch.zeros(max(ws_bytes, 256), dtype=torch.uint8, device=dev) for m in MS}

    def make_args(c, m, par=0):
        a = _lib.LinearArgs()
        a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
        a.layout, a.io_dtype = _lib.LAYOUT_OUT_IN, _lib.DTYPE_BF16
        a.rows, a.d_in, a.d_out = m, K, N
        a.x = xs[m].data_ptr()
        a.packed = weights[c].codes.data_ptr()
        a.absmax = weights[c].absmax.data_ptr()
        a.lora_a, a.lora_b = lora_a.data_ptr(), lora_b.data_ptr()
        a.lora_rank, a.lora_scale = RANK, SCALE
        a.y, a.ldy = ys[(m, par)].data_ptr(), N
        a.workspace, a.workspace_bytes = workspaces[m].data_ptr(), workspaces[m].numel()
        return a

    call_args = {(c, m, par): make_args(c, m, par) for c in range(N_COPIES) for m in MS for par in range(2)}
    # A step's last forward signals (one arrival per rank on every rank's counter of the step's
    # output); the next step's first forward waits for them inside the kernel before it reads its
    # input, as the next layer of a sharded model would; the first step of a sequence waits for
    # nothing and a wait kernel closes the sequence.
    peer_out = {}
    if peer_stores:
        row0 = 0
        for j, m in enumerate(MS):
            for par in range(2):
                for first in (False, True):
                    po = _lib.PeerOutputs()
                    po.struct_bytes = ctypes.sizeof(_lib.PeerOutputs)
                    po.world, po.rank, po.ldy_full = world, rank, world * N
                    for r in range(world):
                        po.y_full[r] = peer_y[par][r][row0:].data_ptr()
                        po.arrivals[r] = peer_arr[r][par:par + 1].data_ptr()
                    po.signal = 1 if j == len(MS) - 1 else 0
                    if j == 0 and not first:
                        po.wait_arrivals = arrivals[(par ^ 1):(par ^ 1) + 1].data_ptr()
                        po.wait_expected = world
                    peer_out[(m, par, first)] = po
            row0 += m
    log("weights quantized, arguments built")

    def step(i: int, first: bool = False) -> None:
        cur = torch.cuda.current_stream()
        stream = ctypes.c_void_p(cur.cuda_stream)
        par = i & 1
        for j, m in enumerate(MS):
            c = (len(MS) * i + j) % N_COPIES  # a different weight copy for every pass
            if peer_stores:
                _lib.check(lib.nf4_linear_forward_scatter_dev(ctypes.byref(call_args[(c, m, par)]),
                                                              ctypes.byref(peer_out[(m, par, first)]), stream))
            else:
                _lib.check(lib.nf4_linear_forward_dev(ctypes.byref(call_args[(c, m, par)]), stream))
        if world > 1 and not peer_stores:
            # without peer mapping: the step's slabs are all-gathered behind it on the same stream
            # and placed side by side
            dist.all_gather_into_tensor(gathered_flat, y_all[par])
            y_full[par].view(sum(MS), world, N).copy_(gathered_flat.permute(1, 0, 2))

    def drain(last: int) -> None:
        """Closes a sequence of steps: the last step's outputs are whole on this rank once every
        rank has signalled."""
        if peer_stores:
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            _lib.check(lib.nf4_peer_arrivals_wait_dev(ctypes.c_void_p(arrivals[(last & 1):(last & 1) + 1].data_ptr()),
                                                      world, 2_000_000_000, stream))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up, then K steps captured in one CUDA graph ---------------------------------
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(max(args.warmup, 3)):
            step(i, i == 0)
        drain(max(args.warmup, 3) - 1)
    barrier()
    scatter_check = "n/a"
    if world > 1:
        # the last warm-up step's output on this rank against every rank's own columns (computed
        # with the plain forward into a local buffer and exchanged with NCCL, off the timed path)
        last = max(args.warmup, 3) - 1
        mine = torch.zeros(sum(MS), N, device=dev, dtype=torch.bfloat16)
        with torch.cuda.stream(side):
            r0 = 0
            for j, m in enumerate(MS):
                a = make_args((len(MS) * last + j) % N_COPIES, m, 0)
                a.y = mine[r0:].data_ptr()
                _lib.check(lib.nf4_linear_forward_dev(ctypes.byref(a), ctypes.c_void_p(side.cuda_stream)))
                r0 += m
        torch.cuda.synchronize()
        everyone = torch.zeros(world, sum(MS), N, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(everyone, mine)
        got = y_full[last & 1].view(sum(MS), world, N).transpose(0, 1)
        same = torch.tensor([1 if torch.equal(got, everyone) else 0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        scatter_check = "ok" if int(same.item()) else "MISMATCH"
        barrier()
    log("warm-up done")
    launches0 = _lib.launch_count()
    launch_mode = "cuda-graph"
    graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(args.steps):
                step(i, i == 0)
            drain(args.steps - 1)
    except Exception as e:  # capture refused
        graph = None
        launch_mode = f"eager ({type(e).__name__})"
        torch.cuda.synchronize()
    gpu_launches = _lib.launch_count() - launches0
    if world > 1:
        # every rank must take the same path: one rank replaying a graph while another launches
        # eagerly would leave the collectives mismatched
        flag = torch.tensor([1 if graph is not None else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0 and graph is not None:
            graph = None
            launch_mode = "eager (capture failed on another rank)"
    log(f"launch mode: {launch_mode}")

    # K steps per measurement; the measurement is repeated and the median taken (the minimum is
    # reported beside it), each repetition bracketed by a barrier and CUDA events on the stream
    reps = 11
    rep_ms = []
    if graph is not None:
        with torch.cuda.stream(side):
            graph.replay()  # one untimed replay: graph upload
    else:
        launches0 = _lib.launch_count()
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with torch.cuda.stream(side):
            e0.record()
            if graph is not None:
                graph.replay()
            else:
                for i in range(args.steps):
                    step(i, i == 0)
                drain(args.steps - 1)
            e1.record()
        barrier()
        rep_ms.append(e0.elapsed_time(e1))
    if graph is None:
        gpu_launches = (_lib.launch_count() - launches0) // reps
    log("timed region done")
    ms = torch.tensor(rep_ms, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)  # per repetition: the slowest rank
    rep_ms = sorted(float(v) for v in ms.tolist())
    total_ms = rep_ms[len(rep_ms) // 2]
    min_ms = rep_ms[0]
    value = STEP_BYTES * args.steps * world / (total_ms * 1e-3) / 1e9

    # ---- roofline of the dominant kernel (decode GEMV incl. its LoRA pre-pass) ----------
    per_launch_ms = total_ms / (args.steps * len(MS))
    achieved = (STEP_BYTES / len(MS)) / (per_launch_ms * 1e-3) / 1e9
    roofline = {
        "kernel": "decode_kernel (one launch per forward), mean over M in {1,4,16}",
        "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
        "frac": achieved / hbm_peak, "peak_kind": f"of {peak_kind}",
        "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
        "algorithmic_bytes_per_launch": STEP_BYTES // len(MS),
        # dram__bytes_read.sum + dram__bytes_write.sum per launch of decode_kernel, from an ncu
        # capture of this kernel on this workload (not measured in this run): the weights are read
        # once, y stays in L2
        "traffic": 25892864, "traffic_source": "ncu capture (M = 1), not this run",
    }

    # ---- end to end through the host-pointer C ABI ------------------------------------------
    e2e = None
    cpu_baseline = None
    extras = {}
    if not args.device_only:
        handles = []
        vp = ctypes.c_void_p
        for c in range(N_COPIES):
            h = vp()
            codes = weights[c].codes.cpu().numpy()
            absmax = weights[c].absmax.cpu().numpy()
            _lib.check(lib.nf4_weight_from_packed_host(
                codes.ctypes.data_as(vp), absmax.ctypes.data_as(vp), None, 0.0, K, N,
                _lib.LAYOUT_OUT_IN, ctypes.byref(h)))
            a_h, b_h = lora_a.cpu().contiguous(), lora_b.cpu().contiguous()
            _lib.check(lib.nf4_weight_attach_lora_host(h, vp(a_h.data_ptr()), vp(b_h.data_ptr()),
                                                       RANK, SCALE, _lib.DTYPE_BF16))
            handles.append(h)
        x_host = {m: xs[m].cpu().pin_memory() for m in MS}
        y_host = {m: torch.zeros(m, N, dtype=torch.bfloat16).pin_memory() for m in MS}

        y_all_host = torch.zeros(sum(MS), world * N, dtype=torch.bfloat16).pin_memory()

        def host_step(i):
            if world == 1:
                # the reference-facing call: host x in, host y out, one synchronous call per forward
                for j, m in enumerate(MS):
                    h = handles[(len(MS) * i + j) % N_COPIES]
                    _lib.check(lib.nf4_weight_linear_forward_host(
                        h, vp(x_host[m].data_ptr()), m, _lib.DTYPE_BF16, None, None, None, 0, 0.0,
                        vp(y_host[m].data_ptr())))
                return
            # a sharded layer end to end: host x in, the shard's forwards storing into every rank's
            # output, the wait for all ranks' columns, the whole output out to the host
            cur = torch.cuda.current_stream()
            for m in MS:
                xs[m].copy_(x_host[m], non_blocking=True)
            step(i, True)
            drain(i)
            y_all_host.copy_(y_full[i & 1], non_blocking=True)
            cur.synchronize()

        for i in range(max(args.warmup, 3)):
            host_step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            host_step(i)
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {
            "value": STEP_BYTES * args.steps * world / float(dt.item()) / 1e9, "unit": UNIT,
            "h2d_bytes_per_step": sum(m * K * 2 for m in MS),
            "d2h_bytes_per_step": sum(m * N * 2 for m in MS) * world,
            "api": "nf4_weight_linear_forward_host (pinned host x in, host y out, synchronous)"
                   if world == 1 else
                   "per rank: pinned host x in, nf4_linear_forward_scatter_dev on the shard (its columns go to every "
                   "rank's output, the last forward signals), nf4_peer_arrivals_wait_dev, the whole [rows, world * N] "
                   "output out to the host, synchronous",
        }
        for h in handles:
            lib.nf4_weight_free(h)
        log("end-to-end region done")

    # ---- the configurations that are sharded by definition (every rank takes part) -------------
    if world > 1 and not args.device_only:
        log("sharded sections")
        extras.update(sharded_sections(torch, dist, lib, _lib, dev, rank, world, peer_stores=peer_stores))

    # ---- other kernels of the path (not part of `value`) -----------------------------------
    if rank == 0 and not args.device_only:
        extras.update(aux_sections(torch, lib, _lib, dev, hbm_peak, peak_kind))
        if world == 1:  # the other named configurations, measured on the one GPU
            log("side sections: block, sweep")
            extras["qwen2_7b_block"] = block_section(torch, lib, _lib, dev)
            extras["quantize_sweep"] = sweep_section(torch, lib, _lib, dev)

    # ---- CPU baseline beside it (rank 0, one GPU only) -----------------------------------------
    if rank == 0 and world == 1 and not args.device_only:
        st = cpu_reference_setup()
        cpu_reference_step(st)
        cpu_reps = 2
        t0 = time.perf_counter()
        for _ in range(cpu_reps):
            cpu_reference_step(st)
        cdt = (time.perf_counter() - t0) / cpu_reps
        log("CPU baselines of the side sections")
        side = cpu_side_baselines()
        for name in ("quantize", "dequantize", "prefill", "quantize_sweep"):
            if name in extras:
                extras[name]["cpu_baseline"] = side[name]
        if "qwen2_7b_block" in extras:
            extras["qwen2_7b_block"]["cpu_baseline_decode"] = side["qwen2_7b_block_decode"]
        cpu_baseline = {
            "value": STEP_BYTES / cdt / 1e9, "unit": UNIT, "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": f"{cpu_reps} full steps after 1 warm-up: scalar single-thread dequantize + torch "
                      f"f32 matmul on {torch.get_num_threads()} threads, {cdt:.2f} s per step",
        }

    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
            "timing": {"repetitions": reps, "statistic": "median of the repetitions (each: the K steps, "
                       "CUDA events on the stream, max over ranks)", "ms_median": total_ms, "ms_min": min_ms,
                       "ms_max": rep_ms[-1],
                       "value_at_min": STEP_BYTES * args.steps * world / (min_ms * 1e-3) / 1e9},
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 tensor-core MMA on bf16 activations, f32 accumulate, bf16 out",
            "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "cache": f"{N_COPIES} distinct weight copies "
                                f"({N_COPIES * algorithmic_bytes(1) / 1e6:.0f} MB > 126 MB L2) rotated "
                                "per pass",
                       "launch": launch_mode,
                       "sharding": "none" if world == 1 else
                       (f"{world} column shards of a [{world * N}, {K}] layer: every rank's kernel stores its columns "
                        "into every rank's output over NVLink, a step's last forward signals and the next step's "
                        f"first forward waits for all ranks inside the kernel (scatter_check: {scatter_check})"
                        if peer_stores else
                        f"{world} column shards of a [{world * N}, {K}] layer, one NCCL all-gather of y per step "
                        f"(no peer mapping on this machine; scatter_check: {scatter_check})")},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": int(gpu_launches), "clocks": clocks,
            "frac_of_nominal_8TBs": value / world / NOMINAL_HBM_GBS,
        }
        line.update(extras)
        print(json.dumps(line))
        sys.stdout.flush()
    if world > 1:
        # Leave without tearing NCCL down: destroying a process group whose collectives were
        # captured in a CUDA graph was seen to block for minutes.  Every rank has finished its
        # work once the barrier returns.
        dist.barrier()
        torch.cuda.synchronize()
        log("done")
        sys.stderr.flush()
        os._exit(0)


def time_loop(torch, fn, iters: int, warm: int = 5) -> float:
    """Mean milliseconds per call of fn(i), CUDA events on the current stream."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def time_flushed(torch, fn, flush, iters: int, warm: int = 3):
    """Median and minimum milliseconds of fn(i), each call timed by its own pair of CUDA events
    with a write of `flush` (larger than the L2) before it, outside the events."""
    for i in range(warm):
        fn(i)
    times = []
    for i in range(iters):
        flush.fill_(i & 1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn(i)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2], times[0]


def aux_sections(torch, lib, _lib, dev, hbm_peak, peak_kind):
    """Quantize / dequantize of the 4096x4096 round-trip configuration, reported in GB/s."""
    out = {}
    n = 4096 * 4096
    reps = 4  # 4 x 67 MB inputs rotate through more than the L2
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device=dev).manual_seed(1)
    vals = [torch.randn(n, device=dev, generator=g) * 0.02 for _ in range(reps)]
    packed = [torch.zeros(n // 2, dtype=torch.uint8, device=dev) for _ in range(reps)]
    absmax = [torch.zeros(n // 64, dtype=torch.float32, device=dev) for _ in range(reps)]
    ms_q = time_loop(torch, lambda i: _lib.check(lib.nf4_quantize_dev(
        p(vals[i % reps]), n, p(packed[i % reps]), p(absmax[i % reps]), stream())), 40)
    ms_d = time_loop(torch, lambda i: _lib.check(lib.nf4_dequantize_dev(
        p(packed[i % reps]), n, p(absmax[i % reps]), None, None, p(vals[i % reps]), stream())), 40)
    b = n * 4.5625
    for name, ms in (("quantize", ms_q), ("dequantize", ms_d)):
        gbs = b / (ms * 1e-3) / 1e9
        out[name] = {"workload": "4096x4096 f32, block 64", "us": ms * 1e3, "GB/s": gbs,
                     "frac": gbs / hbm_peak, "peak_kind": f"of {peak_kind}",
                     "algorithmic_bytes": int(b)}
    del vals, packed, absmax
    out["prefill"] = prefill_section(torch, lib, _lib, dev)
    out["reference_orientation"] = reference_orientation_section(torch, lib, _lib, dev)
    out["f32_tensors"] = f32_tensors_section(torch, lib, _lib, dev)
    out.update(load_and_embedding_section(torch, lib, _lib, dev))
    out["backward"] = backward_section(torch, lib, _lib, dev)
    return out


def reference_orientation_section(torch, lib, _lib, dev, iters: int = 20):
    """The decode configuration's layer as the reference itself stores and calls it: x f32 [M, 4096],
    W [4096, 11008] with the 64-blocks along d_out, adapter A [4096, 16], B [16, 11008] in f32
    (Nf4Linear::forward / QloraLinear::forward, src/qwennet.rs:230-241, 325-344)."""
    from unifur_b200.quantize import PackedNf4Tensor

    hbm_peak, _tf, peak_kind = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(12)
    w = torch.randn(K * N, device=dev, generator=g) * 0.02
    wq = PackedNf4Tensor.quantize(w)
    del w
    la = torch.randn(K, RANK, device=dev, generator=g) * 0.01
    lb = torch.randn(RANK, N, device=dev, generator=g) * 0.01
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)
    out = {"workload": "x f32 [M, 4096], W NF4 [4096, 11008] (blocks along d_out), LoRA rank 16 in f32; "
                       "up to 16 rows the CUDA-core strip kernel (f32 dequantisation and sums), more rows the "
                       "tensor-core GEMM over the repacked weight; 160 MB flush write before every forward, "
                       "outside the timed events"}
    for m in MS:
        x = torch.randn(m, K, device=dev, generator=g)
        y = torch.zeros(m, N, device=dev)
        ws = torch.zeros(max(int(lib.nf4_linear_workspace_bytes(m, K, N, RANK)), 256), dtype=torch.uint8, device=dev)
        a = _lib.LinearArgs()
        a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
        a.layout, a.io_dtype = _lib.LAYOUT_IN_OUT, _lib.DTYPE_F32
        a.rows, a.d_in, a.d_out = m, K, N
        a.x, a.packed, a.absmax = x.data_ptr(), wq.codes.data_ptr(), wq.absmax.data_ptr()
        a.lora_a, a.lora_b, a.lora_rank, a.lora_scale = la.data_ptr(), lb.data_ptr(), RANK, SCALE
        a.y, a.ldy = y.data_ptr(), N
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        ms, _ = time_flushed(torch, lambda _i: _lib.check(lib.nf4_linear_forward_dev(ctypes.byref(a), stream())),
                             flush, iters)
        by = K * N // 2 + K * N // 64 * 4 + RANK * (K + N) * 4 + m * (K + N) * 4
        gbs = by / (ms * 1e-3) / 1e9
        out[f"M={m}"] = {"us": ms * 1e3, "GB/s": gbs, "algorithmic_bytes": by, "frac": gbs / hbm_peak,
                         "peak_kind": f"of {peak_kind}"}
    # more than 16 rows: nibbles and scales repacked into the workspace, then the tensor-core GEMM
    pm = 2048
    x = torch.randn(pm, K, device=dev, generator=g)
    y = torch.zeros(pm, N, device=dev)
    ws = torch.zeros(max(int(lib.nf4_linear_workspace_bytes(pm, K, N, RANK)), 256), dtype=torch.uint8, device=dev)
    a = _lib.LinearArgs()
    a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
    a.layout, a.io_dtype = _lib.LAYOUT_IN_OUT, _lib.DTYPE_F32
    a.rows, a.d_in, a.d_out = pm, K, N
    a.x, a.packed, a.absmax = x.data_ptr(), wq.codes.data_ptr(), wq.absmax.data_ptr()
    a.lora_a, a.lora_b, a.lora_rank, a.lora_scale = la.data_ptr(), lb.data_ptr(), RANK, SCALE
    a.y, a.ldy = y.data_ptr(), N
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    ms, _ = time_flushed(torch, lambda _i: _lib.check(lib.nf4_linear_forward_dev(ctypes.byref(a), stream())),
                         flush, iters)
    flops = 2.0 * pm * N * K + 2.0 * pm * RANK * (K + N)
    out[f"M={pm}"] = {"ms": ms, "TFLOP/s": flops / (ms * 1e-3) / 1e12, "flops": flops,
                      "frac": flops / (ms * 1e-3) / 1e12 / _tf, "peak_kind": f"of {peak_kind} (burst)",
                      "path": "repacking kernels + f16 conversion + tcgen05 GEMM, f32 in and out"}
    return out


def f32_tensors_section(torch, lib, _lib, dev, iters: int = 20):
    """The decode configuration's layer in the measured layout (W [11008, 4096]) called with f32 tensors,
    the reference's own tensor type: up to 16 rows go through the decode kernel as bf16 high / low
    halves of every row, 2048 rows through the tensor-core GEMM after a conversion to f16."""
    from unifur_b200.quantize import PackedNf4Tensor

    hbm_peak, tf_peak, peak_kind = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(13)
    w = torch.randn(K * N, device=dev, generator=g) * 0.02
    wq = PackedNf4Tensor.quantize(w)
    del w
    la = torch.randn(RANK, K, device=dev, generator=g) * 0.01
    lb = torch.randn(N, RANK, device=dev, generator=g) * 0.01
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)
    out = {"workload": "x f32 [M, 4096], W NF4 [11008, 4096] (blocks along d_in), LoRA rank 16 in f32, f32 out; "
                       "160 MB flush write before every forward, outside the timed events"}
    for m in list(MS) + [2048]:
        x = torch.randn(m, K, device=dev, generator=g)
        y = torch.zeros(m, N, device=dev)
        ws = torch.zeros(max(int(lib.nf4_linear_workspace_bytes(m, K, N, RANK)), 256), dtype=torch.uint8, device=dev)
        a = _lib.LinearArgs()
        a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
        a.layout, a.io_dtype = _lib.LAYOUT_OUT_IN, _lib.DTYPE_F32
        a.rows, a.d_in, a.d_out = m, K, N
        a.x, a.packed, a.absmax = x.data_ptr(), wq.codes.data_ptr(), wq.absmax.data_ptr()
        a.lora_a, a.lora_b, a.lora_rank, a.lora_scale = la.data_ptr(), lb.data_ptr(), RANK, SCALE
        a.y, a.ldy = y.data_ptr(), N
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        ms, _ = time_flushed(torch, lambda _i: _lib.check(lib.nf4_linear_forward_dev(ctypes.byref(a), stream())),
                             flush, iters)
        if m <= 16:
            by = K * N // 2 + K * N // 64 * 4 + RANK * (K + N) * 4 + m * (K + N) * 4
            gbs = by / (ms * 1e-3) / 1e9
            out[f"M={m}"] = {"us": ms * 1e3, "GB/s": gbs, "algorithmic_bytes": by, "frac": gbs / hbm_peak,
                             "peak_kind": f"of {peak_kind}"}
        else:
            flops = 2.0 * m * N * K + 2.0 * m * RANK * (K + N)
            out[f"M={m}"] = {"ms": ms, "TFLOP/s": flops / (ms * 1e-3) / 1e12, "flops": flops,
                             "frac": flops / (ms * 1e-3) / 1e12 / tf_peak, "peak_kind": f"of {peak_kind} (burst)"}
    return out


def load_and_embedding_section(torch, lib, _lib, dev, iters: int = 10):
    """The checkpoint load path (a bf16 [4096, 14336] matrix as a checkpoint stores it, quantized as its
    transpose without materialising it: src/qwennet.rs:1375-1390, 1709-1711) and the embedding gather
    (4096 ids out of a double-quantized [151936, 3584] table, f32 rows out: src/qwennet.rs:285-291, where the
    reference rebuilds the whole f32 table per call)."""
    hbm_peak, _tf, peak_kind = measured_peaks()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(21)
    out = {}
    rows, cols = 4096, 14336
    w = (torch.randn(rows, cols, device=dev, generator=g) * 0.02).bfloat16()
    n = rows * cols
    codes = torch.empty(n // 2, dtype=torch.uint8, device=dev)
    absmax = torch.empty(n // 64, dtype=torch.float32, device=dev)
    ws = torch.empty(max(int(lib.nf4_quantize_transposed_workspace_bytes(rows, cols)), 16), dtype=torch.uint8, device=dev)
    ms, _ = time_flushed(torch, lambda _i: _lib.check(lib.nf4_quantize_transposed_dev(
        p(w), _lib.DTYPE_BF16, rows, cols, p(codes), p(absmax), p(ws), ws.numel(), stream())), flush, iters)
    by = n * 2 + n // 2 + n // 64 * 4
    out["load_path"] = {"workload": "bf16 [4096, 14336] -> packed NF4 of its transpose", "us": ms * 1e3,
                        "GB/s": by / (ms * 1e-3) / 1e9, "algorithmic_bytes": by, "frac": by / (ms * 1e-3) / 1e9 / hbm_peak,
                        "peak_kind": f"of {peak_kind}"}
    del w, codes, absmax, ws
    from unifur_b200.quantize import PackedNf4Tensor

    n_emb, d_model, n_ids = 151936, 3584, 4096
    table = PackedNf4Tensor.quantize(torch.randn(n_emb * d_model, device=dev, generator=g) * 0.02).with_double_quantization()
    ids = torch.randint(0, n_emb, (n_ids,), device=dev, generator=g, dtype=torch.int64)
    rows_out = torch.empty(n_ids, d_model, device=dev)
    ms, _ = time_flushed(torch, lambda _i: _lib.check(lib.nf4_embedding_gather_dev(
        p(table.codes), None, p(table.scale_codes), p(table.scale_of_scales), n_emb, d_model, p(ids), n_ids,
        p(rows_out), _lib.DTYPE_F32, stream())), flush, iters)
    by = n_ids * (d_model // 2 + d_model // 64 + d_model * 4 + 8)
    out["embedding_gather"] = {"workload": "4096 ids, table [151936, 3584] NF4 with u8 scales, f32 rows out",
                               "us": ms * 1e3, "GB/s": by / (ms * 1e-3) / 1e9, "algorithmic_bytes": by,
                               "frac": by / (ms * 1e-3) / 1e9 / hbm_peak, "peak_kind": f"of {peak_kind}",
                               "whole_table_f32_bytes_the_reference_rebuilds": n_emb * d_model * 4}
    return out


def backward_section(torch, lib, _lib, dev, iters: int = 10):
    """Backward of the QLoRA linear of configuration 3 (base weight frozen): grad_x = grad_y W + s (grad_y B) A
    over the same packed bytes read in the other orientation (tensor cores), grad_A and grad_B as
    small dense products (nf4_qlora_backward_dev; used by src/qwentrain.rs:421-470 through
    src/qwennet.rs:226-241)."""
    from unifur_b200.quantize import PackedNf4Tensor

    pm, pk, pn, pr = 2048, 4096, 14336, 64
    _hbm, tf_peak, peak_kind = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(15)
    w = torch.randn(pn * pk, device=dev, generator=g) * 0.02
    wq = PackedNf4Tensor.quantize(w)
    del w
    la = (torch.randn(pr, pk, device=dev, generator=g) * 0.01).bfloat16()
    lb = (torch.randn(pn, pr, device=dev, generator=g) * 0.01).bfloat16()
    x = torch.randn(pm, pk, device=dev, generator=g).bfloat16()
    gy = torch.randn(pm, pn, device=dev, generator=g).bfloat16()
    gx = torch.empty_like(x)
    ga, gb = torch.empty_like(la), torch.empty_like(lb)
    ws = torch.zeros(max(int(lib.nf4_qlora_backward_workspace_bytes(pm, pk, pn, pr)), 256), dtype=torch.uint8, device=dev)
    a = _lib.LinearArgs()
    a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
    a.layout, a.io_dtype = _lib.LAYOUT_OUT_IN, _lib.DTYPE_BF16
    a.rows, a.d_in, a.d_out = pm, pk, pn
    a.x, a.packed, a.absmax = x.data_ptr(), wq.codes.data_ptr(), wq.absmax.data_ptr()
    a.lora_a, a.lora_b, a.lora_rank, a.lora_scale = la.data_ptr(), lb.data_ptr(), pr, SCALE
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    vp = ctypes.c_void_p
    stream = lambda: vp(torch.cuda.current_stream().cuda_stream)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def run(_i):
        _lib.check(lib.nf4_qlora_backward_dev(ctypes.byref(a), vp(gy.data_ptr()), vp(gx.data_ptr()), vp(ga.data_ptr()),
                                              vp(gb.data_ptr()), stream()))

    ms, ms_min = time_flushed(torch, run, flush, iters)
    # grad_x: 2 M N K and its adapter term; U = grad_y B^T and T = x A; grad_A and grad_B
    flops = 2.0 * pm * pn * pk + 2.0 * pm * pr * (pk + pn) + 2.0 * pm * pr * (pk + pn) + 2.0 * pm * pr * (pk + pn)
    return {"workload": "backward of configuration 3's layer: x, grad_y bf16 [2048, 4096] / [2048, 14336], W NF4 "
                        "[14336, 4096] frozen, rank 64; grad_x, grad_A, grad_B",
            "ms": ms, "ms_min": ms_min, "TFLOP/s": flops / (ms * 1e-3) / 1e12, "flops": flops,
            "frac": flops / (ms * 1e-3) / 1e12 / tf_peak, "peak_kind": f"of {peak_kind} (burst)",
            "cache": "160 MB flush write before every call, outside the timed events"}


def prefill_section(torch, lib, _lib, dev, pn: int = 14336, iters: int = 20):
    """QLoRA prefill GEMM of configuration 3: x bf16 [2048, 4096], W NF4 [14336, 4096], rank 64,
    scale 2.0 (the configuration names none; the decode configuration's value is used)."""
    from unifur_b200.quantize import PackedNf4Tensor

    pm, pk, pr = 2048, 4096, 64
    _hbm, tf_peak, peak_kind = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(5)
    w = torch.randn(pn * pk, device=dev, generator=g) * 0.02
    wq = PackedNf4Tensor.quantize(w)
    del w
    g = torch.Generator(device=dev).manual_seed(6)
    la = (torch.randn(pr, pk, device=dev, generator=g) * 0.01).bfloat16()
    lb = (torch.randn(pn, pr, device=dev, generator=g) * 0.01).bfloat16()
    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(pm, pk, device=dev, generator=g).bfloat16()
    y = torch.zeros(pm, pn, device=dev, dtype=torch.bfloat16)
    wsb = int(lib.nf4_linear_workspace_bytes(pm, pk, pn, pr))
    ws = torch.zeros(max(wsb, 256), dtype=torch.uint8, device=dev)
    a = _lib.LinearArgs()
    a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
    a.layout, a.io_dtype = _lib.LAYOUT_OUT_IN, _lib.DTYPE_BF16
    a.rows, a.d_in, a.d_out = pm, pk, pn
    a.x, a.packed, a.absmax = x.data_ptr(), wq.codes.data_ptr(), wq.absmax.data_ptr()
    a.lora_a, a.lora_b, a.lora_rank, a.lora_scale = la.data_ptr(), lb.data_ptr(), pr, SCALE
    a.y, a.ldy = y.data_ptr(), pn
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def run(_i):
        _lib.check(lib.nf4_linear_forward_dev(ctypes.byref(a), stream()))

    ms, ms_min = time_flushed(torch, run, flush, iters)
    flops = 2.0 * pm * pn * pk + 2.0 * pm * pr * (pk + pn)
    tflops = flops / (ms * 1e-3) / 1e12
    return {"workload": f"QLoRA prefill GEMM: x bf16 [2048, 4096], W NF4 [{pn}, 4096] block 64, "
                        "LoRA rank 64 fused, f32 accumulate, bf16 out (pre-pass + GEMM kernel)",
            "ms": ms, "TFLOP/s": tflops, "flops": flops,
            "roofline": {"bound": "tensor", "achieved": tflops, "peak": tf_peak, "unit": "TFLOP/s",
                         "frac": tflops / tf_peak, "peak_kind": f"of {peak_kind} (burst)",
                         "frac_of_nominal_2250": tflops / 2250.0},
            "ms_min": ms_min,
            "cache": "160 MB flush write before every launch, outside the timed events (median of the launches)"}


def build_linear(torch, lib, _lib, dev, m: int, k: int, n: int, r: int, seed: int):
    """One NF4 linear with an adapter, resident on the device: argument block + what it points to."""
    from unifur_b200.quantize import PackedNf4Tensor

    g = torch.Generator(device=dev).manual_seed(seed)
    w = torch.randn(n * k, device=dev, generator=g) * 0.02
    wq = PackedNf4Tensor.quantize(w)
    del w
    la = (torch.randn(r, k, device=dev, generator=g) * 0.01).bfloat16()
    lb = (torch.randn(n, r, device=dev, generator=g) * 0.01).bfloat16()
    x = torch.randn(m, k, device=dev, generator=g).bfloat16()
    y = torch.zeros(m, n, device=dev, dtype=torch.bfloat16)
    ws = torch.zeros(max(int(lib.nf4_linear_workspace_bytes(m, k, n, r)), 256), dtype=torch.uint8,
                     device=dev)
    a = _lib.LinearArgs()
    a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
    a.layout, a.io_dtype = _lib.LAYOUT_OUT_IN, _lib.DTYPE_BF16
    a.rows, a.d_in, a.d_out = m, k, n
    a.x, a.packed, a.absmax = x.data_ptr(), wq.codes.data_ptr(), wq.absmax.data_ptr()
    a.lora_a, a.lora_b, a.lora_rank, a.lora_scale = la.data_ptr(), lb.data_ptr(), r, SCALE
    a.y, a.ldy = y.data_ptr(), n
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    return a, (wq, la, lb, x, y, ws)


QWEN2_7B_BLOCK = (("q", 3584, 3584), ("k", 3584, 512), ("v", 3584, 512), ("o", 3584, 3584),
                  ("gate", 3584, 18944), ("up", 3584, 18944), ("down", 18944, 3584))


def block_section(torch, lib, _lib, dev, iters: int = 20):
    """Configuration 5 on one GPU: the seven NF4 projections of a Qwen2-7B-shaped decoder block,
    rank-16 adapters, run back to back (decode batch 8, then prefill of 4096 tokens).  The glue
    between projections is not on the measured path; each projection reads its own synthetic
    input of the right shape."""
    hbm_peak, tf_peak, peak_kind = measured_peaks()
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)
    out = {}
    for label, m in (("decode_batch_8", 8), ("prefill_4096", 4096)):
        lins = [build_linear(torch, lib, _lib, dev, m, k, n, 16, 200 + i)
                for i, (_nm, k, n) in enumerate(QWEN2_7B_BLOCK)]

        def run(_i):
            for a, _keep in lins:
                _lib.check(lib.nf4_linear_forward_dev(ctypes.byref(a), stream()))

        if m == 8:
            # the projections that read the same activations go out as one call (and one launch):
            # q | k | v, then o, then gate | up, then down
            by_name = {nm: lins[i][0] for i, (nm, _k, _n) in enumerate(QWEN2_7B_BLOCK)}
            for nm, src in (("k", "q"), ("v", "q"), ("up", "gate")):
                by_name[nm].x = by_name[src].x
            calls = []
            for names in (("q", "k", "v"), ("o",), ("gate", "up"), ("down",)):
                block = (_lib.LinearArgs * len(names))(*[by_name[nm] for nm in names])
                calls.append((block, len(names)))

            def run_grouped(_i):
                for block, cnt in calls:
                    _lib.check(lib.nf4_linear_forward_grouped_dev(block, cnt, stream()))

            l0 = _lib.launch_count()
            run_grouped(0)
            launches = _lib.launch_count() - l0
            ms_each, _ = time_flushed(torch, run, flush, iters)
            ms, _ms_min = time_flushed(torch, run_grouped, flush, iters)
            by = sum(k * n // 2 + k * n // 64 * 4 + 16 * (k + n) * 2 + m * (k + n) * 2
                     for _nm, k, n in QWEN2_7B_BLOCK)
            gbs = by / (ms * 1e-3) / 1e9
            out[label] = {"us": ms * 1e3, "GB/s": gbs, "algorithmic_bytes": by,
                          "frac": gbs / hbm_peak, "peak_kind": f"of {peak_kind}",
                          "calls": "nf4_linear_forward_grouped_dev: q|k|v, o, gate|up, down",
                          "launches": launches, "us_one_call_per_projection": ms_each * 1e3}
            del calls, lins
            continue
        ms, _ms_min = time_flushed(torch, run, flush, iters)
        fl = sum(2.0 * m * k * n + 2.0 * m * 16 * (k + n) for _nm, k, n in QWEN2_7B_BLOCK)
        tf = fl / (ms * 1e-3) / 1e12
        out[label] = {"ms": ms, "TFLOP/s": tf, "flops": fl, "frac": tf / tf_peak,
                      "peak_kind": f"of {peak_kind} (burst)"}
        del lins
    out["workload"] = ("Qwen2-7B-shaped block, 7 NF4 linears (233,046,016 weights), block 64, rank 16; "
                       "160 MB flush write before each pass over the block, outside the timed events")
    return out


def sweep_section(torch, lib, _lib, dev):
    """Configuration 4: 32 f32 matrices (8 each of 4096x4096, 4096x14336, 14336x4096, 1024x4096),
    Student-t(4) * 0.02, quantized to packed NF4 with one call per matrix."""
    hbm_peak, _tf, peak_kind = measured_peaks()
    shapes = [(4096, 4096), (4096, 14336), (14336, 4096), (1024, 4096)]
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device=dev).manual_seed(100)
    mats = []
    for rep in range(8):
        for r, c in shapes:
            n = r * c
            z = torch.randn(n, device=dev, generator=g)
            chi = torch.randn(4, n, device=dev, generator=g).square_().sum(0).div_(4.0).sqrt_()
            mats.append((z.div_(chi).mul_(0.02), torch.empty(n // 2, dtype=torch.uint8, device=dev),
                         torch.empty(n // 64, dtype=torch.float32, device=dev)))
            del chi

    def run(_i):
        for v, c, am in mats:
            _lib.check(lib.nf4_quantize_dev(p(v), v.numel(), p(c), p(am), stream()))

    ms = time_loop(torch, run, 5, warm=2)
    elems = sum(v.numel() for v, _c, _a in mats)
    by = elems * 4.5625
    gbs = by / (ms * 1e-3) / 1e9
    return {"workload": "32 f32 matrices, Student-t(4) * 0.02, one quantize call per matrix",
            "elements": elems, "ms": ms, "GB/s": gbs, "algorithmic_bytes": int(by),
            "frac": gbs / hbm_peak, "peak_kind": f"of {peak_kind}"}


def sharded_sections(torch, dist, lib, _lib, dev, rank: int, world: int, iters: int = 10, peer_stores: bool = True):
    """The two configurations that are sharded by definition, on `world` GPUs, through
    ShardedNf4Linear: every rank owns a contiguous range of output columns of each weight (its rows
    of the packed weight, of the scales and of LoRA B), runs the single-GPU kernels on it, and the
    ranks all-gather y.  Before timing, every rank compares the gathered y with its own unsharded
    forward of the full weight (`gather_check`).  Times are CUDA events on the stream, max over ranks,
    median of `iters`, with a write larger than the L2 before each timed call."""
    from unifur_b200.quantize import PackedNf4Tensor, linear_forward
    from unifur_b200.sharded import ShardedNf4Linear

    _hbm, tf_peak, peak_kind = measured_peaks()
    hbm_peak = _hbm
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def reduce_max(v: float) -> float:
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def check(y_sharded, y_full, k: int) -> str:
        if torch.equal(y_sharded, y_full):
            verdict = 0.0
        else:
            # one bf16 ulp, plus what f32 sums of k terms added in another order (other tile splits
            # on a shard than on the whole weight) can differ by where the terms cancel
            d = (y_sharded.float() - y_full.float()).abs()
            tol = y_full.float().abs() * 2.0 ** -7 + 2e-6 * (k / 64) ** 0.5 * float(y_full.float().abs().max())
            verdict = 1.0 if bool((d <= tol).all()) else 2.0
        worst = reduce_max(verdict)
        return {0.0: "ok", 1.0: "ok_within_one_bf16_ulp"}.get(worst, "MISMATCH")

    def build(seed: int, m: int, k: int, n: int, r: int):
        """Same seed on every rank: the same full weight everywhere; each rank keeps its rows."""
        g = torch.Generator(device=dev).manual_seed(seed)
        w = torch.randn(n * k, device=dev, generator=g) * 0.02
        full = PackedNf4Tensor.quantize(w)
        del w
        la = (torch.randn(r, k, device=dev, generator=g) * 0.01).bfloat16()
        lb = (torch.randn(n, r, device=dev, generator=g) * 0.01).bfloat16()
        x = torch.randn(m, k, device=dev, generator=g).bfloat16()
        lin = ShardedNf4Linear.from_full(full, k, n, world, rank, lora_a=la, lora_b=lb, lora_scale=SCALE,
                                         granule=64)
        return full, la, lb, x, lin

    def timed(fn):
        times = []
        for i in range(iters + 2):
            flush.fill_(i & 1)
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(e0.elapsed_time(e1))
        t = torch.tensor(times, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.median().item())

    out = {}
    # ---- configuration 3: x [2048, 4096], W [14336, 4096], rank 64 ----
    pm, pk, pn, pr = 2048, 4096, 14336, 64
    full, la, lb, x, lin = build(5, pm, pk, pn, pr)
    plan = lin.plan(x)
    y_sharded = plan.run().clone()
    y_full = linear_forward(x, full, pk, pn, _lib.LAYOUT_OUT_IN, lora_a=la, lora_b=lb, lora_scale=SCALE)
    torch.cuda.synchronize()
    verdict = check(y_sharded, y_full, pk)
    del y_full, y_sharded
    ms_local = timed(plan.run_local)
    ms_all = timed(plan.run)
    flops = 2.0 * pm * pn * pk + 2.0 * pm * pr * (pk + pn)
    peer = {}
    if peer_stores:
        # the same without a collective: the GEMM writes its columns into this rank's output in
        # place, one kernel pushes them into every rank's output over NVLink and signals, a wait
        # for all ranks' arrivals closes the forward
        pp = lin.peer_store_plan(x, signal=True)

        def run_peer():
            pp.run()
            pp.wait(world)

        run_peer()
        torch.cuda.synchronize()
        dist.barrier()
        peer_verdict = check(pp.y, plan.run().clone(), pk)
        torch.cuda.synchronize()
        dist.barrier()
        ms_peer = timed(run_peer)
        peer = {"ms_with_peer_stores": ms_peer, "peer_store_check": peer_verdict,
                "TFLOP/s_with_peer_stores": flops / (ms_peer * 1e-3) / 1e12}
        del pp
    out["prefill_sharded"] = {
        "workload": f"QLoRA prefill GEMM x bf16 [2048, 4096], W NF4 [14336, 4096] in {world} column shards "
                    f"of {pn // world}, rank 64; all-gather of y (58.7 MB in all) into [2048, 14336]",
        "gather_check": verdict, "ms_local_forward": ms_local, "ms_with_gather": ms_all,
        "TFLOP/s": flops / (ms_all * 1e-3) / 1e12,
        "TFLOP/s_per_gpu_local": flops / world / (ms_local * 1e-3) / 1e12,
        "frac_per_gpu_local": flops / world / (ms_local * 1e-3) / 1e12 / tf_peak,
        "peak_kind": f"of {peak_kind} (burst)",
        "gather_share": max(0.0, (ms_all - ms_local) / ms_all), "n_gpus": world,
        "limiter": "the all-gather and the permuting copy of y follow the GEMM on the same stream",
    }
    if peer:  # the section's figure is the faster exchange; the all-gather's stays beside it
        sec = out["prefill_sharded"]
        sec["TFLOP/s_with_gather"] = sec["TFLOP/s"]
        sec["TFLOP/s"] = peer.pop("TFLOP/s_with_peer_stores")
        sec.update(peer)
        sec["limiter"] = ("with peer stores: the push of the shard's columns (NVLink) follows the GEMM on the same "
                          "stream; with the all-gather: the gather and the permuting copy do")
    del full, la, lb, x, lin, plan
    torch.cuda.empty_cache()

    # ---- configuration 5: the seven projections of the Qwen2-7B-shaped block ----
    blk = {}
    for label, m in (("decode_batch_8", 8), ("prefill_4096", 4096)):
        plans, checks = [], {}
        for i, (nm, k, n) in enumerate(QWEN2_7B_BLOCK):
            full, la, lb, x, lin = build(200 + i, m, k, n, 16)
            plan = lin.plan(x)
            y_sharded = plan.run().clone()
            y_full = linear_forward(x, full, k, n, _lib.LAYOUT_OUT_IN, lora_a=la, lora_b=lb, lora_scale=SCALE)
            torch.cuda.synchronize()
            checks[nm] = check(y_sharded, y_full, k)
            del y_full, y_sharded, full
            plans.append(plan)
        ms_local = timed(lambda: [pl.run_local() for pl in plans])
        ms_all = timed(lambda: [pl.run() for pl in plans])
        worst = "MISMATCH" if "MISMATCH" in checks.values() else (
            "ok" if all(v == "ok" for v in checks.values()) else "ok_within_one_bf16_ulp")
        if m == 8 and not peer_stores:
            by = sum(k * n // 2 + k * n // 64 * 4 + 16 * (k + n) * 2 + m * (k + n) * 2
                     for _nm, k, n in QWEN2_7B_BLOCK)
            blk[label] = {"us_local": ms_local * 1e3, "us_with_gather": ms_all * 1e3,
                          "GB/s": by / (ms_all * 1e-3) / 1e9,
                          "GB/s_per_gpu_local": by / world / (ms_local * 1e-3) / 1e9,
                          "frac_per_gpu_local": by / world / (ms_local * 1e-3) / 1e9 / hbm_peak,
                          "gather_check": worst, "per_projection": checks}
        elif m == 8:
            # the same seven sharded projections without a collective: every rank's kernels store
            # their columns into every rank's outputs; the last projection signals for the block
            # (kernel boundaries order the earlier launches' stores before it), one wait for the
            # ranks' arrivals closes the block
            pplans, pchecks, arr = [], {}, None
            for i, pl in enumerate(plans):
                pp = pl.lin.peer_store_plan(pl.x, signal=(i == len(plans) - 1), peer_arrivals=arr)
                arr = pp.peer_arrivals
                pplans.append(pp)

            def run_peer():
                for pp in pplans:
                    pp.run()
                pplans[0].wait(world)

            run_peer()
            torch.cuda.synchronize()
            dist.barrier()
            for (nm, k, n), pl, pp in zip(QWEN2_7B_BLOCK, plans, pplans):
                pchecks[nm] = check(pp.y, pl.run().clone(), k)   # against the all-gathered output, checked above
            torch.cuda.synchronize()
            dist.barrier()
            ms_peer = timed(run_peer)
            peer_worst = "MISMATCH" if "MISMATCH" in pchecks.values() else (
                "ok" if all(v == "ok" for v in pchecks.values()) else "ok_within_one_bf16_ulp")
            by = sum(k * n // 2 + k * n // 64 * 4 + 16 * (k + n) * 2 + m * (k + n) * 2
                     for _nm, k, n in QWEN2_7B_BLOCK)
            blk[label] = {"us_local": ms_local * 1e3, "us_with_gather": ms_all * 1e3,
                          "us_with_peer_stores": ms_peer * 1e3, "peer_store_check": peer_worst,
                          "GB/s": by / (ms_peer * 1e-3) / 1e9,
                          "GB/s_with_gather": by / (ms_all * 1e-3) / 1e9,
                          "GB/s_per_gpu_local": by / world / (ms_local * 1e-3) / 1e9,
                          "frac_per_gpu_local": by / world / (ms_local * 1e-3) / 1e9 / hbm_peak,
                          "gather_check": worst, "per_projection": checks}
            del pplans
        else:
            fl = sum(2.0 * m * k * n + 2.0 * m * 16 * (k + n) for _nm, k, n in QWEN2_7B_BLOCK)
            peer = {}
            if peer_stores:
                pplans, arr = [], None
                for i, pl in enumerate(plans):
                    pp = pl.lin.peer_store_plan(pl.x, signal=(i == len(plans) - 1), peer_arrivals=arr)
                    arr = pp.peer_arrivals
                    pplans.append(pp)

                def run_peer():
                    for pp in pplans:
                        pp.run()
                    pplans[0].wait(world)

                run_peer()
                torch.cuda.synchronize()
                dist.barrier()
                pchecks = [check(pp.y, pl.run().clone(), k) for (_nm, k, _n), pl, pp in zip(QWEN2_7B_BLOCK, plans, pplans)]
                torch.cuda.synchronize()
                dist.barrier()
                ms_peer = timed(run_peer)
                peer = {"ms_with_peer_stores": ms_peer, "TFLOP/s_with_peer_stores": fl / (ms_peer * 1e-3) / 1e12,
                        "peer_store_check": "MISMATCH" if "MISMATCH" in pchecks else (
                            "ok" if all(v == "ok" for v in pchecks) else "ok_within_one_bf16_ulp")}
                del pplans
            blk[label] = {"ms_local": ms_local, "ms_with_gather": ms_all,
                          "TFLOP/s": fl / (ms_all * 1e-3) / 1e12,
                          "TFLOP/s_per_gpu_local": fl / world / (ms_local * 1e-3) / 1e12,
                          "frac_per_gpu_local": fl / world / (ms_local * 1e-3) / 1e12 / tf_peak,
                          "gather_check": worst, "per_projection": checks}
            if peer:
                blk[label]["TFLOP/s_with_gather"] = blk[label]["TFLOP/s"]
                blk[label]["TFLOP/s"] = peer.pop("TFLOP/s_with_peer_stores")
                blk[label].update(peer)
        del plans
        torch.cuda.empty_cache()
    blk["workload"] = (f"Qwen2-7B-shaped block, 7 NF4 linears in {world} column shards each "
                       f"(per-GPU widths {3584 // world}/{512 // world}/{18944 // world}), rank 16, "
                       "one all-gather per projection")
    blk["n_gpus"] = world
    out["qwen2_7b_block_sharded"] = blk
    return out


def cpu_side_baselines():
    """The reference's CPU algorithm beside the side sections, on bounded samples: the oracle's C
    restatement (scalar, one thread, as the reference's loops are) for quantize / dequantize, and
    dequantize + f32 matmul on all cores (torch standing in for burn-ndarray) for the forwards."""
    import torch
    from oracle import nf4_oracle as o

    o.build()
    cores = torch.get_num_threads()
    out = {}
    rng = np.random.default_rng(1)
    n = 4096 * 4096
    w = (rng.standard_normal(n) * 0.02).astype(np.float32)
    t0 = time.perf_counter()
    packed, absmax = o.quantize_packed(w)
    tq = time.perf_counter() - t0
    t0 = time.perf_counter()
    o.dequantize_packed(packed, n, absmax)
    td = time.perf_counter() - t0
    b = n * 4.5625
    out["quantize"] = {"value": b / tq / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                       "sample": "the whole 4096x4096 matrix, once"}
    out["dequantize"] = {"value": b / td / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                         "sample": "the whole 4096x4096 matrix, once"}
    # sweep: the smallest and the square shape, once each (2 of the 32 matrices)
    t_sweep, elems = 0.0, 0
    for r, c in ((4096, 4096), (1024, 4096)):
        z = rng.standard_normal(r * c)
        chi = np.sqrt((rng.standard_normal((4, r * c)) ** 2).sum(0) / 4.0)
        v = (0.02 * z / chi).astype(np.float32)
        del z, chi
        t0 = time.perf_counter()
        o.quantize_packed(v)
        t_sweep += time.perf_counter() - t0
        elems += r * c
    out["quantize_sweep"] = {"value": elems * 4.5625 / t_sweep / 1e9, "unit": "GB/s", "cores": 1,
                             "kind": "port", "sample": "one 4096x4096 and one 1024x4096 Student-t matrix (2 of the 32)"}
    # prefill of configuration 3 on the first 2048 weight rows (a seventh of the 14336)
    pm, pk, pn_s, pr = 2048, 4096, 2048, 64
    wq = (rng.standard_normal(pn_s * pk) * 0.02).astype(np.float32)
    pk_codes, pk_absmax = o.quantize_packed(wq)
    x = torch.from_numpy(o.round_bf16(rng.standard_normal((pm, pk))))
    a = torch.from_numpy(o.round_bf16(rng.standard_normal((pk, pr)) * 0.01))
    bb = torch.from_numpy(o.round_bf16(rng.standard_normal((pr, pn_s)) * 0.01))
    t0 = time.perf_counter()
    wd = torch.from_numpy(o.dequantize_packed(pk_codes, pn_s * pk, pk_absmax)).view(pn_s, pk)
    y = x @ wd.t() + ((x @ a) @ bb) * np.float32(SCALE)
    tp = time.perf_counter() - t0
    fl = 2.0 * pm * pn_s * pk + 2.0 * pm * pr * (pk + pn_s)
    out["prefill"] = {"value": fl / tp / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                      "sample": f"the first {pn_s} of 14336 weight rows: scalar dequantize (1 thread) + "
                                f"f32 matmul on {cores} threads", "sink": float(y[0, 0])}
    # the block's decode pass: the down projection (a seventh of the block's linears, 29 % of its weights)
    k, n_, m = 18944, 3584, 8
    wq = (rng.standard_normal(n_ * k) * 0.02).astype(np.float32)
    c2, a2 = o.quantize_packed(wq)
    x = torch.from_numpy(o.round_bf16(rng.standard_normal((m, k))))
    t0 = time.perf_counter()
    wd = torch.from_numpy(o.dequantize_packed(c2, n_ * k, a2)).view(n_, k)
    y = x @ wd.t()
    tb = time.perf_counter() - t0
    by = k * n_ // 2 + k * n_ // 64 * 4 + m * (k + n_) * 2
    out["qwen2_7b_block_decode"] = {"value": by / tb / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": "the down projection only (67.9 M of the block's 233 M weights), "
                                              "no adapter", "sink": float(y[0, 0])}
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--prefill-only", type=int, default=0, metavar="N",
                    help="run only the prefill GEMM section with d_out = N (used under the profiler)")
    ap.add_argument("--sections", default="",
                    help="comma list of side sections to run alone on one GPU: block (the seven "
                         "projections of a Qwen2-7B-shaped block), sweep (32-matrix quantization "
                         "sweep), aux (quantize / dequantize / prefill)")
    ap.add_argument("--device-only", action="store_true",
                    help="time only the device-resident decode region (used under the profiler)")
    args = ap.parse_args()
    if args.prefill_only:
        import torch
        from unifur_b200 import _lib
        torch.cuda.set_device(0)
        print(json.dumps(prefill_section(torch, _lib.load(), _lib, torch.device("cuda", 0),
                                         pn=args.prefill_only, iters=max(args.steps, 1))))
        return
    if args.sections:
        import torch
        from unifur_b200 import _lib
        torch.cuda.set_device(0)
        dev, lib = torch.device("cuda", 0), _lib.load()
        res = {}
        for name in args.sections.split(","):
            if name == "block":
                res["qwen2_7b_block"] = block_section(torch, lib, _lib, dev)
            elif name == "sweep":
                res["quantize_sweep"] = sweep_section(torch, lib, _lib, dev)
            elif name == "aux":
                hbm, _tf, kind = measured_peaks()
                res.update(aux_sections(torch, lib, _lib, dev, hbm, kind))
            else:
                raise SystemExit(f"unknown section {name!r} (block, sweep, aux)")
        print(json.dumps(res))
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_own(args)


if __name__ == "__main__":
    main()
