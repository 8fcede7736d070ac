#!/usr/bin/env python
"""Benchmark of the rotated-quant Linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl k2q|reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Default workload ``mlp_int4``: the int4 quantized MLP pair  Linear 3072->12288, GELU-tanh,
Linear 12288->3072  on X bf16 [8192, 3072], forward only (weights N(0,0.02) rotated + group-128
int4, activations int8 per token after the online FWHT).  A step = K2 -> W4A8 GEMM(+GELU) -> K2 ->
W4A8 GEMM over one batch of synthetic tokens.  Metric: rotated-quant linear TOP/s counted on the
two GEMMs (2*M*N*K each, 1237 GOP per step).

One JSON line is printed by rank 0.  ``value`` is measured with the inputs resident in HBM;
``e2e`` goes through the public host-tensor call (``convrot_mlp_gelu_host``: pinned HOST input and
output, copies inside the timed region, overlapped with the kernels chunk by chunk).  With N>1 every rank processes its own batch (data parallel by
tokens, no collective on the data path): weak scaling.

With N>1 the line also carries ``multi_gpu``: the two partitioned DiT workloads (data-parallel
training with one all-reduce, tensor-parallel inference with all-gathers) at this world size, a few
steps each.

``--impl reference`` times the reference's own CPU path for this workload: the MLP pair built from
``Fp8Linear`` (quantize.py:23-51: per-row e4m3 weights + bf16 scale, dequantised on every forward,
``F.linear`` in bf16) with ``F.gelu(approximate="tanh")`` between, restated in ``oracle/`` and pinned
bit for bit to the reference module by ``tests/golden/ref_fp8_lora.pt`` (the reference is Python and
cannot travel to the GPU box).  All rows of the workload, all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "krea-2_b200"))
sys.path.insert(0, str(ROOT))
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
# stdout carries ONE JSON line and nothing else: libraries that write to file descriptor 1 (NCCL prints its
# version banner there) are sent to stderr for the whole run, and the line goes out through a private copy of
# the original descriptor
_JSON_FD = os.dup(1)
os.dup2(2, 1)


def emit_json(line: dict) -> None:
    os.write(_JSON_FD, (json.dumps(line) + "\n").encode())


import torch  # noqa: E402

WORKLOADS = {
    # MLP pair (the default): M tokens, K -> H -> K
    "mlp_int4": dict(kind="mlp", M=8192, K=3072, H=12288, bits=4),
    "mlp_int8": dict(kind="mlp", M=8192, K=3072, H=12288, bits=8),
    # the int4 pair evaluated on its per-channel int8 re-expression (ConvRotLinear(fast=True)): W8A8 rate,
    # 1.5 bytes per weight resident, not bit-exact with the group-scaled definition (deviation reported)
    "mlp_int4_fast": dict(kind="mlp", M=8192, K=3072, H=12288, bits=4, fast=True),
    # single ConvRot int8 Linear 3072x3072 with bias and a rank-16 adapter, M=4096, forward
    "linear_int8": dict(kind="layer", M=4096, K=3072, N=3072, bits=8, rank=16, alpha=16.0, backward=False),
    # the same layer with a rank-32 adapter, forward + backward (dX through the codes, dA, dB)
    "lora_train_int8": dict(kind="layer", M=4096, K=3072, N=3072, bits=8, rank=32, alpha=32.0, backward=True),
    # random-init DiT (Krea 2 architecture), int8 base + rank-16 adapters, batch 8 at 1024x1024,
    # one flow-matching forward + backward, data parallel by batch
    "dit_train_int8": dict(kind="dit_train", bits=8, rank=16, batch=8, grid=64, text=512, layers=28, text_side=True),
    # the same DiT with an int4 base, one 2048x2048 denoise forward, column-split tensor parallel
    "dit_denoise_int4": dict(kind="dit_denoise", bits=4, batch=1, grid=128, text=512, layers=28),
    # the same step with every int4 base evaluated on its per-channel int8 re-expression (fast=True: W8A8
    # rate, 1.5 bytes per weight, outputs within the path's tolerance of the int4 definition, not bit-exact)
    "dit_denoise_int4_fast": dict(kind="dit_denoise", bits=4, fast=True, batch=1, grid=128, text=512, layers=28),
}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel (mean of the step's
# two GEMM launches at full size), from the ncu captures summarised under profiles/
NCU_TRAFFIC_BYTES = {"mlp_int4": 179.4e6, "mlp_int8": 246.9e6}

# ms/step of the DiT workloads on ONE GPU (this repository's own runs of `bench.py --workload ...`,
# listed in profiles/scaling.md); the multi_gpu object of an N>1 run quotes them beside its figures
SINGLE_GPU_MS = {"dit_train_int8": 2819.0, "dit_denoise_int4_columns": 615.0, "dit_denoise_int4_sequence": 615.0}


def synth_inputs(cfg, rank: int):
    """Seeded synthetic tensors with the workload's shapes and distributions (CPU, bf16)."""
    g = torch.Generator(device="cpu")
    w1 = (torch.randn(cfg["H"], cfg["K"], generator=g.manual_seed(1000)) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(cfg["K"], cfg["H"], generator=g.manual_seed(1001)) * 0.02).to(torch.bfloat16)
    x = torch.randn(cfg["M"], cfg["K"], generator=g.manual_seed(2000 + rank)).to(torch.bfloat16)
    return w1, w2, x


def step_ops(cfg) -> float:
    return 2.0 * 2.0 * cfg["M"] * cfg["K"] * cfg["H"]


def block_linear_ops(tokens: int, features=6144, kv=1536, hidden=16384) -> float:
    """2*M*N*K summed over the eight Linears of one DiT block (wq, gate, wo: F->F; wk, wv: F->kv;
    mlp.gate, mlp.up: F->hidden; mlp.down: hidden->F)."""
    per_token = 3 * features * features + 2 * features * kv + 3 * features * hidden
    return 2.0 * tokens * per_token


def bind_to_gpu_cores(index: int) -> str:
    """Pins this rank's process (and the threads it starts later: pinned-memory copies, the clock sampler)
    to the host cores NVML lists as local to its GPU, so that with several ranks on a two-socket host each
    rank's pinned staging buffers and copy threads sit on its GPU's NUMA node.  Read-only towards the GPU;
    returns a note for the JSON line.  A host whose GPUs share one core set is left as it is."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if vis:
                ids = [v.strip() for v in vis.split(",") if v.strip()]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            words = (os.cpu_count() + 63) // 64
            mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
            cores = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1}
        finally:
            pynvml.nvmlShutdown()
        allowed = os.sched_getaffinity(0)
        want = cores & allowed
        if want and want != allowed:
            os.sched_setaffinity(0, want)
            return f"bound to {len(want)} GPU-local cores"
        return f"GPU-local core set equals the allowed set ({len(allowed)} cores): not narrowed"
    except Exception as ex:      # affinity is an optimisation, never a reason to fail a run
        return f"not bound ({type(ex).__name__})"


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while the timed region runs (read-only;
    nothing is set).  Falls back to an ``nvidia-smi`` query loop if the NVML binding is missing."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period, self.samples, self.stop = index, period_s, [], threading.Event()
        self.max_mhz, self.thread = None, None

    def _visible_to_physical(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.index < len(ids) and ids[self.index].isdigit():
                return int(ids[self.index])
        return self.index

    def _run_nvml(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            h = pynvml.nvmlDeviceGetHandleByIndex(self._visible_to_physical())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            while not self.stop.is_set():
                mhz = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                try:
                    mask = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                except Exception:
                    mask = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                self.samples.append((mhz, mask))
                time.sleep(self.period)
        finally:
            pynvml.nvmlShutdown()

    def _run_smi(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        bits = [0x8, 0x40, 0x20, 0x4]
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self._visible_to_physical()), f"--query-gpu={q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10).stdout
                c = [v.strip() for v in out.strip().split(",")]
                self.max_mhz = float(c[1])
                mask = sum(b for b, v in zip(bits, c[2:6]) if v.lower().startswith("active"))
                self.samples.append((float(c[0]), mask))
            except Exception:
                return

    def _run(self):
        try:
            self._run_nvml()
        except Exception:
            self._run_smi()

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def mark(self):
        """Samples taken from here on belong to the timed region."""
        self.first = len(self.samples)

    def __exit__(self, *exc):
        self.stop.set()
        self.thread.join(timeout=15)

    def summary(self):
        rows = self.samples[getattr(self, "first", 0):]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        mask = 0
        for _, m in rows:
            mask |= m
        return {"sm_mhz": statistics.median(r[0] for r in rows), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(k for k, b in self.REASONS.items() if mask & b), "samples": len(rows)}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


# --------------------------------------------------------------------------------------------------
# CPU arm (oracle port of the reference-shaped path)
# --------------------------------------------------------------------------------------------------
def cpu_reference_step_factory(cfg, rows: int):
    """The reference's path for this workload on the host: Fp8Linear -> GELU(tanh) -> Fp8Linear
    (quantize.py:33-51 restated by ``oracle.fp8_linear_ref``; the weights are quantised once, as the
    reference does at start-up; every step dequantises them and runs ``F.linear`` in bf16)."""
    import torch.nn.functional as F
    from oracle import convrot_ref as R
    w1, w2, x = synth_inputs(cfg, 0)
    x = x[:rows].contiguous()
    _, wq1, sc1 = R.fp8_linear_ref(w1, None, x[:1])
    _, wq2, sc2 = R.fp8_linear_ref(w2, None, torch.zeros(1, cfg["H"], dtype=torch.bfloat16))

    def step():
        h = F.linear(x, wq1.to(x.dtype) * sc1.to(x.dtype))            # quantize.py:49-51
        h = F.gelu(h, approximate="tanh")
        return F.linear(h, wq2.to(x.dtype) * sc2.to(x.dtype))

    ops = 2.0 * 2.0 * rows * cfg["K"] * cfg["H"]
    return step, ops


def time_cpu(step, n_warm: int, n_timed: int):
    for _ in range(n_warm):
        step()
    ts = []
    for _ in range(n_timed):
        t0 = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t0)
    return ts


def run_reference(args, cfg, rank: int, world: int):
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    rows = cfg["M"]
    step, ops = cpu_reference_step_factory(cfg, rows)
    ts = time_cpu(step, min(args.warmup, 2), args.steps)
    total = sum(ts)
    value = ops * args.steps / total / 1e12
    line = {
        "impl": "reference", "metric": "rotated-quant linear TOPS at DiT shapes", "value": value, "unit": "TOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, **cfg,
                   "note": "the reference's Fp8Linear MLP pair (dequantise + F.linear, bf16) on the host, all "
                           f"{rows} token rows per step; restated in oracle/ and pinned bit for bit to "
                           "quantize.Fp8Linear by tests/golden/ref_fp8_lora.pt",
                   "warmup_steps_run": min(args.warmup, 2)},
        "cpu_baseline": {"value": value, "unit": "TOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"all {rows} token rows, all weights, mean of {args.steps} steps"},
        "e2e": {"value": value, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit_json(line)


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def run_k2q(args, cfg, rank: int, world: int, local_rank: int):
    import torch.distributed as dist
    from k2q import modules, ops

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the k2q path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    host_binding = bind_to_gpu_cores(local_rank) if world > 1 else "single rank: not bound"
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w1, w2, x_cpu = synth_inputs(cfg, rank)
    bits = cfg["bits"]
    lin1 = torch.nn.Linear(cfg["K"], cfg["H"], bias=False, device=dev, dtype=torch.bfloat16)
    lin2 = torch.nn.Linear(cfg["H"], cfg["K"], bias=False, device=dev, dtype=torch.bfloat16)
    lin1.weight.data.copy_(w1)
    lin2.weight.data.copy_(w2)
    fast = bool(cfg.get("fast"))
    fc1 = modules.ConvRotLinear(lin1, bits=bits, backward_copy=fast, fast=fast)
    fc2 = modules.ConvRotLinear(lin2, bits=bits, backward_copy=fast, fast=fast)
    del lin1, lin2
    gemm1, codes1, scale1 = fc1.forward_operands()
    gemm2, codes2, scale2 = fc2.forward_operands()
    int8_kernel = bits == 8 or fast

    x = x_cpu.to(dev)
    x_host = x_cpu.pin_memory()
    y_host = torch.empty(cfg["M"], cfg["K"], dtype=torch.bfloat16).pin_memory()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    M, K, H = cfg["M"], cfg["K"], cfg["H"]
    h = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
    y = torch.empty(M, K, dtype=torch.bfloat16, device=dev)

    gemm_events = []

    def step(record_gemm: bool):
        xq_, sx_ = ops.fwht_quant_act(x)
        if record_gemm:
            e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            e[0].record()
        gemm1(xq_, sx_, codes1, scale1, None, act="gelu_tanh", out=h)
        if record_gemm:
            e[1].record()
        hq_, sh_ = ops.fwht_quant_act(h)
        if record_gemm:
            e[2].record()
        gemm2(hq_, sh_, codes2, scale2, None, out=y)
        if record_gemm:
            e[3].record()
            gemm_events.append(e)

    def e2e_step():
        # public host-tensor entry: copies and kernels of successive token chunks overlap
        modules.convrot_mlp_gelu_host(x_host, fc1, fc2, out_host=y_host)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        evs = []
        for _ in range(steps):
            flush.fill_(1)                      # L2 flush between steps (outside the timed events)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            evs.append((s, e))
        torch.cuda.synchronize()
        return sum(s.elapsed_time(e) for s, e in evs)

    for _ in range(max(args.warmup, 3)):
        step(False)
        e2e_step()
    ops.check_status(dev)
    deviation = None
    if fast:      # the same pair through the group-scaled W4A8 kernel (bit-exact with the oracle) on 1024 rows
        with torch.no_grad():
            fc1.fast = fc2.fast = False
            y_exact = modules.convrot_mlp_gelu(x[:1024], fc1, fc2).float()
            fc1.fast = fc2.fast = True
            y_fast = modules.convrot_mlp_gelu(x[:1024], fc1, fc2).float()
        deviation = float((y_fast - y_exact).abs().max() / y_exact.abs().max())

    # Timed region: blocks of exactly `steps` steps, each bracketed by barrier + synchronize, repeated
    # until at least MIN_TIMED_S of device time has been measured (a single 20-step block lasts 20-30 ms,
    # too short for the clock sampler and for a sustained-power reading); the MEDIAN block is reported.
    MIN_TIMED_S, MAX_BLOCKS = 0.6, 64
    with ClockSampler(local_rank) as clk:
        for _ in range(3):          # lets the sampler thread start and the clocks settle under load
            step(False)
        barrier()
        clk.mark()
        blocks, spent = [], 0.0
        while True:
            barrier()
            ms = timed(lambda: step(True), args.steps)
            barrier()
            blocks.append(ms)
            spent += ms * 1e-3
            go = torch.tensor([1.0 if (spent < MIN_TIMED_S and len(blocks) < MAX_BLOCKS) else 0.0], device=dev)
            if world > 1:
                dist.all_reduce(go, op=dist.ReduceOp.MAX)     # every rank runs the same number of blocks
            if float(go) == 0.0:
                break
        e2e_blocks = []
        for _ in range(max(1, min(len(blocks), 8))):
            barrier()
            e2e_blocks.append(timed(e2e_step, args.steps))
            barrier()
    ops.check_status(dev)

    gemm_ms = sum(e[0].elapsed_time(e[1]) + e[2].elapsed_time(e[3]) for e in gemm_events) / (2 * len(gemm_events))

    # max over ranks per block, then the median block
    tb = torch.tensor(blocks, dtype=torch.float64, device=dev)
    te = torch.tensor(e2e_blocks, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tb, op=dist.ReduceOp.MAX)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = float(tb.median()), float(te.median())

    multi = None
    if world > 1 and not args.no_multi:
        import bench_workloads
        multi = bench_workloads.multi_gpu_summary(args, WORKLOADS, rank, world, dev, ClockSampler, measured_peaks,
                                                  block_linear_ops, SINGLE_GPU_MS)

    if rank == 0:
        ops_step = step_ops(cfg)
        value = world * ops_step * args.steps / (total_ms * 1e-3) / 1e12
        e2e_value = world * ops_step * args.steps / (e2e_ms * 1e-3) / 1e12
        bf16_peak, hbm_peak, src = measured_peaks()
        gemm_tops = (ops_step / 2) / (gemm_ms * 1e-3) / 1e12
        try:
            probe = ops.measure_i8_peak(8192, dev)
        except Exception as ex:  # calibration only
            probe = None
            print(f"[bench] int8 peak probe failed: {ex}", file=sys.stderr)
        # MEASURED_PEAKS.json holds no int8 figure: the denominator is the int8 tensor rate measured in
        # this run by back-to-back tcgen05.mma kind::i8 from resident shared memory; twice the measured
        # cuBLAS bf16 figure is reported beside it
        int8_peak = probe if probe else 2.0 * bf16_peak
        e2e_s = e2e_ms * 1e-3 / args.steps
        line = {
            "metric": "rotated-quant linear TOPS at DiT shapes", "value": value, "unit": "TOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8" if bits == 8 else "int4xint8", "data": "synthetic",
            "config": {"workload": args.workload, **cfg, "global_tokens": world * cfg["M"],
                       "parallelism": f"dp{world}", "l2": "flushed between steps (256 MiB write); inputs+weights "
                       "+hidden = 340 MB > L2", "ops_counted": "2 GEMMs, 2*M*N*K each",
                       "timed_blocks": len(blocks), "timed_seconds": sum(blocks) * 1e-3,
                       "statistic": f"median of {len(blocks)} blocks of {args.steps} steps, max over ranks per block",
                       "parity": "unpinned by the reference: it ships no Hadamard / int8 / int4 arithmetic; the "
                                 "oracle is this repository's CPU restatement (oracle/convrot_ref.py)"},
            "roofline": {"bound": "tensor", "achieved": gemm_tops, "peak": int8_peak, "unit": "TOP/s",
                         "frac": gemm_tops / int8_peak, "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                         "kernel": "gemm_w8a8_kernel" if int8_kernel else "gemm_w4a8_kernel",
                         "peak_note": ("int8 tensor rate measured in this run (tcgen05.mma kind::i8 probe)" if probe else
                                       f"2 x {src} cuBLAS bf16 dense (the in-run int8 probe failed)"),
                         "ms_per_launch": gemm_ms, "ops_per_launch": ops_step / 2,
                         "frac_of_2x_bf16_measured": gemm_tops / (2.0 * bf16_peak),
                         "peak_2x_bf16_measured": 2.0 * bf16_peak, "peaks_source": src,
                         "frac_of_nominal_4500": gemm_tops / 4500.0, "i8_mma_probe_tops": probe},
            "e2e": {"value": e2e_value, "unit": "TOP/s", "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": y_host.numel() * 2, "ms_per_step": e2e_ms / args.steps,
                    "h2d_gbs_per_rank": x_host.numel() * 2 / e2e_s / 1e9, "d2h_gbs_per_rank": y_host.numel() * 2 / e2e_s / 1e9,
                    "blocks": len(e2e_blocks), "host_binding": host_binding},
            "gpu_launches": 4 * args.steps,
            "clocks": clk.summary(),
        }
        if deviation is not None:
            line["config"]["max_rel_dev_from_int4_exact"] = deviation
            line["config"]["note"] = ("forward on the per-channel int8 re-expression of the int4 codes: outputs differ "
                                      "from the group-scaled definition by the figure above (first 1024 rows)")
        if multi is not None:
            line["multi_gpu"] = multi
        if world == 1:
            torch.set_num_threads(os.cpu_count() or 1)
            cstep, cops = cpu_reference_step_factory(cfg, cfg["M"])
            ts = time_cpu(cstep, 1, 3)
            line["cpu_baseline"] = {"value": cops * len(ts) / sum(ts) / 1e12, "unit": "TOP/s",
                                    "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"the reference's Fp8Linear MLP pair on all {cfg['M']} token rows, all "
                                              "weights; mean of 3 steps after 1 warm-up (the statistic of --impl reference)"}
        emit_json(line)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="k2q", choices=["k2q", "reference"])
    ap.add_argument("--workload", default="mlp_int4", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", dest="no_cpu", action="store_true",
                    help="DiT workloads: skip the bounded CPU baseline (one block on the host cores, extrapolated)")
    ap.add_argument("--layers", type=int, default=None, help="DiT workloads: override the depth (reported)")
    ap.add_argument("--batch", type=int, default=None,
                    help="DiT workloads: override the batch (reported); small profiling captures use it")
    ap.add_argument("--no-checkpoint", action="store_true", help="dit_train: disable gradient checkpointing")
    ap.add_argument("--no-text-side", action="store_true",
                    help="dit_train: leave the text-fusion / text-MLP Linears in bf16 as quantize_dit_fp8 does (default: "
                         "ALL base Linears carry ConvRot codes, k2q.serialize.quantize_text_side)")
    ap.add_argument("--tp-scheme", default="sequence", choices=["sequence", "heads", "columns"],
                    help="dit_denoise at N>1: attention heads / MLP hidden units split over the ranks with a "
                         "token-sharded residual stream (sequence, the default), the same with replicated tokens and "
                         "two all-reduces per block (heads), or every Linear's output columns split with an "
                         "all-gather (columns, bit-exact)")
    ap.add_argument("--no-multi", action="store_true",
                    help="N>1: skip the DiT side measurements (the multi_gpu object of the line)")
    ap.add_argument("--no-graph", action="store_true",
                    help="layer workloads: launch every kernel from Python instead of replaying a captured CUDA graph")
    args = ap.parse_args()
    cfg = dict(WORKLOADS[args.workload])
    if args.layers is not None and "layers" in cfg:
        cfg["layers"] = args.layers
    if args.batch is not None and "batch" in cfg:
        cfg["batch"] = args.batch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if cfg["kind"] != "mlp":
        import bench_workloads
        args.emit = emit_json
        bench_workloads.run(args, cfg, rank, world, local_rank, ClockSampler, measured_peaks, block_linear_ops)
    elif args.impl == "reference":
        run_reference(args, cfg, rank, world)
    else:
        run_k2q(args, cfg, rank, world, local_rank)


if __name__ == "__main__":
    main()
