"""Benchmark harness beside ``bench.py`` (not part of the library): the workloads beyond the default
MLP pair -- the single-layer forward / training step and the two DiT steps (data-parallel training,
tensor-parallel inference).  ``bench.py`` dispatches here.  Each runner returns its JSON line as a
dict on rank 0 (``None`` elsewhere); ``run`` prints it, ``multi_gpu_summary`` condenses the DiT
runs into the ``multi_gpu`` object of the default benchmark line.
"""
from __future__ import annotations

import os
import sys
import time

import torch
import torch.distributed as dist

from k2q import dit as ditmod
from k2q import lora, modules, ops, parallel


def _sync_barrier(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def _timed(fn, steps, flush):
    evs = []
    for _ in range(steps):
        if flush is not None:
            flush.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        evs.append((s, e))
    torch.cuda.synchronize()
    return sum(s.elapsed_time(e) for s, e in evs)


def _max_over_ranks(values, dev, world):
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def _seeded_cpu(shape, std, seed, dtype=torch.float32):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


# ---------------------------------------------------------------------------------------------
# single layer: forward (config "linear_int8") or forward+backward (config "lora_train_int8")
# ---------------------------------------------------------------------------------------------
def run_layer(args, cfg, rank, world, dev, ClockSampler, peaks):
    M, K, N, r = cfg["M"], cfg["K"], cfg["N"], cfg["rank"]
    w = _seeded_cpu((N, K), 0.02, 1000, torch.bfloat16)
    x = _seeded_cpu((M, K), 1.0, 2000 + rank)
    cols = torch.randperm(K, generator=torch.Generator().manual_seed(2001))[:8]
    x[:, cols] *= 20.0                                           # eight outlier channels
    x = x.to(torch.bfloat16)
    lin = torch.nn.Linear(K, N, bias=True, device=dev, dtype=torch.bfloat16)
    lin.weight.data.copy_(w)
    lin.bias.data.copy_(_seeded_cpu((N,), 0.01, 3000))
    base = modules.ConvRotLinear(lin, bits=cfg["bits"], backward_copy=cfg["backward"])
    ad = lora.LoRALinear(base, r, cfg["alpha"])
    ad.lora_A.data.copy_(_seeded_cpu((r, K), 0.01, 4000))
    ad.lora_B.data.copy_(_seeded_cpu((N, r), 0.01, 5000))
    lora.fuse_lora(ad)
    gy = _seeded_cpu((M, N), 1e-2, 6000, torch.bfloat16).to(dev)
    xd = x.to(dev)
    x_host, gy_host = x.pin_memory(), gy.cpu().pin_memory()
    y_host = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    gx_host = torch.empty(M, K, dtype=torch.bfloat16).pin_memory()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    train = cfg["backward"]

    def step():
        if train:   # dX, dA, dB returned directly (no .grad accumulation nodes: the step is graph-capturable)
            xin = xd.detach().requires_grad_(True)
            y = ad(xin)
            return (y, *torch.autograd.grad(y, [xin, ad.lora_A, ad.lora_B], gy))
        with torch.no_grad():
            return (ad(xd),)

    def e2e_step():
        xin = x_host.to(dev, non_blocking=True)
        if train:
            xin.requires_grad_(True)
            y = ad(xin)
            gx, _, _ = torch.autograd.grad(y, [xin, ad.lora_A, ad.lora_B], gy_host.to(dev, non_blocking=True))
            gx_host.copy_(gx, non_blocking=True)
        else:
            with torch.no_grad():
                y = ad(xin)
        y_host.copy_(y, non_blocking=True)

    # The device-resident step is a dozen short kernels: launched one by one from Python the host
    # cannot keep up, so the step is captured once and replayed (same kernels, same buffers).
    # Warm-up and capture share one side stream and come before any autograd work on the default
    # stream (autograd ties a parameter's gradient node to the stream that first used it).
    use_graph = not getattr(args, "no_graph", False)
    timed_step = step
    if use_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(args.warmup, 3)):
                step()
        torch.cuda.synchronize()
        ops.check_status(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            graph_out = step()          # keeps the replayed step's outputs alive
        timed_step = graph.replay
    for _ in range(max(args.warmup, 3)):
        timed_step()
        e2e_step()
    ops.check_status(dev)
    with ClockSampler(dev.index) as clk:
        for _ in range(3):
            timed_step()
        _sync_barrier(world)
        clk.mark()
        total_ms = _timed(timed_step, args.steps, flush)
        _sync_barrier(world)
        e2e_ms = _timed(e2e_step, args.steps, flush)
        _sync_barrier(world)
    ops.check_status(dev)
    total_ms, e2e_ms = _max_over_ranks([total_ms, e2e_ms], dev, world)
    if rank != 0:
        return None
    gemm_ops = 2.0 * M * N * K * (2 if train else 1)
    bf16_peak, hbm_peak, src = peaks()
    tops = world * gemm_ops * args.steps / (total_ms * 1e-3) / 1e12
    bytes_h2d = x_host.numel() * 2 * (2 if train else 1)
    bytes_d2h = y_host.numel() * 2 + (gx_host.numel() * 2 if train else 0)
    launches = (3 + 8) if train else 3     # K2, lora_down, GEMM | + quant_rows, lora_down, fwht(A), GEMM, fwht, 2x(lora_tn + reduce)... counted below
    line = {
        "metric": "rotated-quant linear TOPS at DiT shapes", "value": tops, "unit": "TOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": args.workload, **cfg, "parallelism": f"dp{world}",
                   "l2": "flushed between steps (256 MiB write)", "cuda_graph": use_graph,
                   "ops_counted": "2*M*N*K per GEMM (forward; plus dX when training); adapter GEMMs not counted",
                   "kernels_per_step": "fwd: fwht_quant_act, lora_down, gemm_w8a8" +
                                       ("; bwd: quant_rows, lora_down, fwht_rows(A), gemm_w8a8(dX), fwht_rows, "
                                        "2x lora_tn(+reduce)" if train else "")},
        "roofline": {"bound": "tensor", "achieved": tops / world, "peak": 2 * bf16_peak, "unit": "TOP/s",
                     "frac": tops / world / (2 * bf16_peak), "traffic": None,
                     "note": f"whole step (all kernels) against 2 x {src} bf16 dense; not a single-kernel figure"},
        "e2e": {"value": world * gemm_ops * args.steps / (e2e_ms * 1e-3) / 1e12, "unit": "TOP/s",
                "h2d_bytes_per_step": bytes_h2d, "d2h_bytes_per_step": bytes_d2h, "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": (3 + (10 if train else 0)) * args.steps,
        "clocks": clk.summary(),
    }
    del launches
    return line


# ---------------------------------------------------------------------------------------------
# DiT builders
# ---------------------------------------------------------------------------------------------
def build_quantized_dit(cfg, dev, seed=1234):
    """Random-init DiT in the Krea 2 architecture (nn.Linear default init, zero norm / modulation
    parameters as in the reference), bf16, every Linear under ``blocks`` replaced by ConvRot codes."""
    conf = ditmod.krea2_large_wide()
    conf.layers = cfg["layers"]
    torch.manual_seed(seed)
    with torch.device(dev):
        model = ditmod.SingleStreamDiT(conf)
    model = model.to(torch.bfloat16)
    for p in model.parameters():          # norm scales stay fp32 like the reference keeps them
        p.requires_grad_(False)
    n = modules.quantize_dit_convrot(model, bits=cfg["bits"], fast=bool(cfg.get("fast")))
    torch.cuda.empty_cache()
    return model, n


def _dit_inputs(cfg, batch_rows: slice, dev, seed=7000):
    """Global-batch synthetic inputs (drawn once for all ranks), sliced to this rank's rows."""
    b, g, l = cfg["batch"], cfg["grid"], cfg["text"]
    gen = torch.Generator(device="cpu").manual_seed(seed)
    z0 = torch.randn(b, g * g, 64, generator=gen)
    ctx = torch.randn(b, l, 12, 2560, generator=gen).to(torch.bfloat16)
    t = ditmod.shift_schedule(g * g)(torch.rand(b, generator=gen)).float()
    noise = torch.randn(b, g * g, 64, generator=gen)
    mask = torch.ones(b, l, dtype=torch.bool)
    return tuple(v[batch_rows] for v in (z0, ctx, t, noise, mask))


# ---------------------------------------------------------------------------------------------
# config "dit_train_int8": one flow-matching fwd+bwd, data parallel by batch
# ---------------------------------------------------------------------------------------------
class _Fp8RefLinear(torch.nn.Module):
    """The reference's Fp8Linear on the host (quantize.py:23-51 as restated by ``oracle.fp8_linear_ref``):
    e4m3 codes + bf16 row scale, dequantised to bf16 on every forward, then ``F.linear``."""

    is_quant_linear = True

    def __init__(self, lin: torch.nn.Linear):
        super().__init__()
        from oracle import convrot_ref as R
        _, wq, sc = R.fp8_linear_ref(lin.weight.data, None, torch.zeros(1, lin.in_features, dtype=torch.bfloat16))
        self.wq, self.sc = wq, sc
        self.in_features, self.out_features = lin.in_features, lin.out_features

    @property
    def weight(self):
        return self.wq

    def forward(self, x):
        return torch.nn.functional.linear(x, self.wq.to(x.dtype) * self.sc.to(x.dtype))


def cpu_block_baseline(cfg, train: bool) -> dict:
    """CPU baseline of the DiT workloads, bounded: ONE block of the harness DiT with the reference's
    Fp8Linear bases (and, for training, the reference's un-fused rank-r adapters) on the host cores,
    one sample's tokens, timed once after one warm-up and scaled to layers x batch.  Attention, norms
    and everything else in the block run as the reference's torch ops on the CPU."""
    import time
    from k2q import dit as ditmod
    from k2q import lora
    torch.set_num_threads(os.cpu_count() or 1)
    torch.manual_seed(11)
    tokens = cfg["text"] + cfg["grid"] ** 2
    blk = ditmod.SingleStreamBlock(6144, 48, 4, kvheads=12).to(torch.bfloat16)
    for prm in blk.parameters():
        prm.data.normal_(0, 0.02)
        prm.requires_grad_(False)
    params = []
    for parent in (blk.attn, blk.mlp):
        for name, child in list(parent.named_children()):
            if isinstance(child, torch.nn.Linear):
                base = _Fp8RefLinear(child)
                if train:
                    ad = lora.LoRALinear(base, cfg["rank"], float(cfg["rank"]))
                    ad.lora_B.data.normal_(0, 0.01)
                    params += [ad.lora_A, ad.lora_B]
                    base = ad
                setattr(parent, name, base)
    x = torch.randn(1, tokens, 6144).to(torch.bfloat16)
    vec = (torch.randn(1, 1, 6 * 6144) * 0.1).to(torch.bfloat16)
    pos = torch.zeros(1, tokens, 3)
    rope = ditmod.rope_tables(pos, [32, 48, 48], 100.0)

    def step():
        if train:
            xg = x.clone().requires_grad_(True)
            blk(xg, vec, rope, None).float().pow(2).mean().backward()
        else:
            with torch.no_grad():
                blk(x, vec, rope, None)

    step()
    t0 = time.perf_counter()
    step()
    one = time.perf_counter() - t0
    scale = cfg["layers"] * cfg["batch"]
    return {"value": one * scale * 1e3, "unit": "ms/step", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"one block ({'forward + backward' if train else 'forward'}) of the reference's model code with "
                      f"Fp8Linear bases{' and rank-%d adapters' % cfg['rank'] if train else ''} on {tokens} tokens (one "
                      f"sample), {one:.2f} s measured once after a warm-up, extrapolated x {cfg['layers']} blocks x "
                      f"{cfg['batch']} samples (embedders, text fusion and the last layer not counted; no gradient "
                      "checkpointing on the CPU side)"}


def run_dit_train(args, cfg, rank, world, dev, ClockSampler, peaks, block_linear_ops):
    if cfg["batch"] % world:
        raise SystemExit(f"batch {cfg['batch']} does not divide over {world} GPUs")
    model, nq = build_quantized_dit(cfg, dev)
    text_side = bool(cfg.get("text_side")) and not getattr(args, "no_text_side", False)
    if text_side:                          # "all base Linears": the text-fusion blocks and the text MLP as well
        from k2q import serialize
        nq += serialize.quantize_text_side(model, bits=cfg["bits"], backward_copy=True)
    adapters = lora.inject_lora(model, rank=cfg["rank"], alpha=float(cfg["rank"]))
    gen = torch.Generator(device="cpu").manual_seed(5000)
    for ad in adapters.values():           # non-zero B so that dA is exercised
        ad.lora_B.data.copy_((torch.randn(ad.lora_B.shape, generator=gen) * 0.01).to(dev))
    params = lora.lora_parameters(adapters)
    model.gradient_checkpointing = not args.no_checkpoint
    model.train()
    per = cfg["batch"] // world
    rows = slice(rank * per, (rank + 1) * per)
    z0, ctx, t, noise, tmask = _dit_inputs(cfg, rows, dev)
    host = [v.pin_memory() for v in (z0, ctx, t, noise)]
    dz0, dctx, dt, dnoise = (v.to(dev) for v in host)
    tmask = tmask.to(dev)
    g = cfg["grid"]
    bytes_wire = 0

    # adapter gradients live in one flat buffer per block; a block's all-reduce starts as soon as its
    # last gradient has been accumulated, under the backward of the blocks in front of it
    buckets = parallel.AdapterGradBuckets(parallel.block_buckets(adapters), average=False)

    def fwd_bwd(z0_, ctx_, t_, noise_):
        nonlocal bytes_wire
        buckets.zero()
        loss = ditmod.flow_training_step(model, z0=z0_, context=ctx_, text_mask=tmask, grid_h=g, grid_w=g, t=t_,
                                         noise=noise_)
        (loss / world).backward()          # mean over the global batch = mean of per-rank means / world
        bytes_wire = buckets.finish()
        return loss

    def step():
        return fwd_bwd(dz0, dctx, dt, dnoise)

    loss_host = torch.zeros(1).pin_memory()

    def e2e_step():
        tensors = [v.to(dev, non_blocking=True) for v in host]
        loss = fwd_bwd(*tensors)
        loss_host.copy_(loss.detach().reshape(1), non_blocking=True)

    warm = max(args.warmup, 3) if cfg["layers"] < 8 else max(min(args.warmup, 3), 1)
    for _ in range(warm):
        step()
    ops.check_status(dev)
    torch.cuda.reset_peak_memory_stats(dev)
    with ClockSampler(dev.index) as clk:
        _sync_barrier(world)
        clk.mark()
        total_ms = _timed(step, args.steps, None)
        _sync_barrier(world)
        e2e_ms = _timed(e2e_step, args.steps, None)
        _sync_barrier(world)
    ops.check_status(dev)
    loss_val = float(step().detach())
    total_ms, e2e_ms = _max_over_ranks([total_ms, e2e_ms], dev, world)
    if rank != 0:
        return None
    tokens = cfg["batch"] * (cfg["text"] + g * g)
    mult = 3 if model.gradient_checkpointing else 2       # forward (+ recompute) + dX
    lin_ops = cfg["layers"] * block_linear_ops(tokens) * mult
    ms = total_ms / args.steps
    bf16_peak, _, src = peaks()
    line = {
        "metric": "quantized DiT LoRA fwd+bwd ms/step", "value": ms, "unit": "ms/step", "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 base / bf16 activations / fp32 adapters", "data": "synthetic",
        "config": {"workload": args.workload, **cfg, "global_batch": cfg["batch"], "tokens_per_step": tokens,
                   "parallelism": f"dp{world}", "quantized_linears": nq, "adapters": len(adapters),
                   "gradient_checkpointing": model.gradient_checkpointing, "text_side_quantized": text_side,
                   "l2": "working set (weights 12 GB int8 + activations) far larger than L2",
                   "collective": f"{len(buckets.buckets)} all-reduces (one per block, launched from gradient hooks under "
                                 f"the backward) of fp32 adapter gradients, {bytes_wire} bytes per step in total"},
        "linear_tops": lin_ops / (ms * 1e-3) / 1e12,
        "roofline": {"bound": "tensor", "achieved": lin_ops / (ms * 1e-3) / 1e12 / world, "peak": 2 * bf16_peak,
                     "unit": "TOP/s", "frac": lin_ops / (ms * 1e-3) / 1e12 / world / (2 * bf16_peak), "traffic": None,
                     "note": f"block Linear ops (x{mult}: fwd{', recompute' if mult == 3 else ''}, dX) over the WHOLE "
                             f"step time (attention, norms and adapters included), per GPU, against 2 x {src} bf16 dense"},
        "e2e": {"value": e2e_ms / args.steps, "unit": "ms/step",
                "h2d_bytes_per_step": sum(v.numel() * v.element_size() for v in host), "d2h_bytes_per_step": 4},
        "loss": loss_val, "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 2 ** 30,
        "gpu_launches": None, "clocks": clk.summary(),
    }
    if world == 1 and not getattr(args, "no_cpu", False):
        line["cpu_baseline"] = cpu_block_baseline(cfg, train=True)
    return line


# ---------------------------------------------------------------------------------------------
# config "dit_denoise_int4": one denoise forward, column-split tensor parallel
# ---------------------------------------------------------------------------------------------
def run_dit_denoise(args, cfg, rank, world, dev, ClockSampler, peaks, block_linear_ops):
    model, nq = build_quantized_dit(cfg, dev)
    scheme = getattr(args, "tp_scheme", "sequence")
    if world > 1:
        if scheme == "columns":
            parallel.shard_dit_columns(model, rank, world)
        elif scheme == "heads":
            parallel.shard_dit_heads(model, rank, world)
        else:
            parallel.shard_dit_sequence(model, rank, world)
        torch.cuda.empty_cache()
    groups = 0
    groups = modules.group_shared_input_linears(model)
    torch.cuda.empty_cache()
    model.eval()
    z0, ctx, t, noise, tmask = _dit_inputs(cfg, slice(0, cfg["batch"]), dev)
    g = cfg["grid"]
    img_host = noise.to(torch.bfloat16).pin_memory()
    ctx_host = ctx.pin_memory()
    img, dctx, tmask = img_host.to(dev), ctx_host.to(dev), tmask.to(dev)
    pos, mask = ditmod.position_ids(g, g, tmask)
    out_host = torch.empty_like(img_host)

    def step():
        return ditmod.denoise_step(model, img, dctx, 1.0, 0.875, pos, mask)

    def e2e_step():
        out = ditmod.denoise_step(model, img_host.to(dev, non_blocking=True), ctx_host.to(dev, non_blocking=True),
                                  1.0, 0.875, pos, mask)
        out_host.copy_(out, non_blocking=True)

    warm = max(min(args.warmup, 3), 1) if cfg["layers"] >= 8 else max(args.warmup, 3)
    for _ in range(warm):
        step()
    ops.check_status(dev)
    b0 = parallel.tp_gather_bytes(model)
    with ClockSampler(dev.index) as clk:
        _sync_barrier(world)
        clk.mark()
        total_ms = _timed(step, args.steps, None)
        _sync_barrier(world)
        e2e_ms = _timed(e2e_step, args.steps, None)
        _sync_barrier(world)
    ops.check_status(dev)
    gathered = (parallel.tp_gather_bytes(model) - b0) / (2 * args.steps)
    checksum = float(step().float().abs().mean())
    total_ms, e2e_ms = _max_over_ranks([total_ms, e2e_ms], dev, world)
    if rank != 0:
        return None
    tokens = cfg["batch"] * (cfg["text"] + g * g)
    lin_ops = cfg["layers"] * block_linear_ops(tokens)
    ms = total_ms / args.steps
    bf16_peak, _, src = peaks()
    line = {
        "metric": "quantized DiT denoise forward ms/step", "value": ms, "unit": "ms/step", "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "int4 base / int8 activations / bf16 output", "data": "synthetic",
        "config": {"workload": args.workload, **cfg, "tokens_per_step": tokens, "parallelism": f"tp{world}",
                   "quantized_linears": nq, "grouped_launches": groups,
                   "l2": "weights 6.3 GB int4 + activations, far larger than L2",
                   "tp_scheme": scheme if world > 1 else "none",
                   "collective": ("column shards that follow the attention heads / hidden units; all-gather of the gated "
                                  "attention output, wo's output, the SwiGLU product and down's output: "
                                  f"{gathered / 1e9:.2f} GB received per rank per step") if scheme == "columns" else
                                 (f"head / hidden-unit shards, one bf16 all-reduce after wo and after mlp.down: "
                                  f"{gathered / 1e9:.2f} GB received per rank per step") if scheme == "heads" else
                                 (f"head / hidden-unit shards and token-sharded residual stream: all-gather of int8 "
                                  f"codes before, reduce-scatter of bf16 partials after each half block: "
                                  f"{gathered / 1e9:.2f} GB received per rank per step")},
        "linear_tops": lin_ops / (ms * 1e-3) / 1e12,
        "roofline": {"bound": "tensor", "achieved": lin_ops / (ms * 1e-3) / 1e12 / world, "peak": 2 * bf16_peak,
                     "unit": "TOP/s", "frac": lin_ops / (ms * 1e-3) / 1e12 / world / (2 * bf16_peak), "traffic": None,
                     "note": f"block Linear ops over the WHOLE forward (attention, norms, gathers included), per GPU, "
                             f"against 2 x {src} bf16 dense"},
        "e2e": {"value": e2e_ms / args.steps, "unit": "ms/step",
                "h2d_bytes_per_step": img_host.numel() * 2 + ctx_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2},
        "output_checksum": checksum, "gpu_launches": None, "clocks": clk.summary(),
    }
    if world == 1 and not getattr(args, "no_cpu", False):
        line["cpu_baseline"] = cpu_block_baseline(cfg, train=False)
    return line


def run(args, cfg, rank, world, local_rank, ClockSampler, peaks, block_linear_ops):
    if args.impl == "reference":
        if rank == 0:
            args.emit({"impl": "reference", "unavailable":
                       f"workload {args.workload}: the CPU arm is defined for the default MLP workload only"})
        return
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the k2q path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # the reference trainer's runtime default (training_config.py:57,321-327): TF32 for fp32 matmuls,
    # which only the un-fused adapters on the bf16 text-side Linears use here
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    t0 = time.time()
    try:
        if cfg["kind"] == "layer":
            line = run_layer(args, cfg, rank, world, dev, ClockSampler, peaks)
        elif cfg["kind"] == "dit_train":
            line = run_dit_train(args, cfg, rank, world, dev, ClockSampler, peaks, block_linear_ops)
        elif cfg["kind"] == "dit_denoise":
            line = run_dit_denoise(args, cfg, rank, world, dev, ClockSampler, peaks, block_linear_ops)
        else:
            raise SystemExit(f"unknown workload kind {cfg['kind']}")
        if rank == 0:
            args.emit(line)
    finally:
        if world > 1:
            dist.destroy_process_group()
    if rank == 0:
        print(f"[bench] {args.workload} finished in {time.time() - t0:.1f} s", file=sys.stderr)


def multi_gpu_summary(args, workloads, rank, world, dev, ClockSampler, peaks, block_linear_ops, single_gpu_ms):
    """The two partitioned DiT workloads at this world size, a few steps each, inside the process
    group the caller has already set up: data-parallel training (one all-reduce of the adapter
    gradients) and tensor-parallel inference (column split with all-gathers, and the head split with a
    token-sharded residual stream).  Returns the ``multi_gpu`` object on rank 0."""
    import copy
    out = {}
    sub = copy.copy(args)
    sub.steps, sub.warmup = 2, 1
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True

    def keep(line, extra=()):
        if line is None:
            return None
        d = {k: line[k] for k in ("metric", "ms_per_step", "n_gpus", "steps", "warmup", "scaling") if k in line}
        d["collective"] = line["config"].get("collective")
        d["parallelism"] = line["config"].get("parallelism")
        d["e2e_ms_per_step"] = line["e2e"]["value"]
        d["clocks"] = line.get("clocks")
        for k in extra:
            d[k] = line.get(k, line["config"].get(k))
        return d

    for name, scheme in (("dit_train_int8", None), ("dit_denoise_int4", "columns"), ("dit_denoise_int4", "sequence")):
        cfg = dict(workloads[name])
        sub.workload = name
        if scheme is not None:
            sub.tp_scheme = scheme
        t0 = time.time()
        try:
            if cfg["kind"] == "dit_train":
                line = run_dit_train(sub, cfg, rank, world, dev, ClockSampler, peaks, block_linear_ops)
                res = keep(line, ("loss", "peak_mem_gb", "gradient_checkpointing"))
            else:
                line = run_dit_denoise(sub, cfg, rank, world, dev, ClockSampler, peaks, block_linear_ops)
                res = keep(line, ("output_checksum", "tp_scheme"))
        except Exception as ex:           # a failed side measurement must not cost the headline line
            res = {"error": f"{type(ex).__name__}: {ex}"} if rank == 0 else None
        torch.cuda.synchronize()
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        if rank == 0 and res is not None:
            res["wall_s"] = round(time.time() - t0, 1)
            key = name if scheme is None else f"{name}_{scheme}"
            ref = single_gpu_ms.get(key)
            if ref and "ms_per_step" in res:
                res["single_gpu_ms_per_step"] = ref
                res["speedup_vs_single_gpu"] = ref / res["ms_per_step"]
            out[key] = res
    return out if rank == 0 else None
