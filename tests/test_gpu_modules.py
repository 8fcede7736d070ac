"""Module-level parity on the GPU: ConvRotLinear and the fused LoRA adapter against the CPU
oracle and against the reference-shaped adapter formula (lora.py:43-48), forward and backward,
under no_grad, gradient checkpointing, parameter paging and slider scaling."""
import pytest
import torch
import torch.nn as nn
import torch.utils.checkpoint

from oracle import convrot_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _make(n, k, bits, bias=True, seed=0, rank=0, alpha=None, b_std=0.01):
    from k2q import lora, modules
    w = R.synth_weight(n, k, seed=1000 + seed)
    # the module keeps the bias in the Linear's dtype (bf16) as Fp8Linear does (quantize.py:40-41)
    b = R.synth_vec(n, 0.01, 3000 + seed).to(torch.bfloat16).float() if bias else None
    lin = nn.Linear(k, n, bias=bias, device=DEV, dtype=torch.bfloat16)
    lin.weight.data.copy_(w)
    if bias:
        lin.bias.data.copy_(b)
    base = modules.ConvRotLinear(lin, bits=bits)
    if not rank:
        return base, w, b, None
    ad = lora.LoRALinear(base, rank, float(alpha if alpha is not None else rank))
    ad.lora_A.data.copy_(R.synth_mat(rank, k, 0.01, 4000 + seed))
    ad.lora_B.data.copy_(R.synth_mat(n, rank, b_std, 5000 + seed))
    return base, w, b, ad


@pytest.mark.parametrize("bits", [8, 4])
def test_convrot_linear_forward_bit_exact_and_protocol(bits):
    base, w, b, _ = _make(272, 768, bits)
    x = R.synth_act(6 * 50, 768, seed=2000, outliers=8).reshape(6, 50, 768)
    with torch.no_grad():
        y = base(x.to(DEV))
    ref_mod = R.ConvRotLinearRef(nn.Linear(768, 272, bias=True), bits=bits)
    q, s = (R.quantize_weight_int8 if bits == 8 else R.quantize_weight_int4)(w)
    assert torch.equal(base.weight_q.cpu(), q)
    assert torch.equal(base.scale.cpu().view(torch.int16 if bits == 4 else torch.int32),
                       s.view(torch.int16 if bits == 4 else torch.int32))
    ref_mod.weight_q.data, ref_mod.scale.data, ref_mod.bias.data = q, s, b
    y_ref = ref_mod(x)
    assert y.shape == (6, 50, 272) and y.dtype == torch.bfloat16
    assert torch.equal(y.cpu().view(torch.int16), y_ref.view(torch.int16))
    assert base.is_quant_linear and base.weight.is_cuda and not any(p.requires_grad for p in base.parameters())
    # quality figures (reported, gated loosely): weight-only dequant and the unquantised Linear
    assert R.max_rel_err(y.cpu(), R.linear_ref_weight_only(x.reshape(-1, 768), q, s, bits, b).reshape(6, 50, 272)) < 6e-2
    assert R.max_rel_err(y.cpu(), torch.nn.functional.linear(x, w, b.to(torch.bfloat16))) < (0.2 if bits == 4 else 6e-2)


def _reference_adapter_grads(x, w_eff, bias, a, b, s, gy):
    """Backward oracle: autograd through F.linear(x, W_eff) + the reference adapter formula, fp32."""
    x = x.float().clone().requires_grad_(True)
    a = a.clone().requires_grad_(True)
    b = b.clone().requires_grad_(True)
    y = torch.nn.functional.linear(x, w_eff, bias) + s * ((x @ a.t()) @ b.t())
    y.backward(gy.float())
    return x.grad, a.grad, b.grad


@pytest.mark.parametrize("rank,alpha,mul,m,n,k", [(16, 16, 1.0, 300, 384, 768), (32, 32, 1.0, 512, 768, 1024),
                                                  (32, 32, -1.5, 130, 256, 512), (8, 16, 0.5, 64, 128, 256)])
def test_fused_lora_forward_backward_vs_oracle(rank, alpha, mul, m, n, k):
    from k2q import lora, ops
    base, w, bias, ad = _make(n, k, 8, rank=rank, alpha=alpha, seed=rank)
    assert lora.fuse_lora(ad) == 1 and lora.fuse_lora(ad) == 0
    ad.scale_mul = mul
    x = R.synth_act(m, k, seed=2000 + rank, outliers=4)
    gy = R.synth_mat(m, n, 1e-2, 6000).to(torch.bfloat16)
    xd = x.to(DEV).requires_grad_(True)
    y = ad(xd)
    y.backward(gy.to(DEV))
    ops.check_status()

    q, sw = R.quantize_weight_int8(w)
    xq, sx = R.quantize_act_int8(x)
    a, b = ad.lora_A.detach().cpu(), ad.lora_B.detach().cpu()
    s = alpha / rank * mul
    y_ref = R.lora_forward_ref(R.linear_int8_exact(xq, sx, q, sw, bias), x, a, b, alpha / rank, mul)
    assert R.max_rel_err(y.detach().cpu(), y_ref) <= 2e-2
    gx, ga, gb = _reference_adapter_grads(x, R.effective_weight(q, sw, 8), bias, a, b, s, gy)
    assert R.max_rel_err(xd.grad.cpu(), gx) <= 2e-2
    assert R.max_rel_err(ad.lora_A.grad.cpu(), ga) <= 2e-2
    assert R.max_rel_err(ad.lora_B.grad.cpu(), gb) <= 2e-2
    assert ad.lora_A.grad.dtype == torch.float32 and ad.lora_A.grad.shape == (rank, k)
    assert ad.lora_B.grad.shape == (n, rank) and xd.grad.dtype == torch.bfloat16
    assert all(p.grad is None for p in base.parameters())


def test_zero_init_b_gives_zero_dA_and_identity_forward():
    """lora_B = 0 at step 0 (lora.py:40): the adapter is a no-op and dA is exactly zero."""
    from k2q import lora
    base, w, bias, ad = _make(256, 512, 8, rank=16, b_std=0.0)
    lora.fuse_lora(ad)
    x = R.synth_act(100, 512, seed=1).to(DEV).requires_grad_(True)
    y = ad(x)
    with torch.no_grad():
        y0 = base(x)
    assert torch.equal(y, y0)
    y.backward(torch.ones_like(y) * 1e-2)
    assert float(ad.lora_A.grad.abs().max()) == 0.0 and float(ad.lora_B.grad.abs().max()) > 0.0


def test_scale_mul_zero_and_lora_scaled_context():
    from k2q import lora
    base, w, bias, ad = _make(256, 512, 8, rank=16)
    lora.fuse_lora(ad)
    x = R.synth_act(64, 512, seed=2).to(DEV)
    with torch.no_grad():
        y1 = ad(x)
        with lora.lora_disabled(ad):
            y0 = ad(x)
        with lora.lora_scaled(ad, -1.0):
            ym = ad(x)
        assert torch.equal(y0, base(x))
        assert not torch.equal(y1, y0)
        d_plus, d_minus = (y1.float() - y0.float()), (ym.float() - y0.float())
        assert (d_plus + d_minus).abs().max() <= 0.02 * d_plus.abs().max() + 2 ** -6 * y0.float().abs().max()
        assert ad.scale_mul == 1.0


def test_fused_matches_unfused_reference_formula():
    """Same adapter, fused epilogue vs the reference's three-op formula over the same ConvRot base."""
    from k2q import lora
    base, w, bias, ad = _make(384, 768, 8, rank=16)
    x = R.synth_act(200, 768, seed=3).to(DEV)
    with torch.no_grad():
        y_plain = ad(x)
        lora.fuse_lora(ad)
        y_fused = ad(x)
    assert R.max_rel_err(y_fused.cpu(), y_plain.cpu()) <= 1e-2


def test_gradient_checkpointing_and_determinism():
    """mmdit.py:477-481 runs blocks under checkpoint(use_reentrant=False): the forward is executed
    twice and must reproduce itself bit for bit."""
    from k2q import lora
    base, w, bias, ad = _make(256, 512, 8, rank=16)
    lora.fuse_lora(ad)
    x = R.synth_act(96, 512, seed=4).to(DEV)
    xa = x.clone().requires_grad_(True)
    ya = ad(xa)
    ya.float().pow(2).sum().backward()
    ga, gA = xa.grad.clone(), ad.lora_A.grad.clone()
    ad.zero_grad()
    xb = x.clone().requires_grad_(True)
    yb = torch.utils.checkpoint.checkpoint(ad, xb, use_reentrant=False)
    yb.float().pow(2).sum().backward()
    assert torch.equal(ya, yb) and torch.equal(ga, xb.grad) and torch.equal(gA, ad.lora_A.grad)


def test_parameter_paging_like_block_swap():
    """_swap_move pages frozen params with p.data = p.data.to(device) (mmdit.py:409-414)."""
    base, w, bias, _ = _make(256, 512, 8)
    x = R.synth_act(32, 512, seed=5).to(DEV)
    with torch.no_grad():
        y0 = base(x)
        for p in base.parameters():
            p.data = p.data.to("cpu")
        with pytest.raises(RuntimeError):
            base(x)
        for p in base.parameters():
            p.data = p.data.to(DEV)
        assert torch.equal(base(x), y0)


def test_int4_forward_and_backward_with_adapter():
    """int4 base under an adapter: forward against the oracle; dX through the per-channel int8
    re-expression of the int4 weights, dA / dB as for the int8 base."""
    from k2q import lora, ops
    m, n, k, rank = 192, 256, 512, 16
    base, w, bias, ad = _make(n, k, 4, rank=rank)
    lora.fuse_lora(ad)
    x = R.synth_act(m, k, seed=6)
    gy = R.synth_mat(m, n, 1e-2, 6000).to(torch.bfloat16)
    xg = x.to(DEV).requires_grad_(True)
    y = ad(xg)
    y.backward(gy.to(DEV))
    ops.check_status()
    q, s = R.quantize_weight_int4(w)
    xq, sx = R.quantize_act_int8(x)
    a, b = ad.lora_A.detach().cpu(), ad.lora_B.detach().cpu()
    y_ref = R.lora_forward_ref(R.linear_int4_exact(xq, sx, q, s, bias), x, a, b, 1.0)
    assert R.max_rel_err(y.detach().cpu(), y_ref) <= 2e-2
    gx, ga, gb = _reference_adapter_grads(x, R.effective_weight(q, s, 4), bias, a, b, 1.0, gy)
    assert R.max_rel_err(xg.grad.cpu(), gx) <= 2e-2
    assert R.max_rel_err(ad.lora_A.grad.cpu(), ga) <= 2e-2
    assert R.max_rel_err(ad.lora_B.grad.cpu(), gb) <= 2e-2
    assert base.weight_q8.shape == (n, k) and base.weight_q8.dtype == torch.int8 and base.backward_scale.shape == (n,)


def test_mlp_gelu_pair_int4():
    """Linear -> GELU(tanh) -> Linear over int4 bases, the benchmark's workload at a small size."""
    from k2q import modules, ops
    k, h, m = 512, 1024, 200
    fc1, w1, _, _ = _make(h, k, 4, bias=False, seed=1)
    fc2, w2, _, _ = _make(k, h, 4, bias=False, seed=2)
    x = R.synth_act(m, k, seed=7)
    y = modules.convrot_mlp_gelu(x.to(DEV), fc1, fc2)
    ops.check_status()
    q1, s1 = R.quantize_weight_int4(w1)
    q2, s2 = R.quantize_weight_int4(w2)
    xq, sx = R.quantize_act_int8(x)
    hid = R.linear_int4_exact(xq, sx, q1, s1, None, act="gelu_tanh")
    hq, sh = R.quantize_act_int8(hid)
    y_ref = R.linear_int4_exact(hq, sh, q2, s2, None)
    assert R.max_rel_err(y.cpu(), y_ref) <= 2e-2
    hs = R.linear_sim_dequant(xq, sx, q1, s1, 4, None, act="gelu_tanh")
    hq2, sh2 = R.quantize_act_int8(hs)
    assert R.max_rel_err(y.cpu(), R.linear_sim_dequant(hq2, sh2, q2, s2, 4)) <= 2e-2


def test_shared_input_quantisation_is_scoped_reused_and_invalidated():
    """wq / wk / wv / gate read one tensor (mmdit.py:199): inside a ``shared_input_quant`` scope its K2
    pass runs once; an in-place change of the tensor, another tensor, a raw-pointer write by the
    library or leaving the scope quantises again; outside a scope nothing is remembered."""
    from k2q import modules, ops
    a, _, _, _ = _make(256, 512, 8, bias=False, seed=1)
    b, _, _, _ = _make(128, 512, 8, bias=False, seed=2)
    calls = {"n": 0}
    real = ops.fwht_quant_act

    def counting(x):
        calls["n"] += 1
        return real(x)

    ops.fwht_quant_act = counting
    try:
        x = R.synth_act(64, 512, seed=8).to(DEV)
        with torch.no_grad():
            a(x), a(x)
            assert calls["n"] == 2                        # no scope: every call quantises
            calls["n"] = 0
            with modules.shared_input_quant():
                ya, yb = a(x), b(x.view(64, 512))
                assert calls["n"] == 1
                x.mul_(2.0)                               # version bump -> stale codes must not be used
                ya2 = a(x)
                assert calls["n"] == 2 and not torch.equal(ya, ya2)
                y_other = a(x.clone())
                assert calls["n"] == 3 and torch.equal(y_other, ya2)
                a(x)
                assert calls["n"] == 4                    # x.clone() replaced the entry
                ops.note_raw_write()                      # e.g. a GEMM that wrote into x through out=
                a(x)
                assert calls["n"] == 5
            with modules.shared_input_quant():
                a(x)
                assert calls["n"] == 6                    # nothing survives the scope
        xq, sx = R.quantize_act_int8((x / 2.0).cpu())
        assert torch.equal(yb.cpu().view(torch.int16),
                           R.linear_int8_exact(xq, sx.reshape(-1), b.weight_q.cpu(), b.scale.cpu()).view(torch.int16))
    finally:
        ops.fwht_quant_act = real


def test_cuda_graph_replay_requantises_new_input():
    """Warm-up, capture on a static input, copy new data in, replay: the replay must quantise the new
    data (the K2 pass is part of the graph) and equal an eager call on it."""
    from k2q import modules
    lin, _, _, _ = _make(256, 512, 8, bias=True, seed=3)
    block = torch.nn.Sequential(lin)
    modules.share_block_inputs(block)
    static = R.synth_act(96, 512, seed=21).to(DEV)
    with torch.no_grad():
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                block(static)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = block(static)
        fresh = R.synth_act(96, 512, seed=22).to(DEV)
        static.copy_(fresh)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, block(fresh))


def test_mlp_gelu_host_pipeline_matches_device_call():
    """The chunked host-tensor entry point gives the same bits as the device-tensor call."""
    from k2q import modules
    k, h, m = 512, 1024, 1000
    fc1, _, _, _ = _make(h, k, 8, bias=False, seed=1)
    fc2, _, _, _ = _make(k, h, 8, bias=False, seed=2)
    x = R.synth_act(m, k, seed=9)
    y_dev = modules.convrot_mlp_gelu(x.to(DEV), fc1, fc2).cpu()
    x_host = x.pin_memory()
    out = torch.full((m, k), float("nan"), dtype=torch.bfloat16).pin_memory()
    y_host = modules.convrot_mlp_gelu_host(x_host, fc1, fc2, out_host=out, chunks=3)
    torch.cuda.current_stream().synchronize()
    assert y_host is out and torch.equal(y_host, y_dev)
    y2 = modules.convrot_mlp_gelu_host(x_host, fc1, fc2, chunks=1)
    torch.cuda.synchronize()
    assert torch.equal(y2, y_dev)


@pytest.mark.parametrize("bits", [4, 8])
def test_mlp_gelu_host_ramp_schedule_and_refusals(bits):
    """The default (ramped) schedule through the library's one-call pipeline: an int4 and an int8 pair with
    biases, a token count that leaves ragged pieces, a pageable (not pinned) input, work queued on the
    stream before and after the call; then the calls the library must refuse."""
    import ctypes as C
    from k2q import _lib, modules, ops
    k, h, m = 384, 768, 4099
    fc1, _, _, _ = _make(h, k, bits, bias=True, seed=3)
    fc2, _, _, _ = _make(k, h, bits, bias=True, seed=4)
    x = R.synth_act(m, k, seed=11)
    sched = modules.host_chunk_schedule(m, w4a8_out=k if bits == 4 else None)
    assert len(sched) >= 4 and sum(sched) == m and sched[0] < max(sched) > sched[-1]
    y_dev = modules.convrot_mlp_gelu(x.to(DEV), fc1, fc2)
    out = torch.full((m, k), float("nan"), dtype=torch.bfloat16).pin_memory()
    busy = torch.randn(2048, 2048, device=DEV)
    busy = busy @ busy                                     # the copies must start after this, not before
    modules.convrot_mlp_gelu_host(x, fc1, fc2, out_host=out)       # pageable input
    after = out.to(DEV, non_blocking=True)                 # ordered behind the last copy-out by the stream alone
    assert torch.equal(after, y_dev)
    torch.cuda.synchronize()
    assert torch.equal(out, y_dev.cpu())
    ops.check_status()
    # refusals: a schedule that does not add up, rows <= 0, one stream given twice, a short workspace
    keep = []
    d1, d2 = modules._linear_desc(fc1, keep), modules._linear_desc(fc2, keep)
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    xp = x.pin_memory()
    with pytest.raises(ValueError):
        ops.mlp_gelu_host(xp, d1, d2, out, [m - 1], k, h, k, torch.device(DEV), s_in, s_out)
    with pytest.raises(ValueError):
        ops.mlp_gelu_host(xp, d1, d2, out, [m + 5, -5], k, h, k, torch.device(DEV), s_in, s_out)
    with pytest.raises(ValueError, match="distinct"):
        ops.mlp_gelu_host(xp, d1, d2, out, [m], k, h, k, torch.device(DEV), s_in, s_in)
    lib = _lib.load()
    need = lib.k2q_mlp_gelu_host_workspace_bytes(m, k, h, k, m)
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    rows = (C.c_int64 * 1)(m)
    args = [C.c_void_p(xp.data_ptr()), m, C.byref(d1), C.byref(d2), C.c_void_p(out.data_ptr()), rows, 1,
            C.c_void_p(ws.data_ptr()), need - 1, C.c_void_p(ops.status_block(torch.device(DEV)).data_ptr()),
            C.c_void_p(torch.cuda.current_stream().cuda_stream), C.c_void_p(s_in.cuda_stream), C.c_void_p(s_out.cuda_stream)]
    assert lib.k2q_mlp_gelu_host(*args) == _lib.K2Q_EINVAL and "workspace" in _lib.last_error()
    bad = _lib.Linear(d2.bits, 0, d2.codes, d2.scale, d2.bias, d2.N, d2.K + 128)       # fc2 does not chain to fc1
    args[3], args[8] = C.byref(bad), need
    assert lib.k2q_mlp_gelu_host(*args) == _lib.K2Q_EINVAL
    torch.cuda.synchronize()
    assert torch.equal(out, y_dev.cpu())                   # the refused calls wrote nothing


def test_fused_adapter_step_matches_torch_adamw_with_clipping():
    """clip_grad_norm_ + AdamW.step + zero_grad (train_t2i_lora_cached.py:327-332) as two launches over
    flat buffers: parameters follow torch's own optimizer to fp32 rounding over several steps, with the
    clip active (large gradients) and inactive (small ones)."""
    from k2q import parallel, trainer
    torch.manual_seed(0)
    shapes = [(16, 512), (384, 16), (32, 768), (256, 32), (7,)]
    mine = [nn.Parameter(torch.randn(s, device=DEV) * 0.1) for s in shapes]
    ref = [nn.Parameter(p.detach().clone()) for p in mine]
    buckets = parallel.AdapterGradBuckets([mine[:2], mine[2:]], average=False)
    opt = trainer.FusedAdapterStep(buckets, lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.05, max_grad_norm=1.0)
    topt = torch.optim.AdamW(ref, lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.05)
    assert all(p.data.data_ptr() >= opt.param.data_ptr() for p in mine)                 # parameters live in the flat buffer
    for step in range(4):
        scale = 10.0 if step < 2 else 1e-3                                              # clipped, then not
        gs = [torch.randn(s, device=DEV) * scale for s in shapes]
        for p, q, g in zip(mine, ref, gs):
            p.grad.copy_(g)
            q.grad = g.clone()
        norm = torch.nn.utils.clip_grad_norm_(ref, 1.0)
        topt.step()
        topt.zero_grad(set_to_none=True)
        opt.step()
        assert abs(float(opt.grad_norm()) - float(norm)) <= 1e-5 * float(norm)
        for p, q in zip(mine, ref):
            assert torch.allclose(p.data, q.data, rtol=2e-5, atol=1e-7), step
        assert float(buckets.flat.abs().max()) == 0.0                                   # zero_grad


def test_prefetching_block_swap_on_gpu_gives_the_same_output():
    from k2q import dit as ditmod
    from k2q import modules, trainer
    torch.manual_seed(2)
    holder = nn.Module()
    holder.blocks = nn.ModuleList([ditmod.SingleStreamBlock(256, 2, 2, kvheads=1) for _ in range(3)]).to(DEV).to(torch.bfloat16)
    for p in holder.parameters():
        p.data.normal_(0, 0.05)
        p.requires_grad_(False)
    modules.quantize_dit_convrot(holder, bits=8)
    x = torch.randn(1, 128, 256, device=DEV).to(torch.bfloat16)
    vec = (torch.randn(1, 1, 6 * 256, device=DEV) * 0.1).to(torch.bfloat16)

    def run():
        y = x
        with torch.no_grad():
            for b in holder.blocks:
                y = b(y, vec, None, None)
        return y

    ref = run()
    st = trainer.enable_prefetching_block_swap(holder, 2, DEV)
    assert all(p.device.type == "cpu" and p.is_pinned() for p in holder.blocks[2].parameters())
    out = run()
    torch.cuda.synchronize()
    assert torch.equal(out, ref) and st.copies == 2
    assert all(p.device.type == "cpu" for p in holder.blocks[1].parameters())           # dropped again, nothing copied back
    assert torch.equal(run(), ref) and st.copies == 4


def test_int4_transient_backward_and_fast_forward():
    """backward_copy="transient" gives the same dX as the resident re-expression with nothing stored;
    fast=True runs the forward on the int8 re-expression: equal to W8A8 on those codes bit for bit,
    within the path's tolerance of the group-scaled definition."""
    from k2q import modules, ops
    n, k, m = 384, 512, 300
    w = R.synth_weight(n, k, seed=41)
    lin = nn.Linear(k, n, bias=True, device=DEV, dtype=torch.bfloat16)
    lin.weight.data.copy_(w)
    res = modules.ConvRotLinear(lin, bits=4, backward_copy=True)
    tr = modules.ConvRotLinear(lin, bits=4, backward_copy="transient")
    fast = modules.ConvRotLinear(lin, bits=4, backward_copy=True, fast=True)
    assert tr.weight_q8 is None and sum(p.numel() * p.element_size() for p in tr.parameters()) < \
        0.6 * sum(p.numel() * p.element_size() for p in res.parameters())
    x = R.synth_act(m, k, seed=42).to(DEV)
    gy = R.synth_mat(m, n, 1e-2, 43).to(torch.bfloat16).to(DEV)
    grads = []
    for mod in (res, tr):
        xg = x.clone().requires_grad_(True)
        mod(xg).backward(gy)
        grads.append(xg.grad)
    ops.check_status()
    assert torch.equal(grads[0], grads[1])
    with torch.no_grad():
        y_exact, y_fast = res(x), fast(x)
        xq, sx = ops.fwht_quant_act(x)
        y_w8 = ops.gemm_w8a8(xq, sx, fast.weight_q8.data, fast.backward_scale, fast.bias.data.float())
    ops.check_status()
    assert torch.equal(y_fast, y_w8)
    assert R.max_rel_err(y_fast.cpu(), y_exact.cpu()) <= 2e-2
    q4, s4 = R.quantize_weight_int4(w)
    xq_c, sx_c = R.quantize_act_int8(x.cpu())
    assert R.max_rel_err(y_fast.cpu(), R.linear_sim_dequant(xq_c, sx_c, q4, s4, 4, lin.bias.data.cpu())) <= 2e-2
