"""Model-level parity on the GPU: a small DiT with ConvRot blocks and fused adapters against the
same network evaluated on the CPU through the oracle's ConvRotLinearRef, forward and backward,
with gradient checkpointing and with block paging."""
import copy
import zlib

import pytest
import torch
import torch.nn as nn

from oracle import convrot_ref as R

pytestmark = pytest.mark.gpu

CFG = dict(features=256, tdim=64, txtdim=128, heads=2, kvheads=1, multiplier=2, layers=2, patch=2, channels=16,
           txtheads=2, txtkvheads=2, txtlayers=3)


def _fill(model, scale=0.05):
    for name, p in model.named_parameters():
        g = torch.Generator().manual_seed(zlib.crc32(name.encode()))
        p.data = (torch.randn(p.shape, generator=g) * scale).to(p.dtype)


def _oracle_quantize(dit, bits):
    for block in dit.blocks:
        for mod in list(block.modules()):
            for name, child in list(mod.named_children()):
                if isinstance(child, nn.Linear):
                    setattr(mod, name, R.ConvRotLinearRef(child, bits=bits))


def _set_adapters(adapters):
    for name, ad in adapters.items():
        g = torch.Generator().manual_seed(zlib.crc32(name.encode()))
        ad.lora_A.data.copy_(torch.randn(ad.lora_A.shape, generator=g) * 0.02)
        ad.lora_B.data.copy_(torch.randn(ad.lora_B.shape, generator=g) * 0.02)


def _inputs():
    g = torch.Generator().manual_seed(3)
    b, gh, gw, l = 2, 8, 8, 24
    z0 = torch.randn(b, gh * gw, 64, generator=g)
    ctx = torch.randn(b, l, 3, 128, generator=g).to(torch.bfloat16)
    tm = torch.ones(b, l, dtype=torch.bool)
    tm[1, 20:] = False
    t = torch.tensor([0.3, 0.8])
    noise = torch.randn(b, gh * gw, 64, generator=g)
    return z0, ctx, tm, t, noise, gh, gw


@pytest.mark.parametrize("checkpoint", [False, True])
def test_tiny_dit_train_step_matches_cpu_oracle(checkpoint):
    from k2q import dit, lora, modules, ops
    base = dit.SingleStreamDiT(dit.DiTConfig(**CFG))
    _fill(base)
    base = base.to(torch.bfloat16)
    cpu = copy.deepcopy(base)
    gpu = copy.deepcopy(base).cuda()
    _oracle_quantize(cpu, 8)
    assert modules.quantize_dit_convrot(gpu, bits=8) == 16
    ad_cpu = lora.inject_lora(cpu, rank=8, alpha=8.0, fuse=False)
    ad_gpu = lora.inject_lora(gpu, rank=8, alpha=8.0)
    _set_adapters(ad_cpu)
    _set_adapters(ad_gpu)
    assert sum(getattr(m, "is_fused_lora", False) for m in ad_gpu.values()) == 16
    z0, ctx, tm, t, noise, gh, gw = _inputs()
    cpu.train()
    gpu.train()
    gpu.gradient_checkpointing = checkpoint
    loss_c = dit.flow_training_step(cpu, z0=z0, context=ctx, text_mask=tm, grid_h=gh, grid_w=gw, t=t, noise=noise)
    loss_c.backward()
    loss_g = dit.flow_training_step(gpu, z0=z0.cuda(), context=ctx.cuda(), text_mask=tm.cuda(), grid_h=gh, grid_w=gw,
                                    t=t.cuda(), noise=noise.cuda())
    loss_g.backward()
    ops.check_status()
    assert abs(float(loss_g) - float(loss_c)) <= 2e-2 * abs(float(loss_c))
    worst = 0.0
    for name in ("blocks.0.attn.wq", "blocks.1.mlp.down", "blocks.1.attn.wo", "blocks.0.mlp.gate"):
        for which in ("lora_A", "lora_B"):
            gc = getattr(ad_cpu[name], which).grad
            gg = getattr(ad_gpu[name], which).grad.cpu()
            worst = max(worst, R.max_rel_err(gg, gc))
    assert worst <= 5e-2, worst        # bf16 attention / norm differences between CPU and GPU add to the 2e-2
    assert all(p.grad is None for n, p in gpu.named_parameters() if "lora_" not in n)


def test_tiny_dit_int4_denoise_and_block_swap():
    from k2q import dit, modules, ops
    base = dit.SingleStreamDiT(dit.DiTConfig(**CFG))
    _fill(base)
    base = base.to(torch.bfloat16)
    cpu = copy.deepcopy(base)
    gpu = copy.deepcopy(base).cuda()
    _oracle_quantize(cpu, 4)
    modules.quantize_dit_convrot(gpu, bits=4)
    z0, ctx, tm, t, noise, gh, gw = _inputs()
    pos, mask = dit.position_ids(gh, gw, tm)
    img = noise.to(torch.bfloat16)
    cpu.eval()
    gpu.eval()
    out_c = dit.denoise_step(cpu, img, ctx, 1.0, 0.9, pos, mask)
    out_g = dit.denoise_step(gpu, img.cuda(), ctx.cuda(), 1.0, 0.9, pos.cuda(), mask.cuda())
    ops.check_status()
    assert R.max_rel_err(out_g.cpu(), out_c) <= 3e-2
    # deepest block parked on the CPU between uses (mmdit.py:389-428); output unchanged
    assert gpu.enable_block_swap(1, "cuda") == [1]
    assert gpu.blocks[1].attn.wq.weight_q.device.type == "cpu"
    out_s = dit.denoise_step(gpu, img.cuda(), ctx.cuda(), 1.0, 0.9, pos.cuda(), mask.cuda())
    assert torch.equal(out_s, out_g) and gpu.blocks[1].attn.wq.weight_q.device.type == "cpu"


@pytest.mark.parametrize("bits", [8, 4])
def test_head_sharded_block_matches_the_unsharded_quantized_block(bits):
    """Both ranks' shards of one quantized block, evaluated on one GPU and summed by hand (no process
    group: RowParallelLinear then returns the partial product), against the unsharded block."""
    from k2q import dit, modules, ops, parallel
    torch.manual_seed(5)
    dim, heads, kvheads = 768, 6, 3                       # KV head 1 is shared by the two ranks
    attn = dit.Attention(dim, heads, kvheads, bias=True)
    mlp = dit.SwiGLU(dim, 3, bias=True)
    for prm in list(attn.parameters()) + list(mlp.parameters()):
        prm.data.normal_(0.0, 0.04)
    holder = nn.ModuleDict(dict(attn=attn, mlp=mlp)).to(torch.bfloat16).cuda()
    for parent in (holder["attn"], holder["mlp"]):
        for name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear):
                setattr(parent, name, modules.ConvRotLinear(child, bits=bits, backward_copy=False))
    x = torch.randn(2, 40, dim, device="cuda").to(torch.bfloat16)
    pos = torch.arange(40, device="cuda")[None, :, None].expand(2, 40, 3)
    rope = dit.rope_tables(pos, [128 - 12 * 8, 48, 48], 1e4)
    with torch.no_grad():
        ref_a, ref_m = holder["attn"](x, rope).float(), holder["mlp"](x).float()
        sum_a = sum(parallel.HeadParallelAttention(holder["attn"], r, 2)(x, rope).float() for r in range(2))
        sum_m = sum(parallel.HiddenParallelSwiGLU(holder["mlp"], r, 2)(x).float() for r in range(2))
    ops.check_status(x.device)
    # two bf16 partials and per-shard activation scales instead of one product: float tolerance of the path
    assert (sum_a - ref_a).abs().max() <= 2e-2 * ref_a.abs().max()
    assert (sum_m - ref_m).abs().max() <= 2e-2 * ref_m.abs().max()


@pytest.mark.parametrize("bits", [8, 4])
def test_sequence_parallel_block_on_one_rank_equals_the_plain_block(bits):
    """With a single rank the token-sharded block degenerates to the plain one, except that the
    projections consume int8 codes handed over explicitly instead of quantizing their input
    themselves: same kernels, same codes, so the outputs must be identical."""
    from k2q import dit, modules, ops, parallel
    torch.manual_seed(9)
    dim, heads, kvheads, tokens = 768, 6, 3, 64
    blk = dit.SingleStreamBlock(dim, heads, 3, bias=True, kvheads=kvheads)
    for prm in blk.parameters():
        prm.data.normal_(0.0, 0.04)
    blk = blk.to(torch.bfloat16).cuda()
    for parent in (blk.attn, blk.mlp):
        for name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear):
                setattr(parent, name, modules.ConvRotLinear(child, bits=bits, backward_copy=False))
    x = torch.randn(2, tokens, dim, device="cuda").to(torch.bfloat16)
    vec = (torch.randn(2, 1, 6 * dim, device="cuda") * 0.1).to(torch.bfloat16)
    pos = torch.arange(tokens, device="cuda")[None, :, None].expand(2, tokens, 3)
    rope = dit.rope_tables(pos, [128 - 12 * 8, 48, 48], 1e4)
    with torch.no_grad():
        ref = blk(x, vec, rope)
        sp = parallel.SequenceParallelBlock(blk, 0, 1, first=True, last=True)
        assert sp.codes_attn and sp.codes_mlp
        got = sp(x, vec, rope)
    ops.check_status(x.device)
    assert torch.equal(got, ref)


def test_fused_prologue_block_matches_the_unfused_block(monkeypatch):
    """Inference over ConvRot bases takes the fused route (norm + modulation, SwiGLU and the sigmoid
    gate inside the quantisation passes); it must agree with the op-by-op block."""
    from k2q import dit as ditmod
    from k2q import modules
    torch.manual_seed(0)
    blk = ditmod.SingleStreamBlock(256, 2, 2, kvheads=1).cuda().to(torch.bfloat16)
    for p in blk.parameters():
        p.data.normal_(0, 0.05)
    holder = nn.Module()
    holder.blocks = nn.ModuleList([blk])
    assert modules.quantize_dit_convrot(holder, bits=8) == 8
    x = torch.randn(2, 96, 256, device="cuda").to(torch.bfloat16)
    vec = (torch.randn(2, 1, 6 * 256, device="cuda") * 0.1).to(torch.bfloat16)
    pos = torch.stack((torch.zeros(96), torch.arange(96) // 8, torch.arange(96) % 8), dim=-1)[None].expand(2, -1, -1).cuda()
    rope = ditmod.rope_tables(pos, [32, 48, 48], 100.0)        # head dimension 128: QK-norm + rotation as one kernel
    calls = {"n": 0, "qk": 0}
    real = modules.ops.norm_mod_quant
    real_qk = modules.ops.qknorm_rope_

    def counting_qk(*a, **k):
        calls["qk"] += 1
        return real_qk(*a, **k)

    monkeypatch.setattr(modules.ops, "qknorm_rope_", counting_qk)

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    monkeypatch.setattr(modules.ops, "norm_mod_quant", counting)
    with torch.no_grad():
        y_fused = blk(x, vec, rope, None)
        assert calls["n"] == 2 and calls["qk"] == 1
        monkeypatch.setattr(ditmod, "fused_prologue_ok", lambda *a: False)
        monkeypatch.setattr(ditmod, "qk_inplace_ok", lambda *a: False)
        y_plain = blk(x, vec, rope, None)
        assert calls["n"] == 2 and calls["qk"] == 1
    err = float((y_fused.float() - y_plain.float()).abs().max() / y_plain.float().abs().max())
    assert err <= 2e-2, err
    # with autograd on (training) the op-by-op route is taken
    monkeypatch.undo()
    xg = x.clone().requires_grad_(True)
    blk(xg, vec, None, None).float().sum().backward()
    assert xg.grad is not None


@pytest.mark.parametrize("bits", [8, 4])
def test_grouped_launches_equal_separate_launches(bits):
    """wq | wk | wv | gate and mlp.gate | mlp.up as one GEMM each over concatenated codes: the same bits
    as four + two launches (integer accumulation, same epilogue), no second copy of the codes, and a
    fall-back when a member is paged to other storage (mmdit.py:409-414)."""
    from k2q import dit as ditmod
    from k2q import modules
    torch.manual_seed(1)
    blk = ditmod.SingleStreamBlock(256, 2, 2, kvheads=1).cuda().to(torch.bfloat16)
    for p in blk.parameters():
        p.data.normal_(0, 0.05)
    holder = nn.Module()
    holder.blocks = nn.ModuleList([blk])
    modules.quantize_dit_convrot(holder, bits=bits)
    x = torch.randn(2, 200, 256, device="cuda").to(torch.bfloat16)
    vec = (torch.randn(2, 1, 6 * 256, device="cuda") * 0.1).to(torch.bfloat16)
    with torch.no_grad():
        y_sep = blk(x, vec, None, None)
        before = {k: v.clone() for k, v in blk.state_dict().items()}
        assert modules.group_shared_input_linears(holder) == 2
        g = blk.attn.qkvg_group
        assert g.out_features == 256 + 128 + 128 + 256 and blk.attn.wk.weight_q.data_ptr() != g.weight_q.data_ptr()
        assert blk.attn.wq.weight_q.data_ptr() == g.weight_q.data_ptr()          # members alias the group's storage
        after = blk.state_dict()
        assert all(torch.equal(before[k], after[k]) for k in before)             # nothing changed for the members
        y_grp = blk(x, vec, None, None)
        assert torch.equal(y_grp, y_sep)
        for p in blk.attn.wk.parameters():                                       # paged elsewhere: the group lets go
            p.data = p.data.clone()
        assert not g._aliased()
        assert torch.equal(blk(x, vec, None, None), y_sep)


@pytest.mark.parametrize("bits", [8, 4])
def test_column_parallel_block_on_one_rank_equals_the_plain_block(bits):
    """With a single rank the column split with local attention degenerates to the plain block (the gathers
    are identities); the sigmoid gate and SwiGLU then run as dense kernels followed by K2 instead of inside
    K2's load: the same roundings, so the outputs must be identical, grouped launches included."""
    from k2q import dit, modules, ops, parallel
    torch.manual_seed(13)
    dim, heads, kvheads, tokens = 768, 6, 3, 72
    holder = nn.Module()
    holder.blocks = nn.ModuleList([dit.SingleStreamBlock(dim, heads, 3, bias=True, kvheads=kvheads)])
    for prm in holder.parameters():
        prm.data.normal_(0.0, 0.04)
    holder = holder.to(torch.bfloat16).cuda()
    modules.quantize_dit_convrot(holder, bits=bits)
    x = torch.randn(2, tokens, dim, device="cuda").to(torch.bfloat16)
    vec = (torch.randn(2, 1, 6 * dim, device="cuda") * 0.1).to(torch.bfloat16)
    pos = torch.arange(tokens, device="cuda")[None, :, None].expand(2, tokens, 3)
    rope = dit.rope_tables(pos, [128 - 12 * 8, 48, 48], 1e4)
    with torch.no_grad():
        ref = holder.blocks[0](x, vec, rope)
        assert parallel.shard_dit_columns(holder, 0, 1) == 8 and isinstance(holder.blocks[0], parallel.ColumnParallelBlock)
        got = holder.blocks[0](x, vec, rope)
        assert modules.group_shared_input_linears(holder) == 2
        got_grouped = holder.blocks[0](x, vec, rope)
    ops.check_status(x.device)
    assert torch.equal(got, ref) and torch.equal(got_grouped, ref)
