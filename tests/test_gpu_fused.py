"""The fused elementwise steps of a DiT block (k2q.fused) against the op-by-op expressions of the
model code they replace: forward values equal up to one bf16 step where an fp32 sum was taken in
another order, gradients within 1e-2 (max relative error) of the same expression evaluated in fp32
-- no further from it than the eager bf16 autograd chain is."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close_bf16(got, ref, frac=0.99):
    g, r = got.float(), ref.float()
    step = r.abs().clamp_min(2.0 ** -120) * 2.0 ** -7
    assert bool(((g - r).abs() <= step).all()), float(((g - r).abs() / step).max())
    assert float((g == r).float().mean()) >= frac


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-30))


def _grads(fn, inputs, gy):
    xs = [t.clone().requires_grad_(True) for t in inputs]
    out = fn(*xs)
    out.backward(gy.to(out.dtype))
    return out.detach(), [x.grad for x in xs]


def test_norm_modulate_forward_and_backward():
    from k2q import dit as ditmod
    from k2q import fused
    torch.manual_seed(0)
    b, s, k = 2, 150, 768
    x = torch.randn(b, s, k, device=DEV).to(torch.bfloat16) * 1.7
    x[1, 3] = 0
    sc = (torch.randn(b, 1, k, device=DEV) * 0.2).to(torch.bfloat16)
    sh = (torch.randn(b, 1, k, device=DEV) * 0.2).to(torch.bfloat16)
    norm = ditmod.RMSNorm(k).to(DEV)
    norm.scale.data.normal_(0, 0.2)
    norm.scale.requires_grad_(False)
    gy = torch.randn(b, s, k, device=DEV).to(torch.bfloat16)
    for mods in ((sc, sh), (None, None)):
        eager = lambda t: ((1 + mods[0]) * norm(t) + mods[1]) if mods[0] is not None else norm(t)      # noqa: E731

        def exact(t):
            y = F.rms_norm(t.float(), (k,), weight=norm.scale + 1.0, eps=norm.eps)
            return (1 + mods[0].float()) * y + mods[1].float() if mods[0] is not None else y

        y_f, (g_f,) = _grads(lambda t: fused.norm_modulate(t, norm, *mods), [x], gy)
        y_e, (g_e,) = _grads(eager, [x], gy)
        _, (g_x,) = _grads(exact, [x], gy)
        _close_bf16(y_f, y_e)
        assert g_f.dtype == torch.bfloat16 and _rel(g_f, g_x) <= 1e-2 and _rel(g_f, g_x) <= 2 * _rel(g_e, g_x) + 1e-3
    # a modulation vector that needs its own gradient takes the op-by-op route
    scg = sc.clone().requires_grad_(True)
    fused.norm_modulate(x, norm, scg, sh).float().sum().backward()
    assert scg.grad is not None


def test_qk_norm_rope_training_forward_and_backward():
    from k2q import dit as ditmod
    from k2q import fused
    torch.manual_seed(1)
    b, s, hq, hk, d = 2, 96, 3, 1, 128
    q = torch.randn(b, s, hq * d, device=DEV).to(torch.bfloat16)
    k = torch.randn(b, s, hk * d, device=DEV).to(torch.bfloat16)
    norm = ditmod.QKNorm(d).to(DEV)
    norm.qnorm.scale.data.normal_(0, 0.2)
    norm.knorm.scale.data.normal_(0, 0.2)
    for p in norm.parameters():
        p.requires_grad_(False)
    pos = torch.stack((torch.zeros(s), torch.arange(s) // 8, torch.arange(s) % 8), dim=-1)[None].expand(b, -1, -1).to(DEV)
    rope = ditmod.rope_tables(pos, [32, 48, 48], 100.0)
    gq = torch.randn(b, hq, s, d, device=DEV).to(torch.bfloat16)
    gk = torch.randn(b, hk, s, d, device=DEV).to(torch.bfloat16)

    def eager(qt, kt, f32=False):
        qh = qt.view(b, s, hq, d).transpose(1, 2)
        kh = kt.view(b, s, hk, d).transpose(1, 2)
        if f32:
            qh = F.rms_norm(qh.float(), (d,), weight=norm.qnorm.scale + 1.0, eps=1e-5)
            kh = F.rms_norm(kh.float(), (d,), weight=norm.knorm.scale + 1.0, eps=1e-5)
        else:
            qh, kh = norm(qh, kh)
        return ditmod.rope_rotate(qh, *rope), ditmod.rope_rotate(kh, *rope)

    def run(fn):
        qt, kt = q.clone().requires_grad_(True), k.clone().requires_grad_(True)
        qo, ko = fn(qt, kt)
        torch.autograd.backward([qo, ko], [gq.to(qo.dtype), gk.to(ko.dtype)])
        return qo.detach(), ko.detach(), qt.grad, kt.grad

    assert fused.qk_norm_rope_trainable(q, k, norm, d)
    qo_f, ko_f, dq_f, dk_f = run(lambda a, c: fused.qk_norm_rope_train(a, c, norm, rope, b, s, hq, hk))
    qo_e, ko_e, dq_e, dk_e = run(eager)
    _, _, dq_x, dk_x = run(lambda a, c: eager(a, c, f32=True))
    _close_bf16(qo_f, qo_e)
    _close_bf16(ko_f, ko_e)
    assert qo_f.shape == (b, hq, s, d) and ko_f.shape == (b, hk, s, d)
    for got, ref, eag in ((dq_f, dq_x, dq_e), (dk_f, dk_x, dk_e)):
        assert got.dtype == torch.bfloat16 and _rel(got, ref) <= 1e-2 and _rel(got, ref) <= 2 * _rel(eag, ref) + 1e-3
    # gradients that arrive as [B, S, H, D] memory behind a transposed view (what flash attention returns)
    gq2 = gq.transpose(1, 2).contiguous().transpose(1, 2)
    qt, kt = q.clone().requires_grad_(True), k.clone().requires_grad_(True)
    qo, ko = fused.qk_norm_rope_train(qt, kt, norm, rope, b, s, hq, hk)
    torch.autograd.backward([qo, ko], [gq2, gk])
    assert torch.equal(qt.grad, dq_f)


@pytest.mark.parametrize("kind", ["swiglu", "sigmoid_gate"])
def test_pair_ops_forward_and_backward(kind):
    from k2q import fused
    torch.manual_seed(2)
    m, k = 333, 1032
    a = (torch.randn(2, m, k, device=DEV) * 2).to(torch.bfloat16)
    c = (torch.randn(2, m, k, device=DEV) * 2).to(torch.bfloat16)
    gy = torch.randn(2, m, k, device=DEV).to(torch.bfloat16)
    if kind == "swiglu":
        fn, eager = fused.swiglu, lambda g, u: F.silu(g) * u
        exact = lambda g, u: F.silu(g.float()) * u.float()                      # noqa: E731
    else:
        fn, eager = fused.sigmoid_gate, lambda t, g: t * torch.sigmoid(g)
        exact = lambda t, g: t.float() * torch.sigmoid(g.float())               # noqa: E731
    y_f, g_f = _grads(fn, [a, c], gy)
    y_e, g_e = _grads(eager, [a, c], gy)
    _, g_x = _grads(exact, [a, c], gy)
    _close_bf16(y_f, y_e, frac=0.98)
    for got, ref, eag in zip(g_f, g_x, g_e):
        assert got.dtype == torch.bfloat16 and _rel(got, ref) <= 1e-2 and _rel(got, ref) <= 2 * _rel(eag, ref) + 1e-3
    # a strided first operand (column block of a wider tensor) is read in place
    wide = torch.randn(m, 2 * k, device=DEV).to(torch.bfloat16)
    assert torch.equal(fn(wide[:, :k], c[0]), fn(wide[:, :k].contiguous(), c[0]))


def test_gate_residual_forward_and_backward():
    from k2q import fused
    torch.manual_seed(3)
    b, s, k = 2, 77, 640
    x = torch.randn(b, s, k, device=DEV).to(torch.bfloat16)
    y = torch.randn(b, s, k, device=DEV).to(torch.bfloat16)
    gate = torch.randn(b, 1, k, device=DEV).to(torch.bfloat16)
    gy = torch.randn(b, s, k, device=DEV).to(torch.bfloat16)
    out_f, (dx_f, dy_f) = _grads(lambda t, u: fused.gate_residual(t, gate, u), [x, y], gy)
    out_e, (dx_e, dy_e) = _grads(lambda t, u: t + gate * u, [x, y], gy)
    assert torch.equal(out_f, out_e) and torch.equal(dx_f, dx_e) and torch.equal(dy_f, dy_e)
    gg = gate.clone().requires_grad_(True)           # a gate that needs a gradient: op-by-op route
    fused.gate_residual(x, gg, y).float().sum().backward()
    assert gg.grad is not None and gg.grad.shape == gate.shape


def test_block_with_fused_steps_trains_like_the_op_by_op_block(monkeypatch):
    """One block of the harness DiT at head dimension 128, forward + backward through ConvRot bases with
    adapters: with the fused steps and with every step forced onto its op-by-op expression."""
    import torch.nn as nn
    from k2q import dit as ditmod
    from k2q import fused, lora, modules
    torch.manual_seed(4)
    blk = ditmod.SingleStreamBlock(256, 2, 2, kvheads=1).to(DEV).to(torch.bfloat16)
    for p in blk.parameters():
        p.data.normal_(0, 0.05)
        p.requires_grad_(False)
    holder = nn.Module()
    holder.blocks = nn.ModuleList([blk])
    modules.quantize_dit_convrot(holder, bits=8)
    ads = {}
    for tag, parent in (("attn", blk.attn), ("mlp", blk.mlp)):
        for name, child in list(parent.named_children()):
            if isinstance(child, modules.ConvRotLinear):
                ad = ads[f"{tag}.{name}"] = lora.LoRALinear(child, 8, 8.0)
                ad.lora_B.data.normal_(0, 0.05)
                setattr(parent, name, ad)
    assert len(ads) == 8 and lora.fuse_lora(holder) == 8
    params = lora.lora_parameters(ads)
    x = torch.randn(2, 96, 256, device=DEV).to(torch.bfloat16)
    vec = (torch.randn(2, 1, 6 * 256, device=DEV) * 0.1).to(torch.bfloat16)
    pos = torch.stack((torch.zeros(96), torch.arange(96) // 8, torch.arange(96) % 8), dim=-1)[None].expand(2, -1, -1).to(DEV)
    rope = ditmod.rope_tables(pos, [32, 48, 48], 100.0)

    def run():
        for p in params:
            p.grad = None
        xg = x.clone().requires_grad_(True)
        out = blk(xg, vec, rope, None)
        out.float().pow(2).mean().backward()
        return out.detach(), xg.grad, [p.grad.clone() for p in params]

    out_f, dx_f, gp_f = run()
    monkeypatch.setattr(fused, "_kernel_ok", lambda *a: False)
    out_e, dx_e, gp_e = run()
    assert _rel(out_f, out_e) <= 2e-2 and _rel(dx_f, dx_e) <= 3e-2
    worst = max(_rel(a, c) for a, c in zip(gp_f, gp_e))
    assert worst <= 5e-2, worst


def test_sibling_adapters_share_one_down_projection(monkeypatch):
    """Adapters of wq|wk|wv|gate and of mlp gate|up read one tensor: after ``fuse_lora`` their x . A^T runs as
    one pass with the A matrices stacked.  Outputs and every gradient agree with the unlinked adapters, the pass
    count drops from 6 to 2 per block forward, ``lora_scaled(0)`` on the whole model and a changed A are seen."""
    import torch.nn as nn
    from k2q import dit as ditmod
    from k2q import lora, modules, ops
    torch.manual_seed(6)
    blk = ditmod.SingleStreamBlock(256, 2, 2, kvheads=1).to(DEV).to(torch.bfloat16)
    for p in blk.parameters():
        p.data.normal_(0, 0.05)
        p.requires_grad_(False)
    holder = nn.Module()
    holder.blocks = nn.ModuleList([blk])
    modules.quantize_dit_convrot(holder, bits=8)
    ads = []
    for parent in (blk.attn, blk.mlp):
        for name, child in list(parent.named_children()):
            if isinstance(child, modules.ConvRotLinear):
                ad = lora.LoRALinear(child, 8, 8.0)
                ad.lora_B.data.normal_(0, 0.05)
                setattr(parent, name, ad)
                ads.append(ad)
    assert lora.fuse_lora(holder) == 8
    linked = [a for a in ads if getattr(a, "_k2q_sibs", None)]
    assert len(linked) == 6 and blk.attn.wq._k2q_sibs == (blk.attn.wq, blk.attn.wk, blk.attn.wv, blk.attn.gate)
    assert [m._k2q_sib_off for m in blk.attn.wq._k2q_sibs] == [0, 8, 16, 24] and blk.mlp.up._k2q_sib_off == 8
    params = lora.lora_parameters({str(i): a for i, a in enumerate(ads)})
    x = torch.randn(2, 96, 256, device=DEV).to(torch.bfloat16)
    vec = (torch.randn(2, 1, 6 * 256, device=DEV) * 0.1).to(torch.bfloat16)
    pos = torch.stack((torch.zeros(96), torch.arange(96) // 8, torch.arange(96) % 8), dim=-1)[None].expand(2, -1, -1).to(DEV)
    rope = ditmod.rope_tables(pos, [32, 48, 48], 100.0)
    downs = {"n": 0}
    real_down = ops.lora_down

    def counting_down(xx, a, *args, **kw):
        if not kw.get("transposed", False) and not (len(args) > 1 and args[1]):
            downs["n"] += 1
        return real_down(xx, a, *args, **kw)

    monkeypatch.setattr(ops, "lora_down", counting_down)

    def run():
        for p in params:
            p.grad = None
        downs["n"] = 0
        xg = x.clone().requires_grad_(True)
        out = blk(xg, vec, rope, None)
        fwd_downs = downs["n"]
        out.float().pow(2).mean().backward()
        return out.detach(), xg.grad, [p.grad.clone() for p in params], fwd_downs

    out_s, dx_s, gp_s, n_s = run()
    saved = [(a._k2q_sibs, a._k2q_sib_off) for a in linked]
    for a in linked:
        del a._k2q_sibs, a._k2q_sib_off
    out_u, dx_u, gp_u, n_u = run()
    assert (n_s, n_u) == (4, 8)                 # qkvg and gate|up once each, wo and down on their own
    assert _rel(out_s, out_u) <= 1e-3 and _rel(dx_s, dx_u) <= 1e-3
    assert max(_rel(a, c) for a, c in zip(gp_s, gp_u)) <= 1e-3
    for a, (sibs, off) in zip(linked, saved):
        a._k2q_sibs, a._k2q_sib_off = sibs, off
    # a changed A is seen by the next forward (nothing outlives the block scope); adapters switched off bypass it
    blk.attn.wk.lora_A.data.mul_(2.0)
    out_2, _, _, _ = run()
    assert not torch.equal(out_2, out_s)
    with lora.lora_scaled(holder, 0.0):
        downs["n"] = 0
        with torch.no_grad():
            blk(x, vec, rope, None)
        assert downs["n"] == 0
    ops.check_status()
