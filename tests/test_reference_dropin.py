"""Drop-in test against the REFERENCE's own modules (CPU, skipped where the reference checkout is
absent): the ConvRot replacement must work under the reference's ``SingleStreamDiT`` (mmdit.py),
``inject_lora`` / ``lora_scaled`` / ``lora_disabled`` / ``lora_parameters`` (lora.py:51-123), gradient
checkpointing (mmdit.py:474-481) and block swap (mmdit.py:389-428) exactly where ``Fp8Linear``
(quantize.py:23-68) does -- with nothing of the reference edited.

There is no GPU here, so the two device quantisers and the functional forward are replaced by the
CPU oracle for the duration of a test (``monkeypatch``); everything else -- module surgery, the
duck type, the hooks that scope the shared input quantisation, the class retargeting of
``fuse_lora`` on the reference's ``LoRALinear`` -- is the shipped code.
"""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

from oracle import convrot_ref as R

# the reference checkout: K2Q_REFERENCE_DIR, or a directory "reference" beside this repository
REF = Path(os.environ.get("K2Q_REFERENCE_DIR", Path(__file__).resolve().parents[2] / "reference"))
pytestmark = pytest.mark.skipif(not (REF / "mmdit.py").exists(), reason="reference checkout not present")

TINY = dict(features=128, tdim=32, txtdim=64, heads=2, kvheads=1, multiplier=1, layers=2, patch=2, channels=4,
            txtheads=2, txtkvheads=2, txtlayers=3)


@pytest.fixture()
def ref(monkeypatch):
    """The reference's modules, importable as it ships them, with its CUDA-only attention backend
    pin (mmdit.py:41) replaced by the plain SDPA call for the CPU run."""
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    monkeypatch.syspath_prepend(str(REF))
    import lora as ref_lora
    import mmdit as ref_mmdit
    import quantize as ref_quant
    from einops import rearrange

    def cpu_attention(q, k, v, mask=None, scale=None, gqa=False):
        return rearrange(F.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=scale, enable_gqa=gqa),
                         "B H L D -> B L (H D)")

    monkeypatch.setattr(ref_mmdit, "attention", cpu_attention)
    yield ref_mmdit, ref_lora, ref_quant
    for name in ("lora", "mmdit", "quantize"):
        sys.modules.pop(name, None)


class _OracleLinearFn(torch.autograd.Function):
    """O-exact forward from the module's codes, straight-through backward dX = dY . W_eff."""

    @staticmethod
    def forward(ctx, x, mod):
        x2 = x.reshape(-1, x.shape[-1])
        xq, sx = R.quantize_act_int8(x2)
        exact = R.linear_int8_exact if mod.bits == 8 else R.linear_int4_exact
        bias = mod.bias.data.float() if mod.bias is not None else None
        y = exact(xq, sx.reshape(-1), mod.weight_q.data, mod.scale, bias)
        ctx.mod = mod
        return y.reshape(*x.shape[:-1], mod.out_features).to(x.dtype)

    @staticmethod
    def backward(ctx, gy):
        mod = ctx.mod
        w_eff = R.effective_weight(mod.weight_q.data, mod.scale, mod.bits)
        return (gy.float() @ w_eff).to(gy.dtype), None


def _cpu_convrot(monkeypatch):
    from k2q import lora as klora
    from k2q import modules, ops
    calls = {"quant": 0}
    monkeypatch.setattr(ops, "quant_weight_i8", lambda w: R.quantize_weight_int8(w))
    monkeypatch.setattr(ops, "quant_weight_i4", lambda w: R.quantize_weight_int4(w))
    monkeypatch.setattr(ops, "transpose_i8", lambda q: q.t().contiguous())

    def convrot_linear(x, mod, lora_a=None, lora_b=None, lora_scale=0.0, sibs=None, sib_off=0):
        calls["quant"] += 1
        y = _OracleLinearFn.apply(x, mod)
        if lora_a is not None and lora_scale != 0.0:
            y = y + lora_scale * ((x.to(lora_a.dtype) @ lora_a.t()) @ lora_b.t()).to(y.dtype)
        return y

    monkeypatch.setattr(modules, "convrot_linear", convrot_linear)
    monkeypatch.setattr(klora, "convrot_linear", convrot_linear)
    return calls


def _inputs(seed=11):
    g = torch.Generator().manual_seed(seed)
    b, gh, gw, l = 2, 4, 6, 9
    z = torch.randn(b, gh * gw, 16, generator=g)
    ctx = torch.randn(b, l, 3, 64, generator=g)
    t = torch.tensor([0.25, 0.9])
    ys, xs = torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij")
    img_pos = torch.stack([torch.zeros_like(ys), ys, xs], dim=-1).reshape(1, gh * gw, 3).expand(b, -1, -1)
    txt_pos = torch.zeros(b, l, 3, dtype=img_pos.dtype)
    pos = torch.cat([txt_pos, img_pos], dim=1).float()
    mask = torch.ones(b, l + gh * gw, dtype=torch.bool)
    return z, ctx, t, pos, mask


def _seeded(model, scale=0.05):
    import zlib
    for name, p in model.named_parameters():
        g = torch.Generator().manual_seed(zlib.crc32(name.encode()))
        p.data = (torch.randn(p.shape, generator=g) * scale).to(p.dtype)


@pytest.mark.parametrize("bits", [8, 4])
def test_reference_dit_with_convrot_base_lora_checkpoint_and_block_swap(ref, monkeypatch, bits):
    ref_mmdit, ref_lora, ref_quant = ref
    from k2q import lora as klora
    from k2q import modules
    calls = _cpu_convrot(monkeypatch)

    twin = ref_mmdit.SingleStreamDiT(ref_mmdit.SingleMMDiTConfig(**TINY))
    n_fp8 = ref_quant.quantize_dit_fp8(twin)                       # the function being replaced

    dit = ref_mmdit.SingleStreamDiT(ref_mmdit.SingleMMDiTConfig(**TINY))
    _seeded(dit)
    n = modules.quantize_dit_convrot(dit, bits=bits)
    assert n == n_fp8                                               # same traversal, same count
    for (ka, ma), (kb, mb) in zip(dit.named_modules(), twin.named_modules()):
        assert ka == kb
        assert isinstance(ma, modules.ConvRotLinear) == isinstance(mb, ref_quant.Fp8Linear), ka
    assert isinstance(dit.first, torch.nn.Module) and not isinstance(dit.first, modules.ConvRotLinear)

    z, ctx, t, pos, mask = _inputs()
    dit.eval()
    with torch.no_grad():
        calls["quant"] = 0
        y_base = dit(z, ctx, t, pos, mask)
    assert torch.isfinite(y_base).all() and calls["quant"] == n

    # the reference's own adapter surgery on the ConvRot bases (is_quant_linear duck type, lora.py:100)
    adapters = ref_lora.inject_lora(dit, rank=4, alpha=4.0)
    on_convrot = [a for a in adapters.values() if isinstance(a.base, modules.ConvRotLinear)]
    assert len(on_convrot) == n and all(type(a) is ref_lora.LoRALinear for a in adapters.values())
    g = torch.Generator().manual_seed(3)
    for a in adapters.values():
        a.lora_B.data = torch.randn(a.lora_B.shape, generator=g) * 0.05
    params = ref_lora.lora_parameters(adapters)
    assert len(params) == 2 * len(adapters) and all(p.requires_grad for p in params)
    assert not any(p.requires_grad for a in on_convrot for p in a.base.parameters())

    with torch.no_grad():
        y_plain = dit(z, ctx, t, pos, mask)                         # reference LoRALinear.forward, unfused
    assert klora.fuse_lora(dit) == n                                # only adapters on ConvRot bases are retargeted
    assert all(isinstance(a, ref_lora.LoRALinear) for a in adapters.values())   # lora_scaled finds them by isinstance
    assert all(getattr(a, "is_fused_lora", False) == isinstance(a.base, modules.ConvRotLinear) for a in adapters.values())
    # adapters of Linears that read one tensor (wq|wk|wv|gate, mlp gate|up) are linked for a shared down-projection
    linked = [a for a in adapters.values() if getattr(a, "_k2q_sibs", None)]
    assert linked and all(a._k2q_sibs[0]._k2q_sib_off == 0 and any(a is m for m in a._k2q_sibs) for a in linked)
    assert all(sum(m.rank for m in a._k2q_sibs) <= 64 and len({m.base.in_features for m in a._k2q_sibs}) == 1 for a in linked)
    with torch.no_grad():
        y_fused = dit(z, ctx, t, pos, mask)
        assert torch.allclose(y_fused, y_plain, rtol=1e-4, atol=1e-5)
        with ref_lora.lora_scaled(dit, -1.5):
            assert all(a.scale_mul == -1.5 for a in adapters.values())
            y_neg = dit(z, ctx, t, pos, mask)
        with ref_lora.lora_disabled(dit):
            y_off = dit(z, ctx, t, pos, mask)
        assert all(a.scale_mul == 1.0 for a in adapters.values())
    assert torch.equal(y_off, y_base)                               # scale_mul == 0 early-out: the frozen base
    assert not torch.equal(y_neg, y_fused) and not torch.equal(y_fused, y_base)

    # training step as the trainer runs it: checkpointed blocks, the deepest block paged (mmdit.py:389-418)
    swapped = dit.enable_block_swap(1, "cpu")
    assert swapped == [TINY["layers"] - 1]
    dit.gradient_checkpointing = True
    dit.train()
    out = dit(z, ctx, t, pos, mask)
    out.float().pow(2).mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in params)
    assert any(float(p.grad.abs().max()) > 0 for p in params)
    assert all(p.grad is None for a in on_convrot for p in a.base.parameters())
    state = dit.blocks[-1].state_dict()
    assert any(k.endswith("weight_q") for k in state) and all(v.device.type == "cpu" for v in state.values())

    # leaving a block forward leaves the shared-quantisation scope, even through checkpoint recompute
    assert modules._scope.depth == 0 and modules._scope.codes is None

    # un-fusing restores the reference class itself
    assert klora.unfuse_lora(dit) == n and all(type(a) is ref_lora.LoRALinear for a in adapters.values())
