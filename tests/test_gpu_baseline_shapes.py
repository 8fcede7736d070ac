"""Parity at the shapes BASELINE.json's single-layer configurations are quoted on, against the CPU
oracle at full size (seconds of CPU work each):

* configs[0]: ConvRot int8 Linear 3072x3072 with bias and a rank-16 adapter, X [4096, 3072] with
  eight x20 outlier channels -- spread over the row (canonical) and all inside ONE Hadamard block
  (channels 0..7, the adversarial case for a per-token quantiser); forward.
* configs[2]: the same layer with a rank-32 adapter (alpha 32), forward + backward with
  dY ~ N(0, 1e-2): y, dX through the quantised weights, dA, dB.
* the real architecture's long contractions: a forward GEMM at K = 16384 (mlp.down, 16384 -> 6144)
  and a backward dX whose contraction runs over N = 16384 (mlp.gate / mlp.up, 6144 -> 16384), where
  the error of the per-token int8 dY grows with the contraction length; int4 dX at 3072 x 3072.

Tolerances: base outputs bit-exact against O-exact; everything that involves an adapter or a backward
<= 2e-2 max-relative-error (max|y - y_ref| / max|y_ref|), the bound the path is specified with.
"""
import pytest
import torch
import torch.nn as nn

from oracle import convrot_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _layer(n, k, bits, rank, alpha, bias=True, seed=0, backward_copy=True):
    from k2q import lora, modules
    w = R.synth_weight(n, k, seed=1000 + seed)
    b = R.synth_vec(n, 0.01, 3000 + seed).to(torch.bfloat16).float() if bias else None
    lin = nn.Linear(k, n, bias=bias, device=DEV, dtype=torch.bfloat16)
    lin.weight.data.copy_(w)
    if bias:
        lin.bias.data.copy_(b)
    base = modules.ConvRotLinear(lin, bits=bits, backward_copy=backward_copy)
    ad = None
    if rank:
        ad = lora.LoRALinear(base, rank, float(alpha))
        ad.lora_A.data.copy_(R.synth_mat(rank, k, 0.01, 4000 + seed))
        ad.lora_B.data.copy_(R.synth_mat(n, rank, 0.01, 5000 + seed))
        lora.fuse_lora(ad)
    return base, w, b, ad


def _oracle_grads(x, w_eff, bias, a, b, s, gy):
    """Autograd through the reference formula (lora.py:47-48 over F.linear with the de-rotated
    dequantised weight) in fp32 on CPU."""
    x = x.float().clone().requires_grad_(True)
    a = a.clone().requires_grad_(True)
    b = b.clone().requires_grad_(True)
    y = torch.nn.functional.linear(x, w_eff, bias) + s * ((x @ a.t()) @ b.t())
    y.backward(gy.float())
    return x.grad, a.grad, b.grad


@pytest.mark.parametrize("adversarial", [False, True])
def test_config0_int8_linear_rank16_forward(adversarial):
    from k2q import ops
    m, n, k, rank = 4096, 3072, 3072, 16
    base, w, bias, ad = _layer(n, k, 8, rank, 16.0)
    x = R.synth_act(m, k, seed=2000, outliers=8, adversarial=adversarial)
    with torch.no_grad():
        y_base = base(x.to(DEV)).cpu()
        y = ad(x.to(DEV)).cpu()
    ops.check_status()
    q, sw = R.quantize_weight_int8(w)
    assert torch.equal(base.weight_q.cpu(), q) and torch.equal(base.scale.cpu(), sw)
    xq, sx = R.quantize_act_int8(x)
    exact = R.linear_int8_exact(xq, sx, q, sw, bias)
    assert torch.equal(y_base.view(torch.int16), exact.view(torch.int16))
    assert R.max_rel_err(y_base, R.linear_sim_dequant(xq, sx, q, sw, 8, bias.to(torch.bfloat16))) <= 2e-2
    a, b = ad.lora_A.detach().cpu(), ad.lora_B.detach().cpu()
    assert R.max_rel_err(y, R.lora_forward_ref(exact, x, a, b, 1.0)) <= 2e-2


def test_config2_int8_linear_rank32_forward_backward():
    from k2q import ops
    m, n, k, rank = 4096, 3072, 3072, 32
    base, w, bias, ad = _layer(n, k, 8, rank, 32.0)
    x = R.synth_act(m, k, seed=2000, outliers=8)
    gy = R.synth_mat(m, n, 1e-2, 6000).to(torch.bfloat16)
    xd = x.to(DEV).requires_grad_(True)
    y = ad(xd)
    y.backward(gy.to(DEV))
    ops.check_status()
    q, sw = R.quantize_weight_int8(w)
    xq, sx = R.quantize_act_int8(x)
    a, b = ad.lora_A.detach().cpu(), ad.lora_B.detach().cpu()
    y_ref = R.lora_forward_ref(R.linear_int8_exact(xq, sx, q, sw, bias), x, a, b, 1.0)
    assert R.max_rel_err(y.detach().cpu(), y_ref) <= 2e-2
    gx, ga, gb = _oracle_grads(x, R.effective_weight(q, sw, 8), bias, a, b, 1.0, gy)
    assert R.max_rel_err(xd.grad.cpu(), gx) <= 2e-2
    assert R.max_rel_err(ad.lora_A.grad.cpu(), ga) <= 2e-2
    assert R.max_rel_err(ad.lora_B.grad.cpu(), gb) <= 2e-2
    assert all(p.grad is None for p in base.parameters())       # the frozen base gets no gradient


@pytest.mark.parametrize("bits", [8, 4])
def test_forward_gemm_with_contraction_16384(bits):
    """mlp.down of the real architecture: 16384 -> 6144 (128 rotation blocks / int4 groups per row)."""
    from k2q import ops
    m, n, k = 256, 6144, 16384
    base, w, _, _ = _layer(n, k, bits, 0, 0, bias=False, seed=3, backward_copy=False)
    x = R.synth_act(m, k, seed=2003, outliers=8)
    with torch.no_grad():
        y = base(x.to(DEV)).cpu()
    ops.check_status()
    xq, sx = R.quantize_act_int8(x)
    if bits == 8:
        q, s = R.quantize_weight_int8(w)
        exact = R.linear_int8_exact(xq, sx, q, s)
    else:
        q, s = R.quantize_weight_int4(w)
        exact = R.linear_int4_exact(xq, sx, q, s)
    assert torch.equal(base.weight_q.cpu(), q)
    assert torch.equal(y.view(torch.int16), exact.view(torch.int16))
    assert R.max_rel_err(y, R.linear_sim_dequant(xq, sx, q, s, bits)) <= 2e-2


def test_backward_dx_with_contraction_16384():
    """mlp.gate / mlp.up of the real architecture: 6144 -> 16384; dX = dY . W contracts over 16384
    output channels with dY quantised to int8 per token."""
    from k2q import ops
    m, n, k = 512, 16384, 6144
    base, w, _, _ = _layer(n, k, 8, 0, 0, bias=False, seed=4)
    x = R.synth_act(m, k, seed=2004, outliers=8)
    gy = R.synth_mat(m, n, 1e-2, 6004).to(torch.bfloat16)
    xd = x.to(DEV).requires_grad_(True)
    base(xd).backward(gy.to(DEV))
    ops.check_status()
    q, sw = R.quantize_weight_int8(w)
    gx = gy.float() @ R.effective_weight(q, sw, 8)
    assert R.max_rel_err(xd.grad.cpu(), gx) <= 2e-2


def test_int4_backward_dx_at_3072():
    from k2q import ops
    m, n, k = 1024, 3072, 3072
    base, w, _, _ = _layer(n, k, 4, 0, 0, bias=False, seed=5)
    x = R.synth_act(m, k, seed=2005, outliers=8)
    gy = R.synth_mat(m, n, 1e-2, 6005).to(torch.bfloat16)
    xd = x.to(DEV).requires_grad_(True)
    base(xd).backward(gy.to(DEV))
    ops.check_status()
    q, s = R.quantize_weight_int4(w)
    gx = gy.float() @ R.effective_weight(q, s, 4)
    assert R.max_rel_err(xd.grad.cpu(), gx) <= 2e-2
