"""Parity at the benchmark's full sizes (M = 8192 tokens, 3072 <-> 12288 features), where the CPU
oracle would take minutes.  Two kinds of check, both independent of the problem size:

* properties of the arithmetic: the rotation is an involution, every quantised row reaches +-127,
  codes times scale reproduce the rotated row to within half a quantisation step;
* the integer products against an independent integer GEMM on the same device
  (``torch._int_mm``, cuBLASLt int32 accumulation), followed by the oracle's epilogue order
  (``float(acc) * sx * sw + bias`` for int8; per-group ``float(acc_g) * s_g`` summed in group
  order, then ``* sx + bias`` for int4) evaluated with separate fp32 torch ops: bit-exact.

The small-size tests in test_gpu_kernels.py pin the same kernels to the CPU oracle itself.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

M, K, H = 8192, 3072, 12288


@pytest.fixture(scope="module")
def ops():
    from k2q import ops as _ops
    return _ops


def _int_mm(a, bt):
    """int32 = a[int8 M,K] @ bt[int8 K,N] on the GPU's library int8 path."""
    try:
        return torch._int_mm(a, bt)
    except (RuntimeError, AttributeError) as e:   # pragma: no cover - depends on the torch build
        pytest.skip(f"torch._int_mm unavailable here: {e}")


def _x(rows, cols, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    x[:, torch.randperm(cols, generator=g)[:8]] *= 20.0          # outlier channels
    return x.to(torch.bfloat16).cuda()


@pytest.mark.parametrize("cols", [K, H])
def test_k2_properties_at_full_size(ops, cols):
    x = _x(M, cols, 11)
    q, s = ops.fwht_quant_act(x)
    rot = ops.fwht_rows(x, out_dtype=torch.float32)
    # the row maximum maps to +-127 and nothing exceeds it
    assert int(q.abs().max()) == 127
    assert bool((q.abs().amax(dim=1) == 127).all())
    # scale = max|H(x)| / 127 exactly (IEEE fp32 division as in the oracle; evaluated on the CPU because
    # torch's CUDA division by a Python scalar multiplies by the reciprocal)
    assert torch.equal(s.cpu(), torch.clamp(rot.abs().amax(dim=1).cpu(), min=1e-8) / 127.0)
    # codes * scale reproduce the rotated row to half a step
    err = (q.float() * s[:, None] - rot).abs()
    assert bool((err <= 0.5 * s[:, None] * (1 + 1e-4)).all())   # the quotient itself is rounded to fp32 before rint
    # H(H(x)) = x up to fp32 rounding (orthonormal, symmetric blocks)
    back = ops.fwht_rows(rot, out_dtype=torch.float32)
    assert float((back - x.float()).abs().max()) <= 1e-5 * float(x.float().abs().max())
    ops.check_status()


def test_w8a8_against_library_int_gemm_at_full_size(ops):
    g = torch.Generator().manual_seed(5)
    x = _x(M, K, 12)
    w = (torch.randn(H, K, generator=g) * 0.02).to(torch.bfloat16).cuda()
    bias = (torch.randn(H, generator=g) * 0.01).cuda()
    wq, sw = ops.quant_weight_i8(w)
    xq, sx = ops.fwht_quant_act(x)
    y = ops.gemm_w8a8(xq, sx, wq, sw, bias)
    acc = _int_mm(xq, wq.t())                              # [M, H] int32; wq.t() is the column-major [K, H] view
    ref = acc.float()
    ref = ref * sx[:, None]
    ref = ref * sw[None, :]
    ref = ref + bias[None, :]
    assert torch.equal(y, ref.to(torch.bfloat16))
    # a second product with K = 12288 (the MLP's down projection)
    w2 = (torch.randn(K, H, generator=g) * 0.02).to(torch.bfloat16).cuda()
    wq2, sw2 = ops.quant_weight_i8(w2)
    hq, sh = ops.fwht_quant_act(y)
    y2 = ops.gemm_w8a8(hq, sh, wq2, sw2, None)
    ref2 = (_int_mm(hq, wq2.t()).float() * sh[:, None]) * sw2[None, :]
    assert torch.equal(y2, ref2.to(torch.bfloat16))
    ops.check_status()


def _unpack_int4(q4):
    """[N, K/2] packed (low nibble = even k, two's complement) -> [N, K] int8."""
    lo = (q4 & 0xF).to(torch.int16)
    hi = (q4 >> 4).to(torch.int16)
    lo = torch.where(lo > 7, lo - 16, lo)
    hi = torch.where(hi > 7, hi - 16, hi)
    return torch.stack([lo, hi], dim=-1).reshape(q4.shape[0], -1).to(torch.int8)


def test_w4a8_against_library_int_gemm_at_full_size(ops):
    g = torch.Generator().manual_seed(6)
    x = _x(M, K, 13)
    w = (torch.randn(H, K, generator=g) * 0.02).to(torch.bfloat16).cuda()
    wq4, sw4 = ops.quant_weight_i4(w)                     # [H, K/2] uint8, [H, K/128] bf16
    xq, sx = ops.fwht_quant_act(x)
    y = ops.gemm_w4a8(xq, sx, wq4, sw4, None)
    w8 = _unpack_int4(wq4)
    run = torch.zeros(M, H, device="cuda")
    for grp in range(K // 128):
        sl = slice(grp * 128, (grp + 1) * 128)
        acc = _int_mm(xq[:, sl].contiguous(), w8[:, sl].contiguous().t())
        run = (acc.double() * sw4[:, grp].double()[None, :] + run.double()).float()   # fused multiply-add
    ref = run * sx[:, None]
    assert torch.equal(y, ref.to(torch.bfloat16))
    ops.check_status()


def test_adapter_gemms_at_full_size(ops):
    g = torch.Generator().manual_seed(7)
    x = _x(M, K, 14)
    a = (torch.randn(32, K, generator=g) * 0.01).cuda()
    u = ops.lora_down(x, a)
    ref = x.double() @ a.double().t()
    assert float((u.double() - ref).abs().max()) <= 2e-4 * float(ref.abs().max())
    p = torch.randn(M, 32, generator=g).cuda()
    gA = ops.lora_tn(p, x)
    refA = p.double().t() @ x.double()
    assert float((gA.double() - refA).abs().max()) <= 2e-4 * float(refA.abs().max())
    assert torch.equal(gA, ops.lora_tn(p, x))              # fixed reduction order
    ops.check_status()
