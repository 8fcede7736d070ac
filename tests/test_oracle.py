"""CPU tests of the oracle: against golden vectors produced by the reference's own modules, against
an independent numpy restatement, and through size-independent properties."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import convrot_ref as R

GOLD = Path(__file__).resolve().parent / "golden"


def test_fp8_and_lora_restatements_match_reference_goldens():
    """quantize.Fp8Linear and lora.LoRALinear (run from the reference's source) vs the oracle's
    restatements: bit-exact forward, and the gradients autograd gives through the restated formula."""
    cases = torch.load(GOLD / "ref_fp8_lora.pt")
    assert len(cases) == 3
    for c in cases:
        y_fp8, wq, scale = R.fp8_linear_ref(c["w"], c["bias"], c["x"])
        assert torch.equal(wq.view(torch.uint8), c["fp8_weight"])
        assert torch.equal(scale, c["fp8_scale"])
        assert torch.equal(y_fp8, c["y_fp8"])
        a = c["lora_A"].clone().requires_grad_(True)
        b = c["lora_B"].clone().requires_grad_(True)
        x = c["x"].clone().requires_grad_(True)
        base, _, _ = R.fp8_linear_ref(c["w"], c["bias"], x)
        y = R.lora_forward_ref(base, x, a, b, c["alpha"] / c["rank"], c["scale_mul"])
        assert torch.equal(y.detach(), c["y"])
        y.backward(c["gy"])
        assert torch.equal(x.grad, c["dx"])
        if c["scale_mul"] == 0.0:
            assert c["dA"] is None and a.grad is None       # adapters off: early return (lora.py:45-46)
        else:
            assert torch.equal(a.grad, c["dA"]) and torch.equal(b.grad, c["dB"])


def test_convrot_goldens_reproduce():
    for c in torch.load(GOLD / "convrot_small.pt"):
        q8, s8 = R.quantize_weight_int8(c["w"])
        q4, s4 = R.quantize_weight_int4(c["w"])
        xq, sx = R.quantize_act_int8(c["x"])
        assert torch.equal(q8, c["q8"]) and torch.equal(s8, c["s8"])
        assert torch.equal(q4, c["q4"]) and torch.equal(s4.view(torch.int16), c["s4"].view(torch.int16))
        assert torch.equal(xq, c["xq"]) and torch.equal(sx, c["sx"])
        assert torch.equal(R.linear_int8_exact(xq, sx, q8, s8, c["bias"]).view(torch.int16), c["y8"].view(torch.int16))
        assert torch.equal(R.linear_int4_exact(xq, sx, q4, s4, c["bias"]).view(torch.int16), c["y4"].view(torch.int16))


def _hadamard_numpy(x: np.ndarray) -> np.ndarray:
    """Independent restatement: explicit index loops over one 128-block, float32 arithmetic."""
    v = x.astype(np.float32).copy()
    h = 1
    while h < 128:
        for i in range(128):
            if (i & h) == 0:
                a, b = v[i], v[i + h]
                v[i], v[i + h] = np.float32(a + b), np.float32(a - b)
        h *= 2
    return (v * np.float32(2.0 ** -3.5)).astype(np.float32)


def test_hadamard_matches_index_loop_and_matrix():
    x = torch.randn(3, 256, generator=torch.Generator().manual_seed(0))
    y = R.hadamard128(x)
    for r in range(3):
        for blk in range(2):
            ref = _hadamard_numpy(x[r, blk * 128:(blk + 1) * 128].numpy())
            assert np.array_equal(y[r, blk * 128:(blk + 1) * 128].numpy(), ref)
    hmat = torch.tensor([[1.0]], dtype=torch.float64)
    while hmat.shape[0] < 128:
        hmat = torch.cat((torch.cat((hmat, hmat), 1), torch.cat((hmat, -hmat), 1)), 0)
    ym = (x.double().reshape(3, 2, 128) @ hmat).reshape(3, 256) * 2.0 ** -3.5
    assert (y.double() - ym).abs().max() < 1e-5


def test_hadamard_properties():
    x = torch.randn(16, 1024, generator=torch.Generator().manual_seed(1))
    y = R.hadamard128(x)
    assert (R.hadamard128(y) - x).abs().max() < 1e-5                       # involution
    assert torch.allclose(y.pow(2).sum(-1), x.pow(2).sum(-1), rtol=1e-5)   # orthonormal
    a, b = x[:8], x[8:]
    assert (R.hadamard128(a + b) - (R.hadamard128(a) + R.hadamard128(b))).abs().max() < 1e-4   # linear
    with pytest.raises(ValueError):
        R.hadamard128(torch.zeros(2, 100))


def test_quantizers_numpy_cross_check_and_edges():
    x = torch.zeros(5, 256)
    x[1, 7] = 3.0
    x[2] = torch.randn(256, generator=torch.Generator().manual_seed(2))
    x[3] = 0.25
    x[4, 128:] = torch.randn(128, generator=torch.Generator().manual_seed(3)) * 100
    q, s = R.quantize_act_int8(x)
    xr = R.hadamard128(x).numpy()
    s_np = np.maximum(np.abs(xr).max(axis=1, keepdims=True), np.float32(1e-8)) / np.float32(127)
    q_np = np.clip(np.rint(xr / s_np), -127, 127).astype(np.int8)
    assert np.array_equal(q.numpy(), q_np) and np.array_equal(s.numpy(), s_np)
    assert float(s[0]) == pytest.approx(1e-8 / 127, rel=1e-6) and int(q[0].abs().max()) == 0
    assert int(q.abs().max()) == 127
    p, s4 = R.quantize_weight_int4(x)
    codes = R.unpack_int4(p)
    assert codes.abs().max() <= 7 and s4.shape == (5, 2) and s4.dtype == torch.bfloat16
    lo = (p & 0xF).to(torch.int16)
    assert torch.equal(torch.where(lo >= 8, lo - 16, lo).to(torch.int8), codes[:, 0::2])   # low nibble = even k


def test_pack_unpack_round_trip_all_codes():
    codes = torch.arange(-8, 8, dtype=torch.int16).repeat(16).reshape(2, 128)
    packed = ((codes[:, 0::2] & 0xF) | ((codes[:, 1::2] & 0xF) << 4)).to(torch.uint8)
    assert torch.equal(R.unpack_int4(packed), codes.to(torch.int8))


def test_int_matmul_exact_and_forward_oracles_agree():
    g = torch.Generator().manual_seed(4)
    xq = torch.randint(-127, 128, (40, 2304), generator=g, dtype=torch.int8)
    wq = torch.randint(-127, 128, (24, 2304), generator=g, dtype=torch.int8)
    assert torch.equal(R.int_matmul(xq, wq).to(torch.int64), xq.to(torch.int64) @ wq.to(torch.int64).t())
    xs = torch.full((40, 1), 127, dtype=torch.int8).repeat(1, 2304)          # worst case magnitude
    assert int(R.int_matmul(xs, xs[:3])[0, 0]) == 127 * 127 * 2304
    w = R.synth_weight(64, 512, seed=9)
    x = R.synth_act(32, 512, seed=10, outliers=4)
    q8, s8 = R.quantize_weight_int8(w)
    q4, s4 = R.quantize_weight_int4(w)
    xq, sx = R.quantize_act_int8(x)
    for bits, q, s, exact in ((8, q8, s8, R.linear_int8_exact), (4, q4, s4, R.linear_int4_exact)):
        y = exact(xq, sx, q, s)
        assert R.max_rel_err(y, R.linear_sim_dequant(xq, sx, q, s, bits)) <= 2e-2
        assert R.max_rel_err(y, R.linear_ref_weight_only(x, q, s, bits)) <= 5e-2
    # rotation identity behind the backward oracle: x . W_eff^T == H(x) . W_dq^T
    w_eff = R.effective_weight(q8, s8, 8)
    lhs = x.float() @ w_eff.t()
    rhs = R.hadamard128(x.float()) @ R.dequant_weight_rot(q8, s8, 8).t()
    assert (lhs - rhs).abs().max() <= 1e-4 * rhs.abs().max()


def test_ref_module_has_quant_linear_protocol_and_ste_backward():
    lin = torch.nn.Linear(256, 32, bias=True)
    mod = R.ConvRotLinearRef(lin, bits=8)
    assert mod.is_quant_linear and mod.weight.dtype == torch.int8 and not any(p.requires_grad for p in mod.parameters())
    x = torch.randn(3, 5, 256, requires_grad=True)
    y = mod(x)
    assert y.shape == (3, 5, 32)
    y.sum().backward()
    w_eff = R.effective_weight(mod.weight_q, mod.scale, 8)
    assert torch.allclose(x.grad[0, 0], w_eff.sum(0), atol=1e-5)


def test_requant_int4_to_int8_definition():
    """The per-channel re-expression of an int4 base: codes within half an int8 step of the group-scaled
    weight, the largest group of a row maps 7 -> 127, all-zero rows give zeros (no NaN)."""
    w = R.synth_weight(48, 512, seed=31)
    w[5] = 0
    q4, s4 = R.quantize_weight_int4(w)
    w8, s8 = R.requant_int4_to_int8(q4, s4)
    assert w8.dtype == torch.int8 and w8.shape == (48, 512) and s8.shape == (48,)
    assert int(w8.abs().max()) <= 127 and torch.isfinite(s8).all()
    assert int(w8[5].abs().max()) == 0                           # the quantiser's floor keeps the scale > 0
    z8, zs = R.requant_int4_to_int8(q4[:2], torch.zeros(2, 4, dtype=torch.bfloat16))
    assert int(z8.abs().max()) == 0 and float(zs.abs().max()) == 0.0        # zero scales: zeros, no NaN
    dense4 = R.unpack_int4(q4).float().reshape(48, 4, 128) * s4.float()[:, :, None]
    dense8 = w8.float().reshape(48, 4, 128) * s8[:, None, None]
    assert float((dense8 - dense4).abs().max()) <= 0.5 * float(s8.max()) * (1 + 1e-6)
    g = int(s4[0].float().argmax())
    assert int(R.unpack_int4(q4)[0].reshape(4, 128)[g].abs().max()) in (7, 8)
    assert int(w8[0].reshape(4, 128)[g].abs().max()) >= 127 - 19     # |code| 7 -> 127, -8 clamps at -127
