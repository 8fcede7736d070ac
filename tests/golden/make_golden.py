"""Generates the golden fixtures under tests/golden/.

Run from the repository root in a container that has the reference checked out:

    python tests/golden/make_golden.py [/path/to/reference]

Two kinds of fixture are written (small .pt files, seeded inputs + expected outputs):

* ``ref_*.pt``      outputs of the REFERENCE's own modules imported from its source tree
                    (quantize.Fp8Linear, lora.LoRALinear, fwd and autograd bwd, on CPU).  They pin
                    the oracle's restatements ``fp8_linear_ref`` / ``lora_forward_ref`` and the
                    conventions the ConvRot functions inherit.
* ``convrot_*.pt``  outputs of the CPU oracle itself for the ConvRot arithmetic, which has no
                    counterpart in the reference (regression pins for oracle and kernels).
"""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
OUT = Path(__file__).resolve().parent


def reference_fixtures(ref_dir: str):
    sys.path.insert(0, ref_dir)
    import lora as ref_lora          # noqa: E402  (reference module)
    import quantize as ref_quant     # noqa: E402  (reference module)

    g = torch.Generator().manual_seed(0)
    cases = []
    for (m, k, n, rank, alpha, mul, with_bias) in [(24, 64, 48, 4, 4.0, 1.0, True), (17, 128, 32, 8, 16.0, -1.5, False),
                                                   (8, 96, 16, 2, 2.0, 0.0, True)]:
        lin = torch.nn.Linear(k, n, bias=with_bias).to(torch.bfloat16)
        lin.weight.data = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
        if with_bias:
            lin.bias.data = (torch.randn(n, generator=g) * 0.01).to(torch.bfloat16)
        x = torch.randn(m, k, generator=g).to(torch.bfloat16)
        gy = (torch.randn(m, n, generator=g) * 1e-2).to(torch.bfloat16)
        fp8 = ref_quant.Fp8Linear(lin)
        y_fp8 = fp8(x)
        ad = ref_lora.LoRALinear(fp8, rank, alpha)
        ad.lora_A.data = torch.randn(rank, k, generator=g) * 0.01
        ad.lora_B.data = torch.randn(n, rank, generator=g) * 0.01
        ad.scale_mul = mul
        xr = x.clone().requires_grad_(True)
        y = ad(xr)
        y.backward(gy)
        cases.append(dict(
            w=lin.weight.data.clone(), bias=lin.bias.data.clone() if with_bias else None, x=x, gy=gy,
            rank=rank, alpha=alpha, scale_mul=mul, lora_A=ad.lora_A.data.clone(), lora_B=ad.lora_B.data.clone(),
            fp8_weight=fp8.weight_fp8.data.view(torch.uint8).clone(), fp8_scale=fp8.scale.data.clone(),
            y_fp8=y_fp8.detach().clone(), y=y.detach().clone(), dx=xr.grad.clone(),
            dA=None if ad.lora_A.grad is None else ad.lora_A.grad.clone(),
            dB=None if ad.lora_B.grad is None else ad.lora_B.grad.clone()))
    torch.save(cases, OUT / "ref_fp8_lora.pt")
    print("wrote ref_fp8_lora.pt:", len(cases), "cases")


def convrot_fixtures():
    from oracle import convrot_ref as R
    cases = []
    for (m, k, n, seed) in [(9, 128, 16, 0), (20, 256, 48, 1), (33, 384, 32, 2)]:
        w = R.synth_weight(n, k, seed=1000 + seed)
        x = R.synth_act(m, k, seed=2000 + seed, outliers=2)
        bias = R.synth_vec(n, 0.01, 3000 + seed)
        q8, s8 = R.quantize_weight_int8(w)
        q4, s4 = R.quantize_weight_int4(w)
        xq, sx = R.quantize_act_int8(x)
        cases.append(dict(w=w, x=x, bias=bias, q8=q8, s8=s8, q4=q4, s4=s4, xq=xq, sx=sx,
                          y8=R.linear_int8_exact(xq, sx, q8, s8, bias),
                          y4=R.linear_int4_exact(xq, sx, q4, s4, bias)))
    torch.save(cases, OUT / "convrot_small.pt")
    print("wrote convrot_small.pt:", len(cases), "cases")


TINY_DIT = dict(features=128, tdim=32, txtdim=64, heads=2, kvheads=1, multiplier=1, layers=2, patch=2, channels=4,
                txtheads=2, txtkvheads=2, txtlayers=3)


def seeded_fill(model, scale=0.05):
    """Deterministic weights that do not depend on construction order: one generator per name."""
    import zlib
    for name, p in model.named_parameters():
        g = torch.Generator().manual_seed(zlib.crc32(name.encode()))
        p.data = (torch.randn(p.shape, generator=g) * scale).to(p.dtype)


def dit_fixture(ref_dir: str):
    """Forward + flow-matching loss/grad of the REFERENCE SingleStreamDiT (mmdit.py, train_t2i.py) on a
    tiny configuration, on CPU; pins the harness model in k2q/dit.py."""
    import torch.nn.functional as F
    from einops import rearrange
    sys.path.insert(0, ref_dir)
    import mmdit as ref_mmdit          # noqa: E402
    import scheduler as ref_sched      # noqa: E402
    import train_t2i as ref_train      # noqa: E402
    from training_config import FlowConfig  # noqa: E402

    def cpu_attention(q, k, v, mask=None, scale=None, gqa=False):   # the reference pins a CUDA-only backend
        return rearrange(F.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=scale, enable_gqa=gqa),
                         "B H L D -> B L (H D)")
    ref_mmdit.attention = cpu_attention
    model = ref_mmdit.SingleStreamDiT(ref_mmdit.SingleMMDiTConfig(**TINY_DIT))
    seeded_fill(model)
    g = torch.Generator().manual_seed(11)
    b, gh, gw, l = 2, 4, 6, 9
    z0 = torch.randn(b, gh * gw, 16, generator=g)
    ctx = torch.randn(b, l, 3, 64, generator=g)
    tm = torch.ones(b, l, dtype=torch.bool)
    tm[1, 6:] = False
    t = torch.tensor([0.25, 0.9])
    pos, mask = ref_train.build_pos_mask(gh, gw, tm)
    y = model(z0, ctx, t, pos, mask)
    loss = ref_train.t2i_training_step(model, z0=z0, context=ctx, text_mask=tm, grid_h=gh, grid_w=gw,
                                       schedule=ref_sched.get_schedule_for_seqlen(gh * gw), flow_cfg=FlowConfig(),
                                       generator=torch.Generator().manual_seed(5))
    loss.backward()
    torch.save(dict(config=TINY_DIT, z0=z0, ctx=ctx, text_mask=tm, t=t, grid=(gh, gw), y=y.detach(),
                    loss=loss.detach(), grad_wq=model.blocks[1].attn.wq.weight.grad.clone(),
                    grad_first_bias=model.first.bias.grad.clone(), n_params=sum(p.numel() for p in model.parameters()),
                    keys=sorted(model.state_dict().keys())),
               OUT / "ref_dit_tiny.pt")
    print("wrote ref_dit_tiny.pt")


if __name__ == "__main__":
    torch.manual_seed(0)
    torch.set_num_threads(1)
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference project> | --convrot-only")
    if sys.argv[1] == "--convrot-only":      # the oracle's own regression pins need no reference checkout
        convrot_fixtures()
        raise SystemExit(0)
    ref = sys.argv[1]
    reference_fixtures(ref)
    convrot_fixtures()
    dit_fixture(ref)
