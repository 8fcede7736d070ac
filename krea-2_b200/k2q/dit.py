"""Caller side of the path: a single-stream DiT with the Krea 2 layout, and the two step functions
the benchmark configurations time.

The reference model code (mmdit.py, train_t2i.py, sampling.py) stays what users run; it is not
importable where this package is benchmarked, so this module rebuilds the same network from its
description -- same module and parameter names (a reference ``state_dict`` loads here and vice
versa), same forward arithmetic -- purely as the harness around the quantized Linears:

* ``SingleStreamDiT``      mmdit.py:322-501 (``first``, ``tmlp``, ``tproj``, ``txtfusion``, ``txtmlp``,
                           ``blocks`` of RMSNorm -> modulate -> attention(wq wk wv gate wo) -> SwiGLU, ``last``)
* ``flow_training_step``   train_t2i.py:67-127 with the default FlowConfig (uniform weighting)
* ``denoise_step``         the inner call of sampling.py:129-137 without CFG

Attention itself stays a library call (``F.scaled_dot_product_attention``), as in the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint

from . import fused, ops
from .modules import convrot_linear_quantized, fused_prologue_ok


@dataclass
class DiTConfig:
    """Field names of ``SingleMMDiTConfig`` (mmdit.py:73-88)."""
    features: int
    tdim: int
    txtdim: int
    heads: int
    multiplier: int
    layers: int
    patch: int
    channels: int
    bias: bool = False
    theta: float = 1e3
    kvheads: int | None = None
    txtlayers: int = 1
    txtheads: int = 20
    txtkvheads: int = 20


def krea2_large_wide() -> DiTConfig:
    """``single_mmdit_large_wide`` (inference.py:12-25): the only architecture the reference ships."""
    return DiTConfig(features=6144, tdim=256, txtdim=2560, heads=48, kvheads=12, multiplier=4, layers=28, patch=2,
                     channels=16, txtheads=20, txtkvheads=20, txtlayers=12)


# ---------------------------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------------------------
class RMSNorm(nn.Module):
    """fp32 RMS norm with weight (1 + scale), scale initialised to zero (mmdit.py:143-160)."""

    def __init__(self, features: int, eps: float = 1e-5):
        super().__init__()
        self.features, self.eps = features, eps
        self.scale = nn.Parameter(torch.zeros(features, dtype=torch.float32))

    def forward(self, x):
        y = F.rms_norm(x.float(), (self.features,), weight=self.scale.float() + 1.0, eps=self.eps)
        return y.to(x.dtype)


class QKNorm(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.qnorm, self.knorm = RMSNorm(dim), RMSNorm(dim)

    def forward(self, q, k):
        return self.qnorm(q), self.knorm(k)


def rope_tables(pos: torch.Tensor, axes: list[int], theta: float):
    """cos/sin tables [B, S, head_dim/2]: axis i of ``pos`` drives ``axes[i]/2`` frequencies
    theta^(-2j/axes[i]) (mmdit.py:13-22, 119-133), computed in float64 like the reference."""
    parts = []
    for i, d in enumerate(axes):
        freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=pos.device) / d))
        parts.append(pos[..., i, None].to(torch.float64) * freq)
    ang = torch.cat(parts, dim=-1)
    return torch.cos(ang).float(), torch.sin(ang).float()


def rope_rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotates consecutive pairs of the head dimension (mmdit.py:25-31).  x: [B, H, S, D]."""
    xf = x.float().unflatten(-1, (-1, 2))
    x0, x1 = xf[..., 0], xf[..., 1]
    c, s = cos[:, None], sin[:, None]
    out = torch.stack((c * x0 - s * x1, s * x0 + c * x1), dim=-1)
    return out.flatten(-2).to(x.dtype)


def qk_inplace_ok(q2: torch.Tensor, k2: torch.Tensor, headdim: int) -> bool:
    """Inference on bf16 CUDA projections with head dimension 128: the in-place kernel applies."""
    return (headdim == 128 and not torch.is_grad_enabled() and q2.is_cuda and q2.dtype == torch.bfloat16
            and q2.stride(1) == 1 and k2.stride(1) == 1)


def qk_norm_rope(q, k, qknorm: "QKNorm", rope, b: int, s: int, heads: int, kvheads: int, headdim: int):
    """QK-norm and rotary embedding of the projections' outputs q [B*S, heads*D] / k [B*S, kvheads*D]
    (or [B, S, ...]); returns them as [B, heads, S, D] / [B, kvheads, S, D] for the attention call
    (mmdit.py:199-208).  In inference with head dimension 128 both steps are ONE in-place kernel over
    the GEMM outputs (``ops.qknorm_rope_``); otherwise the composed torch ops."""
    q2, k2 = q.reshape(b * s, heads * headdim), k.reshape(b * s, kvheads * headdim)
    if qk_inplace_ok(q2, k2, headdim):
        cos = sin = None
        if rope is not None:
            cos, sin = (t.reshape(b * s, headdim // 2) for t in rope)
            if cos.dtype != torch.float32 or not cos.is_contiguous() or not sin.is_contiguous():
                cos, sin = cos.float().contiguous(), sin.float().contiguous()
        ops.qknorm_rope_(q2, k2, qknorm.qnorm.scale.float(), qknorm.knorm.scale.float(), cos, sin, qknorm.qnorm.eps)
        return (q2.view(b, s, heads, headdim).transpose(1, 2), k2.view(b, s, kvheads, headdim).transpose(1, 2))
    if fused.qk_norm_rope_trainable(q2, k2, qknorm, headdim):      # training: one kernel each way
        return fused.qk_norm_rope_train(q2, k2, qknorm, rope, b, s, heads, kvheads)
    qh = q2.view(b, s, heads, headdim).transpose(1, 2)
    kh = k2.view(b, s, kvheads, headdim).transpose(1, 2)
    qh, kh = qknorm(qh, kh)
    if rope is not None:
        qh, kh = rope_rotate(qh, *rope), rope_rotate(kh, *rope)
    return qh, kh


def timestep_embedding(t: torch.Tensor, dim: int, dtype, period: float = 1e4, tfactor: float = 1e3):
    """[B] -> [B, 1, dim] (cos | sin) embedding (mmdit.py:52-70)."""
    half = dim // 2
    freqs = torch.exp(-math.log(period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = (t.float() * tfactor)[:, None, None] * freqs
    return torch.cat((torch.cos(args), torch.sin(args)), dim=-1).to(dtype)


def pair_mask(mask: torch.Tensor) -> torch.Tensor:
    """(B, L) key-padding mask -> (B, 1, L, L) attention mask (mmdit.py:47-49)."""
    return mask[:, None, None, :] * mask[:, None, :, None]


class SwiGLU(nn.Module):
    def __init__(self, features: int, multiplier: int, bias: bool = False, multiple: int = 128):
        super().__init__()
        hidden = int(2 * features / 3) * multiplier
        hidden = multiple * ((hidden + multiple - 1) // multiple)
        self.gate = nn.Linear(features, hidden, bias=bias)
        self.up = nn.Linear(features, hidden, bias=bias)
        self.down = nn.Linear(hidden, features, bias=bias)

    def forward(self, x):
        return self.down(fused.swiglu(self.gate(x), self.up(x)))

    def forward_codes(self, xq, sx, lead):
        """The same from rotated int8 codes of the input ([T, F] + per-token scales): gate / up GEMMs,
        silu(g) * u folded into the quantisation of ``down``'s input.  Inference, ConvRot Linears."""
        grp = getattr(self, "gu_group", None)
        if grp is not None:
            g, u = grp.forward_codes(xq, sx)          # one launch, two column slices
        else:
            g = convrot_linear_quantized(xq, sx, self.gate)
            u = convrot_linear_quantized(xq, sx, self.up)
        hq, hs = ops.swiglu_quant(g, u)
        return convrot_linear_quantized(hq, hs, self.down).view(*lead, -1)


class Attention(nn.Module):
    """q/k/v/gate projections of one input, QK-RMSNorm, RoPE, SDPA (GQA), sigmoid output gate, wo
    (mmdit.py:181-212)."""

    def __init__(self, dim: int, heads: int, kvheads: int | None = None, bias: bool = False):
        super().__init__()
        self.heads = heads
        self.kvheads = kvheads if kvheads is not None else heads
        self.headdim = dim // heads
        self.wq = nn.Linear(dim, self.headdim * self.heads, bias=bias)
        self.wk = nn.Linear(dim, self.headdim * self.kvheads, bias=bias)
        self.wv = nn.Linear(dim, self.headdim * self.kvheads, bias=bias)
        self.gate = nn.Linear(dim, dim, bias=bias)
        self.qknorm = QKNorm(self.headdim)
        self.wo = nn.Linear(dim, dim, bias=bias)

    def forward(self, x, rope=None, mask=None):
        b, s, _ = x.shape
        q, k, v, g = self.wq(x), self.wk(x), self.wv(x), self.gate(x)
        v = v.view(b, s, self.kvheads, self.headdim).transpose(1, 2)
        q, k = qk_norm_rope(q, k, self.qknorm, rope, b, s, self.heads, self.kvheads, self.headdim)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=self.heads != self.kvheads)
        o = o.transpose(1, 2).reshape(b, s, self.heads * self.headdim)
        return self.wo(fused.sigmoid_gate(o, g))

    def forward_codes(self, xq, sx, lead, rope=None, mask=None):
        """The same from rotated int8 codes of the input: four GEMMs on one set of codes, and
        attention * sigmoid(gate) folded into the quantisation of ``wo``'s input."""
        b, s = lead
        grp = getattr(self, "qkvg_group", None)
        if grp is not None:
            q, k, v, g = grp.forward_codes(xq, sx)    # one launch over 2 F + 2 kv columns
        else:
            q, k, v, g = (convrot_linear_quantized(xq, sx, m) for m in (self.wq, self.wk, self.wv, self.gate))
        v = v.view(b, s, self.kvheads, self.headdim).transpose(1, 2)
        q, k = qk_norm_rope(q, k, self.qknorm, rope, b, s, self.heads, self.kvheads, self.headdim)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=self.heads != self.kvheads)
        o = o.transpose(1, 2).reshape(b * s, self.heads * self.headdim)
        oq, so = ops.gate_quant(o, g)
        return convrot_linear_quantized(oq, so, self.wo).view(b, s, -1)


class DoubleSharedModulation(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.lin = nn.Parameter(torch.zeros(6 * dim))

    def forward(self, vec):
        return (vec + self.lin).chunk(6, dim=-1)


class SimpleModulation(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.lin = nn.Parameter(torch.zeros(2, dim))

    def forward(self, vec):
        return (vec + self.lin[None]).chunk(2, dim=1)


class SingleStreamBlock(nn.Module):
    def __init__(self, features, heads, multiplier, bias=False, kvheads=None):
        super().__init__()
        self.mod = DoubleSharedModulation(features)
        self.prenorm, self.postnorm = RMSNorm(features), RMSNorm(features)
        self.attn = Attention(features, heads, kvheads, bias)
        self.mlp = SwiGLU(features, multiplier, bias)

    def forward(self, x, vec, rope, mask=None):
        prescale, preshift, pregate, postscale, postshift, postgate = self.mod(vec)
        a, m = self.attn, self.mlp
        if (type(a) is Attention and type(m) is SwiGLU and
                fused_prologue_ok(x, a.wq, a.wk, a.wv, a.gate, a.wo, m.gate, m.up, m.down)):
            # inference on ConvRot bases: norm + modulation, SwiGLU and the sigmoid gate run inside the
            # quantisation passes (one read of the residual stream gives the codes of four Linears)
            lead = x.shape[:2]
            xq, sx = ops.norm_mod_quant(x, self.prenorm.scale.float(), prescale, preshift, self.prenorm.eps)
            x = fused.gate_residual(x, pregate, a.forward_codes(xq, sx, lead, rope, mask))
            xq, sx = ops.norm_mod_quant(x, self.postnorm.scale.float(), postscale, postshift, self.postnorm.eps)
            return fused.gate_residual(x, postgate, m.forward_codes(xq, sx, lead))
        x = fused.gate_residual(x, pregate, a(fused.norm_modulate(x, self.prenorm, prescale, preshift), rope, mask))
        return fused.gate_residual(x, postgate, m(fused.norm_modulate(x, self.postnorm, postscale, postshift)))


class TextFusionBlock(nn.Module):
    def __init__(self, features, heads, multiplier, bias=False, kvheads=None):
        super().__init__()
        self.prenorm, self.postnorm = RMSNorm(features), RMSNorm(features)
        self.attn = Attention(features, heads, kvheads, bias)
        self.mlp = SwiGLU(features, multiplier, bias)

    def forward(self, x, mask=None):
        x = x + self.attn(fused.norm_modulate(x, self.prenorm), None, mask)
        return x + self.mlp(fused.norm_modulate(x, self.postnorm))


class TextFusionTransformer(nn.Module):
    """Two blocks across the tapped encoder layers of each token, a learned projection of the layer
    axis to one vector, two blocks across tokens (mmdit.py:252-292)."""

    def __init__(self, num_txt_layers, txt_dim, heads, multiplier, bias=False, kvheads=None):
        super().__init__()
        mk = lambda: TextFusionBlock(txt_dim, heads, multiplier, bias, kvheads)   # noqa: E731
        self.layerwise_blocks = nn.ModuleList([mk() for _ in range(2)])
        self.projector = nn.Linear(num_txt_layers, 1, bias=False)
        self.refiner_blocks = nn.ModuleList([mk() for _ in range(2)])

    def forward(self, x, mask=None):
        b, l, n, d = x.shape
        x = x.reshape(b * l, n, d)
        for blk in self.layerwise_blocks:
            x = blk(x.contiguous(), None)
        x = self.projector(x.view(b, l, n, d).transpose(2, 3)).squeeze(-1)
        for blk in self.refiner_blocks:
            x = blk(x, mask)
        return x


class LastLayer(nn.Module):
    def __init__(self, features, patch, channels):
        super().__init__()
        self.norm = RMSNorm(features)
        self.linear = nn.Linear(features, patch * patch * channels, bias=True)
        self.modulation = SimpleModulation(features)

    def forward(self, x, tvec):
        scale, shift = self.modulation(tvec)
        return self.linear((1 + scale) * self.norm(x) + shift)


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
class SingleStreamDiT(nn.Module):
    def __init__(self, config: DiTConfig):
        super().__init__()
        self.config = c = config
        hd = c.features // c.heads
        self.rope_axes = [hd - 12 * (hd // 16), 6 * (hd // 16), 6 * (hd // 16)]
        if sum(self.rope_axes) != hd or any(a % 2 for a in self.rope_axes):
            raise ValueError(f"head dim {hd} cannot be split over the three position axes")
        self.first = nn.Linear(c.channels * c.patch ** 2, c.features, bias=True)
        self.blocks = nn.ModuleList([SingleStreamBlock(c.features, c.heads, c.multiplier, c.bias, c.kvheads)
                                     for _ in range(c.layers)])
        self.tmlp = nn.Sequential(nn.Linear(c.tdim, c.features), nn.GELU(approximate="tanh"),
                                  nn.Linear(c.features, c.features))
        self.txtfusion = TextFusionTransformer(c.txtlayers, c.txtdim, c.txtheads, c.multiplier, c.bias, c.txtkvheads)
        self.txtmlp = nn.Sequential(RMSNorm(c.txtdim), nn.Linear(c.txtdim, c.features), nn.GELU(approximate="tanh"),
                                    nn.Linear(c.features, c.features))
        self.last = LastLayer(c.features, c.patch, c.channels)
        self.tproj = nn.Sequential(nn.GELU(approximate="tanh"), nn.Linear(c.features, c.features * 6))
        self.gradient_checkpointing = False
        self._swap_blocks: set[int] = set()
        self._swap_device = None
        self._swap_skip_trainable = True

    # -- block swap (mmdit.py:389-428): deepest blocks live on the CPU between uses ----------------
    def enable_block_swap(self, num_blocks: int, device, *, skip_trainable: bool = True) -> list[int]:
        n = max(0, min(int(num_blocks), len(self.blocks)))
        self._swap_device = torch.device(device)
        self._swap_skip_trainable = bool(skip_trainable)
        self._swap_blocks = set(range(len(self.blocks) - n, len(self.blocks)))
        for i in self._swap_blocks:
            self._page(self.blocks[i], torch.device("cpu"))
            self.blocks[i].register_forward_pre_hook(lambda mod, args: self._page(mod, self._swap_device))
        return sorted(self._swap_blocks)

    def _page(self, block: nn.Module, device: torch.device) -> None:
        for p in block.parameters():
            if self._swap_skip_trainable and p.requires_grad:
                continue
            p.data = p.data.to(device, non_blocking=True)

    def _page_out_after_backward(self, block, inp):
        def hook(grad):
            self._page(block, torch.device("cpu"))
        inp.register_hook(hook)

    def forward(self, img, context, t, pos, mask=None):
        c = self.config
        img = self.first(img)
        temb = self.tmlp(timestep_embedding(t, c.tdim, img.dtype))
        tvec = self.tproj(temb)
        context = self.txtfusion(context, pair_mask(mask[:, :context.shape[1]]))
        context = self.txtmlp(context)
        txtlen, imglen = context.shape[1], img.shape[1]
        x = torch.cat((context, img), dim=1)
        pad = (-x.shape[1]) % 256                       # mmdit.py:458-464
        if pad:
            x = F.pad(x, (0, 0, 0, pad))
            mask = F.pad(mask, (0, pad), value=False)
            pos = F.pad(pos, (0, 0, 0, pad))
        amask = pair_mask(mask)
        rope = rope_tables(pos, self.rope_axes, c.theta)
        for i, blk in enumerate(self.blocks):
            swapped = i in self._swap_blocks
            inp = x
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(blk, inp, tvec, rope, amask, use_reentrant=False)
                if swapped:
                    self._page(blk, torch.device("cpu"))
                    if inp.requires_grad:
                        self._page_out_after_backward(blk, inp)
            else:
                x = blk(inp, tvec, rope, amask)
                if swapped:
                    if not self.training:
                        self._page(blk, torch.device("cpu"))
                    elif inp.requires_grad:
                        self._page_out_after_backward(blk, inp)
        out = self.last(x, temb)
        return out[:, txtlen:txtlen + imglen]


# ---------------------------------------------------------------------------------------------
# step functions
# ---------------------------------------------------------------------------------------------
def shift_schedule(image_tokens: int, base_shift=0.5, max_shift=1.15, base_len=256, max_len=6400, sigma=1.0):
    """Resolution-aware timestep shift t -> e^mu / (e^mu + (1/t - 1)^sigma), mu linear in the image
    token count (scheduler.py:28-58, constants.py:33-39)."""
    mu = base_shift + (max_shift - base_shift) * (image_tokens - base_len) / (max_len - base_len)
    em = math.exp(mu)

    def schedule(u: torch.Tensor) -> torch.Tensor:
        u = u.to(torch.float64).clamp(1e-6, 1.0 - 1e-6)
        return (em / (em + (1.0 / u - 1.0) ** sigma)).to(torch.float32)

    return schedule


def position_ids(grid_h: int, grid_w: int, text_mask: torch.Tensor):
    """pos (B, S, 3) and mask (B, S) for [text][image]: text at the origin, image tokens carry their
    grid row/column on axes 1/2 (train_t2i.py:29-58 for plain text-to-image)."""
    b, l = text_mask.shape
    dev = text_mask.device
    ids = torch.zeros(grid_h, grid_w, 3, device=dev)
    ids[..., 1] = torch.arange(grid_h, device=dev)[:, None]
    ids[..., 2] = torch.arange(grid_w, device=dev)[None, :]
    pos = torch.cat((torch.zeros(l, 3, device=dev), ids.reshape(-1, 3)), dim=0)[None].expand(b, -1, -1)
    mask = torch.cat((text_mask, torch.ones(b, grid_h * grid_w, dtype=torch.bool, device=dev)), dim=1)
    return pos, mask


def flow_training_step(dit, *, z0, context, text_mask, grid_h, grid_w, t=None, noise=None, generator=None):
    """Flow-matching loss of one batch (train_t2i.py:67-127, uniform timestep weighting):
    x_t = t*noise + (1-t)*z0, target v = noise - z0, loss = mean over samples of the per-sample MSE.
    ``t`` / ``noise`` may be passed in (data-parallel runs draw them once for the global batch)."""
    b = z0.shape[0]
    dev = z0.device
    if t is None:
        t = shift_schedule(grid_h * grid_w)(torch.rand(b, device=dev, generator=generator)).float()
    if noise is None:
        noise = torch.randn(z0.shape, device=dev, generator=generator, dtype=torch.float32)
    z0f = z0.float()
    tt = t.view(b, 1, 1)
    x_t = tt * noise + (1.0 - tt) * z0f
    target = noise - z0f
    pos, mask = position_ids(grid_h, grid_w, text_mask)
    dtype = next(dit.parameters()).dtype if not hasattr(dit, "compute_dtype") else dit.compute_dtype
    pred = dit(img=x_t.to(dtype), context=context.to(dtype), t=t, pos=pos, mask=mask)
    per_sample = ((pred.float() - target) ** 2).mean(dim=(1, 2))
    return per_sample.mean()


@torch.no_grad()
def denoise_step(dit, img, context, t_curr: float, t_prev: float, pos, mask):
    """One Euler step of the flow ODE without guidance (sampling.py:129-137 for guidance 0)."""
    t = torch.full((img.shape[0],), t_curr, dtype=img.dtype, device=img.device)
    v = dit(img=img, context=context, t=t, pos=pos, mask=mask)
    return img + (t_prev - t_curr) * v
