"""The elementwise steps of a DiT block between the quantised Linears as single kernels with
hand-written backwards (training; inference folds the same steps into the quantisation passes, see
``ops.norm_mod_quant`` / ``swiglu_quant`` / ``gate_quant`` / ``qknorm_rope_``).

Each function mirrors one expression of the reference's model code and falls back to that expression,
op by op, whenever its kernel does not apply (CPU tensors, other dtypes, head dimension != 128, a
modulation vector that itself needs a gradient):

    norm_modulate(x, norm, scale, shift)        (1 + scale) * norm(x) + shift         mmdit.py:313-317
    qk_norm_rope(q, k, qknorm, rope, ...)       QKNorm + ropeapply                     mmdit.py:135-141, 25-31
    swiglu(g, u)                                silu(g) * u                            mmdit.py:178
    sigmoid_gate(a, g)                          a * sigmoid(g)                         mmdit.py:210
    gate_residual(x, gate, y)                   x + gate * y                           mmdit.py:318-321
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.nn.functional as F

from . import _lib
from .ops import _ptr, _stream


def _rows(t: torch.Tensor) -> torch.Tensor:
    """[..., K] -> [rows, K] with unit inner stride and a 16-byte friendly row stride (copy if not)."""
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(1) != 1 or t2.stride(0) % 8 or t2.data_ptr() % 16 or (t2.shape[0] > 1 and t2.stride(0) < t2.shape[1]):
        t2 = t2.contiguous()
    return t2


def _kernel_ok(*tensors) -> bool:
    return all(t is None or (t.is_cuda and t.dtype == torch.bfloat16) for t in tensors)


def _call(name: str, dev, *args) -> None:
    with torch.cuda.device(dev):
        rc = getattr(_lib.load(), name)(*args, _stream(dev))
    _lib.check(rc, name)


# ---------------------------------------------------------------------------------------------
# RMSNorm + modulation
# ---------------------------------------------------------------------------------------------
class _NormMod(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, norm_scale, mod_scale, mod_shift, eps):
        x2 = _rows(x)
        m, k = x2.shape
        rows_per_batch = x.shape[-2] if x.dim() >= 3 else m
        nb = m // rows_per_batch
        sc = None if mod_scale is None else mod_scale.reshape(nb, k).contiguous()
        sh = None if mod_shift is None else mod_shift.reshape(nb, k).contiguous()
        y = torch.empty(m, k, dtype=torch.bfloat16, device=x.device)
        rstd = torch.empty(m, dtype=torch.float32, device=x.device)
        _call("k2q_norm_mod_fwd", x.device, _ptr(x2), x2.stride(0), m, k, _ptr(norm_scale), _ptr(sc), _ptr(sh),
              rows_per_batch, float(eps), _ptr(y), k, _ptr(rstd))
        ctx.save_for_backward(x2, rstd, norm_scale, sc)
        ctx.rows_per_batch = rows_per_batch
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        x2, rstd, norm_scale, sc = ctx.saved_tensors
        m, k = x2.shape
        g2 = _rows(gy if gy.dtype == torch.bfloat16 else gy.to(torch.bfloat16))
        dx = torch.empty(m, k, dtype=torch.bfloat16, device=x2.device)
        _call("k2q_norm_mod_bwd", x2.device, _ptr(g2), g2.stride(0), _ptr(x2), x2.stride(0), _ptr(rstd), m, k,
              _ptr(norm_scale), _ptr(sc), ctx.rows_per_batch, _ptr(dx), k)
        return dx.view(ctx.shape), None, None, None, None


def norm_modulate(x: torch.Tensor, norm, mod_scale: torch.Tensor | None = None, mod_shift: torch.Tensor | None = None):
    """``(1 + mod_scale) * norm(x) + mod_shift`` for an RMSNorm-like ``norm`` (attributes ``scale`` fp32 [K],
    ``eps``; weight 1 + scale), x [B, L, K], mod_* [B, 1, K] (or None: the norm alone)."""
    k = x.shape[-1]
    fused = (_kernel_ok(x, mod_scale, mod_shift) and k % 8 == 0 and k <= 8192 and not norm.scale.requires_grad
             and not (mod_scale is not None and mod_scale.requires_grad)
             and not (mod_shift is not None and mod_shift.requires_grad))
    if not fused:
        y = norm(x)
        if mod_scale is not None:
            y = (1 + mod_scale) * y
        if mod_shift is not None:
            y = y + mod_shift
        return y
    scale = norm.scale if norm.scale.dtype == torch.float32 else norm.scale.float()
    return _NormMod.apply(x, scale.detach(), None if mod_scale is None else mod_scale.detach(),
                          None if mod_shift is None else mod_shift.detach(), norm.eps)


# ---------------------------------------------------------------------------------------------
# QK norm + rotary embedding
# ---------------------------------------------------------------------------------------------
class _QkNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, wq, wk, cos, sin, eps, b, s, heads, kvheads):
        q2, k2 = _rows(q), _rows(k)
        t = q2.shape[0]
        qo = torch.empty(t, heads * 128, dtype=torch.bfloat16, device=q.device)
        ko = torch.empty(t, kvheads * 128, dtype=torch.bfloat16, device=q.device)
        _call("k2q_qknorm_rope_fwd", q.device, _ptr(q2), q2.stride(0), heads, _ptr(wq), _ptr(qo), heads * 128,
              _ptr(k2), k2.stride(0), kvheads, _ptr(wk), _ptr(ko), kvheads * 128, t, _ptr(cos), _ptr(sin), float(eps))
        ctx.save_for_backward(q2, k2, wq, wk, cos, sin)
        ctx.dims = (eps, b, s, heads, kvheads, q.shape, k.shape)
        return qo.view(b, s, heads, 128).transpose(1, 2), ko.view(b, s, kvheads, 128).transpose(1, 2)

    @staticmethod
    def backward(ctx, gq, gk):
        q2, k2, wq, wk, cos, sin = ctx.saved_tensors
        eps, b, s, heads, kvheads, qshape, kshape = ctx.dims

        def grad4(g):      # [B, H, S, 128] bf16 with unit inner stride and 8-byte friendly strides
            if g.dtype != torch.bfloat16:
                g = g.to(torch.bfloat16)
            if g.stride(3) != 1 or any(st % 4 for st in g.stride()[:3]) or g.data_ptr() % 8:
                g = g.contiguous()
            return g

        gq, gk = grad4(gq), grad4(gk)
        dq = torch.empty(b * s, heads * 128, dtype=torch.bfloat16, device=q2.device)
        dk = torch.empty(b * s, kvheads * 128, dtype=torch.bfloat16, device=q2.device)
        _call("k2q_qknorm_rope_bwd", q2.device,
              _ptr(q2), q2.stride(0), heads, _ptr(wq), _ptr(gq), gq.stride(0), gq.stride(2), gq.stride(1), _ptr(dq), heads * 128,
              _ptr(k2), k2.stride(0), kvheads, _ptr(wk), _ptr(gk), gk.stride(0), gk.stride(2), gk.stride(1), _ptr(dk), kvheads * 128,
              b, s, _ptr(cos), _ptr(sin), float(eps))
        return dq.view(qshape), dk.view(kshape), None, None, None, None, None, None, None, None, None


def qk_norm_rope_train(q, k, qknorm, rope, b: int, s: int, heads: int, kvheads: int):
    """Differentiable QK-norm + rotation for head dimension 128: q [B, S, heads*128] / k [B, S, kvheads*128]
    -> ([B, heads, S, 128], [B, kvheads, S, 128]) views of freshly written [B, S, H, 128] tensors."""
    cos = sin = None
    if rope is not None:
        cos, sin = (t.reshape(b * s, 64) for t in rope)
        if cos.dtype != torch.float32 or not cos.is_contiguous() or not sin.is_contiguous():
            cos, sin = cos.float().contiguous(), sin.float().contiguous()
    wq, wk = qknorm.qnorm.scale, qknorm.knorm.scale
    wq = wq if wq.dtype == torch.float32 else wq.float()
    wk = wk if wk.dtype == torch.float32 else wk.float()
    return _QkNormRope.apply(q, k, wq.detach(), wk.detach(), cos, sin, qknorm.qnorm.eps, b, s, heads, kvheads)


def qk_norm_rope_trainable(q, k, qknorm, headdim: int) -> bool:
    return (headdim == 128 and _kernel_ok(q, k) and not qknorm.qnorm.scale.requires_grad
            and not qknorm.knorm.scale.requires_grad)


# ---------------------------------------------------------------------------------------------
# SwiGLU, sigmoid gate, gated residual
# ---------------------------------------------------------------------------------------------
class _Pair(torch.autograd.Function):
    """kind 'swiglu': silu(a) * b;  kind 'sigmoid_gate': a * sigmoid(b)."""

    @staticmethod
    def forward(ctx, a, b, kind):
        a2, b2 = _rows(a), _rows(b)
        m, k = a2.shape
        out = torch.empty(m, k, dtype=torch.bfloat16, device=a.device)
        if kind == "swiglu":
            _call("k2q_swiglu_fwd", a.device, _ptr(a2), a2.stride(0), _ptr(b2), b2.stride(0), m, k, _ptr(out), k)
        else:
            _call("k2q_sigmoid_gate_fwd", a.device, _ptr(a2), a2.stride(0), _ptr(b2), b2.stride(0), m, k, _ptr(out), k)
        ctx.save_for_backward(a2, b2)
        ctx.kind, ctx.ashape, ctx.bshape = kind, a.shape, b.shape
        return out.view(a.shape)

    @staticmethod
    def backward(ctx, gy):
        a2, b2 = ctx.saved_tensors
        m, k = a2.shape
        g2 = _rows(gy if gy.dtype == torch.bfloat16 else gy.to(torch.bfloat16))
        da = torch.empty(m, k, dtype=torch.bfloat16, device=a2.device)
        db = torch.empty(m, k, dtype=torch.bfloat16, device=a2.device)
        if ctx.kind == "swiglu":      # a = g, b = u
            _call("k2q_swiglu_bwd", a2.device, _ptr(g2), g2.stride(0), _ptr(a2), a2.stride(0), _ptr(b2), b2.stride(0), m, k,
                  _ptr(da), k, _ptr(db), k)
        else:                         # a = attention output, b = gate
            _call("k2q_sigmoid_gate_bwd", a2.device, _ptr(g2), g2.stride(0), _ptr(a2), a2.stride(0), _ptr(b2), b2.stride(0),
                  m, k, _ptr(da), k, _ptr(db), k)
        return da.view(ctx.ashape), db.view(ctx.bshape), None


def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    if _kernel_ok(g, u) and g.shape == u.shape and g.shape[-1] % 8 == 0:
        return _Pair.apply(g, u, "swiglu")
    return F.silu(g) * u


def sigmoid_gate(a: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    if _kernel_ok(a, g) and a.shape == g.shape and a.shape[-1] % 8 == 0:
        return _Pair.apply(a, g, "sigmoid_gate")
    return a * torch.sigmoid(g)


class _GateResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, y):
        x2, y2 = _rows(x), _rows(y)
        m, k = y2.shape
        rows_per_batch = y.shape[-2] if y.dim() >= 3 else m
        gt = gate.reshape(m // rows_per_batch, k).contiguous()
        out = torch.empty(m, k, dtype=torch.bfloat16, device=y.device)
        _call("k2q_gate_residual", y.device, _ptr(x2), x2.stride(0), _ptr(y2), y2.stride(0), _ptr(gt), rows_per_batch, m, k,
              _ptr(out), k)
        ctx.save_for_backward(gt)
        ctx.rows_per_batch = rows_per_batch
        return out.view(y.shape)

    @staticmethod
    def backward(ctx, gout):
        (gt,) = ctx.saved_tensors
        g2 = _rows(gout if gout.dtype == torch.bfloat16 else gout.to(torch.bfloat16))
        m, k = g2.shape
        dy = torch.empty(m, k, dtype=torch.bfloat16, device=g2.device)
        _call("k2q_gate_residual", g2.device, C.c_void_p(0), 0, _ptr(g2), g2.stride(0), _ptr(gt), ctx.rows_per_batch, m, k,
              _ptr(dy), k)
        return gout, None, dy.view(gout.shape)


def gate_residual(x: torch.Tensor, gate: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """``x + gate * y`` with gate [B, 1, K] broadcast over the tokens of a batch element."""
    if (_kernel_ok(x, gate, y) and x.shape == y.shape and y.dim() == 3 and y.shape[-1] % 8 == 0
            and gate.numel() == y.shape[0] * y.shape[-1] and not gate.requires_grad):
        return _GateResidual.apply(x, gate.detach(), y)
    return x + gate * y


__all__ = ["norm_modulate", "qk_norm_rope_train", "qk_norm_rope_trainable", "swiglu", "sigmoid_gate", "gate_residual"]
