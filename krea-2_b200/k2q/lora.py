"""LoRA side of the drop-in boundary.

The reference's ``lora.py`` keeps working unchanged on :class:`k2q.modules.ConvRotLinear` bases
(it only asks for ``is_quant_linear`` / ``in_features`` / ``out_features`` / ``weight``,
lora.py:38-40,99-101).  This module adds

* :func:`fuse_lora`: a post-pass that retargets every adapter whose base is a ConvRot linear to a
  fused forward/backward (adapter term inside the GEMM epilogue, hand-written gradients).  The
  adapter object keeps its class identity (the new class derives from the old one), its attributes
  (``base, rank, scale, scale_mul, lora_A, lora_B``) and its parameters, so ``lora_scaled``
  (lora.py:51-65), ``save_lora`` / ``load_lora_weights`` (lora.py:154-193) and optimizer state
  are unaffected.
* a self-contained mirror of the reference's adapter API (``LoRALinear``, ``inject_lora``,
  ``lora_scaled``, ``lora_disabled``, ``lora_parameters``) for environments where the reference
  package is not importable (benchmarks, GPU tests).  Same names, arguments and behaviour.
"""
from __future__ import annotations

import contextlib
import math

import torch
import torch.nn as nn

from .modules import ConvRotLinear, convrot_linear

# leaf paths adapted inside each DiT / text-fusion block (lora.py:23-24)
DEFAULT_TARGETS = ("attn.wq", "attn.wk", "attn.wv", "attn.wo", "attn.gate", "mlp.gate", "mlp.up", "mlp.down")


def _is_linear_like(m) -> bool:
    return isinstance(m, nn.Linear) or getattr(m, "is_quant_linear", False)


class LoRALinear(nn.Module):
    """``base(x) + (alpha/rank)*scale_mul * (x A^T) B^T``; A [rank,in] fp32 ~ U(+-1/sqrt(in)),
    B [out,rank] fp32 zeros; the base is frozen (lora.py:27-48)."""

    def __init__(self, base: nn.Module, rank: int, alpha: float):
        super().__init__()
        self.base = base
        for p in base.parameters():
            p.requires_grad_(False)
        self.rank = rank
        self.scale = alpha / rank
        self.scale_mul = 1.0
        dev = base.weight.device
        a = torch.empty(rank, base.in_features, device=dev, dtype=torch.float32)
        nn.init.kaiming_uniform_(a, a=math.sqrt(5))
        self.lora_A = nn.Parameter(a)
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, rank, device=dev, dtype=torch.float32))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.base(x)
        if self.scale_mul == 0.0:
            return y
        low = x.to(self.lora_A.dtype) @ self.lora_A.t()
        return y + (self.scale * self.scale_mul) * (low @ self.lora_B.t()).to(y.dtype)


class _FusedLoRAForward:
    """Mixin placed in front of an adapter class by :func:`fuse_lora`."""

    is_fused_lora = True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        base = self.base
        if self.scale_mul == 0.0:                      # lora.py:45-46: adapters off
            return base(x)
        if not getattr(base, "is_convrot_linear", False):
            return super().forward(x)
        if self.rank > 64 or (base.bits == 4 and self.rank > 32):
            return super().forward(x)                  # rank beyond the epilogue's register budget
        return convrot_linear(x, base, self.lora_A, self.lora_B, self.scale * self.scale_mul,
                              sibs=getattr(self, "_k2q_sibs", None), sib_off=getattr(self, "_k2q_sib_off", 0))


_fused_classes: dict[type, type] = {}


def _fused_class(cls: type) -> type:
    fused = _fused_classes.get(cls)
    if fused is None:
        fused = type("Fused" + cls.__name__, (_FusedLoRAForward, cls), {"__module__": __name__})
        _fused_classes[cls] = fused
    return fused


def _looks_like_adapter(m: nn.Module) -> bool:
    return all(hasattr(m, a) for a in ("base", "rank", "scale", "scale_mul", "lora_A", "lora_B"))


def fuse_lora(model: nn.Module) -> int:
    """Switches every adapter on a ConvRot base to the fused path; returns how many were switched.
    Works on this module's :class:`LoRALinear` and on the reference's (duck-typed)."""
    n = 0
    for m in model.modules():
        if getattr(m, "is_fused_lora", False) or not _looks_like_adapter(m):
            continue
        if isinstance(m.base, ConvRotLinear):
            m.__class__ = _fused_class(type(m))
            n += 1
    _link_siblings(model)
    return n


# Linears of the reference's block that read one tensor (mmdit.py:199 and :178): their adapters' down-projections
# x . A^T run as one pass over x with the A matrices stacked
_SIBLING_SETS = (("wq", "wk", "wv", "gate"), ("gate", "up"))


def _link_siblings(model: nn.Module) -> None:
    for parent in model.modules():
        for names in _SIBLING_SETS:
            members = [getattr(parent, nm, None) for nm in names]
            if any(m is None or not getattr(m, "is_fused_lora", False) for m in members):
                continue
            feats = {m.base.in_features for m in members}
            if (len(feats) != 1 or sum(m.rank for m in members) > 64
                    or any(m.lora_A.dtype != torch.float32 for m in members)):
                continue
            off = 0
            for m in members:
                m._k2q_sibs, m._k2q_sib_off = tuple(members), off
                off += m.rank
            break


def unfuse_lora(model: nn.Module) -> int:
    n = 0
    for m in model.modules():
        if getattr(m, "is_fused_lora", False):
            m.__class__ = type(m).__mro__[2]
            for attr in ("_k2q_sibs", "_k2q_sib_off"):
                if hasattr(m, attr):
                    delattr(m, attr)
            n += 1
    return n


@contextlib.contextmanager
def lora_scaled(model: nn.Module, factor: float):
    """Temporarily sets ``scale_mul`` of every adapter (negative inverts, 0 disables); restores
    the previous values on exit (lora.py:51-65)."""
    mods = [m for m in model.modules() if _looks_like_adapter(m)]
    prev = [m.scale_mul for m in mods]
    try:
        for m in mods:
            m.scale_mul = float(factor)
        yield
    finally:
        for m, p in zip(mods, prev):
            m.scale_mul = p


def lora_disabled(model: nn.Module):
    return lora_scaled(model, 0.0)


def _walk(parent: nn.Module, dotted: str):
    parts = dotted.split(".")
    for p in parts[:-1]:
        parent = getattr(parent, p)
    return parent, parts[-1]


def inject_lora(dit, rank: int, alpha: float | None = None, *, targets=DEFAULT_TARGETS,
                include_txtfusion: bool = True, include_txtmlp: bool = True, fuse: bool = True) -> dict:
    """Freezes ``dit`` and wraps each target Linear (plain or quantized) with an adapter; returns
    ``{dotted name: adapter}`` in traversal order (lora.py:81-116).  ``fuse`` additionally runs
    :func:`fuse_lora`."""
    alpha = float(rank) if alpha is None else alpha
    dit.requires_grad_(False)
    groups = [("blocks", dit.blocks)]
    if include_txtfusion:
        groups += [("txtfusion.layerwise_blocks", dit.txtfusion.layerwise_blocks),
                   ("txtfusion.refiner_blocks", dit.txtfusion.refiner_blocks)]
    adapters: dict[str, LoRALinear] = {}
    for prefix, blocks in groups:
        for i, blk in enumerate(blocks):
            for tgt in targets:
                try:
                    parent, leaf = _walk(blk, tgt)
                    base = getattr(parent, leaf)
                except AttributeError:
                    continue
                if not _is_linear_like(base):
                    continue
                ad = LoRALinear(base, rank, alpha)
                setattr(parent, leaf, ad)
                adapters[f"{prefix}.{i}.{tgt}"] = ad
    if include_txtmlp:
        for name, base in list(dit.txtmlp.named_modules()):
            if not name or not _is_linear_like(base):
                continue
            parent, leaf = _walk(dit.txtmlp, name)
            ad = LoRALinear(base, rank, alpha)
            setattr(parent, leaf, ad)
            adapters[f"txtmlp.{name}"] = ad
    if not adapters:
        raise RuntimeError("inject_lora matched no Linear targets; check target names vs the DiT")
    if fuse:
        fuse_lora(dit)
    return adapters


def lora_parameters(adapters: dict) -> list:
    out = []
    for m in adapters.values():
        out += [m.lora_A, m.lora_B]
    return out
