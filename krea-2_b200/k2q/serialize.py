"""On-disk form of a ConvRot-quantized base: codes and scales in one safetensors file, so that a
start-up loads them instead of rotating and quantising 12 B bf16 weights again
(train_t2i_lora_cached.py:83-88 re-quantises at every start).

Keys follow the adapter files' convention of lora.py:154-172 (``<key_prefix>.<module path>.<tensor>``,
atomic replace of a ``.tmp`` file, string metadata):

    diffusion_model.blocks.3.attn.wq.weight_q      int8 [N,K]   or uint8 [N,K/2] (low nibble = even k)
    diffusion_model.blocks.3.attn.wq.scale         fp32 [N]     or bf16 [N,K/128]
    diffusion_model.blocks.3.attn.wq.bias          the Linear's bias, when it has one
    diffusion_model.blocks.3.attn.wq.weight_q8 / .scale_bwd     int4 bases quantised for training

metadata: ``format = krea2-convrot``, ``bits``, ``group``, ``had_block``, ``count``.
"""
from __future__ import annotations

import os

import torch
import torch.nn as nn

from .modules import GROUP, HAD_BLOCK, ConvRotLinear, share_block_inputs

FORMAT = "krea2-convrot"


def convrot_modules(model: nn.Module) -> dict:
    """name -> ConvRotLinear for every quantized Linear in ``model`` (also below LoRA wrappers, whose
    ``.base`` then appears in the path exactly as it does in ``state_dict()``)."""
    return {name: m for name, m in model.named_modules() if isinstance(m, ConvRotLinear)}


def save_quantized_base(model: nn.Module, path: str, *, key_prefix: str = "diffusion_model",
                        metadata: dict | None = None) -> int:
    """Writes every ConvRotLinear of ``model``; returns how many.  All must share one bit width."""
    from safetensors.torch import save_file
    mods = convrot_modules(model)
    if not mods:
        raise RuntimeError("save_quantized_base: the model holds no ConvRotLinear")
    bits = {m.bits for m in mods.values()}
    if len(bits) != 1:
        raise ValueError(f"save_quantized_base: mixed bit widths {sorted(bits)}")
    sd = {}
    for name, m in mods.items():
        base = f"{key_prefix}.{name}"
        sd[f"{base}.weight_q"] = m.weight_q.data.cpu().contiguous()
        sd[f"{base}.scale"] = m.scale.cpu().contiguous()
        if m.bias is not None:
            sd[f"{base}.bias"] = m.bias.data.cpu().contiguous()
        if m.weight_q8 is not None:
            sd[f"{base}.weight_q8"] = m.weight_q8.data.cpu().contiguous()
            sd[f"{base}.scale_bwd"] = m.backward_scale.cpu().contiguous()
    meta = {"format": FORMAT, "bits": str(bits.pop()), "group": str(GROUP), "had_block": str(HAD_BLOCK),
            "count": str(len(mods))}
    if metadata:
        meta.update({k: str(v) for k, v in metadata.items()})
    tmp = path + ".tmp"
    save_file(sd, tmp, metadata=meta)
    os.replace(tmp, path)
    return len(mods)


def _set_submodule(root: nn.Module, dotted: str, new: nn.Module) -> nn.Module:
    parent = root.get_submodule(dotted.rsplit(".", 1)[0]) if "." in dotted else root
    leaf = dotted.rsplit(".", 1)[-1]
    old = getattr(parent, leaf)
    setattr(parent, leaf, new)
    return old


def load_quantized_base(model: nn.Module, path: str, *, key_prefix: str = "diffusion_model", device=None,
                        share_inputs: bool = True) -> int:
    """Replaces the ``nn.Linear`` (or ConvRotLinear) at every saved module path of ``model`` by a
    ConvRotLinear built from the stored codes -- no rotation, no quantisation, the bf16 weight is
    never needed (the model may be built on the ``meta`` device).  Call it where the reference calls
    ``quantize_dit_fp8`` (before ``inject_lora``).  Returns the number of modules replaced; raises if a
    saved path does not exist in the model or its shape disagrees."""
    from safetensors import safe_open
    with safe_open(path, framework="pt", device="cpu") as f:
        meta = f.metadata() or {}
        if meta.get("format") != FORMAT:
            raise ValueError(f"{path}: not a {FORMAT} file (format={meta.get('format')!r})")
        if int(meta.get("group", GROUP)) != GROUP or int(meta.get("had_block", HAD_BLOCK)) != HAD_BLOCK:
            raise ValueError(f"{path}: group / rotation block {meta.get('group')}/{meta.get('had_block')} not built here")
        bits = int(meta["bits"])
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    pre = key_prefix + "."
    names = sorted({k[len(pre):].rsplit(".", 1)[0] for k in tensors if k.startswith(pre) and k.endswith(".weight_q")})
    if not names:
        raise ValueError(f"{path}: no '{pre}*.weight_q' tensors")

    def dev_of(t):
        return t.to(device) if device is not None else t

    for name in names:
        base = pre + name
        q, s = tensors[f"{base}.weight_q"], tensors[f"{base}.scale"]
        bias = tensors.get(f"{base}.bias")
        q8, sb = tensors.get(f"{base}.weight_q8"), tensors.get(f"{base}.scale_bwd")
        mod = ConvRotLinear.from_codes(dev_of(q), dev_of(s), None if bias is None else dev_of(bias), bits,
                                       None if q8 is None else dev_of(q8), None if sb is None else dev_of(sb))
        try:
            old = model.get_submodule(name)
        except AttributeError as ex:
            raise KeyError(f"{path}: the model has no module '{name}'") from ex
        if (getattr(old, "in_features", mod.in_features), getattr(old, "out_features", mod.out_features)) != \
                (mod.in_features, mod.out_features):
            raise ValueError(f"{name}: stored {mod.out_features}x{mod.in_features}, model "
                             f"{old.out_features}x{old.in_features}")
        _set_submodule(model, name, mod)
    if share_inputs and hasattr(model, "blocks"):
        for block in model.blocks:
            share_block_inputs(block)
    return len(names)


def quantize_text_side(dit, bits: int = 8, backward_copy: bool | None = None) -> int:
    """Extends the replacement to the Linears that ``quantize_dit_fp8`` leaves in bf16 but that are
    part of "all base Linears" of the model: the text-fusion blocks and the text MLP (mmdit.py:360-375;
    quantize.py:60-65 covers ``dit.blocks`` only).  Linears whose in_features is not a multiple of the
    rotation block, or out_features not a multiple of 16, stay as they are.  Returns the count."""
    if backward_copy is None:
        backward_copy = False
    roots = []
    tf = getattr(dit, "txtfusion", None)
    if tf is not None:
        roots += list(getattr(tf, "layerwise_blocks", [])) + list(getattr(tf, "refiner_blocks", []))
    if getattr(dit, "txtmlp", None) is not None:
        roots.append(dit.txtmlp)
    targets = []
    for root in roots:
        for mod in root.modules():
            for name, child in mod.named_children():
                if isinstance(child, nn.Linear) and child.in_features % HAD_BLOCK == 0 and child.out_features % 16 == 0:
                    targets.append((mod, name, child))
    for mod, name, child in targets:
        setattr(mod, name, ConvRotLinear(child, bits=bits, backward_copy=backward_copy))
    for root in roots:
        share_block_inputs(root)
    return len(targets)
