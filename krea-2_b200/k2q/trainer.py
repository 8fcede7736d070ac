"""Trainer-level pieces around the path (train_t2i_lora_cached.py:83-97, 327-332; mmdit.py:389-428):

* :class:`FusedAdapterStep`  ``clip_grad_norm_`` + ``AdamW.step`` + ``zero_grad`` of all adapter
  parameters as two kernel launches over flat buffers (the reference runs them as a few thousand
  small launches over 516 tensors).
* :func:`enable_prefetching_block_swap`  block swap whose frozen blocks live in pinned host memory:
  the next swapped block is copied in on a side stream while the current one computes, and paging a
  block out is free -- its codes never change, so the device copy is simply dropped.
* :func:`quantized_training_defaults`  what the quantised base lets the trainer relax.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.nn as nn

from . import _lib, ops
from .parallel import AdapterGradBuckets


class FusedAdapterStep:
    """AdamW (torch.optim.AdamW's update rule, decoupled weight decay) with global-norm gradient
    clipping over the parameters of an :class:`~k2q.parallel.AdapterGradBuckets`.

    Parameters, gradients and both moments are flat fp32 buffers in the buckets' order; every
    parameter's ``.data`` is re-pointed at its slice (values kept), so modules, ``state_dict`` and
    ``save_lora`` (lora.py:154-172) see ordinary tensors.  ``step()`` = ``buckets.finish()`` (the
    exchange) -> gradient norm -> update -> gradients zeroed; call ``buckets.zero()`` is not needed
    afterwards, the arrival counters are re-armed here.
    """

    def __init__(self, buckets: AdapterGradBuckets, lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, max_grad_norm: float = 1.0):
        self.buckets = buckets
        self.lr, self.betas, self.eps, self.weight_decay, self.max_grad_norm = lr, betas, eps, weight_decay, max_grad_norm
        g = buckets.flat
        if not g.is_cuda:
            raise RuntimeError("FusedAdapterStep runs on CUDA tensors only; there is no CPU fallback")
        self.param = torch.empty_like(g)
        off = 0
        for b in buckets.buckets:
            for p in b["params"]:
                n = p.numel()
                self.param[off:off + n].copy_(p.data.reshape(-1))
                p.data = self.param[off:off + n].view_as(p)
                off += n
        self.m = torch.zeros_like(g)
        self.v = torch.zeros_like(g)
        self.normsq = torch.zeros(1, dtype=torch.float32, device=g.device)
        self.ws = torch.empty(int(_lib.load().k2q_sumsq_workspace_bytes()) // 4, dtype=torch.float32, device=g.device)
        self.step_count = 0

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the last clipped step's gradients (device scalar, no synchronisation)."""
        return self.normsq.sqrt()

    @torch.no_grad()
    def step(self, lr: float | None = None) -> None:
        bk = self.buckets
        bk.finish()
        g = bk.flat
        dev = g.device
        lib = _lib.load()
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        self.step_count += 1
        with torch.cuda.device(dev):
            norm_ptr = C.c_void_p(0)
            if self.max_grad_norm and self.max_grad_norm > 0:
                _lib.check(lib.k2q_sumsq_f32(C.c_void_p(g.data_ptr()), g.numel(), C.c_void_p(self.normsq.data_ptr()), 0,
                                             C.c_void_p(self.ws.data_ptr()), self.ws.numel() * 4, stream), "k2q_sumsq_f32")
                norm_ptr = C.c_void_p(self.normsq.data_ptr())
            _lib.check(lib.k2q_adamw_clip_f32(C.c_void_p(self.param.data_ptr()), C.c_void_p(g.data_ptr()),
                                              C.c_void_p(self.m.data_ptr()), C.c_void_p(self.v.data_ptr()), g.numel(),
                                              float(self.lr if lr is None else lr), float(self.betas[0]),
                                              float(self.betas[1]), float(self.eps), float(self.weight_decay),
                                              self.step_count, float(self.max_grad_norm or 0.0), norm_ptr, 1, stream),
                       "k2q_adamw_clip_f32")
        for b in bk.buckets:                       # gradients are zero again: re-arm the arrival counters
            b["pending"], b["launched"] = len(b["params"]), False

    def state_dict(self) -> dict:
        return {"step": self.step_count, "m": self.m, "v": self.v}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])


class _PrefetchSwap:
    """State of :func:`enable_prefetching_block_swap` for one model."""

    def __init__(self, blocks, swapped, device, checkpointed=True):
        self.blocks, self.swapped, self.device, self.checkpointed = blocks, swapped, torch.device(device), checkpointed
        self.order = sorted(swapped)
        self.host: dict[int, list] = {}          # block -> [(param, pinned host tensor)]
        self.ready: dict[int, object] = {}       # block -> event of the copy in flight (cuda) / True
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.copies = 0                          # host -> device block copies issued (for tests / reports)

    def frozen(self, block):
        return [p for p in block.parameters() if not p.requires_grad]

    def park(self, i):
        pairs = []
        for p in self.frozen(self.blocks[i]):
            h = p.data.to("cpu")
            if self.device.type == "cuda":
                h = h.pin_memory()
            p.data = h
            pairs.append((p, h))
        self.host[i] = pairs

    def fetch(self, i, asynchronous: bool):
        if i in self.ready or i not in self.host:
            return
        self.copies += 1
        if self.stream is not None and asynchronous:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                for p, h in self.host[i]:
                    p.data = h.to(self.device, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            self.ready[i] = ev
        else:
            for p, h in self.host[i]:
                p.data = h.to(self.device, non_blocking=self.stream is not None)
            self.ready[i] = True

    def drop(self, i):
        """Page block i out: the codes are frozen, the pinned host copy is still valid."""
        if i in self.ready:
            ev = self.ready.pop(i)
            if ev is not True:
                torch.cuda.current_stream(self.device).wait_event(ev)
            for p, h in self.host[i]:
                if self.stream is not None:
                    p.data.record_stream(torch.cuda.current_stream(self.device))
                p.data = h

    @staticmethod
    def _in_backward() -> bool:
        return torch._C._current_graph_task_id() != -1      # a checkpoint recompute runs inside backward

    def pre_hook(self, i):
        def hook(module, args):
            self.fetch(i, asynchronous=False)              # normally already in flight
            ev = self.ready.get(i)
            if ev is not None and ev is not True:
                torch.cuda.current_stream(self.device).wait_event(ev)
                self.ready[i] = True
            pos = self.order.index(i)
            nxt = pos - 1 if self._in_backward() else pos + 1     # the backward walks the blocks in reverse
            if 0 <= nxt < len(self.order):
                self.fetch(self.order[nxt], asynchronous=True)    # overlaps with this block's kernels
        return hook

    def post_hook(self, i):
        def hook(module, args, output):
            if not torch.is_grad_enabled() or (self.checkpointed and not self._in_backward()):
                self.drop(i)                               # inference, or the first pass of a checkpointed block
                return
            # a forward whose graph autograd will walk (the recompute inside backward, or training without
            # checkpointing): the backward reads the codes again, so the block leaves after its backward
            x = next((a for a in args if isinstance(a, torch.Tensor) and a.requires_grad), None)
            if x is not None:
                x.register_hook(lambda grad: self.drop(i))
        return hook


def enable_prefetching_block_swap(dit, num_blocks: int, device, checkpointed: bool = True) -> _PrefetchSwap:
    """Block swap (mmdit.py:389-428) for a quantised base: the ``num_blocks`` deepest blocks keep their
    frozen parameters in pinned host memory; a block's codes are copied in on a side stream while the
    block before it runs and are dropped (not copied back) after its forward.  Under gradient
    checkpointing the recompute in the backward pages the block in again through the same hook, as in
    the reference (``checkpointed=True``, what the trainers use with a quantised base: a block's
    first pass is not differentiated, so it can leave at once); with ``checkpointed=False`` a block that
    ran with autograd on stays until its backward is done.  Trainable parameters (adapters) stay
    resident.  Returns the state object (``.copies`` counts host-to-device block copies)."""
    n = max(0, min(int(num_blocks), len(dit.blocks)))
    swapped = set(range(len(dit.blocks) - n, len(dit.blocks)))
    st = _PrefetchSwap(dit.blocks, swapped, device, checkpointed)
    for i in sorted(swapped):
        st.park(i)
        dit.blocks[i].register_forward_pre_hook(st.pre_hook(i))
        dit.blocks[i].register_forward_hook(st.post_hook(i), always_call=True)
    dit._k2q_prefetch_swap = st
    return st


def quantized_training_defaults(quantize_base: str) -> dict:
    """The reference forces gradient checkpointing whenever the base is quantised
    (train_t2i_lora_cached.py:93-97: autograd would keep a dequantised bf16 weight per layer).  The
    ConvRot backward keeps nothing of the sort -- it reads the stored codes again -- so checkpointing
    becomes a memory / time choice like for a bf16 base.  Returned: the settings a trainer may apply."""
    convrot = quantize_base in ("convrot_int8", "convrot_int4")
    return {"force_gradient_checkpointing": quantize_base == "fp8",
            "gradient_checkpointing_optional": convrot,
            "optimizer": "k2q.trainer.FusedAdapterStep" if convrot else "torch.optim.AdamW"}
