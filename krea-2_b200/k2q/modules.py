"""Drop-in quantized base Linear for the Krea 2 DiT: the module-replacement face of the path.

Mirrors the reference's ``quantize.py``:

* :class:`ConvRotLinear`   takes the place of ``Fp8Linear``       (quantize.py:23-51)
* :func:`quantize_dit_convrot` takes the place of ``quantize_dit_fp8`` (quantize.py:54-68)

The module keeps the reference's duck type (``is_quant_linear``, ``in_features`` / ``out_features``
/ ``weight`` / ``bias``, every tensor a ``requires_grad=False`` Parameter) so that the reference's
``LoRALinear`` / ``inject_lora`` (lora.py:27-116), gradient checkpointing and block-swap
(mmdit.py:389-428, 474-496) work on it unchanged.  All arithmetic happens in ``libk2q.so``;
device pointers are read at call time, never cached.
"""
from __future__ import annotations

import contextlib
import threading

import torch
import torch.nn as nn

from . import ops

HAD_BLOCK = ops.HAD_BLOCK
GROUP = ops.GROUP


class ConvRotLinear(nn.Module):
    """Frozen ``nn.Linear`` stored as Hadamard-rotated int8 (per-out-channel scale) or int4
    (group-128 bf16 scales, two codes per byte) and evaluated as

        y = int32(Q8(H x) . Wq^T) * sx * sw + bias          (W8A8 / W4A8 on tcgen05)

    * ``weight_q``   int8 [N,K]  or uint8 [N,K/2]
    * ``scale``      fp32 [N] (held as its int32 bit pattern in ``scale_bits`` so that a later
                     ``module.to(dtype=bf16)`` cannot round it)  or bf16 [N,K/128]

    The training backward dX = Q8(dY*sw) . Wq contracts over the output channels straight from
    ``weight_q`` as stored (the tensor core reads it as an MN-major operand): an 8-bit base costs one
    byte per weight, nothing else.  Group scales of a 4-bit base sit on both indices of dX's
    contraction, so its backward runs on the codes re-expressed against one scale per output channel
    (``ops.requant_i4_to_i8``): ``backward_copy=True`` keeps them resident (``weight_q8`` int8 [N,K] +
    ``scale_bwd`` fp32 [N], 1.5 bytes per weight in all), ``backward_copy="transient"`` rebuilds them
    inside every backward (0.5 byte per weight resident, one HBM pass over the layer per backward),
    ``False`` stores nothing and refuses a backward.

    ``fast=True`` (4-bit bases, needs the resident re-expression) evaluates the FORWARD on those int8
    codes too, with the W8A8 kernel at more than twice the W4A8 rate; the outputs then differ from the
    group-scaled definition by the re-expression's rounding (at most half an int8 step of the row
    scale per weight) and are no longer bit-exact with the int4 oracle.  Off by default.
    """

    is_quant_linear = True
    is_convrot_linear = True

    def __init__(self, lin: nn.Linear | None, bits: int = 8, group: int = GROUP, had_block: int = HAD_BLOCK,
                 backward_copy: bool | str = True, fast: bool = False):
        super().__init__()
        if bits not in (8, 4):
            raise ValueError(f"bits must be 8 or 4, got {bits}")
        if group != GROUP or had_block != HAD_BLOCK:
            raise ValueError(f"only group={GROUP} and had_block={HAD_BLOCK} are built")
        if backward_copy not in (True, False, "transient"):
            raise ValueError(f"backward_copy must be True, False or 'transient', got {backward_copy!r}")
        if fast and (bits != 4 or backward_copy is not True):
            raise ValueError("fast=True is the int8-rate forward of a 4-bit base and needs backward_copy=True")
        self.bits = bits
        self.fast = bool(fast)
        self.transient_backward = bits == 4 and backward_copy == "transient"
        self.weight_q8 = None
        self.scale_bwd = None
        if lin is None:          # filled by from_codes()
            return
        if lin.in_features % HAD_BLOCK:
            raise ValueError(f"in_features={lin.in_features} is not a multiple of the rotation block {HAD_BLOCK}")
        if lin.out_features % 16:
            raise ValueError(f"out_features={lin.out_features} is not a multiple of 16")
        w = lin.weight.data
        self.in_features, self.out_features = lin.in_features, lin.out_features
        if bits == 8:
            q, s = ops.quant_weight_i8(w)
            self.weight_q = nn.Parameter(q, requires_grad=False)
            self.scale_bits = nn.Parameter(s.view(torch.int32), requires_grad=False)
        else:
            q, s = ops.quant_weight_i4(w)
            self.weight_q = nn.Parameter(q, requires_grad=False)
            self.scale_bits = nn.Parameter(s, requires_grad=False)
            if backward_copy is True:
                self.ensure_backward_copy()
        self.bias = (nn.Parameter(lin.bias.data.clone(), requires_grad=False)
                     if lin.bias is not None else None)

    # -- construction from stored codes (serialised bases, host-side tests) -------------------
    @classmethod
    def from_codes(cls, weight_q: torch.Tensor, scale: torch.Tensor, bias: torch.Tensor | None, bits: int,
                   weight_q8: torch.Tensor | None = None, scale_bwd: torch.Tensor | None = None) -> "ConvRotLinear":
        self = cls(None, bits=bits)
        n = weight_q.shape[0]
        k = weight_q.shape[1] * (2 if bits == 4 else 1)
        if bits == 8:
            if weight_q.dtype != torch.int8 or scale.dtype != torch.float32 or scale.numel() != n:
                raise ValueError("int8 base needs int8 codes [N,K] and an fp32 scale [N]")
            scale = scale.reshape(n).contiguous().view(torch.int32)
        else:
            if weight_q.dtype != torch.uint8 or scale.dtype != torch.bfloat16 or tuple(scale.shape) != (n, k // GROUP):
                raise ValueError("int4 base needs packed uint8 codes [N,K/2] and a bf16 scale [N,K/128]")
        self.weight_q = nn.Parameter(weight_q, requires_grad=False)
        self.scale_bits = nn.Parameter(scale, requires_grad=False)
        self.bias = nn.Parameter(bias, requires_grad=False) if bias is not None else None
        self.in_features, self.out_features = k, n
        if weight_q8 is not None:
            if bits != 4 or scale_bwd is None or tuple(weight_q8.shape) != (n, k) or weight_q8.dtype != torch.int8:
                raise ValueError("weight_q8 [N,K] int8 + scale_bwd [N] fp32 belong to an int4 base")
            self.weight_q8 = nn.Parameter(weight_q8, requires_grad=False)
            self.scale_bwd = nn.Parameter(scale_bwd.reshape(n).contiguous().view(torch.int32), requires_grad=False)
        return self

    # -- protocol of quantize.py:44-46 ------------------------------------------------------------
    @property
    def weight(self) -> torch.Tensor:   # device probe for LoRALinear (lora.py:38)
        return self.weight_q

    @property
    def scale(self) -> torch.Tensor:
        s = self.scale_bits.data
        return s.view(torch.float32) if self.bits == 8 else s

    def ensure_backward_copy(self) -> None:
        """4-bit bases only: stores what dX = Q8(dY*s) . W needs.  Group scales sit on BOTH indices of
        dX's contraction, so the codes are re-expressed once per layer against one scale per output
        channel, ``s_n = max_g(sw4[n,g]) * 7/127`` and ``w8[n,k] = rint(q4[n,k] * (sw4[n,g] / s_n))``
        (|w8| <= 127; this adds at most half an int8 step of s_n to each weight, 5 % of the int4
        rounding step of the row's largest group).  Build it when the module is made
        (``backward_copy=True``), before optimizers or block swap take their snapshot of
        ``parameters()``."""
        if self.bits == 8 or self.weight_q8 is not None:
            return
        w8, s_n = ops.requant_i4_to_i8(self.weight_q.data, self.scale_bits.data)
        self.weight_q8 = nn.Parameter(w8, requires_grad=False)
        self.scale_bwd = nn.Parameter(s_n.contiguous().view(torch.int32), requires_grad=False)
        self.transient_backward = False

    def backward_operands(self):
        """(int8 codes [N,K], fp32 scale [N]) that the backward GEMM contracts with."""
        if self.bits == 8:
            return self.weight_q.data, self.scale
        if self.weight_q8 is not None:
            return self.weight_q8.data, self.scale_bwd.data.view(torch.float32)
        if self.transient_backward:
            return ops.requant_i4_to_i8(self.weight_q.data, self.scale_bits.data)
        raise RuntimeError("this int4 base was quantised for inference (backward_copy=False): quantise with "
                           "backward_copy=True or 'transient' to train through it")

    def forward_operands(self):
        """(GEMM wrapper, codes, scales) of the forward product."""
        if self.bits == 8:
            return ops.gemm_w8a8, self.weight_q.data, self.scale
        if self.fast:
            if self.weight_q8 is None:
                raise RuntimeError("fast=True needs the resident int8 re-expression (backward_copy=True)")
            return ops.gemm_w8a8, self.weight_q8.data, self.scale_bwd.data.view(torch.float32)
        return ops.gemm_w4a8, self.weight_q.data, self.scale

    @property
    def backward_codes(self) -> torch.Tensor:
        """int8 [N,K] codes the backward GEMM contracts with."""
        if self.bits == 8:
            return self.weight_q.data
        return self.backward_operands()[0]

    @property
    def backward_scale(self) -> torch.Tensor:
        """Per-output-channel fp32 scale that goes with ``backward_codes``."""
        return self.backward_operands()[1]

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}, "
                f"bias={self.bias is not None}")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return convrot_linear(x, self)


def _bias_f32(mod: ConvRotLinear):
    if mod.bias is None:
        return None
    b = mod.bias.data
    return b if b.dtype == torch.float32 else b.float()


class _QuantScope(threading.local):
    """Per-thread state of :func:`shared_input_quant`."""

    def __init__(self):
        self.depth = 0
        self.key = None
        self.src = None      # keeps the quantised tensor alive while its codes are cached
        self.codes = None
        self.u_key = None    # the same for the stacked adapter down-projection of sibling Linears
        self.u_src = None
        self.u_all = None


_scope = _QuantScope()


@contextlib.contextmanager
def shared_input_quant():
    """Scope in which Linears that read the SAME tensor share one rotation + quantisation pass:
    wq / wk / wv / gate of a block (mmdit.py:199) and mlp.gate / mlp.up (mmdit.py:178).

    Inside the scope the last quantised input is remembered and recognised by address, layout,
    in-place version, the stream it was quantised on, whether that stream was being captured into a
    CUDA graph, and a counter that every k2q call writing through a raw pointer into a caller's
    buffer advances (``ops.note_raw_write``; such writes do not change ``Tensor._version``).  Leaving
    the outermost scope drops the entry, so nothing outlives a block forward: a CUDA graph captured
    after a warm-up run re-quantises inside the capture, and no activation stays pinned.
    Outside any scope every call quantises its own input."""
    _scope.depth += 1
    try:
        yield
    finally:
        _scope.depth -= 1
        if _scope.depth == 0:
            _scope.key = _scope.src = _scope.codes = None
            _scope.u_key = _scope.u_src = _scope.u_all = None


def _quantize_input(x2: torch.Tensor):
    if _scope.depth == 0:
        return ops.fwht_quant_act(x2)
    key = _input_key(x2)
    if _scope.key == key:
        return _scope.codes
    codes = ops.fwht_quant_act(x2)
    _scope.key, _scope.src, _scope.codes = key, x2, codes
    return codes


def _input_key(x2: torch.Tensor):
    stream = torch.cuda.current_stream(x2.device)
    return (x2.data_ptr(), tuple(x2.shape), x2.stride(), x2.dtype, x2._version, x2.device.index,
            stream.cuda_stream, torch.cuda.is_current_stream_capturing(), ops.raw_write_epoch())


def _adapter_down(x2: torch.Tensor, lora_a: torch.Tensor, sibs, off: int) -> torch.Tensor:
    """u = x . A^T of one adapter.  Adapters that ``fuse_lora`` found to read one tensor (wq / wk / wv / gate
    of a block, mlp.gate / mlp.up: ``sibs``) share ONE pass over x inside :func:`shared_input_quant`: the first
    of them stacks all their A matrices, and each takes its columns of the result (a strided view)."""
    if sibs is None or _scope.depth == 0:
        return ops.lora_down(x2, lora_a.detach())
    key = _input_key(x2) + tuple(id(m) for m in sibs)
    if _scope.u_key != key:
        a_cat = torch.cat([m.lora_A.detach() for m in sibs], dim=0)
        _scope.u_key, _scope.u_src, _scope.u_all = key, x2, ops.lora_down(x2, a_cat)
    return _scope.u_all[:, off:off + lora_a.shape[0]]


def _enter_scope_hook(module, args):
    module._k2q_scope = shared_input_quant()
    module._k2q_scope.__enter__()


def _exit_scope_hook(module, args, output):
    scope = getattr(module, "_k2q_scope", None)
    if scope is not None:
        module._k2q_scope = None
        scope.__exit__(None, None, None)


def share_block_inputs(block: nn.Module) -> None:
    """Makes every forward of ``block`` run inside :func:`shared_input_quant` (forward hooks; the
    scope is left even when the forward raises).  ``quantize_dit_convrot`` does this for each DiT
    block, so the reference's ``SingleStreamBlock.forward`` (mmdit.py:310-319) needs no change."""
    if getattr(block, "_k2q_shared_hooks", False):
        return
    block.register_forward_pre_hook(_enter_scope_hook)
    block.register_forward_hook(_exit_scope_hook, always_call=True)
    block._k2q_shared_hooks = True


class _ConvRotFn(torch.autograd.Function):
    """y = base(x) [+ s * (x A^T) B^T] with the hand-written backward:

        dX = H( Q8(dY*sw) . Wq  +  du . H(A) )        du = s * dY . B      (Wq as stored, [N, K])
        dA = du^T x ,  dB = s * dY^T u                 (autograd of lora.py:47-48)

    No gradient reaches codes or scales (quantize.py:38-41: frozen Parameters).
    """

    @staticmethod
    def forward(ctx, x, mod, lora_a, lora_b, lora_scale, sibs=None, sib_off=0):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        x2 = x2.contiguous()
        use_lora = lora_a is not None and lora_scale != 0.0
        u = _adapter_down(x2, lora_a, sibs, sib_off) if use_lora else None
        xq, sx = _quantize_input(x2)
        gemm, codes, scale = mod.forward_operands()
        y = gemm(xq, sx, codes, scale, _bias_f32(mod), u=u, bm=lora_b.detach() if use_lora else None,
                 lora_scale=lora_scale)
        ctx.mod = mod
        ctx.lora_scale = lora_scale
        ctx.use_lora = use_lora
        ctx.lead = lead
        need_w = use_lora and (lora_a.requires_grad or lora_b.requires_grad)
        if use_lora:
            ctx.save_for_backward(x2 if need_w else None, u if need_w else None, lora_a, lora_b)
        else:
            ctx.save_for_backward(None, None, None, None)
        return y.reshape(*lead, mod.out_features).to(x.dtype)

    @staticmethod
    def backward(ctx, gy):
        mod: ConvRotLinear = ctx.mod
        x2, u, lora_a, lora_b = ctx.saved_tensors
        s = ctx.lora_scale
        gy2 = gy.reshape(-1, mod.out_features)
        if gy2.dtype != torch.bfloat16:
            gy2 = gy2.to(torch.bfloat16)
        gy2 = gy2.contiguous()
        need_dx = ctx.needs_input_grad[0]
        need_a = ctx.use_lora and ctx.needs_input_grad[2]
        need_b = ctx.use_lora and ctx.needs_input_grad[3]

        du = None
        if ctx.use_lora and (need_dx or need_a):
            du = ops.lora_down(gy2, lora_b.detach(), scale=s, transposed=True)          # [T, r]

        gx = None
        if need_dx:
            wq8, sb = mod.backward_operands()
            gq, sg = ops.quant_rows(gy2, sb)
            bm = None
            if du is not None:
                bm = ops.fwht_rows(lora_a.detach()).t().contiguous()                    # H(A)^T  [K, r]
            gxr = ops.gemm_dx_w8(gq, sg, wq8, u=du, bm=bm, lora_scale=1.0)
            gx = ops.fwht_rows(gxr).reshape(*ctx.lead, mod.in_features).to(gy.dtype)
        ga = ops.lora_tn(du, x2) if need_a else None                                     # [r, K]
        gb = ops.lora_tn(u, gy2, scale=s).t().contiguous() if need_b else None           # [N, r]
        return gx, None, ga, gb, None, None, None


def convrot_linear(x: torch.Tensor, mod: ConvRotLinear, lora_a=None, lora_b=None, lora_scale: float = 0.0,
                   sibs=None, sib_off: int = 0):
    """Functional form; ``lora_*`` fuse an adapter term into the same GEMM epilogue.  ``sibs`` (adapter
    modules that read the same tensor, this one's A at row ``sib_off`` of their stack) lets them share the
    down-projection pass."""
    if not x.is_cuda:
        raise RuntimeError("ConvRotLinear runs on CUDA tensors only; there is no CPU fallback")
    if x.shape[-1] != mod.in_features:
        raise ValueError(f"last dim {x.shape[-1]} != in_features {mod.in_features}")
    return _ConvRotFn.apply(x, mod, lora_a, lora_b, float(lora_scale), sibs, int(sib_off))


@torch.no_grad()
def convrot_linear_quantized(xq: torch.Tensor, sx: torch.Tensor, mod: ConvRotLinear) -> torch.Tensor:
    """``mod`` applied to activations that are already rotated and quantized (codes ``xq`` [T, K] int8,
    per-token scales ``sx`` [T]): the GEMM alone.  Inference only, no adapter term.  Used where the
    codes rather than the activations travel between GPUs."""
    if xq.shape[-1] != mod.in_features:
        raise ValueError(f"last dim {xq.shape[-1]} != in_features {mod.in_features}")
    gemm, codes, scale = mod.forward_operands()
    return gemm(xq, sx, codes, scale, _bias_f32(mod))


class ConvRotGroup:
    """Linears that read the SAME tensor (wq | wk | wv | gate, mmdit.py:199; mlp.gate | mlp.up,
    mmdit.py:178) evaluated by ONE GEMM launch over their concatenated output channels.

    The members' codes, scales and biases are laid end to end in one allocation and every member's
    parameters are re-pointed at its slice, so nothing is stored twice and each member still works on
    its own (``state_dict``, adapters, sharding, paging).  If a member is later given other storage
    (block swap pages ``p.data``, mmdit.py:409-414) the group notices and falls back to one launch per
    member.  Not an ``nn.Module`` on purpose: it owns no parameters of its own."""

    def __init__(self, members):
        members = list(members)
        if len(members) < 2 or not all(type(m) is ConvRotLinear for m in members):
            raise TypeError("ConvRotGroup takes two or more bare ConvRotLinear modules")
        bits, k = members[0].bits, members[0].in_features
        if any(m.bits != bits or m.in_features != k for m in members):
            raise ValueError("grouped Linears must share bit width and in_features")
        if any(m.fast for m in members):
            raise ValueError("members with fast=True run from their own int8 codes and are not grouped")
        if len({m.bias is None for m in members}) != 1:
            raise ValueError("grouped Linears must all have a bias or all have none")
        self.members, self.bits, self.in_features = members, bits, k
        self.splits = [m.out_features for m in members]
        self.out_features = sum(self.splits)
        self.weight_q = torch.cat([m.weight_q.data for m in members], dim=0)
        self.scale_bits = torch.cat([m.scale_bits.data for m in members], dim=0)
        self.bias = None if members[0].bias is None else torch.cat([m.bias.data.float() for m in members], dim=0)
        off = 0
        for m, n in zip(members, self.splits):
            m.weight_q.data = self.weight_q[off:off + n]
            m.scale_bits.data = self.scale_bits[off:off + n]
            off += n

    def _aliased(self) -> bool:
        off = 0
        row = self.weight_q.stride(0) * self.weight_q.element_size()
        for m, n in zip(self.members, self.splits):
            if m.weight_q.data.data_ptr() != self.weight_q.data_ptr() + off * row or \
                    m.weight_q.data.device != self.weight_q.device:
                return False
            off += n
        return True

    @torch.no_grad()
    def forward_codes(self, xq: torch.Tensor, sx: torch.Tensor):
        """Outputs of all members for activations given as rotated codes: a tuple of [T, N_i] tensors
        (column slices of one [T, sum N_i] result when the group is intact).  Inference only."""
        if not self._aliased():
            return tuple(convrot_linear_quantized(xq, sx, m) for m in self.members)
        scale = self.scale_bits.view(torch.float32) if self.bits == 8 else self.scale_bits
        gemm = ops.gemm_w8a8 if self.bits == 8 else ops.gemm_w4a8
        y = gemm(xq, sx, self.weight_q, scale, self.bias)
        return tuple(y.split(self.splits, dim=1))


def group_shared_input_linears(dit) -> int:
    """Builds a :class:`ConvRotGroup` for the q/k/v/gate projections and one for mlp.gate/up of every
    block under ``dit.blocks`` whose members are bare ConvRotLinear modules (call after
    ``quantize_dit_convrot`` and any sharding, before inference).  The groups are stored as
    ``attn.qkvg_group`` / ``mlp.gu_group`` and used by the code paths that work from codes.  Returns the
    number of groups built."""
    n = 0
    for block in dit.blocks:
        attn, mlp = getattr(block, "attn", None), getattr(block, "mlp", None)
        for owner, names, attr in ((attn, ("wq", "wk", "wv", "gate"), "qkvg_group"), (mlp, ("gate", "up"), "gu_group")):
            if owner is None:
                continue
            members = [getattr(owner, nm, None) for nm in names]
            if all(type(m) is ConvRotLinear and not m.fast for m in members):
                object.__setattr__(owner, attr, ConvRotGroup(members))
                n += 1
    return n


def fused_prologue_ok(x: torch.Tensor, *linears) -> bool:
    """True when the elementwise step in front of ``linears`` can be folded into their quantisation
    pass (``ops.norm_mod_quant`` / ``swiglu_quant`` / ``gate_quant``): inference (no autograd), bf16
    CUDA activations, and every Linear a bare ConvRotLinear (an adapter needs the dense input)."""
    return (not torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.bfloat16
            and all(type(m) is ConvRotLinear for m in linears))


def quantize_dit_convrot(dit, bits: int = 8, group: int = GROUP, had_block: int = HAD_BLOCK,
                         backward_copy: bool | str | None = None, share_inputs: bool = True,
                         fast: bool = False) -> int:
    """Replaces every ``nn.Linear`` under ``dit.blocks`` with :class:`ConvRotLinear`, in place, and
    returns how many were replaced -- the traversal and contract of ``quantize_dit_fp8``
    (quantize.py:54-68): ``first`` / ``last`` / text fusion / time MLP stay bf16; call it BEFORE
    ``inject_lora``.  ``backward_copy`` matters for 4-bit bases only (default off: inference): it also
    stores the per-channel int8 re-expression the training backward needs (``"transient"``: rebuilt in
    every backward instead); 8-bit bases train from the stored codes.  ``fast`` (4-bit, implies the
    resident re-expression): forward at the int8 rate, see :class:`ConvRotLinear`.  ``share_inputs`` wraps each block's forward in
    :func:`shared_input_quant` so that Linears reading one tensor quantise it once."""
    if backward_copy is None:
        backward_copy = bool(fast)
    targets = []
    for block in dit.blocks:
        for mod in block.modules():
            for name, child in mod.named_children():
                if isinstance(child, nn.Linear):
                    targets.append((mod, name, child))
    for mod, name, child in targets:
        setattr(mod, name, ConvRotLinear(child, bits=bits, group=group, had_block=had_block,
                                         backward_copy=backward_copy, fast=fast and bits == 4))
    if share_inputs:
        for block in dit.blocks:
            share_block_inputs(block)
    return len(targets)


@torch.no_grad()
def convrot_mlp_gelu(x: torch.Tensor, fc1: ConvRotLinear, fc2: ConvRotLinear) -> torch.Tensor:
    """Forward of ``Sequential(Linear, GELU(approximate="tanh"), Linear)`` (the shape of the DiT's
    ``tmlp`` / ``txtmlp`` stages, mmdit.py:360-375) over two ConvRot bases with the GELU fused into
    the first GEMM's epilogue: K2 -> GEMM(+GELU) -> K2 -> GEMM.  Inference only."""
    if not x.is_cuda:
        raise RuntimeError("convrot_mlp_gelu runs on CUDA tensors only; there is no CPU fallback")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    g1, c1, s1 = fc1.forward_operands()
    g2, c2, s2 = fc2.forward_operands()
    xq, sx = ops.fwht_quant_act(x2)
    h = g1(xq, sx, c1, s1, _bias_f32(fc1), act="gelu_tanh")
    hq, sh = ops.fwht_quant_act(h)
    y = g2(hq, sh, c2, s2, _bias_f32(fc2))
    return y.reshape(*lead, fc2.out_features)


_side_streams: dict[int, tuple] = {}


def host_chunk_schedule(m: int, chunks: int | None = None, w4a8_out: int | None = None, sms: int = 148) -> list[int]:
    """Rows per piece for :func:`convrot_mlp_gelu_host`.  An integer gives that many equal pieces
    (multiples of 256 rows).  ``None`` picks the schedule that measured best on a B200:

    * W8A8 pair (``w4a8_out`` None): a ramp.  The first piece's copy-in and the last piece's kernels and
      copy-out are all that nothing hides, so the pieces grow 192, 384, 768 rows at the front, run at
      about 1152 rows in the middle and shrink 768, 384 at the back.
    * a W4A8 base (``w4a8_out`` = out_features of the second Linear): the kernels of a piece cost a fixed
      ~0.1 ms below ~800 rows, and the second GEMM wants its 128 x 192 tiles to fill the SMs exactly once,
      so every piece but the ends is 192 * k rows with k in 4..8 chosen for the fullest waves (1152 rows for
      3072 features on 148 SMs: 144 tiles), the first is 768 rows and the last takes what is left."""
    if m <= 0:
        return []
    if chunks is not None:
        step = max(256, -(-m // max(int(chunks), 1) // 256) * 256)
        return [min(step, m - a) for a in range(0, m, step)]
    if w4a8_out is not None:
        n_tiles = max(1, -(-int(w4a8_out) // 128))
        fill = lambda k: (k * n_tiles) / (-(-(k * n_tiles) // sms) * sms)      # how full the GEMM's waves are  # noqa: E731
        body = 192 * max(range(4, 9), key=lambda k: (round(fill(k), 2), k))
        if m <= 768 + body // 2:
            return [m]
        sched, left = [768], m - 768
        while left > 0:
            take = min(body, left)
            if 0 < left - take < 192:          # a sliver at the end joins the piece before it
                take = left
            sched.append(take)
            left -= take
        return sched
    head, tail, mid = [192, 384, 768], [768, 384], 1152
    inner = m - sum(head) - sum(tail)
    if inner < mid:                       # short inputs: equal pieces of at most 768 rows
        n = -(-m // 768)
        step = -(-m // n // 64) * 64
        return [min(step, m - a) for a in range(0, m, step)]
    n = max(1, round(inner / mid))
    step = -(-inner // n // 192) * 192
    return head + [min(step, inner - a) for a in range(0, inner, step)] + tail


def _linear_desc(mod: "ConvRotLinear", keep: list):
    """``k2q_linear`` of a base for the host pipeline (its forward operands, whichever kernel they go to)."""
    gemm, codes, scale = mod.forward_operands()
    bias = _bias_f32(mod)
    keep.extend((codes, scale, bias))
    return ops.linear_desc(8 if gemm is ops.gemm_w8a8 else 4, codes, scale, bias, mod.out_features, mod.in_features)


@torch.no_grad()
def convrot_mlp_gelu_host(x_host: torch.Tensor, fc1: ConvRotLinear, fc2: ConvRotLinear,
                          out_host: torch.Tensor | None = None, chunks: int | None = None) -> torch.Tensor:
    """:func:`convrot_mlp_gelu` for (pinned) HOST tensors: tokens are cut in pieces
    (:func:`host_chunk_schedule`) and the host-to-device copy of piece i+1, the kernels of piece i and
    the device-to-host copy of piece i-1 run on three streams at once, all enqueued by one call into
    the library (``k2q_mlp_gelu_host``), so the call costs little more than the slower of the two
    copies running together and the kernels.  Returns ``out_host`` (allocated pinned when not given);
    it is complete when the current stream is."""
    dev = fc1.weight.device
    if x_host.is_cuda:
        raise ValueError("convrot_mlp_gelu_host takes host tensors; use convrot_mlp_gelu for device tensors")
    if x_host.dtype != torch.bfloat16:
        raise ValueError("convrot_mlp_gelu_host takes bf16 tokens")
    if dev.type != "cuda":
        raise RuntimeError("convrot_mlp_gelu_host needs the bases on a CUDA device; there is no CPU fallback")
    lead = x_host.shape[:-1]
    x2 = x_host.reshape(-1, x_host.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    m = x2.shape[0]
    if x2.shape[1] != fc1.in_features or fc2.in_features != fc1.out_features:
        raise ValueError("convrot_mlp_gelu_host: feature sizes of the tokens and the two bases do not chain")
    if out_host is None:
        out_host = torch.empty(*lead, fc2.out_features, dtype=torch.bfloat16).pin_memory()
    if out_host.is_cuda or out_host.dtype != torch.bfloat16 or not out_host.is_contiguous() \
            or out_host.numel() != m * fc2.out_features:
        raise ValueError("out_host must be a contiguous bf16 host tensor of [tokens, out_features]")
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _side_streams:
        _side_streams[idx] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    s_in, s_out = _side_streams[idx]
    keep: list = []
    d1, d2 = _linear_desc(fc1, keep), _linear_desc(fc2, keep)
    int4 = d1.bits == 4 or d2.bits == 4
    sched = host_chunk_schedule(m, chunks, w4a8_out=fc2.out_features if int4 else None,
                                sms=torch.cuda.get_device_properties(dev).multi_processor_count)
    with torch.cuda.device(dev):
        ops.mlp_gelu_host(x2, d1, d2, out_host, sched, fc1.in_features, fc1.out_features, fc2.out_features, dev, s_in, s_out)
    return out_host


QUANTIZE_BASE_CHOICES = {"": None, "fp8": "fp8", "convrot_int8": 8, "convrot_int4": 4}


def apply_quantize_base(dit, flag: str) -> int:
    """Dispatch for the trainer flag ``optim.quantize_base`` (training_config.py:112,
    train_t2i_lora_cached.py:84-88) extended with the two ConvRot values."""
    if flag not in QUANTIZE_BASE_CHOICES:
        raise ValueError(f"unknown quantize_base {flag!r}; choose from {sorted(QUANTIZE_BASE_CHOICES)}")
    kind = QUANTIZE_BASE_CHOICES[flag]
    if kind is None:
        return 0
    if kind == "fp8":
        raise ValueError("quantize_base='fp8' is the reference's own Fp8Linear path (quantize.quantize_dit_fp8)")
    return quantize_dit_convrot(dit, bits=kind, backward_copy=True)     # the trainer's flag: trained through
