"""Multi-GPU side of the path: one process per GPU, ``torch.distributed`` (NCCL over NVLink on the
GPU box, gloo in CPU tests) for the plumbing.  The reference is single-GPU; both schemes are new.

* Data parallel (training, batch split): every rank holds the whole quantized base and its own
  samples.  The only exchange is ONE all-reduce of the flattened fp32 adapter gradients
  (:func:`allreduce_adapter_grads`).  Timesteps and noise are drawn for the global batch and sliced
  (:func:`shard_batch`), so the result does not depend on the number of ranks.
* Column-split tensor parallel (single-image inference): every quantized Linear under ``dit.blocks``
  keeps only its ``N / world`` output rows (codes, scales, bias) -- the rotation runs along K, so an
  N split never cuts a Hadamard block.  Each rank quantizes the (replicated) activations itself,
  runs its column slice of the GEMM and the slices are joined by one all-gather per Linear
  (:class:`ColumnParallelLinear`).  Integer accumulation is exact, so the gathered output equals
  the single-GPU output bit for bit.  Eight gathers per block and replicated attention: it scales
  poorly and is kept as the bit-exact scheme.
* Head-sharded tensor parallel (:func:`shard_dit_heads`, the default for inference): the column
  split follows the attention heads and the MLP hidden units, so attention, gating and SwiGLU run
  on the local slice with no exchange, and the closing projections (``wo``, ``mlp.down``) are split
  along K instead (:class:`RowParallelLinear`) at multiples of 128, so no Hadamard block or int4
  group is cut.  Each rank quantizes its own K slice of the activations (per-token scale of the
  slice), dequantizes its partial product and the partials are summed by ONE all-reduce per
  projection: two exchanges per block instead of eight, a third of the bytes, and every
  per-token operation between them divided by the number of ranks.  The sum of bf16 partials is
  not bit-identical with the single-GPU output; it stays within the path's float tolerance.
* Sequence-parallel residual stream on top of the head split (:func:`shard_dit_sequence`): between
  the blocks' projections every rank keeps only its T / world tokens, so the RMSNorms, the
  modulation, the residual updates and the activation quantisation K2 run on a slice.  The slices
  meet again as int8 codes + per-token scales (an all-gather of half the bytes of bf16 activations;
  the local Linears consume the codes directly), and the all-reduce after ``wo`` / ``mlp.down``
  becomes a reduce-scatter over tokens.  Per-token quantisation does not depend on which rank does
  it, so the results equal the head split's up to the order of the collective's additions.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from . import ops
from . import fused
from .fused import gate_residual
from .modules import GROUP, ConvRotLinear, convrot_linear_quantized, fused_prologue_ok, share_block_inputs


def world_info(group=None) -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


# ---------------------------------------------------------------------------------------------
# data parallel
# ---------------------------------------------------------------------------------------------
def shard_batch(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Contiguous slice of the leading (batch) axis owned by ``rank``; the batch must divide."""
    b = t.shape[0]
    if b % world:
        raise ValueError(f"global batch {b} does not divide over {world} ranks")
    per = b // world
    return t[rank * per:(rank + 1) * per]


def allreduce_adapter_grads(params, group=None, average: bool = True) -> int:
    """Sums (or averages) the gradients of ``params`` over the ranks with a single all-reduce of one
    flat fp32 bucket.  Parameters without a gradient contribute zeros.  Returns the bucket size in
    bytes (the bytes one rank puts on the wire per step)."""
    params = [p for p in params if p.requires_grad]
    if not params:
        return 0
    rank, world = world_info(group)
    dev = params[0].device
    sizes = [p.numel() for p in params]
    flat = torch.zeros(sum(sizes), dtype=torch.float32, device=dev)
    off = 0
    for p, n in zip(params, sizes):
        if p.grad is not None:
            flat[off:off + n].copy_(p.grad.reshape(-1))
        off += n
    if world > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat.div_(world)
    off = 0
    for p, n in zip(params, sizes):
        g = flat[off:off + n].view_as(p)
        if p.grad is None:
            p.grad = g.clone()
        else:
            p.grad.copy_(g)
        off += n
    if dev.type == "cuda":
        ops.step_check(dev)          # an expired device-side wait invalidates this step's gradients
    return flat.numel() * 4


class AdapterGradBuckets:
    """Data-parallel exchange of the adapter gradients that overlaps with the backward pass.

    The parameters are grouped in buckets (one per DiT block is the natural choice: the backward
    walks the blocks from the last to the first).  Each bucket owns one flat fp32 buffer and every
    parameter's ``.grad`` is a view into it, so autograd accumulates straight into the buffer and
    nothing is copied.  A post-accumulate hook counts the gradients of a bucket as they arrive; when
    the last one is in, the bucket's all-reduce is launched asynchronously while the backward of the
    earlier blocks is still running.  ``finish()`` waits for the reductions (launching those of
    buckets that stayed incomplete), optionally averages, and checks the device status block.

    Usage per step:  ``buckets.zero()``  ->  forward / backward  ->  ``buckets.finish()``  ->  optimizer.
    """

    def __init__(self, buckets, group=None, average: bool = False):
        self.group, self.average = group, average
        self.rank, self.world = world_info(group)
        self.buckets = []
        self._handles = []
        groups = [[p for p in params if p.requires_grad] for params in buckets]
        groups = [g for g in groups if g]
        total = sum(p.numel() for g in groups for p in g)
        dev = groups[0][0].device if groups else torch.device("cpu")
        # ONE flat gradient buffer; a bucket is a contiguous slice of it (what the fused optimizer
        # step and the gradient-norm kernel stream over), a parameter's .grad a view into its bucket
        self.flat = torch.zeros(total, dtype=torch.float32, device=dev)
        base = 0
        for params in groups:
            n = sum(p.numel() for p in params)
            flat = self.flat[base:base + n]
            b = {"params": params, "flat": flat, "pending": len(params), "launched": False, "offset": base}
            off = 0
            for p in params:
                if p.dtype != torch.float32:
                    raise TypeError("adapter parameters are fp32 (lora.py:39-40)")
                p.grad = flat[off:off + p.numel()].view_as(p)
                off += p.numel()
                p.register_post_accumulate_grad_hook(self._make_hook(b))
            self.buckets.append(b)
            base += n
        self.bytes_per_step = sum(b["flat"].numel() * 4 for b in self.buckets)

    def _launch(self, b):
        b["launched"] = True
        if self.world > 1:
            self._handles.append(dist.all_reduce(b["flat"], op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    def _make_hook(self, b):
        def hook(param):
            b["pending"] -= 1
            if b["pending"] == 0 and not b["launched"]:
                self._launch(b)
        return hook

    def zero(self) -> None:
        """Start of a step: gradients to zero (the views stay attached), arrival counters reset."""
        self.flat.zero_()
        for b in self.buckets:
            b["pending"], b["launched"] = len(b["params"]), False
            off = 0
            for p in b["params"]:          # an optimizer may have replaced .grad (set_to_none): re-attach
                if p.grad is None or p.grad.data_ptr() != b["flat"].data_ptr() + 4 * off:
                    p.grad = b["flat"][off:off + p.numel()].view_as(p)
                off += p.numel()
        self._handles = []

    def finish(self) -> int:
        """End of backward: every bucket reduced and visible to the current stream.  Returns the
        bytes one rank put on the wire."""
        for b in self.buckets:
            if not b["launched"]:
                self._launch(b)            # a parameter of this bucket got no gradient this step
        for h in self._handles:
            h.wait()
        self._handles = []
        if self.average and self.world > 1:
            self.flat.div_(self.world)
        dev = self.buckets[0]["flat"].device if self.buckets else None
        if dev is not None and dev.type == "cuda":
            ops.step_check(dev)
        return self.bytes_per_step


def block_buckets(adapters: dict) -> list:
    """Groups the adapter parameters of ``inject_lora``'s name -> module dict (lora.py:81-116) by the
    block they sit in (``blocks.7.attn.wq`` -> ``blocks.7``), keeping the dict's order."""
    groups: dict[str, list] = {}
    for name, mod in adapters.items():
        parts = name.split(".")
        cut = next((i for i, part in enumerate(parts) if part.isdigit()), None)
        key = ".".join(parts[:cut + 1]) if cut is not None else parts[0]
        groups.setdefault(key, []).extend([mod.lora_A, mod.lora_B])
    return list(groups.values())


# ---------------------------------------------------------------------------------------------
# column-split tensor parallel
# ---------------------------------------------------------------------------------------------
def column_slice(n: int, rank: int, world: int) -> slice:
    if n % (16 * world):
        raise ValueError(f"out_features={n} cannot be split in {world} column shards that are multiples of 16")
    per = n // world
    return slice(rank * per, (rank + 1) * per)


def shard_convrot_columns(mod: ConvRotLinear, rank: int, world: int, sl: slice | None = None) -> ConvRotLinear:
    """A ConvRotLinear holding only this rank's rows of the codes / scales / bias (or the rows ``sl``)."""
    sl = column_slice(mod.out_features, rank, world) if sl is None else sl
    scale = mod.scale[sl].contiguous().clone()
    bias = mod.bias.data[sl].contiguous().clone() if mod.bias is not None else None
    q8 = sb = None
    if mod.bits == 4 and mod.weight_q8 is not None:      # rows of the per-channel re-expression go with the shard
        q8 = mod.weight_q8.data[sl].contiguous().clone()
        sb = mod.backward_scale[sl].contiguous().clone()
    shard = ConvRotLinear.from_codes(mod.weight_q.data[sl].contiguous().clone(), scale, bias, mod.bits, q8, sb)
    shard.fast, shard.transient_backward = mod.fast, mod.transient_backward
    return shard


class ColumnParallelLinear(nn.Module):
    """Column shard of a quantized Linear followed by an all-gather of the output columns.

    ``local`` computes y[:, rank*N/G:(rank+1)*N/G]; the gather collects the G slices ([G, T, N/G],
    written by NCCL straight into local memory) and they are laid side by side into [T, N].
    """

    is_quant_linear = True

    def __init__(self, local: nn.Module, out_features: int, group=None):
        super().__init__()
        self.local = local
        self.group = group
        self.in_features, self.out_features = local.in_features, out_features
        self.gathered_bytes = 0      # bytes received from peers so far (for the benchmark report)

    @property
    def weight(self):
        return self.local.weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local(x)
        rank, world = world_info(self.group)
        if world == 1:
            return y
        lead = y.shape[:-1]
        y2 = y.reshape(-1, y.shape[-1]).contiguous()
        out = torch.empty(world * y2.shape[0], y2.shape[1], dtype=y2.dtype, device=y2.device)
        dist.all_gather_into_tensor(out, y2, group=self.group)       # rank r's slice lands in rows [r*T, (r+1)*T)
        self.gathered_bytes += (world - 1) * y2.numel() * y2.element_size()
        return out.view(world, *y2.shape).permute(1, 0, 2).reshape(*lead, self.out_features)


def _gather_columns(y: torch.Tensor, world: int, group, owner) -> torch.Tensor:
    """[..., C/G] column block of every rank -> [..., C] (rank r's block at columns [r C/G, (r+1) C/G))."""
    if world == 1:
        return y
    lead = y.shape[:-1]
    y2 = y.reshape(-1, y.shape[-1]).contiguous()
    out = torch.empty(world * y2.shape[0], y2.shape[1], dtype=y2.dtype, device=y2.device)
    dist.all_gather_into_tensor(out, y2, group=group)
    owner.gathered_bytes += (world - 1) * y2.numel() * y2.element_size()
    return out.view(world, *y2.shape).permute(1, 0, 2).reshape(*lead, world * y2.shape[1])


class ColumnLocalAttention(nn.Module):
    """``Attention`` of the DiT harness under the column split, without gathering what the next step
    consumes column by column: this rank's columns of wq / gate are its query heads, its columns of
    wk / wv the KV heads those use, so QK-norm, rotation, attention and the sigmoid gate run on the
    local columns and ONE all-gather joins the gated attention output before ``wo`` (itself a column
    shard followed by a gather).  Every value is computed exactly as on one GPU: outputs are
    bit-identical with the unsharded block."""

    def __init__(self, attn: nn.Module, rank: int, world: int, group=None):
        super().__init__()
        from . import dit as ditmod
        self._qk_norm_rope = ditmod.qk_norm_rope
        hd = attn.headdim
        q, kv, kvmap = head_partition(attn.heads, attn.kvheads, rank, world)
        qs = slice(q[0] * hd, (q[-1] + 1) * hd)
        ks = slice(kv[0] * hd, (kv[-1] + 1) * hd)
        self.group, self.world = group, world
        self.headdim, self.lheads, self.lkv = hd, len(q), len(kv)
        self.register_buffer("kvmap", torch.tensor(kvmap, dtype=torch.long), persistent=False)
        self.uniform = kvmap == [i * len(kv) // len(q) for i in range(len(q))] and len(q) % len(kv) == 0
        self.wq, self.gate = _take_columns(attn.wq, qs), _take_columns(attn.gate, qs)
        self.wk, self.wv = _take_columns(attn.wk, ks), _take_columns(attn.wv, ks)
        self.qknorm = attn.qknorm
        self.wo = ColumnParallelLinear(_take_columns(attn.wo, column_slice(attn.wo.out_features, rank, world)),
                                       attn.wo.out_features, group)
        self.gathered_bytes = 0

    def _finish(self, q, k, v, g, b, s, rope, mask):
        v = v.view(b, s, self.lkv, self.headdim).transpose(1, 2)
        q, k = self._qk_norm_rope(q, k, self.qknorm, rope, b, s, self.lheads, self.lkv, self.headdim)
        if self.uniform:
            o = nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=self.lheads != self.lkv)
        else:   # uneven sharing of the local KV heads: one K / V per query head
            kvmap = self.kvmap.to(k.device)
            o = nn.functional.scaled_dot_product_attention(q, k.index_select(1, kvmap), v.index_select(1, kvmap),
                                                           attn_mask=mask)
        o = o.transpose(1, 2).reshape(b, s, self.lheads * self.headdim)
        gated = fused.sigmoid_gate(o, g.reshape(b, s, -1))
        return self.wo(_gather_columns(gated, self.world, self.group, self))

    def forward(self, x, rope=None, mask=None):
        b, s, _ = x.shape
        return self._finish(self.wq(x), self.wk(x), self.wv(x), self.gate(x), b, s, rope, mask)

    @torch.no_grad()
    def forward_codes(self, xq, sx, lead, rope=None, mask=None):
        """The same from the rotated int8 codes of the input (inference, ConvRot bases)."""
        b, s = lead
        grp = getattr(self, "qkvg_group", None)
        if grp is not None:
            q, k, v, g = grp.forward_codes(xq, sx)
        else:
            q, k, v, g = (convrot_linear_quantized(xq, sx, m) for m in (self.wq, self.wk, self.wv, self.gate))
        return self._finish(q, k, v, g, b, s, rope, mask)


class ColumnLocalSwiGLU(nn.Module):
    """``SwiGLU`` under the column split: gate / up column shards, ``silu(g) * u`` on the local columns,
    one all-gather of the product, ``down`` as a column shard followed by a gather."""

    def __init__(self, mlp: nn.Module, rank: int, world: int, group=None):
        super().__init__()
        hs = column_slice(mlp.gate.out_features, rank, world)
        self.group, self.world = group, world
        self.gate, self.up = _take_columns(mlp.gate, hs), _take_columns(mlp.up, hs)
        self.down = ColumnParallelLinear(_take_columns(mlp.down, column_slice(mlp.down.out_features, rank, world)),
                                         mlp.down.out_features, group)
        self.gathered_bytes = 0

    def _finish(self, g, u):
        return self.down(_gather_columns(fused.swiglu(g, u), self.world, self.group, self))

    def forward(self, x):
        return self._finish(self.gate(x), self.up(x))

    @torch.no_grad()
    def forward_codes(self, xq, sx, lead):
        grp = getattr(self, "gu_group", None)
        if grp is not None:
            g, u = grp.forward_codes(xq, sx)
        else:
            g, u = convrot_linear_quantized(xq, sx, self.gate), convrot_linear_quantized(xq, sx, self.up)
        return self._finish(g.view(*lead, -1), u.view(*lead, -1))


class ColumnParallelBlock(nn.Module):
    """``SingleStreamBlock`` (mmdit.py:258-276) under the column split with local attention: the residual
    stream and both norms are replicated, every Linear is a column shard, and four all-gathers per block
    (gated attention output, ``wo`` output, SwiGLU product, ``down`` output) replace the eight of a
    Linear-by-Linear split.  Bit-identical with the unsharded block."""

    def __init__(self, block: nn.Module, rank: int, world: int, group=None):
        super().__init__()
        self.mod, self.prenorm, self.postnorm = block.mod, block.prenorm, block.postnorm
        self.attn = ColumnLocalAttention(block.attn, rank, world, group)
        self.mlp = ColumnLocalSwiGLU(block.mlp, rank, world, group)

    def forward(self, x, vec, rope, mask=None):
        prescale, preshift, pregate, postscale, postshift, postgate = self.mod(vec)
        a, m = self.attn, self.mlp
        if fused_prologue_ok(x, a.wq, a.wk, a.wv, a.gate, m.gate, m.up):
            lead = x.shape[:2]
            xq, sx = ops.norm_mod_quant(x, self.prenorm.scale.float(), prescale, preshift, self.prenorm.eps)
            x = gate_residual(x, pregate, a.forward_codes(xq, sx, lead, rope, mask))
            xq, sx = ops.norm_mod_quant(x, self.postnorm.scale.float(), postscale, postshift, self.postnorm.eps)
            return gate_residual(x, postgate, m.forward_codes(xq, sx, lead))
        x = gate_residual(x, pregate, a(fused.norm_modulate(x, self.prenorm, prescale, preshift), rope, mask))
        return gate_residual(x, postgate, m(fused.norm_modulate(x, self.postnorm, postscale, postshift)))


def _block_splits_by_heads(block, world: int) -> bool:
    attn, mlp = getattr(block, "attn", None), getattr(block, "mlp", None)
    need = ("wq", "wk", "wv", "gate", "wo", "qknorm", "heads", "kvheads", "headdim")
    if attn is None or mlp is None or not all(hasattr(attn, n) for n in need):
        return False
    if not all(hasattr(mlp, n) for n in ("gate", "up", "down")) or not all(hasattr(block, n) for n in ("mod", "prenorm", "postnorm")):
        return False
    return (attn.heads % world == 0 and attn.heads % attn.kvheads == 0 and mlp.gate.out_features % (16 * world) == 0
            and attn.wo.out_features % (16 * world) == 0 and mlp.down.out_features % (16 * world) == 0)


def shard_dit_columns(dit, rank: int | None = None, world: int | None = None, group=None,
                      local_attention: bool = True) -> int:
    """Column split of every Linear under ``dit.blocks`` with NCCL all-gathers; returns how many Linears
    were sharded.  Blocks with the harness's attention / SwiGLU layout become :class:`ColumnParallelBlock`
    (column shards that follow the attention heads, four gathers per block); anything else, or
    ``local_attention=False``, gets the Linear-by-Linear form (column shard + gather of every output).
    Both are bit-identical with one GPU.  Call after ``quantize_dit_convrot`` on every rank (same seeds)."""
    r, w = world_info(group)
    rank = r if rank is None else rank
    world = w if world is None else world
    n_block = 0
    if local_attention:
        for i, block in enumerate(dit.blocks):
            if _block_splits_by_heads(block, world):
                dit.blocks[i] = ColumnParallelBlock(block, rank, world, group)
                share_block_inputs(dit.blocks[i])      # Linears that read one tensor quantise it once
                n_block += 8
    targets = []
    for block in dit.blocks:
        if isinstance(block, ColumnParallelBlock):
            continue
        for mod in block.modules():
            for name, child in mod.named_children():
                if isinstance(child, ConvRotLinear):
                    targets.append((mod, name, child))
    for mod, name, child in targets:
        local = shard_convrot_columns(child, rank, world)
        setattr(mod, name, ColumnParallelLinear(local, child.out_features, group))
    return n_block + len(targets)


def tp_gather_bytes(dit) -> int:
    kinds = (ColumnParallelLinear, RowParallelLinear, SequenceParallelBlock, ColumnLocalAttention, ColumnLocalSwiGLU)
    return sum(m.gathered_bytes for m in dit.modules() if isinstance(m, kinds))


# ---------------------------------------------------------------------------------------------
# head-sharded tensor parallel (column split by heads / hidden units, K split of the closing projection)
# ---------------------------------------------------------------------------------------------
def row_slice(k: int, rank: int, world: int) -> slice:
    """This rank's range of the contraction axis; boundaries fall on multiples of 128."""
    if k % (GROUP * world):
        raise ValueError(f"in_features={k} cannot be split in {world} K shards that are multiples of {GROUP}")
    per = k // world
    return slice(rank * per, (rank + 1) * per)


def _take_columns(mod: nn.Module, sl: slice) -> nn.Module:
    """Output rows ``sl`` of a Linear-like module (ConvRotLinear or nn.Linear)."""
    if isinstance(mod, ConvRotLinear):
        return shard_convrot_columns(mod, 0, 1, sl)
    out = nn.Linear(mod.in_features, sl.stop - sl.start, bias=mod.bias is not None,
                    device=mod.weight.device, dtype=mod.weight.dtype)
    out.weight.data.copy_(mod.weight.data[sl])
    if mod.bias is not None:
        out.bias.data.copy_(mod.bias.data[sl])
    return out


def _take_k(mod: nn.Module, sl: slice, keep_bias: bool) -> nn.Module:
    """The K range ``sl`` of a Linear-like module: a partial product; the bias rides on one rank only."""
    if isinstance(mod, ConvRotLinear):
        if mod.bits == 8:
            codes = mod.weight_q.data[:, sl].contiguous().clone()
            scale = mod.scale.clone()                                       # per output channel: unchanged
        else:
            codes = mod.weight_q.data[:, sl.start // 2:sl.stop // 2].contiguous().clone()
            scale = mod.scale[:, sl.start // GROUP:sl.stop // GROUP].contiguous().clone()
        bias = mod.bias.data.clone() if (mod.bias is not None and keep_bias) else None
        return ConvRotLinear.from_codes(codes, scale, bias, mod.bits)
    out = nn.Linear(sl.stop - sl.start, mod.out_features, bias=mod.bias is not None and keep_bias,
                    device=mod.weight.device, dtype=mod.weight.dtype)
    out.weight.data.copy_(mod.weight.data[:, sl])
    if out.bias is not None:
        out.bias.data.copy_(mod.bias.data)
    return out


class RowParallelLinear(nn.Module):
    """K shard of a Linear: ``local`` multiplies this rank's slice of the input features with the
    matching slice of the weight; one all-reduce adds the partial products of all ranks."""

    is_quant_linear = True

    def __init__(self, local: nn.Module, in_features: int, group=None):
        super().__init__()
        self.local = local
        self.group = group
        self.in_features, self.out_features = in_features, local.out_features
        self.gathered_bytes = 0
        self.reduce = True           # False: return the partial product (the caller reduce-scatters it)

    @property
    def weight(self):
        return self.local.weight

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        return self.finish(self.local(x_shard))

    def finish(self, y: torch.Tensor) -> torch.Tensor:
        """The exchange step on a partial product that the caller has already computed."""
        rank, world = world_info(self.group)
        if world > 1 and self.reduce:
            y = y.contiguous()
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
            # ring all-reduce: every rank receives 2 (G-1)/G of the tensor
            self.gathered_bytes += 2 * (world - 1) * y.numel() * y.element_size() // world
        return y


def head_partition(heads: int, kvheads: int, rank: int, world: int):
    """Query heads of ``rank`` (a contiguous range), the KV heads those need, and for every local
    query head the index of its KV head among the local ones.  KV heads may be shared by two ranks
    when ``kvheads`` does not divide by ``world``; those ranks both project them."""
    if heads % world or heads % kvheads:
        raise ValueError(f"{heads} heads / {kvheads} KV heads cannot be split over {world} ranks")
    per = heads // world
    q = list(range(rank * per, (rank + 1) * per))
    group = heads // kvheads
    kv = sorted({h // group for h in q})
    if kv != list(range(kv[0], kv[-1] + 1)):
        raise AssertionError("KV heads of a contiguous query range are contiguous")
    return q, kv, [h // group - kv[0] for h in q]


class HeadParallelAttention(nn.Module):
    """``Attention`` of the DiT harness on this rank's heads: q / gate columns of the local query
    heads, k / v columns of the KV heads they use, attention and gating local, ``wo`` split along K."""

    def __init__(self, attn: nn.Module, rank: int, world: int, group=None):
        super().__init__()
        from . import dit as ditmod
        self._qk_norm_rope = ditmod.qk_norm_rope
        hd = attn.headdim
        q, kv, kvmap = head_partition(attn.heads, attn.kvheads, rank, world)
        qs = slice(q[0] * hd, (q[-1] + 1) * hd)
        ks = slice(kv[0] * hd, (kv[-1] + 1) * hd)
        if (qs.stop - qs.start) % GROUP:
            raise ValueError("the local head columns must be a multiple of 128 wide")
        self.headdim, self.lheads, self.lkv = hd, len(q), len(kv)
        self.register_buffer("kvmap", torch.tensor(kvmap, dtype=torch.long), persistent=False)
        self.uniform = kvmap == [i * len(kv) // len(q) for i in range(len(q))] and len(q) % len(kv) == 0
        self.wq, self.gate = _take_columns(attn.wq, qs), _take_columns(attn.gate, qs)
        self.wk, self.wv = _take_columns(attn.wk, ks), _take_columns(attn.wv, ks)
        self.qknorm = attn.qknorm
        self.wo = RowParallelLinear(_take_k(attn.wo, qs, keep_bias=rank == 0), attn.wo.in_features, group)

    def forward(self, x, rope=None, mask=None):
        if isinstance(x, TokenPayload):       # all tokens, as int8 codes or dense, gathered from the ranks
            b, s = x.batch, x.tokens
            grp = getattr(self, "qkvg_group", None)
            if grp is not None and x.xq is not None:
                q, k, v, g = grp.forward_codes(x.xq, x.sx)
            else:
                q, k, v, g = x.apply(self.wq), x.apply(self.wk), x.apply(self.wv), x.apply(self.gate)
        else:
            b, s, _ = x.shape
            q, k, v, g = self.wq(x), self.wk(x), self.wv(x), self.gate(x)
        v = v.view(b, s, self.lkv, self.headdim).transpose(1, 2)
        q, k = self._qk_norm_rope(q, k, self.qknorm, rope, b, s, self.lheads, self.lkv, self.headdim)
        if self.uniform:
            o = nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=self.lheads != self.lkv)
        else:   # uneven sharing of the local KV heads: one K / V per query head
            kvmap = self.kvmap.to(k.device)
            o = nn.functional.scaled_dot_product_attention(q, k.index_select(1, kvmap), v.index_select(1, kvmap),
                                                           attn_mask=mask)
        o = o.transpose(1, 2).reshape(b, s, self.lheads * self.headdim)
        if fused_prologue_ok(o, self.wo.local):      # sigmoid gate folded into the quantisation of wo's input
            oq, so = ops.gate_quant(o.reshape(b * s, -1), g.reshape(b * s, -1))
            return self.wo.finish(convrot_linear_quantized(oq, so, self.wo.local).view(b, s, -1))
        return self.wo(o * torch.sigmoid(g))


class HiddenParallelSwiGLU(nn.Module):
    """``SwiGLU`` on this rank's hidden units: gate / up column shards, ``down`` split along K."""

    def __init__(self, mlp: nn.Module, rank: int, world: int, group=None):
        super().__init__()
        hidden = mlp.gate.out_features
        hs = row_slice(hidden, rank, world)
        self.gate, self.up = _take_columns(mlp.gate, hs), _take_columns(mlp.up, hs)
        self.down = RowParallelLinear(_take_k(mlp.down, hs, keep_bias=rank == 0), hidden, group)

    def forward(self, x):
        grp = getattr(self, "gu_group", None)
        if grp is not None and isinstance(x, TokenPayload) and x.xq is not None:
            g, u = grp.forward_codes(x.xq, x.sx)
            g, u = g.view(x.batch, x.tokens, -1), u.view(x.batch, x.tokens, -1)
        else:
            g, u = (x.apply(self.gate), x.apply(self.up)) if isinstance(x, TokenPayload) else (self.gate(x), self.up(x))
        if fused_prologue_ok(g, self.down.local):    # silu(g) * u folded into the quantisation of down's input
            lead = g.shape[:-1]
            hq, hs = ops.swiglu_quant(g.reshape(-1, g.shape[-1]), u.reshape(-1, u.shape[-1]))
            return self.down.finish(convrot_linear_quantized(hq, hs, self.down.local).view(*lead, -1))
        return self.down(nn.functional.silu(g) * u)


def shard_dit_heads(dit, rank: int | None = None, world: int | None = None, group=None) -> int:
    """Replaces ``attn`` and ``mlp`` of every block under ``dit.blocks`` by their head-sharded /
    hidden-sharded versions; returns the number of Linears that were sharded.  Call after
    ``quantize_dit_convrot`` on every rank (same seeds)."""
    r, w = world_info(group)
    rank = r if rank is None else rank
    world = w if world is None else world
    n = 0
    for block in dit.blocks:
        block.attn = HeadParallelAttention(block.attn, rank, world, group)
        block.mlp = HiddenParallelSwiGLU(block.mlp, rank, world, group)
        n += 8
    return n


# ---------------------------------------------------------------------------------------------
# sequence-parallel residual stream (token shards between the projections)
# ---------------------------------------------------------------------------------------------
class TokenPayload:
    """Activations of ``batch`` x ``tokens`` tokens in the form the next Linears consume: rotated int8
    codes with per-token scales (for ConvRot Linears) or the dense tensor."""

    def __init__(self, batch: int, tokens: int, dense=None, xq=None, sx=None):
        self.batch, self.tokens, self.dense, self.xq, self.sx = batch, tokens, dense, xq, sx

    def apply(self, lin: nn.Module) -> torch.Tensor:
        if self.xq is not None:
            if not isinstance(lin, ConvRotLinear):
                raise TypeError("int8 codes can only feed a ConvRotLinear")
            return convrot_linear_quantized(self.xq, self.sx, lin).view(self.batch, self.tokens, -1)
        return lin(self.dense)


def _gather_tokens(t: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """[B, T/G, ...] on every rank -> [B, T, ...] (rank r's tokens at [r T/G, (r+1) T/G))."""
    if world == 1:
        return t
    t = t.contiguous()
    out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out.view(world * t.shape[0], *t.shape[1:]), t, group=group)
    if t.shape[0] == 1:
        return out.view(1, world * t.shape[1], *t.shape[2:])
    return out.transpose(0, 1).reshape(t.shape[0], world * t.shape[1], *t.shape[2:])


def _reduce_scatter_tokens(y: torch.Tensor, rank: int, world: int, group=None) -> torch.Tensor:
    """Sum of every rank's [B, T, F] partial, of which this rank keeps its T/G tokens: [B, T/G, F]."""
    if world == 1:
        return y
    b, t, f = y.shape
    tl = t // world
    if dist.get_backend(group) == "nccl":
        src = y.contiguous() if b == 1 else y.view(b, world, tl, f).transpose(0, 1).contiguous()
        out = torch.empty(b, tl, f, dtype=y.dtype, device=y.device)
        dist.reduce_scatter_tensor(out.view(b * tl, f), src.view(world * b * tl, f), group=group)
        return out
    y = y.contiguous()                        # backends without reduce-scatter (CPU tests)
    dist.all_reduce(y, group=group)
    return y[:, rank * tl:(rank + 1) * tl].contiguous()


class SequenceParallelBlock(nn.Module):
    """``SingleStreamBlock`` (mmdit.py:258-276) with head-sharded attention / hidden-sharded SwiGLU and
    a token-sharded residual stream.  The first block of the stack takes the full sequence and keeps its
    slice, the last one gathers the slices again; in between only slices are passed on."""

    def __init__(self, block: nn.Module, rank: int, world: int, group=None, first=False, last=False):
        super().__init__()
        self.rank, self.world, self.group, self.first, self.last = rank, world, group, first, last
        self.mod, self.prenorm, self.postnorm = block.mod, block.prenorm, block.postnorm
        self.attn = HeadParallelAttention(block.attn, rank, world, group)
        self.mlp = HiddenParallelSwiGLU(block.mlp, rank, world, group)
        self.attn.wo.reduce = False
        self.mlp.down.reduce = False
        self.codes_attn = all(isinstance(m, ConvRotLinear) for m in (self.attn.wq, self.attn.wk, self.attn.wv, self.attn.gate))
        self.codes_mlp = all(isinstance(m, ConvRotLinear) for m in (self.mlp.gate, self.mlp.up))
        self.gathered_bytes = 0

    def _all_tokens(self, n_local, as_codes: bool) -> TokenPayload:
        """``n_local``: this rank's normalised + modulated tokens, or a zero-argument callable that
        returns their codes directly (norm and modulation folded into the quantisation pass)."""
        w = self.world
        if callable(n_local):
            xq, sx, (b, tl, f) = n_local()
            xq = _gather_tokens(xq.view(b, tl, f), w, self.group)
            sx = _gather_tokens(sx.view(b, tl), w, self.group)
            self.gathered_bytes += (w - 1) * b * tl * (f + 4)
            return TokenPayload(b, tl * w, xq=xq.reshape(b * tl * w, f), sx=sx.reshape(b * tl * w))
        b, tl, f = n_local.shape
        if as_codes:
            xq, sx = ops.fwht_quant_act(n_local.reshape(b * tl, f))
            xq = _gather_tokens(xq.view(b, tl, f), w, self.group)
            sx = _gather_tokens(sx.view(b, tl), w, self.group)
            self.gathered_bytes += (w - 1) * b * tl * (f + 4)
            return TokenPayload(b, tl * w, xq=xq.reshape(b * tl * w, f), sx=sx.reshape(b * tl * w))
        self.gathered_bytes += (w - 1) * n_local.numel() * n_local.element_size()
        return TokenPayload(b, tl * w, dense=_gather_tokens(n_local, w, self.group))

    def _my_tokens(self, partial: torch.Tensor) -> torch.Tensor:
        self.gathered_bytes += (self.world - 1) * partial.numel() * partial.element_size() // self.world
        return _reduce_scatter_tokens(partial, self.rank, self.world, self.group)

    def forward(self, x, vec, rope, mask=None):
        if self.first:
            t = x.shape[1]
            if t % self.world:
                raise ValueError(f"{t} tokens do not divide over {self.world} ranks")
            tl = t // self.world
            x = x[:, self.rank * tl:(self.rank + 1) * tl]
        prescale, preshift, pregate, postscale, postshift, postgate = self.mod(vec)
        fused = not torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.bfloat16

        def codes_of(x_, norm, scale, shift):
            x_ = x_.contiguous()
            return lambda: (*ops.norm_mod_quant(x_, norm.scale.float(), scale, shift, norm.eps), tuple(x_.shape))

        n = codes_of(x, self.prenorm, prescale, preshift) if (fused and self.codes_attn) else \
            (1 + prescale) * self.prenorm(x) + preshift
        x = gate_residual(x.contiguous(), pregate, self._my_tokens(self.attn(self._all_tokens(n, self.codes_attn), rope, mask)))
        n = codes_of(x, self.postnorm, postscale, postshift) if (fused and self.codes_mlp) else \
            (1 + postscale) * self.postnorm(x) + postshift
        x = gate_residual(x, postgate, self._my_tokens(self.mlp(self._all_tokens(n, self.codes_mlp))))
        if self.last:
            self.gathered_bytes += (self.world - 1) * x.numel() * x.element_size()
            x = _gather_tokens(x, self.world, self.group)
        return x


def shard_dit_sequence(dit, rank: int | None = None, world: int | None = None, group=None) -> int:
    """Head / hidden-unit shards plus a token-sharded residual stream for every block under
    ``dit.blocks`` (inference; call after ``quantize_dit_convrot`` on every rank with the same seeds).
    Returns the number of Linears that were sharded."""
    r, w = world_info(group)
    rank = r if rank is None else rank
    world = w if world is None else world
    n = len(dit.blocks)
    for i in range(n):
        dit.blocks[i] = SequenceParallelBlock(dit.blocks[i], rank, world, group, first=i == 0, last=i == n - 1)
    return 8 * n


__all__ = ["world_info", "shard_batch", "allreduce_adapter_grads", "column_slice", "shard_convrot_columns",
           "ColumnParallelLinear", "shard_dit_columns", "tp_gather_bytes", "row_slice", "RowParallelLinear",
           "head_partition", "HeadParallelAttention", "HiddenParallelSwiGLU", "shard_dit_heads", "TokenPayload",
           "SequenceParallelBlock", "shard_dit_sequence", "GROUP"]
