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
  the single-GPU output bit for bit.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .modules import GROUP, ConvRotLinear


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
    return flat.numel() * 4


# ---------------------------------------------------------------------------------------------
# column-split tensor parallel
# ---------------------------------------------------------------------------------------------
def column_slice(n: int, rank: int, world: int) -> slice:
    if n % (16 * world):
        raise ValueError(f"out_features={n} cannot be split in {world} column shards that are multiples of 16")
    per = n // world
    return slice(rank * per, (rank + 1) * per)


def shard_convrot_columns(mod: ConvRotLinear, rank: int, world: int) -> ConvRotLinear:
    """A ConvRotLinear holding only this rank's rows of the codes / scales / bias."""
    sl = column_slice(mod.out_features, rank, world)
    scale = mod.scale[sl].contiguous().clone()
    bias = mod.bias.data[sl].contiguous().clone() if mod.bias is not None else None
    # the 4-bit backward copy is rebuilt from the shard's own codes on demand (its scale is per shard)
    qt = mod.weight_qt.data[:, sl].contiguous().clone() if (mod.weight_qt is not None and mod.bits == 8) else None
    return ConvRotLinear.from_codes(mod.weight_q.data[sl].contiguous().clone(), scale, bias, mod.bits, qt)


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


def shard_dit_columns(dit, rank: int | None = None, world: int | None = None, group=None) -> int:
    """Replaces every ConvRotLinear under ``dit.blocks`` by its column shard + all-gather; returns
    how many were replaced.  Call after ``quantize_dit_convrot`` on every rank (same seeds)."""
    r, w = world_info(group)
    rank = r if rank is None else rank
    world = w if world is None else world
    targets = []
    for block in dit.blocks:
        for mod in block.modules():
            for name, child in mod.named_children():
                if isinstance(child, ConvRotLinear):
                    targets.append((mod, name, child))
    for mod, name, child in targets:
        local = shard_convrot_columns(child, rank, world)
        setattr(mod, name, ColumnParallelLinear(local, child.out_features, group))
    return len(targets)


def tp_gather_bytes(dit) -> int:
    return sum(m.gathered_bytes for m in dit.modules() if isinstance(m, ColumnParallelLinear))


__all__ = ["world_info", "shard_batch", "allreduce_adapter_grads", "column_slice", "shard_convrot_columns",
           "ColumnParallelLinear", "shard_dit_columns", "tp_gather_bytes", "GROUP"]
