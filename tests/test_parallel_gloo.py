"""Host-side logic of the multi-GPU schemes, run as two gloo ranks on the CPU: the data-parallel
gradient bucket and the column-split / all-gather plumbing (the GEMM itself is GPU-only, so a plain
Linear slice stands in for the local shard here)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

from oracle import convrot_ref as R


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def _run(fn, world=2):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port_holder[0], fn, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    return [ret[r] for r in range(world)]


port_holder = [0]


@pytest.fixture(autouse=True)
def _port():
    port_holder[0] = _free_port()


def _dp_job(rank, world):
    from k2q import parallel
    torch.manual_seed(0)
    a = nn.Parameter(torch.zeros(4, 8))
    b = nn.Parameter(torch.zeros(6, 4))
    c = nn.Parameter(torch.zeros(3))                     # never receives a gradient on rank 1
    x = torch.arange(16, dtype=torch.float32).reshape(4, 4)   # "global batch" of 4 samples
    xs = parallel.shard_batch(x, rank, world)
    a.grad = xs.sum() * torch.ones_like(a)
    b.grad = (rank + 1.0) * torch.ones_like(b)
    if rank == 0:
        c.grad = torch.ones_like(c)
    nbytes = parallel.allreduce_adapter_grads([a, b, c], average=True)
    return dict(a=a.grad.clone(), b=b.grad.clone(), c=c.grad.clone(), nbytes=nbytes, rows=xs.shape[0])


def test_data_parallel_gradient_bucket():
    out = _run(_dp_job)
    total = float(torch.arange(16, dtype=torch.float32).sum())
    for r in out:
        assert r["rows"] == 2 and r["nbytes"] == (32 + 24 + 3) * 4
        assert torch.equal(r["a"], torch.full((4, 8), total / 2))     # mean over ranks of per-rank sums
        assert torch.equal(r["b"], torch.full((6, 4), 1.5))
        assert torch.equal(r["c"], torch.full((3,), 0.5))
    assert torch.equal(out[0]["a"], out[1]["a"])


def _bucket_job(rank, world):
    """Two 'blocks' of adapters trained through autograd: bucketed, overlapped reduction vs the
    single flat all-reduce; a parameter that receives no gradient must not stall its bucket."""
    from k2q import parallel
    torch.manual_seed(0)
    blocks = [[nn.Parameter(torch.randn(4, 8)), nn.Parameter(torch.randn(6, 4))],
              [nn.Parameter(torch.randn(5, 8)), nn.Parameter(torch.randn(3))]]     # the last one stays unused
    adapters = {"blocks.0.attn.wq": type("A", (), {"lora_A": blocks[0][0], "lora_B": blocks[0][1]})(),
                "blocks.1.mlp.up": type("A", (), {"lora_A": blocks[1][0], "lora_B": blocks[1][1]})()}
    grouped = parallel.block_buckets(adapters)
    assert [len(g) for g in grouped] == [2, 2] and grouped[0][0] is blocks[0][0]
    buckets = parallel.AdapterGradBuckets(grouped, average=True)
    x = torch.arange(8, dtype=torch.float32) + rank
    out = []
    for step in range(2):                                  # second step: counters and views are re-armed
        buckets.zero()
        loss = (blocks[0][0] @ x).sum() * (rank + 1) + (x[:4] @ blocks[0][1].t()).sum() + (blocks[1][0] @ x).pow(2).sum()
        loss.backward()
        nbytes = buckets.finish()
        out.append([p.grad.clone() for b in blocks for p in b])
    # the same gradients through the single-bucket call
    flat_params = [p for b in blocks for p in b]
    for p in flat_params:
        p.grad = None
    loss = (blocks[0][0] @ x).sum() * (rank + 1) + (x[:4] @ blocks[0][1].t()).sum() + (blocks[1][0] @ x).pow(2).sum()
    loss.backward()
    parallel.allreduce_adapter_grads(flat_params, average=True)
    ref = [p.grad.clone() for p in flat_params]
    return dict(out=out, ref=ref, nbytes=nbytes)


def test_bucketed_gradient_exchange_matches_flat_all_reduce():
    res = _run(_bucket_job)
    for r in res:
        assert r["nbytes"] == (32 + 24 + 40 + 3) * 4
        for step in range(2):
            for got, want in zip(r["out"][step], r["ref"]):
                assert torch.allclose(got, want, rtol=1e-6, atol=1e-6)
        assert float(r["out"][0][3].abs().max()) == 0.0          # the unused parameter: zeros, not a hang
    for a, b in zip(res[0]["out"][1], res[1]["out"][1]):
        assert torch.equal(a, b)


class _Slice(nn.Module):
    """Stand-in for the local GEMM shard: rows [lo, hi) of a dense Linear."""

    def __init__(self, w, lo, hi):
        super().__init__()
        self.w = w[lo:hi]
        self.in_features, self.out_features = w.shape[1], hi - lo
        self.weight = self.w

    def forward(self, x):
        return x @ self.w.t()


def _tp_job(rank, world):
    from k2q import parallel
    g = torch.Generator().manual_seed(3)
    w = torch.randn(64, 32, generator=g)
    x = torch.randn(2, 5, 32, generator=g)
    sl = parallel.column_slice(64, rank, world)
    layer = parallel.ColumnParallelLinear(_Slice(w, sl.start, sl.stop), 64)
    y = layer(x)
    # sharding of real codes: rows of codes / scales / bias / transposed copy
    from k2q import modules
    wq, sw = R.quantize_weight_int8(R.synth_weight(64, 256))
    full = modules.ConvRotLinear.from_codes(wq, sw, torch.arange(64.0), 8)
    shard = parallel.shard_convrot_columns(full, rank, world)
    q4, s4 = R.quantize_weight_int4(R.synth_weight(64, 256))
    shard4 = parallel.shard_convrot_columns(modules.ConvRotLinear.from_codes(q4, s4, None, 4), rank, world)
    return dict(y=y, ref=x @ w.t(), bytes=layer.gathered_bytes, q=shard.weight_q.data, s=shard.scale, b=shard.bias.data,
                q4=shard4.weight_q.data, s4=shard4.scale, wq=wq, sw=sw, q4f=q4, s4f=s4,
                shape=(shard.out_features, shard.in_features))


def test_column_split_all_gather_and_sharding():
    out = _run(_tp_job)
    for rank, r in enumerate(out):
        assert torch.equal(r["y"], r["ref"])                          # gathered columns in the right order
        assert r["bytes"] == 10 * 32 * 4 and r["shape"] == (32, 256)
        lo, hi = rank * 32, (rank + 1) * 32
        assert torch.equal(r["q"], r["wq"][lo:hi]) and torch.equal(r["s"], r["sw"][lo:hi])
        assert torch.equal(r["b"], torch.arange(64.0)[lo:hi])
        assert torch.equal(r["q4"], r["q4f"][lo:hi]) and torch.equal(r["s4"].view(torch.int16), r["s4f"][lo:hi].view(torch.int16))


def _head_tp_job(rank, world):
    from k2q import dit as ditmod
    from k2q import modules, parallel
    out = {}
    for heads, kvheads in ((6, 3), (4, 2)):          # (6, 3) over two ranks shares KV head 1 between them
        torch.manual_seed(11)
        dim = heads * 128
        attn = ditmod.Attention(dim, heads, kvheads, bias=True)
        mlp = ditmod.SwiGLU(dim, 3, bias=True)
        for prm in list(attn.parameters()) + list(mlp.parameters()):
            prm.data.normal_(0.0, 0.05)
        x = torch.randn(2, 7, dim)
        pos = torch.arange(7)[None, :, None].expand(2, 7, 3)
        rope = ditmod.rope_tables(pos, [128 - 12 * 8, 48, 48], 1e4)
        tp_a = parallel.HeadParallelAttention(attn, rank, world)
        tp_m = parallel.HiddenParallelSwiGLU(mlp, rank, world)
        with torch.no_grad():
            out[(heads, kvheads)] = dict(a=tp_a(x, rope), ra=attn(x, rope), m=tp_m(x), rm=mlp(x), uniform=tp_a.uniform,
                                         bytes=tp_a.wo.gathered_bytes)
    # K shards of real codes: int8 keeps the per-channel scale, int4 takes the groups of the range
    wq, sw = R.quantize_weight_int8(R.synth_weight(64, 512))
    k8 = parallel._take_k(modules.ConvRotLinear.from_codes(wq, sw, torch.arange(64.0), 8), parallel.row_slice(512, rank, world),
                          keep_bias=rank == 0)
    q4, s4 = R.quantize_weight_int4(R.synth_weight(64, 512))
    k4 = parallel._take_k(modules.ConvRotLinear.from_codes(q4, s4, None, 4), parallel.row_slice(512, rank, world), False)
    out["codes"] = dict(q8=k8.weight_q.data, s8=k8.scale, b8=None if k8.bias is None else k8.bias.data, wq=wq, sw=sw,
                        q4=k4.weight_q.data, s4=k4.scale, q4f=q4, s4f=s4, shape=(k8.out_features, k8.in_features))
    return out


def test_head_sharded_attention_and_swiglu_match_the_unsharded_modules():
    world = 2
    res = _run(_head_tp_job, world)
    for rank, r in enumerate(res):
        for key in ((6, 3), (4, 2)):
            d = r[key]
            assert (d["a"] - d["ra"]).abs().max() <= 2e-5 * d["ra"].abs().max()
            assert (d["m"] - d["rm"]).abs().max() <= 2e-5 * d["rm"].abs().max()
            assert d["bytes"] == d["a"].numel() * 4         # 2 (G-1)/G of the tensor at G = 2
        assert res[rank][(6, 3)]["uniform"] is False and res[rank][(4, 2)]["uniform"] is True
        c = r["codes"]
        lo, hi = rank * 256, (rank + 1) * 256
        assert c["shape"] == (64, 256)
        assert torch.equal(c["q8"], c["wq"][:, lo:hi]) and torch.equal(c["s8"], c["sw"])
        assert (c["b8"] is not None) == (rank == 0)
        assert torch.equal(c["q4"], c["q4f"][:, lo // 2:hi // 2]) and torch.equal(c["s4"], c["s4f"][:, lo // 128:hi // 128])


def _sp_job(rank, world):
    from k2q import dit as ditmod
    from k2q import parallel
    torch.manual_seed(21)
    dim, heads, kvheads, tokens = 512, 4, 2, 8
    blocks = [ditmod.SingleStreamBlock(dim, heads, 3, bias=True, kvheads=kvheads) for _ in range(3)]
    for blk in blocks:
        for prm in blk.parameters():
            prm.data.normal_(0.0, 0.05)
    x = torch.randn(2, tokens, dim)
    vec = torch.randn(2, 1, 6 * dim) * 0.1
    pos = torch.arange(tokens)[None, :, None].expand(2, tokens, 3)
    rope = ditmod.rope_tables(pos, [128 - 12 * 8, 48, 48], 1e4)
    with torch.no_grad():
        ref = x
        for blk in blocks:
            ref = blk(ref, vec, rope)
        sp = [parallel.SequenceParallelBlock(blk, rank, world, first=i == 0, last=i == len(blocks) - 1)
              for i, blk in enumerate(blocks)]
        y = x
        shapes = []
        for blk in sp:
            y = blk(y, vec, rope)
            shapes.append(tuple(y.shape))
    return dict(y=y, ref=ref, shapes=shapes, bytes=sum(b.gathered_bytes for b in sp))


def test_sequence_parallel_blocks_match_the_plain_stack():
    world = 2
    res = _run(_sp_job, world)
    for r in res:
        assert r["shapes"] == [(2, 4, 512), (2, 4, 512), (2, 8, 512)]      # token slices between blocks, full at the end
        assert (r["y"] - r["ref"]).abs().max() <= 2e-5 * r["ref"].abs().max()
        assert r["bytes"] > 0
    assert torch.equal(res[0]["y"], res[1]["y"])


def test_head_partition_covers_every_head_once():
    from k2q import parallel
    for heads, kvheads, world in ((48, 12, 8), (48, 12, 4), (48, 12, 2), (6, 3, 2), (8, 8, 4)):
        seen = []
        for rank in range(world):
            q, kv, kvmap = parallel.head_partition(heads, kvheads, rank, world)
            seen += q
            assert [kv[i] for i in kvmap] == [h // (heads // kvheads) for h in q]
        assert seen == list(range(heads))
    with pytest.raises(ValueError):
        parallel.head_partition(48, 12, 0, 5)
    with pytest.raises(ValueError):
        parallel.row_slice(16384, 0, 3)


def test_column_slice_rejects_ragged_splits():
    from k2q import parallel
    assert parallel.column_slice(1536, 7, 8) == slice(1344, 1536)
    with pytest.raises(ValueError):
        parallel.column_slice(1536, 0, 5)
    with pytest.raises(ValueError):
        parallel.shard_batch(torch.zeros(8, 2), 0, 3)


def _column_block_job(rank, world):
    from k2q import dit as ditmod
    from k2q import parallel
    out = {}
    for heads, kvheads in ((4, 2), (6, 3)):           # (6, 3) over two ranks: KV head 1 is used by both
        torch.manual_seed(31)
        dim, tokens = heads * 128, 9
        holder = nn.Module()
        holder.blocks = nn.ModuleList([ditmod.SingleStreamBlock(dim, heads, 3, bias=True, kvheads=kvheads) for _ in range(2)])
        for prm in holder.parameters():
            prm.data.normal_(0.0, 0.05)
        x = torch.randn(2, tokens, dim)
        vec = torch.randn(2, 1, 6 * dim) * 0.1
        pos = torch.arange(tokens)[None, :, None].expand(2, tokens, 3)
        rope = ditmod.rope_tables(pos, [128 - 12 * 8, 48, 48], 1e4)
        with torch.no_grad():
            ref = x
            for blk in holder.blocks:
                ref = blk(ref, vec, rope)
            n = parallel.shard_dit_columns(holder, rank, world)
            y = x
            for blk in holder.blocks:
                y = blk(y, vec, rope)
        out[(heads, kvheads)] = dict(y=y, ref=ref, n=n, kinds=[type(b).__name__ for b in holder.blocks],
                                     bytes=parallel.tp_gather_bytes(holder), tokens=2 * tokens, dim=dim,
                                     hidden=holder.blocks[0].mlp.gate.out_features * world)
    return out


def test_column_split_with_local_attention_matches_the_unsharded_blocks():
    """Column shards that follow the heads (q / gate by query head, k / v by the KV heads those use, SwiGLU by
    hidden unit), four all-gathers per block; the same numbers as the unsharded blocks (dense fp32 Linears
    stand in for the GEMM shards here, so equality holds up to the BLAS's summation order)."""
    res = _run(_column_block_job, 2)
    for r in res:
        for key, d in r.items():
            assert d["n"] == 16 and d["kinds"] == ["ColumnParallelBlock"] * 2
            assert (d["y"] - d["ref"]).abs().max() <= 2e-5 * d["ref"].abs().max(), key
            # per block: gated attention output, wo output, down output [T, dim] and the SwiGLU product [T, hidden],
            # of which (G-1)/G arrives from the peer: fp32 here
            per_block = d["tokens"] * (3 * d["dim"] + d["hidden"]) * 4 // 2
            assert d["bytes"] == 2 * per_block
    assert torch.equal(res[0][(4, 2)]["y"], res[1][(4, 2)]["y"])            # replicated residual stream
