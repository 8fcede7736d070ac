"""Guard bands around every buffer the library writes (the sanitizer substitute for a pool where
compute-sanitizer is closed): while these tests run, each ``torch.empty`` the op wrappers issue is
served from a larger allocation whose first and last 256 bytes hold a pattern; after the op the
bands must be untouched.  Shapes are ragged on purpose (rows that do not fill a tile, a single row,
column counts that are odd multiples of 16) and every op family is driven once, with and without
the adapter epilogue.  A write before or past an output -- a wrong tile origin, a tail that is not
masked, a workspace sized for the wrong operand -- lands in a band."""
import pytest
import torch

from oracle import convrot_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda"
GUARD = 256
PATTERN = 0xA5


class _GuardedTorch:
    """Stands in for the ``torch`` module inside ``k2q.ops``: everything is forwarded, except that
    ``empty`` returns a contiguous view into the middle of a guarded allocation."""

    def __init__(self):
        self.buffers = []

    def __getattr__(self, name):
        return getattr(torch, name)

    def empty(self, *shape, dtype=torch.float32, device=None, **kw):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            shape = tuple(shape[0])
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        padded = (nbytes + 15) // 16 * 16
        raw = torch.full((padded + 2 * GUARD,), PATTERN, dtype=torch.uint8, device=device)
        self.buffers.append((raw, nbytes))
        return raw[GUARD:GUARD + nbytes].view(dtype).view(*shape)

    def check(self):
        torch.cuda.synchronize()
        for i, (raw, nbytes) in enumerate(self.buffers):
            front, back = raw[:GUARD], raw[GUARD + nbytes:]
            assert int((front != PATTERN).sum()) == 0, f"buffer {i} ({nbytes} bytes): write in front of it"
            assert int((back != PATTERN).sum()) == 0, f"buffer {i} ({nbytes} bytes): write past its end"
        n = len(self.buffers)
        self.buffers.clear()
        return n


@pytest.fixture()
def guarded(monkeypatch):
    from k2q import ops
    g = _GuardedTorch()
    monkeypatch.setattr(ops, "torch", g)
    yield g
    g.check()


SHAPES = [(193, 144, 384), (1, 16, 128), (300, 272, 1024), (130, 400, 256)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_row_kernels_stay_inside_their_outputs(guarded, m, n, k):
    from k2q import ops
    w = R.synth_weight(n, k, seed=900).to(DEV)
    x = R.synth_act(m, k, seed=901).to(DEV)
    q8, s8 = ops.quant_weight_i8(w)
    q4, s4 = ops.quant_weight_i4(w)
    ops.requant_i4_to_i8(q4, s4)
    ops.fwht_quant_act(x)
    ops.fwht_quant_act(x.float())
    ops.swiglu_quant(x, x.flip(0))
    ops.gate_quant(x, x.flip(0))
    ops.norm_mod_quant(x.reshape(1, m, k), torch.zeros(k, device=DEV), x[:1].reshape(1, 1, k), x[:1].reshape(1, 1, k))
    ops.quant_rows(x, torch.rand(k, device=DEV) + 0.5)
    ops.fwht_rows(x)
    ops.fwht_rows(x, out_dtype=torch.float32)
    ops.transpose_i8(q8)
    assert guarded.check() >= 18
    ops.check_status()


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("rank", [0, 8, 32])
def test_gemms_and_adapter_kernels_stay_inside_their_outputs(guarded, m, n, k, rank):
    from k2q import ops
    w = R.synth_weight(n, k, seed=910).to(DEV)
    x = R.synth_act(m, k, seed=911).to(DEV)
    bias = R.synth_vec(n, 0.01, 912).to(DEV)
    q8, s8 = ops.quant_weight_i8(w)
    q4, s4 = ops.quant_weight_i4(w)
    xq, sx = ops.fwht_quant_act(x)
    u = bm = None
    if rank:
        a = R.synth_mat(rank, k, 0.01, 913).to(DEV)
        b = R.synth_mat(n, rank, 0.01, 914).to(DEV)
        u = ops.lora_down(x, a)
        bm = b
    ops.gemm_w8a8(xq, sx, q8, s8, bias, u=u, bm=bm, lora_scale=1.0 if rank else 0.0)
    ops.gemm_w8a8(xq, sx, q8, s8, None, act="gelu_tanh")
    ops.gemm_w4a8(xq, sx, q4, s4, bias, u=u, bm=bm, lora_scale=1.0 if rank else 0.0)
    ops.gemm_w4a8(xq, sx, q4, s4, None, act="gelu_tanh")
    # the backward contracts over the output channels: N must be a multiple of 128 there
    n2 = (n + 127) // 128 * 128
    w2 = R.synth_weight(n2, k, seed=915).to(DEV)
    q2, s2 = ops.quant_weight_i8(w2)
    gy = R.synth_mat(m, n2, 1e-2, 916).to(torch.bfloat16).to(DEV)
    gq, sg = ops.quant_rows(gy, s2)
    du = hb = None
    if rank:
        b2 = R.synth_mat(n2, rank, 0.01, 917).to(DEV)
        du = ops.lora_down(gy, b2, scale=0.5, transposed=True)
        hb = ops.fwht_rows(a).t().contiguous()
        ops.lora_tn(du, x)
        ops.lora_tn(u, gy, scale=0.5)
    ops.gemm_dx_w8(gq, sg, q2, u=du, bm=hb, lora_scale=1.0 if rank else 0.0)
    assert guarded.check() >= 10
    ops.check_status()
