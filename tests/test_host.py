"""CPU tests of the host side: the C-ABI library loads and exports what include/k2q.h declares,
the module boundary keeps the reference's protocol, and nothing computes on the CPU."""
import re
from pathlib import Path

import pytest
import torch
import torch.nn as nn

from oracle import convrot_ref as R

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    ge.build()
    from k2q import _lib
    return _lib


def test_library_exports_every_declared_symbol(lib):
    header = (ROOT / "include" / "k2q.h").read_text()
    declared = set(re.findall(r"\b(k2q_[a-z0-9_]+)\s*\(", header))
    declared.discard("k2q_epilogue")
    assert declared == set(lib.SIGNATURES), declared ^ set(lib.SIGNATURES)
    handle = lib.load()
    for name in declared:
        assert hasattr(handle, name), name
    assert handle.k2q_version() == int(re.search(r"#define K2Q_VERSION (\d+)", header).group(1))
    assert handle.k2q_status_bytes() == 16
    assert handle.k2q_lora_tn_workspace_bytes(4096, 32, 3072) > 0


def test_epilogue_struct_layout_matches_header(lib):
    import ctypes as C
    assert C.sizeof(lib.Epilogue) == 64
    assert lib.Epilogue.ldu.offset == 32 and lib.Epilogue.rank.offset == 48 and lib.Epilogue.act.offset == 56


def test_linear_struct_layout_and_host_schedule(lib):
    import ctypes as C
    from k2q import modules
    assert C.sizeof(lib.Linear) == 48 and lib.Linear.codes.offset == 8 and lib.Linear.N.offset == 32
    assert lib.load().k2q_mlp_gelu_host_workspace_bytes(8192, 3072, 12288, 3072, 1152) >= 2 * 8192 * 3072 * 2
    for m in (0, 1, 191, 768, 769, 3647, 3648, 8192, 16896, 100003):
        for chunks in (None, 1, 3, 16):
            sched = modules.host_chunk_schedule(m, chunks)
            assert sum(sched) == m and all(r > 0 for r in sched), (m, chunks, sched)
    assert modules.host_chunk_schedule(8192) == [192, 384, 768, 1152, 1152, 1152, 1152, 1088, 768, 384]
    assert modules.host_chunk_schedule(8192, w4a8_out=3072) == [768] + [1152] * 6 + [512]
    assert modules.host_chunk_schedule(8192, w4a8_out=6144) == [768] + [1152] * 6 + [512]
    for m in (1, 700, 1345, 2000, 4099, 8200, 16896):
        for n2 in (1024, 3072, 6144, 32768):
            sched = modules.host_chunk_schedule(m, w4a8_out=n2)
            assert sum(sched) == m and min(sched) >= min(m, 192), (m, n2, sched)
    with pytest.raises(ValueError):
        modules.convrot_mlp_gelu_host(torch.zeros(4, 128), _codes_module(32, 128, 8), _codes_module(128, 32, 8))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        modules.convrot_mlp_gelu_host(torch.zeros(4, 128, dtype=torch.bfloat16), _codes_module(256, 128, 8),
                                      _codes_module(128, 256, 8))


def test_no_cpu_fallback(lib):
    from k2q import modules, ops
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.fwht_quant_act(torch.zeros(4, 128, dtype=torch.bfloat16))
    q, s = R.quantize_weight_int8(R.synth_weight(32, 128))
    mod = modules.ConvRotLinear.from_codes(q, s, None, 8)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        mod(torch.zeros(2, 128, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        modules.ConvRotLinear(nn.Linear(128, 32), bits=8)          # quantising needs the device


def _codes_module(n, k, bits, bias=False):
    from k2q import modules
    w = R.synth_weight(n, k)
    q, s = (R.quantize_weight_int8 if bits == 8 else R.quantize_weight_int4)(w)
    b = torch.zeros(n) if bias else None
    return modules.ConvRotLinear.from_codes(q, s, b, bits)


def test_module_protocol_matches_fp8linear(lib):
    """quantize.py:31-51 / lora.py:38-40: flag, sizes, weight probe, frozen Parameters; and an fp32
    scale that survives module.to(dtype=bf16)."""
    for bits in (8, 4):
        mod = _codes_module(48, 256, bits, bias=True)
        assert mod.is_quant_linear and (mod.in_features, mod.out_features) == (256, 48)
        assert mod.weight is mod.weight_q and mod.weight.device.type == "cpu"
        params = dict(mod.named_parameters())
        assert set(params) == {"weight_q", "scale_bits", "bias"}
        assert not any(p.requires_grad for p in params.values())
        s_before = mod.scale.clone()
        mod.to(dtype=torch.bfloat16)
        assert mod.scale.dtype == (torch.float32 if bits == 8 else torch.bfloat16)
        assert torch.equal(mod.scale, s_before)
        assert mod.weight_q.dtype == (torch.int8 if bits == 8 else torch.uint8)
    with pytest.raises(ValueError):
        from k2q import modules
        modules.ConvRotLinear.from_codes(torch.zeros(4, 128, dtype=torch.int8), torch.zeros(4, dtype=torch.bfloat16),
                                         None, 8)


class _TinyAttn(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.wq, self.wk, self.wv = nn.Linear(d, d, bias=False), nn.Linear(d, d // 2, bias=False), nn.Linear(d, d // 2, bias=False)
        self.gate, self.wo = nn.Linear(d, d, bias=False), nn.Linear(d, d, bias=False)
        self.norm = nn.LayerNorm(d)


class _TinyMlp(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.gate, self.up, self.down = nn.Linear(d, 2 * d, bias=False), nn.Linear(d, 2 * d, bias=False), nn.Linear(2 * d, d, bias=False)


class _TinyBlock(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.attn, self.mlp = _TinyAttn(d), _TinyMlp(d)


class _TinyDit(nn.Module):
    def __init__(self, d=128, layers=2):
        super().__init__()
        self.first = nn.Linear(64, d)
        self.blocks = nn.ModuleList([_TinyBlock(d) for _ in range(layers)])
        self.txtfusion = nn.Module()
        self.txtfusion.layerwise_blocks = nn.ModuleList([_TinyBlock(d)])
        self.txtfusion.refiner_blocks = nn.ModuleList([_TinyBlock(d)])
        self.txtmlp = nn.Sequential(nn.LayerNorm(d), nn.Linear(d, d), nn.GELU(approximate="tanh"), nn.Linear(d, d))
        self.last = nn.Linear(d, 64)


def _oracle_quantizers(monkeypatch):
    """Stand-ins for the device quantisers so the traversal logic can run without a GPU."""
    from k2q import ops
    monkeypatch.setattr(ops, "quant_weight_i8", lambda w: R.quantize_weight_int8(w))
    monkeypatch.setattr(ops, "quant_weight_i4", lambda w: R.quantize_weight_int4(w))
    monkeypatch.setattr(ops, "transpose_i8", lambda q: q.t().contiguous())
    monkeypatch.setattr(ops, "requant_i4_to_i8", lambda q4, s4, out=None: R.requant_int4_to_int8(q4, s4))


def test_quantize_dit_convrot_traversal_and_lora_surgery(lib, monkeypatch):
    """Same targets, order and return value as quantize_dit_fp8 (quantize.py:54-68): every nn.Linear
    under dit.blocks, nothing else; then inject_lora wraps them (lora.py:81-116) and fuse_lora
    retargets only adapters on ConvRot bases, keeping class identity and parameters."""
    from k2q import lora, modules
    _oracle_quantizers(monkeypatch)
    dit = _TinyDit()
    n = modules.quantize_dit_convrot(dit, bits=8)
    assert n == 2 * 8
    assert all(isinstance(m, modules.ConvRotLinear) for b in dit.blocks for m in (b.attn.wq, b.mlp.down))
    assert isinstance(dit.first, nn.Linear) and isinstance(dit.txtmlp[1], nn.Linear)
    assert isinstance(dit.txtfusion.refiner_blocks[0].attn.wq, nn.Linear)
    # an 8-bit base is codes + scale and nothing else: one byte per weight, trained through as stored
    assert set(dict(dit.blocks[0].attn.wq.named_parameters())) == {"weight_q", "scale_bits"}
    adapters = lora.inject_lora(dit, rank=4, alpha=8.0)
    assert len(adapters) == 2 * 8 + 2 * 8 + 2
    assert list(adapters)[0] == "blocks.0.attn.wq" and "txtmlp.3" in adapters
    fused = [m for m in adapters.values() if getattr(m, "is_fused_lora", False)]
    assert len(fused) == 16 and all(isinstance(m, lora.LoRALinear) for m in fused)
    assert not getattr(adapters["txtmlp.1"], "is_fused_lora", False)
    trainable = [p for p in dit.parameters() if p.requires_grad]
    assert len(trainable) == 2 * len(adapters) and all(p.dtype == torch.float32 for p in trainable)
    ad = adapters["blocks.1.mlp.up"]
    assert ad.scale == 2.0 and ad.scale_mul == 1.0 and float(ad.lora_B.detach().abs().max()) == 0.0
    with lora.lora_scaled(dit, -1.5):
        assert all(m.scale_mul == -1.5 for m in adapters.values())
        with lora.lora_disabled(dit):
            assert all(m.scale_mul == 0.0 for m in adapters.values())
    assert all(m.scale_mul == 1.0 for m in adapters.values())
    # adapters on plain bf16 bases keep the reference formula (CPU-runnable): B = 0 -> identity
    x = torch.randn(3, 128)
    assert torch.equal(adapters["txtmlp.1"](x), dit.txtmlp[1].base(x))
    # adapters of Linears that read one tensor are linked for one shared down-projection pass
    wq = adapters["blocks.0.attn.wq"]
    assert wq._k2q_sibs == tuple(adapters[f"blocks.0.attn.{n}"] for n in ("wq", "wk", "wv", "gate"))
    assert [m._k2q_sib_off for m in wq._k2q_sibs] == [0, 4, 8, 12]
    assert adapters["blocks.1.mlp.up"]._k2q_sib_off == 4 and adapters["blocks.1.mlp.up"]._k2q_sibs[0] is adapters["blocks.1.mlp.gate"]
    assert not hasattr(adapters["blocks.0.attn.wo"], "_k2q_sibs") and not hasattr(adapters["blocks.0.mlp.down"], "_k2q_sibs")
    assert not hasattr(adapters["txtmlp.1"], "_k2q_sibs")           # plain bf16 bases are never linked
    assert lora.unfuse_lora(dit) == 16 and type(ad) is lora.LoRALinear
    assert not any(hasattr(m, "_k2q_sibs") or hasattr(m, "_k2q_sib_off") for m in adapters.values())
    with pytest.raises(RuntimeError, match="matched no Linear"):
        lora.inject_lora(_EmptyDit(), rank=2, include_txtfusion=False,
                         include_txtmlp=False)


class _EmptyDit(nn.Module):
    def __init__(self):
        super().__init__()
        self.blocks = nn.ModuleList([nn.Module()])


def test_quantize_base_flag_dispatch(lib, monkeypatch):
    from k2q import modules
    _oracle_quantizers(monkeypatch)
    dit = _TinyDit(layers=1)
    assert modules.apply_quantize_base(dit, "") == 0
    assert modules.apply_quantize_base(dit, "convrot_int4") == 8
    gate = dit.blocks[0].mlp.gate                      # the trainer flag means training: the int4 base keeps what dX needs
    assert gate.bits == 4 and gate.weight_q8.shape == (256, 128) and gate.backward_scale.shape == (256,)
    inf = _TinyDit(layers=1)
    modules.quantize_dit_convrot(inf, bits=4)
    assert inf.blocks[0].mlp.gate.weight_q8 is None
    with pytest.raises(RuntimeError, match="backward_copy=True"):
        inf.blocks[0].mlp.gate.backward_codes
    # "transient": nothing resident, the re-expression is rebuilt on demand; fast: needs it resident
    lin = nn.Linear(128, 32, bias=False)
    tr = modules.ConvRotLinear(lin, bits=4, backward_copy="transient")
    res = modules.ConvRotLinear(lin, bits=4, backward_copy=True, fast=True)
    assert tr.weight_q8 is None and tr.transient_backward and not res.transient_backward
    codes, scale = tr.backward_operands()
    assert torch.equal(codes, res.weight_q8.data) and torch.equal(scale, res.backward_scale)
    assert res.forward_operands()[1].data_ptr() == res.weight_q8.data_ptr()
    assert tr.forward_operands()[1].data_ptr() == tr.weight_q.data_ptr()
    with pytest.raises(ValueError, match="fast=True"):
        modules.ConvRotLinear(lin, bits=4, backward_copy=False, fast=True)
    with pytest.raises(ValueError, match="fast=True"):
        modules.ConvRotLinear(lin, bits=8, fast=True)
    with pytest.raises(ValueError, match="backward_copy must be"):
        modules.ConvRotLinear(lin, bits=4, backward_copy="sometimes")
    with pytest.raises(ValueError):
        modules.apply_quantize_base(dit, "int3")
    with pytest.raises(ValueError, match="multiple of the rotation block"):
        modules.ConvRotLinear(nn.Linear(100, 32), bits=8)


def test_block_swap_style_paging_keeps_codes(lib):
    """enable_block_swap pages parameters with p.data = p.data.to(device) (mmdit.py:409-414); the
    module must expose everything it needs as Parameters and read them at call time."""
    mod = _codes_module(32, 256, 8)
    before = {k: v.clone() for k, v in mod.state_dict().items()}
    for p in mod.parameters():
        p.data = p.data.to("cpu", copy=True)
    after = mod.state_dict()
    assert all(torch.equal(before[k], after[k]) for k in before)
    assert mod.scale.data_ptr() == mod.scale_bits.data_ptr()


def test_serialised_base_round_trip_and_text_side(lib, monkeypatch, tmp_path):
    """Codes and scales written with the adapter files' key convention (lora.py:154-172) come back bit
    for bit into a model that never saw the bf16 weights; the text-side extension covers the Linears
    quantize_dit_fp8 leaves out (quantize.py:60-65)."""
    from safetensors import safe_open
    from k2q import modules, serialize
    _oracle_quantizers(monkeypatch)
    for bits in (8, 4):
        dit = _TinyDit()
        assert modules.quantize_dit_convrot(dit, bits=bits, backward_copy=True) == 16
        extra = serialize.quantize_text_side(dit, bits=bits)
        assert extra == 2 * 8 + 2 and isinstance(dit.txtmlp[1], modules.ConvRotLinear)
        assert isinstance(dit.first, nn.Linear) and isinstance(dit.last, nn.Linear)     # 64 wide: left alone
        path = str(tmp_path / f"base{bits}.safetensors")
        assert serialize.save_quantized_base(dit, path, metadata={"note": "test"}) == 16 + extra
        with safe_open(path, framework="pt") as f:
            meta = f.metadata()
            assert meta["format"] == "krea2-convrot" and meta["bits"] == str(bits) and meta["note"] == "test"
            assert "diffusion_model.blocks.1.mlp.down.weight_q" in f.keys()
        fresh = _TinyDit()
        with torch.device("meta"):
            skeleton = _TinyDit()                           # no bf16 weights at all
        for target in (fresh, skeleton):
            assert serialize.load_quantized_base(target, path) == 16 + extra
            for name, m in serialize.convrot_modules(dit).items():
                got = target.get_submodule(name)
                assert isinstance(got, modules.ConvRotLinear) and got.bits == bits
                assert torch.equal(got.weight_q.data, m.weight_q.data) and torch.equal(got.scale, m.scale)
                assert (got.weight_q8 is None) == (m.weight_q8 is None)
                if m.weight_q8 is not None:
                    assert torch.equal(got.weight_q8.data, m.weight_q8.data) and torch.equal(got.backward_scale, m.backward_scale)
            assert getattr(target.blocks[0], "_k2q_shared_hooks", False)
    with pytest.raises(ValueError, match="not a krea2-convrot file"):
        from safetensors.torch import save_file
        bad = str(tmp_path / "bad.safetensors")
        save_file({"x": torch.zeros(1)}, bad, metadata={"format": "krea2-lora"})
        serialize.load_quantized_base(_TinyDit(), bad)


def test_prefetching_block_swap_logic_on_cpu(lib):
    """Host logic of the block swap for frozen codes (mmdit.py:389-428): the deepest blocks are parked,
    paged in by the pre-hook (the next one ahead of time), dropped after their forward, and paged in
    again for a checkpoint recompute, leaving after the block's backward."""
    from k2q import trainer

    class Blk(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(8, 8)
            self.lin.weight.requires_grad_(False)
            self.lin.bias.requires_grad_(False)
            self.ad = nn.Parameter(torch.zeros(8))          # trainable: stays put

        def forward(self, x):
            return self.lin(x) + self.ad

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = nn.ModuleList([Blk() for _ in range(4)])

        def forward(self, x, ckpt=False):
            for b in self.blocks:
                x = torch.utils.checkpoint.checkpoint(b, x, use_reentrant=False) if ckpt else b(x)
            return x

    torch.manual_seed(0)
    net = Net()
    x = torch.randn(3, 8)
    ref = net(x)
    st = trainer.enable_prefetching_block_swap(net, 2, "cpu")
    assert st.order == [2, 3] and set(st.host) == {2, 3} and len(st.host[2]) == 2      # weight + bias, not the adapter
    with torch.no_grad():
        out = net(x)
    assert torch.equal(out, ref) and st.copies == 2 and not st.ready                    # each paged in once, both dropped
    xg = x.clone().requires_grad_(True)
    st.copies = 0
    net(xg, ckpt=True).sum().backward()
    assert st.copies == 4 and not st.ready                                              # forward + recompute, all dropped again
    assert xg.grad is not None and all(b.ad.grad is not None for b in net.blocks)
    assert trainer.quantized_training_defaults("convrot_int8")["gradient_checkpointing_optional"]
    assert trainer.quantized_training_defaults("fp8")["force_gradient_checkpointing"]
