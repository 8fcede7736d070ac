"""Tensor-level wrappers over the C ABI (``include/k2q.h``).

torch supplies device memory and the current CUDA stream; every computation below is one call
into ``libk2q.so``.  Inputs must live on a CUDA device: there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
import threading

import torch

from . import _lib
from ._lib import ACT_GELU_TANH, ACT_NONE, K2Q_BF16, K2Q_F32, Epilogue

HAD_BLOCK = 128
GROUP = 128

_ACTS = {None: ACT_NONE, "none": ACT_NONE, "gelu_tanh": ACT_GELU_TANH}
_status_lock = threading.Lock()
_raw_writes = 0


def note_raw_write() -> None:
    """Called by every wrapper that lets the library write through a raw pointer into a tensor the
    caller supplied (``out=`` arguments, in-place transforms): such writes do not advance
    ``Tensor._version``, so caches keyed on it also key on this counter."""
    global _raw_writes
    _raw_writes += 1


def raw_write_epoch() -> int:
    return _raw_writes

_status_blocks: dict[int, torch.Tensor] = {}


def _dtype_tag(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return K2Q_BF16
    if t.dtype == torch.float32:
        return K2Q_F32
    raise TypeError(f"expected a bf16 or fp32 tensor, got {t.dtype}")


def _need_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "k2q kernels run on CUDA tensors only (got a tensor on "
                f"{t.device}); there is no CPU fallback")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev


def _stream(dev: torch.device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _ptr(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _rows2d(t: torch.Tensor) -> torch.Tensor:
    """View as [rows, last] with unit inner stride (copies only if it has to)."""
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(-1) != 1 or (t2.shape[0] > 1 and t2.stride(0) < t2.shape[1]):
        t2 = t2.contiguous()
    return t2


def status_block(dev: torch.device) -> torch.Tensor:
    """Per-device status block the GEMM kernels report expired waits into."""
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    with _status_lock:
        blk = _status_blocks.get(idx)
        if blk is None:
            nbytes = int(_lib.load().k2q_status_bytes())
            blk = torch.zeros(nbytes // 4, dtype=torch.int32, device=torch.device("cuda", idx))
            _status_blocks[idx] = blk
    return blk


def check_status(dev: torch.device | None = None) -> None:
    """Synchronises and raises if a bounded device-side wait expired in an earlier GEMM."""
    dev = dev or torch.device("cuda", torch.cuda.current_device())
    blk = status_block(dev)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_check_status(_ptr(blk), _stream(dev))
    if rc != 0:
        msg = _lib.last_error()
        blk.zero_()
        raise RuntimeError(f"k2q device status: {msg}")


def step_check(dev: torch.device | None = None) -> None:
    """Call once per optimizer step or sampler step, at a point that may synchronise: raises if a
    bounded device-side wait expired in any GEMM since the last check (their results are invalid
    then).  ``parallel.allreduce_adapter_grads`` calls it; single-GPU loops call it themselves."""
    check_status(dev)


# --------------------------------------------------------------------------------------------
# K1 / K2
# --------------------------------------------------------------------------------------------
def quant_weight_i8(w: torch.Tensor):
    """W [N,K] (bf16/fp32) -> (int8 codes [N,K], fp32 scale [N]); rotation + quantize.py:34-37."""
    dev = _need_cuda(w)
    w2 = _rows2d(w)
    n, k = w2.shape
    q = torch.empty(n, k, dtype=torch.int8, device=dev)
    s = torch.empty(n, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_quant_weight_i8(_ptr(w2), _dtype_tag(w2), n, k, w2.stride(0), _ptr(q), _ptr(s),
                                             _stream(dev))
    _lib.check(rc, "k2q_quant_weight_i8")
    return q, s


def quant_weight_i4(w: torch.Tensor):
    """W [N,K] -> (packed uint8 [N,K/2], bf16 group scale [N,K/128])."""
    dev = _need_cuda(w)
    w2 = _rows2d(w)
    n, k = w2.shape
    q = torch.empty(n, k // 2, dtype=torch.uint8, device=dev)
    s = torch.empty(n, k // GROUP, dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_quant_weight_i4(_ptr(w2), _dtype_tag(w2), n, k, w2.stride(0), _ptr(q), _ptr(s),
                                             _stream(dev))
    _lib.check(rc, "k2q_quant_weight_i4")
    return q, s


def requant_i4_to_i8(q4: torch.Tensor, scale4: torch.Tensor, out: torch.Tensor | None = None):
    """Packed int4 codes [N,K/2] + bf16 group scales [N,K/128] -> (int8 codes [N,K], fp32 scale [N])
    against one scale per output channel (what the backward of a 4-bit base contracts with)."""
    dev = _need_cuda(q4)
    if q4.dtype != torch.uint8 or q4.dim() != 2 or not q4.is_contiguous():
        raise ValueError("q4 must be a contiguous uint8 [N, K/2] tensor")
    n, k = q4.shape[0], q4.shape[1] * 2
    if scale4.dtype != torch.bfloat16 or tuple(scale4.shape) != (n, k // GROUP) or not scale4.is_contiguous():
        raise ValueError("scale4 must be a contiguous bf16 [N, K/128] tensor")
    if out is None:
        out = torch.empty(n, k, dtype=torch.int8, device=dev)
    elif out.dtype != torch.int8 or tuple(out.shape) != (n, k) or out.stride(1) != 1 or out.device != dev:
        raise ValueError("out must be an int8 [N, K] tensor with unit inner stride on the same device")
    s8 = torch.empty(n, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_requant_i4_to_i8(_ptr(q4), _ptr(scale4), n, k, _ptr(out), out.stride(0), _ptr(s8),
                                              _stream(dev))
    _lib.check(rc, "k2q_requant_i4_to_i8")
    note_raw_write()
    return out, s8


# below this many elements the general row kernel's many small CTAs win over one persistent CTA per SM
STREAMING_MIN_ELEMENTS = 8 << 20


def fwht_quant_act(x: torch.Tensor, streaming: bool | None = None):
    """x [..., K] -> (int8 codes [M,K], fp32 per-token scale [M]) with M = prod(leading dims).

    Contiguous bf16 rows with K a multiple of 1024 (and at least ``STREAMING_MIN_ELEMENTS`` elements)
    go to the streaming kernel (rows by TMA through a shared-memory ring,
    ``k2q_fwht_quant_act_i8_stream``), everything else to the general row kernel;
    both give the same bits.  ``streaming`` forces one or the other (True raises if the problem does
    not qualify)."""
    dev = _need_cuda(x)
    x2 = _rows2d(x)
    m, k = x2.shape
    xq = torch.empty(m, k, dtype=torch.int8, device=dev)
    sx = torch.empty(m, dtype=torch.float32, device=dev)
    lib = _lib.load()
    fits = m > 0 and x2.dtype == torch.bfloat16 and bool(lib.k2q_fwht_quant_act_i8_stream_ok(_dtype_tag(x2), m, k, x2.stride(0)))
    if streaming and not fits and m > 0:
        raise ValueError("fwht_quant_act: the streaming kernel takes contiguous bf16 rows with K a multiple of 1024")
    with torch.cuda.device(dev):
        if fits and (streaming or (streaming is None and m * k >= STREAMING_MIN_ELEMENTS)):
            rc = lib.k2q_fwht_quant_act_i8_stream(_ptr(x2), m, k, _ptr(xq), _ptr(sx), _ptr(status_block(dev)), _stream(dev))
            _lib.check(rc, "k2q_fwht_quant_act_i8_stream")
        else:
            rc = lib.k2q_fwht_quant_act_i8(_ptr(x2), _dtype_tag(x2), m, k, x2.stride(0), _ptr(xq), _ptr(sx), _stream(dev))
            _lib.check(rc, "k2q_fwht_quant_act_i8")
    return xq, sx


def _pair_quant(name, fn, a: torch.Tensor, b: torch.Tensor):
    dev = _need_cuda(a, b)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.shape != b.shape:
        raise ValueError(f"{name}: two bf16 tensors of one shape expected")
    a2, b2 = _rows2d(a), _rows2d(b)
    m, k = a2.shape
    xq = torch.empty(m, k, dtype=torch.int8, device=dev)
    sx = torch.empty(m, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = fn(_ptr(a2), a2.stride(0), _ptr(b2), b2.stride(0), m, k, _ptr(xq), _ptr(sx), _stream(dev))
    _lib.check(rc, name)
    return xq, sx


def swiglu_quant(g: torch.Tensor, u: torch.Tensor):
    """codes, scales of ``F.silu(g) * u`` (mmdit.py:178) without writing that tensor."""
    return _pair_quant("k2q_swiglu_fwht_quant", _lib.load().k2q_swiglu_fwht_quant, g, u)


def gate_quant(attn: torch.Tensor, gate: torch.Tensor):
    """codes, scales of ``attn * torch.sigmoid(gate)`` (mmdit.py:210)."""
    return _pair_quant("k2q_gate_fwht_quant", _lib.load().k2q_gate_fwht_quant, attn, gate)


def norm_mod_quant(x: torch.Tensor, norm_scale: torch.Tensor, mod_scale: torch.Tensor | None = None,
                   mod_shift: torch.Tensor | None = None, eps: float = 1e-5):
    """codes, scales of ``(1 + mod_scale) * RMSNorm(x) + mod_shift`` (mmdit.py:158-160, 313-317) for
    x [B, L, K] bf16, norm_scale [K] fp32 (the norm's weight is 1 + norm_scale), mod_* [B, 1, K] or [B, K]
    bf16 (or None: the plain norm)."""
    dev = _need_cuda(x, norm_scale, mod_scale, mod_shift)
    if x.dtype != torch.bfloat16 or x.dim() < 2:
        raise ValueError("norm_mod_quant: x must be a bf16 tensor [..., L, K]")
    k = x.shape[-1]
    rows_per_batch = x.shape[-2] if x.dim() >= 3 else x.shape[0]
    x2 = _rows2d(x)
    m = x2.shape[0]
    nb = m // rows_per_batch
    if norm_scale.dtype != torch.float32 or norm_scale.numel() != k or not norm_scale.is_contiguous():
        raise ValueError("norm_mod_quant: norm_scale must be a contiguous fp32 vector of length K")

    def vec(t, what):
        if t is None:
            return None
        if t.dtype != torch.bfloat16 or t.numel() != nb * k:
            raise ValueError(f"norm_mod_quant: {what} must be bf16 with {nb} x {k} elements")
        return t.reshape(nb, k).contiguous()

    sc, sh = vec(mod_scale, "mod_scale"), vec(mod_shift, "mod_shift")
    xq = torch.empty(m, k, dtype=torch.int8, device=dev)
    sx = torch.empty(m, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_norm_mod_fwht_quant(_ptr(x2), x2.stride(0), m, k, _ptr(norm_scale), _ptr(sc), _ptr(sh),
                                                 rows_per_batch, float(eps), _ptr(xq), _ptr(sx), _stream(dev))
    _lib.check(rc, "k2q_norm_mod_fwht_quant")
    return xq, sx


def qknorm_rope_(q: torch.Tensor, k: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor,
                 cos: torch.Tensor | None = None, sin: torch.Tensor | None = None, eps: float = 1e-5) -> None:
    """In place: QK-RMSNorm (weights 1 + wq / 1 + wk, fp32 [128]) and the rotary embedding of
    q [T, Hq*128] and k [T, Hk*128] (bf16, unit inner stride, any row stride: column blocks of a wider
    result are fine); cos / sin [T, 64] fp32 or None for the norm alone."""
    dev = _need_cuda(q, k, wq, wk, cos, sin)
    for name, t in (("q", q), ("k", k)):
        if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1 or t.shape[1] % 128:
            raise ValueError(f"qknorm_rope_: {name} must be bf16 [T, heads*128] with unit inner stride")
    t_rows = q.shape[0]
    if k.shape[0] != t_rows:
        raise ValueError("qknorm_rope_: q and k must have the same number of rows")
    for name, w in (("wq", wq), ("wk", wk)):
        if w.dtype != torch.float32 or w.numel() != 128 or not w.is_contiguous():
            raise ValueError(f"qknorm_rope_: {name} must be a contiguous fp32 vector of 128")
    if (cos is None) != (sin is None):
        raise ValueError("qknorm_rope_: cos and sin go together")
    if cos is not None:
        for name, t in (("cos", cos), ("sin", sin)):
            if t.dtype != torch.float32 or t.numel() != t_rows * 64 or not t.is_contiguous():
                raise ValueError(f"qknorm_rope_: {name} must be contiguous fp32 [T, 64]")
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_qknorm_rope(_ptr(q), q.stride(0), q.shape[1] // 128, _ptr(wq), _ptr(k), k.stride(0),
                                         k.shape[1] // 128, _ptr(wk), t_rows, _ptr(cos), _ptr(sin), float(eps),
                                         _stream(dev))
    _lib.check(rc, "k2q_qknorm_rope")
    note_raw_write()


def quant_rows(g: torch.Tensor, colscale: torch.Tensor | None = None):
    """Per-row int8 quantisation of g * colscale without rotation."""
    dev = _need_cuda(g, colscale)
    g2 = _rows2d(g)
    m, n = g2.shape
    if colscale is not None:
        colscale = colscale.reshape(-1)
        if colscale.dtype != torch.float32 or colscale.numel() != n or not colscale.is_contiguous():
            raise ValueError("colscale must be a contiguous fp32 vector of length N")
    gq = torch.empty(m, n, dtype=torch.int8, device=dev)
    sg = torch.empty(m, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_quant_rows_i8(_ptr(g2), _dtype_tag(g2), m, n, g2.stride(0), _ptr(colscale), _ptr(gq),
                                           _ptr(sg), _stream(dev))
    _lib.check(rc, "k2q_quant_rows_i8")
    return gq, sg


def fwht_rows(x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """y = H(x) along the last axis (block 128)."""
    dev = _need_cuda(x)
    x2 = _rows2d(x)
    m, k = x2.shape
    y = torch.empty(m, k, dtype=out_dtype or x.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_fwht_rows(_ptr(x2), _dtype_tag(x2), m, k, x2.stride(0), _ptr(y), _dtype_tag(y), k,
                                       _stream(dev))
    _lib.check(rc, "k2q_fwht_rows")
    return y.reshape(*x.shape[:-1], k)


# --------------------------------------------------------------------------------------------
# K3 / K4
# --------------------------------------------------------------------------------------------
def _epilogue(sx, bias, u, bm, lora_scale, act) -> Epilogue:
    ep = Epilogue()
    ep.sx = 0 if sx is None else sx.data_ptr()
    ep.bias = 0 if bias is None else bias.data_ptr()
    if u is not None:
        if u.dtype != torch.float32 or bm.dtype != torch.float32:
            raise TypeError("LoRA operands u and B must be fp32")
        if u.stride(-1) != 1 or bm.stride(-1) != 1:
            raise ValueError("LoRA operands need unit inner stride")
        ep.u, ep.Bm = u.data_ptr(), bm.data_ptr()
        ep.ldu, ep.ldb = u.stride(0), bm.stride(0)
        ep.rank = u.shape[1]
        ep.lora_scale = float(lora_scale)
    ep.act = _ACTS[act]
    return ep


def _check_out(name, out, m, n, dev):
    """A caller-supplied output must be what the kernel will write: [M, N] bf16 on the operands' device
    with unit inner stride (rows may be padded)."""
    if out.dtype != torch.bfloat16 or out.dim() != 2 or tuple(out.shape) != (m, n):
        raise ValueError(f"{name}: out must be a bf16 tensor of shape [{m}, {n}], got {out.dtype} {tuple(out.shape)}")
    if out.device != dev:
        raise RuntimeError(f"{name}: out lives on {out.device}, the operands on {dev}")
    if out.stride(1) != 1 or (m > 1 and out.stride(0) < n):
        raise ValueError(f"{name}: out needs unit inner stride and a row stride >= {n}")
    note_raw_write()


def _check_lora(name, u, bm, m, n):
    if (u is None) != (bm is None):
        raise ValueError(f"{name}: u and bm go together")
    if u is not None and (u.dim() != 2 or bm.dim() != 2 or u.shape[0] != m or bm.shape[0] != n
                          or u.shape[1] != bm.shape[1]):
        raise ValueError(f"{name}: LoRA operand shapes do not match (u [M, r], bm [N, r])")


def _check_vec(name, t, n):
    if t is None:
        return
    if t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous fp32 vector of length {n}")


def gemm_w8a8(xq, sx, wq, sw, bias=None, u=None, bm=None, lora_scale: float = 0.0, act=None,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """y[M,N] bf16 = act(int32(xq.wq^T)*sx*sw + bias) + lora_scale * u.bm^T."""
    dev = _need_cuda(xq, sx, wq, sw, bias, u, bm)
    m, k = xq.shape
    n = wq.shape[0]
    if wq.shape[1] != k or xq.dtype != torch.int8 or wq.dtype != torch.int8:
        raise ValueError("gemm_w8a8: xq [M,K] and wq [N,K] must be int8 with equal K")
    if not (xq.is_contiguous() and wq.is_contiguous()):
        raise ValueError("gemm_w8a8: codes must be contiguous")
    _check_vec("sx", sx, m)
    _check_vec("sw", sw, n)
    _check_vec("bias", bias, n)
    _check_lora("gemm_w8a8", u, bm, m, n)
    if out is not None:
        _check_out("gemm_w8a8", out, m, n, dev)
    y = out if out is not None else torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    ep = _epilogue(sx, bias, u, bm, lora_scale, act)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_gemm_w8a8(_ptr(xq), _ptr(wq), _ptr(sw), m, n, k, C.byref(ep), _ptr(y), y.stride(0),
                                       _ptr(status_block(dev)), _stream(dev))
    _lib.check(rc, "k2q_gemm_w8a8")
    return y


def gemm_w4a8(xq, sx, wq4, sw4, bias=None, u=None, bm=None, lora_scale: float = 0.0, act=None,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """W4A8 variant: wq4 [N,K/2] packed uint8, sw4 [N,K/128] bf16."""
    dev = _need_cuda(xq, sx, wq4, sw4, bias, u, bm)
    m, k = xq.shape
    n = wq4.shape[0]
    if wq4.shape[1] * 2 != k or xq.dtype != torch.int8 or wq4.dtype != torch.uint8:
        raise ValueError("gemm_w4a8: xq [M,K] int8 and wq4 [N,K/2] uint8 expected")
    if sw4.dtype != torch.bfloat16 or tuple(sw4.shape) != (n, k // GROUP) or not sw4.is_contiguous():
        raise ValueError("gemm_w4a8: sw4 must be contiguous bf16 [N, K/128]")
    if not (xq.is_contiguous() and wq4.is_contiguous()):
        raise ValueError("gemm_w4a8: codes must be contiguous")
    _check_vec("sx", sx, m)
    _check_vec("bias", bias, n)
    _check_lora("gemm_w4a8", u, bm, m, n)
    if out is not None:
        _check_out("gemm_w4a8", out, m, n, dev)
    y = out if out is not None else torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    ep = _epilogue(sx, bias, u, bm, lora_scale, act)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_gemm_w4a8(_ptr(xq), _ptr(wq4), _ptr(sw4), m, n, k, C.byref(ep), _ptr(y), y.stride(0),
                                       _ptr(status_block(dev)), _stream(dev))
    _lib.check(rc, "k2q_gemm_w4a8")
    return y


def linear_desc(bits: int, codes: torch.Tensor, scale: torch.Tensor, bias: torch.Tensor | None, n: int, k: int):
    """``k2q_linear`` over the operands of a quantised base (8: int8 [N,K] + f32 [N]; 4: packed uint8
    [N,K/2] + bf16 [N,K/128]).  The tensors must outlive the call that takes the descriptor."""
    _need_cuda(codes, scale, bias)
    if bits == 8:
        ok = codes.dtype == torch.int8 and tuple(codes.shape) == (n, k) and scale.dtype == torch.float32 and scale.numel() == n
    elif bits == 4:
        ok = (codes.dtype == torch.uint8 and tuple(codes.shape) == (n, k // 2) and scale.dtype == torch.bfloat16
              and tuple(scale.shape) == (n, k // GROUP))
    else:
        raise ValueError(f"linear_desc: bits = {bits}")
    if not ok or not codes.is_contiguous() or not scale.is_contiguous():
        raise ValueError("linear_desc: codes / scales do not have the layout of a %d-bit base [%d, %d]" % (bits, n, k))
    _check_vec("bias", bias, n)
    return _lib.Linear(bits, 0, codes.data_ptr(), scale.data_ptr(), 0 if bias is None else bias.data_ptr(), n, k)


def mlp_gelu_host(x_host: torch.Tensor, fc1, fc2, y_host: torch.Tensor, schedule: list[int], k: int, h: int, n2: int,
                  dev: torch.device, copy_in: torch.cuda.Stream, copy_out: torch.cuda.Stream) -> None:
    """``k2q_mlp_gelu_host`` on contiguous bf16 HOST tensors x [M, k] -> y [M, n2] through the bases
    described by ``fc1`` / ``fc2`` (:func:`linear_desc`), rows cut as ``schedule`` says.  The workspace
    comes from torch's allocator on the current stream; the call rejoins both copy streams into the
    current one, so handing the block back afterwards is safe."""
    m = x_host.shape[0]
    if x_host.is_cuda or y_host.is_cuda or x_host.dtype != torch.bfloat16 or y_host.dtype != torch.bfloat16:
        raise ValueError("mlp_gelu_host: bf16 host tensors expected")
    if not (x_host.is_contiguous() and y_host.is_contiguous()) or x_host.numel() != m * k or y_host.numel() != m * n2:
        raise ValueError("mlp_gelu_host: x [M, K] and y [M, N] must be contiguous")
    if m == 0:
        return
    if sum(schedule) != m or min(schedule) <= 0:
        raise ValueError("mlp_gelu_host: the schedule's rows must be positive and add up to M")
    lib = _lib.load()
    need = int(lib.k2q_mlp_gelu_host_workspace_bytes(m, k, h, n2, max(schedule)))
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    rows = (C.c_int64 * len(schedule))(*schedule)
    rc = lib.k2q_mlp_gelu_host(C.c_void_p(x_host.data_ptr()), m, C.byref(fc1), C.byref(fc2), C.c_void_p(y_host.data_ptr()),
                               rows, len(schedule), _ptr(ws), need, _ptr(status_block(dev)), _stream(dev),
                               C.c_void_p(copy_in.cuda_stream), C.c_void_p(copy_out.cuda_stream))
    _lib.check(rc, "k2q_mlp_gelu_host")
    note_raw_write()


def gemm_dx_w8(gq, sg, wq, u=None, bm=None, lora_scale: float = 0.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """dx[M,K] bf16 = int32(gq . wq) * sg + lora_scale * u.bm^T with gq [M,N] int8 and wq [N,K] int8 as the
    forward stores it (contraction over N, read as an MN-major operand: no transposed weights)."""
    dev = _need_cuda(gq, sg, wq, u, bm)
    m, n = gq.shape
    k = wq.shape[1]
    if wq.shape[0] != n or gq.dtype != torch.int8 or wq.dtype != torch.int8:
        raise ValueError("gemm_dx_w8: gq [M,N] and wq [N,K] must be int8 with equal N")
    if not (gq.is_contiguous() and wq.is_contiguous()):
        raise ValueError("gemm_dx_w8: codes must be contiguous")
    if n % 128:
        raise ValueError(f"gemm_dx_w8: out_features={n} (the contraction of dX) must be a multiple of 128")
    _check_vec("sg", sg, m)
    _check_lora("gemm_dx_w8", u, bm, m, k)
    if out is not None:
        _check_out("gemm_dx_w8", out, m, k, dev)
    y = out if out is not None else torch.empty(m, k, dtype=torch.bfloat16, device=dev)
    ep = _epilogue(sg, None, u, bm, lora_scale, None)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_gemm_dx_w8(_ptr(gq), _ptr(wq), m, n, k, C.byref(ep), _ptr(y), y.stride(0),
                                        _ptr(status_block(dev)), _stream(dev))
    _lib.check(rc, "k2q_gemm_dx_w8")
    return y


def transpose_i8(q: torch.Tensor) -> torch.Tensor:
    dev = _need_cuda(q)
    if q.dtype != torch.int8 or q.dim() != 2 or not q.is_contiguous():
        raise ValueError("transpose_i8: contiguous int8 matrix expected")
    r, c = q.shape
    out = torch.empty(c, r, dtype=torch.int8, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_transpose_i8(_ptr(q), r, c, _ptr(out), _stream(dev))
    _lib.check(rc, "k2q_transpose_i8")
    return out


# --------------------------------------------------------------------------------------------
# K5 / K7
# --------------------------------------------------------------------------------------------
def lora_down(x: torch.Tensor, a: torch.Tensor, scale: float = 1.0, transposed: bool = False) -> torch.Tensor:
    """out[M,r] fp32 = scale * x[M,K] . A^T.  ``a`` is [r,K]; with ``transposed`` it is given as
    [K,r] (e.g. lora_B [N,r] for du = s*dY.B)."""
    dev = _need_cuda(x, a)
    if x.dtype != torch.bfloat16:
        raise TypeError("lora_down: x must be bf16")
    if a.dtype != torch.float32:
        raise TypeError("lora_down: the low-rank factor must be fp32")
    x2 = _rows2d(x)
    m, k = x2.shape
    if transposed:
        if a.shape[0] != k:
            raise ValueError("lora_down: factor [K,r] does not match x")
        a = a.t().contiguous()          # [r, K]: tiny copy, lets the kernel read the factor with 128-bit loads
        r, rs, cs = a.shape[0], a.stride(0), a.stride(1)
    else:
        if a.shape[1] != k:
            raise ValueError("lora_down: factor [r,K] does not match x")
        r, rs, cs = a.shape[0], a.stride(0), a.stride(1)
    out = torch.empty(m, r, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_lora_down(_ptr(x2), m, k, x2.stride(0), _ptr(a), rs, cs, r, float(scale), _ptr(out), r,
                                       _stream(dev))
    _lib.check(rc, "k2q_lora_down")
    return out


def lora_tn(p: torch.Tensor, q: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[r,C] fp32 = scale * p[T,r]^T . q[T,C]   (p fp32, q bf16)."""
    dev = _need_cuda(p, q)
    if p.dtype != torch.float32 or q.dtype != torch.bfloat16:
        raise TypeError("lora_tn: p must be fp32 and q bf16")
    q2 = _rows2d(q)
    p2 = _rows2d(p)
    t, c = q2.shape
    if p2.shape[0] != t:
        raise ValueError("lora_tn: row counts differ")
    r = p2.shape[1]
    lib = _lib.load()
    ws_bytes = int(lib.k2q_lora_tn_workspace_bytes(t, r, c))
    ws = torch.empty(max(ws_bytes, 4) // 4, dtype=torch.float32, device=dev)
    out = torch.empty(r, c, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.k2q_lora_tn(_ptr(p2), p2.stride(0), _ptr(q2), q2.stride(0), t, r, c, float(scale), _ptr(out), c,
                             _ptr(ws), ws_bytes, _stream(dev))
    _lib.check(rc, "k2q_lora_tn")
    return out


def measure_i8_peak(iters: int = 4096, dev: torch.device | None = None) -> float:
    """TOP/s of back-to-back tcgen05 int8 MMAs from resident shared memory (calibration only)."""
    dev = dev or torch.device("cuda", torch.cuda.current_device())
    out = C.c_double(0.0)
    with torch.cuda.device(dev):
        rc = _lib.load().k2q_measure_i8_peak(int(iters), _ptr(status_block(dev)), C.byref(out), _stream(dev))
    _lib.check(rc, "k2q_measure_i8_peak")
    return float(out.value)
