"""Kernel-level parity on the GPU: every op goes through the C ABI (libk2q.so) and is compared
with the CPU oracle on the same seeded inputs.  Integer outputs (codes, packed nibbles) and
scales are bit-exact; GEMM outputs without activation/adapter are bit-exact against O-exact."""
import pytest
import torch

from oracle import convrot_ref as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from k2q import ops as _ops
    return _ops


def _dev(t):
    return t.cuda()


# ------------------------------------------------------------------------------------------------
# K2 / K1: rotation + quantisation, bit-exact
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("m,k", [(1, 128), (5, 256), (33, 1024), (64, 1536), (256, 3072), (48, 2560),
                                 (16, 6912), (8, 12288), (8, 16384)])
def test_fwht_quant_act_bit_exact(ops, m, k):
    x = R.synth_act(m, k, seed=2000 + k, outliers=8 if k >= 1024 else 1)
    q_ref, s_ref = R.quantize_act_int8(x)
    q, s = ops.fwht_quant_act(_dev(x))
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(s.cpu(), s_ref.reshape(-1))


def test_fwht_quant_act_edge_rows(ops):
    k = 512
    x = torch.zeros(6, k)
    x[1, 3] = 1.0                       # single spike -> flat rotated block, ties at +-amax
    x[2] = 0.5                          # constant row -> energy in one coefficient per block
    x[3] = torch.arange(k) % 7 - 3.0    # small integers, exact .5 boundaries after scaling
    x[4, :128] = -2.0 ** -120           # tiny values: scale clamps at 1e-8/127
    x[5] = torch.randn(k, generator=torch.Generator().manual_seed(5)) * 1e4
    x = x.to(torch.bfloat16)
    q_ref, s_ref = R.quantize_act_int8(x)
    q, s = ops.fwht_quant_act(_dev(x))
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(s.cpu(), s_ref.reshape(-1))
    assert float(s_ref[0]) == pytest.approx(1e-8 / 127, rel=1e-6)  # all-zero row takes the clamp path


@pytest.mark.parametrize("m,k", [(1, 1024), (7, 2048), (333, 3072), (1000, 6144), (37, 12288), (150, 16384),
                                 (2500, 1024), (2100, 4096)])
def test_fwht_quant_act_streaming_kernel_bit_exact(ops, m, k):
    """The TMA-fed streaming form of K2 (teams of K/1024 warps per row, several rounds of rows per CTA at the
    larger M, ragged last rounds) against the oracle and against the general row kernel; rows of zeros, a
    single spike and tiny values among them."""
    x = R.synth_act(m, k, seed=4000 + k + m, outliers=8)
    if m > 4:
        x[1] = 0
        x[2] = 0
        x[2, k - 1] = 1.0
        x[3, :256] = -2.0 ** -120
    xd = _dev(x)
    q, s = ops.fwht_quant_act(xd, streaming=True)
    q0, s0 = ops.fwht_quant_act(xd, streaming=False)
    assert torch.equal(q, q0) and torch.equal(s, s0)
    if m * k <= 4_000_000:
        q_ref, s_ref = R.quantize_act_int8(x)
        assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref.reshape(-1))
    qa, sa = ops.fwht_quant_act(xd)                  # the automatic choice (streaming from 8 Mi elements on)
    assert torch.equal(qa, q) and torch.equal(sa, s)
    ops.check_status()
    with pytest.raises(ValueError):
        ops.fwht_quant_act(xd[:, :k - 128] if k > 1024 else xd.float(), streaming=True)


def test_fwht_quant_act_fp32_input_and_strided(ops):
    x = torch.randn(40, 768, generator=torch.Generator().manual_seed(1))
    q_ref, s_ref = R.quantize_act_int8(x)
    q, s = ops.fwht_quant_act(_dev(x))
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref.reshape(-1))
    big = _dev(R.synth_act(40, 1024, seed=7))
    view = big[:, :768]                 # ld = 1024 > K
    q_ref, s_ref = R.quantize_act_int8(view.cpu())
    q, s = ops.fwht_quant_act(view)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref.reshape(-1))


@pytest.mark.parametrize("n,k,dtype", [(128, 128, torch.bfloat16), (768, 1024, torch.bfloat16),
                                       (304, 3072, torch.bfloat16), (96, 2560, torch.float32)])
def test_quant_weight_int8_bit_exact(ops, n, k, dtype):
    w = R.synth_weight(n, k, seed=1000 + n).to(dtype)
    q_ref, s_ref = R.quantize_weight_int8(w)
    q, s = ops.quant_weight_i8(_dev(w))
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(s.cpu(), s_ref)


@pytest.mark.parametrize("n,k,dtype", [(128, 128, torch.bfloat16), (768, 1024, torch.bfloat16),
                                       (304, 3072, torch.bfloat16), (96, 2560, torch.float32)])
def test_quant_weight_int4_bit_exact(ops, n, k, dtype):
    w = R.synth_weight(n, k, seed=1100 + n).to(dtype)
    w[0] = 0                           # all-zero row: clamp path in every group
    p_ref, s_ref = R.quantize_weight_int4(w)
    p, s = ops.quant_weight_i4(_dev(w))
    assert torch.equal(p.cpu(), p_ref)
    assert torch.equal(s.cpu().view(torch.int16), s_ref.view(torch.int16))
    assert torch.equal(R.unpack_int4(p.cpu()), R.unpack_int4(p_ref))


def test_quant_rows_bit_exact(ops):
    g = (torch.randn(70, 1536, generator=torch.Generator().manual_seed(6000)) * 1e-2).to(torch.bfloat16)
    cs = torch.rand(1536, generator=torch.Generator().manual_seed(3)) * 1e-3 + 1e-4
    q_ref, s_ref = R.quantize_rows_int8(g, cs)
    q, s = ops.quant_rows(_dev(g), _dev(cs))
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref.reshape(-1))
    q_ref, s_ref = R.quantize_rows_int8(g, None)
    q, s = ops.quant_rows(_dev(g), None)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref.reshape(-1))


def test_fwht_rows_matches_oracle_and_is_involution(ops):
    x = torch.randn(50, 2048, generator=torch.Generator().manual_seed(11))
    y = ops.fwht_rows(_dev(x))
    assert torch.equal(y.cpu(), R.hadamard128(x))
    back = ops.fwht_rows(y)
    assert (back.cpu() - x).abs().max() < 1e-5
    xb = x.to(torch.bfloat16)
    yb = ops.fwht_rows(_dev(xb))
    assert torch.equal(yb.cpu(), R.hadamard128(xb.float()).to(torch.bfloat16))
    # bf16 in, fp32 out: the output rows need twice the staging space of the input rows
    yf = ops.fwht_rows(_dev(xb), out_dtype=torch.float32)
    assert torch.equal(yf.cpu(), R.hadamard128(xb.float()))


# ------------------------------------------------------------------------------------------------
# K3: W8A8 GEMM
# ------------------------------------------------------------------------------------------------
def _int8_problem(m, n, k, seed=0, bias=True):
    w = R.synth_weight(n, k, seed=1000 + seed)
    x = R.synth_act(m, k, seed=2000 + seed, outliers=8)
    wq, sw = R.quantize_weight_int8(w)
    xq, sx = R.quantize_act_int8(x)
    b = R.synth_vec(n, 0.01, 3000 + seed) if bias else None
    return x, w, xq, sx.reshape(-1), wq, sw, b


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 256, 512), (256, 512, 1024), (100, 272, 384),
                                   (1, 16, 128), (513, 768, 1536), (300, 3072, 3072)])
def test_gemm_w8a8_bit_exact(ops, m, n, k):
    x, w, xq, sx, wq, sw, b = _int8_problem(m, n, k)
    y_ref = R.linear_int8_exact(xq, sx, wq, sw, b)
    y = ops.gemm_w8a8(_dev(xq), _dev(sx), _dev(wq), _dev(sw), _dev(b))
    ops.check_status()
    assert torch.equal(y.cpu().view(torch.int16), y_ref.view(torch.int16))
    # the 2e-2 gate: against the torch dequant-matmul path on the same codes
    y_sim = R.linear_sim_dequant(xq, sx, wq, sw, 8, b)
    assert R.max_rel_err(y.cpu(), y_sim) <= 2e-2


def test_gemm_w8a8_no_bias_no_scales(ops):
    x, w, xq, sx, wq, sw, _ = _int8_problem(200, 512, 256, seed=3, bias=False)
    y = ops.gemm_w8a8(_dev(xq), None, _dev(wq), None)
    ops.check_status()
    acc = R.int_matmul(xq, wq).float().to(torch.bfloat16)
    assert torch.equal(y.cpu().view(torch.int16), acc.view(torch.int16))


@pytest.mark.parametrize("rank,scale", [(16, 1.0), (32, -1.5), (8, 0.5), (64, 1.0)])
def test_gemm_w8a8_lora_epilogue(ops, rank, scale):
    m, n, k = 260, 528, 768
    x, w, xq, sx, wq, sw, b = _int8_problem(m, n, k, seed=rank)
    a = R.synth_mat(rank, k, 0.01, 4000)
    bm = R.synth_mat(n, rank, 0.01, 5000)
    u = x.float() @ a.t()
    y = ops.gemm_w8a8(_dev(xq), _dev(sx), _dev(wq), _dev(sw), _dev(b), u=_dev(u), bm=_dev(bm), lora_scale=scale)
    ops.check_status()
    base = R.linear_int8_exact(xq, sx, wq, sw, b)
    ref = R.lora_forward_ref(base, x, a, bm, scale)
    fused = (R.int_matmul(xq, wq).float() * sx.reshape(-1, 1) * sw.reshape(1, -1) + b + scale * (u @ bm.t()))
    assert (y.cpu().float() - fused).abs().max() <= 2 ** -7 * fused.abs().max()   # one bf16 rounding
    assert R.max_rel_err(y.cpu(), ref) <= 2e-2


@pytest.mark.parametrize("rank,act", [(32, None), (24, "gelu_tanh"), (16, None)])
def test_gemm_w8a8_lora_epilogue_long_contraction(ops, rank, act):
    """Ranks 17..32 take the adapter term on the fp32 pipe from K = 12288 on (warp-level MMAs below that), rank
    <= 16 from M = 8192 on: those instantiations against the same composition, ragged M and N, a rank that
    is not a multiple of 8, an activation in front of the adapter term."""
    m, n, k = (8200, 272, 1024) if rank == 16 else (333, 272, 12288)
    g = torch.Generator().manual_seed(rank)
    xq = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8)
    wq = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    sx, sw = torch.rand(m, generator=g) * 1e-3 + 1e-4, torch.rand(n, generator=g) * 1e-2 + 1e-3
    b = torch.randn(n, generator=g) * 0.1
    u, bm = torch.randn(m, rank, generator=g), torch.randn(n, rank, generator=g) * 0.3
    y = ops.gemm_w8a8(_dev(xq), _dev(sx), _dev(wq), _dev(sw), _dev(b), u=_dev(u), bm=_dev(bm), lora_scale=-0.75, act=act)
    ops.check_status()
    base = R.int_matmul(xq, wq).float() * sx.reshape(-1, 1) * sw.reshape(1, -1) + b
    if act:
        base = torch.nn.functional.gelu(base, approximate="tanh")
    fused = base - 0.75 * (u @ bm.t())
    tol = 2 ** -7 * fused.abs().max() + (4e-3 * base.abs().max() if act else 0.0)
    assert (y.cpu().float() - fused).abs().max() <= tol
    # dX through the MN-major operand with the same long contraction (N of the forward): equal to the K-major
    # kernel on a transposed copy, which runs the same epilogue
    u2, bm2 = torch.randn(m, rank, generator=g), torch.randn(n, rank, generator=g) * 0.1
    gq = xq
    w2 = torch.randint(-127, 128, (k, n), generator=g, dtype=torch.int8)
    out = ops.gemm_dx_w8(_dev(gq), _dev(sx), _dev(w2), u=_dev(u2), bm=_dev(bm2), lora_scale=1.0)
    ref = ops.gemm_w8a8(_dev(gq), _dev(sx), _dev(w2.t().contiguous()), None, None, u=_dev(u2), bm=_dev(bm2), lora_scale=1.0)
    ops.check_status()
    assert torch.equal(out, ref)
    exact = R.int_matmul(gq, w2.t().contiguous()).float() * sx.reshape(-1, 1) + u2 @ bm2.t()
    assert (out.cpu().float() - exact).abs().max() <= 2 ** -7 * exact.abs().max()


def test_gemm_w8a8_gelu_epilogue(ops):
    x, w, xq, sx, wq, sw, b = _int8_problem(192, 512, 512, seed=9)
    y = ops.gemm_w8a8(_dev(xq), _dev(sx), _dev(wq), _dev(sw), _dev(b), act="gelu_tanh")
    ops.check_status()
    ref = R.linear_int8_exact(xq, sx, wq, sw, b, act="gelu_tanh")
    assert R.max_rel_err(y.cpu(), ref) <= 4e-3


# ------------------------------------------------------------------------------------------------
# K4: W4A8 GEMM
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (128, 128, 512), (256, 384, 1024), (100, 272, 384),
                                   (1, 16, 128), (300, 1024, 3072)])
def test_gemm_w4a8_bit_exact(ops, m, n, k):
    w = R.synth_weight(n, k, seed=1200)
    x = R.synth_act(m, k, seed=2200)
    wq4, sw4 = R.quantize_weight_int4(w)
    xq, sx = R.quantize_act_int8(x)
    sx = sx.reshape(-1)
    b = R.synth_vec(n, 0.01, 3200)
    y_ref = R.linear_int4_exact(xq, sx, wq4, sw4, b)
    y = ops.gemm_w4a8(_dev(xq), _dev(sx), _dev(wq4), _dev(sw4), _dev(b))
    ops.check_status()
    assert torch.equal(y.cpu().view(torch.int16), y_ref.view(torch.int16))
    y_sim = R.linear_sim_dequant(xq, sx, wq4, sw4, 4, b)
    assert R.max_rel_err(y.cpu(), y_sim) <= 2e-2


def test_gemm_w4a8_gelu_and_lora(ops):
    m, n, k, rank = 200, 384, 768, 16
    w = R.synth_weight(n, k, seed=1300)
    x = R.synth_act(m, k, seed=2300)
    wq4, sw4 = R.quantize_weight_int4(w)
    xq, sx = R.quantize_act_int8(x)
    sx = sx.reshape(-1)
    y = ops.gemm_w4a8(_dev(xq), _dev(sx), _dev(wq4), _dev(sw4), None, act="gelu_tanh")
    ops.check_status()
    ref = R.linear_int4_exact(xq, sx, wq4, sw4, None, act="gelu_tanh")
    assert R.max_rel_err(y.cpu(), ref) <= 4e-3
    a = R.synth_mat(rank, k, 0.01, 4000)
    bm = R.synth_mat(n, rank, 0.01, 5000)
    u = x.float() @ a.t()
    y = ops.gemm_w4a8(_dev(xq), _dev(sx), _dev(wq4), _dev(sw4), None, u=_dev(u), bm=_dev(bm), lora_scale=2.0)
    ops.check_status()
    fused = R.linear_int4_exact(xq, sx, wq4, sw4, None, fp32_out=True) + 2.0 * (u @ bm.t())
    assert (y.cpu().float() - fused).abs().max() <= 2 ** -7 * fused.abs().max()


# ------------------------------------------------------------------------------------------------
# K5 / K7 and the transpose
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("m,k,r", [(16, 128, 16), (100, 768, 16), (333, 3072, 32), (64, 1536, 8), (40, 512, 64),
                                   (4096, 3072, 32),      # 64-row tiles, K split over a cluster of 2
                                   (2048, 1024, 16),      # cluster of 4
                                   (700, 776, 24),        # 32-row tiles, K tail (776 = 24 * 32 + 8), ragged M
                                   (1200, 2048, 64)])     # widest factor
def test_lora_down(ops, m, k, r):
    x = R.synth_act(m, k, seed=2000)
    a = R.synth_mat(r, k, 0.01, 4000)
    ref = (x.double() @ a.double().t()).float()
    u = ops.lora_down(_dev(x), _dev(a))
    assert (u.cpu() - ref).abs().max() <= 2e-4 * ref.abs().max()
    bt = R.synth_mat(k, r, 0.01, 5000)                    # factor given as [K, r]
    ref2 = (0.5 * x.double() @ bt.double()).float()
    u2 = ops.lora_down(_dev(x), _dev(bt), scale=0.5, transposed=True)
    assert (u2.cpu() - ref2).abs().max() <= 2e-4 * ref2.abs().max()


def test_lora_down_strided_factor(ops):
    """The factor handed over as a strided view ([K, r] storage read as [r, K]): the register-prefetch
    kernel that serves factors without unit stride along K."""
    import ctypes as C
    from k2q import _lib
    lib = _lib.load()
    m, k, r = 1500, 640, 32
    x = _dev(R.synth_act(m, k, seed=2000))
    bt = _dev(R.synth_mat(k, r, 0.01, 5000))               # [K, r]: element (j, kk) at kk * r + j
    out = torch.full((m, r), float("nan"), device="cuda")
    rc = lib.k2q_lora_down(C.c_void_p(x.data_ptr()), m, k, k, C.c_void_p(bt.data_ptr()), 1, r, r, 0.5,
                           C.c_void_p(out.data_ptr()), r, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.k2q_last_error()
    ref = (0.5 * x.double() @ bt.double()).float()
    assert (out - ref).abs().max() <= 2e-4 * ref.abs().max()


@pytest.mark.parametrize("t,r,c", [(16, 16, 128), (100, 16, 384), (1000, 32, 1536), (4096, 32, 3072), (77, 8, 136),
                                   (50, 6, 128),          # rank not a multiple of 4: the register-staged kernel
                                   (3000, 64, 1024)])
def test_lora_tn(ops, t, r, c):
    p = R.synth_mat(t, r, 1.0, 1)
    q = R.synth_mat(t, c, 1e-2, 2).to(torch.bfloat16)
    ref = (2.0 * p.double().t() @ q.double()).float()
    out = ops.lora_tn(_dev(p), _dev(q), scale=2.0)
    assert (out.cpu() - ref).abs().max() <= 2e-4 * ref.abs().max()
    out2 = ops.lora_tn(_dev(p), _dev(q), scale=2.0)
    assert torch.equal(out, out2)                         # fixed reduction order


@pytest.mark.parametrize("m,n,k,rank", [(100, 128, 256, 0), (300, 384, 768, 0), (260, 512, 272, 16), (1024, 3072, 3072, 32)])
def test_gemm_dx_reads_stored_codes_like_a_transposed_copy(ops, m, n, k, rank):
    """dX = gq . wq with wq [N, K] as the forward stores it (MN-major operand) equals, bit for bit, the
    K-major GEMM on an explicit transpose -- integer accumulation is exact."""
    g = torch.Generator().manual_seed(m + rank)
    gq = torch.randint(-127, 128, (m, n), generator=g, dtype=torch.int8)
    wq = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    sg = torch.rand(m, generator=g) * 1e-3 + 1e-4
    u = bm = None
    if rank:
        u, bm = torch.randn(m, rank, generator=g), torch.randn(k, rank, generator=g) * 0.1
    out = ops.gemm_dx_w8(_dev(gq), _dev(sg), _dev(wq), u=None if u is None else _dev(u),
                         bm=None if bm is None else _dev(bm), lora_scale=1.0 if rank else 0.0)
    ref = ops.gemm_w8a8(_dev(gq), _dev(sg), _dev(wq.t().contiguous()), None, None, u=None if u is None else _dev(u),
                        bm=None if bm is None else _dev(bm), lora_scale=1.0 if rank else 0.0)
    ops.check_status()
    assert torch.equal(out, ref)
    if not rank:
        exact = (R.int_matmul(gq, wq.t().contiguous()).float() * sg.reshape(-1, 1)).to(torch.bfloat16)
        assert torch.equal(out.cpu().view(torch.int16), exact.view(torch.int16))
    with pytest.raises(ValueError, match="multiple of 128"):
        ops.gemm_dx_w8(_dev(gq[:, :64].contiguous()), _dev(sg), _dev(wq[:64].contiguous()))


def test_transpose_i8(ops):
    q = torch.randint(-127, 128, (272, 1536), dtype=torch.int8)
    assert torch.equal(ops.transpose_i8(_dev(q)).cpu(), q.t().contiguous())


# ------------------------------------------------------------------------------------------------
# argument validation through the C ABI
# ------------------------------------------------------------------------------------------------
def test_bad_arguments_raise(ops):
    with pytest.raises(ValueError):
        ops.fwht_quant_act(torch.zeros(4, 100, dtype=torch.bfloat16, device="cuda"))     # K % 128
    with pytest.raises(RuntimeError):
        ops.fwht_quant_act(torch.zeros(4, 128, dtype=torch.bfloat16))                    # CPU tensor
    xq = torch.zeros(8, 128, dtype=torch.int8, device="cuda")
    wq = torch.zeros(24, 128, dtype=torch.int8, device="cuda")                           # N % 16
    with pytest.raises(ValueError):
        ops.gemm_w8a8(xq, None, wq, None)


# ------------------------------------------------------------------------------------------------
# bounded waits: the path an expired wait takes, walked without hanging or faulting anything
# ------------------------------------------------------------------------------------------------
def test_status_block_written_from_the_host_is_decoded_and_cleared(ops):
    dev = torch.device("cuda", torch.cuda.current_device())
    ops.check_status(dev)
    blk = ops.status_block(dev)
    blk.copy_(torch.tensor([207, 33, 5, 0], dtype=torch.int32))       # wait id, CTA, detail as a kernel would leave them
    with pytest.raises(RuntimeError, match=r"wait id 207, CTA 33, detail 5"):
        ops.check_status(dev)
    assert int(blk.abs().sum()) == 0                                    # cleared by the raise
    ops.step_check(dev)                                                 # and quiet again


def test_expired_device_wait_reports_and_leaves_the_context_usable(ops):
    """A warp waits a few microseconds on a barrier nobody signals: the wait gives up, the status
    block names it, K2Q_ETIMEOUT comes back, and the next GEMM is still bit-exact."""
    import ctypes as C
    from k2q import _lib
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    blk = ops.status_block(dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.k2q_selftest_wait_expiry(C.c_void_p(blk.data_ptr()), 42, stream) == 0
    rc = lib.k2q_check_status(C.c_void_p(blk.data_ptr()), stream)
    assert rc == _lib.K2Q_ETIMEOUT and b"wait id 901" in lib.k2q_last_error() and b"detail 42" in lib.k2q_last_error()
    with pytest.raises(RuntimeError, match="wait id 901"):
        ops.check_status(dev)
    x, w, xq, sx, wq, sw, b = _int8_problem(128, 256, 256, seed=1)
    y = ops.gemm_w8a8(_dev(xq), _dev(sx), _dev(wq), _dev(sw), _dev(b))
    ops.check_status(dev)
    assert torch.equal(y.cpu().view(torch.int16), R.linear_int8_exact(xq, sx, wq, sw, b).view(torch.int16))


# ------------------------------------------------------------------------------------------------
# K2 with the step in front of the Linear folded in (mmdit.py:158-160, 178, 210, 313-317)
# ------------------------------------------------------------------------------------------------
def _codes_close(xq, sx, ref_rows, exact):
    q_ref, s_ref = R.quantize_act_int8(ref_rows)
    s_ref = s_ref.reshape(-1)
    if exact:
        assert torch.equal(xq.cpu(), q_ref) and torch.equal(sx.cpu(), s_ref)
        return
    # fp32 statistics summed in another order than torch's kernel: a code may move by one step
    assert float(((sx.cpu() - s_ref).abs() / s_ref).max()) <= 1e-4
    d = (xq.cpu().int() - q_ref.int()).abs()
    assert int(d.max()) <= 1 and float((d == 0).float().mean()) >= 0.999


@pytest.mark.parametrize("b,l,k", [(2, 100, 512), (1, 300, 6144), (3, 64, 16384), (1, 1, 128)])
def test_fused_prologues_match_the_composed_reference_ops(ops, b, l, k):
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(k + l)
    x = torch.randn(b, l, k, generator=g).to(torch.bfloat16)
    u = torch.randn(b, l, k, generator=g).to(torch.bfloat16)
    xq, sx = ops.swiglu_quant(_dev(x), _dev(u))                       # F.silu(gate(x)) * up(x), mmdit.py:178
    _codes_close(xq, sx, (F.silu(x) * u).reshape(-1, k), exact=True)
    xq, sx = ops.gate_quant(_dev(x), _dev(u))                         # attention * sigmoid(gate), mmdit.py:210
    _codes_close(xq, sx, (x * torch.sigmoid(u)).reshape(-1, k), exact=True)
    w = torch.randn(k, generator=g) * 0.1
    sc = (torch.randn(b, 1, k, generator=g) * 0.1).to(torch.bfloat16)
    sh = (torch.randn(b, 1, k, generator=g) * 0.1).to(torch.bfloat16)
    x3 = (x * 3).to(torch.bfloat16)
    normed = F.rms_norm(x3.float(), (k,), weight=w + 1.0, eps=1e-5).to(torch.bfloat16)       # mmdit.py:158-160
    xq, sx = ops.norm_mod_quant(_dev(x3), _dev(w), _dev(sc), _dev(sh))
    _codes_close(xq, sx, ((1 + sc) * normed + sh).reshape(-1, k), exact=False)            # mmdit.py:313-317
    xq, sx = ops.norm_mod_quant(_dev(x3), _dev(w))
    _codes_close(xq, sx, normed.reshape(-1, k), exact=False)
    with pytest.raises(ValueError):
        ops.swiglu_quant(_dev(x), _dev(u[:, :, :k // 2].contiguous()))


def test_requant_i4_to_i8_matches_host_restatement():
    """k2q_requant_i4_to_i8 against oracle.requant_int4_to_int8: codes and scales bit for bit, ragged row
    counts, a padded output (ldw8 > K), an all-zero row."""
    from k2q import ops
    for n, k in [(16, 128), (100, 384), (257, 3072), (48, 16384)]:
        w = R.synth_weight(n, k, seed=700 + n)
        w[n // 2] = 0
        q4, s4 = R.quantize_weight_int4(w)
        ref8, refs = R.requant_int4_to_int8(q4, s4)
        got8, gots = ops.requant_i4_to_i8(q4.cuda(), s4.cuda())
        assert torch.equal(got8.cpu(), ref8), (n, k)
        assert torch.equal(gots.cpu().view(torch.int32), refs.view(torch.int32)), (n, k)
        wide = torch.full((n, k + 32), 99, dtype=torch.int8, device="cuda")
        ops.requant_i4_to_i8(q4.cuda(), s4.cuda(), out=wide[:, :k])
        assert torch.equal(wide[:, :k].cpu(), ref8) and int((wide[:, k:] != 99).sum()) == 0
    with pytest.raises(ValueError):
        ops.requant_i4_to_i8(torch.zeros(4, 64, dtype=torch.int8, device="cuda"), torch.zeros(4, 1, dtype=torch.bfloat16, device="cuda"))


def test_qknorm_rope_matches_the_composed_ops():
    """k2q_qknorm_rope (in place, q and k as column blocks of one wider GEMM result) against the
    harness's op-by-op QKNorm + rope_rotate (the restatement of mmdit.py:135-141 and :25-31 that
    tests/golden/ref_dit_tiny.pt pins): the same bf16 values except where the fp32 mean of squares,
    summed in another order, moves a result across a rounding boundary (one bf16 step)."""
    from k2q import dit as ditmod
    from k2q import ops
    torch.manual_seed(5)
    b, s, hq, hk, d = 2, 173, 3, 1, 128
    wide = torch.randn(b * s, (hq + hk) * d + 256, device="cuda").to(torch.bfloat16)
    wide[7] = 0                                                    # an all-zero token: rsqrt(eps), zeros out
    q, k = wide[:, :hq * d], wide[:, hq * d:(hq + hk) * d]
    tail = wide[:, (hq + hk) * d:].clone()
    norm = ditmod.QKNorm(d).cuda()
    norm.qnorm.scale.data.normal_(0, 0.2)
    norm.knorm.scale.data.normal_(0, 0.2)
    pos = torch.stack((torch.zeros(s), torch.arange(s) // 16, torch.arange(s) % 16), dim=-1)[None].expand(b, -1, -1).cuda()
    cos, sin = ditmod.rope_tables(pos, [32, 48, 48], 100.0)
    for rope in ((cos, sin), None):
        q0, k0 = q.clone(), k.clone()
        qr, kr = norm(q0.view(b, s, hq, d).transpose(1, 2), k0.view(b, s, hk, d).transpose(1, 2))
        if rope is not None:
            qr, kr = ditmod.rope_rotate(qr, *rope), ditmod.rope_rotate(kr, *rope)
        qg, kg = q.clone(), k.clone()
        wq_, wk_ = qg.clone(), kg.clone()     # contiguous copies too
        ops.qknorm_rope_(wq_, wk_, norm.qnorm.scale.data, norm.knorm.scale.data,
                         None if rope is None else cos.reshape(b * s, d // 2), None if rope is None else sin.reshape(b * s, d // 2))
        for got, ref, h in ((wq_, qr, hq), (wk_, kr, hk)):
            ref2 = ref.transpose(1, 2).reshape(b * s, h * d).float()
            g2 = got.float()
            assert torch.isfinite(g2).all()
            step = ref2.abs().clamp_min(2.0 ** -120) * 2.0 ** -7          # one bf16 step at the value's size
            assert bool(((g2 - ref2).abs() <= step).all())
            assert float((g2 == ref2).float().mean()) >= 0.99
    # in place on strided column blocks: the neighbouring columns stay as they were
    wq_, wk_ = q.clone(), k.clone()
    ops.qknorm_rope_(wq_, wk_, norm.qnorm.scale.data, norm.knorm.scale.data, cos.reshape(b * s, d // 2), sin.reshape(b * s, d // 2))
    ops.qknorm_rope_(q, k, norm.qnorm.scale.data, norm.knorm.scale.data, cos.reshape(b * s, d // 2), sin.reshape(b * s, d // 2))
    assert torch.equal(q, wq_) and torch.equal(k, wk_) and torch.equal(wide[:, (hq + hk) * d:], tail)
    with pytest.raises(ValueError):
        ops.qknorm_rope_(q[:, :100], k, norm.qnorm.scale.data, norm.knorm.scale.data)
