/*
 * k2q.h -- C ABI of the B200 (sm_100a) rotated-quant ("ConvRot") Linear path.
 *
 * Every entry point is `extern "C"`, takes raw device pointers, explicit sizes and
 * leading dimensions (in ELEMENTS) and a CUDA stream (`void*` = cudaStream_t, NULL =
 * legacy default stream).  Return value: 0 on success or a negative K2Q_E* code;
 * `k2q_last_error()` then holds a thread-local, human readable message.  No entry
 * point allocates or frees device memory (workspaces are passed in), none keeps a
 * device pointer after it returns, none throws, none aborts.  All of them may be
 * called from any host thread (PyTorch's autograd thread included).
 *
 * The reference project (RyukoMatoiFan/krea-2) has no FFI; its boundary is the Python
 * duck type in quantize.py / lora.py.  Each function below names the reference lines
 * whose work it takes over.
 *
 * Layout conventions
 *   weights   W   [N, K]  row-major (out_features x in_features), as nn.Linear.weight
 *   codes     q8  [N, K]  int8                        (per-out-channel scale  sw[N]    f32)
 *             q4  [N, K/2] uint8, low nibble = even k (group scale sw4[N, K/128] bf16)
 *   tokens    x   [M, K]  bf16 row-major,  xq [M, K] int8, sx[M] f32 per-token scale
 *   rotation  block-diagonal Sylvester-Hadamard, block 128 along K, orthonormal.
 *   K must be a multiple of 128, N a multiple of 16; M is arbitrary (>= 0).
 */
#ifndef K2Q_H_
#define K2Q_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define K2Q_VERSION 106

#define K2Q_OK 0
#define K2Q_EINVAL (-1)   /* bad shape / alignment / null pointer / unsupported rank  */
#define K2Q_EARCH (-2)    /* current device is not compute capability 10.x            */
#define K2Q_ECUDA (-3)    /* CUDA runtime / driver call or launch failed              */
#define K2Q_ETIMEOUT (-4) /* a bounded device-side wait expired (see k2q_check_status) */

/* element type tags for `*_dtype` arguments */
#define K2Q_BF16 0
#define K2Q_F32 1

/* activation fused into a GEMM epilogue */
#define K2Q_ACT_NONE 0
#define K2Q_ACT_GELU_TANH 1

int k2q_version(void);
const char* k2q_last_error(void);

/* Number of bytes of the device status block every GEMM call needs (zero it once). */
int64_t k2q_status_bytes(void);
/* Reads a status block back (synchronises `stream`); returns 0, or K2Q_ETIMEOUT with
 * the place of the expired wait in k2q_last_error().  Host logic only, no kernel. */
int k2q_check_status(const void* status_dev, void* stream);

/* ---- K1: offline weight rotation + quantisation -------------------------------------
 * Replaces Fp8Linear.__init__ (quantize.py:33-42): per-row absmax scale + cast, with the
 * block-128 Walsh-Hadamard rotation along K in front.  Codes and scales are bit-exact
 * with the CPU restatement the tests check against (quantize_weight_int8 / _int4).
 *   w        [N, ldw] bf16 or f32 (w_dtype)
 *   q        [N, K]   int8          scale [N]        f32   (s = max(amax,1e-8)/127)
 *   q4       [N, K/2] uint8 packed  scale4 [N,K/128] bf16  (s = max(amax_g,1e-8)/7,
 *            codes use the f32 scale, the stored scale is its bf16 rounding)          */
int k2q_quant_weight_i8(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw,
                        int8_t* q, float* scale, void* stream);
int k2q_quant_weight_i4(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw,
                        uint8_t* q4, void* scale4_bf16, void* stream);

/* ---- K2: online activation rotation + per-token int8 quantisation ---------------------
 * New work in front of F.linear (quantize.py:51): warp-shuffle FWHT fused with the
 * per-token absmax/int8 quantiser.  x [M, ldx] bf16 (or f32) -> xq [M, K] int8, sx [M].
 * Bit-exact with the CPU restatement (quantize_act_int8).                                 */
int k2q_fwht_quant_act_i8(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                          int8_t* xq, float* sx, void* stream);

/* The same transform as a streaming kernel for the common case -- contiguous bf16 rows (ldx == K) with K a
 * multiple of 1024 up to 24576: whole rows are requested by TMA into a shared-memory ring by a producer
 * thread, a team of K/1024 warps works on each row, codes leave by TMA stores.  Same codes and scales, bit
 * for bit.  k2q_fwht_quant_act_i8_stream_ok() answers 1 when a problem qualifies.  The kernel's waits are
 * bounded, hence the status block (as for the GEMMs).                                                    */
int k2q_fwht_quant_act_i8_stream_ok(int x_dtype, int64_t M, int64_t K, int64_t ldx);
int k2q_fwht_quant_act_i8_stream(const void* x_bf16, int64_t M, int64_t K, int8_t* xq, float* sx, void* status,
                                 void* stream);

/* K2 with the elementwise step in front of the quantised Linear folded into its load (the callers of
 * the path, mmdit.py:158-160, 178, 210, 313-317): each reads bf16 rows, applies the step with the
 * reference's bf16 rounding points, rotates and quantises, and writes only codes + per-token scales --
 * the intermediate bf16 tensor never reaches memory.  Outputs as k2q_fwht_quant_act_i8.
 *   swiglu    v = silu(g) * u                               (input of mlp.down)
 *   gate      v = attention * sigmoid(gate)                 (input of attn.wo)
 *   norm_mod  v = (1 + mod_scale[b]) * rmsnorm(x) * ... + mod_shift[b]: RMS norm over K in fp32 with
 *             weight 1 + norm_scale[K] (f32), then the block's modulation, b = row / rows_per_batch,
 *             mod_scale / mod_shift [B, K] bf16 or NULL (plain norm)    (input of wq|wk|wv|gate, mlp.gate|up) */
int k2q_swiglu_fwht_quant(const void* g_bf16, int64_t ldg, const void* u_bf16, int64_t ldu, int64_t M,
                          int64_t K, int8_t* xq, float* sx, void* stream);
int k2q_gate_fwht_quant(const void* attn_bf16, int64_t lda, const void* gate_bf16, int64_t ldg, int64_t M,
                        int64_t K, int8_t* xq, float* sx, void* stream);
int k2q_norm_mod_fwht_quant(const void* x_bf16, int64_t ldx, int64_t M, int64_t K, const float* norm_scale,
                            const void* mod_scale_bf16, const void* mod_shift_bf16, int64_t rows_per_batch,
                            float eps, int8_t* xq, float* sx, void* stream);

/* QK-RMSNorm + rotary embedding of the q and k projections, in place, head dimension 128
 * (mmdit.py:135-141 QKNorm, :25-31 ropeapply, as Attention.forward :199-208 applies them between the
 * projections and the attention call).  q [T, ldq] bf16 with heads_q * 128 used columns, k likewise;
 * wq / wk [128] f32 (norm weight = 1 + w); cos_t / sin_t [T, 64] f32 (NULL: norm only); the bf16
 * rounding points of the reference's two steps are kept (norm output rounded before the rotation). */
int k2q_qknorm_rope(void* q_bf16, int64_t ldq, int heads_q, const float* wq,
                    void* k_bf16, int64_t ldk, int heads_k, const float* wk, int64_t T,
                    const float* cos_t, const float* sin_t, float eps, void* stream);

/* ---- the elementwise steps of a DiT block between the quantised Linears, forward and backward ----
 * One kernel per step and direction for TRAINING (the fused quantisation prologues above serve
 * inference, where no dense tensor is needed in between): in eager model code each step is a chain of
 * casts, norms, multiplies and adds with a bf16 rounding after every op.  bf16 rows with row strides
 * (multiples of 8 elements, 16-byte aligned bases); forward values keep the reference's bf16 rounding
 * points, gradients are computed in fp32 from the saved inputs and rounded once.
 *   norm_mod      y = (1 + sc_b) * rmsnorm(x) * ... + sh_b, b = row / rows_per_batch   mmdit.py:158-160, 313-317
 *                 (fwd also returns rstd [M]; bwd gives dx; K <= 8192)
 *   qknorm_rope   out-of-place form of k2q_qknorm_rope and its backward; the upstream gradients are read
 *                 as (b, s, h, d) tensors through element strides (what the attention backward returns)
 *   swiglu        h = silu(g) * u            mmdit.py:178       sigmoid_gate  y = a * sigmoid(g)   mmdit.py:210
 *   gate_residual out = x + gate_b * y       mmdit.py:318-321   (x NULL: gate_b * y, the step's backward)   */
int k2q_norm_mod_fwd(const void* x_bf16, int64_t ldx, int64_t M, int64_t K, const float* norm_scale,
                     const void* mod_scale_bf16, const void* mod_shift_bf16, int64_t rows_per_batch, float eps,
                     void* y_bf16, int64_t ldy, float* rstd, void* stream);
int k2q_norm_mod_bwd(const void* dy_bf16, int64_t lddy, const void* x_bf16, int64_t ldx, const float* rstd, int64_t M,
                     int64_t K, const float* norm_scale, const void* mod_scale_bf16, int64_t rows_per_batch,
                     void* dx_bf16, int64_t lddx, void* stream);
int k2q_qknorm_rope_fwd(const void* q_bf16, int64_t ldq, int heads_q, const float* wq, void* qo_bf16, int64_t ldqo,
                        const void* k_bf16, int64_t ldk, int heads_k, const float* wk, void* ko_bf16, int64_t ldko,
                        int64_t T, const float* cos_t, const float* sin_t, float eps, void* stream);
int k2q_qknorm_rope_bwd(const void* q_bf16, int64_t ldq, int heads_q, const float* wq, const void* dqo_bf16,
                        int64_t dq_sb, int64_t dq_ss, int64_t dq_sh, void* dq_bf16, int64_t lddq,
                        const void* k_bf16, int64_t ldk, int heads_k, const float* wk, const void* dko_bf16,
                        int64_t dk_sb, int64_t dk_ss, int64_t dk_sh, void* dk_bf16, int64_t lddk,
                        int64_t B, int64_t S, const float* cos_t, const float* sin_t, float eps, void* stream);
int k2q_swiglu_fwd(const void* g, int64_t ldg, const void* u, int64_t ldu, int64_t M, int64_t K, void* h, int64_t ldh,
                   void* stream);
int k2q_swiglu_bwd(const void* dh, int64_t lddh, const void* g, int64_t ldg, const void* u, int64_t ldu, int64_t M,
                   int64_t K, void* dg, int64_t lddg, void* du, int64_t lddu, void* stream);
int k2q_sigmoid_gate_fwd(const void* a, int64_t lda, const void* g, int64_t ldg, int64_t M, int64_t K, void* y,
                         int64_t ldy, void* stream);
int k2q_sigmoid_gate_bwd(const void* dy, int64_t lddy, const void* a, int64_t lda, const void* g, int64_t ldg, int64_t M,
                         int64_t K, void* da, int64_t ldda, void* dg, int64_t lddg, void* stream);
int k2q_gate_residual(const void* x_or_null, int64_t ldx, const void* y, int64_t ldy, const void* gate_bk,
                      int64_t rows_per_batch, int64_t M, int64_t K, void* out, int64_t ldo, void* stream);

/* Per-token int8 quantisation WITHOUT rotation of g[m,n] * colscale[n] (colscale may be
 * NULL).  Used by the backward (autograd of quantize.py:51): dY is folded with the
 * per-out-channel weight scale, which sits on the contraction index of dX = dY.W.      */
int k2q_quant_rows_i8(const void* g, int g_dtype, int64_t M, int64_t N, int64_t ldg,
                      const float* colscale, int8_t* gq, float* sg, void* stream);

/* Block-128 FWHT of every row, no quantisation: y = H(x).  in/out bf16 or f32 (same
 * shape [M, K]); in-place allowed when dtypes match.  Used to de-rotate dX and to
 * rotate the LoRA A matrix for the backward epilogue.                                   */
int k2q_fwht_rows(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                  void* y, int y_dtype, int64_t ldy, void* stream);

/* ---- K3/K4: W8A8 and W4A8 GEMMs on tcgen05 int8 tensor cores ---------------------------
 * Replace Fp8Linear.forward (quantize.py:48-51: dequantise the whole weight, F.linear)
 * and the adapter term of LoRALinear.forward (lora.py:47-48) with one kernel:
 *   y[m,n] = act( acc[m,n]*sx[m]*sw[n] + bias[n] ) + lora_scale * sum_j u[m,j]*Bm[n,j]
 * acc is the exact int32 dot product of codes (W4A8: sum over K-groups of acc_g*sw4[n,g]).
 * `act` is applied before the adapter term (the reference never combines both).
 *   xq [M,K] int8, sx [M] f32 (NULL = 1), wq [N,K] int8, sw [N] f32 (NULL = 1)
 *   bias [N] f32 or NULL;  u [M, ldu] f32 and Bm [N, ldb] f32 with rank <= 64, or both NULL
 *   y [M, ldy] bf16.  `status` = device block of k2q_status_bytes() bytes (zeroed by the
 *   caller once); a bounded in-kernel wait that expires records its place there.       */
typedef struct k2q_epilogue {
  const float* sx;      /* [M] per-token scale, or NULL                       */
  const float* bias;    /* [N] or NULL                                         */
  const float* u;       /* [M, ldu] LoRA down-projection x.A^T, or NULL        */
  const float* Bm;      /* [N, ldb] LoRA up matrix, or NULL                    */
  int64_t ldu, ldb;
  int32_t rank;         /* 0 when u/Bm are NULL                                */
  float lora_scale;     /* (alpha/rank) * scale_mul; may be negative or zero   */
  int32_t act;          /* K2Q_ACT_*                                           */
} k2q_epilogue;

int k2q_gemm_w8a8(const int8_t* xq, const int8_t* wq, const float* sw, int64_t M, int64_t N,
                  int64_t K, const k2q_epilogue* ep, void* y_bf16, int64_t ldy, void* status,
                  void* stream);
int k2q_gemm_w4a8(const int8_t* xq, const uint8_t* wq4, const void* sw4_bf16, int64_t M,
                  int64_t N, int64_t K, const k2q_epilogue* ep, void* y_bf16, int64_t ldy,
                  void* status, void* stream);

/* Backward of K3 through the SAME stored codes (autograd of quantize.py:51, dX = dY . w):
 *   dx[m,k] = acc[m,k]*sx[m] + lora_scale * sum_j u[m,j]*Bm[k,j],   acc = sum_n gq[m,n]*wq[n,k]
 * gq [M, N] int8 = per-token quantised dY*sw (k2q_quant_rows_i8, scale in ep->sx), wq [N, K] int8 exactly
 * as the forward uses it: the tensor core reads it as an MN-major operand, no transposed copy of the
 * weights exists.  N (the contraction) must be a multiple of 128, K of 16; the result is still in the
 * rotated basis (k2q_fwht_rows de-rotates it).  ep->u = du [M, r], ep->Bm = H(A)^T [K, r] add the
 * adapter's share of dX; ep->bias / ep->act are normally unset.                                  */
int k2q_gemm_dx_w8(const int8_t* gq, const int8_t* wq, int64_t M, int64_t N, int64_t K,
                   const k2q_epilogue* ep, void* dx_bf16, int64_t lddx, void* status, void* stream);

/* A group-128 int4 base re-expressed against ONE scale per output channel, for the backward of a
 * 4-bit base (an int4 group scale sits on both indices of dX's contraction) and for its optional
 * int8-rate forward:   scale8[n] = max_g scale4[n,g] * 7/127,
 *                      w8[n,k]   = rint(q4[n,k] * (scale4[n,k/128] / scale8[n])),  |w8| <= 127
 * (fp32 division, multiplication, round-half-even: a host restatement gives the same codes).  No
 * counterpart in the reference, whose Fp8Linear dequantises to bf16 for both directions
 * (quantize.py:48-51).  w8 [N, ldw8] int8 with ldw8 >= K a multiple of 16; q4 and w8 16-byte aligned. */
int k2q_requant_i4_to_i8(const uint8_t* q4, const void* scale4_bf16, int64_t N, int64_t K,
                         int8_t* w8, int64_t ldw8, float* scale8, void* stream);

/* int8 [R, C] -> int8 [C, R] transpose (builds the [K, N] copy of the codes that the
 * backward GEMM dX = dYq . Wq contracts over N with; done once per layer).              */
int k2q_transpose_i8(const int8_t* src, int64_t R, int64_t C, int8_t* dst, void* stream);

/* ---- K5/K7: LoRA skinny GEMMs ---------------------------------------------------------
 * K5 replaces `x.to(f32) @ A.t()` (lora.py:47) and autograd's du = s*dY.B:
 *   out[M, r] = scale * X[M, K](bf16) . A[r, K]^T      A given as f32 with element strides
 *   (a_rs, a_cs): A[j,k] = a[j*a_rs + k*a_cs], so B[N,r] can be passed as its transpose.
 * K7 replaces autograd of lora.py:47-48 for the adapter weights:
 *   out[r, C] = scale * P[T, r]^T (f32) . Q[T, C] (bf16)           (dA = du^T x, dB^T = u^T dY)
 *   ws = workspace of k2q_lora_tn_workspace_bytes(T, r, C) bytes (split-T partial sums,
 *   reduced in a fixed order, so results are run-to-run identical).                    */
int k2q_lora_down(const void* x_bf16, int64_t M, int64_t K, int64_t ldx, const float* a,
                  int64_t a_rs, int64_t a_cs, int32_t r, float scale, float* out, int64_t ldo,
                  void* stream);
int64_t k2q_lora_tn_workspace_bytes(int64_t T, int32_t r, int64_t C);
int k2q_lora_tn(const float* p, int64_t ldp, const void* q_bf16, int64_t ldq, int64_t T,
                int32_t r, int64_t C, float scale, float* out, int64_t ldo, void* ws,
                int64_t ws_bytes, void* stream);

/* ---- K7 without a workspace (no counterpart in the reference) -------------------------------
 * Same result as k2q_lora_tn, for callers that must not allocate device memory and therefore
 * cannot supply a workspace: code running under a host that hands out a fixed set of buffers, or
 * a latency-critical loop where a device allocation (which may synchronise the whole GPU) is not
 * acceptable.  The split-T partial sums go to a 16 MiB array built into the library image
 * (k2q_lora_tn_static_max_bytes()); each GPU that loads the library holds that array until exit.
 *   - problems whose partial sums exceed the array are refused with K2Q_EINVAL
 *     (need = k2q_lora_tn_workspace_bytes(T, r, C));
 *   - the first call on a device looks up the array's device address (a host-side query, no
 *     allocation); make that first call outside any stream capture;
 *   - all calls on a device share the one array, which keeps the last call's partial sums: every
 *     value the reduction reads is rewritten by the same call, so nothing needs clearing, but two
 *     calls that overlap on the GPU (different streams) race -- serialise them;
 *   - no cudaMalloc / cudaFree or other allocating routine is called.                          */
int64_t k2q_lora_tn_static_max_bytes(void);
int k2q_lora_tn_static(const float* p, int64_t ldp, const void* q_bf16, int64_t ldq, int64_t T,
                       int32_t r, int64_t C, float scale, float* out, int64_t ldo, void* stream);

/* ---- the MLP pair over HOST buffers (no counterpart in the reference, whose modules take device tensors;
 * the call stands where a host program hands tokens to Sequential(Linear, GELU(tanh), Linear) of two
 * quantised bases, mmdit.py:360-375 over quantize.py:48-51, and wants the result back in host memory) ---
 *   y_host[M, fc2.N] = fc2( gelu_tanh( fc1( x_host[M, fc1.K] ) ) ),  bf16 rows, both buffers in (ideally
 *   page-locked) host memory; each Linear = K2 + K3/K4 exactly as the device entry points compute it.
 * The rows are cut into n_chunks pieces of chunk_rows[i] rows (positive, adding up to M); the copy-in of
 * piece i+1, the kernels of piece i and the copy-out of piece i-1 overlap on `copy_in_stream`, `stream` and
 * `copy_out_stream` (three distinct streams of the current device, made by the caller).  The copies start
 * after the work `stream` holds at the time of the call, and `stream` waits for the last copy before
 * anything enqueued on it later: y_host is complete when `stream` is.  Short first and last pieces keep
 * the part that cannot overlap small.  `workspace` (256-byte aligned device memory of
 * k2q_mlp_gelu_host_workspace_bytes(M, fc1.K, fc1.N, fc2.N, max_i chunk_rows[i]) bytes) holds the tokens,
 * the result and one piece's intermediates; nothing is allocated on the device.  The events that order
 * the streams are host objects created on first use, per host thread and device, and kept.       */
typedef struct k2q_linear {
  int32_t bits;          /* 8: codes int8 [N, K], scale f32 [N];  4: codes uint8 [N, K/2], scale bf16 [N, K/128] */
  int32_t pad_;
  const void* codes;
  const void* scale;
  const float* bias;     /* [N] or NULL */
  int64_t N, K;
} k2q_linear;

int64_t k2q_mlp_gelu_host_workspace_bytes(int64_t M, int64_t K, int64_t H, int64_t N2, int64_t max_rows);
int k2q_mlp_gelu_host(const void* x_host_bf16, int64_t M, const k2q_linear* fc1, const k2q_linear* fc2,
                      void* y_host_bf16, const int64_t* chunk_rows, int n_chunks, void* workspace,
                      int64_t workspace_bytes, void* status, void* stream, void* copy_in_stream,
                      void* copy_out_stream);

/* ---- calibration helper (no counterpart in the reference) ----------------------------------
 * Runs back-to-back tcgen05.mma kind::i8 (M128 N256 K32) on every SM from operands that stay in
 * shared memory and returns the rate in TOP/s: the practical int8 tensor ceiling of this GPU
 * at its present clocks.  Synchronises `stream`.  `iters` = K-blocks of 4 MMAs per SM.        */
int k2q_measure_i8_peak(int iters, void* status, double* tops_out, void* stream);

/* ---- optimizer step of the adapters (train_t2i_lora_cached.py:327-332) ------------------------------
 * clip_grad_norm_ + AdamW.step + zero_grad over flat fp32 buffers (parameters, gradients, moments of all
 * adapters laid end to end).  k2q_sumsq_f32 leaves sum(g^2) in out[0] (a device scalar; accumulate != 0
 * adds to what is there: several gradient buffers) using a workspace of k2q_sumsq_workspace_bytes();
 * the sum is formed in a fixed order.  k2q_adamw_clip_f32 applies the update rule of torch.optim.AdamW
 * for step number `step` (1-based) with every gradient first scaled by min(1, max_norm / (sqrt(*normsq_dev)
 * + 1e-6)) (max_norm <= 0 or normsq_dev NULL: no clipping) and zeroes g when zero_grad != 0.          */
int64_t k2q_sumsq_workspace_bytes(void);
int k2q_sumsq_f32(const float* g, int64_t n, float* out, int accumulate, void* ws, int64_t ws_bytes, void* stream);
int k2q_adamw_clip_f32(float* p, float* g, float* m, float* v, int64_t n, float lr, float beta1, float beta2,
                       float eps, float weight_decay, int64_t step, float max_norm, const float* normsq_dev,
                       int zero_grad, void* stream);

/* ---- self-test of the bounded waits (no counterpart in the reference) ------------------------
 * Launches one warp that waits, with a limit of a few microseconds, on a barrier nobody signals.
 * The wait expires, the kernel writes wait id 901 and `detail` to `status` and returns normally; a
 * following k2q_check_status(status) must answer K2Q_ETIMEOUT.  Used by the tests to walk the path
 * an expired wait takes in the GEMM kernels without hanging or faulting anything.               */
int k2q_selftest_wait_expiry(void* status, int detail, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* K2Q_H_ */
