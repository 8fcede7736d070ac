// The MLP pair K2 -> GEMM(+GELU) -> K2 -> GEMM for callers whose tokens live in HOST memory.
//
// Tokens are cut into row chunks; the host-to-device copy of chunk i+1, the four kernels of chunk i
// and the device-to-host copy of chunk i-1 run on three streams at once.  Everything is enqueued by
// this one call (a few microseconds per chunk), so the chunks can be small enough that the call costs
// little more than the slower of "both copies over PCIe at once" and "the kernels": the first chunk's
// copy-in and the last chunk's kernels + copy-out are all that is not overlapped, which is why the
// caller may give the chunks different sizes (short first and last chunks, long ones between).
//
// No device memory is allocated here: inputs, outputs and intermediates live in the caller's
// workspace.  The whole input and output have room there (no buffer is reused while a copy may still
// read or write it); the per-chunk intermediates are used by one stream only, in order.  The events
// that order the three streams are host objects, created once per host thread and device and reused.
#include <vector>

#include "k2q_common.cuh"

namespace k2q {
namespace {

constexpr size_t kAlign = 256;
size_t round_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

struct Layout {
  size_t x, y, xq, sx, h, hq, sh, total;
};

Layout layout(int64_t M, int64_t K, int64_t H, int64_t N2, int64_t max_rows) {
  Layout l;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += round_up(bytes);
    return at;
  };
  l.x = take(static_cast<size_t>(M) * K * 2);
  l.y = take(static_cast<size_t>(M) * N2 * 2);
  l.xq = take(static_cast<size_t>(max_rows) * K);
  l.sx = take(static_cast<size_t>(max_rows) * 4);
  l.h = take(static_cast<size_t>(max_rows) * H * 2);
  l.hq = take(static_cast<size_t>(max_rows) * H);
  l.sh = take(static_cast<size_t>(max_rows) * 4);
  l.total = off;
  return l;
}

// Events of this host thread for the current device: 2 per chunk + 2.
int events_for(int count, cudaEvent_t** out) {
  thread_local std::vector<cudaEvent_t> pool[64];
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= 64) return fail(K2Q_EINVAL, "device index %d out of range", dev);
  std::vector<cudaEvent_t>& p = pool[dev];
  while (static_cast<int>(p.size()) < count) {
    cudaEvent_t e;
    if (int rc = check_cuda(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreateWithFlags")) return rc;
    p.push_back(e);
  }
  *out = p.data();
  return K2Q_OK;
}

int check_linear(const char* which, const k2q_linear* l) {
  if (!l) return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: %s is NULL", which);
  if (l->bits != 4 && l->bits != 8) return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: %s.bits = %d (4 or 8)", which, l->bits);
  if (!l->codes || !l->scale) return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: %s has no codes / scales", which);
  if (l->N <= 0 || l->K <= 0 || l->K % 128 != 0 || l->N % 16 != 0)
    return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: %s is [%lld, %lld]; K must be a multiple of 128, N of 16", which,
                (long long)l->N, (long long)l->K);
  return K2Q_OK;
}

int gemm(const k2q_linear* l, const int8_t* xq, const float* sx, int64_t rows, int act, void* y, void* status,
         cudaStream_t s) {
  k2q_epilogue ep;
  ep.sx = sx;
  ep.bias = l->bias;
  ep.u = nullptr;
  ep.Bm = nullptr;
  ep.ldu = ep.ldb = 0;
  ep.rank = 0;
  ep.lora_scale = 0.0f;
  ep.act = act;
  if (l->bits == 4)
    return k2q_gemm_w4a8(xq, static_cast<const uint8_t*>(l->codes), l->scale, rows, l->N, l->K, &ep, y, l->N, status, s);
  return k2q_gemm_w8a8(xq, static_cast<const int8_t*>(l->codes), static_cast<const float*>(l->scale), rows, l->N, l->K,
                       &ep, y, l->N, status, s);
}

// K2 of one piece: the streaming kernel when the rows qualify and are many enough for one persistent CTA per
// SM to beat the general row kernel's many small CTAs, that kernel otherwise
int k2(const void* x, int64_t rows, int64_t K, int8_t* xq, float* sx, void* status, cudaStream_t s) {
  if (rows * K >= (int64_t(8) << 20) && k2q_fwht_quant_act_i8_stream_ok(K2Q_BF16, rows, K, K)) return k2q_fwht_quant_act_i8_stream(x, rows, K, xq, sx, status, s);
  return k2q_fwht_quant_act_i8(x, K2Q_BF16, rows, K, K, xq, sx, s);
}

int64_t max_chunk(int64_t M, const int64_t* chunk_rows, int n_chunks) {
  int64_t mx = 0, sum = 0;
  for (int i = 0; i < n_chunks; ++i) {
    if (chunk_rows[i] <= 0) return -1;
    mx = chunk_rows[i] > mx ? chunk_rows[i] : mx;
    sum += chunk_rows[i];
  }
  return sum == M ? mx : -1;
}

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" int64_t k2q_mlp_gelu_host_workspace_bytes(int64_t M, int64_t K, int64_t H, int64_t N2, int64_t max_rows) {
  if (M < 0 || K <= 0 || H <= 0 || N2 <= 0 || max_rows < 0) return 0;
  return static_cast<int64_t>(layout(M, K, H, N2, max_rows).total);
}

extern "C" int k2q_mlp_gelu_host(const void* x_host_bf16, int64_t M, const k2q_linear* fc1, const k2q_linear* fc2,
                                 void* y_host_bf16, const int64_t* chunk_rows, int n_chunks, void* workspace,
                                 int64_t workspace_bytes, void* status, void* stream, void* copy_in_stream,
                                 void* copy_out_stream) {
  if (int rc = check_device_arch()) return rc;
  if (int rc = check_linear("fc1", fc1)) return rc;
  if (int rc = check_linear("fc2", fc2)) return rc;
  if (fc2->K != fc1->N)
    return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: fc2 takes %lld features, fc1 gives %lld", (long long)fc2->K, (long long)fc1->N);
  if (M < 0) return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: M = %lld", (long long)M);
  if (M == 0) return K2Q_OK;
  if (!x_host_bf16 || !y_host_bf16 || !workspace || !status)
    return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: NULL host buffer, workspace or status block");
  if (!copy_in_stream || !copy_out_stream || copy_in_stream == stream || copy_out_stream == stream ||
      copy_in_stream == copy_out_stream)
    return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: the two copy streams must be distinct streams other than the compute stream");
  if (!chunk_rows || n_chunks <= 0 || n_chunks > 4096)
    return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: no chunk schedule (n_chunks = %d)", n_chunks);
  const int64_t max_rows = max_chunk(M, chunk_rows, n_chunks);
  if (max_rows < 0) return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: chunk rows must be positive and add up to M = %lld", (long long)M);
  const int64_t K = fc1->K, H = fc1->N, N2 = fc2->N;
  const Layout l = layout(M, K, H, N2, max_rows);
  if (workspace_bytes < static_cast<int64_t>(l.total))
    return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: workspace of %lld bytes, %lld needed", (long long)workspace_bytes,
                (long long)l.total);
  if ((reinterpret_cast<uintptr_t>(workspace) & (kAlign - 1)) != 0)
    return fail(K2Q_EINVAL, "k2q_mlp_gelu_host: workspace must be 256-byte aligned");

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaStream_t s_in = static_cast<cudaStream_t>(copy_in_stream);
  cudaStream_t s_out = static_cast<cudaStream_t>(copy_out_stream);
  cudaEvent_t* ev = nullptr;
  if (int rc = events_for(2 * n_chunks + 2, &ev)) return rc;
  cudaEvent_t ev_start = ev[2 * n_chunks], ev_end = ev[2 * n_chunks + 1];

  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* x_dev = ws + l.x;
  uint8_t* y_dev = ws + l.y;
  int8_t* xq = reinterpret_cast<int8_t*>(ws + l.xq);
  float* sx = reinterpret_cast<float*>(ws + l.sx);
  uint8_t* h = ws + l.h;
  int8_t* hq = reinterpret_cast<int8_t*>(ws + l.hq);
  float* sh = reinterpret_cast<float*>(ws + l.sh);
  const uint8_t* xh = static_cast<const uint8_t*>(x_host_bf16);
  uint8_t* yh = static_cast<uint8_t*>(y_host_bf16);

  // the copies start after whatever the compute stream holds at this point (a consumer of y_host's
  // previous contents, the producer of x_host's)
  if (int rc = check_cuda(cudaEventRecord(ev_start, s), "cudaEventRecord")) return rc;
  if (int rc = check_cuda(cudaStreamWaitEvent(s_in, ev_start, 0), "cudaStreamWaitEvent")) return rc;
  if (int rc = check_cuda(cudaStreamWaitEvent(s_out, ev_start, 0), "cudaStreamWaitEvent")) return rc;

  int rc = K2Q_OK;
  int64_t a = 0;
  for (int i = 0; i < n_chunks && rc == K2Q_OK; ++i) {
    const int64_t rows = chunk_rows[i];
    const size_t xo = static_cast<size_t>(a) * K * 2, yo = static_cast<size_t>(a) * N2 * 2;
    rc = check_cuda(cudaMemcpyAsync(x_dev + xo, xh + xo, static_cast<size_t>(rows) * K * 2, cudaMemcpyHostToDevice, s_in),
                    "cudaMemcpyAsync(tokens to the device)");
    if (rc == K2Q_OK) rc = check_cuda(cudaEventRecord(ev[2 * i], s_in), "cudaEventRecord");
    if (rc == K2Q_OK) rc = check_cuda(cudaStreamWaitEvent(s, ev[2 * i], 0), "cudaStreamWaitEvent");
    if (rc == K2Q_OK) rc = k2(x_dev + xo, rows, K, xq, sx, status, s);
    if (rc == K2Q_OK) rc = gemm(fc1, xq, sx, rows, K2Q_ACT_GELU_TANH, h, status, s);
    if (rc == K2Q_OK) rc = k2(h, rows, H, hq, sh, status, s);
    if (rc == K2Q_OK) rc = gemm(fc2, hq, sh, rows, K2Q_ACT_NONE, y_dev + yo, status, s);
    if (rc == K2Q_OK) rc = check_cuda(cudaEventRecord(ev[2 * i + 1], s), "cudaEventRecord");
    if (rc == K2Q_OK) rc = check_cuda(cudaStreamWaitEvent(s_out, ev[2 * i + 1], 0), "cudaStreamWaitEvent");
    if (rc == K2Q_OK)
      rc = check_cuda(cudaMemcpyAsync(yh + yo, y_dev + yo, static_cast<size_t>(rows) * N2 * 2, cudaMemcpyDeviceToHost, s_out),
                      "cudaMemcpyAsync(result to the host)");
    a += rows;
  }
  // whatever happened, the compute stream rejoins both copy streams: the workspace may be reused,
  // and y_host is complete, when `stream` reaches this point
  cudaError_t e1 = cudaEventRecord(ev_end, s_out);
  if (e1 == cudaSuccess) e1 = cudaStreamWaitEvent(s, ev_end, 0);
  cudaError_t e2 = cudaEventRecord(ev_start, s_in);
  if (e2 == cudaSuccess) e2 = cudaStreamWaitEvent(s, ev_start, 0);
  if (rc != K2Q_OK) return rc;
  if (int r2 = check_cuda(e1, "joining the copy-out stream")) return r2;
  return check_cuda(e2, "joining the copy-in stream");
}
