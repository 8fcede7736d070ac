// Optimizer step of the adapter parameters (train_t2i_lora_cached.py:327-332: clip_grad_norm_, AdamW
// step, zero_grad) on ONE flat fp32 buffer each for parameters, gradients and the two moments:
//   sumsq   deterministic sum of squares of the gradients (per-block partial sums, then one block
//           adds them in index order): the global gradient norm without a host round trip
//   adamw   decoupled-weight-decay Adam (the update rule of torch.optim.AdamW) with the clipping
//           factor min(1, max_norm / (norm + 1e-6)) of clip_grad_norm_ folded into the gradient read,
//           and the gradient buffer zeroed on the way out (zero_grad)
// Both are HBM-bound streams: 4 B/element read for the norm, 16 B read + 16 B written for the update.
#include "k2q_common.cuh"

namespace k2q {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxPartials = 2048;

__global__ void __launch_bounds__(kThreads) sumsq_partial_kernel(const float* __restrict__ g, int64_t n, float* partials) {
  __shared__ float warp_sums[kThreads / 32];
  const int64_t n4 = n / 4;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  float acc = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x; i < n4; i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const float4 v = __ldg(g4 + i);
    acc = fmaf(v.x, v.x, acc);
    acc = fmaf(v.y, v.y, acc);
    acc = fmaf(v.z, v.z, acc);
    acc = fmaf(v.w, v.w, acc);
  }
  if (blockIdx.x == 0 && threadIdx.x < n - n4 * 4) {   // ragged tail
    const float v = g[n4 * 4 + threadIdx.x];
    acc = fmaf(v, v, acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < kThreads / 32; ++w) s += warp_sums[w];
    partials[blockIdx.x] = s;
  }
}

__global__ void __launch_bounds__(32) sumsq_final_kernel(const float* partials, int count, float* out, int accumulate) {
  if (threadIdx.x == 0) {
    float s = accumulate ? out[0] : 0.f;
    for (int i = 0; i < count; ++i) s += partials[i];   // fixed order: run-to-run identical
    out[0] = s;
  }
}

struct AdamParams {
  float* p; float* g; float* m; float* v;
  int64_t n;
  float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, max_norm;
  const float* normsq;   // device scalar or NULL (no clipping)
  int zero_grad;
};

__global__ void __launch_bounds__(kThreads) adamw_kernel(const AdamParams a) {
  float clip = 1.0f;
  if (a.normsq != nullptr && a.max_norm > 0.f) {
    const float norm = sqrtf(__ldg(a.normsq));
    clip = fminf(1.0f, a.max_norm / (norm + 1e-6f));        // torch.nn.utils.clip_grad_norm_
  }
  const float decay = 1.0f - a.lr * a.wd;
  const float step = a.lr / a.bc1;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x; i < a.n; i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const float g = a.g[i] * clip;
    float p = a.p[i] * decay;                               // decoupled weight decay
    const float m = a.beta1 * a.m[i] + (1.0f - a.beta1) * g;
    const float v = a.beta2 * a.v[i] + (1.0f - a.beta2) * g * g;
    const float denom = sqrtf(v) / a.bc2_sqrt + a.eps;
    p -= step * (m / denom);
    a.p[i] = p; a.m[i] = m; a.v[i] = v;
    if (a.zero_grad) a.g[i] = 0.f;
  }
}

}  // namespace
}  // namespace k2q

using namespace k2q;

extern "C" {

int64_t k2q_sumsq_workspace_bytes(void) { return kMaxPartials * (int64_t)sizeof(float); }

int k2q_sumsq_f32(const float* g, int64_t n, float* out, int accumulate, void* ws, int64_t ws_bytes, void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (n < 0 || !out) return fail(K2Q_EINVAL, "k2q_sumsq_f32: bad arguments");
  if (!ws || ws_bytes < k2q_sumsq_workspace_bytes()) return fail(K2Q_EINVAL, "k2q_sumsq_f32: workspace too small");
  if (n > 0 && (!g || (reinterpret_cast<uintptr_t>(g) & 15u))) return fail(K2Q_EINVAL, "k2q_sumsq_f32: g must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int sms = sm_count() > 0 ? sm_count() : 148;
  int64_t blocks = (n / 4 + kThreads - 1) / kThreads;
  if (blocks > 8LL * sms) blocks = 8LL * sms;
  if (blocks > kMaxPartials) blocks = kMaxPartials;
  if (blocks < 1) blocks = 1;
  sumsq_partial_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(g, n, static_cast<float*>(ws));
  sumsq_final_kernel<<<1, 32, 0, s>>>(static_cast<const float*>(ws), static_cast<int>(blocks), out, accumulate);
  return check_cuda(cudaGetLastError(), "sumsq launch");
}

int k2q_adamw_clip_f32(float* p, float* g, float* m, float* v, int64_t n, float lr, float beta1, float beta2, float eps,
                       float weight_decay, int64_t step, float max_norm, const float* normsq_dev, int zero_grad,
                       void* stream) {
  if (int rc = check_device_arch()) return rc;
  if (n < 0 || step < 1) return fail(K2Q_EINVAL, "k2q_adamw_clip_f32: bad n or step");
  if (n == 0) return K2Q_OK;
  if (!p || !g || !m || !v) return fail(K2Q_EINVAL, "k2q_adamw_clip_f32: NULL operand");
  AdamParams a{};
  a.p = p; a.g = g; a.m = m; a.v = v; a.n = n;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = weight_decay;
  a.bc1 = 1.0f - powf(beta1, static_cast<float>(step));
  a.bc2_sqrt = sqrtf(1.0f - powf(beta2, static_cast<float>(step)));
  a.max_norm = max_norm; a.normsq = normsq_dev; a.zero_grad = zero_grad;
  const int sms = sm_count() > 0 ? sm_count() : 148;
  int64_t blocks = (n + kThreads - 1) / kThreads;
  if (blocks > 16LL * sms) blocks = 16LL * sms;
  adamw_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_cuda(cudaGetLastError(), "adamw launch");
}

}  // extern "C"
