// layer_norm.cu — the f32 residual stream of architectures whose layers read ONE normalised copy of the stream and add
// several branch outputs back (parallel blocks):
//   nvllm_residual_layernorm:  h += s0 a0 + s1 a1 + s2 a2 + sb bias;   out = (h - mean) / sqrt(var + eps) * w
//   nvllm_concat_cast:         out = [a | b] per row in the operand type (the input of a projection that mixes two streams)
//   nvllm_embedding_gather_scaled: rows of an embedding table times a constant, as f32 (both the stream and a copy of it)
// Statistics are two-pass (mean, then the mean of squared deviations) in f32 over a row held in shared memory.
#include "common.cuh"

namespace nvllm {
namespace {

struct Addend { const void* p; float s; int dt; };

__device__ __forceinline__ float ld_any(const void* p, int dt, int64_t i) {
  return dt == NVLLM_F32 ? static_cast<const float*>(p)[i] : __bfloat162float(static_cast<const bf16*>(p)[i]);
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();  // red may still be read from a previous call
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];  // same order in every thread: all threads hold the same sum
  return t;
}

template <typename TO>
__global__ void __launch_bounds__(256) residual_layernorm_kernel(TO* __restrict__ out, float* __restrict__ h, Addend a0, Addend a1,
                                                                 Addend a2, const float* __restrict__ bias, float sb,
                                                                 const float* __restrict__ w, int hidden, float eps) {
  extern __shared__ float row[];
  __shared__ float red[8];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * hidden;
  float sum = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = h[base + c];
    if (a0.p) v = fmaf(a0.s, ld_any(a0.p, a0.dt, base + c), v);
    if (a1.p) v = fmaf(a1.s, ld_any(a1.p, a1.dt, base + c), v);
    if (a2.p) v = fmaf(a2.s, ld_any(a2.p, a2.dt, base + c), v);
    if (bias) v = fmaf(sb, bias[c], v);
    if (a0.p || a1.p || a2.p || bias) h[base + c] = v;
    row[c] = v;
    sum += v;
  }
  if (out == nullptr) return;
  const float mean = block_sum(sum, red) / hidden;
  float sq = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) { const float d = row[c] - mean; sq = fmaf(d, d, sq); }
  const float rstd = rsqrtf(block_sum(sq, red) / hidden + eps);
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = (row[c] - mean) * rstd * w[c];
    if (sizeof(TO) == 2) reinterpret_cast<bf16*>(out)[base + c] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(out)[base + c] = v;
  }
}

template <typename TO>
__global__ void concat_cast_kernel(TO* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, int64_t n, int wa, int wb) {
  const int wo = wa + wb;
  const int64_t total = n * wo;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / wo;
    const int c = static_cast<int>(i - r * wo);
    const float v = c < wa ? a[r * wa + c] : b[r * wb + (c - wa)];
    if (sizeof(TO) == 2) reinterpret_cast<bf16*>(out)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(out)[i] = v;
  }
}

template <typename T>
__global__ void embedding_scaled_kernel(float* __restrict__ h, float* __restrict__ h2, const T* __restrict__ table,
                                        const int64_t* __restrict__ ids, int64_t n, int hidden, int vocab, float scale) {
  const int64_t total = n * hidden;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / hidden, c = i - r * hidden;
    int64_t id = ids[r];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    float v;
    if (sizeof(T) == 2) v = __bfloat162float(reinterpret_cast<const bf16*>(table)[id * hidden + c]);
    else v = reinterpret_cast<const float*>(table)[id * hidden + c];
    v *= scale;
    h[i] = v;
    if (h2) h2[i] = v;
  }
}

inline unsigned grid_for(int64_t total) {
  int64_t b = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<unsigned>(b > cap ? cap : (b < 1 ? 1 : b));
}

}  // namespace
}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_residual_layernorm(void* out, float* h, const void* a0, float s0, int32_t dt0, const void* a1, float s1,
                                        int32_t dt1, const void* a2, float s2, int32_t dt2, const float* bias, float bias_scale,
                                        const float* w, int32_t n, int32_t hidden, float eps, int32_t out_dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && hidden > 0 && hidden <= 49152, NVLLM_ERR_ARG, "residual_layernorm: n=%d hidden=%d", n, hidden);
  NVLLM_CHECK_ARG(out_dtype == NVLLM_BF16 || out_dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "residual_layernorm: dtype %d", out_dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(h && (!out || w), NVLLM_ERR_ARG, "residual_layernorm: NULL");
  const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const Addend A0{a0, s0, dt0}, A1{a1, s1, dt1}, A2{a2, s2, dt2};
  if (out_dtype == NVLLM_BF16) {
    if (smem > 48 * 1024) NVLLM_CUDA(cudaFuncSetAttribute(residual_layernorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 192 * 1024));
    residual_layernorm_kernel<bf16><<<n, 256, smem, st>>>(static_cast<bf16*>(out), h, A0, A1, A2, bias, bias_scale, w, hidden, eps);
  } else {
    if (smem > 48 * 1024) NVLLM_CUDA(cudaFuncSetAttribute(residual_layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 192 * 1024));
    residual_layernorm_kernel<float><<<n, 256, smem, st>>>(static_cast<float*>(out), h, A0, A1, A2, bias, bias_scale, w, hidden, eps);
  }
  NVLLM_LAUNCH_CHECK("residual_layernorm_kernel");
  return 0;
}

extern "C" int nvllm_concat_cast(void* out, const float* a, const float* b, int32_t n, int32_t width_a, int32_t width_b,
                                 int32_t out_dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && width_a > 0 && width_b > 0, NVLLM_ERR_ARG, "concat_cast: sizes");
  NVLLM_CHECK_ARG(out_dtype == NVLLM_BF16 || out_dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "concat_cast: dtype %d", out_dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && a && b, NVLLM_ERR_ARG, "concat_cast: NULL");
  const int64_t total = static_cast<int64_t>(n) * (width_a + width_b);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == NVLLM_BF16) concat_cast_kernel<bf16><<<grid_for(total), 256, 0, st>>>(static_cast<bf16*>(out), a, b, n, width_a, width_b);
  else concat_cast_kernel<float><<<grid_for(total), 256, 0, st>>>(static_cast<float*>(out), a, b, n, width_a, width_b);
  NVLLM_LAUNCH_CHECK("concat_cast_kernel");
  return 0;
}

extern "C" int nvllm_embedding_gather_scaled(float* h, float* h_copy, const void* table, const int64_t* ids, int32_t n,
                                             int32_t hidden, int32_t vocab, float scale, int32_t table_dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && hidden > 0 && vocab > 0, NVLLM_ERR_ARG, "embedding_gather_scaled: sizes");
  NVLLM_CHECK_ARG(table_dtype == NVLLM_BF16 || table_dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "embedding_gather_scaled: dtype %d", table_dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(h && table && ids, NVLLM_ERR_ARG, "embedding_gather_scaled: NULL");
  const int64_t total = static_cast<int64_t>(n) * hidden;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (table_dtype == NVLLM_BF16) embedding_scaled_kernel<bf16><<<grid_for(total), 256, 0, st>>>(h, h_copy, static_cast<const bf16*>(table), ids, n, hidden, vocab, scale);
  else embedding_scaled_kernel<float><<<grid_for(total), 256, 0, st>>>(h, h_copy, static_cast<const float*>(table), ids, n, hidden, vocab, scale);
  NVLLM_LAUNCH_CHECK("embedding_scaled_kernel");
  return 0;
}
