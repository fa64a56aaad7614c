// dyt_norm.cu — Dynamic Tanh normalisation, dyt(x) = tanh(alpha * x) * w + b: an element-wise stand-in for a norm layer
// that computes no mean and no variance (alpha is a learned scalar, w and b are vectors).  Models that use it keep the
// residual stream in f32; the fused step of a sandwich-normed block is
//     h += dyt_post(y);  out = dyt_pre(h)
// i.e. the sublayer's output norm, the residual add and the next sublayer's input norm in one pass over the row, as
// nvllm_add_rmsnorm does for RMSNorm models.  All arithmetic is f32; `y` and `out` are bf16 or f32 (dtype), the residual
// and the parameters are always f32.  Also here: the embedding gather into an f32 residual stream and a row gather.
#include "common.cuh"

namespace nvllm {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

struct DytParams { const float* alpha; const float* w; const float* b; };

// 8 bf16 values <-> one 16-byte vector
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

// bf16 rows whose length is a multiple of 8: 16-byte vectors (the residual as two float4)
__global__ void dyt_residual_norm_vec8_kernel(bf16* __restrict__ out, float* __restrict__ h, const bf16* __restrict__ y,
                                              DytParams post, DytParams pre, int64_t total8, int hidden8) {
  const float a_post = y ? *post.alpha : 0.f, a_pre = out ? *pre.alpha : 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % hidden8) * 8;
    float v[8];
    *reinterpret_cast<float4*>(v) = reinterpret_cast<const float4*>(h)[2 * i];
    *reinterpret_cast<float4*>(v + 4) = reinterpret_cast<const float4*>(h)[2 * i + 1];
    if (y) {
      float yv[8];
      unpack8(reinterpret_cast<const uint4*>(y)[i], yv);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += tanhf(a_post * yv[j]) * post.w[c + j] + post.b[c + j];
      reinterpret_cast<float4*>(h)[2 * i] = *reinterpret_cast<float4*>(v);
      reinterpret_cast<float4*>(h)[2 * i + 1] = *reinterpret_cast<float4*>(v + 4);
    }
    if (out) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = tanhf(a_pre * v[j]) * pre.w[c + j] + pre.b[c + j];
      reinterpret_cast<uint4*>(out)[i] = pack8(o);
    }
  }
}

template <typename T>
__global__ void dyt_residual_norm_kernel(T* __restrict__ out, float* __restrict__ h, const T* __restrict__ y, DytParams post,
                                         DytParams pre, int64_t total, int hidden) {
  const float a_post = y ? *post.alpha : 0.f, a_pre = out ? *pre.alpha : 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % hidden);
    float v = h[i];
    if (y) {
      v += tanhf(a_post * ldf(y + i)) * post.w[c] + post.b[c];
      h[i] = v;
    }
    if (out) stf(out + i, tanhf(a_pre * v) * pre.w[c] + pre.b[c]);
  }
}

template <typename T>
__global__ void embedding_f32_kernel(float* __restrict__ h, const T* __restrict__ table, const int64_t* __restrict__ ids,
                                     int n, int hidden, int vocab) {
  const int64_t total = static_cast<int64_t>(n) * hidden;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / hidden, c = i - r * hidden;
    int64_t id = ids[r];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    h[i] = ldf(table + id * hidden + c);
  }
}

// rows whose byte length is a multiple of 16: plain 16-byte copies
__global__ void gather_rows_vec_kernel(uint4* __restrict__ out, const uint4* __restrict__ x, const int32_t* __restrict__ rows, int n,
                                       int vecs, int n_src) {
  const int64_t total = static_cast<int64_t>(n) * vecs;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vecs, c = i - r * vecs;
    int32_t s = rows[r];
    s = s < 0 ? 0 : (s >= n_src ? n_src - 1 : s);
    out[i] = x[static_cast<int64_t>(s) * vecs + c];
  }
}

template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ x, const int32_t* __restrict__ rows, int n,
                                   int hidden, int n_src) {
  const int64_t total = static_cast<int64_t>(n) * hidden;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / hidden, c = i - r * hidden;
    int32_t s = rows[r];
    s = s < 0 ? 0 : (s >= n_src ? n_src - 1 : s);
    out[i] = x[static_cast<int64_t>(s) * hidden + c];
  }
}

inline unsigned blocks_for(int64_t total) {
  int64_t b = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<unsigned>(b > cap ? cap : (b < 1 ? 1 : b));
}

}  // namespace
}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_dyt_residual_norm(void* out, float* h, const void* y, const float* post_alpha, const float* post_w,
                                       const float* post_b, const float* pre_alpha, const float* pre_w, const float* pre_b,
                                       int32_t n, int32_t hidden, int32_t dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && hidden > 0, NVLLM_ERR_ARG, "dyt_residual_norm: n=%d hidden=%d", n, hidden);
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "dyt_residual_norm: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(h && (out || y), NVLLM_ERR_ARG, "dyt_residual_norm: NULL");
  NVLLM_CHECK_ARG(!y || (post_alpha && post_w && post_b), NVLLM_ERR_ARG, "dyt_residual_norm: output-norm parameters");
  NVLLM_CHECK_ARG(!out || (pre_alpha && pre_w && pre_b), NVLLM_ERR_ARG, "dyt_residual_norm: input-norm parameters");
  const int64_t total = static_cast<int64_t>(n) * hidden;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const DytParams post{post_alpha, post_w, post_b}, pre{pre_alpha, pre_w, pre_b};
  if (dtype == NVLLM_BF16 && hidden % 8 == 0 && aligned16(h) && aligned16(out) && aligned16(y))
    dyt_residual_norm_vec8_kernel<<<blocks_for(total / 8), 256, 0, st>>>(static_cast<bf16*>(out), h, static_cast<const bf16*>(y), post, pre,
                                                                          total / 8, hidden / 8);
  else if (dtype == NVLLM_BF16)
    dyt_residual_norm_kernel<bf16><<<blocks_for(total), 256, 0, st>>>(static_cast<bf16*>(out), h, static_cast<const bf16*>(y), post, pre, total, hidden);
  else
    dyt_residual_norm_kernel<float><<<blocks_for(total), 256, 0, st>>>(static_cast<float*>(out), h, static_cast<const float*>(y), post, pre, total, hidden);
  NVLLM_LAUNCH_CHECK("dyt_residual_norm_kernel");
  return 0;
}

extern "C" int nvllm_embedding_gather_f32(float* h, const void* table, const int64_t* ids, int32_t n, int32_t hidden,
                                          int32_t vocab, int32_t table_dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && hidden > 0 && vocab > 0, NVLLM_ERR_ARG, "embedding_gather_f32: sizes");
  NVLLM_CHECK_ARG(table_dtype == NVLLM_BF16 || table_dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "embedding_gather_f32: dtype %d", table_dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(h && table && ids, NVLLM_ERR_ARG, "embedding_gather_f32: NULL");
  const int64_t total = static_cast<int64_t>(n) * hidden;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (table_dtype == NVLLM_BF16)
    embedding_f32_kernel<bf16><<<blocks_for(total), 256, 0, st>>>(h, static_cast<const bf16*>(table), ids, n, hidden, vocab);
  else
    embedding_f32_kernel<float><<<blocks_for(total), 256, 0, st>>>(h, static_cast<const float*>(table), ids, n, hidden, vocab);
  NVLLM_LAUNCH_CHECK("embedding_f32_kernel");
  return 0;
}

extern "C" int nvllm_gather_rows(void* out, const void* x, const int32_t* rows, int32_t n, int32_t hidden, int32_t n_src,
                                 int32_t dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && hidden > 0 && n_src > 0, NVLLM_ERR_ARG, "gather_rows: sizes");
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "gather_rows: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && x && rows, NVLLM_ERR_ARG, "gather_rows: NULL");
  const int64_t total = static_cast<int64_t>(n) * hidden;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t row_bytes = static_cast<int64_t>(hidden) * (dtype == NVLLM_BF16 ? 2 : 4);
  if (row_bytes % 16 == 0 && aligned16(out) && aligned16(x)) {
    const int vecs = static_cast<int>(row_bytes / 16);
    gather_rows_vec_kernel<<<blocks_for(static_cast<int64_t>(n) * vecs), 256, 0, st>>>(static_cast<uint4*>(out), static_cast<const uint4*>(x), rows, n, vecs, n_src);
    NVLLM_LAUNCH_CHECK("gather_rows_vec_kernel");
    return 0;
  }
  if (dtype == NVLLM_BF16)
    gather_rows_kernel<bf16><<<blocks_for(total), 256, 0, st>>>(static_cast<bf16*>(out), static_cast<const bf16*>(x), rows, n, hidden, n_src);
  else
    gather_rows_kernel<float><<<blocks_for(total), 256, 0, st>>>(static_cast<float*>(out), static_cast<const float*>(x), rows, n, hidden, n_src);
  NVLLM_LAUNCH_CHECK("gather_rows_kernel");
  return 0;
}
