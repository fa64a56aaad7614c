// latent_attn.cu — attention over a compressed (latent) KV cache.
//
// A latent-attention layer caches, per token, only a normalised latent vector c (kv_rank values) and ONE rotated key part
// shared by all heads (rot_dim values): cache row = [c | k_rot].  Keys and values of head h are linear maps of c
// (k_h = Uk_h c, v_h = Uv_h c), so with the key map folded into the query the layer is multi-query attention over the
// cache rows themselves:
//     qa_h = Uk_h^T q_h[:dim]                              (nvllm_linear, batched over heads, f32)
//     s_hj = scale * (qa_h . c_j + q_h[dim:] . k_rot_j)     j <= position of the query
//     o_h  = sum_j softmax(s_h)_j c_j                      (this file; kv_rank values per head)
//     out_h = Uv_h o_h                                     (nvllm_linear, batched over heads)
// Entry points: the interleaved-pair rotary table (f64 angles), the per-token preparation (RMS norm of the latent, rotary
// on the shared key part and on the queries' rotated part, store into the paged cache) and the paged attention itself, which
// takes every query token with its own sequence index and position — prompt portions, single decoded tokens and any mix of
// them are one launch.  Softmax, norms and all accumulation are f32; cache and activations are bf16 or f32 (dtype).
#include "common.cuh"

namespace nvllm {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// table[p][i] = (cos, sin)(p * base^(-2i/dims)), i < dims/2, angles in f64
__global__ void rope_table_interleaved_kernel(float2* __restrict__ tab, int max_pos, int half, int dims, double base) {
  const int64_t total = static_cast<int64_t>(max_pos) * half;
  for (int64_t e = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t p = e / half;
    const int i = static_cast<int>(e - p * half);
    const double f = pow(base, -2.0 * i / dims), a = static_cast<double>(p) * f;
    tab[e] = make_float2(static_cast<float>(cos(a)), static_cast<float>(sin(a)));
  }
}

struct PrepArgs {
  void* q; int64_t ldq;
  const void* dkv; int64_t lddkv;
  const float* c_norm_w; float eps;
  const int64_t* positions; const float2* table; int rot_dims, max_pos;
  int n, heads, dim, rot_dim, kv_rank;
  void* cache; int64_t cache_row; const int32_t* slots;
};

// One warp per token: c = rms_norm(dkv[:kv_rank]) * w -> cache row; rotary (pairs (2i, 2i+1), first rot_dims of the
// rotated part) on dkv[kv_rank:] -> cache row, and in place on the rotated part of every query head.
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(const PrepArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= a.n) return;
  const T* row = static_cast<const T*>(a.dkv) + static_cast<int64_t>(t) * a.lddkv;
  const int32_t slot = a.slots[t];
  int64_t pos = a.positions[t];
  pos = pos < 0 ? 0 : (pos >= a.max_pos ? a.max_pos - 1 : pos);
  const float2* tab = a.table + pos * (a.rot_dims / 2);
  T* crow = slot >= 0 ? static_cast<T*>(a.cache) + static_cast<int64_t>(slot) * a.cache_row : nullptr;
  float ss = 0.f;
  for (int i = lane; i < a.kv_rank; i += 32) { const float v = ldf(row + i); ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(a.kv_rank) + a.eps);
  if (crow) {
    for (int i = lane; i < a.kv_rank; i += 32) stf(crow + i, ldf(row + i) * inv * a.c_norm_w[i]);
    for (int i = lane; i < a.rot_dim; i += 32) {
      float v = ldf(row + a.kv_rank + i);
      if (i < a.rot_dims) {
        const float2 cs = tab[i >> 1];
        const float o = ldf(row + a.kv_rank + (i ^ 1));
        v = (i & 1) ? fmaf(v, cs.x, o * cs.y) : fmaf(v, cs.x, -o * cs.y);  // (u cos - v sin, v cos + u sin)
      }
      stf(crow + a.kv_rank + i, v);
    }
  }
  T* q = static_cast<T*>(a.q) + static_cast<int64_t>(t) * a.ldq;
  const int half = a.rot_dims / 2;
  for (int e = lane; e < a.heads * half; e += 32) {
    const int h = e / half, i = e - h * half;
    T* p = q + static_cast<int64_t>(h) * (a.dim + a.rot_dim) + a.dim + 2 * i;
    const float u = ldf(p), v = ldf(p + 1);
    const float2 cs = tab[i];
    stf(p, fmaf(u, cs.x, -v * cs.y));
    stf(p + 1, fmaf(v, cs.x, u * cs.y));
  }
}

struct AttnArgs {
  void* out; int64_t ldo;           // [n, heads, kv_rank]
  const float* q_abs; int64_t ldqa;  // [n, heads, kv_rank] f32
  const void* q; int64_t ldq;        // [n, heads, dim + rot_dim]: only the rotated part is read
  const int32_t* tok_seq; const int64_t* positions;
  const int32_t* tables; int table_cap, block_size;
  const void* cache; int64_t cache_row;
  int n, heads, dim, rot_dim, kv_rank;
  float scale;
};

constexpr int kKeyTile = 32;

// CTA = one query token x up to 8 heads (one warp per head).  Key tiles of 32 cache rows are staged once in shared memory
// (f32) and shared by the CTA's heads; lane j scores key j, then every lane owns kv_rank/32 output columns.
template <typename T, int RI>
__global__ void __launch_bounds__(256) latent_attn_kernel(const AttnArgs a) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int t = blockIdx.x, h = blockIdx.y * nwarps + warp;
  const bool active = h < a.heads;
  const int D = a.kv_rank + a.rot_dim, stride = D | 1;
  float* qs = smem;                       // [nwarps][D]
  float* ks = smem + nwarps * D;          // [kKeyTile][stride]
  const int seq = a.tok_seq[t];
  const int64_t pos = a.positions[t];
  const int nkeys = static_cast<int>(pos) + 1;
  if (active) {
    const float* qa = a.q_abs + static_cast<int64_t>(t) * a.ldqa + static_cast<int64_t>(h) * a.kv_rank;
    const T* qr = static_cast<const T*>(a.q) + static_cast<int64_t>(t) * a.ldq + static_cast<int64_t>(h) * (a.dim + a.rot_dim) + a.dim;
    for (int d = lane; d < a.kv_rank; d += 32) qs[warp * D + d] = qa[d] * a.scale;
    for (int d = lane; d < a.rot_dim; d += 32) qs[warp * D + a.kv_rank + d] = ldf(qr + d) * a.scale;
  }
  float m = -INFINITY, l = 0.f, acc[RI];
#pragma unroll
  for (int i = 0; i < RI; ++i) acc[i] = 0.f;
  const int32_t* table = a.tables + static_cast<int64_t>(seq) * a.table_cap;
  for (int j0 = 0; j0 < nkeys; j0 += kKeyTile) {
    const int cnt = min(kKeyTile, nkeys - j0);
    __syncthreads();
    for (int e = threadIdx.x; e < cnt * D; e += blockDim.x) {
      const int jj = e / D, d = e - jj * D, j = j0 + jj;
      const int32_t blk = table[j / a.block_size];
      float v = 0.f;
      if (blk >= 0)
        v = ldf(static_cast<const T*>(a.cache) + (static_cast<int64_t>(blk) * a.block_size + j % a.block_size) * a.cache_row + d);
      ks[jj * stride + d] = v;
    }
    __syncthreads();
    if (!active) continue;
    float s = -INFINITY;
    if (lane < cnt && table[(j0 + lane) / a.block_size] >= 0) {
      s = 0.f;
      const float* k = ks + lane * stride;
      const float* q = qs + warp * D;
      for (int d = 0; d < D; ++d) s = fmaf(q[d], k[d], s);
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float p = s == -INFINITY ? 0.f : expf(s - m_new);
    const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < RI; ++i) acc[i] *= corr;
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const float* k = ks + jj * stride;
#pragma unroll
      for (int i = 0; i < RI; ++i)
        if (lane + 32 * i < a.kv_rank) acc[i] = fmaf(pj, k[lane + 32 * i], acc[i]);
    }
  }
  if (!active) return;
  T* o = static_cast<T*>(a.out) + static_cast<int64_t>(t) * a.ldo + static_cast<int64_t>(h) * a.kv_rank;
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < RI; ++i)
    if (lane + 32 * i < a.kv_rank) stf(o + lane + 32 * i, acc[i] * inv);
}

template <typename T, int RI>
int launch_attn(const AttnArgs& a, cudaStream_t st) {
  const int hpb = a.heads < 8 ? a.heads : 8;
  const int D = a.kv_rank + a.rot_dim;
  const size_t smem = (static_cast<size_t>(hpb) * D + static_cast<size_t>(kKeyTile) * (D | 1)) * sizeof(float);
  NVLLM_CHECK_ARG(smem <= 220 * 1024, NVLLM_ERR_ARG, "latent_attention: kv_rank + rot_dim = %d needs %zu bytes of shared memory", D, smem);
  NVLLM_SMEM_ATTR_ONCE((latent_attn_kernel<T, RI>), 220 * 1024);
  dim3 grid(a.n, (a.heads + hpb - 1) / hpb);
  latent_attn_kernel<T, RI><<<grid, 32 * hpb, smem, st>>>(a);
  NVLLM_LAUNCH_CHECK("latent_attn_kernel");
  return 0;
}

template <typename T>
int dispatch_attn(const AttnArgs& a, cudaStream_t st) {
  if (a.kv_rank <= 128) return launch_attn<T, 4>(a, st);
  if (a.kv_rank <= 512) return launch_attn<T, 16>(a, st);
  return launch_attn<T, 32>(a, st);
}

}  // namespace
}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_rope_table_interleaved(float* cos_sin, int32_t max_pos, int32_t dims, double base, void* stream) {
  NVLLM_CHECK_ARG(cos_sin && max_pos > 0 && dims > 0 && dims % 2 == 0 && base > 0, NVLLM_ERR_ARG,
                  "rope_table_interleaved: max_pos=%d dims=%d (even) base=%g", max_pos, dims, base);
  const int64_t total = static_cast<int64_t>(max_pos) * (dims / 2);
  int64_t blocks = (total + 255) / 256;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  rope_table_interleaved_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<float2*>(cos_sin), max_pos, dims / 2, dims, base);
  NVLLM_LAUNCH_CHECK("rope_table_interleaved_kernel");
  return 0;
}

extern "C" int nvllm_latent_prepare(void* q, int64_t ldq, const void* dkv, int64_t lddkv, const float* c_norm_w, float eps,
                                    const int64_t* positions, const float* rope_table, int32_t rot_dims, int32_t max_pos,
                                    int32_t n, int32_t heads, int32_t dim, int32_t rot_dim, int32_t kv_rank, void* cache,
                                    int64_t cache_row, const int32_t* slots, int32_t dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && heads > 0 && dim >= 0 && rot_dim >= 0 && kv_rank > 0, NVLLM_ERR_ARG, "latent_prepare: sizes");
  NVLLM_CHECK_ARG(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot_dim, NVLLM_ERR_ARG,
                  "latent_prepare: rot_dims=%d must be even and at most rot_dim=%d", rot_dims, rot_dim);
  NVLLM_CHECK_ARG(cache_row >= kv_rank + rot_dim && ldq >= static_cast<int64_t>(heads) * (dim + rot_dim) && lddkv >= kv_rank + rot_dim,
                  NVLLM_ERR_ARG, "latent_prepare: strides");
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "latent_prepare: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(q && dkv && c_norm_w && positions && (rope_table || rot_dims == 0) && cache && slots, NVLLM_ERR_ARG, "latent_prepare: NULL");
  const PrepArgs a{q, ldq, dkv, lddkv, c_norm_w, eps, positions, reinterpret_cast<const float2*>(rope_table), rot_dims, max_pos,
                   n, heads, dim, rot_dim, kv_rank, cache, cache_row, slots};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == NVLLM_BF16) latent_prepare_kernel<bf16><<<(n + 3) / 4, 128, 0, st>>>(a);
  else latent_prepare_kernel<float><<<(n + 3) / 4, 128, 0, st>>>(a);
  NVLLM_LAUNCH_CHECK("latent_prepare_kernel");
  return 0;
}

extern "C" int nvllm_latent_attention(void* out, int64_t ldo, const float* q_abs, int64_t ldqa, const void* q, int64_t ldq,
                                      const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables,
                                      int32_t table_cap, int32_t block_size, const void* cache, int64_t cache_row, int32_t n,
                                      int32_t heads, int32_t dim, int32_t rot_dim, int32_t kv_rank, float scale,
                                      int32_t dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && heads > 0 && dim >= 0 && rot_dim >= 0 && kv_rank > 0 && kv_rank <= 1024 && table_cap > 0 && block_size > 0,
                  NVLLM_ERR_ARG, "latent_attention: sizes (kv_rank <= 1024)");
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "latent_attention: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && q_abs && q && tok_seq && positions && block_tables && cache, NVLLM_ERR_ARG, "latent_attention: NULL");
  const AttnArgs a{out, ldo, q_abs, ldqa, q, ldq, tok_seq, positions, block_tables, table_cap, block_size, cache, cache_row,
                   n, heads, dim, rot_dim, kv_rank, scale};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == NVLLM_BF16 ? dispatch_attn<bf16>(a, st) : dispatch_attn<float>(a, st);
}
