// capped_attn.cu — grouped-query softmax attention over a paged key / value cache with
//   * no rotary: position enters through a per-position query temperature  1 + coef * ln(floor((p + 1) / every) + 1),
//   * a soft cap on the scores:  s <- cap * tanh(s / cap)   (cap <= 0: none),
//   * an optional output gate:   out *= sigmoid(gate)       (gate: f32 pre-activations, same layout as the output),
//   * key and value sizes that may differ (dim, vdim).
// Every query token carries its sequence (a row of the block tables) and its position, so one launch serves whole prompts,
// portions of prompts and single decoded tokens side by side; position p sees the keys 0..p of its sequence.
//
// nvllm_attn_bias_store: the step before it — adds the projection biases, writes the queries in the operand type and the
// keys / values into their cache rows.
// Scores, softmax and the accumulation of P.V are f32.
#include "common.cuh"

namespace nvllm {
namespace {

template <typename T> __device__ __forceinline__ float ldv(const T* p);
template <> __device__ __forceinline__ float ldv<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldv<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stv(T* p, float v);
template <> __device__ __forceinline__ void stv<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stv<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// proj row: [q (qn) | k (kn) | v (vn) | ...] f32.  CTA per token.
template <typename T>
__global__ void attn_bias_store_kernel(T* __restrict__ q, int64_t ldq, T* __restrict__ kc, T* __restrict__ vc, int64_t k_row, int64_t v_row,
                                       const float* __restrict__ proj, int64_t ldp, const float* __restrict__ qb,
                                       const float* __restrict__ kb, const float* __restrict__ vb, const int32_t* __restrict__ slots,
                                       int qn, int kn, int vn) {
  const int64_t t = blockIdx.x;
  const float* p = proj + t * ldp;
  for (int c = threadIdx.x; c < qn; c += blockDim.x) stv(q + t * ldq + c, p[c] + (qb ? qb[c] : 0.f));
  const int32_t slot = slots[t];
  if (slot < 0) return;
  for (int c = threadIdx.x; c < kn; c += blockDim.x) stv(kc + slot * k_row + c, p[qn + c] + (kb ? kb[c] : 0.f));
  for (int c = threadIdx.x; c < vn; c += blockDim.x) stv(vc + slot * v_row + c, p[qn + kn + c] + (vb ? vb[c] : 0.f));
}

struct AttnArgs {
  void* out; int64_t ldo;
  const void* q; int64_t ldq;
  const float* gate; int64_t ldg;
  const void *kc, *vc; int64_t k_row, v_row;
  const int32_t* tok_seq; const int64_t* positions; const int32_t* tables;
  int table_cap, block_size, n, heads, kv_heads, dim, vdim;
  float scale, softcap, temp_coef; int temp_every;
};

constexpr int kMaxVPerLane = 8;  // vdim <= 256

// One warp per (token, head): 32 keys per round, lane j scores key j (q broadcast from shared memory), the warp shares
// the online-softmax statistics, then every lane accumulates its output dimensions over the 32 keys.
template <typename T>
__global__ void __launch_bounds__(128) capped_attn_warp_kernel(const AttnArgs a) {
  extern __shared__ float qs[];  // [4 warps][dim]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  if (item >= static_cast<int64_t>(a.n) * a.heads) return;
  const int t = static_cast<int>(item / a.heads), h = static_cast<int>(item % a.heads);
  const int g = h / (a.heads / a.kv_heads);
  float* qw = qs + warp * a.dim;
  const int64_t pos = a.positions[t];
  const float temp = 1.0f + a.temp_coef * logf(floorf(static_cast<float>((pos + 1) / a.temp_every)) + 1.0f);
  const float qscale = a.scale * temp;
  const T* q = static_cast<const T*>(a.q) + t * a.ldq + static_cast<int64_t>(h) * a.dim;
  for (int c = lane; c < a.dim; c += 32) qw[c] = ldv(q + c) * qscale;
  __syncwarp();
  const int32_t* table = a.tables + static_cast<int64_t>(a.tok_seq[t]) * a.table_cap;
  const T* kc = static_cast<const T*>(a.kc) + static_cast<int64_t>(g) * a.dim;
  const T* vc = static_cast<const T*>(a.vc) + static_cast<int64_t>(g) * a.vdim;
  float m = -INFINITY, l = 0.f, acc[kMaxVPerLane];
#pragma unroll
  for (int i = 0; i < kMaxVPerLane; ++i) acc[i] = 0.f;
  const int nkeys = static_cast<int>(pos) + 1;
  for (int j0 = 0; j0 < nkeys; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    int64_t slot = -1;
    if (j < nkeys) {
      const int32_t blk = table[j / a.block_size];
      if (blk >= 0) {
        slot = static_cast<int64_t>(blk) * a.block_size + j % a.block_size;
        const T* kr = kc + slot * a.k_row;
        float d = 0.f;
        for (int c = 0; c < a.dim; ++c) d = fmaf(qw[c], ldv(kr + c), d);
        s = a.softcap > 0.f ? a.softcap * tanhf(d / a.softcap) : d;
      }
    }
    const float mt = warp_max(s);
    const float mn = fmaxf(m, mt);
    if (mn == -INFINITY) continue;
    const float corr = expf(m - mn);   // m = -inf on the first round: 0
    const float p = s == -INFINITY ? 0.f : expf(s - mn);
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int i = 0; i < kMaxVPerLane; ++i) acc[i] *= corr;
    const int cnt = min(32, nkeys - j0);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int64_t sj = __shfl_sync(0xffffffffu, slot, jj);
      if (pj == 0.f || sj < 0) continue;
      const T* vr = vc + sj * a.v_row;
#pragma unroll
      for (int i = 0; i < kMaxVPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < a.vdim) acc[i] = fmaf(pj, ldv(vr + c), acc[i]);
      }
    }
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  T* o = static_cast<T*>(a.out) + t * a.ldo + static_cast<int64_t>(h) * a.vdim;
  const float* gt = a.gate ? a.gate + t * a.ldg + static_cast<int64_t>(h) * a.vdim : nullptr;
#pragma unroll
  for (int i = 0; i < kMaxVPerLane; ++i) {
    const int c = lane + 32 * i;
    if (c < a.vdim) {
      float v = acc[i] * inv;
      if (gt) v *= 1.0f / (1.0f + expf(-gt[c]));
      stv(o + c, v);
    }
  }
}

}  // namespace
}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_attn_bias_store(void* q, int64_t ldq, void* k_cache, void* v_cache, int64_t k_row, int64_t v_row,
                                     const float* proj, int64_t ldp, const float* q_bias, const float* k_bias, const float* v_bias,
                                     const int32_t* slots, int32_t n, int32_t q_cols, int32_t k_cols, int32_t v_cols, int32_t dtype,
                                     void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && q_cols > 0 && k_cols > 0 && v_cols > 0 && ldq >= q_cols && k_row >= k_cols && v_row >= v_cols &&
                      ldp >= q_cols + k_cols + v_cols, NVLLM_ERR_ARG, "attn_bias_store: sizes");
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "attn_bias_store: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(q && k_cache && v_cache && proj && slots, NVLLM_ERR_ARG, "attn_bias_store: NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == NVLLM_BF16)
    attn_bias_store_kernel<bf16><<<n, 256, 0, st>>>(static_cast<bf16*>(q), ldq, static_cast<bf16*>(k_cache), static_cast<bf16*>(v_cache), k_row,
                                                    v_row, proj, ldp, q_bias, k_bias, v_bias, slots, q_cols, k_cols, v_cols);
  else
    attn_bias_store_kernel<float><<<n, 256, 0, st>>>(static_cast<float*>(q), ldq, static_cast<float*>(k_cache), static_cast<float*>(v_cache),
                                                     k_row, v_row, proj, ldp, q_bias, k_bias, v_bias, slots, q_cols, k_cols, v_cols);
  NVLLM_LAUNCH_CHECK("attn_bias_store_kernel");
  return 0;
}

extern "C" int nvllm_capped_attention(void* out, int64_t ldo, const void* q, int64_t ldq, const float* gate, int64_t ldg,
                                      const void* k_cache, const void* v_cache, int64_t k_row, int64_t v_row,
                                      const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables,
                                      int32_t table_cap, int32_t block_size, int32_t n, int32_t heads, int32_t kv_heads, int32_t dim,
                                      int32_t vdim, float scale, float softcap, float temp_coef, int32_t temp_every, int32_t dtype,
                                      void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0 && vdim <= 32 * kMaxVPerLane &&
                      dim <= 2048 && block_size > 0 && table_cap > 0 && temp_every > 0, NVLLM_ERR_ARG,
                  "capped_attention: n=%d heads=%d/%d dim=%d vdim=%d (vdim <= 256)", n, heads, kv_heads, dim, vdim);
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "capped_attention: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && q && k_cache && v_cache && tok_seq && positions && block_tables, NVLLM_ERR_ARG, "capped_attention: NULL");
  AttnArgs a{out, ldo, q, ldq, gate, ldg, k_cache, v_cache, k_row, v_row, tok_seq, positions, block_tables, table_cap, block_size,
             n, heads, kv_heads, dim, vdim, scale, softcap, temp_coef, temp_every};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>((static_cast<int64_t>(n) * heads + 3) / 4);
  const size_t smem = static_cast<size_t>(4) * dim * sizeof(float);
  if (dtype == NVLLM_BF16) capped_attn_warp_kernel<bf16><<<grid, 128, smem, st>>>(a);
  else capped_attn_warp_kernel<float><<<grid, 128, smem, st>>>(a);
  NVLLM_LAUNCH_CHECK("capped_attn_warp_kernel");
  return 0;
}
