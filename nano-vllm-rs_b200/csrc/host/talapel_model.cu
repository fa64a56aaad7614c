// talapel_model.cu — the Talapel architecture on the runner's model interface (model.hpp).
//
// Talapel is a decoder-only model of PARALLEL blocks on an f32 residual stream: one layer norm per layer, and the mixer and
// the feed-forward both read its output,  x <- x + mixer(ln(x)) + ff(ln(x)).  Two kinds of mixer:
//   "parallel"   two mixers side by side, c_l * attention + c_r * ssd:
//                attention — grouped-query softmax attention without rotary (capped_attn.cu): biased q / k / v, a query
//                temperature that grows with the logarithm of the position, tanh-capped scores, a sigmoid output gate, biased
//                output projection; keys and values live in the paged cache;
//                ssd — state-space duality (recurrence.cu): one input projection [z | x | B | C | dt], a short causal
//                convolution + SiLU over (x, B, C), S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x, gated group RMS norm;
//   "retention"  decayed linear attention (recurrence.cu): half-split rotary on q and k, S <- decay_h S + k v^T, o = S^T q,
//                per-head RMS norm, SiLU gate.
// Recurrent states (and the convolution's last inputs) live in per-sequence state slots that the scheduler hands out.
// Feed-forward: dense SiLU-gated, or experts chosen by a table indexed with the token id (equal weights, squared-ReLU
// experts); a layer may have none.  A contiguous range of layers may run several times over the same weights (`loop`);
// every pass starts with x <- W_loop [x ; x0] (x0: the scaled embedding) and every layer run has its own cache and state.
// Every size, constant and the layer order come from the configuration.
//
// configuration keys read here: architecture, vocab, width, norm.eps, embedding.scale, loop.{start,stop,times},
// layers[i].type ("parallel" | "retention"), layers[i].mixer (parallel: left.{heads,kv_heads,dim,vdim,scale,softcap,
// q_temp.{coef,every}}, right.{heads,groups,state,vdim,conv,norm_groups}, left_scale, right_scale; retention: heads, dim,
// vdim, rot.{base,dims}, decay[]), layers[i].mlp (null | kind "dense", ff | kind "moe", expert.ff, router.{experts,top}).
// tensors: embed, head, final.norm, loop.in, l<i>.norm1, l<i>.mix.left.{q,k,v,o}{,.b}, l<i>.mix.left.g,
// l<i>.mix.right.{in,conv,conv.b,dt_bias,A_log,D,norm,o}, l<i>.mix.{q,k,v,g,o}, l<i>.mlp.{gate,up,down},
// l<i>.mlp.e<j>.{up,down}, l<i>.mlp.table (int32).
#include <algorithm>
#include <cmath>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "../common.cuh"
#include "model.hpp"

namespace nvllm {
namespace {

#define RUN(expr)                   \
  do {                              \
    int _rc = (expr);               \
    if (_rc != 0) return _rc;       \
  } while (0)

inline int pad8(int n) { return (n + 7) / 8 * 8; }

enum MixKind { kParallel = 0, kRetention = 1 };
enum FfKind { kNone = 0, kDense = 1, kExperts = 2 };

struct Layer {
  int mix = kParallel, ffk = kNone;
  // attention (parallel.left)
  int H = 0, G = 0, D = 0, V = 0, temp_every = 1;
  float scale = 1.f, softcap = 0.f, temp_coef = 0.f, left_scale = 1.f, right_scale = 1.f;
  // ssd (parallel.right)
  int sH = 0, sG = 0, sN = 0, sP = 0, taps = 1, norm_groups = 1;
  // retention
  int rH = 0, rD = 0, rV = 0, rot_dims = 0;
  double rot_base = 10000.0;
  std::vector<float> decay_h;
  // feed-forward
  int ff = 0, experts = 0, top = 0, tile_rows = 32;
  // weights: projections in the operand type (bf16 | f32), vectors f32
  float* norm1 = nullptr;
  void *a_in = nullptr, *a_o = nullptr, *s_in = nullptr, *s_o = nullptr, *r_in = nullptr, *r_o = nullptr;
  float *qb = nullptr, *kb = nullptr, *vb = nullptr, *ob = nullptr;
  float *conv_w = nullptr, *conv_b = nullptr, *dt_bias = nullptr, *a_log = nullptr, *skip = nullptr, *s_norm = nullptr, *decay = nullptr, *kscale = nullptr;
  void *gu = nullptr, *down = nullptr, *eup = nullptr, *edown = nullptr;
  int32_t* table = nullptr;
  const float* rope = nullptr;
  // packed projection layouts (f32 output rows, padded to 8 columns)
  int a_cols() const { return H * D + G * D + G * V + H * V; }
  int s_inner() const { return sH * sP; }
  int s_ch() const { return s_inner() + 2 * sG * sN; }
  int s_cols() const { return 2 * s_inner() + 2 * sG * sN + sH; }
  int r_cols() const { return 2 * rH * rD + 2 * rH * rV; }
};

struct RunState {
  void *kc = nullptr, *vc = nullptr;         // attention cache of this layer run
  float *ssd = nullptr, *conv = nullptr;     // [slots, sH, sN, sP], [slots, taps - 1, channels]
  float* ret = nullptr;                      // [slots, rH, rD, rV]
};

class Talapel : public ModelImpl {
 public:
  int vocab_ = 0, width_ = 0;
  float eps_ = 1e-5f, embed_scale_ = 1.f;
  bool has_loop_ = false;
  std::vector<Layer> layers_;
  std::vector<std::pair<int, bool>> runs_;  // (layer, first of its pass) in execution order
  std::vector<RunState> state_;
  ModelLimits lim_{};
  int dt_ = NVLLM_BF16;
  size_t esz_ = 2;
  void *embed_ = nullptr, *head_ = nullptr, *loop_in_ = nullptr;
  float* final_norm_ = nullptr;
  std::map<std::pair<double, int>, float*> rope_tables_;
  // activations
  float *h_ = nullptr, *x0_ = nullptr, *proj_ = nullptr, *left_out_ = nullptr, *right_out_ = nullptr, *conv_out_ = nullptr,
        *step_ = nullptr, *decay_t_ = nullptr, *y_ = nullptr, *topk_w_ = nullptr;
  void *normed_ = nullptr, *cat_ = nullptr, *q_ = nullptr, *mix_in_ = nullptr, *gu_buf_ = nullptr, *act_ = nullptr, *ff_out_ = nullptr,
       *eout_ = nullptr, *xg_ = nullptr, *eup_buf_ = nullptr, *head_in_ = nullptr;
  int32_t *topk_idx_ = nullptr, *row_token_ = nullptr, *tile_expert_ = nullptr, *slot_row_ = nullptr;
  int max_rows_ = 0, head_rows_ = 0;
  std::vector<void*> allocs_;
  std::set<std::string> needed_, loaded_;
  bool ready_ = false;

  ~Talapel() override { for (void* p : allocs_) cudaFree(p); }
  int vocab() const override { return vocab_; }
  int hidden() const override { return width_; }
  int layer_runs() const override { return static_cast<int>(runs_.size()); }
  bool recurrent_state() const override { return true; }
  bool weights_ready() const override { return ready_; }

  int parse(const json::Value& c) {
    vocab_ = c["vocab"].need_int("vocab");
    width_ = c["width"].need_int("width");
    eps_ = static_cast<float>(c["norm"]["eps"].as_double(1e-5));
    embed_scale_ = static_cast<float>(c["embedding"]["scale"].as_double(1.0));
    const json::Value& ls = c["layers"];
    NVLLM_CHECK_ARG(ls.is_array() && ls.size() > 0 && vocab_ > 0 && width_ > 0, NVLLM_ERR_ARG, "Talapel config: layers / vocab / width");
    for (size_t i = 0; i < ls.size(); ++i) {
      const json::Value& l = ls[i];
      Layer L;
      const std::string type = l["type"].as_string();
      const json::Value& m = l["mixer"];
      if (type == "parallel") {
        L.mix = kParallel;
        const json::Value &a = m["left"], &s = m["right"];
        L.H = a["heads"].need_int("left.heads"); L.G = a["kv_heads"].as_int(L.H);
        L.D = a["dim"].need_int("left.dim"); L.V = a["vdim"].as_int(L.D);
        L.scale = static_cast<float>(a["scale"].need_double("left.scale"));
        L.softcap = static_cast<float>(a["softcap"].as_double(0.0));
        L.temp_coef = static_cast<float>(a["q_temp"]["coef"].as_double(0.0));
        L.temp_every = a["q_temp"]["every"].as_int(1);
        L.left_scale = static_cast<float>(m["left_scale"].as_double(1.0));
        L.right_scale = static_cast<float>(m["right_scale"].as_double(1.0));
        L.sH = s["heads"].need_int("right.heads"); L.sG = s["groups"].as_int(1);
        L.sN = s["state"].need_int("right.state"); L.sP = s["vdim"].need_int("right.vdim");
        L.taps = s["conv"].as_int(1); L.norm_groups = s["norm_groups"].as_int(1);
        NVLLM_CHECK_ARG(L.H > 0 && L.G > 0 && L.H % L.G == 0 && L.D > 0 && L.V > 0 && L.V <= 512 && L.temp_every > 0, NVLLM_ERR_ARG,
                        "Talapel config: layer %zu attention sizes (heads %d / %d, dim %d, vdim %d <= 512)", i, L.H, L.G, L.D, L.V);
        NVLLM_CHECK_ARG(L.sH > 0 && L.sG > 0 && L.sH % L.sG == 0 && L.sN > 0 && L.sN <= 512 && L.sP > 0 && L.taps >= 1 && L.taps <= 16 &&
                            L.norm_groups > 0 && (L.sH * L.sP) % L.norm_groups == 0, NVLLM_ERR_ARG,
                        "Talapel config: layer %zu state-space sizes (heads %d / %d, state %d <= 512, vdim %d, conv %d <= 16, norm_groups %d)",
                        i, L.sH, L.sG, L.sN, L.sP, L.taps, L.norm_groups);
      } else if (type == "retention") {
        L.mix = kRetention;
        L.rH = m["heads"].need_int("mixer.heads"); L.rD = m["dim"].need_int("mixer.dim"); L.rV = m["vdim"].as_int(L.rD);
        L.rot_dims = m["rot"]["dims"].as_int(0);
        L.rot_base = m["rot"]["base"].as_double(10000.0);
        const json::Value& d = m["decay"];
        NVLLM_CHECK_ARG(L.rH > 0 && L.rD > 0 && L.rD <= 512 && L.rV > 0 && L.rot_dims >= 0 && L.rot_dims % 2 == 0 && L.rot_dims <= L.rD &&
                            L.rot_base > 0 && d.is_array() && static_cast<int>(d.size()) == L.rH, NVLLM_ERR_ARG,
                        "Talapel config: layer %zu retention sizes (heads %d, dim %d <= 512, vdim %d, rot dims %d, one decay per head)", i,
                        L.rH, L.rD, L.rV, L.rot_dims);
        for (size_t k = 0; k < d.size(); ++k) L.decay_h.push_back(static_cast<float>(d[k].as_double(1.0)));
      } else {
        NVLLM_CHECK_ARG(false, NVLLM_ERR_ARG, "Talapel config: layer %zu has mixer type '%s' (known: parallel, retention)", i, type.c_str());
      }
      const json::Value& f = l["mlp"];
      if (!f.is_null()) {
        const std::string kind = f["kind"].as_string("dense");
        if (kind == "dense") {
          L.ffk = kDense;
          L.ff = f["ff"].need_int("mlp.ff");
        } else if (kind == "moe") {
          L.ffk = kExperts;
          L.ff = f["expert"]["ff"].need_int("expert.ff");
          L.experts = f["router"]["experts"].need_int("router.experts");
          L.top = f["router"]["top"].need_int("router.top");
          NVLLM_CHECK_ARG(L.experts > 0 && L.experts <= 8192 && L.top > 0 && L.top <= L.experts, NVLLM_ERR_ARG, "Talapel config: layer %zu experts / top", i);
        } else {
          NVLLM_CHECK_ARG(false, NVLLM_ERR_ARG, "Talapel config: layer %zu feed-forward kind '%s' (known: dense, moe)", i, kind.c_str());
        }
        NVLLM_CHECK_ARG(L.ff > 0, NVLLM_ERR_ARG, "Talapel config: layer %zu feed-forward size", i);
      }
      layers_.push_back(L);
    }
    const int n = static_cast<int>(layers_.size());
    if (c["loop"].is_object()) {
      const int start = c["loop"]["start"].as_int(0), stop = c["loop"]["stop"].as_int(0), times = c["loop"]["times"].as_int(1);
      NVLLM_CHECK_ARG(0 <= start && start <= stop && stop <= n && times >= 0, NVLLM_ERR_ARG, "Talapel config: loop %d..%d x %d", start, stop, times);
      has_loop_ = times > 0 && stop > start;   // only then does a pass begin somewhere and W_loop get used
      for (int i = 0; i < start; ++i) runs_.push_back({i, false});
      for (int t = 0; t < times; ++t)
        for (int i = start; i < stop; ++i) runs_.push_back({i, i == start});
      for (int i = stop; i < n; ++i) runs_.push_back({i, false});
    } else {
      for (int i = 0; i < n; ++i) runs_.push_back({i, false});
    }
    NVLLM_CHECK_ARG(!runs_.empty(), NVLLM_ERR_ARG, "Talapel config: no layer runs");
    return 0;
  }

  template <typename T>
  int dalloc(T** p, size_t count, size_t elt = sizeof(T), bool zero = false) {
    void* q = nullptr;
    const size_t bytes = (count * elt + 255) & ~static_cast<size_t>(255);
    cudaError_t e = cudaMalloc(&q, bytes ? bytes : 256);
    if (e != cudaSuccess) { set_error("cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e)); return static_cast<int>(e); }
    allocs_.push_back(q);
    if (zero) cudaMemset(q, 0, bytes ? bytes : 256);
    *p = static_cast<T*>(q);
    return 0;
  }
  int oalloc(void** p, size_t count, bool zero = false) { return dalloc(p, count, esz_, zero); }  // operand-typed buffer
  int valloc(float** p, size_t count, const std::string& name) { needed_.insert(name); return dalloc(p, count); }

  int create(const ModelLimits& lim, cudaStream_t stream) override {
    lim_ = lim;
    dt_ = lim.dtype;
    esz_ = dt_ == NVLLM_F32 ? 4 : 2;
    const size_t W = width_, T = lim.max_tokens, S = lim.max_seqs;
    RUN(oalloc(&embed_, static_cast<size_t>(vocab_) * W)); RUN(oalloc(&head_, static_cast<size_t>(vocab_) * W));
    needed_.insert("embed"); needed_.insert("head");
    RUN(valloc(&final_norm_, W, "final.norm"));
    if (has_loop_) { RUN(oalloc(&loop_in_, W * 2 * W)); needed_.insert("loop.in"); }
    size_t m_proj = 8, m_q = 8, m_mix = 8, m_ch = 1, m_sh = 1, m_y = 1, m_ff = 0, m_eff = 0, m_top = 1;
    for (size_t i = 0; i < layers_.size(); ++i) {
      Layer& L = layers_[i];
      const std::string p = "l" + std::to_string(i) + ".";
      RUN(valloc(&L.norm1, W, p + "norm1"));
      if (L.mix == kParallel) {
        const std::string a = p + "mix.left.", s = p + "mix.right.";
        RUN(oalloc(&L.a_in, static_cast<size_t>(pad8(L.a_cols())) * W, true)); RUN(oalloc(&L.a_o, W * L.H * L.V));
        for (const char* t : {"q", "k", "v", "g", "o"}) needed_.insert(a + t);
        RUN(valloc(&L.qb, L.H * L.D, a + "q.b")); RUN(valloc(&L.kb, L.G * L.D, a + "k.b")); RUN(valloc(&L.vb, L.G * L.V, a + "v.b"));
        RUN(valloc(&L.ob, W, a + "o.b"));
        RUN(oalloc(&L.s_in, static_cast<size_t>(pad8(L.s_cols())) * W, true)); RUN(oalloc(&L.s_o, W * L.s_inner()));
        needed_.insert(s + "in"); needed_.insert(s + "o");
        RUN(valloc(&L.conv_w, static_cast<size_t>(L.s_ch()) * L.taps, s + "conv")); RUN(valloc(&L.conv_b, L.s_ch(), s + "conv.b"));
        RUN(valloc(&L.dt_bias, L.sH, s + "dt_bias")); RUN(valloc(&L.a_log, L.sH, s + "A_log")); RUN(valloc(&L.skip, L.sH, s + "D"));
        RUN(valloc(&L.s_norm, L.s_inner(), s + "norm"));
        m_proj = std::max<size_t>(m_proj, std::max(pad8(L.a_cols()), pad8(L.s_cols())));
        m_q = std::max<size_t>(m_q, L.H * L.D);
        m_mix = std::max<size_t>(m_mix, std::max(L.H * L.V, L.s_inner()));
        m_ch = std::max<size_t>(m_ch, L.s_ch()); m_sh = std::max<size_t>(m_sh, L.sH); m_y = std::max<size_t>(m_y, L.s_inner());
      } else {
        const std::string a = p + "mix.";
        RUN(oalloc(&L.r_in, static_cast<size_t>(pad8(L.r_cols())) * W, true)); RUN(oalloc(&L.r_o, W * L.rH * L.rV));
        for (const char* t : {"q", "k", "v", "g", "o"}) needed_.insert(a + t);
        RUN(dalloc(&L.decay, L.rH)); RUN(dalloc(&L.kscale, L.rH));
        NVLLM_CUDA(cudaMemcpy(L.decay, L.decay_h.data(), sizeof(float) * L.rH, cudaMemcpyHostToDevice));
        const std::vector<float> ks(L.rH, 1.0f / sqrtf(static_cast<float>(L.rD)));   // k <- k dim^-1/2, applied as the recurrence's step
        NVLLM_CUDA(cudaMemcpy(L.kscale, ks.data(), sizeof(float) * L.rH, cudaMemcpyHostToDevice));
        if (L.rot_dims > 0) {  // rotary table shared by the layers that agree on (base, dims)
          const auto key = std::make_pair(L.rot_base, L.rot_dims);
          auto it = rope_tables_.find(key);
          if (it == rope_tables_.end()) {
            float* tab = nullptr;
            RUN(dalloc(&tab, static_cast<size_t>(lim.max_positions) * L.rot_dims));
            RUN(nvllm_rope_table_interleaved(tab, lim.max_positions, L.rot_dims, L.rot_base, stream));
            it = rope_tables_.emplace(key, tab).first;
          }
          L.rope = it->second;
        }
        m_proj = std::max<size_t>(m_proj, pad8(L.r_cols()));
        m_mix = std::max<size_t>(m_mix, L.rH * L.rV); m_y = std::max<size_t>(m_y, L.rH * L.rV);
      }
      if (L.ffk == kDense) {
        RUN(oalloc(&L.gu, static_cast<size_t>(2) * L.ff * W)); RUN(oalloc(&L.down, W * L.ff));
        for (const char* t : {"gate", "up", "down"}) needed_.insert(p + "mlp." + t);
        m_ff = std::max<size_t>(m_ff, L.ff);
      } else if (L.ffk == kExperts) {
        RUN(oalloc(&L.eup, static_cast<size_t>(L.experts) * L.ff * W)); RUN(oalloc(&L.edown, static_cast<size_t>(L.experts) * W * L.ff));
        RUN(dalloc(&L.table, static_cast<size_t>(vocab_) * L.top));
        for (int e = 0; e < L.experts; ++e)
          for (const char* t : {"up", "down"}) needed_.insert(p + "mlp.e" + std::to_string(e) + "." + t);
        needed_.insert(p + "mlp.table");
        m_eff = std::max<size_t>(m_eff, L.ff); m_top = std::max<size_t>(m_top, L.top);
        if (dt_ == NVLLM_BF16 && W % 64 == 0 && L.ff % 64 == 0) L.tile_rows = 128;  // experts on the tensor-core grouped GEMM
        max_rows_ = std::max(max_rows_, nvllm_moe_max_rows(lim.max_tokens, L.top, L.experts, L.tile_rows));
      }
    }
    // per layer run: the attention cache (paged, addressed through the runner's block tables) and the state slots
    state_.resize(runs_.size());
    for (size_t r = 0; r < runs_.size(); ++r) {
      const Layer& L = layers_[runs_[r].first];
      RunState& st = state_[r];
      if (L.mix == kParallel) {
        const size_t rows = static_cast<size_t>(lim.num_blocks) * lim.block_size;
        RUN(oalloc(&st.kc, rows * L.G * L.D, true)); RUN(oalloc(&st.vc, rows * L.G * L.V, true));
        RUN(dalloc(&st.ssd, S * L.sH * L.sN * L.sP, sizeof(float), true));
        RUN(dalloc(&st.conv, S * std::max(1, L.taps - 1) * L.s_ch(), sizeof(float), true));
      } else {
        RUN(dalloc(&st.ret, S * L.rH * L.rD * L.rV, sizeof(float), true));
      }
    }
    RUN(dalloc(&h_, T * W)); RUN(dalloc(&x0_, T * W)); RUN(oalloc(&normed_, T * W)); RUN(oalloc(&cat_, T * 2 * W));
    RUN(dalloc(&proj_, T * m_proj)); RUN(oalloc(&q_, T * m_q)); RUN(oalloc(&mix_in_, T * m_mix));
    RUN(dalloc(&left_out_, T * W)); RUN(dalloc(&right_out_, T * W)); RUN(dalloc(&conv_out_, T * m_ch));
    RUN(dalloc(&step_, T * m_sh)); RUN(dalloc(&decay_t_, T * m_sh)); RUN(dalloc(&y_, T * m_y));
    RUN(dalloc(reinterpret_cast<float**>(&ff_out_), T * W));
    const size_t m_act = std::max(m_ff, m_eff);
    if (m_ff > 0) RUN(oalloc(&gu_buf_, T * 2 * m_ff));
    if (m_eff > 0) {
      RUN(dalloc(&topk_w_, T * m_top)); RUN(dalloc(&topk_idx_, T * m_top)); RUN(dalloc(&slot_row_, T * m_top));
      RUN(dalloc(&row_token_, static_cast<size_t>(max_rows_) + 32)); RUN(dalloc(&tile_expert_, static_cast<size_t>(max_rows_) / 32 + 1));
      RUN(oalloc(&eout_, static_cast<size_t>(max_rows_) * W)); RUN(oalloc(&xg_, static_cast<size_t>(max_rows_) * W));
      RUN(oalloc(&eup_buf_, static_cast<size_t>(max_rows_) * m_eff));
    }
    if (m_act > 0) RUN(oalloc(&act_, std::max(T, static_cast<size_t>(max_rows_)) * m_act));
    NVLLM_CUDA(cudaStreamSynchronize(stream));
    return 0;
  }

  // ---- weights ---------------------------------------------------------------------------------------------------
  static float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = static_cast<uint32_t>(b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
  }
  // host bf16 [rows, cols] -> device operand tensor at ELEMENT offset `off`
  int put(void* dst, size_t off, const uint16_t* src, int64_t rows, int64_t cols, cudaStream_t st) {
    const size_t n = static_cast<size_t>(rows) * cols;
    const void* from = src;
    std::vector<float> tmp;
    if (esz_ == 4) {
      tmp.resize(n);
      for (size_t i = 0; i < n; ++i) tmp[i] = bf16_bits_to_f32(src[i]);
      from = tmp.data();
    }
    NVLLM_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(dst) + off * esz_, from, n * esz_, cudaMemcpyHostToDevice, st));
    NVLLM_CUDA(cudaStreamSynchronize(st));
    return 0;
  }
  int putf(float* dst, const uint16_t* src, int64_t n, cudaStream_t st) {
    std::vector<float> tmp(n);
    for (int64_t i = 0; i < n; ++i) tmp[i] = bf16_bits_to_f32(src[i]);
    NVLLM_CUDA(cudaMemcpyAsync(dst, tmp.data(), n * 4, cudaMemcpyHostToDevice, st));
    NVLLM_CUDA(cudaStreamSynchronize(st));
    return 0;
  }

  // The tensor's shape and where it goes.  kind: 0 operand matrix at (dst, element offset), 1 f32 vector, 2 int32 table.
  struct Target { int kind = -1; void* dst = nullptr; size_t off = 0; int64_t rows = 0, cols = 0; };
  Target target_of(const std::string& name) const {
    const int64_t W = width_;
    Target t;
    auto mat = [&](void* d, size_t off, int64_t r, int64_t c) { t.kind = 0; t.dst = d; t.off = off; t.rows = r; t.cols = c; return t; };
    auto vec = [&](float* d, int64_t n) { t.kind = 1; t.dst = d; t.rows = 1; t.cols = n; return t; };
    if (name == "embed") return mat(embed_, 0, vocab_, W);
    if (name == "head") return mat(head_, 0, vocab_, W);
    if (name == "final.norm") return vec(final_norm_, W);
    if (name == "loop.in") return mat(loop_in_, 0, W, 2 * W);
    if (name.size() < 4 || name[0] != 'l') return t;
    const size_t dot = name.find('.');
    if (dot == std::string::npos) return t;
    const int li = atoi(name.substr(1, dot - 1).c_str());
    if (li < 0 || li >= static_cast<int>(layers_.size())) return t;
    const Layer& L = layers_[li];
    const std::string rest = name.substr(dot + 1);
    if (rest == "norm1") return vec(L.norm1, W);
    if (L.mix == kParallel) {
      const int64_t qn = L.H * L.D, kn = L.G * L.D, vn = L.G * L.V, gn = L.H * L.V;
      if (rest == "mix.left.q") return mat(L.a_in, 0, qn, W);
      if (rest == "mix.left.k") return mat(L.a_in, qn * W, kn, W);
      if (rest == "mix.left.v") return mat(L.a_in, (qn + kn) * W, vn, W);
      if (rest == "mix.left.g") return mat(L.a_in, (qn + kn + vn) * W, gn, W);
      if (rest == "mix.left.o") return mat(L.a_o, 0, W, gn);
      if (rest == "mix.left.q.b") return vec(L.qb, qn);
      if (rest == "mix.left.k.b") return vec(L.kb, kn);
      if (rest == "mix.left.v.b") return vec(L.vb, vn);
      if (rest == "mix.left.o.b") return vec(L.ob, W);
      if (rest == "mix.right.in") return mat(L.s_in, 0, L.s_cols(), W);
      if (rest == "mix.right.o") return mat(L.s_o, 0, W, L.s_inner());
      if (rest == "mix.right.conv") { t = vec(L.conv_w, static_cast<int64_t>(L.s_ch()) * L.taps); t.rows = L.s_ch(); t.cols = L.taps; return t; }
      if (rest == "mix.right.conv.b") return vec(L.conv_b, L.s_ch());
      if (rest == "mix.right.dt_bias") return vec(L.dt_bias, L.sH);
      if (rest == "mix.right.A_log") return vec(L.a_log, L.sH);
      if (rest == "mix.right.D") return vec(L.skip, L.sH);
      if (rest == "mix.right.norm") return vec(L.s_norm, L.s_inner());
    } else {
      const int64_t qn = L.rH * L.rD, vn = L.rH * L.rV;
      if (rest == "mix.q") return mat(L.r_in, 0, qn, W);
      if (rest == "mix.k") return mat(L.r_in, qn * W, qn, W);
      if (rest == "mix.v") return mat(L.r_in, 2 * qn * W, vn, W);
      if (rest == "mix.g") return mat(L.r_in, (2 * qn + vn) * W, vn, W);
      if (rest == "mix.o") return mat(L.r_o, 0, W, vn);
    }
    if (L.ffk == kDense) {
      if (rest == "mlp.gate") return mat(L.gu, 0, L.ff, W);
      if (rest == "mlp.up") return mat(L.gu, static_cast<size_t>(L.ff) * W, L.ff, W);
      if (rest == "mlp.down") return mat(L.down, 0, W, L.ff);
    } else if (L.ffk == kExperts) {
      if (rest == "mlp.table") { t.kind = 2; t.dst = L.table; t.rows = vocab_; t.cols = L.top; return t; }
      if (rest.compare(0, 5, "mlp.e") == 0) {
        const size_t d2 = rest.find('.', 5);
        if (d2 == std::string::npos) return t;
        const int e = atoi(rest.substr(5, d2 - 5).c_str());
        if (e < 0 || e >= L.experts) return t;
        const std::string which = rest.substr(d2 + 1);
        if (which == "up") return mat(L.eup, static_cast<size_t>(e) * L.ff * W, L.ff, W);
        if (which == "down") return mat(L.edown, static_cast<size_t>(e) * W * L.ff, W, L.ff);
      }
    }
    return t;
  }

  // Operand matrices and f32 vectors arrive as bf16 bit patterns; the expert table (`...mlp.table`) as int32.
  int load_weight(const char* name_c, const void* src_v, int64_t rows, int64_t cols, cudaStream_t st) override {
    NVLLM_CHECK_ARG(name_c && src_v, NVLLM_ERR_ARG, "load_weight: NULL");
    const std::string name(name_c);
    if (name == "loop.in" && !has_loop_) return 0;   // a checkpoint may carry it although no pass ever begins
    NVLLM_CHECK_ARG(needed_.count(name), NVLLM_ERR_ARG, "load_weight: tensor '%s' is not part of this model", name_c);
    const Target t = target_of(name);
    NVLLM_CHECK_ARG(t.kind >= 0, NVLLM_ERR_ARG, "load_weight: unknown tensor '%s'", name_c);
    NVLLM_CHECK_ARG(rows * cols == t.rows * t.cols && (t.kind == 1 || (rows == t.rows && cols == t.cols)), NVLLM_ERR_ARG,
                    "load_weight(%s): expected [%lld, %lld], got [%lld, %lld]", name_c, (long long)t.rows, (long long)t.cols, (long long)rows,
                    (long long)cols);
    const uint16_t* src = static_cast<const uint16_t*>(src_v);
    if (t.kind == 0) RUN(put(t.dst, t.off, src, rows, cols, st));
    else if (t.kind == 1) RUN(putf(static_cast<float*>(t.dst), src, rows * cols, st));
    else {
      const int32_t* tab = static_cast<const int32_t*>(src_v);
      const Layer& L = layers_[atoi(name.substr(1).c_str())];
      for (int64_t i = 0; i < rows * cols; ++i)
        NVLLM_CHECK_ARG(tab[i] >= 0 && tab[i] < L.experts, NVLLM_ERR_ARG, "load_weight(%s): entry %lld names expert %d of %d", name_c, (long long)i, tab[i], L.experts);
      NVLLM_CUDA(cudaMemcpyAsync(t.dst, tab, sizeof(int32_t) * rows * cols, cudaMemcpyHostToDevice, st));
      NVLLM_CUDA(cudaStreamSynchronize(st));
    }
    loaded_.insert(name);
    ready_ = loaded_.size() == needed_.size();
    return 0;
  }

  // Seeded synthetic weights (benchmarks, smoke runs): every needed tensor drawn on the host from a counter-based generator
  // and sent through load_weight, so that synthetic and checkpoint weights take the same path.
  int init_weights(uint64_t seed, float std, cudaStream_t st) override {
    auto mix = [](uint64_t x) {
      x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
      x ^= x >> 27; x *= 0x94D049BB133111EBull;
      x ^= x >> 31;
      return x;
    };
    auto to_bf16 = [](float f) {
      uint32_t u;
      memcpy(&u, &f, 4);
      return static_cast<uint16_t>((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
    };
    auto ends = [](const std::string& s, const char* suf) { const size_t n = strlen(suf); return s.size() >= n && s.compare(s.size() - n, n, suf) == 0; };
    std::vector<uint16_t> buf;
    std::vector<int32_t> tab;
    uint64_t tid = 0;
    for (const std::string& name : needed_) {
      ++tid;
      const Target t = target_of(name);
      NVLLM_CHECK_ARG(t.kind >= 0, NVLLM_ERR_STATE, "init_weights: no target for '%s'", name.c_str());
      if (t.kind == 2) {  // expert table: `top` distinct experts per token id
        const Layer& L = layers_[atoi(name.substr(1).c_str())];
        tab.resize(static_cast<size_t>(t.rows) * t.cols);
        for (int64_t r = 0; r < t.rows; ++r) {
          const int first = static_cast<int>(mix(seed ^ (tid << 40) ^ static_cast<uint64_t>(r + 1)) % L.experts);
          for (int64_t j = 0; j < t.cols; ++j) tab[r * t.cols + j] = static_cast<int32_t>((first + j) % L.experts);
        }
        RUN(load_weight(name.c_str(), tab.data(), t.rows, t.cols, st));
        continue;
      }
      buf.resize(static_cast<size_t>(t.rows) * t.cols);
      const bool norm_w = name.find("norm") != std::string::npos, is_d = ends(name, ".D"), is_alog = ends(name, ".A_log"), is_dtb = ends(name, ".dt_bias");
      const bool is_conv = ends(name, ".conv");
      for (size_t i = 0; i < buf.size(); ++i) {
        const uint64_t hsh = mix(seed ^ (tid << 40) ^ (i + 1) * 0x9E3779B97F4A7C15ull);
        const int s = static_cast<int>((hsh & 0xffff) + ((hsh >> 16) & 0xffff) + ((hsh >> 32) & 0xffff) + (hsh >> 48)) - 131070;
        const float g = static_cast<float>(s) * 2.6428998e-05f;  // ~N(0, 1)
        float v = g * std;
        if (norm_w || is_d) v = 1.0f + 0.1f * g;
        else if (is_alog) v = 0.5f * g;
        else if (is_dtb) v = -1.0f + 0.5f * g;
        else if (is_conv) v = 0.5f * g;
        buf[i] = to_bf16(v);
      }
      RUN(load_weight(name.c_str(), buf.data(), t.rows, t.cols, st));
    }
    return 0;
  }

  // ---- forward ---------------------------------------------------------------------------------------------------
  struct Pending {  // branch outputs of the previous layer, still to be added to the stream
    const void* a[3] = {nullptr, nullptr, nullptr};
    float s[3] = {0.f, 0.f, 0.f};
    int dt[3] = {NVLLM_F32, NVLLM_F32, NVLLM_F32};
    const float* bias = nullptr;
    float sb = 0.f;
    bool any() const { return a[0] || a[1] || a[2] || bias; }
  };

  int forward(const StepView& v) override {
    void* st = v.stream;
    const int N = v.n_tokens, W = width_, S = v.n_seqs;
    launches = 0;
    NVLLM_CHECK_ARG(v.cu_tokens && v.seq_slots && v.tables, NVLLM_ERR_ARG, "Talapel forward: the step carries no token ranges / state slots / block tables");
    auto mk = [&](const char* name) { if (v.mark) v.mark(v.mark_ctx, name); };
    auto lin = [&](void* y, const void* x, const void* w, int n, int k, int64_t ldy, int out_dt, const char* name) {
      ++launches;
      const int rc = nvllm_linear(y, x, w, N, n, k, k, k, ldy, 1, 0, 0, 0, dt_, out_dt, st);
      mk(name);
      return rc;
    };
    // h += pending branch outputs; normed = ln(h) * w (w null: only the sum)
    auto add_norm = [&](Pending& p, const float* w, const char* name) {
      if (!p.any() && w == nullptr) return 0;
      ++launches;
      const int rc = nvllm_residual_layernorm(w ? normed_ : nullptr, h_, p.a[0], p.s[0], p.dt[0], p.a[1], p.s[1], p.dt[1], p.a[2], p.s[2], p.dt[2],
                                              p.bias, p.sb, w, N, W, eps_, dt_, st);
      mk(name);
      p = Pending();
      return rc;
    };
    RUN(nvllm_embedding_gather_scaled(h_, has_loop_ ? x0_ : nullptr, embed_, v.ids, N, W, vocab_, embed_scale_, dt_, st)); ++launches; mk("embedding_gather_scaled");
    Pending pend;
    for (size_t r = 0; r < runs_.size(); ++r) {
      const Layer& L = layers_[runs_[r].first];
      const RunState& rs = state_[r];
      if (runs_[r].second) {  // a pass begins: x <- W_loop [x ; x0]
        RUN(add_norm(pend, nullptr, "residual sum"));
        RUN(nvllm_concat_cast(cat_, h_, x0_, N, W, W, dt_, st)); ++launches; mk("concat_cast");
        RUN(lin(h_, cat_, loop_in_, W, 2 * W, W, NVLLM_F32, "loop input projection"));
      }
      RUN(add_norm(pend, L.norm1, "residual_layernorm"));
      if (L.mix == kParallel) {
        // --- attention: [q | k | v | g] in one projection (f32 rows), biases + cache store, attention with the gate fused, Wo
        const int qn = L.H * L.D, kn = L.G * L.D, vn = L.G * L.V, gn = L.H * L.V, lda = pad8(L.a_cols());
        RUN(lin(proj_, normed_, L.a_in, lda, W, lda, NVLLM_F32, "attention q k v g projection"));
        RUN(nvllm_attn_bias_store(q_, qn, rs.kc, rs.vc, kn, vn, proj_, lda, L.qb, L.kb, L.vb, v.slots, N, qn, kn, vn, dt_, st)); ++launches; mk("attn_bias_store");
        RUN(nvllm_capped_attention(mix_in_, gn, q_, qn, proj_ + qn + kn + vn, lda, rs.kc, rs.vc, kn, vn, v.tok_seq, v.positions, v.tables,
                                   v.table_cap, lim_.block_size, N, L.H, L.G, L.D, L.V, L.scale, L.softcap, L.temp_coef, L.temp_every, v.cu_tokens, S, dt_, st)); ++launches; mk("capped_attention");
        RUN(lin(left_out_, mix_in_, L.a_o, W, gn, W, NVLLM_F32, "attention output projection"));
        // --- ssd: [z | x | B | C | dt] in one projection, convolution + SiLU over (x, B, C), recurrence, gated norm, Wo
        const int inner = L.s_inner(), gns = L.sG * L.sN, ch = L.s_ch(), lds = pad8(L.s_cols());
        RUN(lin(proj_, normed_, L.s_in, lds, W, lds, NVLLM_F32, "ssd input projection"));
        RUN(nvllm_causal_conv(conv_out_, ch, proj_ + inner, lds, L.conv_w, L.conv_b, rs.conv, v.tok_seq, v.seq_slots, v.cu_tokens, v.positions, N, S,
                              ch, L.taps, 1, st)); launches += L.taps > 1 ? 2 : 1; mk("causal_conv");
        RUN(nvllm_ssd_prepare(step_, decay_t_, proj_ + inner + ch, lds, L.dt_bias, L.a_log, N, L.sH, st)); ++launches; mk("ssd_prepare");
        RUN(nvllm_linear_recurrence(y_, inner, conv_out_ + inner + gns, ch, conv_out_ + inner, ch, conv_out_, ch, decay_t_, 1, step_, 1, L.skip,
                                    rs.ssd, v.seq_slots, v.cu_tokens, v.positions, S, L.sH, L.sG, L.sN, L.sP, st)); ++launches; mk("linear_recurrence (ssd)");
        RUN(nvllm_gated_group_norm(mix_in_, inner, y_, inner, proj_, lds, L.s_norm, N, inner, L.norm_groups, eps_, 1, dt_, st)); ++launches; mk("gated_group_norm");
        RUN(lin(right_out_, mix_in_, L.s_o, W, inner, W, NVLLM_F32, "ssd output projection"));
        pend.a[0] = left_out_; pend.s[0] = L.left_scale;
        pend.a[1] = right_out_; pend.s[1] = L.right_scale;
        pend.bias = L.ob; pend.sb = L.left_scale;
      } else {
        // --- retention: [q | k | v | g] in one projection, rotary on q and k, recurrence (k scaled), per-head norm + gate, Wo
        const int qn = L.rH * L.rD, vn = L.rH * L.rV, ldr = pad8(L.r_cols());
        RUN(lin(proj_, normed_, L.r_in, ldr, W, ldr, NVLLM_F32, "retention q k v g projection"));
        // q and k heads lie side by side: one launch rotates both; the key scale dim^-1/2 rides in the recurrence as its step
        RUN(nvllm_rotate_half(proj_, ldr, v.positions, L.rope, lim_.max_positions, N, 2 * L.rH, L.rD, L.rot_dims, 1.0f, st)); ++launches; mk("rotate_half (q, k)");
        RUN(nvllm_linear_recurrence(y_, vn, proj_, ldr, proj_ + qn, ldr, proj_ + 2 * qn, ldr, L.decay, 0, L.kscale, 0, nullptr, rs.ret, v.seq_slots,
                                    v.cu_tokens, v.positions, S, L.rH, L.rH, L.rD, L.rV, st)); ++launches; mk("linear_recurrence (retention)");
        RUN(nvllm_gated_group_norm(mix_in_, vn, y_, vn, proj_ + 2 * qn + vn, ldr, nullptr, N, vn, L.rH, eps_, 0, dt_, st)); ++launches; mk("gated_group_norm");
        RUN(lin(left_out_, mix_in_, L.r_o, W, vn, W, NVLLM_F32, "retention output projection"));
        pend.a[0] = left_out_; pend.s[0] = 1.0f;
      }
      if (L.ffk == kDense) {
        if (dt_ == NVLLM_BF16 && L.ff % 128 == 0 && W % 64 == 0) {  // SiLU gate in the GEMM's epilogue: [N, 2 ff] never reaches HBM
          RUN(nvllm_gemm_silu_mul_bf16(act_, normed_, L.gu, N, L.ff, W, W, W, L.ff, nullptr, 0, st)); ++launches; mk("gate_up projection + SiLU gate");
        } else {
          RUN(lin(gu_buf_, normed_, L.gu, 2 * L.ff, W, 2 * L.ff, dt_, "gate_up projection"));
          RUN(nvllm_ff_activation(act_, gu_buf_, N, L.ff, 0, dt_, st)); ++launches; mk("ff_activation (silu gate)");
        }
        RUN(lin(ff_out_, act_, L.down, W, L.ff, W, NVLLM_F32, "down projection"));
        pend.a[2] = ff_out_; pend.s[2] = 1.0f; pend.dt[2] = NVLLM_F32;
      } else if (L.ffk == kExperts) {
        RUN(nvllm_moe_table_route(topk_idx_, topk_w_, L.table, v.ids, N, L.top, vocab_, st)); ++launches; mk("moe_table_route");
        const int rows = nvllm_moe_max_rows(N, L.top, L.experts, L.tile_rows);
        RUN(nvllm_moe_sort(row_token_, tile_expert_, slot_row_, topk_idx_, N, L.top, L.experts, rows, L.tile_rows, st)); ++launches; mk("moe_sort");
        if (L.tile_rows == 128) {
          RUN(nvllm_gather_rows(xg_, normed_, row_token_, rows, W, N, dt_, st)); ++launches; mk("expert row gather");
          RUN(nvllm_gemm_bf16_grouped(eup_buf_, xg_, L.eup, rows, L.ff, W, L.experts, W, W, L.ff, tile_expert_, st)); ++launches; mk("expert up grouped GEMM");
          RUN(nvllm_ff_activation(act_, eup_buf_, rows, L.ff, 1, dt_, st)); ++launches; mk("ff_activation (relu^2)");
          RUN(nvllm_gemm_bf16_grouped(eout_, act_, L.edown, rows, W, L.ff, L.experts, L.ff, L.ff, W, tile_expert_, st)); ++launches; mk("expert down grouped GEMM");
        } else {
          RUN(nvllm_linear_grouped(act_, normed_, L.eup, rows, L.ff, W, W, W, L.ff, static_cast<int64_t>(L.ff) * W, row_token_, tile_expert_, 2,
                                   0.f, dt_, dt_, st)); ++launches; mk("expert up + relu^2 grouped tile kernel");
          RUN(nvllm_linear_grouped(eout_, act_, L.edown, rows, W, L.ff, L.ff, L.ff, W, static_cast<int64_t>(W) * L.ff, nullptr, tile_expert_, 0,
                                   0.f, dt_, dt_, st)); ++launches; mk("expert down grouped tile kernel");
        }
        RUN(nvllm_moe_combine(ff_out_, eout_, normed_, nullptr, topk_idx_, topk_w_, slot_row_, N, W, L.top, L.experts, dt_, st)); ++launches; mk("moe_combine");
        pend.a[2] = ff_out_; pend.s[2] = 1.0f; pend.dt[2] = dt_;
      }
      if (v.layer_tap != nullptr && !v.capturing) {
        RUN(add_norm(pend, nullptr, "residual sum"));
        NVLLM_CUDA(cudaMemcpyAsync(v.layer_tap + r * static_cast<size_t>(N) * W, h_, static_cast<size_t>(N) * W * 4, cudaMemcpyDeviceToHost,
                                   static_cast<cudaStream_t>(st)));
      }
    }
    RUN(add_norm(pend, final_norm_, "residual_layernorm"));
    if (v.n_logit_rows > 0) {
      if (v.n_logit_rows > head_rows_) {
        NVLLM_CHECK_ARG(!v.capturing, NVLLM_ERR_STATE, "forward: logit rows grew inside a graph capture");
        NVLLM_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(st)));
        head_rows_ = std::max(v.n_logit_rows, lim_.max_seqs);
        RUN(oalloc(&head_in_, static_cast<size_t>(head_rows_) * W));
      }
      RUN(nvllm_gather_rows(head_in_, normed_, v.logit_rows, v.n_logit_rows, W, N, dt_, st)); ++launches; mk("gather_rows");
      ++launches;
      RUN(nvllm_linear(v.logits, head_in_, head_, v.n_logit_rows, vocab_, W, W, W, vocab_, 1, 0, 0, 0, dt_, NVLLM_F32, st));
      mk("head projection");
    }
    return 0;
  }
};

}  // namespace

ModelImpl* make_talapel(const json::Value& cfg) {
  Talapel* m = new Talapel();
  if (m->parse(cfg) != 0) { delete m; return nullptr; }
  return m;
}

}  // namespace nvllm
