// Native CPU engine for Qwen2 / Qwen3 (dense) and Qwen3-MoE checkpoints in GGUF: the model runs straight from the file's (memory-mapped) ggml
// blocks, single process, a pool of worker threads.  It is the counterpart of the reference's CPU engine
// (common/transformer.h: transformer_load :1598, transformer_forward_pos :3499-3548, layer loop :3550-4174, Q8_0 dot
// tf_qmatvec_worker :648-738, sampler :5415-5467) for the configuration that has no GPU in it: Qwen3-0.6B, Q8_0, batch 1.
//
// Numerics follow the reference's fp32 path so that greedy decoding picks the same tokens: fp32 activations, weights decoded
// block by block (Q8_0: d * q), RMSNorm x * rsqrt(mean(x^2) + eps) * w, per-head QK-RMSNorm, NeoX RoPE with
// inv_freq[j] = theta^(-2j / d), fp32 softmax, SiLU(gate) * up, arg-max with ties to the lower id.
//
// What differs is the schedule.  The reference prefills a prompt as n sequential single-token forwards, i.e. it streams every
// weight n times; here the prompt is one batched pass: every weight row is decoded once into registers / L1 and multiplied with
// all prompt tokens, attention is causal over the batch, and only the last token goes through the LM head.  Decode steps are
// GEMVs over the raw blocks (AVX2: int8 -> fp32 in registers, FMA against the activations) split over the threads by rows.
#include "common.h"
#include "ggml_types.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <chrono>
#include <string>
#include <vector>
#if defined(__AVX2__)
#include <immintrin.h>
#endif
#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>
#include <sys/mman.h>

extern "C" {
void* gbh_gguf_open(const char* path);
void gbh_gguf_close(void* h);
int gbh_gguf_find_tensor(void* h, const char* name);
int gbh_gguf_tensor_info(void* h, int i, char* name, int name_cap, int* n_dims, uint64_t* dims4, int* type, uint64_t* nbytes);
const void* gbh_gguf_tensor_data(void* h, int i);
int gbh_gguf_find_key(void* h, const char* key);
int gbh_gguf_kv_scalar(void* h, int i, double* out);
int gbh_gguf_kv_info(void* h, int i, char* key, int key_cap, int* type, int* elem_type, uint64_t* count);
const void* gbh_gguf_kv_array_data(void* h, int i);
const char* gbh_gguf_kv_string(void* h, int i, long j, uint64_t* len);
}

namespace gbh {

int dequant_row(int type, const void* src, float* dst, long n);

namespace {

// Persistent workers: run(n, fn) calls fn(begin, end) on contiguous slices of [0, n), one per thread (the caller takes a slice too),
// and returns when all are done.  Workers spin for a short while between jobs (a decode step issues hundreds of small jobs), then
// sleep on a condition variable.  Counterpart of the reference's thread pool (common/transformer.h:2259-2344).
inline void cpu_relax() {
#if defined(__x86_64__)
  __builtin_ia32_pause();
#endif
}

class Pool {
 public:
  explicit Pool(int n) : n_(std::max(1, n)) {
    for (int i = 1; i < n_; ++i) workers_.emplace_back([this, i] { loop(i); });
  }
  ~Pool() {
    { std::lock_guard<std::mutex> g(mu_); stop_ = true; ++gen_; }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
  }
  int size() const { return n_; }
  void run(int n, const std::function<void(int, int)>& fn) {
    if (n_ == 1 || n <= 1) { fn(0, n); return; }
    { std::lock_guard<std::mutex> g(mu_); fn_ = &fn; total_ = n; pending_.store(n_ - 1); ++gen_; }
    cv_.notify_all();
    slice(0);
    while (pending_.load(std::memory_order_acquire) != 0) cpu_relax();       // the slices are equal, the others finish about now
  }
 private:
  void slice(int i) {
    const int b = (int)((long)total_ * i / n_), e = (int)((long)total_ * (i + 1) / n_);
    if (e > b) (*fn_)(b, e);
  }
  void loop(int i) {
    unsigned long seen = 0;
    for (;;) {
      // a decode step issues a job every few tens of microseconds: keep spinning for about a millisecond before going to sleep
      for (int spin = 0; spin < 60000 && gen_.load(std::memory_order_acquire) == seen; ++spin) cpu_relax();
      if (gen_.load(std::memory_order_acquire) == seen) {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return gen_.load() != seen; });
      }
      seen = gen_.load(std::memory_order_acquire);
      if (stop_) return;
      slice(i);
      pending_.fetch_sub(1, std::memory_order_release);
    }
  }
  int n_;
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::atomic<unsigned long> gen_{0};
  std::atomic<int> pending_{0};
  const std::function<void(int, int)>* fn_ = nullptr;
  int total_ = 0;
  bool stop_ = false;
};

struct QMat {                      // a [rows, k] matrix as it sits in the file
  const uint8_t* data = nullptr;
  int type = 0, rows = 0, k = 0;
  long row_bytes = 0;
};

struct Layer {
  std::vector<float> attn_norm, ffn_norm, q_norm, k_norm, bq, bk, bv;
  QMat wq, wk, wv, wo, wgate, wup, wdown;
  QMat wrouter;                    // MoE layers: [n_experts, hidden]
  std::vector<QMat> eg, eu, ed;    // per expert: gate / up [expert_ffn, hidden], down [hidden, expert_ffn] (slices of the 3-D tensors)
  QMat sh_gate, sh_up, sh_down;    // shared expert (qwen35moe), added to the routed output times sigmoid(sh_inp . x)
  std::vector<float> sh_inp;
  // gated Delta-Net layers of the hybrid models: projections of the layer input, the causal convolution over q | k | v, the
  // per-head decay and write strength, the output norm and projection; and the running state of the one sequence the engine holds
  bool is_ssm = false;
  QMat s_qkv, s_z, s_alpha, s_beta, s_out;
  std::vector<float> conv_w, s_norm, s_a, s_dt;
  std::vector<float> ring;         // the last d_conv - 1 rows of q | k | v in front of the convolution
  std::vector<float> state;        // [v heads][head_dim (value)][head_dim (key)]
};

struct CpuEngine {
  void* gguf = nullptr;
  int n_layers = 0, hidden = 0, n_heads = 0, n_kv = 0, head_dim = 0, ffn = 0, vocab = 0, max_seq = 0, threads = 1;
  int n_experts = 0, n_used = 0, expert_ffn = 0;     // > 0: every layer's FFN is a routed mixture (qwen3moe, qwen35moe)
  int shared_ffn = 0;                                // > 0: plus a shared expert of this width
  // hybrid models (qwen35, qwen35moe): every full_interval-th layer is gated attention, the others are Delta-Net layers
  int full_interval = 0, rope_dim = 0, d_conv = 4, ssm_kh = 0, ssm_vh = 0, ssm_d = 0;
  bool attn_gate = false;
  int ssm_pos = 0;                                   // position the recurrent state stands at
  float eps = 1e-6f, theta = 1e6f;
  bool qk_norm = false, has_bias = false;
  std::vector<Layer> layers;
  std::vector<float> final_norm, inv_freq;
  QMat embed, head;
  std::vector<float> kc, vc;       // [layer][kv head][pos][head_dim]: the positions of one head are contiguous, a decode step streams them
  double t_prefill = 0, t_decode = 0;
  // seconds per phase since the last reset (gbh_cpu_engine_profile): qkv, rope + cache write, attention, o_proj, norms + residual adds,
  // gate / up + SiLU, down, head (final norm + LM head), embedding
  double prof[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  Pool* pool = nullptr;
  void* huge = nullptr;            // the matrices copied out of the file mapping into 2 MB pages (see place_weights)
  size_t huge_bytes = 0;
  ~CpuEngine() { delete pool; if (huge != nullptr) munmap(huge, huge_bytes); }
};

float dot_f32(const float* a, const float* b, int n) {
#if defined(__AVX2__)
  __m256 s0 = _mm256_setzero_ps(), s1 = _mm256_setzero_ps();
  int i = 0;
  for (; i + 16 <= n; i += 16) {
    s0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), s0);
    s1 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 8), _mm256_loadu_ps(b + i + 8), s1);
  }
  s0 = _mm256_add_ps(s0, s1);
  __m128 lo = _mm_add_ps(_mm256_castps256_ps128(s0), _mm256_extractf128_ps(s0, 1));
  lo = _mm_add_ps(lo, _mm_movehl_ps(lo, lo));
  lo = _mm_add_ss(lo, _mm_shuffle_ps(lo, lo, 1));
  float s = _mm_cvtss_f32(lo);
  for (; i < n; ++i) s += a[i] * b[i];
  return s;
#else
  float s = 0.f;
  for (int i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
#endif
}

// Four rows against one vector: every load of x feeds four FMA chains (the batched prefill is bound by re-reading the tokens).
void dot4_f32(const float* r0, const float* r1, const float* r2, const float* r3, const float* x, int n, float* out) {
#if defined(__AVX2__)
  __m256 a0 = _mm256_setzero_ps(), a1 = a0, a2 = a0, a3 = a0;
  int i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m256 xv = _mm256_loadu_ps(x + i);
    a0 = _mm256_fmadd_ps(_mm256_loadu_ps(r0 + i), xv, a0);
    a1 = _mm256_fmadd_ps(_mm256_loadu_ps(r1 + i), xv, a1);
    a2 = _mm256_fmadd_ps(_mm256_loadu_ps(r2 + i), xv, a2);
    a3 = _mm256_fmadd_ps(_mm256_loadu_ps(r3 + i), xv, a3);
  }
  const __m256 acc[4] = {a0, a1, a2, a3};
  const float* rows[4] = {r0, r1, r2, r3};
  for (int r = 0; r < 4; ++r) {
    __m128 lo = _mm_add_ps(_mm256_castps256_ps128(acc[r]), _mm256_extractf128_ps(acc[r], 1));
    lo = _mm_add_ps(lo, _mm_movehl_ps(lo, lo));
    lo = _mm_add_ss(lo, _mm_shuffle_ps(lo, lo, 1));
    float s = _mm_cvtss_f32(lo);
    for (int k2 = i; k2 < n; ++k2) s += rows[r][k2] * x[k2];
    out[r] = s;
  }
#else
  out[0] = dot_f32(r0, x, n); out[1] = dot_f32(r1, x, n); out[2] = dot_f32(r2, x, n); out[3] = dot_f32(r3, x, n);
#endif
}

// Four rows against two vectors: a 4 x 2 register tile (eight accumulators, four row loads and two token loads per step) keeps the
// FMA units busier than the loads.  Every (row, token) sum is accumulated in the order of dot4_f32, so the results are the same bits.
void dot4x2_f32(const float* r0, const float* r1, const float* r2, const float* r3, const float* xa, const float* xb, int n, float* oa,
                float* ob) {
#if defined(__AVX2__)
  __m256 a0 = _mm256_setzero_ps(), a1 = a0, a2 = a0, a3 = a0, b0 = a0, b1 = a0, b2 = a0, b3 = a0;
  int i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m256 va = _mm256_loadu_ps(xa + i), vb = _mm256_loadu_ps(xb + i);
    __m256 w = _mm256_loadu_ps(r0 + i);
    a0 = _mm256_fmadd_ps(w, va, a0); b0 = _mm256_fmadd_ps(w, vb, b0);
    w = _mm256_loadu_ps(r1 + i);
    a1 = _mm256_fmadd_ps(w, va, a1); b1 = _mm256_fmadd_ps(w, vb, b1);
    w = _mm256_loadu_ps(r2 + i);
    a2 = _mm256_fmadd_ps(w, va, a2); b2 = _mm256_fmadd_ps(w, vb, b2);
    w = _mm256_loadu_ps(r3 + i);
    a3 = _mm256_fmadd_ps(w, va, a3); b3 = _mm256_fmadd_ps(w, vb, b3);
  }
  const __m256 acc[8] = {a0, a1, a2, a3, b0, b1, b2, b3};
  const float* rows[4] = {r0, r1, r2, r3};
  for (int j = 0; j < 8; ++j) {
    __m128 lo = _mm_add_ps(_mm256_castps256_ps128(acc[j]), _mm256_extractf128_ps(acc[j], 1));
    lo = _mm_add_ps(lo, _mm_movehl_ps(lo, lo));
    lo = _mm_add_ss(lo, _mm_shuffle_ps(lo, lo, 1));
    float sum = _mm_cvtss_f32(lo);
    const float* x = j < 4 ? xa : xb;
    for (int k2 = i; k2 < n; ++k2) sum += rows[j & 3][k2] * x[k2];
    (j < 4 ? oa : ob)[j & 3] = sum;
  }
#else
  dot4_f32(r0, r1, r2, r3, xa, n, oa);
  dot4_f32(r0, r1, r2, r3, xb, n, ob);
#endif
}

// One row of a Q8_0 matrix times an fp32 vector: per 32-block  d * sum(q * x).  Two blocks per iteration (independent FMA
// chains), the fp16 scales converted by the F16C unit.
float dot_q8_0(const uint8_t* row, const float* x, int k) {
  float total = 0.f;
  const int nb = k / 32;
#if defined(__AVX2__) && defined(__F16C__)
  __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
  auto block = [&](const uint8_t* blk, const float* xb, __m256& acc) {
    uint16_t dh; memcpy(&dh, blk, 2);
    const __m256 d = _mm256_set1_ps(_cvtsh_ss(dh));
    __m256 s0 = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i*)(blk + 2)))), _mm256_loadu_ps(xb));
    __m256 s1 = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i*)(blk + 10)))), _mm256_loadu_ps(xb + 8));
    s0 = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i*)(blk + 18)))), _mm256_loadu_ps(xb + 16), s0);
    s1 = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i*)(blk + 26)))), _mm256_loadu_ps(xb + 24), s1);
    acc = _mm256_fmadd_ps(d, _mm256_add_ps(s0, s1), acc);
  };
  int b = 0;
  for (; b + 2 <= nb; b += 2) {
    block(row + (size_t)b * 34, x + b * 32, acc0);
    block(row + (size_t)(b + 1) * 34, x + (b + 1) * 32, acc1);
  }
  if (b < nb) block(row + (size_t)b * 34, x + b * 32, acc0);
  acc0 = _mm256_add_ps(acc0, acc1);
  __m128 lo = _mm_add_ps(_mm256_castps256_ps128(acc0), _mm256_extractf128_ps(acc0, 1));
  lo = _mm_add_ps(lo, _mm_movehl_ps(lo, lo));
  lo = _mm_add_ss(lo, _mm_shuffle_ps(lo, lo, 1));
  total = _mm_cvtss_f32(lo);
#else
  for (int b = 0; b < nb; ++b) {
    const uint8_t* blk = row + (size_t)b * 34;
    uint16_t dh; memcpy(&dh, blk, 2);
    float s = 0.f;
    for (int j = 0; j < 32; ++j) s += (float)(int8_t)blk[2 + j] * x[b * 32 + j];
    total += fp16_to_f32(dh) * s;
  }
#endif
  return total;
}

#if defined(__x86_64__)
// AVX-512 variants, compiled for their target by attribute and chosen at run time (the library itself is built for AVX2 machines):
// 16 lanes per instruction halve the instruction count of the two kernels the engine spends its time in.  GB_CPU_AVX512=0 keeps AVX2.
#define GB_AVX512 __attribute__((target("avx512f,avx512bw,avx512vl,avx512dq,f16c,fma")))

GB_AVX512 float dot_q8_0_avx512(const uint8_t* row, const float* x, int k) {
  const int nb = k / 32;
  __m512 acc0 = _mm512_setzero_ps(), acc1 = _mm512_setzero_ps();
  auto block = [&](const uint8_t* blk, const float* xb, __m512& acc) GB_AVX512 {
    uint16_t dh; memcpy(&dh, blk, 2);
    const __m512 d = _mm512_set1_ps(_cvtsh_ss(dh));
    const __m512 lo = _mm512_cvtepi32_ps(_mm512_cvtepi8_epi32(_mm_loadu_si128((const __m128i*)(blk + 2))));
    const __m512 hi = _mm512_cvtepi32_ps(_mm512_cvtepi8_epi32(_mm_loadu_si128((const __m128i*)(blk + 18))));
    __m512 sum = _mm512_mul_ps(lo, _mm512_loadu_ps(xb));
    sum = _mm512_fmadd_ps(hi, _mm512_loadu_ps(xb + 16), sum);
    acc = _mm512_fmadd_ps(d, sum, acc);
  };
  int b = 0;
  for (; b + 2 <= nb; b += 2) {
    block(row + (size_t)b * 34, x + b * 32, acc0);
    block(row + (size_t)(b + 1) * 34, x + (b + 1) * 32, acc1);
  }
  if (b < nb) block(row + (size_t)b * 34, x + b * 32, acc0);
  return _mm512_reduce_add_ps(_mm512_add_ps(acc0, acc1));
}

// 4 rows x 4 tokens: sixteen accumulators, four row loads and four token loads per step of 16 features
GB_AVX512 void dot4x4_f32_avx512(const float* r0, const float* r1, const float* r2, const float* r3, const float* const* xs, int n, float* out) {
  __m512 a[16];
  for (int j = 0; j < 16; ++j) a[j] = _mm512_setzero_ps();
  int i = 0;
  for (; i + 16 <= n; i += 16) {
    const __m512 w0 = _mm512_loadu_ps(r0 + i), w1 = _mm512_loadu_ps(r1 + i), w2 = _mm512_loadu_ps(r2 + i), w3 = _mm512_loadu_ps(r3 + i);
#pragma GCC unroll 4
    for (int t = 0; t < 4; ++t) {
      const __m512 xv = _mm512_loadu_ps(xs[t] + i);
      a[t * 4 + 0] = _mm512_fmadd_ps(w0, xv, a[t * 4 + 0]);
      a[t * 4 + 1] = _mm512_fmadd_ps(w1, xv, a[t * 4 + 1]);
      a[t * 4 + 2] = _mm512_fmadd_ps(w2, xv, a[t * 4 + 2]);
      a[t * 4 + 3] = _mm512_fmadd_ps(w3, xv, a[t * 4 + 3]);
    }
  }
  const float* rows[4] = {r0, r1, r2, r3};
  for (int t = 0; t < 4; ++t)
    for (int q = 0; q < 4; ++q) {
      float sum = _mm512_reduce_add_ps(a[t * 4 + q]);
      for (int k2 = i; k2 < n; ++k2) sum += rows[q][k2] * xs[t][k2];
      out[t * 4 + q] = sum;                                   // out[token][row]
    }
}

bool use_avx512() {
  static const bool on = [] {
    const char* e = getenv("GB_CPU_AVX512");
    if (e != nullptr && e[0] == '0') return false;
    return __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512vl") &&
           __builtin_cpu_supports("avx512dq");
  }();
  return on;
}
#else
inline bool use_avx512() { return false; }
#endif

inline float dot_q8_0_best(const uint8_t* row, const float* x, int k) {
#if defined(__x86_64__)
  if (use_avx512()) return dot_q8_0_avx512(row, x, k);
#endif
  return dot_q8_0(row, x, k);
}

// Rows [n0, n1) of y[t, n] = sum_k W[n, k] x[t, k] for t < T.  With several tokens a row is decoded once (four at a time into `row`)
// and multiplied with the tokens two at a time; a single token streams Q8_0 rows straight from their blocks.
void matmul_rows(const QMat& w, const float* x, int ldx, int T, float* y, int ldy, const float* bias, int n0, int n1, std::vector<float>& row) {
  int n = n0;
  const size_t k = (size_t)w.k;
  if (T > 1) {
    if (row.size() < 4 * k) row.resize(4 * k);
    float* r = row.data();
    for (; n + 4 <= n1; n += 4) {                            // four decoded rows share every token load
      for (int q = 0; q < 4; ++q) dequant_row(w.type, w.data + (size_t)(n + q) * w.row_bytes, r + q * k, w.k);
      const float b4[4] = {bias ? bias[n] : 0.f, bias ? bias[n + 1] : 0.f, bias ? bias[n + 2] : 0.f, bias ? bias[n + 3] : 0.f};
      int t = 0;
#if defined(__x86_64__)
      if (use_avx512())
        for (; t + 4 <= T; t += 4) {
          const float* xs[4] = {x + (size_t)t * ldx, x + (size_t)(t + 1) * ldx, x + (size_t)(t + 2) * ldx, x + (size_t)(t + 3) * ldx};
          float o16[16];
          dot4x4_f32_avx512(r, r + k, r + 2 * k, r + 3 * k, xs, w.k, o16);
          for (int tt = 0; tt < 4; ++tt)
            for (int q = 0; q < 4; ++q) y[(size_t)(t + tt) * ldy + n + q] = o16[tt * 4 + q] + b4[q];
        }
#endif
      for (; t + 2 <= T; t += 2) {
        float oa[4], ob[4];
        dot4x2_f32(r, r + k, r + 2 * k, r + 3 * k, x + (size_t)t * ldx, x + (size_t)(t + 1) * ldx, w.k, oa, ob);
        for (int q = 0; q < 4; ++q) { y[(size_t)t * ldy + n + q] = oa[q] + b4[q]; y[(size_t)(t + 1) * ldy + n + q] = ob[q] + b4[q]; }
      }
      if (t < T) {
        float o4[4];
        dot4_f32(r, r + k, r + 2 * k, r + 3 * k, x + (size_t)t * ldx, w.k, o4);
        for (int q = 0; q < 4; ++q) y[(size_t)t * ldy + n + q] = o4[q] + b4[q];
      }
    }
  }
  for (; n < n1; ++n) {
    const uint8_t* src = w.data + (size_t)n * w.row_bytes;
    const float b = bias ? bias[n] : 0.f;
    if (T == 1 && w.type == T_Q8_0) { y[n] = dot_q8_0_best(src, x, w.k) + b; continue; }
    if (row.size() < k) row.resize(k);
    dequant_row(w.type, src, row.data(), w.k);
    for (int t = 0; t < T; ++t) y[(size_t)t * ldy + n] = dot_f32(row.data(), x + (size_t)t * ldx, w.k) + b;
  }
}

// Several projections of the same input (q / k / v) as ONE job of the pool: their rows are laid end to end and split over the
// threads, so a decode step pays one wake-up and one join instead of three.
struct MatJob { const QMat* w; float* y; int ldy; const float* bias; };

void matmul_multi(const CpuEngine& e, const MatJob* jobs, int n_jobs, const float* x, int ldx, int T) {
  int total = 0;
  for (int j = 0; j < n_jobs; ++j) total += jobs[j].w->rows;
  e.pool->run(total, [&](int g0, int g1) {
    std::vector<float> row;
    int base = 0;
    for (int j = 0; j < n_jobs; ++j) {
      const int rows = jobs[j].w->rows;
      const int lo = std::max(g0, base) - base, hi = std::min(g1, base + rows) - base;
      if (hi > lo) matmul_rows(*jobs[j].w, x, ldx, T, jobs[j].y, jobs[j].ldy, jobs[j].bias, lo, hi, row);
      base += rows;
    }
  });
}

void matmul(const CpuEngine& e, const QMat& w, const float* x, int ldx, int T, float* y, int ldy, const float* bias = nullptr) {
  const MatJob j{&w, y, ldy, bias};
  matmul_multi(e, &j, 1, x, ldx, T);
}

// g[t, n] = SiLU(gate[n] . x[t]) * (up[n] . x[t]): the two FFN input projections and the activation as one job (a thread computes
// both sums of an output feature, so nothing is written in between).
void ffn_gate_up_silu(const CpuEngine& e, const QMat& wg, const QMat& wu, const float* x, int ldx, int T, float* g, int ldg) {
  e.pool->run(wg.rows, [&](int n0, int n1) {
    const size_t k = (size_t)wg.k;
    std::vector<float> rg, ru;
    auto act = [](float a, float b) { return a / (1.0f + expf(-a)) * b; };
    int n = n0;
    if (T > 1) {
      rg.resize(4 * k); ru.resize(4 * k);
      for (; n + 4 <= n1; n += 4) {
        for (int q = 0; q < 4; ++q) {
          dequant_row(wg.type, wg.data + (size_t)(n + q) * wg.row_bytes, rg.data() + q * k, wg.k);
          dequant_row(wu.type, wu.data + (size_t)(n + q) * wu.row_bytes, ru.data() + q * k, wu.k);
        }
        int t = 0;
#if defined(__x86_64__)
        if (use_avx512())
          for (; t + 4 <= T; t += 4) {
            const float* xs[4] = {x + (size_t)t * ldx, x + (size_t)(t + 1) * ldx, x + (size_t)(t + 2) * ldx, x + (size_t)(t + 3) * ldx};
            float g16[16], u16[16];
            dot4x4_f32_avx512(rg.data(), rg.data() + k, rg.data() + 2 * k, rg.data() + 3 * k, xs, wg.k, g16);
            dot4x4_f32_avx512(ru.data(), ru.data() + k, ru.data() + 2 * k, ru.data() + 3 * k, xs, wu.k, u16);
            for (int tt = 0; tt < 4; ++tt)
              for (int q = 0; q < 4; ++q) g[(size_t)(t + tt) * ldg + n + q] = act(g16[tt * 4 + q], u16[tt * 4 + q]);
          }
#endif
        for (; t + 2 <= T; t += 2) {
          float ga[4], gb[4], ua[4], ub[4];
          const float* xa = x + (size_t)t * ldx; const float* xb = x + (size_t)(t + 1) * ldx;
          dot4x2_f32(rg.data(), rg.data() + k, rg.data() + 2 * k, rg.data() + 3 * k, xa, xb, wg.k, ga, gb);
          dot4x2_f32(ru.data(), ru.data() + k, ru.data() + 2 * k, ru.data() + 3 * k, xa, xb, wu.k, ua, ub);
          for (int q = 0; q < 4; ++q) { g[(size_t)t * ldg + n + q] = act(ga[q], ua[q]); g[(size_t)(t + 1) * ldg + n + q] = act(gb[q], ub[q]); }
        }
        if (t < T) {
          float g4[4], u4[4];
          dot4_f32(rg.data(), rg.data() + k, rg.data() + 2 * k, rg.data() + 3 * k, x + (size_t)t * ldx, wg.k, g4);
          dot4_f32(ru.data(), ru.data() + k, ru.data() + 2 * k, ru.data() + 3 * k, x + (size_t)t * ldx, wu.k, u4);
          for (int q = 0; q < 4; ++q) g[(size_t)t * ldg + n + q] = act(g4[q], u4[q]);
        }
      }
    }
    for (; n < n1; ++n) {
      const uint8_t* sg = wg.data + (size_t)n * wg.row_bytes;
      const uint8_t* su = wu.data + (size_t)n * wu.row_bytes;
      if (T == 1 && wg.type == T_Q8_0 && wu.type == T_Q8_0) { g[n] = act(dot_q8_0_best(sg, x, wg.k), dot_q8_0_best(su, x, wu.k)); continue; }
      if (rg.size() < k) { rg.resize(k); ru.resize(k); }
      dequant_row(wg.type, sg, rg.data(), wg.k);
      dequant_row(wu.type, su, ru.data(), wu.k);
      for (int t = 0; t < T; ++t) g[(size_t)t * ldg + n] = act(dot_f32(rg.data(), x + (size_t)t * ldx, wg.k), dot_f32(ru.data(), x + (size_t)t * ldx, wu.k));
    }
  });
}

void rmsnorm(const float* x, const float* w, float* y, int n, float eps) {
  float ss = 0.f;
  for (int i = 0; i < n; ++i) ss += x[i] * x[i];
  const float s = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = 0; i < n; ++i) y[i] = x[i] * s * w[i];
}

void rope_neox(float* v, int d, int pos, const float* inv_freq) {
  const int half = d / 2;
  for (int j = 0; j < half; ++j) {
    const float a = (float)pos * inv_freq[j], c = cosf(a), s = sinf(a);
    const float x0 = v[j], x1 = v[j + half];
    v[j] = x0 * c - x1 * s;
    v[j + half] = x0 * s + x1 * c;
  }
}

int get_mat(void* g, const std::string& name, QMat* m, int want_rows, int want_k) {
  const int i = gbh_gguf_find_tensor(g, name.c_str());
  if (i < 0) return fail("cpu engine: tensor %s is missing", name.c_str());
  int nd, type; uint64_t dims[4], nbytes; char nm[8];
  gbh_gguf_tensor_info(g, i, nm, 8, &nd, dims, &type, &nbytes);
  if (nd != 2 || (int)dims[0] != want_k || (int)dims[1] != want_rows)
    return fail("cpu engine: %s has shape [%d, %d], wanted [%d, %d]", name.c_str(), (int)dims[1], (int)dims[0], want_rows, want_k);
  const TypeInfo* ti = type_info(type);
  if (ti == nullptr || want_k % ti->block) return fail("cpu engine: %s: unsupported tensor type %d", name.c_str(), type);
  m->data = (const uint8_t*)gbh_gguf_tensor_data(g, i); m->type = type; m->rows = want_rows; m->k = want_k;
  m->row_bytes = (long)(want_k / ti->block) * ti->bytes;
  return 0;
}

// The experts of a 3-D tensor [n_experts][rows][k] (ggml dims {k, rows, n_experts}) as one matrix each.
int get_experts(void* g, const std::string& name, std::vector<QMat>* out, int n_experts, int want_rows, int want_k) {
  const int i = gbh_gguf_find_tensor(g, name.c_str());
  if (i < 0) return fail("cpu engine: tensor %s is missing", name.c_str());
  int nd, type; uint64_t dims[4], nbytes; char nm[8];
  gbh_gguf_tensor_info(g, i, nm, 8, &nd, dims, &type, &nbytes);
  if (nd != 3 || (int)dims[0] != want_k || (int)dims[1] != want_rows || (int)dims[2] != n_experts)
    return fail("cpu engine: %s has shape [%d, %d, %d], wanted [%d, %d, %d]", name.c_str(), (int)dims[2], (int)dims[1], (int)dims[0], n_experts, want_rows, want_k);
  const TypeInfo* ti = type_info(type);
  if (ti == nullptr || want_k % ti->block) return fail("cpu engine: %s: unsupported tensor type %d", name.c_str(), type);
  const long rb = (long)(want_k / ti->block) * ti->bytes;
  const uint8_t* base = (const uint8_t*)gbh_gguf_tensor_data(g, i);
  out->resize((size_t)n_experts);
  for (int e = 0; e < n_experts; ++e) {
    QMat& m = (*out)[(size_t)e];
    m.data = base + (size_t)e * want_rows * rb; m.type = type; m.rows = want_rows; m.k = want_k; m.row_bytes = rb;
  }
  return 0;
}

int get_vec(void* g, const std::string& name, std::vector<float>* v, int n, bool optional = false) {
  const int i = gbh_gguf_find_tensor(g, name.c_str());
  if (i < 0) return optional ? 1 : fail("cpu engine: tensor %s is missing", name.c_str());
  int nd, type; uint64_t dims[4], nbytes; char nm[8];
  gbh_gguf_tensor_info(g, i, nm, 8, &nd, dims, &type, &nbytes);
  if ((int)dims[0] != n) return fail("cpu engine: %s has %d elements, wanted %d", name.c_str(), (int)dims[0], n);
  v->resize((size_t)n);
  return dequant_row(type, gbh_gguf_tensor_data(g, i), v->data(), n);
}

double kv_num(void* g, const std::string& key, double dflt) {
  const int i = gbh_gguf_find_key(g, key.c_str());
  double v = dflt;
  if (i >= 0) gbh_gguf_kv_scalar(g, i, &v);
  return v;
}

// Layers + final norm over T tokens at positions pos0 .. pos0 + T - 1 (rows of x, [T, hidden], updated in place).
struct Phase {                        // adds its lifetime to one slot of the profile
  double* slot;
  std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
  explicit Phase(double* s) : slot(s) {}
  ~Phase() { *slot += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count(); }
};

// Routed FFN of one layer over the rows h [T, hidden] -> o [T, hidden].  Router: softmax over all experts, the n_used largest
// (ties to the lower index), their weights renormalised to sum 1 (common/transformer.h:4050-4130).  A single token runs its
// experts one after the other, each matrix split over the threads by rows; a batch gathers the rows of each expert and runs them
// through the same register-tiled products as the dense FFN, then scatters the weighted results.
void moe_ffn(CpuEngine& e, const Layer& L, const float* h, int T, float* o) {
  const int H = e.hidden, E = e.n_experts, K = e.n_used, F = e.expert_ffn;
  std::vector<float> logits((size_t)T * E);
  matmul(e, L.wrouter, h, H, T, logits.data(), E);
  std::vector<int> pick((size_t)T * K);
  std::vector<float> wt((size_t)T * K);
  for (int t = 0; t < T; ++t) {
    float* lg = logits.data() + (size_t)t * E;
    float mx = lg[0];
    for (int i = 1; i < E; ++i) mx = std::max(mx, lg[i]);
    float sum = 0.f;
    for (int i = 0; i < E; ++i) { lg[i] = expf(lg[i] - mx); sum += lg[i]; }
    for (int i = 0; i < E; ++i) lg[i] /= sum;
    float chosen = 0.f;
    for (int k = 0; k < K; ++k) {
      int best = -1;
      for (int i = 0; i < E; ++i) {
        bool taken = false;
        for (int j = 0; j < k; ++j) taken = taken || pick[(size_t)t * K + j] == i;
        if (!taken && (best < 0 || lg[i] > lg[best])) best = i;
      }
      pick[(size_t)t * K + k] = best; wt[(size_t)t * K + k] = lg[best]; chosen += lg[best];
    }
    for (int k = 0; k < K; ++k) wt[(size_t)t * K + k] /= chosen;
  }
  for (size_t i = 0; i < (size_t)T * H; ++i) o[i] = 0.f;
  std::vector<float> xe, ge, ye;
  std::vector<int> rows; std::vector<float> rw;
  for (int ex = 0; ex < E; ++ex) {
    rows.clear(); rw.clear();
    for (int t = 0; t < T; ++t)
      for (int k = 0; k < K; ++k)
        if (pick[(size_t)t * K + k] == ex) { rows.push_back(t); rw.push_back(wt[(size_t)t * K + k]); }
    const int n = (int)rows.size();
    if (n == 0) continue;
    const float* xin = h;
    if (!(n == T)) {                                             // gather this expert's rows
      xe.resize((size_t)n * H);
      for (int r = 0; r < n; ++r) memcpy(xe.data() + (size_t)r * H, h + (size_t)rows[r] * H, sizeof(float) * H);
      xin = xe.data();
    }
    ge.resize((size_t)n * F); ye.resize((size_t)n * H);
    ffn_gate_up_silu(e, L.eg[(size_t)ex], L.eu[(size_t)ex], xin, H, n, ge.data(), F);
    matmul(e, L.ed[(size_t)ex], ge.data(), F, n, ye.data(), H);
    for (int r = 0; r < n; ++r) {
      float* dst = o + (size_t)rows[r] * H;
      const float* src = ye.data() + (size_t)r * H;
      const float w = rw[(size_t)r];
      for (int i = 0; i < H; ++i) dst[i] += w * src[i];
    }
  }
  if (e.shared_ffn > 0) {
    const int FS = e.shared_ffn;
    ge.resize((size_t)T * FS); ye.resize((size_t)T * H);
    ffn_gate_up_silu(e, L.sh_gate, L.sh_up, h, H, T, ge.data(), FS);
    matmul(e, L.sh_down, ge.data(), FS, T, ye.data(), H);
    for (int t = 0; t < T; ++t) {
      float g = 1.0f;
      if (!L.sh_inp.empty()) g = 1.0f / (1.0f + expf(-dot_f32(L.sh_inp.data(), h + (size_t)t * H, H)));
      for (int i = 0; i < H; ++i) o[(size_t)t * H + i] += g * ye[(size_t)t * H + i];
    }
  }
}

// One gated Delta-Net layer over the rows h [T, hidden] -> o [T, hidden], continuing the layer's running state
// (common/transformer.h:2861-3113).  Projections and the convolution run over the whole batch; the recurrence walks the tokens in
// order, one thread per value head: S *= decay; delta = (v - S k) * beta; S += delta k^T; out = S q, with L2-normalised q (scaled
// by d^-1/2) and k of the head's key group (value head h uses key head h % key heads).
void deltanet_layer(CpuEngine& e, Layer& L, const float* h, int T, float* o) {
  const int H = e.hidden, KH = e.ssm_kh, VH = e.ssm_vh, D = e.ssm_d, CK = e.d_conv;
  const int QD = 2 * KH * D + VH * D, DI = VH * D;
  std::vector<float> qkv((size_t)T * QD), z((size_t)T * DI), al((size_t)T * VH), be((size_t)T * VH), y((size_t)T * DI);
  const MatJob jobs[4] = {{&L.s_qkv, qkv.data(), QD, nullptr}, {&L.s_z, z.data(), DI, nullptr}, {&L.s_alpha, al.data(), VH, nullptr},
                          {&L.s_beta, be.data(), VH, nullptr}};
  matmul_multi(e, jobs, 4, h, H, T);
  // causal depthwise convolution + SiLU, channel by channel over the ring of earlier rows and this batch
  std::vector<float> conv((size_t)T * QD);
  e.pool->run(QD, [&](int c0, int c1) {
    for (int c = c0; c < c1; ++c) {
      const float* w = L.conv_w.data() + (size_t)c * CK;
      for (int t = 0; t < T; ++t) {
        float acc = 0.f;
        for (int f = 0; f < CK; ++f) {
          const int src = t - (CK - 1) + f;                     // row of this batch, or of the ring when negative
          const float v = src >= 0 ? qkv[(size_t)src * QD + c] : L.ring[(size_t)(CK - 1 + src) * QD + c];
          acc += v * w[f];
        }
        conv[(size_t)t * QD + c] = acc / (1.0f + expf(-acc));
      }
    }
  });
  for (int r = 0; r < CK - 1; ++r) {                             // the ring becomes the last CK - 1 rows seen so far
    const int src = T - (CK - 1) + r;
    if (src >= 0) memcpy(L.ring.data() + (size_t)r * QD, qkv.data() + (size_t)src * QD, sizeof(float) * QD);
    else memmove(L.ring.data() + (size_t)r * QD, L.ring.data() + (size_t)(r + T) * QD, sizeof(float) * QD);
  }
  e.pool->run(VH, [&](int h0, int h1) {
    std::vector<float> qn((size_t)D), kn((size_t)D), sk((size_t)D);
    for (int hv = h0; hv < h1; ++hv) {
      const int hk = hv % KH;
      float* S = L.state.data() + (size_t)hv * D * D;
      for (int t = 0; t < T; ++t) {
        const float* q = conv.data() + (size_t)t * QD + (size_t)hk * D;
        const float* k = conv.data() + (size_t)t * QD + (size_t)(KH + hk) * D;
        const float* v = conv.data() + (size_t)t * QD + (size_t)2 * KH * D + (size_t)hv * D;
        const float qs = 1.0f / sqrtf(dot_f32(q, q, D) + e.eps) / sqrtf((float)D), ks = 1.0f / sqrtf(dot_f32(k, k, D) + e.eps);
        for (int i = 0; i < D; ++i) { qn[i] = q[i] * qs; kn[i] = k[i] * ks; }
        const float a = al[(size_t)t * VH + hv] + L.s_dt[(size_t)hv];
        const float sp = a > 20.0f ? a : log1pf(expf(a));
        const float decay = expf(sp * L.s_a[(size_t)hv]);
        const float beta = 1.0f / (1.0f + expf(-be[(size_t)t * VH + hv]));
        float* out = y.data() + (size_t)t * DI + (size_t)hv * D;
        for (int r = 0; r < D; ++r) {
          float* row = S + (size_t)r * D;
          for (int c = 0; c < D; ++c) row[c] *= decay;
          const float delta = (v[r] - dot_f32(row, kn.data(), D)) * beta;
          for (int c = 0; c < D; ++c) row[c] += delta * kn[c];
          out[r] = dot_f32(row, qn.data(), D);
        }
        // per-head RMSNorm with the shared weight, then the SiLU gate of z
        float ss = 0.f;
        for (int r = 0; r < D; ++r) ss += out[r] * out[r];
        const float inv = 1.0f / sqrtf(ss / D + e.eps);
        const float* zz = z.data() + (size_t)t * DI + (size_t)hv * D;
        for (int r = 0; r < D; ++r) out[r] = out[r] * inv * L.s_norm[(size_t)r] * (zz[r] / (1.0f + expf(-zz[r])));
      }
    }
  });
  matmul(e, L.s_out, y.data(), DI, T, o, H);
}

// x += o (the mixer's output); then the FFN on the normalised rows, added to x.  h, o, g are scratch of the caller.
void ffn_block(CpuEngine& e, const Layer& L, float* x, float* h, float* o, float* g, int T) {
  const int H = e.hidden, F = e.ffn;
  { Phase ph(&e.prof[4]);
  e.pool->run(T, [&](int t0, int t1) {
    for (int t = t0; t < t1; ++t) {
      float* xr = x + (size_t)t * H;
      const float* orow = o + (size_t)t * H;
      for (int i = 0; i < H; ++i) xr[i] += orow[i];
      rmsnorm(xr, L.ffn_norm.data(), h + (size_t)t * H, H, e.eps);
    }
  }); }
  if (e.n_experts > 0) { Phase ph(&e.prof[5]); moe_ffn(e, L, h, T, o); }
  else {
    { Phase ph(&e.prof[5]); ffn_gate_up_silu(e, L.wgate, L.wup, h, H, T, g, F); }
    { Phase ph(&e.prof[6]); matmul(e, L.wdown, g, F, T, o, H); }
  }
  Phase ph_res(&e.prof[4]);
  for (int t = 0; t < T; ++t) {
    float* xr = x + (size_t)t * H;
    const float* orow = o + (size_t)t * H;
    for (int i = 0; i < H; ++i) xr[i] += orow[i];
  }
}

void forward_hidden(CpuEngine& e, float* x, int T, int pos0) {
  const int H = e.hidden, D = e.head_dim, QD = e.n_heads * D, KD = e.n_kv * D, F = e.ffn;
  std::vector<float> h((size_t)T * H), q((size_t)T * QD), k((size_t)T * KD), v((size_t)T * KD), att((size_t)T * QD), o((size_t)T * H);
  std::vector<float> g(e.n_experts > 0 ? 0 : (size_t)T * F), qg(e.attn_gate ? (size_t)T * 2 * QD : 0);
  const float scale = 1.0f / sqrtf((float)D);
  const int group = e.n_heads / e.n_kv;
  for (int li = 0; li < e.n_layers; ++li) {
    const Layer& L = e.layers[li];
    float* kc = e.kc.data() + (size_t)li * e.max_seq * KD;
    float* vc = e.vc.data() + (size_t)li * e.max_seq * KD;
    { Phase ph(&e.prof[4]);
    e.pool->run(T, [&](int t0, int t1) {
      for (int t = t0; t < t1; ++t) rmsnorm(x + (size_t)t * H, L.attn_norm.data(), h.data() + (size_t)t * H, H, e.eps);
    }); }
    if (L.is_ssm) {
      { Phase ph(&e.prof[2]); deltanet_layer(e, e.layers[li], h.data(), T, o.data()); }
      ffn_block(e, L, x, h.data(), o.data(), g.data(), T);
      continue;
    }
    float* qdst = e.attn_gate ? qg.data() : q.data();             // gated attention: attn_q emits [q | gate] per head
    const int QW = e.attn_gate ? 2 * QD : QD;
    const MatJob qkv[3] = {{&L.wq, qdst, QW, e.has_bias ? L.bq.data() : nullptr}, {&L.wk, k.data(), KD, e.has_bias ? L.bk.data() : nullptr},
                           {&L.wv, v.data(), KD, e.has_bias ? L.bv.data() : nullptr}};
    { Phase ph(&e.prof[0]); matmul_multi(e, qkv, 3, h.data(), H, T); }
    if (e.attn_gate)
      for (int t = 0; t < T; ++t)
        for (int hq = 0; hq < e.n_heads; ++hq)
          memcpy(q.data() + (size_t)t * QD + hq * D, qg.data() + (size_t)t * QW + (size_t)hq * 2 * D, sizeof(float) * D);
    { Phase ph(&e.prof[1]);
    e.pool->run(T, [&](int t0, int t1) {
    for (int t = t0; t < t1; ++t) {
      const int pos = pos0 + t;
      for (int hq = 0; hq < e.n_heads; ++hq) {
        float* qh = q.data() + (size_t)t * QD + hq * D;
        if (e.qk_norm) rmsnorm(qh, L.q_norm.data(), qh, D, e.eps);
        rope_neox(qh, e.rope_dim, pos, e.inv_freq.data());
      }
      for (int hk = 0; hk < e.n_kv; ++hk) {
        float* kh = k.data() + (size_t)t * KD + hk * D;
        if (e.qk_norm) rmsnorm(kh, L.k_norm.data(), kh, D, e.eps);
        rope_neox(kh, e.rope_dim, pos, e.inv_freq.data());
      }
      for (int hk = 0; hk < e.n_kv; ++hk) {
        memcpy(kc + ((size_t)hk * e.max_seq + pos) * D, k.data() + (size_t)t * KD + hk * D, sizeof(float) * D);
        memcpy(vc + ((size_t)hk * e.max_seq + pos) * D, v.data() + (size_t)t * KD + hk * D, sizeof(float) * D);
      }
    }
    }); }
    // causal attention: token t sees positions 0 .. pos0 + t
    { Phase ph(&e.prof[2]);
    e.pool->run(T * e.n_heads, [&](int i0, int i1) {
      std::vector<float> sc((size_t)pos0 + T);
      for (int idx = i0; idx < i1; ++idx) {
        // interleave long and short contexts over the threads: item idx -> token (idx % T), head (idx / T)
        const int t = idx % T, hq = idx / T;
        const int n_ctx = pos0 + t + 1, hk = hq / group;
        const float* qh = q.data() + (size_t)t * QD + hq * D;
        float mx = -INFINITY;
        const float* kh = kc + (size_t)hk * e.max_seq * D;
        const float* vhead = vc + (size_t)hk * e.max_seq * D;
        for (int p = 0; p < n_ctx; ++p) { sc[p] = dot_f32(qh, kh + (size_t)p * D, D) * scale; mx = std::max(mx, sc[p]); }
        float sum = 0.f;
        for (int p = 0; p < n_ctx; ++p) { sc[p] = expf(sc[p] - mx); sum += sc[p]; }
        const float inv = 1.0f / sum;
        float* out = att.data() + (size_t)t * QD + hq * D;
        for (int d = 0; d < D; ++d) out[d] = 0.f;
        for (int p = 0; p < n_ctx; ++p) {
          const float w = sc[p] * inv;
          const float* vh = vhead + (size_t)p * D;
          for (int d = 0; d < D; ++d) out[d] += w * vh[d];
        }
      }
    }); }
    if (e.attn_gate)
      for (int t = 0; t < T; ++t)
        for (int hq = 0; hq < e.n_heads; ++hq) {
          const float* gt = qg.data() + (size_t)t * QW + (size_t)hq * 2 * D + D;
          float* a = att.data() + (size_t)t * QD + hq * D;
          for (int d = 0; d < D; ++d) a[d] *= 1.0f / (1.0f + expf(-gt[d]));
        }
    { Phase ph(&e.prof[3]); matmul(e, L.wo, att.data(), QD, T, o.data(), H); }
    ffn_block(e, L, x, h.data(), o.data(), g.data(), T);
  }
}

void embed_rows(const CpuEngine& e, const int* tokens, int T, float* x) {
  for (int t = 0; t < T; ++t) {
    int id = tokens[t];
    if (id < 0 || id >= e.vocab) id = 0;
    dequant_row(e.embed.type, e.embed.data + (size_t)id * e.embed.row_bytes, x + (size_t)t * e.hidden, e.hidden);
  }
}

void logits_of(CpuEngine& e, const float* xrow, float* logits) {
  Phase ph(&e.prof[7]);
  std::vector<float> hn((size_t)e.hidden);
  rmsnorm(xrow, e.final_norm.data(), hn.data(), e.hidden, e.eps);
  matmul(e, e.head, hn.data(), e.hidden, 1, logits, e.vocab);
}

int argmax(const float* v, int n) {
  int bi = 0; float bv = -INFINITY;
  for (int i = 0; i < n; ++i) { const float x = v[i] == v[i] ? v[i] : -3.4e38f; if (x > bv) { bv = x; bi = i; } }
  return bi;
}

}  // namespace
}  // namespace gbh

using namespace gbh;

// Open a GGUF checkpoint of a qwen2 / qwen3 / qwen3moe model for CPU inference.  threads <= 0: all cores.  NULL on error.
// A decode step streams every matrix once; out of the file mapping that is one TLB miss per 4 KB.  Copy the matrices into one
// anonymous region the kernel may back with 2 MB pages (the reference does the same at load: MADV_HUGEPAGE or a 2 MB-aligned
// buffer, common/gguf_loader.h).  Every thread copies, and so first touches, a slice of every matrix.  GB_CPU_HUGEPAGES=0 keeps the mapping.
void place_weights(CpuEngine& e) {
  const char* env = getenv("GB_CPU_HUGEPAGES");
  if (env != nullptr && env[0] == '0') return;
  std::vector<QMat*> mats;
  mats.push_back(&e.embed);
  const bool tied = e.head.data == e.embed.data;
  if (!tied) mats.push_back(&e.head);
  for (Layer& L : e.layers) {
    if (L.is_ssm) { for (QMat* m : {&L.s_qkv, &L.s_z, &L.s_alpha, &L.s_beta, &L.s_out}) mats.push_back(m); }
    else { for (QMat* m : {&L.wq, &L.wk, &L.wv, &L.wo}) mats.push_back(m); }
    if (e.shared_ffn > 0) for (QMat* m : {&L.sh_gate, &L.sh_up, &L.sh_down}) mats.push_back(m);
    if (e.n_experts > 0) {
      mats.push_back(&L.wrouter);
      for (std::vector<QMat>* v : {&L.eg, &L.eu, &L.ed}) for (QMat& m : *v) mats.push_back(&m);
    } else {
      for (QMat* m : {&L.wgate, &L.wup, &L.wdown}) mats.push_back(m);
    }
  }
  size_t total = 0;
  std::vector<size_t> off;
  for (QMat* m : mats) { off.push_back(total); total += ((size_t)m->rows * m->row_bytes + 4095) & ~(size_t)4095; }
  const size_t two_mb = (size_t)2 << 20;
  total = (total + two_mb - 1) & ~(two_mb - 1);
  void* p = mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (p == MAP_FAILED) return;                                  // not enough memory for a second copy: run from the file mapping
#ifdef MADV_HUGEPAGE
  madvise(p, total, MADV_HUGEPAGE);
#endif
  for (size_t i = 0; i < mats.size(); ++i) {
    QMat* m = mats[i];
    uint8_t* dst = (uint8_t*)p + off[i];
    const uint8_t* src = m->data;
    const long rb = m->row_bytes;
    e.pool->run(m->rows, [&](int r0, int r1) { memcpy(dst + (size_t)r0 * rb, src + (size_t)r0 * rb, (size_t)(r1 - r0) * rb); });
    m->data = dst;
  }
  if (tied) e.head = e.embed;
  e.huge = p; e.huge_bytes = total;
}

GBH_API void* gbh_cpu_engine_load(const char* path, int max_seq, int threads) {
  void* g = gbh_gguf_open(path);
  if (g == nullptr) return nullptr;
  auto* e = new CpuEngine();
  e->gguf = g;
  std::string arch = "qwen3";
  const int ai = gbh_gguf_find_key(g, "general.architecture");
  if (ai >= 0) { uint64_t len = 0; const char* s = gbh_gguf_kv_string(g, ai, -1, &len); if (s) arch.assign(s, (size_t)len); }
  if (arch != "qwen2" && arch != "qwen3" && arch != "qwen3moe" && arch != "qwen35" && arch != "qwen35moe") {
    fail("cpu engine: architecture %s is not qwen2 / qwen3 / qwen3moe / qwen35 / qwen35moe", arch.c_str()); delete e; gbh_gguf_close(g); return nullptr;
  }
  const bool hybrid = arch == "qwen35" || arch == "qwen35moe";
  const std::string p = arch + ".";
  e->n_layers = (int)kv_num(g, p + "block_count", 0); e->hidden = (int)kv_num(g, p + "embedding_length", 0);
  e->n_heads = (int)kv_num(g, p + "attention.head_count", 0); e->n_kv = (int)kv_num(g, p + "attention.head_count_kv", e->n_heads);
  e->head_dim = (int)kv_num(g, p + "attention.key_length", e->n_heads ? e->hidden / e->n_heads : 0);
  e->ffn = (int)kv_num(g, p + "feed_forward_length", 0);
  if (hybrid) {
    e->full_interval = (int)kv_num(g, p + "attention.full_attention_interval", 4); e->d_conv = (int)kv_num(g, p + "ssm.conv_kernel", 4);
    e->ssm_d = (int)kv_num(g, p + "ssm.state_size", 0); e->ssm_kh = (int)kv_num(g, p + "ssm.group_count", 0);
    e->ssm_vh = (int)kv_num(g, p + "ssm.time_step_rank", 0);
    e->attn_gate = true;
    if (e->full_interval < 1 || e->d_conv < 2 || e->ssm_d <= 0 || e->ssm_kh <= 0 || e->ssm_vh <= 0 || e->ssm_vh % e->ssm_kh) {
      fail("cpu engine: incomplete Delta-Net hyper-parameters in %s", path); delete e; gbh_gguf_close(g); return nullptr;
    }
  }
  if (arch == "qwen3moe" || arch == "qwen35moe") {
    e->n_experts = (int)kv_num(g, p + "expert_count", 0); e->n_used = (int)kv_num(g, p + "expert_used_count", 0);
    e->expert_ffn = (int)kv_num(g, p + "expert_feed_forward_length", 0);
    if (e->n_experts <= 0 || e->n_used <= 0 || e->n_used > e->n_experts || e->expert_ffn <= 0) {
      fail("cpu engine: incomplete expert hyper-parameters in %s", path); delete e; gbh_gguf_close(g); return nullptr;
    }
    if (e->ffn <= 0) e->ffn = e->expert_ffn;
    e->shared_ffn = (int)kv_num(g, p + "expert_shared_feed_forward_length", 0);
  }
  e->eps = (float)kv_num(g, p + "attention.layer_norm_rms_epsilon", 1e-6); e->theta = (float)kv_num(g, p + "rope.freq_base", 1e6);
  e->max_seq = max_seq > 0 ? max_seq : 4096;
  e->threads = threads > 0 ? threads : (int)std::max(1u, std::thread::hardware_concurrency());
  e->pool = new Pool(e->threads);
  bool ok = e->n_layers > 0 && e->hidden > 0 && e->n_heads > 0 && e->n_kv > 0 && e->head_dim > 0 && e->ffn > 0 && e->n_heads % e->n_kv == 0;
  if (!ok) fail("cpu engine: incomplete hyper-parameters in %s", path);
  const int H = e->hidden, D = e->head_dim;
  if (ok) {
    const int ei = gbh_gguf_find_tensor(g, "token_embd.weight");
    int nd = 0, type = 0; uint64_t dims[4] = {0, 0, 0, 0}, nbytes = 0; char nm[8];
    if (ei < 0) { fail("cpu engine: token_embd.weight is missing"); ok = false; }
    else { gbh_gguf_tensor_info(g, ei, nm, 8, &nd, dims, &type, &nbytes); e->vocab = (int)dims[1]; }
  }
  ok = ok && get_mat(g, "token_embd.weight", &e->embed, e->vocab, H) == 0;
  if (ok) { if (gbh_gguf_find_tensor(g, "output.weight") >= 0) ok = get_mat(g, "output.weight", &e->head, e->vocab, H) == 0; else e->head = e->embed; }
  ok = ok && get_vec(g, "output_norm.weight", &e->final_norm, H) == 0;
  e->layers.resize((size_t)std::max(e->n_layers, 0));
  for (int li = 0; ok && li < e->n_layers; ++li) {
    Layer& L = e->layers[li];
    const std::string b = "blk." + std::to_string(li) + ".";
    L.is_ssm = hybrid && (li + 1) % e->full_interval != 0;
    ok = get_vec(g, b + "attn_norm.weight", &L.attn_norm, H) == 0 &&
         get_vec(g, b + (hybrid ? "post_attention_norm.weight" : "ffn_norm.weight"), &L.ffn_norm, H) == 0;
    if (ok && L.is_ssm) {
      const int SD = e->ssm_d, QDs = 2 * e->ssm_kh * SD + e->ssm_vh * SD, DI = e->ssm_vh * SD;
      ok = get_mat(g, b + "attn_qkv.weight", &L.s_qkv, QDs, H) == 0 && get_mat(g, b + "attn_gate.weight", &L.s_z, DI, H) == 0 &&
           get_mat(g, b + "ssm_alpha.weight", &L.s_alpha, e->ssm_vh, H) == 0 && get_mat(g, b + "ssm_beta.weight", &L.s_beta, e->ssm_vh, H) == 0 &&
           get_mat(g, b + "ssm_out.weight", &L.s_out, H, DI) == 0 && get_vec(g, b + "ssm_norm.weight", &L.s_norm, SD) == 0 &&
           get_vec(g, b + "ssm_a", &L.s_a, e->ssm_vh) == 0 && get_vec(g, b + "ssm_dt.bias", &L.s_dt, e->ssm_vh) == 0;
      if (ok) {                                                  // conv weights: ggml dims {d_conv, channels} = one row of taps per channel
        const int ci = gbh_gguf_find_tensor(g, (b + "ssm_conv1d.weight").c_str());
        int nd = 0, type = 0; uint64_t dims[4] = {0, 0, 0, 0}, nbytes = 0; char nm[8];
        if (ci < 0) { fail("cpu engine: tensor %sssm_conv1d.weight is missing", b.c_str()); ok = false; }
        else {
          gbh_gguf_tensor_info(g, ci, nm, 8, &nd, dims, &type, &nbytes);
          if (nd != 2 || (int)dims[0] != e->d_conv || (int)dims[1] != QDs) { fail("cpu engine: %sssm_conv1d.weight has the wrong shape", b.c_str()); ok = false; }
          else { L.conv_w.resize((size_t)QDs * e->d_conv); ok = dequant_row(type, gbh_gguf_tensor_data(g, ci), L.conv_w.data(), (long)QDs * e->d_conv) == 0; }
        }
      }
      L.ring.assign((size_t)(e->d_conv - 1) * QDs, 0.f);
      L.state.assign((size_t)e->ssm_vh * SD * SD, 0.f);
    } else if (ok) {
      ok = get_mat(g, b + "attn_q.weight", &L.wq, (e->attn_gate ? 2 : 1) * e->n_heads * D, H) == 0 && get_mat(g, b + "attn_k.weight", &L.wk, e->n_kv * D, H) == 0 &&
           get_mat(g, b + "attn_v.weight", &L.wv, e->n_kv * D, H) == 0 && get_mat(g, b + "attn_output.weight", &L.wo, H, e->n_heads * D) == 0;
    }
    if (ok && e->n_experts > 0)
      ok = get_mat(g, b + "ffn_gate_inp.weight", &L.wrouter, e->n_experts, H) == 0 &&
           get_experts(g, b + "ffn_gate_exps.weight", &L.eg, e->n_experts, e->expert_ffn, H) == 0 &&
           get_experts(g, b + "ffn_up_exps.weight", &L.eu, e->n_experts, e->expert_ffn, H) == 0 &&
           get_experts(g, b + "ffn_down_exps.weight", &L.ed, e->n_experts, H, e->expert_ffn) == 0;
    if (ok && e->n_experts > 0 && e->shared_ffn > 0) {
      ok = get_mat(g, b + "ffn_gate_shexp.weight", &L.sh_gate, e->shared_ffn, H) == 0 && get_mat(g, b + "ffn_up_shexp.weight", &L.sh_up, e->shared_ffn, H) == 0 &&
           get_mat(g, b + "ffn_down_shexp.weight", &L.sh_down, H, e->shared_ffn) == 0;
      if (ok && get_vec(g, b + "ffn_gate_inp_shexp.weight", &L.sh_inp, H, true) < 0) ok = false;
    }
    if (ok && e->n_experts == 0)
      ok = get_mat(g, b + "ffn_gate.weight", &L.wgate, e->ffn, H) == 0 && get_mat(g, b + "ffn_up.weight", &L.wup, e->ffn, H) == 0 &&
           get_mat(g, b + "ffn_down.weight", &L.wdown, H, e->ffn) == 0;
    if (!ok) break;
    if (L.is_ssm) continue;
    const int qn = get_vec(g, b + "attn_q_norm.weight", &L.q_norm, D, true);
    if (qn == 0) { e->qk_norm = true; ok = get_vec(g, b + "attn_k_norm.weight", &L.k_norm, D) == 0; } else if (qn < 0) ok = false;
    const int bq = get_vec(g, b + "attn_q.bias", &L.bq, e->n_heads * D, true);
    if (bq == 0) { e->has_bias = true; ok = ok && get_vec(g, b + "attn_k.bias", &L.bk, e->n_kv * D) == 0 && get_vec(g, b + "attn_v.bias", &L.bv, e->n_kv * D) == 0; }
    else if (bq < 0) ok = false;
  }
  if (!ok) { gbh_gguf_close(g); delete e; return nullptr; }
  e->rope_dim = (int)kv_num(g, p + "rope.dimension_count", D);
  {                                                               // M-RoPE files carry the section sizes instead: with one position for
    const int si = gbh_gguf_find_key(g, (p + "rope.dimension_sections").c_str());   // all three axes the rotated width is twice their sum
    int type = 0, elem = 0; uint64_t count = 0;
    if (si >= 0 && gbh_gguf_kv_info(g, si, nullptr, 0, &type, &elem, &count) == 0 && count > 0 && count <= 8) {
      const void* arr = gbh_gguf_kv_array_data(g, si);
      long sum = 0;
      if (arr != nullptr && (elem == 5 || elem == 4)) for (uint64_t i = 0; i < count; ++i) { int32_t v; memcpy(&v, (const uint8_t*)arr + 4 * i, 4); sum += v; }
      if (sum > 0) e->rope_dim = (int)(2 * sum);
    }
  }
  if (e->rope_dim <= 0 || e->rope_dim > D || e->rope_dim % 2) e->rope_dim = D;
  e->inv_freq.resize((size_t)e->rope_dim / 2);
  for (int j = 0; j < e->rope_dim / 2; ++j) e->inv_freq[j] = powf(e->theta, -2.0f * (float)j / (float)e->rope_dim);
  const size_t kvn = (size_t)e->n_layers * e->max_seq * e->n_kv * D;
  e->kc.assign(kvn, 0.f); e->vc.assign(kvn, 0.f);
  place_weights(*e);
  return e;
}

GBH_API void gbh_cpu_engine_free(void* h) {
  auto* e = (CpuEngine*)h;
  if (e == nullptr) return;
  gbh_gguf_close(e->gguf);
  delete e;
}

GBH_API int gbh_cpu_engine_vocab(void* h) { return ((CpuEngine*)h)->vocab; }
GBH_API int gbh_cpu_engine_threads(void* h) { return ((CpuEngine*)h)->threads; }

// Batched pass over `n` tokens at positions pos0 .. pos0 + n - 1 (fills the KV cache); logits [vocab] of the last one.
GBH_API int gbh_cpu_engine_forward(void* h, const int* tokens, int n, int pos0, float* logits) {
  auto* e = (CpuEngine*)h;
  if (n <= 0 || pos0 < 0 || pos0 + n > e->max_seq) return fail("cpu engine: positions %d .. %d leave the cache of %d", pos0, pos0 + n, e->max_seq);
  if (e->full_interval > 0) {                                    // a recurrent state cannot be rewound: start over at 0 or continue
    if (pos0 == 0) for (Layer& L : e->layers) { std::fill(L.ring.begin(), L.ring.end(), 0.f); std::fill(L.state.begin(), L.state.end(), 0.f); }
    else if (pos0 != e->ssm_pos) return fail("cpu engine: the recurrent state stands at position %d, not %d (restart from 0)", e->ssm_pos, pos0);
    e->ssm_pos = pos0 + n;
  }
  std::vector<float> x((size_t)n * e->hidden);
  embed_rows(*e, tokens, n, x.data());
  forward_hidden(*e, x.data(), n, pos0);
  if (logits != nullptr) logits_of(*e, x.data() + (size_t)(n - 1) * e->hidden, logits);
  return 0;
}

// Seconds per phase since the engine was loaded or since the last call with reset != 0 (nine slots: qkv, rope + cache, attention, o_proj,
// norms + residuals, gate / up + SiLU, down, head, unused).  The counterpart of the reference's per-op tables (common/profiler.h).
GBH_API int gbh_cpu_engine_profile(void* h, double* out, int reset) {
  auto* e = (CpuEngine*)h;
  for (int i = 0; i < 9; ++i) { if (out) out[i] = e->prof[i]; if (reset) e->prof[i] = 0; }
  return 9;
}

// Greedy generation: batched prefill of the prompt, then max_new - 1 single-token steps.  Writes max_new token ids and the
// seconds spent in the two phases.
GBH_API int gbh_cpu_engine_generate(void* h, const int* prompt, int n_prompt, int max_new, int* out_tokens, double* prefill_s, double* decode_s) {
  auto* e = (CpuEngine*)h;
  if (max_new <= 0) return 0;
  if (n_prompt + max_new > e->max_seq) return fail("cpu engine: %d + %d tokens exceed the cache of %d", n_prompt, max_new, e->max_seq);
  std::vector<float> logits((size_t)e->vocab);
  auto t0 = std::chrono::steady_clock::now();
  if (gbh_cpu_engine_forward(h, prompt, n_prompt, 0, logits.data()) != 0) return -1;
  auto t1 = std::chrono::steady_clock::now();
  int tok = argmax(logits.data(), e->vocab);
  out_tokens[0] = tok;
  for (int i = 1; i < max_new; ++i) {
    if (gbh_cpu_engine_forward(h, &tok, 1, n_prompt + i - 1, logits.data()) != 0) return -1;
    tok = argmax(logits.data(), e->vocab);
    out_tokens[i] = tok;
  }
  auto t2 = std::chrono::steady_clock::now();
  if (prefill_s) *prefill_s = std::chrono::duration<double>(t1 - t0).count();
  if (decode_s) *decode_s = std::chrono::duration<double>(t2 - t1).count();
  return 0;
}
