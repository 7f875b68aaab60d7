// Gated Delta-Net layers of the Qwen3.5 hybrid models (linear attention with a per-head matrix state) and the sigmoid output
// gate of their full-attention layers.
//
//   gb_ssm_conv_silu     causal depthwise conv1d (kernel conv_k, history carried per sequence) + SiLU over packed tokens
//   gb_deltanet          per (sequence, value head): L2-normalised q, k; S *= exp(alpha); delta = (v - S k) * beta;
//                        S += delta k^T; o = S q; gated RMSNorm: o * rsqrt(mean(o^2) + eps) * w * SiLU(z)
//   gb_sigmoid_gate_mul  a[t, c] *= sigmoid(gate[t, c])
//
// The recurrence keeps one row of the d_state x d_state state per thread in registers and walks the tokens of its sequence
// in order, so one launch serves decode (one token) and prefill chunks alike; the state is read once and written once per
// launch.  Prefill launches take the chunked scan of deltanet_chunk.cu instead.
//
// Math and tensor conventions follow common/transformer.h:2861-3113 (tf_ssm_deltanet_forward) and :2829-2851 (the scalar
// recurrence): qkv channels are ordered [Q (n_group heads) | K (n_group heads) | V (dt_rank heads)], value head h uses the
// q/k group h % n_group, alpha = softplus(alpha_raw + dt_bias) * a, beta = sigmoid(beta_raw), q is scaled by
// 1/sqrt(d_state) after the L2 normalisation (x / sqrt(sum x^2 + eps)).  The reference keeps the conv history in a ring
// buffer (transformer.h:2927-2998); here it is a plain oldest-to-newest window, rewritten at the end of every launch.
#include "sm100.cuh"
#include "host_common.h"

namespace gb {

constexpr int kMaxConvK = 8;

// One thread per (sequence, channel): walks the sequence's tokens with the window in registers.
__global__ void __launch_bounds__(256)
ssm_conv_silu_kernel(const __nv_bfloat16* __restrict__ x, int ld_x, const float* __restrict__ w, float* __restrict__ state,
                     const int* __restrict__ cu_q, const int* __restrict__ seq_slots, __nv_bfloat16* __restrict__ out, int ld_out,
                     int channels, int conv_k) {
  pdl_wait();
  pdl_trigger();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  if (c >= channels) return;
  const int t0 = cu_q[s], t1 = cu_q[s + 1];
  if (t1 <= t0) return;
  const int nh = conv_k - 1;
  float* st = state + ((size_t)seq_slots[s] * nh) * channels + c;
  float win[kMaxConvK], wk[kMaxConvK];
#pragma unroll
  for (int f = 0; f < kMaxConvK; ++f) {
    win[f] = (f < nh) ? st[(size_t)f * channels] : 0.f;
    wk[f] = (f < conv_k) ? w[(size_t)c * conv_k + f] : 0.f;
  }
  for (int t = t0; t < t1; ++t) {
    const float xv = __bfloat162float(x[(size_t)t * ld_x + c]);
    float acc = 0.f;
#pragma unroll
    for (int f = 0; f < kMaxConvK - 1; ++f) if (f < nh) acc += wk[f] * win[f];
    acc += wk[nh] * xv;
    out[(size_t)t * ld_out + c] = __float2bfloat16(acc / (1.0f + __expf(-acc)));
#pragma unroll
    for (int f = 0; f < kMaxConvK - 1; ++f) if (f + 1 < nh) win[f] = win[f + 1];
    win[nh - 1] = xv;
  }
#pragma unroll
  for (int f = 0; f < kMaxConvK - 1; ++f) if (f < nh) st[(size_t)f * channels] = win[f];
}

struct DeltaNetArgs {
  const __nv_bfloat16* qkv;   // [T, ld_qkv] after conv + SiLU: Q | K | V
  int ld_qkv;
  const __nv_bfloat16* z;     // [T, ld_z] gate input (d_inner columns)
  int ld_z;
  const float* ab;            // [T, 2 * dt_rank]: alpha_raw | beta_raw
  const float* a;             // [dt_rank]
  const float* dt_bias;       // [dt_rank]
  const float* norm_w;        // [d_state]
  float* state;               // [slots, dt_rank, d_state, d_state]
  const int* cu_q;
  const int* seq_slots;
  __nv_bfloat16* out;         // [T, dt_rank * d_state]
  int n_group, dt_rank;
  float eps;
};

template <int DS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < DS / 32; ++i) t += red[i];
  __syncthreads();
  return t;
}

// grid (dt_rank, sequences), DS threads: thread r owns row r of the state (the value index), columns are the key index.
template <int DS>
__global__ void __launch_bounds__(DS)
deltanet_kernel(const DeltaNetArgs a) {
  pdl_wait();
  pdl_trigger();
  const int h = blockIdx.x, s = blockIdx.y, r = threadIdx.x;
  const int t0 = a.cu_q[s], t1 = a.cu_q[s + 1];
  if (t1 <= t0) return;
  __shared__ float sq[DS], sk[DS], red[DS / 32];
  const int g = h % a.n_group;
  const int q_off = g * DS, k_off = a.n_group * DS + g * DS, v_off = 2 * a.n_group * DS + h * DS;
  float* st = a.state + (((size_t)a.seq_slots[s] * a.dt_rank + h) * DS + r) * DS;
  float S[DS];
#pragma unroll
  for (int c = 0; c < DS; c += 4) {
    const float4 v4 = *reinterpret_cast<const float4*>(st + c);
    S[c] = v4.x; S[c + 1] = v4.y; S[c + 2] = v4.z; S[c + 3] = v4.w;
  }
  const float a_h = a.a[h], bias_h = a.dt_bias[h], nw = a.norm_w[r];
  const float q_scale = rsqrtf((float)DS);
  for (int t = t0; t < t1; ++t) {
    const __nv_bfloat16* row = a.qkv + (size_t)t * a.ld_qkv;
    const float qv = __bfloat162float(row[q_off + r]), kv = __bfloat162float(row[k_off + r]), vv = __bfloat162float(row[v_off + r]);
    const float qn = block_sum<DS>(qv * qv, red), kn = block_sum<DS>(kv * kv, red);
    sq[r] = qv * rsqrtf(qn + a.eps) * q_scale;
    sk[r] = kv * rsqrtf(kn + a.eps);
    const float ar = a.ab[(size_t)t * 2 * a.dt_rank + h] + bias_h;
    const float sp = ar > 20.0f ? ar : log1pf(__expf(ar));
    const float decay = __expf(sp * a_h);
    const float beta = 1.0f / (1.0f + __expf(-a.ab[(size_t)t * 2 * a.dt_rank + a.dt_rank + h]));
    __syncthreads();
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < DS; ++c) { S[c] *= decay; dot += S[c] * sk[c]; }
    const float delta = (vv - dot) * beta;
    float o = 0.f;
#pragma unroll
    for (int c = 0; c < DS; ++c) { S[c] += delta * sk[c]; o += S[c] * sq[c]; }
    const float ss = block_sum<DS>(o * o, red);          // also the barrier that lets the next token overwrite sq / sk
    const float zv = __bfloat162float(a.z[(size_t)t * a.ld_z + h * DS + r]);
    const float y = o * rsqrtf(ss / (float)DS + a.eps) * nw * (zv / (1.0f + __expf(-zv)));
    a.out[((size_t)t * a.dt_rank + h) * DS + r] = __float2bfloat16(y);
  }
#pragma unroll
  for (int c = 0; c < DS; c += 4) *reinterpret_cast<float4*>(st + c) = make_float4(S[c], S[c + 1], S[c + 2], S[c + 3]);
}

__global__ void sigmoid_gate_mul_kernel(__nv_bfloat16* __restrict__ x, int ld_x, const __nv_bfloat16* __restrict__ gate, int ld_g, long rows,
                                        int cols) {
  pdl_wait();
  pdl_trigger();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vpr = cols >> 3;
  if (idx >= rows * vpr) return;
  const long rr = idx / vpr;
  const int c = (int)(idx % vpr) * 8;
  const uint4 xr = *reinterpret_cast<const uint4*>(x + rr * ld_x + c), gr = *reinterpret_cast<const uint4*>(gate + rr * ld_g + c);
  const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xr);
  const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gr);
  uint4 o;
  uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 xf = __bfloat1622float2(xh[i]), gf = __bfloat1622float2(gh[i]);
    ow[i] = pack_bf16x2(xf.x / (1.0f + __expf(-gf.x)), xf.y / (1.0f + __expf(-gf.y)));
  }
  *reinterpret_cast<uint4*>(x + rr * ld_x + c) = o;
}

}  // namespace gb

using namespace gb;

GB_API int gb_ssm_conv_silu(const void* x, int ld_x, const float* w, float* state, const int* cu_q, const int* seq_slots, void* out, int ld_out,
                            int channels, int conv_k, int n_seqs, cudaStream_t stream) {
  if (conv_k < 2 || conv_k > kMaxConvK) return fail("ssm_conv: conv_k must be in [2, 8]%s");
  if (n_seqs <= 0) return 0;
  launch_k(ssm_conv_silu_kernel, dim3((channels + 255) / 256, n_seqs), 256, 0, stream, (const __nv_bfloat16*)x, ld_x, w, state, cu_q, seq_slots,
           (__nv_bfloat16*)out, ld_out, channels, conv_k);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_deltanet(const void* qkv, int ld_qkv, const void* z, int ld_z, const float* ab, const float* a, const float* dt_bias,
                       const float* norm_w, float* state, const int* cu_q, const int* seq_slots, void* out, int n_group, int dt_rank,
                       int d_state, float eps, int n_seqs, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (n_group <= 0 || dt_rank % n_group) return fail("deltanet: dt_rank must be a multiple of n_group%s");
  DeltaNetArgs g;
  g.qkv = (const __nv_bfloat16*)qkv; g.ld_qkv = ld_qkv; g.z = (const __nv_bfloat16*)z; g.ld_z = ld_z; g.ab = ab; g.a = a; g.dt_bias = dt_bias;
  g.norm_w = norm_w; g.state = state; g.cu_q = cu_q; g.seq_slots = seq_slots; g.out = (__nv_bfloat16*)out; g.n_group = n_group;
  g.dt_rank = dt_rank; g.eps = eps;
  if (d_state == 128) launch_k(deltanet_kernel<128>, dim3(dt_rank, n_seqs), 128, 0, stream, g);
  else if (d_state == 64) launch_k(deltanet_kernel<64>, dim3(dt_rank, n_seqs), 64, 0, stream, g);
  else return fail("deltanet: d_state must be 64 or 128%s");
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}

GB_API int gb_sigmoid_gate_mul(void* x, int ld_x, const void* gate, int ld_g, long rows, int cols, cudaStream_t stream) {
  if (cols % 8 || ld_x % 8 || ld_g % 8) return fail("sigmoid_gate_mul: columns and strides must be multiples of 8%s");
  const long n = rows * (cols / 8);
  if (n <= 0) return 0;
  launch_k(sigmoid_gate_mul_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, (__nv_bfloat16*)x, ld_x, (const __nv_bfloat16*)gate, ld_g, rows, cols);
  GB_CUDA_OK(cudaGetLastError());
  return 0;
}
