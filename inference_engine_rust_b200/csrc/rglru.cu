// The gated linear recurrence of a recurrent block with two branches (a real-gated LRU):
//
//   branch y:  g = gelu_tanh(py + by)                                  (py, px: the two halves of one projection)
//   branch x:  u[t] = cb + sum_j taps[:, K-1-j] (px[t-j] + bx)          (causal, per channel, zeros before the start)
//   gates:     r = sigmoid(Ra u + ra_b),  i = sigmoid(Ri u + ri_b)      (block-diagonal: the channels in `blocks` equal
//                                                                       parts, one square matrix [out, in] per part)
//   decay:     log a = -c r softplus(lam),  a = exp(log a),  m = sqrt(1 - a^2)
//   state:     S[t] = a S[t-1] + m i u[t]            from S = 0 for a new sequence, carried in the cache's state
//   result:    S[t] g[t] * out_scale, in the run's dtype: the input of the output projection
//
// Everything here is fp32 (the gates' weight matrices are read in their stored type and widened).  The state
// of a sequence is [S (C) | the last K-1 inputs px + bx of the convolution, oldest first ((K-1) C)].
//
// Three kernels: the convolution (a thread per token and channel), the gates with decay and input term
// (a tiled product on the CUDA cores: every output sums its k ascending, so a token's result does not
// depend on the batch), and the scan (a thread per sequence and channel walks the step's tokens in order,
// then stores S and the new tail of inputs).
#include "common.cuh"

using namespace iert;

namespace {

__device__ __forceinline__ float sigmoid_f(float x) {
  if (x >= 0.f) return 1.0f / (1.0f + expf(-x));
  const float z = expf(x);
  return z / (1.0f + z);
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// u[t, c] for every token of the step, a thread per token and channel.  proj: fp32 [T, 2C] = [py | px].
constexpr int MAX_TAPS = 16;

__global__ void rglru_conv_kernel(const float* __restrict__ proj, long long ld, const float* __restrict__ bx,
                                  const float* __restrict__ taps, const float* __restrict__ cb, const float* __restrict__ state,
                                  long long state_ld, float* __restrict__ u, int C, int K, IertBatchView b) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int s = sequence_of_token(b, t);
  const int slot = s < 0 ? -1 : b.slot_ids[s];
  if (slot < 0 || c >= C) return;
  const int q_begin = b.cu_q[s];
  const int back = t - q_begin;                    // tokens of this sequence in front of t within the step
  const float bias = bx[c];
  float acc = cb[c];
  pdl_wait();
  const float* tail = state + (size_t)slot * state_ld + C;       // [K-1][C], oldest first
  for (int j = K - 1; j >= 0; --j) {               // oldest input first
    float xin;
    if (j <= back) xin = proj[(size_t)(t - j) * ld + C + c] + bias;
    else xin = tail[(size_t)(K - 1 - (j - back)) * C + c];        // position pos0 - (j - back)
    acc = fmaf(taps[(size_t)c * K + (K - 1 - j)], xin, acc);
  }
  u[(size_t)t * C + c] = acc;
}

// The same with four consecutive channels per thread (16-byte accesses) and CONV_TOKENS tokens per block, which
// brings its channels' taps into shared memory once, transposed (taps of one place side by side).  C a multiple of 4,
// rows aligned.
constexpr int CONV_TOKENS = 4, CONV_THREADS = 128;

__global__ void __launch_bounds__(CONV_THREADS)
rglru_conv4_kernel(const float* __restrict__ proj, long long ld, const float* __restrict__ bx,
                   const float* __restrict__ taps, const float* __restrict__ cb, const float* __restrict__ state,
                   long long state_ld, float* __restrict__ u, int C, int K, int tokens_per_block, IertBatchView b) {
  extern __shared__ __align__(16) float taps_s[];             // [K][4 * CONV_THREADS]
  pdl_launch_dependents();
  constexpr int CH = 4 * CONV_THREADS;
  const int c0 = blockIdx.y * CH;
  const int c = c0 + threadIdx.x * 4;
  const int n_ch = min(CH, C - c0);
  for (int i = threadIdx.x; i < n_ch * K; i += CONV_THREADS) {
    const int ch = i / K, q = i - ch * K;
    taps_s[q * CH + ch] = taps[(size_t)c0 * K + i];
  }
  __syncthreads();
  if (c >= C) return;
  const float4 bias = *reinterpret_cast<const float4*>(bx + c);
  const float4 cbias = *reinterpret_cast<const float4*>(cb + c);
  pdl_wait();
  for (int i = 0; i < tokens_per_block; ++i) {
    const int t = blockIdx.x * tokens_per_block + i;
    if (t >= b.n_tokens) break;
    const int s = sequence_of_token(b, t);
    const int slot = s < 0 ? -1 : b.slot_ids[s];
    if (slot < 0) continue;
    const int back = t - b.cu_q[s];
    const float* tail = state + (size_t)slot * state_ld + C;
    float4 acc = cbias;
    for (int j = K - 1; j >= 0; --j) {
      float4 xin;
      if (j <= back) {
        xin = *reinterpret_cast<const float4*>(proj + (size_t)(t - j) * ld + C + c);
        xin.x += bias.x; xin.y += bias.y; xin.z += bias.z; xin.w += bias.w;
      } else {
        xin = *reinterpret_cast<const float4*>(tail + (size_t)(K - 1 - (j - back)) * C + c);
      }
      const float4 w = *reinterpret_cast<const float4*>(taps_s + (K - 1 - j) * CH + threadIdx.x * 4);
      acc.x = fmaf(w.x, xin.x, acc.x);
      acc.y = fmaf(w.y, xin.y, acc.y);
      acc.z = fmaf(w.z, xin.z, acc.z);
      acc.w = fmaf(w.w, xin.w, acc.w);
    }
    *reinterpret_cast<float4*>(u + (size_t)t * C + c) = acc;
  }
}

// Gates, decay and input term: A[t, c] = a, Bv[t, c] = sqrt(1 - a^2) i u.
// Tile: 32 tokens x 64 output channels of one block, k in chunks of 32.
constexpr int GT = 32, GO = 64, GK = 32, GTHREADS = 256;

template <typename TW>
__global__ void __launch_bounds__(GTHREADS)
rglru_gates_kernel(const float* __restrict__ u, const TW* __restrict__ Ra, const float* __restrict__ ra_b,
                   const TW* __restrict__ Ri, const float* __restrict__ ri_b, const float* __restrict__ lam, float decay_c,
                   float* __restrict__ A, float* __restrict__ Bv, int T, int C, int bw) {
  __shared__ float us[GK][GT + 1];
  __shared__ float wr[GK][GO + 1];
  __shared__ float wi[GK][GO + 1];
  pdl_launch_dependents();
  const int blk = blockIdx.z, o0 = blockIdx.y * GO, t0 = blockIdx.x * GT;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;        // 16 x 16: 4 outputs x 2 tokens per thread
  const TW* ra = Ra + (size_t)blk * bw * bw;
  const TW* ri = Ri + (size_t)blk * bw * bw;
  float ar[2][4], ai[2][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int c = 0; c < 4; ++c) ar[a][c] = ai[a][c] = 0.f;
  pdl_wait();
  for (int k0 = 0; k0 < bw; k0 += GK) {
    for (int i = threadIdx.x; i < GK * GT; i += GTHREADS) {
      const int tt = i / GK, kk = i - tt * GK;
      const int t = t0 + tt, k = k0 + kk;
      us[kk][tt] = (t < T && k < bw) ? u[(size_t)t * C + (size_t)blk * bw + k] : 0.f;
    }
    for (int i = threadIdx.x; i < GK * GO; i += GTHREADS) {
      const int oo = i / GK, kk = i - oo * GK;
      const int o = o0 + oo, k = k0 + kk;
      const bool in = o < bw && k < bw;
      wr[kk][oo] = in ? to_f32(ra[(size_t)o * bw + k]) : 0.f;
      wi[kk][oo] = in ? to_f32(ri[(size_t)o * bw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < GK; ++kk) {
      const float u0 = us[kk][ty * 2], u1 = us[kk][ty * 2 + 1];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float a = wr[kk][tx + 16 * c], bb = wi[kk][tx + 16 * c];
        ar[0][c] = fmaf(a, u0, ar[0][c]);
        ar[1][c] = fmaf(a, u1, ar[1][c]);
        ai[0][c] = fmaf(bb, u0, ai[0][c]);
        ai[1][c] = fmaf(bb, u1, ai[1][c]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int t = t0 + ty * 2 + a;
    if (t >= T) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int o = o0 + tx + 16 * c;
      if (o >= bw) continue;
      const size_t ch = (size_t)blk * bw + o;
      const float r = sigmoid_f(ar[a][c] + ra_b[ch]);
      const float g = sigmoid_f(ai[a][c] + ri_b[ch]);
      const float log_a = -decay_c * r * softplus_f(lam[ch]);
      const float av = expf(log_a);
      const float m = sqrtf(fmaxf(-expm1f(2.0f * log_a), 0.f));       // sqrt(1 - a^2) without cancellation
      A[(size_t)t * C + ch] = av;
      Bv[(size_t)t * C + ch] = m * g * u[(size_t)t * C + ch];
    }
  }
}

// The gates of many tokens with bfloat16 weights, on the tensor cores (mma.sync m16n8k16) without giving up the
// 32-bit input: u is split as hi + lo, two bfloat16 numbers that together carry 16 bits of its mantissa, both are
// multiplied by the (exact) bfloat16 weights and summed in fp32, so a sum differs from the fp32 one by about 2^-17 of
// its terms.  Tile: 64 tokens x 64 output channels of one block, both gates; a warp owns 16 tokens; k in chunks of 32.
constexpr int TM = 64, TN = 64, TK = 32, TLD = TK + 8, TC_THREADS = 128;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(TC_THREADS)
rglru_gates_tc_kernel(const float* __restrict__ u, const __nv_bfloat16* __restrict__ Ra, const float* __restrict__ ra_b,
                      const __nv_bfloat16* __restrict__ Ri, const float* __restrict__ ri_b, const float* __restrict__ lam,
                      float decay_c, float* __restrict__ A, float* __restrict__ Bv, int T, int C, int bw) {
  __shared__ __align__(16) __nv_bfloat16 a_hi[TM][TLD];
  __shared__ __align__(16) __nv_bfloat16 a_lo[TM][TLD];
  __shared__ __align__(16) __nv_bfloat16 w_r[TN][TLD];
  __shared__ __align__(16) __nv_bfloat16 w_i[TN][TLD];
  pdl_launch_dependents();
  const int blk = blockIdx.z, o0 = blockIdx.y * TN, t0 = blockIdx.x * TM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const __nv_bfloat16* ra = Ra + (size_t)blk * bw * bw;
  const __nv_bfloat16* ri = Ri + (size_t)blk * bw * bw;
  float cr[TN / 8][4], ci[TN / 8][4];
#pragma unroll
  for (int n = 0; n < TN / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) cr[n][e] = ci[n][e] = 0.f;
  pdl_wait();
  // A chunk's operands come from memory into registers while the chunk before it is multiplied.
  constexpr int UV = TM * TK / 4 / TC_THREADS, WV = TN * TK / 8 / TC_THREADS;
  float4 ureg[UV];
  uint4 wreg_r[WV], wreg_i[WV];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int q = 0; q < UV; ++q) {                 // u: 64 tokens x 32 k, four consecutive k per load
      const int i = threadIdx.x + q * TC_THREADS;
      const int tt = i / (TK / 4), kk = (i - tt * (TK / 4)) * 4;
      const int t = t0 + tt, k = k0 + kk;
      ureg[q] = (t < T && k < bw) ? *reinterpret_cast<const float4*>(u + (size_t)t * C + (size_t)blk * bw + k)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int q = 0; q < WV; ++q) {                 // weights: 64 output rows x 32 k of either gate, eight k per load
      const int i = threadIdx.x + q * TC_THREADS;
      const int oo = i / (TK / 8), kk = (i - oo * (TK / 8)) * 8;
      const int o = o0 + oo, k = k0 + kk;
      const bool in = o < bw && k < bw;
      wreg_r[q] = in ? *reinterpret_cast<const uint4*>(ra + (size_t)o * bw + k) : make_uint4(0u, 0u, 0u, 0u);
      wreg_i[q] = in ? *reinterpret_cast<const uint4*>(ri + (size_t)o * bw + k) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < bw; k0 += TK) {
#pragma unroll
    for (int q = 0; q < UV; ++q) {                 // u as hi and lo
      const int i = threadIdx.x + q * TC_THREADS;
      const int tt = i / (TK / 4), kk = (i - tt * (TK / 4)) * 4;
      const float4 v = ureg[q];
      const __nv_bfloat162 h0 = __floats2bfloat162_rn(v.x, v.y), h1 = __floats2bfloat162_rn(v.z, v.w);
      const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);
      const __nv_bfloat162 l0 = __floats2bfloat162_rn(v.x - f0.x, v.y - f0.y), l1 = __floats2bfloat162_rn(v.z - f1.x, v.w - f1.y);
      *reinterpret_cast<__nv_bfloat162*>(&a_hi[tt][kk]) = h0;
      *reinterpret_cast<__nv_bfloat162*>(&a_hi[tt][kk + 2]) = h1;
      *reinterpret_cast<__nv_bfloat162*>(&a_lo[tt][kk]) = l0;
      *reinterpret_cast<__nv_bfloat162*>(&a_lo[tt][kk + 2]) = l1;
    }
#pragma unroll
    for (int q = 0; q < WV; ++q) {
      const int i = threadIdx.x + q * TC_THREADS;
      const int oo = i / (TK / 8), kk = (i - oo * (TK / 8)) * 8;
      *reinterpret_cast<uint4*>(&w_r[oo][kk]) = wreg_r[q];
      *reinterpret_cast<uint4*>(&w_i[oo][kk]) = wreg_i[q];
    }
    __syncthreads();
    if (k0 + TK < bw) fetch(k0 + TK);
#pragma unroll
    for (int ks = 0; ks < TK / 16; ++ks) {
      uint32_t ah[4], al[4];
      ldsm_x4(ah, &a_hi[warp * 16 + (lane & 15)][ks * 16 + (lane >> 4) * 8]);
      ldsm_x4(al, &a_lo[warp * 16 + (lane & 15)][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int np = 0; np < TN / 16; ++np) {
        uint32_t br[4], bi[4];
        const int row = np * 16 + (lane & 7) + ((lane >> 4) << 3), col = ks * 16 + ((lane >> 3) & 1) * 8;
        ldsm_x4(br, &w_r[row][col]);
        ldsm_x4(bi, &w_i[row][col]);
        mma_bf16_16816(cr[2 * np], al, br[0], br[1]);          // the small parts first
        mma_bf16_16816(cr[2 * np + 1], al, br[2], br[3]);
        mma_bf16_16816(ci[2 * np], al, bi[0], bi[1]);
        mma_bf16_16816(ci[2 * np + 1], al, bi[2], bi[3]);
        mma_bf16_16816(cr[2 * np], ah, br[0], br[1]);
        mma_bf16_16816(cr[2 * np + 1], ah, br[2], br[3]);
        mma_bf16_16816(ci[2 * np], ah, bi[0], bi[1]);
        mma_bf16_16816(ci[2 * np + 1], ah, bi[2], bi[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int n = 0; n < TN / 8; ++n) {
    const int o = o0 + n * 8 + tq * 2;
    if (o >= bw) continue;                             // bw is even: o + 1 is inside too
    const size_t ch = (size_t)blk * bw + o;
    const float sp0 = softplus_f(lam[ch]), sp1 = softplus_f(lam[ch + 1]);
    const float rb0 = ra_b[ch], rb1 = ra_b[ch + 1], ib0 = ri_b[ch], ib1 = ri_b[ch + 1];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int t = t0 + warp * 16 + g + 8 * half;
      if (t >= T) continue;
      const float2 uv = *reinterpret_cast<const float2*>(u + (size_t)t * C + ch);
      const float la0 = -decay_c * sigmoid_f(cr[n][2 * half] + rb0) * sp0;
      const float la1 = -decay_c * sigmoid_f(cr[n][2 * half + 1] + rb1) * sp1;
      *reinterpret_cast<float2*>(A + (size_t)t * C + ch) = make_float2(expf(la0), expf(la1));
      *reinterpret_cast<float2*>(Bv + (size_t)t * C + ch) =
          make_float2(sqrtf(fmaxf(-expm1f(2.0f * la0), 0.f)) * sigmoid_f(ci[n][2 * half] + ib0) * uv.x,
                      sqrtf(fmaxf(-expm1f(2.0f * la1), 0.f)) * sigmoid_f(ci[n][2 * half + 1] + ib1) * uv.y);
    }
  }
}

// The same for a handful of tokens (one-token steps): a warp per output channel reads its two weight rows once,
// lanes over k, and forms the sums of up to SMALL_T tokens at a time; the weights are the traffic.
constexpr int SMALL_T = 8;

__device__ __forceinline__ void load8(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h[e]);
    o[2 * e] = f.x;
    o[2 * e + 1] = f.y;
  }
}

template <typename TW>
__global__ void __launch_bounds__(256, 4)
rglru_gates_small_kernel(const float* __restrict__ u, const TW* __restrict__ Ra, const float* __restrict__ ra_b,
                         const TW* __restrict__ Ri, const float* __restrict__ ri_b, const float* __restrict__ lam, float decay_c,
                         float* __restrict__ A, float* __restrict__ Bv, int T, int C, int bw, int vec8) {
  pdl_launch_dependents();
  const int ch = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (ch >= C) return;
  const int blk = ch / bw, o = ch - blk * bw;
  const TW* ra = Ra + ((size_t)blk * bw + o) * bw;
  const TW* ri = Ri + ((size_t)blk * bw + o) * bw;
  const float sp = softplus_f(lam[ch]), rb = ra_b[ch], ib = ri_b[ch];
  pdl_wait();
  for (int t0 = 0; t0 < T; t0 += SMALL_T) {
    float ar[SMALL_T], ai[SMALL_T];
#pragma unroll
    for (int j = 0; j < SMALL_T; ++j) ar[j] = ai[j] = 0.f;
    if (vec8) {
      // eight consecutive k per lane and pass: one 16-byte (bf16) or two (fp32) loads of either weight row, two of u per token
      for (int k = lane * 8; k < bw; k += 256) {
        float wr[8], wi[8];
        load8(ra + k, wr);
        load8(ri + k, wi);
#pragma unroll
        for (int j = 0; j < SMALL_T; ++j) {
          if (t0 + j >= T) break;
          const float* up = u + (size_t)(t0 + j) * C + (size_t)blk * bw + k;
          const float4 a = *reinterpret_cast<const float4*>(up), bq = *reinterpret_cast<const float4*>(up + 4);
          const float uv[8] = {a.x, a.y, a.z, a.w, bq.x, bq.y, bq.z, bq.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            ar[j] = fmaf(wr[e], uv[e], ar[j]);
            ai[j] = fmaf(wi[e], uv[e], ai[j]);
          }
        }
      }
    } else {
      for (int k = lane; k < bw; k += 32) {
        const float wr = to_f32(ra[k]), wi = to_f32(ri[k]);
#pragma unroll
        for (int j = 0; j < SMALL_T; ++j) {
          const float uv = t0 + j < T ? u[(size_t)(t0 + j) * C + (size_t)blk * bw + k] : 0.f;
          ar[j] = fmaf(wr, uv, ar[j]);
          ai[j] = fmaf(wi, uv, ai[j]);
        }
      }
    }
    // lane j finishes token t0 + j: the sigmoids, the decay and the input term of all tokens side by side
    float my_r = 0.f, my_i = 0.f;
#pragma unroll
    for (int j = 0; j < SMALL_T; ++j) {
      const float sr = warp_sum(ar[j]), si = warp_sum(ai[j]);
      if (lane == j) { my_r = sr; my_i = si; }
    }
    if (lane < SMALL_T && t0 + lane < T) {
      const size_t at = (size_t)(t0 + lane) * C + ch;
      const float r = sigmoid_f(my_r + rb), g = sigmoid_f(my_i + ib);
      const float log_a = -decay_c * r * sp;
      A[at] = expf(log_a);
      Bv[at] = sqrtf(fmaxf(-expm1f(2.0f * log_a), 0.f)) * g * u[at];
    }
  }
}

// The scan: a thread per (sequence, channel).

template <typename TO>
__global__ void rglru_scan_kernel(const float* __restrict__ A, const float* __restrict__ Bv, const float* __restrict__ proj,
                                  long long ld, const float* __restrict__ by, const float* __restrict__ bx,
                                  float* __restrict__ state, long long state_ld, TO* __restrict__ out, float out_scale, int C,
                                  int K, IertBatchView b) {
  pdl_launch_dependents();
  const int s = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = b.slot_ids[s];
  if (slot < 0 || c >= C) return;
  const int q_begin = b.cu_q[s], q_len = b.cu_q[s + 1] - q_begin;
  const float ybias = by[c], xbias = bx[c];
  pdl_wait();
  float* st = state + (size_t)slot * state_ld;
  float S = st[c];
  int t = q_begin;
  const int t_end = q_begin + q_len;
  for (; t + 4 <= t_end; t += 4) {                 // four tokens' loads in flight
    float a[4], bv[4], py[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      a[j] = A[(size_t)(t + j) * C + c];
      bv[j] = Bv[(size_t)(t + j) * C + c];
      py[j] = proj[(size_t)(t + j) * ld + c];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      S = fmaf(a[j], S, bv[j]);
      out[(size_t)(t + j) * C + c] = from_f32<TO>(S * gelu_tanh_f(py[j] + ybias) * out_scale);
    }
  }
  for (; t < t_end; ++t) {
    S = fmaf(A[(size_t)t * C + c], S, Bv[(size_t)t * C + c]);
    out[(size_t)t * C + c] = from_f32<TO>(S * gelu_tanh_f(proj[(size_t)t * ld + c] + ybias) * out_scale);
  }
  st[c] = S;
  // the convolution's last K-1 inputs, oldest first: from the step's rows, or moved up from the old tail
  float* tail = st + C;
  float keep[MAX_TAPS];
#pragma unroll
  for (int i = 0; i < MAX_TAPS; ++i) {
    if (i >= K - 1) break;
    const int back = K - 2 - i;                     // how many tokens before the sequence's last one
    if (back < q_len) keep[i] = proj[(size_t)(t_end - 1 - back) * ld + C + c] + xbias;
    else keep[i] = tail[(size_t)(i + q_len) * C + c];
  }
#pragma unroll
  for (int i = 0; i < MAX_TAPS; ++i) {
    if (i >= K - 1) break;
    tail[(size_t)i * C + c] = keep[i];
  }
}

// The scan of long prompts in chunks of SCAN_CHUNK tokens.  A chunk's effect on the state is S -> P S + Q (P the
// product of its decays, Q its own scan from zero): a first kernel writes (P, Q) of every chunk and the state each
// sequence starts from; a second one folds the chunks in front of its own, in order, and then walks its chunk as the
// plain scan does.  The thread of a sequence's last chunk stores S and the new tail of inputs.
constexpr int SCAN_CHUNK = 64;

__global__ void rglru_chunk_sums_kernel(const float* __restrict__ A, const float* __restrict__ Bv, const float* __restrict__ state,
                                        long long state_ld, float* __restrict__ PQ, float* __restrict__ S0, int C, int max_chunks,
                                        IertBatchView b) {
  pdl_launch_dependents();
  const int s = blockIdx.z, ch = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = b.slot_ids[s];
  if (slot < 0 || c >= C) return;
  const int q_begin = b.cu_q[s], q_len = b.cu_q[s + 1] - q_begin;
  if (ch * SCAN_CHUNK >= q_len) return;
  pdl_wait();
  if (ch == 0) S0[(size_t)s * C + c] = state[(size_t)slot * state_ld + c];
  const int t0 = q_begin + ch * SCAN_CHUNK, t1 = min(q_begin + q_len, t0 + SCAN_CHUNK);
  float P = 1.f, Q = 0.f;
  int t = t0;
  for (; t + 8 <= t1; t += 8) {
    float a[8], bv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { a[j] = A[(size_t)(t + j) * C + c]; bv[j] = Bv[(size_t)(t + j) * C + c]; }
#pragma unroll
    for (int j = 0; j < 8; ++j) { P *= a[j]; Q = fmaf(a[j], Q, bv[j]); }
  }
  for (; t < t1; ++t) { const float a = A[(size_t)t * C + c]; P *= a; Q = fmaf(a, Q, Bv[(size_t)t * C + c]); }
  float* pq = PQ + (((size_t)s * max_chunks + ch) * 2) * C;
  pq[c] = P;
  pq[C + c] = Q;
}

template <typename TO>
__global__ void rglru_chunk_scan_kernel(const float* __restrict__ A, const float* __restrict__ Bv, const float* __restrict__ proj,
                                        long long ld, const float* __restrict__ by, const float* __restrict__ bx,
                                        float* __restrict__ state, long long state_ld, const float* __restrict__ PQ,
                                        const float* __restrict__ S0, TO* __restrict__ out, float out_scale, int C, int K,
                                        int max_chunks, IertBatchView b) {
  pdl_launch_dependents();
  const int s = blockIdx.z, ch = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = b.slot_ids[s];
  if (slot < 0 || c >= C) return;
  const int q_begin = b.cu_q[s], q_len = b.cu_q[s + 1] - q_begin;
  if (ch * SCAN_CHUNK >= q_len) return;
  const float ybias = by[c], xbias = bx[c];
  pdl_wait();
  float S = S0[(size_t)s * C + c];
  for (int j = 0; j < ch; ++j) {
    const float* pq = PQ + (((size_t)s * max_chunks + j) * 2) * C;
    S = fmaf(pq[c], S, pq[C + c]);
  }
  const int t0 = q_begin + ch * SCAN_CHUNK, t_end = q_begin + q_len, t1 = min(t_end, t0 + SCAN_CHUNK);
  int t = t0;
  for (; t + 4 <= t1; t += 4) {
    float a[4], bv[4], py[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      a[j] = A[(size_t)(t + j) * C + c];
      bv[j] = Bv[(size_t)(t + j) * C + c];
      py[j] = proj[(size_t)(t + j) * ld + c];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      S = fmaf(a[j], S, bv[j]);
      out[(size_t)(t + j) * C + c] = from_f32<TO>(S * gelu_tanh_f(py[j] + ybias) * out_scale);
    }
  }
  for (; t < t1; ++t) {
    S = fmaf(A[(size_t)t * C + c], S, Bv[(size_t)t * C + c]);
    out[(size_t)t * C + c] = from_f32<TO>(S * gelu_tanh_f(proj[(size_t)t * ld + c] + ybias) * out_scale);
  }
  if (t1 != t_end) return;
  float* st = state + (size_t)slot * state_ld;
  st[c] = S;
  float* tail = st + C;
  float keep[MAX_TAPS];
#pragma unroll
  for (int i = 0; i < MAX_TAPS; ++i) {
    if (i >= K - 1) break;
    const int back = K - 2 - i;
    if (back < q_len) keep[i] = proj[(size_t)(t_end - 1 - back) * ld + C + c] + xbias;
    else keep[i] = tail[(size_t)(i + q_len) * C + c];
  }
#pragma unroll
  for (int i = 0; i < MAX_TAPS; ++i) {
    if (i >= K - 1) break;
    tail[(size_t)i * C + c] = keep[i];
  }
}

}  // namespace

IERT_API int iert_rglru_conv(const float* proj, long long ld, const float* bx, const float* taps, const float* cb,
                             const float* state, long long state_ld, float* u, int C, int K, const IertBatchView* batch,
                             cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  if (C <= 0 || K < 1 || K > MAX_TAPS) return IERT_BAD_ARGUMENT;
  if (C % 4 == 0 && ld % 4 == 0 && state_ld % 4 == 0 &&
      (((uintptr_t)proj | (uintptr_t)bx | (uintptr_t)cb | (uintptr_t)state | (uintptr_t)u) & 15) == 0) {
    const int ch = 4 * CONV_THREADS;
    const int per = batch->n_tokens >= 256 ? CONV_TOKENS : 1;
    launch_dep(rglru_conv4_kernel, dim3((batch->n_tokens + per - 1) / per, (C + ch - 1) / ch), dim3(CONV_THREADS),
               (size_t)K * ch * sizeof(float), stream, proj, ld, bx, taps, cb, state, state_ld, u, C, K, per, *batch);
    return iert_check_launch("rglru_conv");
  }
  const int threads = C >= 256 ? 256 : 64;
  launch_dep(rglru_conv_kernel, dim3(batch->n_tokens, (C + threads - 1) / threads), dim3(threads), 0, stream, proj, ld, bx,
             taps, cb, state, state_ld, u, C, K, *batch);
  return iert_check_launch("rglru_conv");
}

// Ra, Ri: [blocks, bw, bw] of `w_dtype`; u, A, Bv: fp32 [T, C]; decay_c: the constant in log a = -c r softplus(lam).
IERT_API int iert_rglru_gates(const float* u, const void* Ra, const float* ra_b, const void* Ri, const float* ri_b,
                              int w_dtype, const float* lam, float decay_c, float* A, float* Bv, int T, int C, int blocks,
                              cudaStream_t stream) {
  if (T <= 0) return IERT_OK;
  if (C <= 0 || blocks <= 0 || C % blocks) return IERT_BAD_ARGUMENT;
  const int bw = C / blocks;
  if (blocks > 65535 || (bw + GO - 1) / GO > 65535) return IERT_BAD_ARGUMENT;
  if (T <= 8 * SMALL_T) {
    const dim3 g((C + 7) / 8);
    const int vec8 = bw % 8 == 0 && (((uintptr_t)u | (uintptr_t)Ra | (uintptr_t)Ri) & 15) == 0;
    if (w_dtype == IERT_F32)
      launch_dep(rglru_gates_small_kernel<float>, g, dim3(256), 0, stream, u, (const float*)Ra, ra_b, (const float*)Ri, ri_b, lam,
                 decay_c, A, Bv, T, C, bw, vec8);
    else if (w_dtype == IERT_BF16)
      launch_dep(rglru_gates_small_kernel<__nv_bfloat16>, g, dim3(256), 0, stream, u, (const __nv_bfloat16*)Ra, ra_b,
                 (const __nv_bfloat16*)Ri, ri_b, lam, decay_c, A, Bv, T, C, bw, vec8);
    else
      return IERT_BAD_ARGUMENT;
    return iert_check_launch("rglru_gates");
  }
  // bfloat16 weights, blocks in whole runs of eight and everything aligned for the vector loads: the tensor cores
  if (w_dtype == IERT_BF16 && bw % 8 == 0 && (((uintptr_t)u | (uintptr_t)A | (uintptr_t)Bv | (uintptr_t)Ra | (uintptr_t)Ri) & 15) == 0 &&
      (bw + TN - 1) / TN <= 65535) {
    launch_dep(rglru_gates_tc_kernel, dim3((T + TM - 1) / TM, (bw + TN - 1) / TN, blocks), dim3(TC_THREADS), 0, stream, u,
               (const __nv_bfloat16*)Ra, ra_b, (const __nv_bfloat16*)Ri, ri_b, lam, decay_c, A, Bv, T, C, bw);
    return iert_check_launch("rglru_gates");
  }
  dim3 grid((T + GT - 1) / GT, (bw + GO - 1) / GO, blocks);
  if (w_dtype == IERT_F32)
    launch_dep(rglru_gates_kernel<float>, grid, dim3(GTHREADS), 0, stream, u, (const float*)Ra, ra_b, (const float*)Ri, ri_b,
               lam, decay_c, A, Bv, T, C, bw);
  else if (w_dtype == IERT_BF16)
    launch_dep(rglru_gates_kernel<__nv_bfloat16>, grid, dim3(GTHREADS), 0, stream, u, (const __nv_bfloat16*)Ra, ra_b,
               (const __nv_bfloat16*)Ri, ri_b, lam, decay_c, A, Bv, T, C, bw);
  else
    return IERT_BAD_ARGUMENT;
  return iert_check_launch("rglru_gates");
}

// Floats of scratch the chunked scan needs for sequences of up to `max_q_len` tokens.
IERT_API long long iert_rglru_scan_scratch_floats(int n_seqs, int max_q_len, int C) {
  const long long chunks = (max_q_len + SCAN_CHUNK - 1) / SCAN_CHUNK;
  return (long long)n_seqs * C * (2 * chunks + 1);
}

// max_q_len: the longest sequence of the step.  With `scratch` (iert_rglru_scan_scratch_floats) sequences of more than
// two chunks are scanned chunk by chunk; without it, or for short ones, a thread walks its whole sequence.
IERT_API int iert_rglru_scan(const float* A, const float* Bv, const float* proj, long long ld, const float* by,
                             const float* bx, float* state, long long state_ld, void* out, int out_dtype, float out_scale,
                             int C, int K, int max_q_len, float* scratch, const IertBatchView* batch, cudaStream_t stream) {
  if (batch->n_tokens <= 0 || batch->n_seqs <= 0) return IERT_OK;
  if (C <= 0 || K < 1 || K > MAX_TAPS || batch->n_seqs > 65535) return IERT_BAD_ARGUMENT;
  if (scratch && max_q_len > 2 * SCAN_CHUNK) {
    const int chunks = (max_q_len + SCAN_CHUNK - 1) / SCAN_CHUNK;
    if (chunks > 65535) return IERT_BAD_ARGUMENT;
    float* S0 = scratch;
    float* PQ = scratch + (size_t)batch->n_seqs * C;
    const int th = 128;
    dim3 grid((C + th - 1) / th, chunks, batch->n_seqs);
    launch_dep(rglru_chunk_sums_kernel, grid, dim3(th), 0, stream, A, Bv, (const float*)state, state_ld, PQ, S0, C, chunks, *batch);
    if (out_dtype == IERT_F32)
      launch_dep(rglru_chunk_scan_kernel<float>, grid, dim3(th), 0, stream, A, Bv, proj, ld, by, bx, state, state_ld,
                 (const float*)PQ, (const float*)S0, (float*)out, out_scale, C, K, chunks, *batch);
    else if (out_dtype == IERT_BF16)
      launch_dep(rglru_chunk_scan_kernel<__nv_bfloat16>, grid, dim3(th), 0, stream, A, Bv, proj, ld, by, bx, state, state_ld,
                 (const float*)PQ, (const float*)S0, (__nv_bfloat16*)out, out_scale, C, K, chunks, *batch);
    else
      return IERT_BAD_ARGUMENT;
    return iert_check_launch("rglru_scan");
  }
  const int threads = C >= 4096 ? 128 : 64;
  dim3 grid((C + threads - 1) / threads, batch->n_seqs);
  if (out_dtype == IERT_F32)
    launch_dep(rglru_scan_kernel<float>, grid, dim3(threads), 0, stream, A, Bv, proj, ld, by, bx, state, state_ld, (float*)out,
               out_scale, C, K, *batch);
  else if (out_dtype == IERT_BF16)
    launch_dep(rglru_scan_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, A, Bv, proj, ld, by, bx, state, state_ld,
               (__nv_bfloat16*)out, out_scale, C, K, *batch);
  else
    return IERT_BAD_ARGUMENT;
  return iert_check_launch("rglru_scan");
}
