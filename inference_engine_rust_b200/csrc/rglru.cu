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

// u[t, c] for every token of the step.  proj: fp32 [T, 2C] = [py | px].
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

// The scan: a thread per (sequence, channel).
constexpr int MAX_TAPS = 16;

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

}  // namespace

IERT_API int iert_rglru_conv(const float* proj, long long ld, const float* bx, const float* taps, const float* cb,
                             const float* state, long long state_ld, float* u, int C, int K, const IertBatchView* batch,
                             cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  if (C <= 0 || K < 1 || K > MAX_TAPS) return IERT_BAD_ARGUMENT;
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

IERT_API int iert_rglru_scan(const float* A, const float* Bv, const float* proj, long long ld, const float* by,
                             const float* bx, float* state, long long state_ld, void* out, int out_dtype, float out_scale,
                             int C, int K, const IertBatchView* batch, cudaStream_t stream) {
  if (batch->n_tokens <= 0 || batch->n_seqs <= 0) return IERT_OK;
  if (C <= 0 || K < 1 || K > MAX_TAPS || batch->n_seqs > 65535) return IERT_BAD_ARGUMENT;
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
