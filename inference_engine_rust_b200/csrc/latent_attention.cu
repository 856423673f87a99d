// Attention whose keys and values are expanded from one low-rank row c per token (the only thing
// the cache keeps), without positions, with a sink in the softmax's denominator:
//
//   weights  p_j = exp(s_j - M) / (sum_j exp(s_j - M) + exp(sink_h - M)),  s_j = (q . k_j) * scale,
//   M = max(max_j s_j, sink_h); the sink is a bare logit per head: it enters the denominator unscaled and
//   adds nothing to the numerator.
//
// latent_norm_store: RMS norm (plain weight, eps inside the root) of the two down-projections of a
//   token (query latent, key/value latent), fp32 statistics; the key/value latent is also written to
//   the paged cache (kv_heads = 1, head_dim = rank).
// latent_attention_prompt: a prompt that starts at position 0 attends over the step's own expanded
//   keys and values, packed per token as q [H*D] | k [H*D] | v [H*V] (D and V may differ).
// latent_attention_decode: one token per sequence over the cached latents, in the absorbed form:
//   qa = W_uk[h]^T q  (rank numbers), s_j = (qa . c_j) * scale, l = sum_j p_j c_j, o = W_uv[h] l.
//   Nothing is expanded per cached position.
// All arithmetic is fp32; one block per (token, head); keys are visited in chunks with a running
// maximum and sum, so the memory needed does not grow with the context.
#include "common.cuh"

using namespace iert;

namespace {

constexpr int THREADS = 128;
constexpr int MAX_PER_THREAD = 8;       // value size / rank up to 1024

template <typename T>
__global__ void latent_norm_store_kernel(const float* __restrict__ x, long long ldx, int q_rank, int kv_rank,
                                         const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                                         T* __restrict__ cq, T* __restrict__ c, IertBatchView b, IertKvView kv,
                                         int store, int* __restrict__ err) {
  __shared__ float scratch[33];
  pdl_wait();
  const int t = blockIdx.x;
  const int s = sequence_of_token(b, t);
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  if (slot < 0) return;
  const float* row = x + (size_t)t * ldx;
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  const float rq = 1.0f / sqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cq[(size_t)t * q_rank + i] = from_f32<T>(row[i] * rq * wq[i]);
  ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) ss = fmaf(row[q_rank + i], row[q_rank + i], ss);
  const float rk = 1.0f / sqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);
  T* dst = nullptr;
  if (store) {
    const int pos = b.pos0[s] + (t - b.cu_q[s]);
    const long long off = kv_row_offset(kv, slot, pos, 0, err);
    if (off >= 0) dst = (T*)kv.k + off;
  }
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
    const T v = from_f32<T>(row[q_rank + i] * rk * wkv[i]);
    c[(size_t)t * kv_rank + i] = v;
    if (dst) dst[i] = v;
  }
}

// Shared by both attention kernels: one chunk of scores is in sc (this thread's key) -> running
// maximum / sum update; returns the factor for what was accumulated so far and leaves p in p_s.
__device__ __forceinline__ float softmax_chunk(float sc, float& m, float& l, float* p_s, float* scratch) {
  const float m_new = fmaxf(m, block_max(sc, scratch));
  const float p = sc == -INFINITY ? 0.f : expf(sc - m_new);
  const float alpha = m == -INFINITY ? 0.f : expf(m - m_new);
  l = l * alpha + block_sum(p, scratch);
  m = m_new;
  p_s[threadIdx.x] = p;
  __syncthreads();
  return alpha;
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
latent_attention_prompt_kernel(const T* __restrict__ qkv, long long ld, T* __restrict__ out, IertBatchView b,
                               int H, int D, int V, float scale, const float* __restrict__ sink) {
  extern __shared__ float smem[];
  float* q_s = smem;                  // [D]
  float* p_s = smem + D;              // [THREADS]
  float* scratch = p_s + THREADS;     // [33]
  pdl_wait();
  const int t = blockIdx.x, head = blockIdx.y;
  T* o = out + ((size_t)t * H + head) * V;
  const int s = sequence_of_token(b, t);
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  if (slot < 0) {
    for (int e = threadIdx.x; e < V; e += THREADS) o[e] = from_f32<T>(0.f);
    return;
  }
  const int q_begin = b.cu_q[s];
  const int pos = t - q_begin;                       // the prompt starts at position 0
  const T* q = qkv + (size_t)t * ld + (size_t)head * D;
  for (int d = threadIdx.x; d < D; d += THREADS) q_s[d] = to_f32(q[d]);
  __syncthreads();
  const float snk = sink ? sink[head] : -INFINITY;
  float m = snk, l = sink ? 1.f : 0.f;               // the sink: a term exp(sink - M) with no value
  float acc[MAX_PER_THREAD];
#pragma unroll
  for (int i = 0; i < MAX_PER_THREAD; ++i) acc[i] = 0.f;
  for (int j0 = 0; j0 <= pos; j0 += THREADS) {
    const int j = j0 + threadIdx.x;
    float sc = -INFINITY;
    if (j <= pos) {
      const T* k = qkv + (size_t)(q_begin + j) * ld + (size_t)(H + head) * D;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(q_s[d], to_f32(k[d]), dot);
      sc = dot * scale;
    }
    const float alpha = softmax_chunk(sc, m, l, p_s, scratch);
    const int n_in = min(THREADS, pos - j0 + 1);
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
      const int e = threadIdx.x + i * THREADS;
      if (e >= V) break;
      float a = acc[i] * alpha;
      const T* v = qkv + (size_t)(q_begin + j0) * ld + (size_t)2 * H * D + (size_t)head * V + e;
      for (int jj = 0; jj < n_in; ++jj) a = fmaf(p_s[jj], to_f32(v[(size_t)jj * ld]), a);
      acc[i] = a;
    }
    __syncthreads();
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < MAX_PER_THREAD; ++i) {
    const int e = threadIdx.x + i * THREADS;
    if (e < V) o[e] = from_f32<T>(acc[i] * inv);
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
latent_attention_decode_kernel(const T* __restrict__ q, long long ldq, const T* __restrict__ w_uk,
                               const T* __restrict__ w_uv, T* __restrict__ out, IertBatchView b, IertKvView kv,
                               int H, int D, int V, float scale, const float* __restrict__ sink,
                               int* __restrict__ err) {
  extern __shared__ float smem[];
  const int rank = kv.head_dim;
  float* qa = smem;                   // [rank]: the query in the latent's coordinates
  float* lat = qa + rank;             // [rank]: the weighted sum of latents
  float* q_s = lat + rank;            // [D]
  float* p_s = q_s + D;               // [THREADS]
  float* scratch = p_s + THREADS;     // [33]
  pdl_wait();
  const int t = blockIdx.x, head = blockIdx.y;
  T* o = out + ((size_t)t * H + head) * V;
  const int s = sequence_of_token(b, t);
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  if (slot < 0) {
    for (int e = threadIdx.x; e < V; e += THREADS) o[e] = from_f32<T>(0.f);
    return;
  }
  const int pos = b.pos0[s] + (t - b.cu_q[s]);
  for (int d = threadIdx.x; d < D; d += THREADS) q_s[d] = to_f32(q[(size_t)t * ldq + (size_t)head * D + d]);
  __syncthreads();
  for (int r = threadIdx.x; r < rank; r += THREADS) {
    const T* w = w_uk + (size_t)head * D * rank + r;
    float a = 0.f;
    for (int d = 0; d < D; ++d) a = fmaf(q_s[d], to_f32(w[(size_t)d * rank]), a);
    qa[r] = a;
  }
  __syncthreads();
  const float snk = sink ? sink[head] : -INFINITY;
  float m = snk, l = sink ? 1.f : 0.f;
  float acc[MAX_PER_THREAD];
#pragma unroll
  for (int i = 0; i < MAX_PER_THREAD; ++i) acc[i] = 0.f;
  const T* cache = (const T*)kv.k;
  for (int j0 = 0; j0 <= pos; j0 += THREADS) {
    const int j = j0 + threadIdx.x;
    float sc = -INFINITY;
    if (j <= pos) {
      const long long off = kv_row_offset(kv, slot, j, 0, err);
      if (off >= 0) {
        const T* c = cache + off;
        float dot = 0.f;
        for (int r = 0; r < rank; ++r) dot = fmaf(qa[r], to_f32(c[r]), dot);
        sc = dot * scale;
      }
    }
    const float alpha = softmax_chunk(sc, m, l, p_s, scratch);
    const int n_in = min(THREADS, pos - j0 + 1);
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
      const int r = threadIdx.x + i * THREADS;
      if (r >= rank) break;
      float a = acc[i] * alpha;
      for (int jj = 0; jj < n_in; ++jj) {
        const float pj = p_s[jj];
        if (pj == 0.f) continue;
        const long long off = kv_row_offset(kv, slot, j0 + jj, 0, nullptr);
        if (off < 0) continue;
        a = fmaf(pj, to_f32(cache[off + r]), a);
      }
      acc[i] = a;
    }
    __syncthreads();
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < MAX_PER_THREAD; ++i) {
    const int r = threadIdx.x + i * THREADS;
    if (r < rank) lat[r] = acc[i] * inv;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = warp; e < V; e += THREADS / 32) {
    const T* w = w_uv + ((size_t)head * V + e) * rank;
    float a = 0.f;
    for (int r = lane; r < rank; r += 32) a = fmaf(to_f32(w[r]), lat[r], a);
    a = warp_sum(a);
    if (lane == 0) o[e] = from_f32<T>(a);
  }
}

}  // namespace

// x: fp32 [T, ldx] = query latent [q_rank] | key/value latent [kv_rank], before their norms.
IERT_API int iert_latent_norm_store(const float* x, long long ldx, int q_rank, int kv_rank, const float* wq,
                                    const float* wkv, float eps, void* cq, void* c, int dtype,
                                    const IertBatchView* batch, const IertKvView* kv, int store, int* err,
                                    cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  if (q_rank <= 0 || kv_rank <= 0 || (store && (kv->head_dim != kv_rank || kv->kv_heads != 1 || kv->dtype != dtype)))
    return IERT_BAD_ARGUMENT;
  if (dtype == IERT_F32)
    launch_dep(latent_norm_store_kernel<float>, dim3(batch->n_tokens), dim3(128), 0, stream, x, ldx, q_rank, kv_rank, wq,
               wkv, eps, (float*)cq, (float*)c, *batch, *kv, store, err);
  else if (dtype == IERT_BF16)
    launch_dep(latent_norm_store_kernel<__nv_bfloat16>, dim3(batch->n_tokens), dim3(128), 0, stream, x, ldx, q_rank,
               kv_rank, wq, wkv, eps, (__nv_bfloat16*)cq, (__nv_bfloat16*)c, *batch, *kv, store, err);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("latent_norm_store");
}

// qkv: [T, ld] packed q [H*D] | k [H*D] | v [H*V]; out [T, H*V]; sink fp32 [H] or nullptr.
IERT_API int iert_latent_attention_prompt(const void* qkv, long long ld, void* out, int dtype,
                                          const IertBatchView* batch, int H, int D, int V, float scale,
                                          const float* sink, cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  if (H <= 0 || H > 65535 || D <= 0 || V <= 0 || V > THREADS * MAX_PER_THREAD || D > 8192) return IERT_BAD_ARGUMENT;
  dim3 grid(batch->n_tokens, H);
  const size_t smem = (size_t)(D + THREADS + 33) * sizeof(float);
  if (dtype == IERT_F32)
    launch_dep(latent_attention_prompt_kernel<float>, grid, dim3(THREADS), smem, stream, (const float*)qkv, ld,
               (float*)out, *batch, H, D, V, scale, sink);
  else if (dtype == IERT_BF16)
    launch_dep(latent_attention_prompt_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream,
               (const __nv_bfloat16*)qkv, ld, (__nv_bfloat16*)out, *batch, H, D, V, scale, sink);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("latent_attention_prompt");
}

// q: [T, ldq] (H*D per token); w_uk [H*D, rank], w_uv [H*V, rank] row-major in the run's dtype;
// the cache view holds the latents (k only).  out [T, H*V].
IERT_API int iert_latent_attention_decode(const void* q, long long ldq, const void* w_uk, const void* w_uv, void* out,
                                          int dtype, const IertBatchView* batch, const IertKvView* kv, int H, int D,
                                          int V, float scale, const float* sink, int* err, cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  const int rank = kv->head_dim;
  if (H <= 0 || H > 65535 || D <= 0 || V <= 0 || rank <= 0 || rank > THREADS * MAX_PER_THREAD || kv->kv_heads != 1 ||
      kv->dtype != dtype || 2 * rank + D > 10000)
    return IERT_BAD_ARGUMENT;
  dim3 grid(batch->n_tokens, H);
  const size_t smem = (size_t)(2 * rank + D + THREADS + 33) * sizeof(float);
  if (dtype == IERT_F32)
    launch_dep(latent_attention_decode_kernel<float>, grid, dim3(THREADS), smem, stream, (const float*)q, ldq,
               (const float*)w_uk, (const float*)w_uv, (float*)out, *batch, *kv, H, D, V, scale, sink, err);
  else if (dtype == IERT_BF16)
    launch_dep(latent_attention_decode_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream,
               (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)w_uk, (const __nv_bfloat16*)w_uv,
               (__nv_bfloat16*)out, *batch, *kv, H, D, V, scale, sink, err);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("latent_attention_decode");
}
