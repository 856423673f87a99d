// Preparation of queries and keys for attention whose keys double as values: from the fp32 projection
// row [q | k] of a token to the packed row [q' | k' | v] that the attention kernels read, plus the cache
// write of k' and v.  All arithmetic fp32, one rounding at the end.
//
//   v  = k as projected, times `value_scale` (a fixed factor on the mixer's result, which is linear in v)
//   norm_mode 1: q and k each divided by the root mean square over their WHOLE projection and multiplied
//                by a weight of that length, before the rotation
//   rotation of the first `rotary_dim` numbers of every head, number i with number i + rotary_dim / 2,
//                by position * inv_freq[i]
//   norm_mode 2: after the rotation every head of q and k divided by its own root mean square (no weight)
//
// One block per token.  The row is held in shared memory.
#include "common.cuh"

using namespace iert;

namespace {

constexpr int THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(THREADS)
qk_prep_kernel(const float* __restrict__ proj, long long ld, T* __restrict__ qkv, IertBatchView b, IertKvView c, int heads,
               const float* __restrict__ inv_freq, int rotary_dim, int norm_mode, const float* __restrict__ wq,
               const float* __restrict__ wk, float eps, float value_scale, int write_cache, int heads_per_block,
               int* __restrict__ err) {
  extern __shared__ float sm[];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int hd = c.head_dim, nkv = c.kv_heads;
  const int qd = heads * hd, kd = nkv * hd, half = rotary_dim / 2;
  float* row = sm;                       // [qd + kd]
  float* cs = sm + qd + kd;              // [half] cos, [half] sin
  const int t = blockIdx.x;
  const int s = sequence_of_token(b, t);
  const int slot = s < 0 ? -1 : b.slot_ids[s];
  if (slot < 0) {
    // a padding token: a defined row (the prompt attention kernels read whole tiles of keys and values, and a masked
    // key's weight of zero times a NaN left in this row would still be NaN)
    pdl_wait();
    T* pad = qkv + (size_t)t * (qd + 2 * kd);
    if (blockIdx.y == 0)
      for (int i = threadIdx.x; i < qd + 2 * kd; i += THREADS) pad[i] = from_f32<T>(0.f);
    return;
  }
  const int q_begin = b.cu_q[s], q_len = b.cu_q[s + 1] - q_begin;
  const int pos = b.pos0[s] + (t - q_begin);
  const int final_len = b.pos0[s] + q_len;
  for (int k = threadIdx.x; k < half; k += THREADS) {
    float sn, co;
    sincosf((float)pos * inv_freq[k], &sn, &co);
    cs[k] = co;
    cs[half + k] = sn;
  }
  pdl_wait();
  const bool store = write_cache && pos >= final_len - c.ring_pages * c.page_tokens;
  const float* pr = proj + (size_t)t * ld;
  T* out = qkv + (size_t)t * (qd + 2 * kd);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_heads = heads + nkv;
  constexpr int WARPS = THREADS / 32;
  // this block's heads of [queries | keys]: [h_lo, h_hi) (few tokens: the heads of a token are spread over blocks)
  const int h_lo = blockIdx.y * heads_per_block, h_hi = min(n_heads, h_lo + heads_per_block);
  float ssq = 0.f, ssk = 0.f;
  if (norm_mode == 1 || heads_per_block >= n_heads) {           // the whole row (its sums of squares are needed)
    for (int i = threadIdx.x; i < qd + kd; i += THREADS) {
      const float v = pr[i];
      row[i] = v;
      if (i < qd) ssq = fmaf(v, v, ssq); else ssk = fmaf(v, v, ssk);
    }
  } else {
    for (int i = h_lo * hd + threadIdx.x; i < h_hi * hd; i += THREADS) row[i] = pr[i];
  }
  if (norm_mode == 1) {
    ssq = block_sum(ssq, scratch);
    ssk = block_sum(ssk, scratch);
  } else {
    __syncthreads();
  }
  // the values: the keys as projected (a warp per head: the place in the cache is worked out once per head)
  for (int h = max(h_lo, heads) - heads + warp; h < h_hi - heads; h += WARPS) {
    const long long off = store ? kv_row_offset(c, slot, pos, h, err) : -1;
    const float* src = row + qd + (size_t)h * hd;
    T* dst = out + qd + kd + (size_t)h * hd;
    for (int d = lane; d < hd; d += 32) {
      const T v = from_f32<T>(src[d] * value_scale);
      dst[d] = v;
      if (off >= 0) ((T*)c.v)[off + d] = v;
    }
  }
  const float rq = 1.0f / sqrtf(ssq / (float)qd + eps), rk = 1.0f / sqrtf(ssk / (float)kd + eps);
  __syncthreads();
  // per head: the whole-projection norm's factor and weight, the rotation, the unit norm, the rounding and the stores
  for (int h = h_lo + warp; h < h_hi; h += WARPS) {
    float* v = row + (size_t)h * hd;
    if (norm_mode == 1) {
      const float r = h < heads ? rq : rk;
      const float* w = h < heads ? wq + (size_t)h * hd : wk + (size_t)(h - heads) * hd;
      for (int d = lane; d < hd; d += 32) v[d] *= r * w[d];
      __syncwarp();
    }
    for (int k = lane; k < half; k += 32) {
      const float a = v[k], bb = v[k + half];
      v[k] = a * cs[k] - bb * cs[half + k];
      v[k + half] = bb * cs[k] + a * cs[half + k];
    }
    __syncwarp();
    float r = 1.f;
    if (norm_mode == 2) {
      float ss = 0.f;
      for (int d = lane; d < hd; d += 32) ss = fmaf(v[d], v[d], ss);
      ss = warp_sum(ss);
      r = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    T* dst = out + (size_t)h * hd;
    const long long off = (store && h >= heads) ? kv_row_offset(c, slot, pos, h - heads, nullptr) : -1;
    for (int d = lane; d < hd; d += 32) {
      const T o = from_f32<T>(v[d] * r);
      dst[d] = o;
      if (off >= 0) ((T*)c.k)[off + d] = o;
    }
  }
}

}  // namespace

// proj: fp32 [T, heads*hd + kv_heads*hd] (row stride ld); qkv: [T, (heads + 2 kv_heads) * hd] of `dtype` (= the cache's).
IERT_API int iert_qk_prep(const float* proj, long long ld, void* qkv, int dtype, const IertBatchView* batch,
                          const IertKvView* cache, int heads, const float* inv_freq, int rotary_dim, int norm_mode,
                          const float* wq, const float* wk, float eps, float value_scale, int write_cache, int* err,
                          cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  const int hd = cache->head_dim;
  if (rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1) || cache->dtype != dtype || norm_mode < 0 || norm_mode > 2 ||
      (norm_mode == 1 && (!wq || !wk)))
    return IERT_BAD_ARGUMENT;
  const size_t smem = ((size_t)(heads + cache->kv_heads) * hd + rotary_dim) * sizeof(float);
  if (smem > 200 * 1024) return IERT_BAD_ARGUMENT;
  // many tokens: a block per token; few: the heads of a token over several blocks, a warp's worth of heads each
  const int n_heads = heads + cache->kv_heads;
  const int per_block = batch->n_tokens >= 256 ? n_heads : (n_heads >= 16 ? 8 : n_heads);
  const int groups = (n_heads + per_block - 1) / per_block;
  // the opt-in for more than 48 KB of dynamic shared memory, asked once per size (and not again inside a stream capture)
#define GO(T)                                                                                                          \
  do {                                                                                                                 \
    static size_t allowed = 48 * 1024;                                                                                 \
    if (smem > allowed) {                                                                                              \
      if (cudaFuncSetAttribute(qk_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { \
        cudaGetLastError();                                                                                            \
        return IERT_BAD_ARGUMENT;                                                                                      \
      }                                                                                                                \
      allowed = smem;                                                                                                  \
    }                                                                                                                  \
    launch_dep(qk_prep_kernel<T>, dim3(batch->n_tokens, groups), dim3(THREADS), smem, stream, proj, ld, (T*)qkv, *batch,   \
               *cache, heads, inv_freq, rotary_dim, norm_mode, wq, wk, eps, value_scale, write_cache, per_block, err);    \
  } while (0)
  if (dtype == IERT_F32) GO(float);
  else if (dtype == IERT_BF16) GO(__nv_bfloat16);
  else return IERT_BAD_ARGUMENT;
#undef GO
  return iert_check_launch("qk_prep");
}
