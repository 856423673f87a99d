// Routing of a mixture-of-experts feed-forward.
//
// router_topk: logits z = x W_r^T (+ bias) arrive in fp32 [T, E]; the `top` largest are chosen (the
//   lower index wins a tie) and their weights are the softmax over the chosen logits only.  Written as
//   a dense map wt [T, E] (zero for experts not chosen) and as lists idx / w [T, top].
// moe_scale: act[t, e*F + i] *= wt[t, e] for the E routed experts' blocks of F activations; columns
//   beyond E*F (an expert that every token uses) are left as they are.
#include "common.cuh"

using namespace iert;

namespace {

constexpr int MAX_TOP = 32;

__global__ void router_topk_kernel(const float* __restrict__ z, long long ldz, const float* __restrict__ bias,
                                   int E, int top, float* __restrict__ wt, int* __restrict__ idx,
                                   float* __restrict__ w) {
  // one warp per token
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x;
  const float* row = z + (size_t)t * ldz;
  int chosen[MAX_TOP];
  float val[MAX_TOP];
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= chosen[j] == e;
      const float v = row[e] + (bias ? bias[e] : 0.f);
      if (!taken && (v > best || (v == best && e < bi))) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    chosen[k] = bi;
    val[k] = best;
  }
  float den = 0.f;
  const float largest = val[0];
  for (int k = 0; k < top; ++k) { val[k] = expf(val[k] - largest); den += val[k]; }
  for (int e = lane; e < E; e += 32) wt[(size_t)t * E + e] = 0.f;
  __syncwarp();
  if (lane == 0)
    for (int k = 0; k < top; ++k) {
      const float p = val[k] / den;
      if (chosen[k] < E) wt[(size_t)t * E + chosen[k]] = p;
      idx[(size_t)t * top + k] = chosen[k];
      w[(size_t)t * top + k] = p;
    }
}

template <typename T>
__global__ void moe_scale_kernel(T* __restrict__ act, long long ld, const float* __restrict__ wt, int E, int F) {
  pdl_wait();
  const int t = blockIdx.x;
  T* row = act + (size_t)t * ld;
  if (sizeof(T) == 2 && F % 8 == 0 && ld % 8 == 0 && ((uintptr_t)act & 15) == 0) {      // eight at a time
    for (int i = threadIdx.x * 8; i < E * F; i += blockDim.x * 8) {
      const float w = wt[(size_t)t * E + i / F];
      uint4 v = *reinterpret_cast<const uint4*>(row + i);
      __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]);
        p[e] = __floats2bfloat162_rn(f.x * w, f.y * w);
      }
      *reinterpret_cast<uint4*>(row + i) = v;
    }
    return;
  }
  for (int i = threadIdx.x; i < E * F; i += blockDim.x)
    row[i] = from_f32<T>(to_f32(row[i]) * wt[(size_t)t * E + i / F]);
}

}  // namespace

IERT_API int iert_router_topk(const float* z, long long ldz, const float* bias, int n_tokens, int E, int top,
                              float* wt, int* idx, float* w, cudaStream_t stream) {
  if (n_tokens <= 0) return IERT_OK;
  if (E <= 0 || top <= 0 || top > E || top > MAX_TOP) return IERT_BAD_ARGUMENT;
  launch_dep(router_topk_kernel, dim3(n_tokens), dim3(32), 0, stream, z, ldz, bias, E, top, wt, idx, w);
  return iert_check_launch("router_topk");
}

IERT_API int iert_moe_scale(void* act, int dtype, long long ld, const float* wt, int n_tokens, int E, int F,
                            cudaStream_t stream) {
  if (n_tokens <= 0) return IERT_OK;
  if (E <= 0 || F <= 0) return IERT_BAD_ARGUMENT;
  if (dtype == IERT_F32) launch_dep(moe_scale_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, (float*)act, ld, wt, E, F);
  else if (dtype == IERT_BF16)
    launch_dep(moe_scale_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, (__nv_bfloat16*)act, ld, wt, E, F);
  else return IERT_BAD_ARGUMENT;
  return iert_check_launch("moe_scale");
}
