// Kernels of layers that norm a sublayer's OUTPUT instead of its input:
//
//   x <- x + y / sqrt(mean(y^2) + eps) * w        (x: fp32 residual rows, y: fp32 sublayer output)
//
// in one pass that also clears y for the sublayer to come (sublayers add into it) and writes the new
// residual rows in the run's dtype, which is what the next sublayer's projections read.  The weight w
// arrives in fp32 with any offset (a weight stored around zero) already added.  Statistics, the
// product and the sum are fp32; the order of the additions depends on the row length alone.
//
// `cast_rows` is the same without a sublayer output: the residual rows in the run's dtype and a
// cleared y, for the first sublayer of a step.
#include "common.cuh"

using namespace iert;

namespace {

constexpr int THREADS = 256;

__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

// Rows of up to 4 * V * THREADS numbers, 16-byte accesses: every load of a row (y, x and the weight) is issued before the
// first is used, so a row costs one round trip to memory, one block-wide sum and the stores.
template <typename TO, int V>
__global__ void __launch_bounds__(THREADS)
add_normed_rows_kernel(float* __restrict__ x, float* __restrict__ y, const float* __restrict__ w, TO* __restrict__ cast,
                       int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int n4 = hidden >> 2;
  float4 g[V], v[V], a[V];
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int i = threadIdx.x + k * THREADS;
    g[k] = i < n4 ? *reinterpret_cast<const float4*>(w + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  const size_t r = blockIdx.x;
  float* yr = y + r * hidden;
  float* xr = x + r * hidden;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int i = threadIdx.x + k * THREADS;
    v[k] = i < n4 ? *reinterpret_cast<const float4*>(yr + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    a[k] = i < n4 ? *reinterpret_cast<const float4*>(xr + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int k = 0; k < V; ++k) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  ss = block_sum(ss, scratch);
  const float rinv = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int i = threadIdx.x + k * THREADS;
    if (i >= n4) continue;
    a[k].x += v[k].x * rinv * g[k].x; a[k].y += v[k].y * rinv * g[k].y;
    a[k].z += v[k].z * rinv * g[k].z; a[k].w += v[k].w * rinv * g[k].w;
    *reinterpret_cast<float4*>(xr + 4 * i) = a[k];
    *reinterpret_cast<float4*>(yr + 4 * i) = make_float4(0.f, 0.f, 0.f, 0.f);
    if (cast) store4(cast + r * hidden + 4 * i, a[k]);
  }
}

template <typename TO>
__global__ void __launch_bounds__(THREADS)
add_normed_kernel(float* __restrict__ x, float* __restrict__ y, const float* __restrict__ w, TO* __restrict__ cast,
                  int hidden, float eps, int vec4) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t r = blockIdx.x;
  float* yr = y + r * hidden;
  float* xr = x + r * hidden;
  float ss = 0.f;
  if (vec4) {
    const int n4 = hidden >> 2;
    for (int i = threadIdx.x; i < n4; i += THREADS) {
      const float4 v = *reinterpret_cast<const float4*>(yr + 4 * i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += THREADS) ss = fmaf(yr[i], yr[i], ss);
  }
  ss = block_sum(ss, scratch);
  const float rinv = 1.0f / sqrtf(ss / (float)hidden + eps);
  if (vec4) {
    const int n4 = hidden >> 2;
    for (int i = threadIdx.x; i < n4; i += THREADS) {
      const float4 v = *reinterpret_cast<const float4*>(yr + 4 * i);
      const float4 g = *reinterpret_cast<const float4*>(w + 4 * i);
      float4 a = *reinterpret_cast<const float4*>(xr + 4 * i);
      a.x += v.x * rinv * g.x; a.y += v.y * rinv * g.y; a.z += v.z * rinv * g.z; a.w += v.w * rinv * g.w;
      *reinterpret_cast<float4*>(xr + 4 * i) = a;
      *reinterpret_cast<float4*>(yr + 4 * i) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (cast) {
        TO* c = cast + r * hidden + 4 * i;
        c[0] = from_f32<TO>(a.x); c[1] = from_f32<TO>(a.y); c[2] = from_f32<TO>(a.z); c[3] = from_f32<TO>(a.w);
      }
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += THREADS) {
      const float a = xr[i] + yr[i] * rinv * w[i];
      xr[i] = a;
      yr[i] = 0.f;
      if (cast) cast[r * hidden + i] = from_f32<TO>(a);
    }
  }
}

template <typename TO>
__global__ void __launch_bounds__(THREADS)
cast_rows_kernel(const float* __restrict__ x, float* __restrict__ y, TO* __restrict__ cast, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * THREADS + threadIdx.x; i < total; i += (size_t)gridDim.x * THREADS) {
    cast[i] = from_f32<TO>(x[i]);
    if (y) y[i] = 0.f;
  }
}

__global__ void scale_values_kernel(float* __restrict__ z, size_t total, float s) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) z[i] *= s;
}

}  // namespace

// x[r, :] += y[r, :] / rms(y[r, :]) * w for `rows` rows of `hidden` numbers; y's rows are cleared; `cast`
// (optional, of `cast_dtype`) receives the new x.
IERT_API int iert_add_normed(float* x, float* y, const float* w, void* cast, int cast_dtype, int rows, int hidden, float eps,
                             cudaStream_t stream) {
  if (rows <= 0) return IERT_OK;
  if (hidden <= 0) return IERT_BAD_ARGUMENT;
  const int vec4 = hidden % 4 == 0 && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)w) & 15) == 0;
  if (vec4 && hidden <= 4 * 8 * THREADS && (cast_dtype == IERT_F32 || cast_dtype == IERT_BF16) && ((uintptr_t)cast & 15) == 0) {
    const int per_thread = (hidden / 4 + THREADS - 1) / THREADS;            // runs of four numbers a thread holds
#define ROWS(TO, V) launch_dep(add_normed_rows_kernel<TO, V>, dim3(rows), dim3(THREADS), 0, stream, x, y, w, (TO*)cast, hidden, eps)
#define PICK(TO) do { if (per_thread <= 1) ROWS(TO, 1); else if (per_thread <= 2) ROWS(TO, 2); else if (per_thread <= 4) ROWS(TO, 4); \
                      else ROWS(TO, 8); } while (0)
    if (cast_dtype == IERT_F32) PICK(float); else PICK(__nv_bfloat16);
#undef PICK
#undef ROWS
    return iert_check_launch("add_normed");
  }
  if (cast_dtype == IERT_F32)
    launch_dep(add_normed_kernel<float>, dim3(rows), dim3(THREADS), 0, stream, x, y, w, (float*)cast, hidden, eps, vec4);
  else if (cast_dtype == IERT_BF16)
    launch_dep(add_normed_kernel<__nv_bfloat16>, dim3(rows), dim3(THREADS), 0, stream, x, y, w, (__nv_bfloat16*)cast, hidden,
               eps, vec4);
  else
    return IERT_BAD_ARGUMENT;
  return iert_check_launch("add_normed");
}

// cast[i] = x[i] in `cast_dtype`; y[i] = 0 (y optional).
IERT_API int iert_cast_rows(const float* x, float* y, void* cast, int cast_dtype, long long total, cudaStream_t stream) {
  if (total <= 0) return IERT_OK;
  const size_t want = ((size_t)total + THREADS - 1) / THREADS, cap = (size_t)iert_sm_count_cached() * 16;
  const int blocks = (int)(want < cap ? want : cap);
  if (cast_dtype == IERT_F32)
    launch_dep(cast_rows_kernel<float>, dim3(blocks), dim3(THREADS), 0, stream, x, y, (float*)cast, (size_t)total);
  else if (cast_dtype == IERT_BF16)
    launch_dep(cast_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(THREADS), 0, stream, x, y, (__nv_bfloat16*)cast,
               (size_t)total);
  else
    return IERT_BAD_ARGUMENT;
  return iert_check_launch("cast_rows");
}

// z[i] *= s (fp32): a fixed factor on the logits.
IERT_API int iert_scale_values(float* z, long long total, float s, cudaStream_t stream) {
  if (total <= 0) return IERT_OK;
  const size_t want = ((size_t)total + 255) / 256, cap = (size_t)iert_sm_count_cached() * 16;
  launch_dep(scale_values_kernel, dim3((unsigned)(want < cap ? want : cap)), dim3(256), 0, stream, z, (size_t)total, s);
  return iert_check_launch("scale_values");
}
