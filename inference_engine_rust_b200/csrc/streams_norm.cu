// LayerNorm (weight and bias) over a residual that is kept as S parallel streams
// (hyper-connections), and the small kernels around it.  One kernel does, per token row:
//
//   1. optional update with a sublayer's output y:   x'_t = sum_s mix[s, t] x_s + outc[t] y
//   2. optional clearing of the row of y (the next sublayer adds its result into it)
//   3. the combination  u = sum_s in[s] x'_s         (in = nullptr: all ones)
//   4. LayerNorm  out = (u - mean(u)) / sqrt(var(u) + eps) * w + b,  var = mean((u - mean)^2)
//
// so that the update after one sublayer and the normed input of the next are one pass over the
// streams.  With S = 1, no update and in = nullptr it is a plain LayerNorm of fp32 rows.  Everything
// is computed in fp32; the sums run in an order that depends on the sizes alone.
#include "common.cuh"

using namespace iert;

namespace {

constexpr int MAX_STREAMS = 8;

struct StreamsNormArgs {
  float* xs;              // [T, S, H] fp32
  int S, H;
  float* y;               // [T, H] fp32 or nullptr
  const float* mix;       // [S, S] indexed [from, to] (update only)
  const float* outc;      // [S] (update only)
  int update, write_back, zero_y;
  const float* in_coef;   // [S] or nullptr
  const float* w;         // [H] or nullptr (no norm: only the update / the sum)
  const float* b;         // [H] or nullptr
  float eps;
  void* out;              // [rows, H] of out_dtype or nullptr
  float* sum_out;         // [rows, H] fp32: u itself, or nullptr
  const int* rows_idx;    // output row i reads token row rows_idx[i], or nullptr (i itself)
};

template <typename TO>
__global__ void streams_norm_kernel(StreamsNormArgs a) {
  extern __shared__ float sm[];
  float* u_row = sm;                       // [H]
  float* coef = sm + a.H;                  // mix [S*S] | outc [S] | in [S]
  float* scratch = coef + MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS;   // [33]
  const int S = a.S, H = a.H;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) coef[i] = a.update ? a.mix[i] : 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    coef[MAX_STREAMS * MAX_STREAMS + i] = a.update ? a.outc[i] : 0.f;
    coef[MAX_STREAMS * MAX_STREAMS + MAX_STREAMS + i] = a.in_coef ? a.in_coef[i] : 1.f;
  }
  pdl_wait();
  __syncthreads();
  const float* mix = coef;
  const float* outc = coef + MAX_STREAMS * MAX_STREAMS;
  const float* inc = outc + MAX_STREAMS;
  const int row = a.rows_idx ? a.rows_idx[blockIdx.x] : (int)blockIdx.x;
  float* xr = a.xs + (size_t)row * S * H;
  float* yr = a.y ? a.y + (size_t)row * H : nullptr;
  float part = 0.f;
  // four columns per thread and pass (16-byte accesses) when the row length allows
  const int W = (H % 4 == 0) ? 4 : 1;
  for (int h = threadIdx.x * W; h < H; h += blockDim.x * W) {
    float x[MAX_STREAMS][4], yv[4] = {0.f, 0.f, 0.f, 0.f};
    if (W == 4) {
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) {
          const float4 v = *reinterpret_cast<const float4*>(xr + (size_t)s * H + h);
          x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w;
        }
      if (a.update) {
        const float4 v = *reinterpret_cast<const float4*>(yr + h);
        yv[0] = v.x; yv[1] = v.y; yv[2] = v.z; yv[3] = v.w;
      }
    } else {
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s) if (s < S) x[s][0] = xr[(size_t)s * H + h];
      if (a.update) yv[0] = yr[h];
    }
    float u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (e >= W) break;
      if (a.update) {
        float nx[MAX_STREAMS];
#pragma unroll
        for (int t = 0; t < MAX_STREAMS; ++t) {
          float v = 0.f;
          if (t < S) {
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s) if (s < S) v = fmaf(mix[s * S + t], x[s][e], v);
            v = fmaf(outc[t], yv[e], v);
          }
          nx[t] = v;
        }
#pragma unroll
        for (int t = 0; t < MAX_STREAMS; ++t) x[t][e] = nx[t];
      }
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s) if (s < S) u[e] = fmaf(inc[s], x[s][e], u[e]);
      part += u[e];
    }
    if (W == 4) *reinterpret_cast<float4*>(u_row + h) = make_float4(u[0], u[1], u[2], u[3]);
    else u_row[h] = u[0];
    if (a.update && a.write_back) {
#pragma unroll
      for (int t = 0; t < MAX_STREAMS; ++t)
        if (t < S) {
          if (W == 4) *reinterpret_cast<float4*>(xr + (size_t)t * H + h) = make_float4(x[t][0], x[t][1], x[t][2], x[t][3]);
          else xr[(size_t)t * H + h] = x[t][0];
        }
    }
    if (a.zero_y && yr) {
      if (W == 4) *reinterpret_cast<float4*>(yr + h) = make_float4(0.f, 0.f, 0.f, 0.f);
      else yr[h] = 0.f;
    }
  }
  if (a.sum_out)
    for (int h = threadIdx.x; h < H; h += blockDim.x) a.sum_out[(size_t)blockIdx.x * H + h] = u_row[h];
  if (!a.out) return;
  const float mean = block_sum(part, scratch) / (float)H;
  float dev = 0.f;
  for (int h = threadIdx.x * W; h < H; h += blockDim.x * W) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (e >= W) break;
      const float d = u_row[h + e] - mean;
      dev = fmaf(d, d, dev);
    }
  }
  const float rstd = 1.0f / sqrtf(block_sum(dev, scratch) / (float)H + a.eps);
  TO* o = (TO*)a.out + (size_t)blockIdx.x * H;
  if (W == 4) {                               // four outputs per thread and pass
    for (int h = threadIdx.x * 4; h < H; h += blockDim.x * 4) {
      const float4 u = *reinterpret_cast<const float4*>(u_row + h);
      const float4 w = *reinterpret_cast<const float4*>(a.w + h);
      const float4 bb = a.b ? *reinterpret_cast<const float4*>(a.b + h) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float v0 = (u.x - mean) * rstd * w.x + bb.x, v1 = (u.y - mean) * rstd * w.y + bb.y;
      const float v2 = (u.z - mean) * rstd * w.z + bb.z, v3 = (u.w - mean) * rstd * w.w + bb.w;
      if (sizeof(TO) == 4) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + h) = make_float4(v0, v1, v2, v3);
      } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v0, v1), hi = __floats2bfloat162_rn(v2, v3);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&lo);
        pk.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(o) + h) = pk;
      }
    }
    return;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float v = (u_row[h] - mean) * rstd * a.w[h] + (a.b ? a.b[h] : 0.f);
    o[h] = from_f32<TO>(v);
  }
}

__global__ void streams_expand_kernel(const float* __restrict__ x, float* __restrict__ xs, int S, int H) {
  const size_t t = blockIdx.x;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float v = x[t * H + h];
    for (int s = 0; s < S; ++s) xs[(t * S + s) * H + h] = v;
  }
}

__global__ void softcap_kernel(float* __restrict__ z, long long n, float cap) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) z[i] = cap * tanhf(z[i] / cap);
}

}  // namespace

// See the head of the file.  `rows` blocks; rows_idx (optional) gathers token rows.  Small vectors
// (mix, outc, in_coef, w, b) are fp32.  out may alias xs when S == 1 (a norm in place).
IERT_API int iert_streams_norm(float* xs, int S, int H, float* y, const float* mix, const float* outc, int update,
                               int write_back, int zero_y, const float* in_coef, const float* w, const float* b,
                               float eps, void* out, int out_dtype, float* sum_out, const int* rows_idx, int rows,
                               cudaStream_t stream) {
  if (rows <= 0) return IERT_OK;
  if (S <= 0 || S > MAX_STREAMS || H <= 0 || H > 11000 || (update && (!y || !mix || !outc)) || (out && !w))
    return IERT_BAD_ARGUMENT;
  StreamsNormArgs a = {xs, S, H, y, mix, outc, update, write_back, zero_y, in_coef, w, b, eps, out, sum_out, rows_idx};
  const int threads = H >= 2048 ? (rows >= 512 ? 256 : 512) : H >= 512 ? 256 : 128;    // many rows: more blocks per SM
  const size_t smem = (size_t)(H + MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS + 33) * sizeof(float);
  if (!out || out_dtype == IERT_F32)
    launch_dep(streams_norm_kernel<float>, dim3(rows), dim3(threads), smem, stream, a);
  else if (out_dtype == IERT_BF16)
    launch_dep(streams_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), smem, stream, a);
  else
    return IERT_BAD_ARGUMENT;
  return iert_check_launch("streams_norm");
}

// xs[t, s, :] = x[t, :] for every stream s.
IERT_API int iert_streams_expand(const float* x, float* xs, int n_tokens, int S, int H, cudaStream_t stream) {
  if (n_tokens <= 0) return IERT_OK;
  streams_expand_kernel<<<n_tokens, 256, 0, stream>>>(x, xs, S, H);
  return iert_check_launch("streams_expand");
}

// z <- cap * tanh(z / cap), in place (fp32 logits).
IERT_API int iert_softcap(float* z, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return IERT_OK;
  if (!(cap > 0.f)) return IERT_BAD_ARGUMENT;
  softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(z, n, cap);
  return iert_check_launch("softcap");
}
