// Recurrences with a matrix state per head, S [DIM x V] in fp32, carried from token to token in the
// sequence's state.  Compiled per key size (-DDIM=...), like the attention kernels per head size.
//
// Work split: a column j of S never meets another column, so a CTA owns (sequence, head, a run of
// columns) and a thread owns RPT = ceil(DIM / R) rows of one column in registers; the R threads of a
// column are neighbouring lanes and add their partial dot products by shuffles.  A CTA walks its
// sequence's tokens in order; the tokens' vectors come through shared memory CHUNK tokens at a time.
// State is read when the CTA starts and written back when it ends, so a step of one token and a
// prompt of thousands run the same code.
//
//   gated delta rule, per token:   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   mLSTM, per token:  m' = max(f + m, i);  S <- e^(f+m-m') S + e^(i-m') k v^T;  n likewise with k;
//                      o = S^T q / (max(|n . q|, e^(-m')) + 1e-6),  m starts at 0
//       with i = cap tanh((zi + bi) / cap),  f = logsigmoid(cap tanh((zf + bf) / cap))
#include "common.cuh"

using namespace iert;

#ifndef DIM
#error "compile with -DDIM=<rows of the state matrix>"
#endif

namespace {

constexpr int lanes_per_column() {
  int r = 1;
  while ((DIM + r - 1) / r > 32 && r < 32) r *= 2;
  return r;
}
constexpr int R = lanes_per_column();
constexpr int RPT = (DIM + R - 1) / R;
constexpr int CHUNK = 8;
constexpr int MAX_COLS = 128 / R > 0 ? (256 / R) : 1;      // columns per CTA (threads = cols * R <= 256)

__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = R / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct DeltaArgs {
  const float* qkv;      // [T, C] fp32: q [G*DIM] | k [G*DIM] | v [H*V]   (from delta_prep)
  const float* beta;     // [T, H]
  const float* decay;    // [T, H]
  float* state;          // per slot at s_off: S [H, DIM, V]
  long long state_stride, s_off;
  float* o;              // [T, H*V] fp32
  int G, H, V, cols;
};

__global__ void __launch_bounds__(256) delta_recur_kernel(DeltaArgs a, IertBatchView b) {
  __shared__ float k_s[CHUNK][DIM], q_s[CHUNK][DIM], v_s[CHUNK][256], bg_s[CHUNK][2];
  pdl_wait();
  const int s = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * a.cols;
  const int slot = b.slot_ids[s];
  const int t0 = b.cu_q[s], t1 = b.cu_q[s + 1];
  if (slot < 0 || t1 <= t0) return;
  const int col = threadIdx.x / R, r = threadIdx.x % R;
  const int j = c0 + col;
  const bool live = col < a.cols && j < a.V;
  const int g = head / (a.H / a.G);
  const int GD = a.G * DIM, C = 2 * GD + a.H * a.V;
  float* Sg = a.state + (size_t)slot * a.state_stride + a.s_off + (size_t)head * DIM * a.V;
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = r * RPT + i;
    S[i] = (live && d < DIM) ? Sg[(size_t)d * a.V + j] : 0.f;
  }
  for (int tc = t0; tc < t1; tc += CHUNK) {
    const int n = min(CHUNK, t1 - tc);
    __syncthreads();
    for (int x = threadIdx.x; x < n * DIM; x += blockDim.x) {
      const int tt = x / DIM, d = x - tt * DIM;
      const float* rowp = a.qkv + (size_t)(tc + tt) * C;
      q_s[tt][d] = rowp[g * DIM + d];
      k_s[tt][d] = rowp[GD + g * DIM + d];
    }
    for (int x = threadIdx.x; x < n * a.cols; x += blockDim.x) {
      const int tt = x / a.cols, cc = x - tt * a.cols;
      v_s[tt][cc] = c0 + cc < a.V ? a.qkv[(size_t)(tc + tt) * C + 2 * GD + head * a.V + c0 + cc] : 0.f;
    }
    if (threadIdx.x < n) {
      bg_s[threadIdx.x][0] = a.beta[(size_t)(tc + threadIdx.x) * a.H + head];
      bg_s[threadIdx.x][1] = a.decay[(size_t)(tc + threadIdx.x) * a.H + head];
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float beta = bg_s[tt][0], gd = bg_s[tt][1];
      float kk[RPT];
      float dk = 0.f;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int d = r * RPT + i;
        kk[i] = d < DIM ? k_s[tt][d] : 0.f;
        S[i] *= gd;
        dk = fmaf(S[i], kk[i], dk);
      }
      dk = group_sum(dk);
      const float u = beta * ((live ? v_s[tt][col] : 0.f) - dk);
      float oq = 0.f;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int d = r * RPT + i;
        S[i] = fmaf(kk[i], u, S[i]);
        oq = fmaf(S[i], d < DIM ? q_s[tt][d] : 0.f, oq);
      }
      oq = group_sum(oq);
      if (live && r == 0) a.o[(size_t)(tc + tt) * a.H * a.V + (size_t)head * a.V + j] = oq;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int d = r * RPT + i;
      if (d < DIM) Sg[(size_t)d * a.V + j] = S[i];
    }
  }
}

struct MlstmArgs {
  const void* proj;      // [T, ld] run dtype: q [H*DIM] | k [H*DIM] | v [H*V] | ...
  long long ld;
  const float* gates;    // [T, gld] fp32: zi [H] | zf [H]
  long long gld;
  const float* bi;       // [H]
  const float* bf;       // [H]
  float cap;
  float* state;          // per slot: S [H, DIM, V] at s_off, n [H, DIM] at n_off, m [H] at m_off
  long long state_stride, s_off, n_off, m_off;
  float* coef;           // [T, H, 3] fp32: e^(f+m-m'), e^(i-m'), the read-out's denominator
  float* o;              // [T, H*V] fp32
  int H, V, cols;
};

__device__ __forceinline__ float logsigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// The part of the recurrence that no column of S takes part in: the gates, the running maximum m,
// the normaliser n and the read-out's denominator.  One warp per (sequence, head) walks the tokens
// and leaves three numbers per token for the CTAs that own the columns.
constexpr int NPL = (DIM + 31) / 32;          // entries of n per lane

template <typename T>
__global__ void __launch_bounds__(32) mlstm_scan_kernel(MlstmArgs a, IertBatchView b) {
  pdl_wait();
  const int s = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
  const int slot = b.slot_ids[s];
  const int t0 = b.cu_q[s], t1 = b.cu_q[s + 1];
  if (slot < 0 || t1 <= t0) return;
  float* base = a.state + (size_t)slot * a.state_stride;
  float* ng = base + a.n_off + (size_t)head * DIM;
  float nn[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) nn[i] = lane + 32 * i < DIM ? ng[lane + 32 * i] : 0.f;
  float m = base[a.m_off + head];
  const float qscale = 1.0f / sqrtf((float)DIM);
  const T* proj = (const T*)a.proj;
  for (int tc = t0; tc < t1; tc += CHUNK) {
    const int n = min(CHUNK, t1 - tc);
    float kq[CHUNK][NPL][2], gi[CHUNK], gf[CHUNK];
#pragma unroll
    for (int tt = 0; tt < CHUNK; ++tt) {
      if (tt < n) {
        const T* rowp = proj + (size_t)(tc + tt) * a.ld;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          const int d = lane + 32 * i;
          kq[tt][i][0] = d < DIM ? to_f32(rowp[a.H * DIM + head * DIM + d]) : 0.f;
          kq[tt][i][1] = d < DIM ? to_f32(rowp[head * DIM + d]) * qscale : 0.f;
        }
        gi[tt] = a.gates[(size_t)(tc + tt) * a.gld + head] + a.bi[head];
        gf[tt] = a.gates[(size_t)(tc + tt) * a.gld + a.H + head] + a.bf[head];
      }
    }
#pragma unroll
    for (int tt = 0; tt < CHUNK; ++tt) {
      if (tt < n) {
        const float li = a.cap * tanhf(gi[tt] / a.cap);
        const float lf = logsigmoid_f(a.cap * tanhf(gf[tt] / a.cap));
        const float m_new = fmaxf(lf + m, li);
        const float ea = expf(lf + m - m_new), eb = expf(li - m_new);
        m = m_new;
        float nq = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          nn[i] = fmaf(ea, nn[i], eb * kq[tt][i][0]);
          nq = fmaf(nn[i], kq[tt][i][1], nq);
        }
        nq = warp_sum(nq);
        if (lane == 0) {
          float* c = a.coef + ((size_t)(tc + tt) * a.H + head) * 3;
          c[0] = ea; c[1] = eb; c[2] = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NPL; ++i) if (lane + 32 * i < DIM) ng[lane + 32 * i] = nn[i];
  if (lane == 0) base[a.m_off + head] = m;
}

template <typename T>
__global__ void __launch_bounds__(256) mlstm_recur_kernel(MlstmArgs a, IertBatchView b) {
  __shared__ float k_s[CHUNK][DIM], q_s[CHUNK][DIM], v_s[CHUNK][256], c_s[CHUNK][3];
  pdl_wait();
  const int s = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * a.cols;
  const int slot = b.slot_ids[s];
  const int t0 = b.cu_q[s], t1 = b.cu_q[s + 1];
  if (slot < 0 || t1 <= t0) return;
  const int col = threadIdx.x / R, r = threadIdx.x % R;
  const int j = c0 + col;
  const bool live = col < a.cols && j < a.V;
  float* Sg = a.state + (size_t)slot * a.state_stride + a.s_off + (size_t)head * DIM * a.V;
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = r * RPT + i;
    S[i] = (live && d < DIM) ? Sg[(size_t)d * a.V + j] : 0.f;
  }
  const float qscale = 1.0f / sqrtf((float)DIM);
  const T* proj = (const T*)a.proj;
  for (int tc = t0; tc < t1; tc += CHUNK) {
    const int n = min(CHUNK, t1 - tc);
    __syncthreads();
    for (int x = threadIdx.x; x < n * DIM; x += blockDim.x) {
      const int tt = x / DIM, d = x - tt * DIM;
      const T* rowp = proj + (size_t)(tc + tt) * a.ld;
      q_s[tt][d] = to_f32(rowp[head * DIM + d]) * qscale;
      k_s[tt][d] = to_f32(rowp[a.H * DIM + head * DIM + d]);
    }
    for (int x = threadIdx.x; x < n * a.cols; x += blockDim.x) {
      const int tt = x / a.cols, cc = x - tt * a.cols;
      v_s[tt][cc] = c0 + cc < a.V ? to_f32(proj[(size_t)(tc + tt) * a.ld + 2 * a.H * DIM + head * a.V + c0 + cc]) : 0.f;
    }
    if (threadIdx.x < n * 3)
      c_s[threadIdx.x / 3][threadIdx.x % 3] = a.coef[((size_t)(tc + threadIdx.x / 3) * a.H + head) * 3 + threadIdx.x % 3];
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float ea = c_s[tt][0], eb = c_s[tt][1], den = c_s[tt][2];
      const float bv = eb * (live ? v_s[tt][col] : 0.f);
      float oq = 0.f;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int d = r * RPT + i;
        const float kd = d < DIM ? k_s[tt][d] : 0.f, qd = d < DIM ? q_s[tt][d] : 0.f;
        S[i] = fmaf(ea, S[i], kd * bv);
        oq = fmaf(S[i], qd, oq);
      }
      oq = group_sum(oq);
      if (live && r == 0) a.o[(size_t)(tc + tt) * a.H * a.V + (size_t)head * a.V + j] = oq / den;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int d = r * RPT + i;
      if (d < DIM) Sg[(size_t)d * a.V + j] = S[i];
    }
  }
}

// Columns per CTA: as many CTAs as fill the device a few times over, not fewer than 8 columns each.
int pick_cols(int n_seqs, int H, int V) {
  int cols = MAX_COLS < V ? MAX_COLS : V;
  const int want = 2 * iert_sm_count_cached();
  while (cols > 8 && (long long)n_seqs * H * ((V + cols - 1) / cols) < want) cols = (cols + 1) / 2;
  return cols;
}

}  // namespace

IERT_API int iert_recurrent_dim() { return DIM; }

IERT_API int iert_delta_recur(const float* qkv, const float* beta, const float* decay, float* state,
                              long long state_stride, long long s_off, float* o, int G, int H, int V,
                              const IertBatchView* batch, cudaStream_t stream) {
  if (batch->n_seqs <= 0 || batch->n_tokens <= 0) return IERT_OK;
  if (G <= 0 || H <= 0 || H % G || V <= 0 || H > 65535) return IERT_BAD_ARGUMENT;
  const int cols = pick_cols(batch->n_seqs, H, V);
  DeltaArgs a = {qkv, beta, decay, state, state_stride, s_off, o, G, H, V, cols};
  dim3 grid(batch->n_seqs, H, (V + cols - 1) / cols);
  const int threads = ((cols * R + 31) / 32) * 32;
  launch_dep(delta_recur_kernel, grid, dim3(threads), 0, stream, a, *batch);
  return iert_check_launch("delta_recur");
}

IERT_API int iert_mlstm_recur(const void* proj, int dtype, long long ld, const float* gates, long long gld,
                              const float* bi, const float* bf, float cap, float* state, long long state_stride,
                              long long s_off, long long n_off, long long m_off, float* coef, float* o, int H, int V,
                              const IertBatchView* batch, cudaStream_t stream) {
  if (batch->n_seqs <= 0 || batch->n_tokens <= 0) return IERT_OK;
  if (H <= 0 || V <= 0 || H > 65535 || !(cap > 0.f) || (dtype != IERT_F32 && dtype != IERT_BF16)) return IERT_BAD_ARGUMENT;
  const int cols = pick_cols(batch->n_seqs, H, V);
  MlstmArgs a = {proj, ld, gates, gld, bi, bf, cap, state, state_stride, s_off, n_off, m_off, coef, o, H, V, cols};
  dim3 grid(batch->n_seqs, H, (V + cols - 1) / cols);
  const int threads = ((cols * R + 31) / 32) * 32;
  if (dtype == IERT_F32) {
    launch_dep(mlstm_scan_kernel<float>, dim3(batch->n_seqs, H), dim3(32), 0, stream, a, *batch);
    launch_dep(mlstm_recur_kernel<float>, grid, dim3(threads), 0, stream, a, *batch);
  } else {
    launch_dep(mlstm_scan_kernel<__nv_bfloat16>, dim3(batch->n_seqs, H), dim3(32), 0, stream, a, *batch);
    launch_dep(mlstm_recur_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, a, *batch);
  }
  return iert_check_launch("mlstm_recur");
}
