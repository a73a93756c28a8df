// Generalized delta rule with a decay per key channel: a recurrence over time whose state is a matrix
// S [key channel i, value channel j] per (request, head), float32, kept in the request's state slot.
//
//   u   = k / sqrt(sum(k^2) + unit_eps)                       (unit key of the head)
//   w   = exp(-decay_scale * sigmoid(wpre + w_bias))          (decay per key channel)
//   a   = sigmoid(apre + a_bias)                              (removal rate per key channel)
//   S_t = diag(w) S_{t-1} - (a * u) (u^T S_{t-1}) + k v^T     (both terms read the old state)
//   o_t = S_t^T r
//
// A column j of S never meets another column, so four neighbouring lanes own one column (rows i = p,
// p + 4, ... for lane p) in registers for the whole step, and a block owns some columns of one
// (request, head).  Tokens are taken in chunks: the block's warps first turn a chunk's projections into
// w, a*u, u, k, r, v in shared memory (a warp a token; the sum over k^2 is a warp reduction in a fixed
// order), then every lane group walks the chunk's tokens without any barrier.  One token (decoding) or a
// portion of a prompt is the same code, so a position's numbers do not depend on the cut.
//
// A second kernel divides each head's o by its root mean square, multiplies by the gain and by
// sigmoid(gate) and writes the activation dtype for the output projection.
#include "common.cuh"

constexpr int DR_LANES = 4;   // lanes that share a column
constexpr int DR_MAX_COLS = 128;   // columns a block (512 threads), so that a lane's rows stay in registers
template <int RPT> struct DrThreads { static constexpr int max = RPT * 16 < 512 ? RPT * 16 : 512; };

template <int RPT>            // rows of the column a lane holds: D <= 4 * RPT
__global__ void __launch_bounds__(DrThreads<RPT>::max, 1)
delta_rule_kernel(const float* __restrict__ proj, int proj_stride, int r_off, int k_off, int v_off, int a_off,
                  const float* __restrict__ wpre, const float* __restrict__ a_bias,
                  const float* __restrict__ w_bias, float* __restrict__ state, float* __restrict__ out,
                  const int* __restrict__ req_start, const int* __restrict__ req_slot, int H, int D,
                  int cols_per_block, int chunk, float decay_scale, float unit_eps) {
  extern __shared__ float sm[];
  constexpr int DP = DR_LANES * RPT;       // padded key channels
  const int r = blockIdx.x, h = blockIdx.y;
  const int col0 = blockIdx.z * cols_per_block;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int p = tid % DR_LANES;
  const int j = col0 + tid / DR_LANES;
  const bool owns = (tid / DR_LANES) < cols_per_block && j < D;
  float* s_w = sm;                          // [chunk][DP] each
  float* s_au = s_w + (size_t)chunk * DP;
  float* s_u = s_au + (size_t)chunk * DP;
  float* s_k = s_u + (size_t)chunk * DP;
  float* s_r = s_k + (size_t)chunk * DP;
  float* s_v = s_r + (size_t)chunk * DP;

  const int t0 = req_start[r], t1 = req_start[r + 1];
  float* S = state + ((size_t)req_slot[r] * H + h) * D * D;
  float col[RPT];
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = p + DR_LANES * ii;
    col[ii] = (owns && i < D) ? S[(size_t)i * D + j] : 0.f;
  }

  for (int c0 = t0; c0 < t1; c0 += chunk) {
    const int n = min(chunk, t1 - c0);
    __syncthreads();                        // the chunk before has been read by everyone
    for (int tt = warp; tt < n; tt += nwarps) {
      const float* row = proj + (size_t)(c0 + tt) * proj_stride + (size_t)h * D;
      const float* wrow = wpre + ((size_t)(c0 + tt) * H + h) * D;
      float ss = 0.f;
      for (int i = lane; i < D; i += 32) { const float kv = row[k_off + i]; ss += kv * kv; }
      ss = qb_warp_sum(ss);
      const float inv = 1.f / sqrtf(ss + unit_eps);
      for (int i = lane; i < DP; i += 32) {
        float wv = 0.f, au = 0.f, uv = 0.f, kv = 0.f, rv = 0.f, vv = 0.f;
        if (i < D) {
          kv = row[k_off + i];
          rv = row[r_off + i];
          vv = row[v_off + i];
          uv = kv * inv;
          const float av = 1.f / (1.f + expf(-(row[a_off + i] + a_bias[h * D + i])));
          au = av * uv;
          const float sg = 1.f / (1.f + expf(-(wrow[i] + w_bias[h * D + i])));
          wv = expf(-decay_scale * sg);
        }
        const size_t o = (size_t)tt * DP + i;
        s_w[o] = wv; s_au[o] = au; s_u[o] = uv; s_k[o] = kv; s_r[o] = rv; s_v[o] = vv;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const size_t o = (size_t)tt * DP;
      float dot = 0.f;
#pragma unroll
      for (int ii = 0; ii < RPT; ++ii) dot += s_u[o + p + DR_LANES * ii] * col[ii];
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      const float vj = owns ? s_v[o + j] : 0.f;
      float acc = 0.f;
#pragma unroll
      for (int ii = 0; ii < RPT; ++ii) {
        const int i = p + DR_LANES * ii;
        const float s_new = s_w[o + i] * col[ii] - s_au[o + i] * dot + s_k[o + i] * vj;
        col[ii] = s_new;
        acc += s_r[o + i] * s_new;
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (owns && p == 0) out[((size_t)(c0 + tt) * H + h) * D + j] = acc;
    }
  }
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = p + DR_LANES * ii;
    if (owns && i < D) S[(size_t)i * D + j] = col[ii];
  }
}

extern "C" int qb_delta_rule(const float* proj, int proj_stride, int r_off, int k_off, int v_off, int a_off,
                             const float* wpre, const float* a_bias, const float* w_bias, float* state,
                             float* out, const int* req_start, const int* req_slot, int R, int T, int H,
                             int D, float decay_scale, float unit_eps, cudaStream_t stream) {
  if (R <= 0 || T <= 0) return 0;
  if (D <= 0 || D > 256 || H <= 0) return QB_ERR_UNSUPPORTED;
  // columns a block: all of them unless that leaves most SMs idle; a multiple of 8 so that the block is whole warps
  int splits = (D + DR_MAX_COLS - 1) / DR_MAX_COLS;
  while ((long)R * H * splits < 132 && (D + 2 * splits - 1) / (2 * splits) >= 8) splits *= 2;
  int cols = (D + splits - 1) / splits;
  cols = (cols + 7) / 8 * 8;
  splits = (D + cols - 1) / cols;
  const int threads = cols * DR_LANES;
  const int rpt = D <= 32 ? 8 : D <= 64 ? 16 : D <= 128 ? 32 : 64;
  const int dp = rpt * DR_LANES;
  const int chunk = dp <= 128 ? 16 : 8;
  const size_t smem = (size_t)6 * chunk * dp * sizeof(float);
  dim3 grid(R, H, splits);
#define DR_LAUNCH(N)                                                                                       \
  do {                                                                                                     \
    auto kern = delta_rule_kernel<N>;                                                                      \
    if (smem > 48 * 1024) {                                                                                \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      if (e != cudaSuccess) return (int)e;                                                                 \
    }                                                                                                      \
    kern<<<grid, threads, smem, stream>>>(proj, proj_stride, r_off, k_off, v_off, a_off, wpre, a_bias,     \
                                          w_bias, state, out, req_start, req_slot, H, D, cols, chunk,      \
                                          decay_scale, unit_eps);                                          \
  } while (0)
  if (rpt == 8) DR_LAUNCH(8);
  else if (rpt == 16) DR_LAUNCH(16);
  else if (rpt == 32) DR_LAUNCH(32);
  else DR_LAUNCH(64);
#undef DR_LAUNCH
  QB_LAUNCH_CHECK();
  return 0;
}

// out[t, h*D + i] = o[t,h,i] / sqrt(mean_i(o[t,h,:]^2) + eps) * gain[h*D + i] * sigmoid(gate[t, h*D + i])
// One warp a (token, head); the sum is a warp reduction in a fixed order.
template <typename O>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                                      int gate_stride, const float* __restrict__ gain, O* __restrict__ out,
                                      int T, int H, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const long wid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (long)T * H) return;
  const int t = (int)(wid / H), h = (int)(wid % H);
  const float* row = o + ((size_t)t * H + h) * D;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) ss += row[i] * row[i];
  ss = qb_warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)D + eps);
  const float* g = gate + (size_t)t * gate_stride + (size_t)h * D;
  for (int i = lane; i < D; i += 32) {
    const float sg = 1.f / (1.f + expf(-g[i]));
    out[((size_t)t * H + h) * D + i] = qb_from_float<O>(row[i] * inv * gain[h * D + i] * sg);
  }
}

extern "C" int qb_head_norm_gate(const float* o, const float* gate, int gate_stride, const float* gain,
                                 void* out, int out_dtype, int T, int H, int D, float eps,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  const long warps = (long)T * H;
  const int blocks = (int)((warps + 3) / 4);
  QB_DISPATCH_DTYPE(out_dtype, O, head_norm_gate_kernel<O><<<blocks, 128, 0, stream>>>(
      o, gate, gate_stride, gain, (O*)out, T, H, D, eps));
  QB_LAUNCH_CHECK();
  return 0;
}

// out[t, c] = tanh(x[t, off + c]) for c < n, in the activation dtype (the inner activation of a
// low-rank pair of projections whose first product sits inside a wider fused product).
template <typename O>
__global__ void tanh_cols_kernel(const float* __restrict__ x, int x_stride, int off, O* __restrict__ out,
                                 int T, int n) {
  const size_t total = (size_t)T * n;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / n, c = i % n;
    out[i] = qb_from_float<O>(tanhf(x[t * x_stride + off + c]));
  }
}

extern "C" int qb_tanh_cols(const float* x, int x_stride, int off, void* out, int out_dtype, int T, int n,
                            cudaStream_t stream) {
  if (T <= 0 || n <= 0) return 0;
  const size_t total = (size_t)T * n;
  const int blocks = (int)((total + 255) / 256 < 2048 ? (total + 255) / 256 : 2048);
  QB_DISPATCH_DTYPE(out_dtype, O, tanh_cols_kernel<O><<<blocks, 256, 0, stream>>>(x, x_stride, off, (O*)out, T, n));
  QB_LAUNCH_CHECK();
  return 0;
}
