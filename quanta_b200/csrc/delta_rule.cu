// Generalized delta rule with a decay per key channel: a recurrence over time whose state is a matrix
// S [key channel i, value channel j] per (request, head), float32, kept in the request's state slot.
//
//   u   = k / sqrt(sum(k^2) + unit_eps)                       (unit key of the head)
//   w   = exp(-decay_scale * sigmoid(wpre + w_bias))          (decay per key channel)
//   a   = sigmoid(apre + a_bias)                              (removal rate per key channel)
//   S_t = diag(w) S_{t-1} - (a * u) (u^T S_{t-1}) + k v^T     (both terms read the old state)
//   o_t = S_t^T r
//
// A first kernel turns the projections of every (token, head) into w, a*u and u (all tokens at once).  The
// recurrence itself is a chain in time.  A column j of S never meets another column, so eight neighbouring
// lanes own one column (rows i = p, p + 8, ... for lane p) in registers for the whole step, and a block owns
// some columns of one (request, head).  Tokens are taken in chunks: w, a*u, u, k, r, v of the next chunk come
// into shared memory by asynchronous copies while every lane group walks the chunk before without any
// barrier.  One token (decoding) or a portion of a prompt is the same code, and a column's numbers do not
// depend on which block owns it, so a position's numbers depend neither on the cut nor on the batch.
//
// The per-head RMS norm with gain and gate that follows is a kernel of the common unit (norm_embed.cu).
#include "common.cuh"

constexpr int DR_LANES = 8;   // lanes that share a column
constexpr int DR_MAX_COLS = 64;    // columns a block (512 threads), so that a lane's rows stay in registers
template <int RPT> struct DrThreads { static constexpr int max = RPT * 64 < 512 ? RPT * 64 : 512; };

// w, a*u and u of every (token, head), float32 [T, H, D] each: one warp a (token, head), the sum over k^2 a
// warp reduction in a fixed order.
__global__ void delta_prep_kernel(const float* __restrict__ proj, int proj_stride, int k_off, int a_off,
                                  const float* __restrict__ wpre, const float* __restrict__ a_bias,
                                  const float* __restrict__ w_bias, float* __restrict__ w_out,
                                  float* __restrict__ au_out, float* __restrict__ u_out, int T, int H, int D,
                                  float decay_scale, float unit_eps) {
  const int lane = threadIdx.x & 31;
  const long wid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (long)T * H) return;
  const int t = (int)(wid / H), h = (int)(wid % H);
  const float* row = proj + (size_t)t * proj_stride + (size_t)h * D;
  const size_t base = ((size_t)t * H + h) * D;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) { const float kv = row[k_off + i]; ss += kv * kv; }
  ss = qb_warp_sum(ss);
  const float inv = 1.f / sqrtf(ss + unit_eps);
  for (int i = lane; i < D; i += 32) {
    const float uv = row[k_off + i] * inv;
    const float av = 1.f / (1.f + expf(-(row[a_off + i] + a_bias[h * D + i])));
    const float sg = 1.f / (1.f + expf(-(wpre[base + i] + w_bias[h * D + i])));
    w_out[base + i] = expf(-decay_scale * sg);
    au_out[base + i] = av * uv;
    u_out[base + i] = uv;
  }
}

__device__ __forceinline__ void dr_copy4(float* dst_smem, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

template <int RPT>            // rows of the column a lane holds: D <= DR_LANES * RPT
__global__ void __launch_bounds__(DrThreads<RPT>::max, 1)
delta_rule_kernel(const float* __restrict__ proj, int proj_stride, int r_off, int k_off, int v_off,
                  const float* __restrict__ w_in, const float* __restrict__ au_in, const float* __restrict__ u_in,
                  float* __restrict__ state, float* __restrict__ out, const int* __restrict__ req_start,
                  const int* __restrict__ req_slot, int H, int D, int cols_per_block, int chunk) {
  extern __shared__ float sm[];
  constexpr int DP = DR_LANES * RPT;       // padded key channels (a power of two)
  const int r = blockIdx.x, h = blockIdx.y;
  const int col0 = blockIdx.z * cols_per_block;
  const int tid = threadIdx.x;
  const int p = tid % DR_LANES;
  const int j = col0 + tid / DR_LANES;
  const bool owns = (tid / DR_LANES) < cols_per_block && j < D;
  const size_t plane = (size_t)chunk * DP;  // one array of a chunk; six arrays a buffer, two buffers
  // the padding rows (i >= D) are read as zeros and never written
  for (size_t i = tid; i < 12 * plane; i += blockDim.x) sm[i] = 0.f;

  const int t0 = req_start[r], t1 = req_start[r + 1];
  float* S = state + ((size_t)req_slot[r] * H + h) * D * D;
  float col[RPT];
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = p + DR_LANES * ii;
    col[ii] = (owns && i < D) ? S[(size_t)i * D + j] : 0.f;
  }
  __syncthreads();

  // a chunk's six arrays come in by asynchronous copies while the chunk before is walked
  auto fetch = [&](int c0, int buf) {
    const int n = min(chunk, t1 - c0);
    float* b = sm + (size_t)buf * 6 * plane;
    for (int idx = tid; idx < n * DP; idx += blockDim.x) {
      const int tt = idx / DP, i = idx % DP;
      if (i < D) {
        const size_t g = ((size_t)(c0 + tt) * H + h) * D + i;
        const float* row = proj + (size_t)(c0 + tt) * proj_stride + (size_t)h * D + i;
        dr_copy4(b + idx, w_in + g);
        dr_copy4(b + plane + idx, au_in + g);
        dr_copy4(b + 2 * plane + idx, u_in + g);
        dr_copy4(b + 3 * plane + idx, row + k_off);
        dr_copy4(b + 4 * plane + idx, row + r_off);
        dr_copy4(b + 5 * plane + idx, row + v_off);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (t0 < t1) fetch(t0, 0);
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += chunk, buf ^= 1) {
    const int n = min(chunk, t1 - c0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                        // this chunk has landed, and everyone is done with the other buffer
    if (c0 + chunk < t1) fetch(c0 + chunk, buf ^ 1);
    const float* s_w = sm + (size_t)buf * 6 * plane;
    const float* s_au = s_w + plane;
    const float* s_u = s_au + plane;
    const float* s_k = s_u + plane;
    const float* s_r = s_k + plane;
    const float* s_v = s_r + plane;
    for (int tt = 0; tt < n; ++tt) {
      const size_t o = (size_t)tt * DP;
      float dot = 0.f;
#pragma unroll
      for (int ii = 0; ii < RPT; ++ii) dot += s_u[o + p + DR_LANES * ii] * col[ii];
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      dot += __shfl_xor_sync(0xffffffffu, dot, 4);
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
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (owns && p == 0) out[((size_t)(c0 + tt) * H + h) * D + j] = acc;
    }
  }
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = p + DR_LANES * ii;
    if (owns && i < D) S[(size_t)i * D + j] = col[ii];
  }
}

// scratch: 3 * T * H * D floats (w, a*u, u of the step's tokens)
extern "C" int qb_delta_rule(const float* proj, int proj_stride, int r_off, int k_off, int v_off, int a_off,
                             const float* wpre, const float* a_bias, const float* w_bias, float* state,
                             float* out, float* scratch, const int* req_start, const int* req_slot, int R,
                             int T, int H, int D, float decay_scale, float unit_eps, cudaStream_t stream) {
  if (R <= 0 || T <= 0) return 0;
  if (D <= 0 || D > 256 || H <= 0) return QB_ERR_UNSUPPORTED;
  const size_t n = (size_t)T * H * D;
  float *w_s = scratch, *au_s = scratch + n, *u_s = scratch + 2 * n;
  const long warps = (long)T * H;
  delta_prep_kernel<<<(int)((warps + 3) / 4), 128, 0, stream>>>(proj, proj_stride, k_off, a_off, wpre, a_bias, w_bias,
                                                              w_s, au_s, u_s, T, H, D, decay_scale, unit_eps);
  QB_LAUNCH_CHECK();
  // columns a block: all of them (at most DR_MAX_COLS) unless that leaves most SMs idle; then fewer, down to 16
  // where requests bring portions (the block's threads also fetch the chunks) and down to 4 where every request
  // brings one token (the state's bytes are what counts, spread over all SMs); a multiple of 4: whole warps
  const int min_cols = T > R ? 16 : 4;
  int splits = (D + DR_MAX_COLS - 1) / DR_MAX_COLS;
  while ((long)R * H * splits < 132 && (D + 2 * splits - 1) / (2 * splits) >= min_cols) splits *= 2;
  int cols = (D + splits - 1) / splits;
  cols = (cols + 3) / 4 * 4;
  splits = (D + cols - 1) / cols;
  const int threads = cols * DR_LANES;
  const int rpt = D <= 32 ? 4 : D <= 64 ? 8 : D <= 128 ? 16 : 32;
  const int dp = rpt * DR_LANES;
  const int chunk = dp <= 128 ? 16 : 8;
  const size_t smem = (size_t)12 * chunk * dp * sizeof(float);
  dim3 grid(R, H, splits);
#define DR_LAUNCH(N)                                                                                       \
  do {                                                                                                     \
    auto kern = delta_rule_kernel<N>;                                                                      \
    if (smem > 48 * 1024) {                                                                                \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      if (e != cudaSuccess) return (int)e;                                                                 \
    }                                                                                                      \
    kern<<<grid, threads, smem, stream>>>(proj, proj_stride, r_off, k_off, v_off, w_s, au_s, u_s, state,   \
                                          out, req_start, req_slot, H, D, cols, chunk);                    \
  } while (0)
  if (rpt == 4) DR_LAUNCH(4);
  else if (rpt == 8) DR_LAUNCH(8);
  else if (rpt == 16) DR_LAUNCH(16);
  else DR_LAUNCH(32);
#undef DR_LAUNCH
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
