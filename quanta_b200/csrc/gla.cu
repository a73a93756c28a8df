// Gated linear attention: a recurrence over time whose state is a matrix S [key channel i, value channel j]
// per (request, head), float32, kept in the request's state slot.
//
//   alpha = sigmoid(z)^(1/tau),  z = W2 (W1 x) + b            (decay per key channel, in (0, 1))
//   S_t   = diag(alpha_t) S_{t-1} + k_t v_t^T                 (the decay scales the rows)
//   o_t   = q_scale * S_t^T q_t
//
// Keys and queries have D channels a head, values and outputs E (any sizes up to 256).
//
// A first kernel finishes the decay of every (token, channel): the second, low-rank product W2 (.) from the
// float32 result of the first (which sits inside the step's wide fused projection), the bias, and
// alpha = exp(logsigmoid(z) / tau), all float32; logsigmoid(z) = min(z, 0) - log1p(exp(-|z|)) keeps decays
// close to 1 exact.  The recurrence is a chain in time.  A column j of S never meets another column, so eight
// neighbouring lanes own one column (rows i = p, p + 8, ... for lane p) in registers for the whole step, and a
// block owns some columns of one (request, head).  Tokens are taken in chunks: alpha, k, q, v of the next chunk
// come into shared memory by asynchronous copies while every lane group walks the chunk before without any
// barrier.  One token (decoding) or a portion of a prompt is the same code, and a column's numbers do not depend
// on which block owns it, so a position's numbers depend neither on the cut nor on the batch.
#include "common.cuh"

constexpr int GLA_LANES = 8;       // lanes that share a column
constexpr int GLA_MAX_COLS = 64;   // columns a block (512 threads), so that a lane's rows stay in registers

// alpha[t, c] for every token and channel c < C (= heads * D): one thread a (token, channel); the inner
// product over the rank L is one sequential float32 sum, the same whatever else the step holds.
template <typename W>
__global__ void gla_decay_kernel(const float* __restrict__ proj, int proj_stride, int inner_off, int L,
                                 const W* __restrict__ w2, const float* __restrict__ bias, float* __restrict__ alpha,
                                 int T, int C, float inv_tau) {
  extern __shared__ float s_inner[];      // the token's L inner values
  const int t = blockIdx.y;
  const float* in = proj + (size_t)t * proj_stride + inner_off;
  for (int i = threadIdx.x; i < L; i += blockDim.x) s_inner[i] = in[i];
  __syncthreads();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const W* row = w2 + (size_t)c * L;
  float z = 0.f;
  for (int i = 0; i < L; ++i) z = fmaf(qb_to_float<W>(row[i]), s_inner[i], z);
  z += bias[c];
  const float ls = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
  alpha[(size_t)t * C + c] = expf(ls * inv_tau);
}

__device__ __forceinline__ void gla_copy4(float* dst_smem, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

template <int RPT>            // rows of the column a lane holds: D <= GLA_LANES * RPT
__global__ void __launch_bounds__(GLA_MAX_COLS * GLA_LANES, 1)
gla_chain_kernel(const float* __restrict__ proj, int proj_stride, int q_off, int k_off, int v_off,
                 const float* __restrict__ alpha, float* __restrict__ state, float* __restrict__ out,
                 const int* __restrict__ req_start, const int* __restrict__ req_slot, int H, int D, int E,
                 int cols_per_block, int chunk, int EP, float q_scale) {
  extern __shared__ float sm[];
  constexpr int DP = GLA_LANES * RPT;       // padded key channels
  const int r = blockIdx.x, h = blockIdx.y;
  const int col0 = blockIdx.z * cols_per_block;
  const int tid = threadIdx.x;
  const int p = tid % GLA_LANES;
  const int j = col0 + tid / GLA_LANES;
  const bool owns = (tid / GLA_LANES) < cols_per_block && j < E;
  // a buffer: alpha, k, q [chunk][DP] and v [chunk][EP]; two buffers
  const size_t plane = (size_t)chunk * DP, vplane = (size_t)chunk * EP, bufsz = 3 * plane + vplane;
  // the padding rows (i >= D) are read as zeros and never written
  for (size_t i = tid; i < 2 * bufsz; i += blockDim.x) sm[i] = 0.f;

  const int t0 = req_start[r], t1 = req_start[r + 1];
  float* S = state + ((size_t)req_slot[r] * H + h) * D * E;
  float col[RPT];
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = p + GLA_LANES * ii;
    col[ii] = (owns && i < D) ? S[(size_t)i * E + j] : 0.f;
  }
  __syncthreads();

  auto fetch = [&](int c0, int buf) {
    const int n = min(chunk, t1 - c0);
    float* b = sm + (size_t)buf * bufsz;
    for (int idx = tid; idx < n * DP; idx += blockDim.x) {
      const int tt = idx / DP, i = idx % DP;
      if (i < D) {
        const float* row = proj + (size_t)(c0 + tt) * proj_stride + (size_t)h * D + i;
        gla_copy4(b + idx, alpha + ((size_t)(c0 + tt) * H + h) * D + i);
        gla_copy4(b + plane + idx, row + k_off);
        gla_copy4(b + 2 * plane + idx, row + q_off);
      }
    }
    for (int idx = tid; idx < n * EP; idx += blockDim.x) {
      const int tt = idx / EP, i = idx % EP;
      if (i < E) gla_copy4(b + 3 * plane + idx, proj + (size_t)(c0 + tt) * proj_stride + v_off + (size_t)h * E + i);
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
    const float* s_a = sm + (size_t)buf * bufsz;
    const float* s_k = s_a + plane;
    const float* s_q = s_k + plane;
    const float* s_v = s_q + plane;
    for (int tt = 0; tt < n; ++tt) {
      const size_t o = (size_t)tt * DP;
      const float vj = owns ? s_v[(size_t)tt * EP + j] : 0.f;
      float acc = 0.f;
#pragma unroll
      for (int ii = 0; ii < RPT; ++ii) {
        const int i = p + GLA_LANES * ii;
        const float s_new = fmaf(s_a[o + i], col[ii], s_k[o + i] * vj);
        col[ii] = s_new;
        acc = fmaf(s_q[o + i], s_new, acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (owns && p == 0) out[((size_t)(c0 + tt) * H + h) * E + j] = acc * q_scale;
    }
  }
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = p + GLA_LANES * ii;
    if (owns && i < D) S[(size_t)i * E + j] = col[ii];
  }
}

// proj: float32 rows of the step's fused projection (q, k at q_off / k_off: heads x D; v at v_off: heads x E; the
// L inner values of the decay at inner_off).  w2: [heads*D, L] in w2_dtype, bias: float32 [heads*D].
// state: float32 [slots, heads, D, E]; out: float32 [T, heads, E]; scratch: T * heads * D floats (alpha).
extern "C" int qb_gla(const float* proj, int proj_stride, int q_off, int k_off, int v_off, int inner_off, int L,
                      const void* w2, int w2_dtype, const float* bias, float* state, float* out, float* scratch,
                      const int* req_start, const int* req_slot, int R, int T, int H, int D, int E, float tau,
                      float q_scale, cudaStream_t stream) {
  if (R <= 0 || T <= 0) return 0;
  if (D <= 0 || D > 256 || E <= 0 || E > 256 || H <= 0 || L <= 0 || tau <= 0.f) return QB_ERR_UNSUPPORTED;
  if (L * sizeof(float) > 48 * 1024 || T > 65535 * 16) return QB_ERR_UNSUPPORTED;
  const int C = H * D;
  {
    dim3 grid((C + 127) / 128, T);
    if (grid.y > 65535) return QB_ERR_UNSUPPORTED;
    QB_DISPATCH_DTYPE(w2_dtype, W, gla_decay_kernel<W><<<grid, 128, L * sizeof(float), stream>>>(
        proj, proj_stride, inner_off, L, (const W*)w2, bias, scratch, T, C, 1.f / tau));
    QB_LAUNCH_CHECK();
  }
  // columns a block: all of them (at most GLA_MAX_COLS) unless that leaves most SMs idle; then fewer, down to 16
  // where requests bring portions (the block's threads also fetch the chunks) and down to 4 where every request
  // brings one token (the state's bytes are what counts, spread over all SMs); a multiple of 4: whole warps
  const int min_cols = T > R ? 16 : 4;
  int splits = (E + GLA_MAX_COLS - 1) / GLA_MAX_COLS;
  while ((long)R * H * splits < 132 && (E + 2 * splits - 1) / (2 * splits) >= min_cols) splits *= 2;
  int cols = (E + splits - 1) / splits;
  cols = (cols + 3) / 4 * 4;
  splits = (E + cols - 1) / cols;
  const int threads = cols * GLA_LANES;
  const int rpt = D <= 32 ? 4 : D <= 64 ? 8 : D <= 128 ? 16 : 32;
  const int dp = rpt * GLA_LANES;
  const int ep = (E + 3) / 4 * 4;
  const int chunk = dp <= 128 ? 16 : 8;
  const size_t smem = (size_t)2 * chunk * (3 * dp + ep) * sizeof(float);
  dim3 grid(R, H, splits);
  if (grid.y > 65535 || grid.z > 65535) return QB_ERR_UNSUPPORTED;
#define GLA_LAUNCH(N)                                                                                      \
  do {                                                                                                     \
    auto kern = gla_chain_kernel<N>;                                                                       \
    if (smem > 48 * 1024) {                                                                                \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      if (e != cudaSuccess) return (int)e;                                                                 \
    }                                                                                                      \
    kern<<<grid, threads, smem, stream>>>(proj, proj_stride, q_off, k_off, v_off, scratch, state, out,     \
                                          req_start, req_slot, H, D, E, cols, chunk, ep, q_scale);         \
  } while (0)
  if (rpt == 4) GLA_LAUNCH(4);
  else if (rpt == 8) GLA_LAUNCH(8);
  else if (rpt == 16) GLA_LAUNCH(16);
  else GLA_LAUNCH(32);
#undef GLA_LAUNCH
  QB_LAUNCH_CHECK();
  return 0;
}
