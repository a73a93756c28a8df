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
// close to 1 exact.  The recurrence is a chain in time.  A column j of S never meets another column, so four
// neighbouring lanes own one or two columns (a quarter of the rows each, contiguous) in registers for the whole
// step, and a block owns some columns of one (request, head).  Tokens are taken in chunks: alpha, k, q, v of the next chunk
// come into shared memory by asynchronous copies while every lane group walks the chunk before without any
// barrier.  A column's numbers do not depend on which block owns it.
//
// Steps that bring long portions (a prompt) cut every request's rows into segments of GLA_SEG tokens and run three
// passes, since a chain of thousands of tokens on the few thousand threads that one request's state occupies
// leaves the GPU idle: (1) every segment's chain from a ZERO state, all segments at once, which gives the
// segment's own contribution L and the product P of its decays per key channel; (2) per request, over its
// segments in order, S <- P * S + L, leaving in L's place the state each segment starts from, and the request's
// new state in its slot; (3) every segment's chain again from its true start state, all at once, now with the
// outputs.  Twice the arithmetic, T / GLA_SEG times the parallelism; the numbers differ from the one chain by
// float32 rounding only (the same sums, associated differently at segment borders).
#include "common.cuh"

constexpr int GLA_LANES = 4;          // lanes that share a column
constexpr int GLA_MAX_THREADS = 256;  // a block: 64 groups of four lanes, each group one or two columns

// alpha[t, c] for every token and channel c < C (= heads * D).  A block takes 128 channels and GLA_DECAY_ROUNDS rounds
// of GLA_DECAY_TOKENS tokens: the channels' rows of W2 (transposed) and the tokens' L inner values (transposed) lie in shared memory,
// a thread owns one channel and walks the rank once for all the block's tokens.  The inner product over the rank
// L is one sequential float32 sum in index order, the same whatever else the step holds.
constexpr int GLA_DECAY_TOKENS = 16, GLA_DECAY_ROUNDS = 4, GLA_DECAY_CHANNELS = 128;
constexpr int GLA_DECAY_WS = GLA_DECAY_CHANNELS + 1;      // floats between two rank rows of W2 in shared memory (no bank conflicts)

template <typename W>
__global__ void __launch_bounds__(GLA_DECAY_CHANNELS)
gla_decay_kernel(const float* __restrict__ proj, int proj_stride, int inner_off, int L,
                 const W* __restrict__ w2, const float* __restrict__ bias, float* __restrict__ alpha,
                 int T, int C, float inv_tau) {
  extern __shared__ __align__(16) float s_dec[];
  float* s_in = s_dec;                                        // [L][GLA_DECAY_TOKENS]
  float* s_w = s_dec + (size_t)L * GLA_DECAY_TOKENS;          // [L][GLA_DECAY_WS]
  const int c0 = blockIdx.x * GLA_DECAY_CHANNELS;
  for (int idx = threadIdx.x; idx < GLA_DECAY_CHANNELS * L; idx += blockDim.x) {
    const int c = idx / L, i = idx % L;                 // consecutive threads read consecutive elements of W2
    s_w[i * GLA_DECAY_WS + c] = c0 + c < C ? qb_to_float<W>(w2[(size_t)(c0 + c) * L + i]) : 0.f;
  }
  const int c = c0 + threadIdx.x;
  const float b = c < C ? bias[c] : 0.f;
  // the block's tokens in rounds of GLA_DECAY_TOKENS: the rows of W2 are staged once for all of them
  for (int round = 0; round < GLA_DECAY_ROUNDS; ++round) {
    const int t0 = (blockIdx.y * GLA_DECAY_ROUNDS + round) * GLA_DECAY_TOKENS;
    if (t0 >= T) break;
    const int nt = min(GLA_DECAY_TOKENS, T - t0);
    __syncthreads();                                    // the round before is done with s_in
    for (int idx = threadIdx.x; idx < GLA_DECAY_TOKENS * L; idx += blockDim.x) {
      const int i = idx / GLA_DECAY_TOKENS, tt = idx % GLA_DECAY_TOKENS;
      s_in[i * GLA_DECAY_TOKENS + tt] = tt < nt ? proj[(size_t)(t0 + tt) * proj_stride + inner_off + i] : 0.f;
    }
    __syncthreads();
    float z[GLA_DECAY_TOKENS];
#pragma unroll
    for (int tt = 0; tt < GLA_DECAY_TOKENS; ++tt) z[tt] = 0.f;
    for (int i = 0; i < L; ++i) {
      const float w = s_w[i * GLA_DECAY_WS + threadIdx.x];
#pragma unroll
      for (int tt = 0; tt < GLA_DECAY_TOKENS; tt += 4) {
        const float4 x = *reinterpret_cast<const float4*>(s_in + i * GLA_DECAY_TOKENS + tt);
        z[tt] = fmaf(w, x.x, z[tt]);
        z[tt + 1] = fmaf(w, x.y, z[tt + 1]);
        z[tt + 2] = fmaf(w, x.z, z[tt + 2]);
        z[tt + 3] = fmaf(w, x.w, z[tt + 3]);
      }
    }
    if (c < C) {
#pragma unroll
      for (int tt = 0; tt < GLA_DECAY_TOKENS; ++tt) {
        if (tt < nt) {
          const float zz = z[tt] + b;
          const float ls = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));
          alpha[(size_t)(t0 + tt) * C + c] = expf(ls * inv_tau);
        }
      }
    }
  }
}

// The same for steps of few tokens: one thread a (token, channel), a block a token and 128 channels, so that the few
// tokens' channels spread over many SMs; the same sum in the same order.
template <typename W>
__global__ void gla_decay_small_kernel(const float* __restrict__ proj, int proj_stride, int inner_off, int L,
                                       const W* __restrict__ w2, const float* __restrict__ bias,
                                       float* __restrict__ alpha, int T, int C, float inv_tau) {
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
__device__ __forceinline__ void gla_copy16(float* dst_smem, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

constexpr int GLA_SEG = 64;        // tokens a segment of the three-pass form
constexpr int GLA_DIRECT = 0, GLA_LOCAL = 1, GLA_REPLAY = 2;

// The segments of a step: request r's rows [t0, t1) in runs of GLA_SEG.  seg[s] = (first row, end row, request row,
// index within the request); req_seg[r] = (first segment, segments).  One block; R <= 1024.
__global__ void gla_segments_kernel(const int* __restrict__ req_start, int R, int4* __restrict__ seg,
                                    int2* __restrict__ req_seg, int* __restrict__ n_seg) {
  __shared__ int s_n[1024];
  const int r = threadIdx.x;
  const int t0 = r < R ? req_start[r] : 0, t1 = r < R ? req_start[r + 1] : 0;
  const int n = (t1 - t0 + GLA_SEG - 1) / GLA_SEG;
  s_n[r] = n;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const int a = r >= o ? s_n[r - o] : 0;
    __syncthreads();
    s_n[r] += a;
    __syncthreads();
  }
  const int first = s_n[r] - n;
  if (r < R) {
    req_seg[r] = make_int2(first, n);
    for (int c = 0; c < n; ++c) seg[first + c] = make_int4(t0 + c * GLA_SEG, min(t1, t0 + (c + 1) * GLA_SEG), r, c);
  }
  if (r == 1023) n_seg[0] = s_n[r];
}

// Pass 2: thread per state element (request, head, i, j); over the request's segments in order.
__global__ void gla_combine_kernel(float* __restrict__ state, float* __restrict__ seg_state, const float* __restrict__ seg_decay,
                                   const int2* __restrict__ req_seg, const int* __restrict__ req_slot, int H, int D, int E) {
  const int r = blockIdx.x, h = blockIdx.y;
  const int2 rs = req_seg[r];
  float* S = state + ((size_t)req_slot[r] * H + h) * D * E;
  for (int idx = blockIdx.z * blockDim.x + threadIdx.x; idx < D * E; idx += gridDim.z * blockDim.x) {
    const int i = idx / E;
    float s = S[idx];
    // eight segments a turn: their loads are in flight together, then the short chain, then the stores
    for (int c0 = 0; c0 < rs.y; c0 += 8) {
      float l[8], p[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (c0 + u < rs.y) {
          const size_t sg = (size_t)(rs.x + c0 + u) * H + h;
          l[u] = __ldcg(seg_state + sg * D * E + idx);
          p[u] = __ldcg(seg_decay + sg * D + i);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (c0 + u < rs.y) {
          const size_t sg = (size_t)(rs.x + c0 + u) * H + h;
          seg_state[sg * D * E + idx] = s;      // the state this segment starts from
          s = fmaf(p[u], s, l[u]);
        }
      }
    }
    S[idx] = s;
  }
}

// RPT: rows (key channels) of a column a lane holds, contiguous, D <= GLA_LANES * RPT; CPT: columns a thread holds.
// A token's decays, keys and queries are read from shared memory as 16-byte vectors that the lanes of all the
// warp's columns share, and serve CPT columns each: the kernel is bound by its multiply-adds, not by those reads.
template <int RPT, int CPT, int MODE>
__global__ void __launch_bounds__(GLA_MAX_THREADS, 1)
gla_chain_kernel(const float* __restrict__ proj, int proj_stride, int q_off, int k_off, int v_off,
                 const float* __restrict__ alpha, float* __restrict__ state, float* __restrict__ out,
                 const int* __restrict__ req_start, const int* __restrict__ req_slot, const int4* __restrict__ seg,
                 const int* __restrict__ n_seg, float* __restrict__ seg_state, float* __restrict__ seg_decay,
                 int H, int D, int E, int cols_per_block, int chunk, int EP, int vec, float q_scale) {
  extern __shared__ __align__(16) float sm[];
  // floats between the rows of two neighbouring lanes: padded where the plain distance would put the four lanes'
  // vectors on the same banks
  constexpr int RS = RPT + (RPT >= 16 ? 4 : 0);
  constexpr int DP = GLA_LANES * RS;
  const int r = blockIdx.x, h = blockIdx.y;
  if (MODE != GLA_DIRECT && r >= n_seg[0]) return;
  const int col0 = blockIdx.z * cols_per_block;
  const int tid = threadIdx.x;
  const int p = tid % GLA_LANES, cg = tid / GLA_LANES;
  const int j0 = col0 + cg * CPT;
  bool owns[CPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c) owns[c] = cg * CPT + c < cols_per_block && j0 + c < E;
  // a buffer: alpha, k, q [chunk][DP] and v [chunk][EP]; two buffers
  const int plane = chunk * DP, bufsz = 3 * plane + chunk * EP;
  // the padding rows (i >= D) are read as zeros and never written
  for (int i = tid; i < 2 * bufsz; i += blockDim.x) sm[i] = 0.f;

  int t0, t1;
  float* S;
  if (MODE == GLA_DIRECT) {
    t0 = req_start[r];
    t1 = req_start[r + 1];
    S = state + ((size_t)req_slot[r] * H + h) * D * E;
  } else {
    const int4 sg = seg[r];
    t0 = sg.x;
    t1 = sg.y;
    S = seg_state + ((size_t)r * H + h) * D * E;
  }
  float col[CPT][RPT], decay[MODE == GLA_LOCAL ? RPT : 1];
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = p * RPT + ii;
#pragma unroll
    for (int c = 0; c < CPT; ++c) col[c][ii] = (MODE != GLA_LOCAL && owns[c] && i < D) ? S[(size_t)i * E + j0 + c] : 0.f;
    if (MODE == GLA_LOCAL) decay[ii] = 1.f;
  }
  __syncthreads();

  // row i of a token lies at (i / RPT) * RS + i % RPT of the token's DP floats
  auto fetch = [&](int c0, int buf) {
    const int n = min(chunk, t1 - c0);
    float* b = sm + buf * bufsz;
    if (vec) {          // D and E multiples of 4, rows that start on 16 bytes: four elements a copy
      const int D4 = D / 4, E4 = E / 4;
      for (int idx = tid; idx < n * D4; idx += blockDim.x) {
        const int tt = idx / D4, i = (idx % D4) * 4;
        const int dst = tt * DP + (i / RPT) * RS + i % RPT;
        const float* row = proj + (size_t)(c0 + tt) * proj_stride + (size_t)h * D + i;
        gla_copy16(b + dst, alpha + ((size_t)(c0 + tt) * H + h) * D + i);
        gla_copy16(b + plane + dst, row + k_off);
        if (MODE != GLA_LOCAL) gla_copy16(b + 2 * plane + dst, row + q_off);
      }
      for (int idx = tid; idx < n * E4; idx += blockDim.x) {
        const int tt = idx / E4, i = (idx % E4) * 4;
        gla_copy16(b + 3 * plane + tt * EP + i, proj + (size_t)(c0 + tt) * proj_stride + v_off + (size_t)h * E + i);
      }
    } else {
      for (int idx = tid; idx < n * D; idx += blockDim.x) {
        const int tt = idx / D, i = idx % D;
        const int dst = tt * DP + (i / RPT) * RS + i % RPT;
        const float* row = proj + (size_t)(c0 + tt) * proj_stride + (size_t)h * D + i;
        gla_copy4(b + dst, alpha + ((size_t)(c0 + tt) * H + h) * D + i);
        gla_copy4(b + plane + dst, row + k_off);
        if (MODE != GLA_LOCAL) gla_copy4(b + 2 * plane + dst, row + q_off);
      }
      for (int idx = tid; idx < n * E; idx += blockDim.x) {
        const int tt = idx / E, i = idx % E;
        gla_copy4(b + 3 * plane + tt * EP + i, proj + (size_t)(c0 + tt) * proj_stride + v_off + (size_t)h * E + i);
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
    const float* s_a = sm + buf * bufsz + p * RS;
    const float* s_k = s_a + plane;
    const float* s_q = s_k + plane;
    const float* s_v = sm + buf * bufsz + 3 * plane;
    auto token = [&](int tt) {
      const int o = tt * DP;
      float vj[CPT], acc[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        vj[c] = owns[c] ? s_v[tt * EP + j0 + c] : 0.f;
        acc[c] = 0.f;
      }
#pragma unroll
      for (int f = 0; f < RPT; f += 4) {
        const float4 a4 = *reinterpret_cast<const float4*>(s_a + o + f);
        const float4 k4 = *reinterpret_cast<const float4*>(s_k + o + f);
        float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (MODE != GLA_LOCAL) q4 = *reinterpret_cast<const float4*>(s_q + o + f);
        const float av[4] = {a4.x, a4.y, a4.z, a4.w}, kv[4] = {k4.x, k4.y, k4.z, k4.w}, qv[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            const float s_new = fmaf(av[e], col[c][f + e], kv[e] * vj[c]);
            col[c][f + e] = s_new;
            if (MODE != GLA_LOCAL) acc[c] = fmaf(qv[e], s_new, acc[c]);
          }
          if (MODE == GLA_LOCAL) decay[f + e] *= av[e];
        }
      }
      if (MODE != GLA_LOCAL) {
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          float v = acc[c];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          if (owns[c] && p == 0) out[((size_t)(c0 + tt) * H + h) * E + j0 + c] = v * q_scale;
        }
      }
    };
    int tt = 0;
    for (; tt + 2 <= n; tt += 2) {          // two tokens a turn: their sums across lanes overlap
      token(tt); token(tt + 1);
    }
    for (; tt < n; ++tt) token(tt);
  }
  if (MODE == GLA_REPLAY) return;
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = p * RPT + ii;
    if (i < D) {
#pragma unroll
      for (int c = 0; c < CPT; ++c)
        if (owns[c]) S[(size_t)i * E + j0 + c] = col[c][ii];
      if (MODE == GLA_LOCAL && j0 == 0 && owns[0]) seg_decay[((size_t)r * H + h) * D + i] = decay[ii];
    }
  }
}

// floats of scratch for the three-pass form of a step of T tokens in R requests (0: the step runs as one chain)
extern "C" long long qb_gla_segment_scratch(int R, int T, int H, int D, int E) {
  if (T < 512 || (long long)T < 64ll * R || R > 1024) return 0;
  const long long max_seg = T / GLA_SEG + R;
  // as int32: seg [max_seg] int4, req_seg [R] int2 (padded to 16 bytes), n_seg (16 bytes); then seg_decay
  // [max_seg, H, D] and seg_state [max_seg, H, D, E]
  return 4 * max_seg + ((2ll * R + 3) & ~3ll) + 4 + max_seg * H * D + max_seg * H * D * E;
}

// proj: float32 rows of the step's fused projection (q, k at q_off / k_off: heads x D; v at v_off: heads x E; the
// L inner values of the decay at inner_off).  w2: [heads*D, L] in w2_dtype, bias: float32 [heads*D].
// state: float32 [slots, heads, D, E]; out: float32 [T, heads, E]; scratch: T * heads * D floats (alpha);
// seg_scratch: qb_gla_segment_scratch(...) floats, 16-byte aligned, or null (then the step runs as one chain).
extern "C" int qb_gla(const float* proj, int proj_stride, int q_off, int k_off, int v_off, int inner_off, int L,
                      const void* w2, int w2_dtype, const float* bias, float* state, float* out, float* scratch,
                      float* seg_scratch, const int* req_start, const int* req_slot, int R, int T, int H, int D, int E,
                      float tau, float q_scale, cudaStream_t stream) {
  if (R <= 0 || T <= 0) return 0;
  if (D <= 0 || D > 256 || E <= 0 || E > 256 || H <= 0 || L <= 0 || tau <= 0.f) return QB_ERR_UNSUPPORTED;
  const int C = H * D;
  {
    const size_t smem = (size_t)L * (GLA_DECAY_WS + GLA_DECAY_TOKENS) * sizeof(float);
    if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
    const int per_block = GLA_DECAY_TOKENS * GLA_DECAY_ROUNDS;
    dim3 grid((C + GLA_DECAY_CHANNELS - 1) / GLA_DECAY_CHANNELS, (T + per_block - 1) / per_block);
    if (grid.y > 65535) return QB_ERR_UNSUPPORTED;
    if (T < 64) {
      QB_DISPATCH_DTYPE(w2_dtype, W, gla_decay_small_kernel<W><<<dim3((C + 127) / 128, T), 128, L * sizeof(float), stream>>>(
          proj, proj_stride, inner_off, L, (const W*)w2, bias, scratch, T, C, 1.f / tau));
    } else QB_DISPATCH_DTYPE(w2_dtype, W, {
      auto kern = gla_decay_kernel<W>;
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
      }
      kern<<<grid, GLA_DECAY_CHANNELS, smem, stream>>>(proj, proj_stride, inner_off, L, (const W*)w2, bias, scratch, T, C,
                                                       1.f / tau);
    });
    QB_LAUNCH_CHECK();
  }
  const bool segmented = seg_scratch != nullptr && qb_gla_segment_scratch(R, T, H, D, E) > 0;
  const int max_seg = T / GLA_SEG + R;
  const int rpt = D <= 16 ? 4 : D <= 32 ? 8 : D <= 64 ? 16 : D <= 128 ? 32 : 64;
  const int cpt = rpt <= 32 ? 2 : 1;          // columns a thread: what its registers hold
  // columns a block: all of them (at most what GLA_MAX_THREADS threads hold) unless that leaves most SMs idle; then
  // fewer, down to 16 where requests bring portions (the block's threads also fetch the chunks) and down to one
  // warp's where every request brings one token (the state's bytes are what counts, spread over all SMs); whole warps
  const int warp_cols = 32 / GLA_LANES * cpt, max_cols = GLA_MAX_THREADS / GLA_LANES * cpt;
  const int min_cols = T > R ? 16 : warp_cols;
  const long units = segmented ? (long)(T / GLA_SEG) : (long)R;
  int splits = (E + max_cols - 1) / max_cols;
  while (units * H * splits < 132 && (E + 2 * splits - 1) / (2 * splits) >= min_cols) splits *= 2;
  int cols = (E + splits - 1) / splits;
  cols = (cols + warp_cols - 1) / warp_cols * warp_cols;
  splits = (E + cols - 1) / cols;
  const int threads = cols / cpt * GLA_LANES;
  const int rs = rpt + (rpt >= 16 ? 4 : 0), dp = rs * GLA_LANES;
  const int ep = (E + 3) / 4 * 4;
  const int chunk = dp <= 160 ? 16 : 8;
  const size_t smem = (size_t)2 * chunk * (3 * dp + ep) * sizeof(float);
  if (H > 65535 || splits > 65535) return QB_ERR_UNSUPPORTED;
  const int vec = (D % 4 == 0 && E % 4 == 0 && proj_stride % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 &&
                   ((uintptr_t)proj & 15) == 0 && ((uintptr_t)scratch & 15) == 0) ? 1 : 0;
  if (segmented && ((uintptr_t)seg_scratch & 15)) return QB_ERR_BAD_ARG;
  int4* seg = reinterpret_cast<int4*>(seg_scratch);
  int2* req_seg = segmented ? reinterpret_cast<int2*>(seg + max_seg) : nullptr;
  int* n_seg = segmented ? reinterpret_cast<int*>(seg_scratch + 4 * (size_t)max_seg + ((2 * (size_t)R + 3) & ~(size_t)3)) : nullptr;
  float* seg_decay = segmented ? reinterpret_cast<float*>(n_seg + 4) : nullptr;
  float* seg_state = segmented ? seg_decay + (size_t)max_seg * H * D : nullptr;
#define GLA_LAUNCH(N, CPT_, MODE_, GRIDX)                                                                  \
  do {                                                                                                     \
    auto kern = gla_chain_kernel<N, CPT_, MODE_>;                                                          \
    if (smem > 48 * 1024) {                                                                                \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      if (e != cudaSuccess) return (int)e;                                                                 \
    }                                                                                                      \
    kern<<<dim3(GRIDX, H, splits), threads, smem, stream>>>(proj, proj_stride, q_off, k_off, v_off, scratch, state, out, \
                                          req_start, req_slot, seg, n_seg, seg_state, seg_decay, H, D, E, cols, chunk, ep, vec, q_scale); \
  } while (0)
#define GLA_LAUNCH_RPT(MODE_, GRIDX)              \
  do {                                            \
    if (rpt == 4) GLA_LAUNCH(4, 2, MODE_, GRIDX);    \
    else if (rpt == 8) GLA_LAUNCH(8, 2, MODE_, GRIDX);   \
    else if (rpt == 16) GLA_LAUNCH(16, 2, MODE_, GRIDX); \
    else if (rpt == 32) GLA_LAUNCH(32, 2, MODE_, GRIDX); \
    else GLA_LAUNCH(64, 1, MODE_, GRIDX);            \
  } while (0)
  if (!segmented) {
    GLA_LAUNCH_RPT(GLA_DIRECT, R);
  } else {
    gla_segments_kernel<<<1, 1024, 0, stream>>>(req_start, R, seg, req_seg, n_seg);
    GLA_LAUNCH_RPT(GLA_LOCAL, max_seg);
    int zsplit = (D * E + 255) / 256;
    while ((long)R * H * zsplit > 4096 && zsplit > 1) zsplit = (zsplit + 1) / 2;
    gla_combine_kernel<<<dim3(R, H, zsplit), 256, 0, stream>>>(state, seg_state, seg_decay, req_seg, req_slot, H, D, E);
    GLA_LAUNCH_RPT(GLA_REPLAY, max_seg);
  }
#undef GLA_LAUNCH_RPT
#undef GLA_LAUNCH
  QB_LAUNCH_CHECK();
  return 0;
}
