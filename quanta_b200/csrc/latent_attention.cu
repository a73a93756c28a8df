// Softmax attention over a cached low-rank latent, all heads reading the same cache row, with a sink.
//
// Per token the cache keeps one row of C + R elements: the normed latent c (C) and one rotated key part
// (R) that every head shares.  With the up-projections folded into the query (q_lat = W_uk^T q_plain,
// a library product per head) a head's score against position j is
//
//   s_j = (q_lat . c_j + q_rot . krot_j) * scale
//
// and its result is sum_j p_j c_j (C numbers, taken through W_uv by another library product).  The
// softmax has a sink: the denominator also holds exp(sink_h), which has no key and no value.
//
//   qb_latent_write : dkv rows -> RMS norm of the first C (gain), rotation of the last R -> cache row
//   qb_latent_query : q rows [T, H, D + R] float32 -> q_plain [H, T, D] (activation dtype) and the rotated
//                     part [T, H, R] float32
//   qb_latent_attend: every (token, group of heads, range of keys): a block walks the keys of its range in
//                     tiles of 32 through the block table, a warp a head, lanes own keys for the scores
//                     and latent channels for the sum; float32 throughout; partial (max, sum, vector)
//   qb_latent_merge : partial results of a (token, head) in range order, the sink, division, output
//                     [H, T, C] in the activation dtype
//
// A token attends positions 0 .. its own whatever else is in the batch; its result depends on the number
// of ranges only through the order of float32 additions.  Rotation: the first rd of the R dimensions, pair
// (i, i + rd/2), angle = position * inv_freq[i], in float32; the rest pass unchanged.
#include "common.cuh"

constexpr int LA_TILE = 32;        // keys a tile
constexpr int LA_MAX_WARPS = 8;    // heads a block
constexpr int LA_MAX_C = 512;      // latent channels (a lane holds C / 32 sums)

// ---------------------------------------------------------------------------------------------
template <typename A>
__global__ void latent_write_kernel(const float* __restrict__ dkv, const float* __restrict__ gain,
                                    const float* __restrict__ inv_freq, A* __restrict__ cache,
                                    const int* __restrict__ tok_pos, const int* __restrict__ tok_req,
                                    const int* __restrict__ block_table, int bt_stride, int T, int C, int R,
                                    int rd, int page_size, int num_pages, float eps, int* status) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  if (t >= T) return;
  const float* row = dkv + (size_t)t * (C + R);
  float ss = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) ss += row[i] * row[i];
  const float total = qb_block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(total / (float)C + eps);
  const int pos = tok_pos[t];
  const int page = block_table[(size_t)tok_req[t] * bt_stride + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) qb_set_status(status, QB_STATUS_BAD_PAGE, page, 2);
    return;
  }
  A* dst = cache + ((size_t)page * page_size + pos % page_size) * (C + R);
  for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = qb_from_float<A>(row[i] * inv * gain[i]);
  const int half = rd / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float ang = (float)pos * inv_freq[i];
    float sn, cs;
    sincosf(ang, &sn, &cs);
    const float u = row[C + i], v = row[C + half + i];
    dst[C + i] = qb_from_float<A>(u * cs - v * sn);
    dst[C + half + i] = qb_from_float<A>(v * cs + u * sn);
  }
  for (int i = rd + threadIdx.x; i < R; i += blockDim.x) dst[C + i] = qb_from_float<A>(row[C + i]);
}

extern "C" int qb_latent_write(const float* dkv, const float* gain, const float* inv_freq, void* cache,
                               int dtype, const int* tok_pos, const int* tok_req, const int* block_table,
                               int bt_stride, int T, int C, int R, int rd, int page_size, int num_pages,
                               float eps, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rd % 2 || rd < 0 || rd > R || C <= 0 || page_size <= 0) return QB_ERR_BAD_ARG;
  QB_DISPATCH_DTYPE(dtype, A, latent_write_kernel<A><<<T, 128, 0, stream>>>(
      dkv, gain, inv_freq, (A*)cache, tok_pos, tok_req, block_table, bt_stride, T, C, R, rd, page_size,
      num_pages, eps, status));
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
template <typename A>
__global__ void latent_query_kernel(const float* __restrict__ q, const float* __restrict__ inv_freq,
                                    A* __restrict__ q_plain, float* __restrict__ q_rot,
                                    const int* __restrict__ tok_pos, int T, int H, int D, int R, int rd) {
  const int t = blockIdx.x, h = blockIdx.y;
  const float* row = q + ((size_t)t * H + h) * (D + R);
  A* qp = q_plain + ((size_t)h * T + t) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) qp[i] = qb_from_float<A>(row[i]);
  const int half = rd / 2;
  const float pos = (float)tok_pos[t];
  float* qr = q_rot + ((size_t)t * H + h) * R;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf(pos * inv_freq[i], &sn, &cs);
    const float u = row[D + i], v = row[D + half + i];
    qr[i] = u * cs - v * sn;
    qr[half + i] = v * cs + u * sn;
  }
  for (int i = rd + threadIdx.x; i < R; i += blockDim.x) qr[i] = row[D + i];
}

extern "C" int qb_latent_query(const float* q, const float* inv_freq, void* q_plain, int dtype, float* q_rot,
                               const int* tok_pos, int T, int H, int D, int R, int rd, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rd % 2 || rd < 0 || rd > R) return QB_ERR_BAD_ARG;
  dim3 grid(T, H);
  QB_DISPATCH_DTYPE(dtype, A, latent_query_kernel<A><<<grid, 64, 0, stream>>>(
      q, inv_freq, (A*)q_plain, q_rot, tok_pos, T, H, D, R, rd));
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Partial results: part[((t * H + h) * n_ranges + s) * (C + 2)] = {max, sum, vector[C]}.
template <typename A, typename QL>
__global__ void latent_attend_kernel(const QL* __restrict__ q_lat, const float* __restrict__ q_rot,
                                     const A* __restrict__ cache, float* __restrict__ part,
                                     const int* __restrict__ tok_pos, const int* __restrict__ tok_req,
                                     const int* __restrict__ block_table, int bt_stride, int T, int H, int C,
                                     int R, int page_size, int num_pages, int heads_per_block, int n_ranges,
                                     float scale, int* status) {
  extern __shared__ float sm[];
  const int W = C + R, WP = W | 1;            // odd row stride: lanes that own keys hit different banks
  float* s_q = sm;                             // [heads_per_block][W]
  float* s_tile = s_q + (size_t)heads_per_block * W;      // [LA_TILE][WP]
  __shared__ long s_row[LA_TILE];             // element offset of each key's cache row, -1: none
  const int t = blockIdx.x, h0 = blockIdx.y * heads_per_block, range = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int h = h0 + warp;
  const bool live = h < H;
  const int pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_req[t] * bt_stride;

  if (live) {
    const QL* ql = q_lat + ((size_t)h * T + t) * C;
    for (int i = lane; i < C; i += 32) s_q[warp * W + i] = qb_to_float<QL>(ql[i]);
    const float* qr = q_rot + ((size_t)t * H + h) * R;
    for (int i = lane; i < R; i += 32) s_q[warp * W + C + i] = qr[i];
  }
  const int n_tiles = pos / LA_TILE + 1;
  const int per = (n_tiles + n_ranges - 1) / n_ranges;
  const int tile_lo = range * per, tile_hi = min(n_tiles, tile_lo + per);

  float m = -INFINITY, l = 0.f;
  float acc[LA_MAX_C / 32];
#pragma unroll
  for (int i = 0; i < LA_MAX_C / 32; ++i) acc[i] = 0.f;

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int k0 = tile * LA_TILE;
    const int n_here = min(LA_TILE, pos - k0 + 1);
    __syncthreads();                           // the tile before has been read (and s_q is written)
    if (threadIdx.x < LA_TILE) {
      long off = -1;
      if ((int)threadIdx.x < n_here) {
        const int key = k0 + threadIdx.x;
        const int page = bt[key / page_size];
        if (page < 0 || page >= num_pages) qb_set_status(status, QB_STATUS_BAD_PAGE, page, 3);
        else off = ((long)page * page_size + key % page_size) * W;
      }
      s_row[threadIdx.x] = off;
    }
    __syncthreads();
    for (int k = warp; k < LA_TILE; k += nwarps) {
      const long off = s_row[k];
      float* dst = s_tile + (size_t)k * WP;
      if (off >= 0) {
        const A* src = cache + off;
        for (int i = lane; i < W; i += 32) dst[i] = qb_to_float<A>(src[i]);
      } else {
        for (int i = lane; i < W; i += 32) dst[i] = 0.f;
      }
    }
    __syncthreads();
    if (!live) continue;
    // scores: this lane's key against the head's query
    const float* qrow = s_q + warp * W;
    const float* krow = s_tile + (size_t)lane * WP;
    float dot = 0.f;
    for (int i = 0; i < W; ++i) dot += qrow[i] * krow[i];
    const bool valid = lane < n_here && s_row[lane] >= 0;
    const float s = valid ? dot * scale : -INFINITY;
    const float mb = qb_warp_max(s);
    if (mb == -INFINITY) continue;
    const float m_new = fmaxf(m, mb);
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + qb_warp_sum(p);
#pragma unroll
    for (int i = 0; i < LA_MAX_C / 32; ++i) acc[i] *= corr;
    for (int k = 0; k < n_here; ++k) {
      const float pk = __shfl_sync(0xffffffffu, p, k);
      const float* crow = s_tile + (size_t)k * WP;
#pragma unroll
      for (int i = 0; i < LA_MAX_C / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < C) acc[i] += pk * crow[d];
      }
    }
    m = m_new;
  }
  if (!live) return;
  float* dst = part + (((size_t)t * H + h) * n_ranges + range) * (C + 2);
  if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
  for (int i = 0; i < LA_MAX_C / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < C) dst[2 + d] = acc[i];
  }
}

extern "C" int qb_latent_attend(const void* q_lat, int q_lat_dtype, const float* q_rot, const void* cache,
                                int dtype, float* part, const int* tok_pos, const int* tok_req,
                                const int* block_table, int bt_stride, int T, int H, int C, int R,
                                int page_size, int num_pages, int n_ranges, float scale, int* status,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C <= 0 || C > LA_MAX_C || R < 0 || n_ranges < 1 || page_size <= 0) return QB_ERR_UNSUPPORTED;
  const int hpb = H < LA_MAX_WARPS ? H : LA_MAX_WARPS;
  const int W = C + R, WP = W | 1;
  const size_t smem = ((size_t)hpb * W + (size_t)LA_TILE * WP) * sizeof(float);
  if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
  dim3 grid(T, (H + hpb - 1) / hpb, n_ranges);
  QB_DISPATCH_DTYPE(dtype, A, QB_DISPATCH_DTYPE(q_lat_dtype, QL, {
    auto kern = latent_attend_kernel<A, QL>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    kern<<<grid, hpb * 32, smem, stream>>>((const QL*)q_lat, q_rot, (const A*)cache, part, tok_pos, tok_req,
                                           block_table, bt_stride, T, H, C, R, page_size, num_pages, hpb,
                                           n_ranges, scale, status);
  }));
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// One warp a (token, head): top = max(sink, every range's max); denominator = exp(sink - top) + sum of the
// ranges' sums scaled to top; out[h, t, :] = sum of the ranges' vectors scaled to top / denominator.
template <typename A>
__global__ void latent_merge_kernel(const float* __restrict__ part, const float* __restrict__ sink,
                                    A* __restrict__ out, int T, int H, int C, int n_ranges) {
  const int lane = threadIdx.x & 31;
  const long wid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (long)T * H) return;
  const int t = (int)(wid / H), h = (int)(wid % H);
  const float* src = part + ((size_t)t * H + h) * n_ranges * (C + 2);
  const float sk = sink ? sink[h] : -INFINITY;
  float top = sk;
  for (int s = 0; s < n_ranges; ++s) top = fmaxf(top, src[(size_t)s * (C + 2)]);
  float denom = sink ? expf(sk - top) : 0.f;
  for (int s = 0; s < n_ranges; ++s) {
    const float ms = src[(size_t)s * (C + 2)];
    if (ms != -INFINITY) denom += src[(size_t)s * (C + 2) + 1] * expf(ms - top);
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  A* dst = out + ((size_t)h * T + t) * C;
  for (int d = lane; d < C; d += 32) {
    float v = 0.f;
    for (int s = 0; s < n_ranges; ++s) {
      const float ms = src[(size_t)s * (C + 2)];
      if (ms != -INFINITY) v += src[(size_t)s * (C + 2) + 2 + d] * expf(ms - top);
    }
    dst[d] = qb_from_float<A>(v * inv);
  }
}

extern "C" int qb_latent_merge(const float* part, const float* sink, void* out, int dtype, int T, int H, int C,
                               int n_ranges, cudaStream_t stream) {
  if (T <= 0) return 0;
  const long warps = (long)T * H;
  const int blocks = (int)((warps + 3) / 4);
  QB_DISPATCH_DTYPE(dtype, A, latent_merge_kernel<A><<<blocks, 128, 0, stream>>>(part, sink, (A*)out, T, H, C,
                                                                                n_ranges));
  QB_LAUNCH_CHECK();
  return 0;
}
