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
    if (smem + 2048 > 48 * 1024) {   /* the kernel also has some static shared memory */
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
// One block a (token, head): top = max(sink, every range's max); denominator = exp(sink - top) + sum of the
// ranges' sums scaled to top; out[h, t, :] = sum of the ranges' vectors scaled to top / denominator.  The
// first warp works out the ranges' weights (a lane a range, two for more than 32), then a thread a channel
// adds the ranges in index order.
constexpr int LA_MAX_RANGES = 64;

template <typename A>
__global__ void latent_merge_kernel(const float* __restrict__ part, const float* __restrict__ sink,
                                    A* __restrict__ out, int T, int H, int C, int n_ranges) {
  __shared__ float s_w[LA_MAX_RANGES];
  __shared__ float s_inv;
  const int t = blockIdx.x / H, h = blockIdx.x % H;
  const float* src = part + ((size_t)t * H + h) * n_ranges * (C + 2);
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float ms[2], ls[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int s = lane + 32 * e;
      ms[e] = s < n_ranges ? src[(size_t)s * (C + 2)] : -INFINITY;
      ls[e] = s < n_ranges ? src[(size_t)s * (C + 2) + 1] : 0.f;
    }
    const float sk = sink ? sink[h] : -INFINITY;
    const float top = fmaxf(sk, qb_warp_max(fmaxf(ms[0], ms[1])));
    float w[2], d = 0.f;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      w[e] = (ms[e] == -INFINITY) ? 0.f : expf(ms[e] - top);
      d += w[e] * ls[e];
      if (lane + 32 * e < LA_MAX_RANGES) s_w[lane + 32 * e] = w[e];
    }
    d = qb_warp_sum(d) + (sink ? expf(sk - top) : 0.f);
    if (lane == 0) s_inv = d > 0.f ? 1.f / d : 0.f;
  }
  __syncthreads();
  const float inv = s_inv;
  A* dst = out + ((size_t)h * T + t) * C;
  for (int d = threadIdx.x; d < C; d += blockDim.x) {
    float v = 0.f;
#pragma unroll 4
    for (int s = 0; s < n_ranges; ++s) v += src[(size_t)s * (C + 2) + 2 + d] * s_w[s];
    dst[d] = qb_from_float<A>(v * inv);
  }
}

extern "C" int qb_latent_merge(const float* part, const float* sink, void* out, int dtype, int T, int H, int C,
                               int n_ranges, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_ranges < 1 || n_ranges > LA_MAX_RANGES) return QB_ERR_UNSUPPORTED;
  const int threads = C >= 256 ? 256 : C >= 128 ? 128 : 64;
  QB_DISPATCH_DTYPE(dtype, A, latent_merge_kernel<A><<<T * H, threads, 0, stream>>>(part, sink, (A*)out, T, H, C,
                                                                                 n_ranges));
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// The same attention on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 sums), for
// bfloat16 caches with C a multiple of 64 and R a multiple of 16.  All heads of a token read the same
// cache rows, so the rows of a tile are (token, head) pairs of one request's portion, flattened, 16 a row
// group: a single token with 16 heads fills an MMA tile, and a portion fills as many as it has.  A block
// has LM_RG row groups of four warps each.  For a tile of 64 keys the four warps of a row group each take
// 16 keys of S = Q K^T, exchange row maxima and sums through shared memory, leave P (bfloat16) there, and
// then each take a quarter of the C channels of O += P V, V being the first C columns of the very rows K
// was read from; the next tile's rows come in by asynchronous copies meanwhile.  Blocks find their rows from the requests' token ranges on the device (no host list), so
// captured decode steps run it too; a block's keys can be one of n_ranges ranges, merged afterwards.
constexpr int LM_RG = 2;                    // row groups a block
constexpr int LM_ROWS = 16 * LM_RG;         // (token, head) rows a block
constexpr int LM_KEYS = 64;                 // keys a tile
constexpr int LM_PPITCH = LM_KEYS + 8;      // row pitch of P in shared memory (elements)
static_assert(LM_RG == 2 && LM_KEYS == 64, "the tile fetch deals four of 256 threads to each of 64 rows");

__device__ __forceinline__ void lm_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int NT>      // n-tiles of 8 channels a warp owns in O: C = 32 * NT
__global__ void __launch_bounds__(128 * LM_RG)
latent_attend_mma_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot,
                         const __nv_bfloat16* __restrict__ cache, float* __restrict__ part,
                         const int* __restrict__ tok_pos, const int* __restrict__ req_start,
                         const int* __restrict__ block_table, int bt_stride, int n_req, int T, int H, int R,
                         int page_size, int num_pages, int n_ranges, float scale, int* status) {
  constexpr int C = 32 * NT;
  extern __shared__ __align__(16) unsigned char lm_smem[];
  const int W = C + R, WP = W + 8;
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(lm_smem);              // [LM_ROWS][WP]
  __nv_bfloat16* sK0 = sQ + (size_t)LM_ROWS * WP;                              // [2][LM_KEYS][WP]: two tiles of keys
  __nv_bfloat16* sP = sK0 + (size_t)2 * LM_KEYS * WP;                          // [LM_ROWS][LM_PPITCH]
  float* sMax = reinterpret_cast<float*>(sP + (size_t)LM_ROWS * LM_PPITCH);    // [LM_RG][4][16]
  float* sSum = sMax + LM_RG * 4 * 16;                                         // [LM_RG][4][16]
  __shared__ long long sRow[2 * LM_KEYS];                                      // places of the two tiles' cache rows, -1: none
  __shared__ int s_item[3];                                                    // request row, first flattened row, found

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rg = warp >> 2, cg = warp & 3;
  const int range = blockIdx.y;
  if (tid == 0) {
    int acc = 0, found = 0;
    for (int r = 0; r < n_req; ++r) {
      const int rows = (req_start[r + 1] - req_start[r]) * H;
      const int tiles = (rows + LM_ROWS - 1) / LM_ROWS;
      if ((int)blockIdx.x < acc + tiles) { s_item[0] = r; s_item[1] = ((int)blockIdx.x - acc) * LM_ROWS; found = 1; break; }
      acc += tiles;
    }
    s_item[2] = found;
  }
  __syncthreads();
  if (!s_item[2]) return;
  const int req = s_item[0], row0 = s_item[1];
  const int t0 = req_start[req], n_rows = (req_start[req + 1] - t0) * H;
  const int rows_here = min(LM_ROWS, n_rows - row0);
  const int* bt = block_table + (size_t)req * bt_stride;
  // queries: latent part and rotated part side by side, times the score scale, bfloat16; rows past the end zero
  for (int i = warp; i < LM_ROWS; i += (int)(blockDim.x >> 5)) {
    __nv_bfloat16* dst = sQ + (size_t)i * WP;
    if (i < rows_here) {
      const int tok = t0 + (row0 + i) / H, head = (row0 + i) % H;
      const float* ql = q_lat + ((size_t)head * T + tok) * C;
      const float* qr = q_rot + ((size_t)tok * H + head) * R;
      for (int c = lane; c < C; c += 32) dst[c] = __float2bfloat16_rn(ql[c] * scale);
      for (int c = lane; c < R; c += 32) dst[C + c] = __float2bfloat16_rn(qr[c] * scale);
    } else {
      for (int c = lane; c < W; c += 32) dst[c] = __float2bfloat16_rn(0.f);
    }
  }
  // the two rows of this lane in its row group's MMA tiles: lane / 4 and lane / 4 + 8
  int my_pos[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int i = rg * 16 + (lane >> 2) + 8 * e;
    my_pos[e] = i < rows_here ? tok_pos[t0 + (row0 + i) / H] : -1;
  }
  const bool rg_active = rg * 16 < rows_here;
  const int last_pos = tok_pos[t0 + (row0 + rows_here - 1) / H];
  const int n_tiles = last_pos / LM_KEYS + 1;
  const int per = (n_tiles + n_ranges - 1) / n_ranges;
  const int tile_lo = range * per, tile_hi = min(n_tiles, tile_lo + per);

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  const int chunks = W / 8;                   // 16-byte pieces of a cache row

  // a tile's cache rows come in by asynchronous copies while the tile before is worked on: 64 threads look the
  // rows' places up (lookup), a barrier later four threads a row issue its 16-byte pieces (fetch)
  // lookup_ask reads the table entry of this thread's row of a tile (the load is not waited for), lookup_put
  // turns it into the row's place later, when the entry has long arrived
  auto lookup_ask = [&](int tile) -> int {
    const int key = tile * LM_KEYS + tid;
    return (tid < LM_KEYS && key <= last_pos) ? bt[key / page_size] : -2;
  };
  auto lookup_put = [&](int tile, int buf, int page) {
    if (tid < LM_KEYS) {
      long long off = -1;
      const int key = tile * LM_KEYS + tid;
      if (page != -2) {
        if (page < 0 || page >= num_pages) qb_set_status(status, QB_STATUS_BAD_PAGE, page, 3);
        else off = ((long long)page * page_size + key % page_size) * W;
      }
      sRow[buf * LM_KEYS + tid] = off;
    }
  };
  auto fetch = [&](int buf) {
    const int key_in = tid >> 2;              // 256 threads: four a row
    const long long off = sRow[buf * LM_KEYS + key_in];
    __nv_bfloat16* dst = sK0 + ((size_t)buf * LM_KEYS + key_in) * WP;
    if (off >= 0) {
      const __nv_bfloat16* src = cache + off;
      for (int c = tid & 3; c < chunks; c += 4) {
        const unsigned d = (unsigned)__cvta_generic_to_shared(dst + c * 8);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + c * 8) : "memory");
      }
    } else {
      for (int c = tid & 3; c < chunks; c += 4) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // the first two tiles are asked for at once; after that tile i + 1 is asked for as soon as tile i has landed
  // (its buffer was read last by tile i - 1), its rows' places having been looked up during tile i - 1
  if (tile_lo < tile_hi) {
    lookup_put(tile_lo, 0, lookup_ask(tile_lo));
    if (tile_lo + 1 < tile_hi) lookup_put(tile_lo + 1, 1, lookup_ask(tile_lo + 1));
    __syncthreads();
    fetch(0);
    if (tile_lo + 1 < tile_hi) fetch(1);
  }
  int buf = 0;
  for (int tile = tile_lo; tile < tile_hi; ++tile, buf ^= 1) {
    const int k0 = tile * LM_KEYS;
    if (tile == tile_lo && tile + 1 < tile_hi) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                          // this tile has landed; the tile before has been read (and sQ is written)
    if (tile > tile_lo && tile + 1 < tile_hi) fetch(buf ^ 1);
    const int page_ahead = tile + 2 < tile_hi ? lookup_ask(tile + 2) : -2;
    const __nv_bfloat16* sK = sK0 + (size_t)buf * LM_KEYS * WP;

    // S = Q K^T for this warp's 16 keys: the fragments of the next 16 channels are asked for before the MMAs of
    // these, and even and odd steps add into accumulators of their own (two chains of MMAs instead of one)
    float s[2][4];
    {
      float acc[2][2][4];
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int y = 0; y < 2; ++y) { acc[x][y][0] = acc[x][y][1] = acc[x][y][2] = acc[x][y][3] = 0.f; }
      const __nv_bfloat16* qa = sQ + (size_t)(rg * 16 + (lane & 15)) * WP + (lane >> 4) * 8;
      const __nv_bfloat16* kb = sK + (size_t)(cg * 16 + (lane & 7) + (lane >> 4) * 8) * WP + ((lane >> 3) & 1) * 8;
      uint32_t a0[4], b0[4], a1[4], b1[4];
      lm_ldmatrix_x4(a0, qa);
      lm_ldmatrix_x4(b0, kb);
      int kk = rg_active ? 0 : W;             // a row group without rows (a single token of few heads) skips the MMAs
      for (; kk + 32 <= W; kk += 32) {
        lm_ldmatrix_x4(a1, qa + kk + 16);
        lm_ldmatrix_x4(b1, kb + kk + 16);
        lm_mma(acc[0][0], a0, b0[0], b0[1]);
        lm_mma(acc[0][1], a0, b0[2], b0[3]);
        if (kk + 32 < W) {
          lm_ldmatrix_x4(a0, qa + kk + 32);
          lm_ldmatrix_x4(b0, kb + kk + 32);
        }
        lm_mma(acc[1][0], a1, b1[0], b1[1]);
        lm_mma(acc[1][1], a1, b1[2], b1[3]);
      }
      if (kk < W) {                           // an odd number of steps: the last fragments are in a0, b0
        lm_mma(acc[0][0], a0, b0[0], b0[1]);
        lm_mma(acc[0][1], a0, b0[2], b0[3]);
      }
#pragma unroll
      for (int y = 0; y < 2; ++y)
#pragma unroll
        for (int v = 0; v < 4; ++v) s[y][v] = acc[0][y][v] + acc[1][y][v];
    }
    // causal mask, row maxima over this warp's keys
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const int key_in = cg * 16 + nt * 8 + (lane & 3) * 2 + (v & 1);
        const int e = v >> 1;
        const bool ok = k0 + key_in <= my_pos[e];
        s[nt][v] = ok ? s[nt][v] : -INFINITY;
        mx[e] = fmaxf(mx[e], s[nt][v]);
      }
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
      mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
      if ((lane & 3) == 0) sMax[(rg * 4 + cg) * 16 + (lane >> 2) + 8 * e] = mx[e];
    }
    __syncthreads();
    float corr[2], ps[2] = {0.f, 0.f};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int row = (lane >> 2) + 8 * e;
      float m_new = m[e];
#pragma unroll
      for (int g = 0; g < 4; ++g) m_new = fmaxf(m_new, sMax[(rg * 4 + g) * 16 + row]);
      corr[e] = (m_new == -INFINITY) ? 1.f : expf(m[e] - m_new);
      m[e] = m_new;
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float p0 = s[nt][2 * e] == -INFINITY ? 0.f : expf(s[nt][2 * e] - m[e]);
        const float p1 = s[nt][2 * e + 1] == -INFINITY ? 0.f : expf(s[nt][2 * e + 1] - m[e]);
        ps[e] += p0 + p1;
        const int row = rg * 16 + (lane >> 2) + 8 * e;
        *reinterpret_cast<__nv_bfloat162*>(sP + (size_t)row * LM_PPITCH + cg * 16 + nt * 8 + (lane & 3) * 2) =
            __floats2bfloat162_rn(p0, p1);
      }
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      ps[e] += __shfl_xor_sync(0xffffffffu, ps[e], 1);
      ps[e] += __shfl_xor_sync(0xffffffffu, ps[e], 2);
      if ((lane & 3) == 0) sSum[(rg * 4 + cg) * 16 + (lane >> 2) + 8 * e] = ps[e];
    }
    __syncthreads();
    if (tile + 2 < tile_hi) lookup_put(tile + 2, buf, page_ahead);   // this tile's places were used when it was asked for
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int row = (lane >> 2) + 8 * e;
      float add = 0.f;
#pragma unroll
      for (int g = 0; g < 4; ++g) add += sSum[(rg * 4 + g) * 16 + row];
      l[e] = l[e] * corr[e] + add;
    }
    // O += P V for this warp's quarter of the channels
#pragma unroll
    for (int n = 0; n < NT; ++n) { o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1]; }
    if (rg_active) {
      const __nv_bfloat16* pa = sP + (size_t)(rg * 16 + (lane & 15)) * LM_PPITCH + (lane >> 4) * 8;
      const __nv_bfloat16* vb = sK + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * WP + cg * (C / 4) + (lane >> 4) * 8;
#pragma unroll
      for (int kk = 0; kk < LM_KEYS; kk += 16) {
        uint32_t a[4];
        lm_ldmatrix_x4(a, pa + kk);
#pragma unroll
        for (int n = 0; n < NT; n += 4) {     // the fragments of four channel tiles are asked for before their MMAs
          uint32_t b0[4], b1[4];
          lm_ldmatrix_x4_trans(b0, vb + (size_t)kk * WP + n * 8);
          if (n + 2 < NT) lm_ldmatrix_x4_trans(b1, vb + (size_t)kk * WP + (n + 2) * 8);
          lm_mma(o[n], a, b0[0], b0[1]);
          lm_mma(o[n + 1], a, b0[2], b0[3]);
          if (n + 2 < NT) {
            lm_mma(o[n + 2], a, b1[0], b1[1]);
            lm_mma(o[n + 3], a, b1[2], b1[3]);
          }
        }
      }
    }
  }
  // partial results of this range
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int i = rg * 16 + (lane >> 2) + 8 * e;
    if (i >= rows_here) continue;
    const int tok = t0 + (row0 + i) / H, head = (row0 + i) % H;
    float* dst = part + (((size_t)tok * H + head) * n_ranges + range) * (C + 2);
    if (cg == 0 && (lane & 3) == 0) { dst[0] = m[e]; dst[1] = l[e]; }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const int ch = cg * (C / 4) + n * 8 + (lane & 3) * 2;
      dst[2 + ch] = o[n][2 * e];
      dst[2 + ch + 1] = o[n][2 * e + 1];
    }
  }
}

extern "C" int qb_latent_attend_mma_supported(int C, int R) {
  return (C == 64 || C == 128 || C == 256 || C == 512) && R >= 0 && R % 16 == 0;
}

// max_tiles: an upper bound on the row tiles of the step: sum over requests of ceil(tokens * H / 32)
extern "C" int qb_latent_attend_mma(const float* q_lat, const float* q_rot, const void* cache, float* part,
                                    const int* tok_pos, const int* req_start, const int* block_table,
                                    int bt_stride, int n_req, int T, int H, int C, int R, int page_size,
                                    int num_pages, int n_ranges, int max_tiles, float scale, int* status,
                                    cudaStream_t stream) {
  if (T <= 0 || n_req <= 0) return 0;
  if (!qb_latent_attend_mma_supported(C, R) || n_ranges < 1 || page_size <= 0) return QB_ERR_UNSUPPORTED;
  const int W = C + R, WP = W + 8;
  const size_t smem = ((size_t)(LM_ROWS + 2 * LM_KEYS) * WP + (size_t)LM_ROWS * LM_PPITCH) * 2 + 2 * LM_RG * 4 * 16 * 4;
  if (smem > 220 * 1024) return QB_ERR_UNSUPPORTED;
  dim3 grid(max_tiles, n_ranges);
#define LM_LAUNCH(N)                                                                                        \
  do {                                                                                                      \
    auto kern = latent_attend_mma_kernel<N>;                                                                \
    if (smem + 2048 > 48 * 1024) {   /* the kernel also has some static shared memory */                                                                                 \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      if (e != cudaSuccess) return (int)e;                                                                  \
    }                                                                                                       \
    kern<<<grid, 128 * LM_RG, smem, stream>>>(q_lat, q_rot, (const __nv_bfloat16*)cache, part, tok_pos,    \
                                              req_start, block_table, bt_stride, n_req, T, H, R, page_size, \
                                              num_pages, n_ranges, scale, status);                          \
  } while (0)
  if (C == 64) LM_LAUNCH(2);
  else if (C == 128) LM_LAUNCH(4);
  else if (C == 256) LM_LAUNCH(8);
  else LM_LAUNCH(16);
#undef LM_LAUNCH
  QB_LAUNCH_CHECK();
  return 0;
}
