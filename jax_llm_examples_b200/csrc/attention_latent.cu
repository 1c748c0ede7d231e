// Attention whose keys and values are up-projections of one cached latent per token, with a rotated key part
// shared by all heads and a per-head sink in the softmax's denominator.  32-bit scores, softmax and sums;
// the cache is 32-bit or bfloat16.
//
// The cache holds, per token, ONE row [c (rank) | k_rot (dr)] (pages: [P, 1, 1, page_size, rank + dr]).  The kernels
// work in the latent space (the up-projections are absorbed into the query and applied to the output by the
// caller, as per-head products):
//   score(t, s, h) = (q_lat[h, t] . c_s + q_rot[t, h] . k_rot_s) * scale          q_lat = W_uk[h]^T q_nope
//   p = exp(score - m) / (sum_s exp(score - m) + exp(sink_h - m))                  causal: s <= t
//   out_lat[h, t] = sum_s p_s c_s                                                  (value = W_uv[h] out_lat)
//
// latent_kv_prep   from the projected row [dq (q_rank) | dkv (rank) | k_rot (dr)]: weighted RMS norms of the two
//                  latents, the rotation of k_rot, and the page write, in one kernel.
// latent_q_prep    from the projected queries [H, dn + dr]: the unrotated parts head-major (for the per-head
//                  products) and the rotated parts, rotated.
// Rotation: pairs (2i, 2i+1), i < dims/2, by the angle position * inv_freq[i] in 32-bit; entries from `dims` on pass.
#include "common.cuh"

__device__ __forceinline__ float row_sum_splits(const float* p, int splits, long long stride) {
  float s = 0.f;
  for (int z = 0; z < splits; ++z) s += p[(size_t)z * stride];
  return s;
}

template <typename TO>
__global__ void latent_kv_prep_kernel(const float* __restrict__ proj, int splits, long long split_stride,
                                      const float* __restrict__ q_norm_w, const float* __restrict__ kv_norm_w, float eps,
                                      const float* __restrict__ inv_freq, int rot_dims, TO* __restrict__ cq, TO* __restrict__ pages,
                                      const int* __restrict__ block_table, int bt_stride, const int* __restrict__ req_of_token,
                                      const int* __restrict__ positions, int q_rank, int rank, int dr, int page_size,
                                      int num_pages, int* status) {
  JLX_TL(TL_ROPE);
  pdl_launch_dependents_if_small();
  pdl_wait();
  __shared__ float scratch[33];
  const int n = blockIdx.x;
  const int C = q_rank + rank + dr;
  const float* row = proj + (size_t)n * C;
  // the query's latent
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float v = row_sum_splits(row + i, splits, split_stride);
    ss = fmaf(v, v, ss);
  }
  float rms = sqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[(size_t)n * q_rank + i] = from_f32<TO>(row_sum_splits(row + i, splits, split_stride) / rms * q_norm_w[i]);
  if (!pages) return;
  const int p = positions[n], r = req_of_token[n];
  const int page = block_table[(size_t)r * bt_stride + p / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, JLX_STATUS_BAD_PAGE);
    return;
  }
  TO* dst = pages + ((size_t)page * page_size + p % page_size) * (rank + dr);
  // the keys' and values' latent
  ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = row_sum_splits(row + q_rank + i, splits, split_stride);
    ss = fmaf(v, v, ss);
  }
  rms = sqrtf(block_sum(ss, scratch) / (float)rank + eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x)
    dst[i] = from_f32<TO>(row_sum_splits(row + q_rank + i, splits, split_stride) / rms * kv_norm_w[i]);
  // the shared rotated key part
  const float* kr = row + q_rank + rank;
  for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
    float sn, cs;
    sincosf((float)p * inv_freq[i], &sn, &cs);
    const float u = row_sum_splits(kr + 2 * i, splits, split_stride), v = row_sum_splits(kr + 2 * i + 1, splits, split_stride);
    dst[rank + 2 * i] = from_f32<TO>(u * cs - v * sn);
    dst[rank + 2 * i + 1] = from_f32<TO>(v * cs + u * sn);
  }
  for (int i = rot_dims + threadIdx.x; i < dr; i += blockDim.x) dst[rank + i] = from_f32<TO>(row_sum_splits(kr + i, splits, split_stride));
}

JLX_API int jlx_latent_kv_prep(const float* proj, int splits, long long split_stride, const float* q_norm_w,
                               const float* kv_norm_w, float eps, const float* inv_freq, int rot_dims, void* cq, void* pages,
                               int dtype, const int* block_table, int bt_stride, const int* req_of_token, const int* positions,
                               int N, int q_rank, int rank, int dr, int page_size, int num_pages, int* status,
                               cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && q_rank > 0 && rank > 0 && dr >= 0 && splits >= 1, "latent_kv_prep: bad sizes");
  JLX_REQUIRE(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0, "latent_kv_prep: %d rotated entries of %d", rot_dims, dr);
  JLX_REQUIRE(eps > 0.f, "latent_kv_prep: eps must be positive");
  if (N == 0) return 0;
  JLX_DISPATCH_DTYPE(dtype, TO, {
    JLX_CUDA(jlx_launch_pdl(latent_kv_prep_kernel<TO>, dim3(N), dim3(128), 0, stream, proj, splits, split_stride, q_norm_w, kv_norm_w,
                            eps, inv_freq, rot_dims, (TO*)cq, (TO*)pages, block_table, bt_stride, req_of_token, positions, q_rank,
                            rank, dr, page_size, num_pages, status));
  });
  JLX_LAUNCH_CHECK("latent_kv_prep");
  return 0;
}

// q: float32 [N, H, dn + dr] (or partials).  q_nope: [H, N, dn] in the activation type; q_rot: float32 [N, H, dr];
// q_full (optional): [H, N, dn + dr] in the activation type, the rotated part rotated (for per-head score products).
template <typename TO>
__global__ void latent_q_prep_kernel(const float* __restrict__ q, int splits, long long split_stride,
                                     const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions,
                                     TO* __restrict__ q_nope, float* __restrict__ q_rot, TO* __restrict__ q_full, int N, int H,
                                     int dn, int dr) {
  JLX_TL(TL_ROPE);
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int n = blockIdx.x, h = blockIdx.y;
  const float* row = q + ((size_t)n * H + h) * (dn + dr);
  TO* full = q_full ? q_full + ((size_t)h * N + n) * (dn + dr) : nullptr;
  for (int i = threadIdx.x; i < dn; i += blockDim.x) {
    const TO v = from_f32<TO>(row_sum_splits(row + i, splits, split_stride));
    q_nope[((size_t)h * N + n) * dn + i] = v;
    if (full) full[i] = v;
  }
  const float* qr = row + dn;
  float* dst = q_rot + ((size_t)n * H + h) * dr;
  const int p = positions[n];
  for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
    float sn, cs;
    sincosf((float)p * inv_freq[i], &sn, &cs);
    const float u = row_sum_splits(qr + 2 * i, splits, split_stride), v = row_sum_splits(qr + 2 * i + 1, splits, split_stride);
    const float a = u * cs - v * sn, b = v * cs + u * sn;
    dst[2 * i] = a;
    dst[2 * i + 1] = b;
    if (full) { full[dn + 2 * i] = from_f32<TO>(a); full[dn + 2 * i + 1] = from_f32<TO>(b); }
  }
  for (int i = rot_dims + threadIdx.x; i < dr; i += blockDim.x) {
    const float v = row_sum_splits(qr + i, splits, split_stride);
    dst[i] = v;
    if (full) full[dn + i] = from_f32<TO>(v);
  }
}

JLX_API int jlx_latent_q_prep(const float* q, int splits, long long split_stride, const float* inv_freq, int rot_dims,
                              const int* positions, void* q_nope, int dtype, float* q_rot, void* q_full, int N, int H, int dn,
                              int dr, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && H > 0 && dn > 0 && dr >= 0 && splits >= 1, "latent_q_prep: bad sizes");
  JLX_REQUIRE(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0, "latent_q_prep: %d rotated entries of %d", rot_dims, dr);
  JLX_REQUIRE(H <= 65535, "latent_q_prep: too many heads (%d)", H);
  if (N == 0) return 0;
  JLX_DISPATCH_DTYPE(dtype, TO, {
    JLX_CUDA(jlx_launch_pdl(latent_q_prep_kernel<TO>, dim3(N, H), dim3(64), 0, stream, q, splits, split_stride, inv_freq, rot_dims,
                            positions, (TO*)q_nope, q_rot, (TO*)q_full, N, H, dn, dr));
  });
  JLX_LAUNCH_CHECK("latent_q_prep");
  return 0;
}

// ------------------------------------------------------------------------------------------------ attention
// One block serves one query token and up to LAT_WARPS * HPW heads; a warp takes HPW heads, a lane one key of the tile for
// the scores and a slice of the latent for the weighted sums, so that every value read from shared memory serves HPW
// products.  All heads share each tile of keys.  Key tiles are aligned to absolute positions (0, 32, 64, ...), so the
// order of a position's sums depends on the position alone.  The sink opens the running maximum and denominator:
// m = sink, l = exp(sink - m) = 1.
// With `rows` the block serves token rows[blockIdx.x] (the single decoded tokens of a step that also holds prompt
// portions).  With splits > 1 block z takes the keys [z * split_keys, (z + 1) * split_keys) (a multiple of the tile, so
// tiles stay aligned) and leaves (m, l, unnormalised sums) for the combine kernel; the sink opens split 0.
#define LAT_TILE 32
#define LAT_WARPS 8
#define LAT_MAX_R32 32  // latent size up to 1024

template <typename TC, typename TO, int HPW, int R32>
__global__ void attention_latent_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot,
                                        const TC* __restrict__ pages, const int* __restrict__ block_table, int bt_stride,
                                        const int* __restrict__ req_of_token, const int* __restrict__ positions,
                                        const float* __restrict__ sink, TO* __restrict__ out_lat, int N, int H, int rank,
                                        int dr, int page_size, int num_pages, float scale, const int* __restrict__ rows,
                                        int splits, int split_keys, float* __restrict__ part_acc, float* __restrict__ part_ml,
                                        int ldk, int* status) {
  JLX_TL(TL_ATTN_GENERIC);
  pdl_launch_dependents_if_small();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  __shared__ long long row_at[LAT_TILE];  // row number of each key of the tile in the pool, -1: a bad page
  const int dk = rank + dr;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  float* qs = smem;                     // [nwarp * HPW][dk]
  float* ks = qs + nwarp * HPW * dk;    // [LAT_TILE][ldk]
  const int n = rows ? rows[blockIdx.x] : blockIdx.x;
  const int h0 = (blockIdx.y * nwarp + warp) * HPW;  // the warp's first head
  const int z = blockIdx.z;
  const int p = positions[n], r = req_of_token[n];
  for (int u = 0; u < HPW; ++u) {  // heads beyond H get a zero query: they run along and write nothing
    const int h = h0 + u;
    float* q = qs + (warp * HPW + u) * dk;
    for (int d = lane; d < rank; d += 32) q[d] = h < H ? q_lat[((size_t)h * N + n) * rank + d] : 0.f;
    for (int d = lane; d < dr; d += 32) q[rank + d] = h < H ? q_rot[((size_t)n * H + h) * dr + d] : 0.f;
  }
  const bool has_sink = sink != nullptr && z == 0;
  float m[HPW], l[HPW], acc[HPW][R32];
#pragma unroll
  for (int u = 0; u < HPW; ++u) {
    m[u] = (has_sink && h0 + u < H) ? sink[h0 + u] : -INFINITY;
    l[u] = has_sink ? 1.f : 0.f;
#pragma unroll
    for (int i = 0; i < R32; ++i) acc[u][i] = 0.f;
  }
  const int nd = (rank + 31) >> 5;
  const int t_begin = splits > 1 ? z * split_keys : 0;
  const int t_end = splits > 1 ? min(p, (z + 1) * split_keys - 1) : p;  // last key of this block

  // 16-byte loads of the cached rows where their size and the pool's address allow
  constexpr int VEC = 16 / (int)sizeof(TC);
  const bool wide = (dk % VEC) == 0 && ((uintptr_t)pages & 15) == 0;
  const bool quads = (dk & 3) == 0 && (ldk & 3) == 0;  // scores with 16-byte reads of shared memory
  bool bad_page = false;
  for (int t0 = t_begin; t0 <= t_end; t0 += LAT_TILE) {
    __syncthreads();  // the previous tile is consumed; qs is visible
    const int cnt = min(LAT_TILE, t_end - t0 + 1);
    if (threadIdx.x < cnt) {  // where the tile's rows lie
      const int pos = t0 + threadIdx.x;
      int page = block_table[(size_t)r * bt_stride + pos / page_size];
      if (page < 0 || page >= num_pages) { bad_page = true; page = -1; }
      row_at[threadIdx.x] = page < 0 ? -1 : (long long)page * page_size + pos % page_size;
    }
    __syncthreads();
    if (wide) {
      const int chunks = dk / VEC;
#pragma unroll 4
      for (int idx = threadIdx.x; idx < cnt * chunks; idx += blockDim.x) {
        const int j = idx / chunks, ch = idx - j * chunks;
        const long long at = row_at[j];
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (at >= 0) raw = *reinterpret_cast<const uint4*>(pages + (size_t)at * dk + ch * VEC);
        const TC* e = reinterpret_cast<const TC*>(&raw);
        float* dst = ks + j * ldk + ch * VEC;
#pragma unroll
        for (int u = 0; u < VEC; ++u) dst[u] = to_f32<TC>(e[u]);
      }
    } else {
      for (int idx = threadIdx.x; idx < cnt * dk; idx += blockDim.x) {
        const int j = idx / dk, d = idx - j * dk;
        const long long at = row_at[j];
        ks[j * ldk + d] = at >= 0 ? to_f32<TC>(pages[(size_t)at * dk + d]) : 0.f;
      }
    }
    __syncthreads();
    float sc[HPW];
#pragma unroll
    for (int u = 0; u < HPW; ++u) sc[u] = -INFINITY;
    if (lane < cnt) {
      float dot[HPW];
#pragma unroll
      for (int u = 0; u < HPW; ++u) dot[u] = 0.f;
      const float* kr = ks + lane * ldk;
      const float* qr = qs + warp * HPW * dk;
      if (quads) {
        for (int d = 0; d < dk; d += 4) {
          const float4 kv = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
          for (int u = 0; u < HPW; ++u) {
            const float4 qv = *reinterpret_cast<const float4*>(qr + u * dk + d);
            dot[u] = fmaf(qv.x, kv.x, dot[u]);
            dot[u] = fmaf(qv.y, kv.y, dot[u]);
            dot[u] = fmaf(qv.z, kv.z, dot[u]);
            dot[u] = fmaf(qv.w, kv.w, dot[u]);
          }
        }
      } else {
        for (int d = 0; d < dk; ++d) {
          const float kv = kr[d];
#pragma unroll
          for (int u = 0; u < HPW; ++u) dot[u] = fmaf(qr[u * dk + d], kv, dot[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < HPW; ++u) sc[u] = dot[u] * scale;
    }
    float pj[HPW];
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
      const float m_new = fmaxf(m[u], warp_max(sc[u]));
      const float corr = expf(m[u] - m_new);  // without a sink m is -inf on the first tile: exp(-inf) = 0
      pj[u] = lane < cnt ? expf(sc[u] - m_new) : 0.f;
      l[u] = l[u] * corr + warp_sum(pj[u]);
      m[u] = m_new;
#pragma unroll
      for (int i = 0; i < R32; ++i) acc[u][i] *= corr;
    }
    for (int j = 0; j < cnt; ++j) {  // key by key: the lane's entries of the latent are independent sums
      float pv[HPW];
#pragma unroll
      for (int u = 0; u < HPW; ++u) pv[u] = __shfl_sync(0xffffffffu, pj[u], j);
      const float* kj = ks + j * ldk + lane;
#pragma unroll
      for (int i = 0; i < R32; ++i) {
        if (i < nd && lane + 32 * i < rank) {
          const float kv = kj[32 * i];
#pragma unroll
          for (int u = 0; u < HPW; ++u) acc[u][i] = fmaf(pv[u], kv, acc[u][i]);
        }
      }
    }
  }
  if (bad_page) atomicOr(status, JLX_STATUS_BAD_PAGE);
#pragma unroll
  for (int u = 0; u < HPW; ++u) {
    const int h = h0 + u;
    if (h >= H) continue;
    if (splits > 1) {
      const size_t slot = ((size_t)blockIdx.x * H + h) * splits + z;
      if (lane == 0) { part_ml[2 * slot] = m[u]; part_ml[2 * slot + 1] = l[u]; }
#pragma unroll
      for (int i = 0; i < R32; ++i) {
        const int d = lane + 32 * i;
        if (i < nd && d < rank) part_acc[slot * rank + d] = acc[u][i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < R32; ++i) {
        const int d = lane + 32 * i;
        if (i < nd && d < rank) out_lat[((size_t)h * N + n) * rank + d] = from_f32<TO>(acc[u][i] / l[u]);
      }
    }
  }
}

// out = sum_z acc_z exp(m_z - m) / sum_z l_z exp(m_z - m), m = max_z m_z, the splits in ascending order.
template <typename TO>
__global__ void attention_latent_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                                TO* __restrict__ out_lat, const int* __restrict__ rows, int N, int H, int rank,
                                                int splits) {
  JLX_TL(TL_ATTN_COMBINE);
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int n = rows ? rows[b] : b;
  const size_t slot0 = ((size_t)b * H + h) * splits;
  float m = -INFINITY;
  for (int z = 0; z < splits; ++z) m = fmaxf(m, part_ml[2 * (slot0 + z)]);
  float l = 0.f;
  for (int z = 0; z < splits; ++z) {
    const float mz = part_ml[2 * (slot0 + z)];
    if (mz > -INFINITY) l += part_ml[2 * (slot0 + z) + 1] * expf(mz - m);
  }
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float a = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float mz = part_ml[2 * (slot0 + z)];
      if (mz > -INFINITY) a = fmaf(part_acc[(slot0 + z) * rank + d], expf(mz - m), a);
    }
    out_lat[((size_t)h * N + n) * rank + d] = from_f32<TO>(a / l);
  }
}

// rows / n_rows: serve these token rows only (N stays the row count of q and out).  splits > 1: part_acc float32
// [n_rows * H * splits * rank], part_ml float32 [n_rows * H * splits * 2].
JLX_API int jlx_attention_latent(const float* q_lat, const float* q_rot, const void* pages, int cache_dtype,
                                 const int* block_table, int bt_stride, const int* req_of_token, const int* positions,
                                 const float* sink, void* out_lat, int out_dtype, int N, int H, int rank, int dr,
                                 int page_size, int num_pages, float scale, const int* rows, int n_rows, int splits,
                                 int split_keys, float* part_acc, float* part_ml, int* status, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && H > 0 && rank > 0 && dr >= 0 && page_size > 0 && num_pages > 0, "attention_latent: bad sizes");
  JLX_REQUIRE(rank <= 32 * LAT_MAX_R32, "attention_latent: latent size %d is above the supported maximum %d", rank, 32 * LAT_MAX_R32);
  JLX_REQUIRE(splits >= 1 && splits <= 65535, "attention_latent: bad split count %d", splits);
  JLX_REQUIRE(splits == 1 || (split_keys > 0 && split_keys % LAT_TILE == 0 && part_acc && part_ml),
              "attention_latent: splits need a key count that is a multiple of %d, and scratch", LAT_TILE);
  const int served = rows ? n_rows : N;
  if (served == 0) return 0;
  const int dk = rank + dr;
  // a key's row in shared memory: padded so that 16-byte reads of a quarter warp's rows fall into different banks
  // (rows a multiple of 4 floats apart with an odd count of 16-byte pieces), else by one float
  const int ldk = (dk & 3) == 0 ? (((dk >> 2) & 1) ? dk : dk + 4) : dk + 1;
  const bool big = rank > 512;             // latents above 512: two heads per warp, else four
  const int hpw = big ? 2 : 4;
  const int groups = (H + hpw - 1) / hpw;  // warps' worth of heads
  int nwarp = groups < LAT_WARPS ? groups : LAT_WARPS;
  auto smem_for = [&](int warps) { return sizeof(float) * ((size_t)warps * hpw * dk + (size_t)LAT_TILE * ldk); };
  while (nwarp > 1 && smem_for(nwarp) > 200 * 1024) nwarp >>= 1;  // fewer heads per block where the rows are long
  const size_t smem = smem_for(nwarp);
  JLX_REQUIRE(smem <= 200 * 1024, "attention_latent: a key tile of %d x %d does not fit into shared memory", LAT_TILE, dk);
  const int hb = (groups + nwarp - 1) / nwarp;
  JLX_REQUIRE(hb <= 65535 && H <= 65535, "attention_latent: too many heads (%d)", H);
#define LAT_GO(HPW, R32)                                                                                                   \
  do {                                                                                                                     \
    if (smem > 48 * 1024)                                                                                                  \
      JLX_CUDA(cudaFuncSetAttribute(attention_latent_kernel<TC, TO, HPW, R32>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                    (int)smem));                                                                           \
    JLX_CUDA(jlx_launch_pdl(attention_latent_kernel<TC, TO, HPW, R32>, dim3(served, hb, splits), dim3(nwarp * 32), smem, stream, \
                            q_lat, q_rot, (const TC*)pages, block_table, bt_stride, req_of_token, positions, sink, (TO*)out_lat, \
                            N, H, rank, dr, page_size, num_pages, scale, rows, splits, split_keys, part_acc, part_ml, ldk,  \
                            status));                                                                                      \
  } while (0)
  JLX_DISPATCH_DTYPE(cache_dtype, TC, JLX_DISPATCH_DTYPE(out_dtype, TO, {
    if (big) LAT_GO(2, 32);
    else LAT_GO(4, 16);
  }));
#undef LAT_GO
  JLX_LAUNCH_CHECK("attention_latent");
  if (splits > 1) {
    JLX_DISPATCH_DTYPE(out_dtype, TO, {
      JLX_CUDA(jlx_launch_pdl(attention_latent_combine_kernel<TO>, dim3(served, H), dim3(128), 0, stream, (const float*)part_acc,
                              (const float*)part_ml, (TO*)out_lat, rows, N, H, rank, splits));
    });
    JLX_LAUNCH_CHECK("attention_latent_combine");
  }
  return 0;
}

// ------------------------------------------------------------------------------------------------ prompt portions
// For a prompt portion the scores and the weighted sums are per-head matrix products on the tensor cores (the caller's,
// from the library), around three kernels of this file: the request's cached rows gathered into two dense matrices,
// the keys put together per head, and the softmax with its causal edge and its sink.

// c[t, :] = cache row t's first `rank` entries, kr[t, :] = its last dr, t < L, for the request of block-table row r.
template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ pages, const int* __restrict__ bt_row, T* __restrict__ c,
                                     T* __restrict__ kr, int rank, int dr, int page_size, int num_pages, int* status) {
  JLX_TL(TL_OTHER);
  const int t = blockIdx.x;
  const int page = bt_row[t / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, JLX_STATUS_BAD_PAGE);
    return;
  }
  const T* src = pages + ((size_t)page * page_size + t % page_size) * (rank + dr);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) c[(size_t)t * rank + i] = src[i];
  for (int i = threadIdx.x; i < dr; i += blockDim.x) kr[(size_t)t * dr + i] = src[rank + i];
}

JLX_API int jlx_latent_gather(const void* pages, int dtype, const int* bt_row, void* c, void* kr, int L, int rank, int dr,
                              int page_size, int num_pages, int* status, cudaStream_t stream) {
  JLX_REQUIRE(L >= 0 && rank > 0 && dr >= 0 && page_size > 0, "latent_gather: bad sizes");
  if (L == 0) return 0;
  JLX_DISPATCH_DTYPE(dtype, T, {
    latent_gather_kernel<T><<<L, 128, 0, stream>>>((const T*)pages, bt_row, (T*)c, (T*)kr, rank, dr, page_size, num_pages, status);
  });
  JLX_LAUNCH_CHECK("latent_gather");
  return 0;
}

// k[h, t, :] = [kv_up[t, h * dn .. (h + 1) * dn) | kr[t, :]]: every head's key with the shared rotated part appended.
template <typename T>
__global__ void latent_key_assemble_kernel(const T* __restrict__ kv_up, long long ld_up, const T* __restrict__ kr,
                                           T* __restrict__ k, int L, int H, int dn, int dr) {
  JLX_TL(TL_OTHER);
  const int t = blockIdx.x, d = dn + dr;
  for (int i = threadIdx.x; i < H * d; i += blockDim.x) {
    const int h = i / d, e = i - h * d;
    k[((size_t)h * L + t) * d + e] = e < dn ? kv_up[(size_t)t * ld_up + h * dn + e] : kr[(size_t)t * dr + (e - dn)];
  }
}

JLX_API int jlx_latent_key_assemble(const void* kv_up, long long ld_up, const void* kr, void* k, int dtype, int L, int H,
                                    int dn, int dr, cudaStream_t stream) {
  JLX_REQUIRE(L >= 0 && H > 0 && dn > 0 && dr >= 0 && ld_up >= (long long)H * dn, "latent_key_assemble: bad sizes");
  if (L == 0) return 0;
  JLX_DISPATCH_DTYPE(dtype, T, {
    latent_key_assemble_kernel<T><<<L, 256, 0, stream>>>((const T*)kv_up, ld_up, (const T*)kr, (T*)k, L, H, dn, dr);
  });
  JLX_LAUNCH_CHECK("latent_key_assemble");
  return 0;
}

// p[h, i, j] = exp(scale * s[h, i, j] - m) / (sum over visible j + exp(sink_h - m)) for j <= q_start + i, else 0.
// s: float32 [H, T, L]; p: [H, T, L] in the activations' type.  One block per (query row, head); 32-bit throughout.
// With `staged` the visible part of the row is read once into shared memory (L floats) and the three passes run there.
template <typename TO>
__global__ void causal_sink_softmax_kernel(const float* __restrict__ s, const float* __restrict__ sink, float scale,
                                           int q_start, TO* __restrict__ p, int T, int L, int staged) {
  JLX_TL(TL_OTHER);
  extern __shared__ __align__(16) float stage[];
  __shared__ float scratch[33];
  const int i = blockIdx.x, h = blockIdx.y;
  const float* row = s + ((size_t)h * T + i) * L;
  TO* out = p + ((size_t)h * T + i) * L;
  const int visible = min(L, q_start + i + 1);
  float m = sink ? sink[h] : -INFINITY;
  if (staged) {
    if ((L & 3) == 0) {  // rows start on 16-byte boundaries
      for (int j = threadIdx.x * 4; j < visible; j += blockDim.x * 4) {
        float4 v = *reinterpret_cast<const float4*>(row + j);
        v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
        *reinterpret_cast<float4*>(stage + j) = v;
        m = fmaxf(m, v.x);
        if (j + 1 < visible) m = fmaxf(m, v.y);
        if (j + 2 < visible) m = fmaxf(m, v.z);
        if (j + 3 < visible) m = fmaxf(m, v.w);
      }
    } else {
      for (int j = threadIdx.x; j < visible; j += blockDim.x) { stage[j] = row[j] * scale; m = fmaxf(m, stage[j]); }
    }
    row = stage;
    scale = 1.f;
  } else {
    for (int j = threadIdx.x; j < visible; j += blockDim.x) m = fmaxf(m, row[j] * scale);
  }
  // the block's maximum: warp maxima, then every thread takes the largest
  m = warp_max(m);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
  __syncthreads();
  m = scratch[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w) m = fmaxf(m, scratch[w]);
  float l = 0.f;
  for (int j = threadIdx.x; j < visible; j += blockDim.x) l += expf(row[j] * scale - m);
  l = block_sum(l, scratch) + (sink ? expf(sink[h] - m) : 0.f);
  for (int j = threadIdx.x; j < L; j += blockDim.x) out[j] = from_f32<TO>(j < visible ? expf(row[j] * scale - m) / l : 0.f);
}

JLX_API int jlx_causal_sink_softmax(const float* s, const float* sink, float scale, int q_start, void* p, int dtype, int H,
                                    int T, int L, cudaStream_t stream) {
  JLX_REQUIRE(H > 0 && T >= 0 && L > 0 && q_start >= 0 && H <= 65535, "causal_sink_softmax: bad sizes");
  if (T == 0) return 0;
  const int staged = (size_t)L * 4 <= 160 * 1024;
  const size_t smem = staged ? (size_t)(L + 4) * 4 : 0;
  JLX_DISPATCH_DTYPE(dtype, TO, {
    if (smem > 48 * 1024)
      JLX_CUDA(cudaFuncSetAttribute(causal_sink_softmax_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    causal_sink_softmax_kernel<TO><<<dim3(T, H), 256, smem, stream>>>(s, sink, scale, q_start, (TO*)p, T, L, staged);
  });
  JLX_LAUNCH_CHECK("causal_sink_softmax");
  return 0;
}

// [H, N, d] -> [N, H * d]: the per-head products' rows back into token rows.
template <typename T>
__global__ void heads_to_rows_kernel(const T* __restrict__ in, T* __restrict__ out, int N, int H, int d) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int n = blockIdx.x;
  for (int i = threadIdx.x; i < H * d; i += blockDim.x) {
    const int h = i / d, c = i - h * d;
    out[(size_t)n * H * d + i] = in[((size_t)h * N + n) * d + c];
  }
}

JLX_API int jlx_heads_to_rows(const void* in, void* out, int dtype, int N, int H, int d, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && H > 0 && d > 0, "heads_to_rows: bad sizes");
  if (N == 0) return 0;
  JLX_DISPATCH_DTYPE(dtype, T, { JLX_CUDA(jlx_launch_pdl(heads_to_rows_kernel<T>, dim3(N), dim3(256), 0, stream, (const T*)in, (T*)out, N, H, d)); });
  JLX_LAUNCH_CHECK("heads_to_rows");
  return 0;
}
