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
    latent_kv_prep_kernel<TO><<<N, 128, 0, stream>>>(proj, splits, split_stride, q_norm_w, kv_norm_w, eps, inv_freq, rot_dims,
                                                      (TO*)cq, (TO*)pages, block_table, bt_stride, req_of_token, positions,
                                                      q_rank, rank, dr, page_size, num_pages, status);
  });
  JLX_LAUNCH_CHECK("latent_kv_prep");
  return 0;
}

// q: float32 [N, H, dn + dr] (or partials).  q_nope: [H, N, dn] in the activation type; q_rot: float32 [N, H, dr].
template <typename TO>
__global__ void latent_q_prep_kernel(const float* __restrict__ q, int splits, long long split_stride,
                                     const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions,
                                     TO* __restrict__ q_nope, float* __restrict__ q_rot, int N, int H, int dn, int dr) {
  JLX_TL(TL_ROPE);
  const int n = blockIdx.x, h = blockIdx.y;
  const float* row = q + ((size_t)n * H + h) * (dn + dr);
  for (int i = threadIdx.x; i < dn; i += blockDim.x)
    q_nope[((size_t)h * N + n) * dn + i] = from_f32<TO>(row_sum_splits(row + i, splits, split_stride));
  const float* qr = row + dn;
  float* dst = q_rot + ((size_t)n * H + h) * dr;
  const int p = positions[n];
  for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
    float sn, cs;
    sincosf((float)p * inv_freq[i], &sn, &cs);
    const float u = row_sum_splits(qr + 2 * i, splits, split_stride), v = row_sum_splits(qr + 2 * i + 1, splits, split_stride);
    dst[2 * i] = u * cs - v * sn;
    dst[2 * i + 1] = v * cs + u * sn;
  }
  for (int i = rot_dims + threadIdx.x; i < dr; i += blockDim.x) dst[i] = row_sum_splits(qr + i, splits, split_stride);
}

JLX_API int jlx_latent_q_prep(const float* q, int splits, long long split_stride, const float* inv_freq, int rot_dims,
                              const int* positions, void* q_nope, int dtype, float* q_rot, int N, int H, int dn, int dr,
                              cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && H > 0 && dn > 0 && dr >= 0 && splits >= 1, "latent_q_prep: bad sizes");
  JLX_REQUIRE(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0, "latent_q_prep: %d rotated entries of %d", rot_dims, dr);
  JLX_REQUIRE(H <= 65535, "latent_q_prep: too many heads (%d)", H);
  if (N == 0) return 0;
  JLX_DISPATCH_DTYPE(dtype, TO, {
    latent_q_prep_kernel<TO><<<dim3(N, H), 64, 0, stream>>>(q, splits, split_stride, inv_freq, rot_dims, positions, (TO*)q_nope,
                                                            q_rot, N, H, dn, dr);
  });
  JLX_LAUNCH_CHECK("latent_q_prep");
  return 0;
}

// ------------------------------------------------------------------------------------------------ attention
// One block serves one query token and up to LAT_WARPS heads (a warp each); all of them share each tile of keys.
// Key tiles are aligned to absolute positions (0, 32, 64, ...), so the order of a position's sums depends on the
// position alone.  The sink opens the running maximum and denominator: m = sink, l = exp(sink - m) = 1.
#define LAT_TILE 32
#define LAT_WARPS 8
#define LAT_MAX_R32 32  // latent size up to 1024

template <typename TC, typename TO>
__global__ void attention_latent_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot,
                                        const TC* __restrict__ pages, const int* __restrict__ block_table, int bt_stride,
                                        const int* __restrict__ req_of_token, const int* __restrict__ positions,
                                        const float* __restrict__ sink, TO* __restrict__ out_lat, int N, int H, int rank,
                                        int dr, int page_size, int num_pages, float scale, int* status) {
  JLX_TL(TL_ATTN_GENERIC);
  extern __shared__ float smem[];
  const int dk = rank + dr, ldk = dk + 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  float* qs = smem;               // [nwarp][dk]
  float* ks = qs + nwarp * dk;    // [LAT_TILE][dk + 1]
  const int n = blockIdx.x;
  const int h = blockIdx.y * nwarp + warp;
  const bool active = h < H;
  const int p = positions[n], r = req_of_token[n];
  if (active) {
    for (int d = lane; d < rank; d += 32) qs[warp * dk + d] = q_lat[((size_t)h * N + n) * rank + d];
    for (int d = lane; d < dr; d += 32) qs[warp * dk + rank + d] = q_rot[((size_t)n * H + h) * dr + d];
  }
  const bool has_sink = sink != nullptr;
  float m = (active && has_sink) ? sink[h] : -INFINITY, l = has_sink ? 1.f : 0.f;
  float acc[LAT_MAX_R32];
#pragma unroll
  for (int i = 0; i < LAT_MAX_R32; ++i) acc[i] = 0.f;
  const int nd = (rank + 31) >> 5;

  for (int t0 = 0; t0 <= p; t0 += LAT_TILE) {
    __syncthreads();  // the previous tile is consumed; qs is visible
    const int cnt = min(LAT_TILE, p - t0 + 1);
    for (int idx = threadIdx.x; idx < cnt * dk; idx += blockDim.x) {
      const int j = idx / dk, d = idx - j * dk;
      const int pos = t0 + j;
      const int page = block_table[(size_t)r * bt_stride + pos / page_size];
      float kv = 0.f;
      if (page < 0 || page >= num_pages) atomicOr(status, JLX_STATUS_BAD_PAGE);
      else kv = to_f32<TC>(pages[((size_t)page * page_size + pos % page_size) * dk + d]);
      ks[j * ldk + d] = kv;
    }
    __syncthreads();
    if (active) {
      float s = -INFINITY;
      if (lane < cnt) {
        float dot = 0.f;
        const float* kr = ks + lane * ldk;
        const float* qr = qs + warp * dk;
        for (int d = 0; d < dk; ++d) dot = fmaf(qr[d], kr[d], dot);
        s = dot * scale;
      }
      const float m_new = fmaxf(m, warp_max(s));
      const float corr = expf(m - m_new);  // without a sink m is -inf on the first tile: exp(-inf) = 0
      const float pj = lane < cnt ? expf(s - m_new) : 0.f;
      l = l * corr + warp_sum(pj);
      m = m_new;
#pragma unroll
      for (int i = 0; i < LAT_MAX_R32; ++i) {
        if (i < nd) {
          const int d = lane + 32 * i;
          float a = acc[i] * corr;
          for (int j = 0; j < cnt; ++j) {
            const float pv = __shfl_sync(0xffffffffu, pj, j);
            if (d < rank) a = fmaf(pv, ks[j * ldk + d], a);
          }
          acc[i] = a;
        }
      }
    }
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < LAT_MAX_R32; ++i) {
      const int d = lane + 32 * i;
      if (i < nd && d < rank) out_lat[((size_t)h * N + n) * rank + d] = from_f32<TO>(acc[i] / l);
    }
  }
}

JLX_API int jlx_attention_latent(const float* q_lat, const float* q_rot, const void* pages, int cache_dtype,
                                 const int* block_table, int bt_stride, const int* req_of_token, const int* positions,
                                 const float* sink, void* out_lat, int out_dtype, int N, int H, int rank, int dr,
                                 int page_size, int num_pages, float scale, int* status, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && H > 0 && rank > 0 && dr >= 0 && page_size > 0 && num_pages > 0, "attention_latent: bad sizes");
  JLX_REQUIRE(rank <= 32 * LAT_MAX_R32, "attention_latent: latent size %d is above the supported maximum %d", rank, 32 * LAT_MAX_R32);
  if (N == 0) return 0;
  const int nwarp = H < LAT_WARPS ? H : LAT_WARPS;
  const int dk = rank + dr;
  const size_t smem = sizeof(float) * ((size_t)nwarp * dk + (size_t)LAT_TILE * (dk + 1));
  JLX_REQUIRE(smem <= 200 * 1024, "attention_latent: a key tile of %d x %d does not fit into shared memory", LAT_TILE, dk);
  const int hb = (H + nwarp - 1) / nwarp;
  JLX_REQUIRE(hb <= 65535, "attention_latent: too many heads (%d)", H);
  JLX_DISPATCH_DTYPE(cache_dtype, TC, JLX_DISPATCH_DTYPE(out_dtype, TO, {
    if (smem > 48 * 1024)
      JLX_CUDA(cudaFuncSetAttribute(attention_latent_kernel<TC, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attention_latent_kernel<TC, TO><<<dim3(N, hb), nwarp * 32, smem, stream>>>(
        q_lat, q_rot, (const TC*)pages, block_table, bt_stride, req_of_token, positions, sink, (TO*)out_lat, N, H, rank, dr,
        page_size, num_pages, scale, status);
  }));
  JLX_LAUNCH_CHECK("attention_latent");
  return 0;
}

// [H, N, d] -> [N, H * d]: the per-head products' rows back into token rows.
template <typename T>
__global__ void heads_to_rows_kernel(const T* __restrict__ in, T* __restrict__ out, int N, int H, int d) {
  JLX_TL(TL_OTHER);
  const int n = blockIdx.x;
  for (int i = threadIdx.x; i < H * d; i += blockDim.x) {
    const int h = i / d, c = i - h * d;
    out[(size_t)n * H * d + i] = in[((size_t)h * N + n) * d + c];
  }
}

JLX_API int jlx_heads_to_rows(const void* in, void* out, int dtype, int N, int H, int d, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && H > 0 && d > 0, "heads_to_rows: bad sizes");
  if (N == 0) return 0;
  JLX_DISPATCH_DTYPE(dtype, T, { heads_to_rows_kernel<T><<<N, 256, 0, stream>>>((const T*)in, (T*)out, N, H, d); });
  JLX_LAUNCH_CHECK("heads_to_rows");
  return 0;
}
