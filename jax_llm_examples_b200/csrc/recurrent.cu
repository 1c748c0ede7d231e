// Gated linear recurrences with a matrix state per head, in 32-bit, over the flattened batch of a step.
//
// HGRN2 form (the forget gate also says how much is written; there is no key):
//   f_t = lower + (1 - lower) * sigmoid(f_pre_t + f_bias)            per head and channel i < dk
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T                         S: [dk, dv] per request and head
//   o_t = S_t^T silu(q_pre_t)
//   out_t = norm_w * o_t / sqrt(mean(o_t^2) + eps)                    per head over dv   (head_rms_norm)
// The projected rows come as float32 [N, 2 H dk + H dv] = [q_pre | f_pre | v] (or split-K partials of them).
// The state lives in a float32 slab [slots, H, dk, dv]; a request's tokens are walked in order, whatever the
// step brings of them (a prompt portion or one decoded token), and every entry of S and of o is computed by the same
// sequence of operations whatever the cut, so the result does not depend on it.
//
// One block per (request, head, slice of DVB value columns).  A thread keeps an 8 x 4 tile of S in registers; the 8-row
// slices of a column group sit in neighbouring lanes, so that o's sum over the rows is a few shuffles.  The update is
// S <- f * (S - v) + v (one subtraction and one fused multiply-add).  The output sum does not feed back into the state:
// a block walks TCH tokens between barriers, with the next TCH tokens' rows on their way into shared memory (cp.async)
// meanwhile; gates and silu are applied there, in place.
#include "common.cuh"

#define REC_RT 8    // state rows per thread
#define REC_CT 4    // state columns per thread
#define REC_TCH 16  // tokens between barriers

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__global__ void __launch_bounds__(512)
hgrn2_scan_kernel(const float* __restrict__ qfv, int splits, long long split_stride, const float* __restrict__ f_bias,
                  const float* __restrict__ lower, float* __restrict__ state, const int* __restrict__ cu_q,
                  const int* __restrict__ slot_ids, float* __restrict__ o32, int H, int dk, int dv, int DVB, int NSP) {
  JLX_TL(TL_OTHER);
  extern __shared__ __align__(16) float smem[];
  const int dkp = NSP * REC_RT;         // dk padded to whole row slices
  const int rowlen = 2 * dkp + DVB;     // a token in shared memory: [f (dkp) | q (dkp) | v (DVB)]
  float* buf0 = smem;
  float* buf1 = smem + REC_TCH * rowlen;
  float* gate_c = buf1 + REC_TCH * rowlen;  // [2][dkp]: f_bias, lower of this head
  const int r = blockIdx.x, hd = blockIdx.y, col0 = blockIdx.z * DVB;
  const int NC = DVB / REC_CT;
  const int c = threadIdx.x / NSP, s = threadIdx.x % NSP;
  const bool live = c < NC;  // the block is rounded up to whole warps
  const int i0 = s * REC_RT, jl = live ? c * REC_CT : 0, j0 = col0 + jl;
  const int n0 = cu_q[r], n1 = cu_q[r + 1];
  const int C = 2 * H * dk + H * dv;
  float* S_g = state + (((size_t)slot_ids[r] * H + hd) * dk) * dv;

  float S[REC_RT][REC_CT];
#pragma unroll
  for (int a = 0; a < REC_RT; ++a)
#pragma unroll
    for (int k = 0; k < REC_CT; ++k)
      S[a][k] = (live && i0 + a < dk && j0 + k < dv) ? S_g[(size_t)(i0 + a) * dv + j0 + k] : 0.f;
  for (int i = threadIdx.x; i < dkp; i += blockDim.x) {
    gate_c[i] = i < dk ? f_bias[hd * dk + i] : 0.f;
    gate_c[dkp + i] = i < dk ? lower[hd * dk + i] : 0.f;
  }

  // raw rows of tokens [t0, t0 + cnt) into b (asynchronously when they are whole)
  auto fill = [&](int t0, int cnt, float* b) {
    for (int idx = threadIdx.x; idx < cnt * rowlen; idx += blockDim.x) {
      const int tt = idx / rowlen, e = idx - tt * rowlen;
      int src = -1;
      if (e < dkp) { if (e < dk) src = H * dk + hd * dk + e; }
      else if (e < 2 * dkp) { if (e - dkp < dk) src = hd * dk + (e - dkp); }
      else if (col0 + (e - 2 * dkp) < dv) src = 2 * H * dk + hd * dv + col0 + (e - 2 * dkp);
      if (src < 0) { b[idx] = 0.f; continue; }
      const float* p = qfv + (size_t)(t0 + tt) * C + src;
      if (splits == 1) cp_async4(b + idx, p);
      else {
        float v = 0.f;
        for (int z = 0; z < splits; ++z) v += p[(size_t)z * split_stride];
        b[idx] = v;
      }
    }
  };
  // gates and silu in place; padded rows get f = 1, q = 0 (their state stays zero and adds nothing)
  auto transform = [&](int cnt, float* b) {
    for (int idx = threadIdx.x; idx < cnt * dkp; idx += blockDim.x) {
      const int tt = idx / dkp, i = idx - tt * dkp;
      float* row = b + tt * rowlen;
      if (i < dk) {
        const float lo = gate_c[dkp + i];
        row[i] = lo + (1.f - lo) * (1.f / (1.f + expf(-(row[i] + gate_c[i]))));
        const float qp = row[dkp + i];
        row[dkp + i] = qp / (1.f + expf(-qp));
      } else {
        row[i] = 1.f;
        row[dkp + i] = 0.f;
      }
    }
  };

  int cnt = min(REC_TCH, n1 - n0);
  fill(n0, cnt, buf0);
  cp_async_wait_all();
  __syncthreads();
  transform(cnt, buf0);
  __syncthreads();
  int p = 0;
  for (int cs = n0; cs < n1; cs += REC_TCH, p ^= 1) {
    float* cur = p ? buf1 : buf0;
    float* nxt = p ? buf0 : buf1;
    const int next = cs + REC_TCH;
    const int ncnt = min(REC_TCH, n1 - next);
    if (next < n1) fill(next, ncnt, nxt);
    cnt = min(REC_TCH, n1 - cs);
    for (int tt = 0; tt < cnt; ++tt) {
      const float* row = cur + tt * rowlen;
      float f[REC_RT], q[REC_RT], v[REC_CT];
      *reinterpret_cast<float4*>(&f[0]) = *reinterpret_cast<const float4*>(row + i0);
      *reinterpret_cast<float4*>(&f[4]) = *reinterpret_cast<const float4*>(row + i0 + 4);
      *reinterpret_cast<float4*>(&q[0]) = *reinterpret_cast<const float4*>(row + dkp + i0);
      *reinterpret_cast<float4*>(&q[4]) = *reinterpret_cast<const float4*>(row + dkp + i0 + 4);
      *reinterpret_cast<float4*>(&v[0]) = *reinterpret_cast<const float4*>(row + 2 * dkp + jl);
      float acc[REC_CT] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int a = 0; a < REC_RT; ++a)
#pragma unroll
        for (int k = 0; k < REC_CT; ++k) {
          S[a][k] = fmaf(f[a], S[a][k] - v[k], v[k]);
          acc[k] = fmaf(S[a][k], q[a], acc[k]);
        }
      for (int o = NSP >> 1; o > 0; o >>= 1)
#pragma unroll
        for (int k = 0; k < REC_CT; ++k) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], o);
      if (live && s == 0) {
        float* dst = o32 + (size_t)(cs + tt) * H * dv + hd * dv + j0;
#pragma unroll
        for (int k = 0; k < REC_CT; ++k)
          if (j0 + k < dv) dst[k] = acc[k];
      }
    }
    cp_async_wait_all();
    __syncthreads();
    if (next < n1) {
      transform(ncnt, nxt);
      __syncthreads();
    }
  }
#pragma unroll
  for (int a = 0; a < REC_RT; ++a)
#pragma unroll
    for (int k = 0; k < REC_CT; ++k)
      if (live && i0 + a < dk && j0 + k < dv) S_g[(size_t)(i0 + a) * dv + j0 + k] = S[a][k];
}

// out[n, h, :] = w * o[n, h, :] / sqrt(mean(o[n, h, :]^2) + eps): one warp per (token, head).
template <typename TO>
__global__ void head_rms_norm_kernel(const float* __restrict__ o32, const float* __restrict__ w, float eps, TO* __restrict__ out,
                                     int rows, int dv) {
  JLX_TL(TL_NORM);
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* p = o32 + (size_t)row * dv;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) ss = fmaf(p[j], p[j], ss);
  const float rms = sqrtf(warp_sum(ss) / (float)dv + eps);
  for (int j = lane; j < dv; j += 32) out[(size_t)row * dv + j] = from_f32<TO>(p[j] / rms * (w ? w[j] : 1.f));
}

JLX_API int jlx_hgrn2_scan(const float* qfv, int splits, long long split_stride, const float* f_bias, const float* lower,
                           float* state, const int* cu_q, const int* slot_ids, const float* norm_w, float eps, float* o32,
                           void* out, int out_dtype, int N, int R, int H, int dk, int dv, int sm_count, cudaStream_t stream) {
  JLX_REQUIRE(R >= 0 && N >= 0 && H > 0 && dk > 0 && dv > 0 && splits >= 1, "hgrn2_scan: bad sizes R=%d H=%d dk=%d dv=%d", R, H, dk, dv);
  JLX_REQUIRE(dk <= 32 * REC_RT, "hgrn2_scan: %d state rows per head are above the supported maximum %d", dk, 32 * REC_RT);
  JLX_REQUIRE(eps > 0.f, "hgrn2_scan: eps must be positive");
  JLX_REQUIRE(((uintptr_t)qfv & 3) == 0, "hgrn2_scan: misaligned input");
  if (R == 0 || N == 0) return 0;
  int NSP = 1;
  while (NSP * REC_RT < dk) NSP *= 2;
  // value columns per block: as many as a block of 512 threads takes, fewer while the grid would not fill the GPU
  int DVB = 4;
  while (DVB < dv && DVB < 64 && (DVB * 2 / REC_CT) * NSP <= 512) DVB *= 2;
  while (DVB > 32 && (long long)R * H * ((dv + DVB - 1) / DVB) < sm_count) DVB /= 2;  // every slice computes the head's gates again
  const int zb = (dv + DVB - 1) / DVB;
  JLX_REQUIRE(H <= 65535 && zb <= 65535, "hgrn2_scan: too many heads or column slices");
  const int threads = ((DVB / REC_CT) * NSP + 31) / 32 * 32;
  const int dkp = NSP * REC_RT;
  const size_t smem = sizeof(float) * (2 * (size_t)REC_TCH * (2 * dkp + DVB) + 2 * dkp);
  if (smem > 48 * 1024) JLX_CUDA(cudaFuncSetAttribute(hgrn2_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  hgrn2_scan_kernel<<<dim3(R, H, zb), threads, smem, stream>>>(qfv, splits, split_stride, f_bias, lower, state, cu_q, slot_ids, o32,
                                                                H, dk, dv, DVB, NSP);
  JLX_LAUNCH_CHECK("hgrn2_scan");
  const int rows = N * H, wpb = 8;
  JLX_DISPATCH_DTYPE(out_dtype, TO, {
    head_rms_norm_kernel<TO><<<(rows + wpb - 1) / wpb, wpb * 32, 0, stream>>>(o32, norm_w, eps, (TO*)out, rows, dv);
  });
  JLX_LAUNCH_CHECK("head_rms_norm");
  return 0;
}
