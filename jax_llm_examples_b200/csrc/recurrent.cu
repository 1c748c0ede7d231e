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
// Two kernels.  hgrn2_gates turns the projected rows into [f | silu(q) | v] once per token (adding split-K partials on
// the way).  hgrn2_scan: one block per (request, head, slice of DVB value columns).  A thread keeps an 8 x 4 tile of S in
// registers; the 8-row slices of a column group sit in neighbouring lanes, so that o's sum over the rows is a few
// shuffles.  The update is S <- f * (S - v) + v (one subtraction and one fused multiply-add).  The output sum does not
// feed back into the state: a block walks TCH tokens between barriers, with the next TCH tokens' rows on their way into
// shared memory (cp.async, 16 bytes each where the sizes allow) meanwhile, and the token loop is unrolled so that one
// token's shuffles overlap the next one's loads and products (a scheduler holds one warp of this kernel at most).
#include "common.cuh"

#ifndef REC_RT
#define REC_RT 8    // state rows per thread (a multiple of 4)
#endif
#define REC_CT 4    // state columns per thread
#ifndef REC_TCH
#define REC_TCH 16  // tokens between barriers
#endif

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* smem_dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// g[n] = [f (H dk) | silu(q) (H dk) | v (H dv)] from qfv[n] = [q_pre | f_pre | v] (the sum of its partials).
__global__ void hgrn2_gates_kernel(const float* __restrict__ qfv, int splits, long long split_stride, const float* __restrict__ f_bias,
                                   const float* __restrict__ lower, float* __restrict__ g, int HK, int HV) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t n = blockIdx.x;
  const int C = 2 * HK + HV;
  const float* row = qfv + n * C;
  float* out = g + n * C;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    float v = 0.f;
    for (int z = 0; z < splits; ++z) v += row[(size_t)z * split_stride + i];
    if (i < HK) {
      out[HK + i] = v / (1.f + expf(-v));  // q
    } else if (i < 2 * HK) {
      const int c = i - HK;
      const float lo = lower[c];
      out[c] = lo + (1.f - lo) * (1.f / (1.f + expf(-(v + f_bias[c]))));  // f
    } else {
      out[i] = v;
    }
  }
}

// Two 32-bit values per instruction (Blackwell's packed fp32 arithmetic; each half is the IEEE operation).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long*>(&a)),
      "l"(*reinterpret_cast<unsigned long long*>(&b)), "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 sub2(float2 a, float2 b) {
  unsigned long long d;
  asm("sub.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}

// One token through a thread's tile.  S is kept as pairs of neighbouring rows: S[a][k] = (S_(2a, k), S_(2a+1, k)).
// acc[k] = the sum over the even rows' products + the sum over the odd rows' products.
__device__ __forceinline__ void rec_token(const float* __restrict__ row, int dkp, int i0, int jl,
                                          float2 (&S)[REC_RT / 2][REC_CT], float (&acc)[REC_CT]) {
  float2 f[REC_RT / 2], q[REC_RT / 2];
  float v[REC_CT];
#pragma unroll
  for (int a = 0; a < REC_RT / 2; a += 2) {
    *reinterpret_cast<float4*>(&f[a]) = *reinterpret_cast<const float4*>(row + i0 + 2 * a);
    *reinterpret_cast<float4*>(&q[a]) = *reinterpret_cast<const float4*>(row + dkp + i0 + 2 * a);
  }
  *reinterpret_cast<float4*>(&v[0]) = *reinterpret_cast<const float4*>(row + 2 * dkp + jl);
#pragma unroll
  for (int k = 0; k < REC_CT; ++k) {
    const float2 vv = make_float2(v[k], v[k]);
    float2 sum = make_float2(0.f, 0.f);
#pragma unroll
    for (int a = 0; a < REC_RT / 2; ++a) {
      S[a][k] = fma2(f[a], sub2(S[a][k], vv), vv);
      sum = fma2(S[a][k], q[a], sum);
    }
    acc[k] = sum.x + sum.y;
  }
}

template <int NSP>
__global__ void __launch_bounds__(512)
hgrn2_scan_kernel(const float* __restrict__ g, float* __restrict__ state, const int* __restrict__ cu_q,
                  const int* __restrict__ slot_ids, float* __restrict__ o32, int H, int dk, int dv, int DVB) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int dkp = NSP * REC_RT;         // dk padded to whole row slices
  const int rowlen = 2 * dkp + DVB;     // a token in shared memory: [f (dkp) | q (dkp) | v (DVB)]
  float* buf0 = smem;
  float* buf1 = smem + REC_TCH * rowlen;
  const int r = blockIdx.x, hd = blockIdx.y, col0 = blockIdx.z * DVB;
  const int NC = DVB / REC_CT;
  const int c = threadIdx.x / NSP, s = threadIdx.x % NSP;
  const bool live = c < NC;  // the block is rounded up to whole warps
  const int i0 = s * REC_RT, jl = live ? c * REC_CT : 0, j0 = col0 + jl;
  const int n0 = cu_q[r], n1 = cu_q[r + 1];
  const int HK = H * dk;
  const int C = 2 * HK + H * dv;
  float* S_g = state + (((size_t)slot_ids[r] * H + hd) * dk) * dv;

  float2 S[REC_RT / 2][REC_CT];
  auto held = [&](int a, int k) { return live && i0 + a < dk && j0 + k < dv; };
#pragma unroll
  for (int a = 0; a < REC_RT / 2; ++a)
#pragma unroll
    for (int k = 0; k < REC_CT; ++k) {
      S[a][k].x = held(2 * a, k) ? S_g[(size_t)(i0 + 2 * a) * dv + j0 + k] : 0.f;
      S[a][k].y = held(2 * a + 1, k) ? S_g[(size_t)(i0 + 2 * a + 1) * dv + j0 + k] : 0.f;
    }
  // padded rows: f = 1, q = 0 (their state stays zero and adds nothing); padded columns: v = 0.  Written once: the
  // copies below never touch them.
  for (int idx = threadIdx.x; idx < 2 * REC_TCH * rowlen; idx += blockDim.x) {
    const int e = idx % rowlen;
    if (e >= dk && e < dkp) smem[idx] = 1.f;
    else if ((e >= dkp + dk && e < 2 * dkp) || (e >= 2 * dkp && col0 + (e - 2 * dkp) >= dv)) smem[idx] = 0.f;
  }
  const int vcols = min(DVB, dv - col0);
  // 16-byte copies where every piece starts on a 16-byte boundary in both memories
  const bool wide = (dk & 3) == 0 && (dv & 3) == 0 && (vcols & 3) == 0 && (((uintptr_t)g) & 15) == 0;
  const float* gf = g + hd * dk;                // + token * C: the head's f
  const float* gq = g + HK + hd * dk;           // its q
  const float* gv = g + 2 * HK + hd * dv + col0;  // its slice of v

  auto fill = [&](int t0, int cnt, float* b) {
    if (wide) {
      const int kq = dk >> 2, vq = vcols >> 2, per = 2 * kq + vq;
      for (int tt = 0; tt < cnt; ++tt) {
        const size_t at = (size_t)(t0 + tt) * C;
        float* row = b + tt * rowlen;
        for (int e = threadIdx.x; e < per; e += blockDim.x) {
          if (e < kq) cp_async16(row + 4 * e, gf + at + 4 * e);
          else if (e < 2 * kq) cp_async16(row + dkp + 4 * (e - kq), gq + at + 4 * (e - kq));
          else cp_async16(row + 2 * dkp + 4 * (e - 2 * kq), gv + at + 4 * (e - 2 * kq));
        }
      }
    } else {
      const int per = 2 * dk + vcols;
      for (int tt = 0; tt < cnt; ++tt) {
        const size_t at = (size_t)(t0 + tt) * C;
        float* row = b + tt * rowlen;
        for (int e = threadIdx.x; e < per; e += blockDim.x) {
          if (e < dk) cp_async4(row + e, gf + at + e);
          else if (e < 2 * dk) cp_async4(row + dkp + (e - dk), gq + at + (e - dk));
          else cp_async4(row + 2 * dkp + (e - 2 * dk), gv + at + (e - 2 * dk));
        }
      }
    }
  };
  auto emit = [&](int t, float (&acc)[REC_CT]) {  // the sum over the row slices, then the first slice's lanes write
#pragma unroll
    for (int o = NSP >> 1; o > 0; o >>= 1)
#pragma unroll
      for (int k = 0; k < REC_CT; ++k) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], o);
    if (live && s == 0) {
      float* dst = o32 + (size_t)t * H * dv + hd * dv + j0;
      if (j0 + REC_CT <= dv && (dv & 3) == 0) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      else
#pragma unroll
        for (int k = 0; k < REC_CT; ++k)
          if (j0 + k < dv) dst[k] = acc[k];
    }
  };

  int cnt = min(REC_TCH, n1 - n0);
  __syncthreads();  // the padding is in place
  fill(n0, cnt, buf0);
  cp_async_wait_all();
  __syncthreads();
  int p = 0;
  for (int cs = n0; cs < n1; cs += REC_TCH, p ^= 1) {
    const float* cur = p ? buf1 : buf0;
    float* nxt = p ? buf0 : buf1;
    const int next = cs + REC_TCH;
    if (next < n1) fill(next, min(REC_TCH, n1 - next), nxt);
    cnt = min(REC_TCH, n1 - cs);
    int tt = 0;
    for (; tt + 3 < cnt; tt += 4) {  // four tokens in flight: the state goes through them in order, the rest overlaps
      float a0[REC_CT], a1[REC_CT], a2[REC_CT], a3[REC_CT];
      rec_token(cur + tt * rowlen, dkp, i0, jl, S, a0);
      rec_token(cur + (tt + 1) * rowlen, dkp, i0, jl, S, a1);
      rec_token(cur + (tt + 2) * rowlen, dkp, i0, jl, S, a2);
      rec_token(cur + (tt + 3) * rowlen, dkp, i0, jl, S, a3);
      emit(cs + tt, a0);
      emit(cs + tt + 1, a1);
      emit(cs + tt + 2, a2);
      emit(cs + tt + 3, a3);
    }
    for (; tt < cnt; ++tt) {
      float a0[REC_CT];
      rec_token(cur + tt * rowlen, dkp, i0, jl, S, a0);
      emit(cs + tt, a0);
    }
    cp_async_wait_all();
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < REC_RT / 2; ++a)
#pragma unroll
    for (int k = 0; k < REC_CT; ++k) {
      if (held(2 * a, k)) S_g[(size_t)(i0 + 2 * a) * dv + j0 + k] = S[a][k].x;
      if (held(2 * a + 1, k)) S_g[(size_t)(i0 + 2 * a + 1) * dv + j0 + k] = S[a][k].y;
    }
}

// out[n, h, :] = w * o[n, h, :] / sqrt(mean(o[n, h, :]^2) + eps): one warp per (token, head).
template <typename TO>
__global__ void head_rms_norm_kernel(const float* __restrict__ o32, const float* __restrict__ w, float eps, TO* __restrict__ out,
                                     int rows, int dv) {
  JLX_TL(TL_NORM);
  pdl_launch_dependents_if_small();
  pdl_wait();
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
                           float* state, const int* cu_q, const int* slot_ids, const float* norm_w, float eps, float* gates,
                           float* o32, void* out, int out_dtype, int N, int R, int H, int dk, int dv, int sm_count,
                           cudaStream_t stream) {
  JLX_REQUIRE(R >= 0 && N >= 0 && H > 0 && dk > 0 && dv > 0 && splits >= 1, "hgrn2_scan: bad sizes R=%d H=%d dk=%d dv=%d", R, H, dk, dv);
  JLX_REQUIRE(dk <= 32 * REC_RT, "hgrn2_scan: %d state rows per head are above the supported maximum %d", dk, 32 * REC_RT);
  JLX_REQUIRE(eps > 0.f, "hgrn2_scan: eps must be positive");
  JLX_REQUIRE(gates && o32, "hgrn2_scan: scratch is missing");
  if (R == 0 || N == 0) return 0;
  JLX_CUDA(jlx_launch_pdl(hgrn2_gates_kernel, dim3(N), dim3(256), 0, stream, qfv, splits, split_stride, f_bias, lower, gates, H * dk, H * dv));
  JLX_LAUNCH_CHECK("hgrn2_gates");
  int NSP = 1;
  while (NSP * REC_RT < dk) NSP *= 2;
  // value columns per block: as many as a block of 512 threads takes, fewer while the grid would not fill the GPU
  int DVB = 4;
  while (DVB < dv && DVB < 64 && (DVB * 2 / REC_CT) * NSP <= 512) DVB *= 2;
  while (DVB > 16 && (long long)R * H * ((dv + DVB - 1) / DVB) < 2 * sm_count) DVB /= 2;  // every slice reads the head's f and q again
  const int zb = (dv + DVB - 1) / DVB;
  JLX_REQUIRE(H <= 65535 && zb <= 65535, "hgrn2_scan: too many heads or column slices");
  const int threads = ((DVB / REC_CT) * NSP + 31) / 32 * 32;
  const int dkp = NSP * REC_RT;
  const size_t smem = sizeof(float) * (2 * (size_t)REC_TCH * (2 * dkp + DVB));
#define REC_GO(NSP_)                                                                                                        \
  case NSP_:                                                                                                                \
    if (smem > 48 * 1024)                                                                                                   \
      JLX_CUDA(cudaFuncSetAttribute(hgrn2_scan_kernel<NSP_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));        \
    JLX_CUDA(jlx_launch_pdl(hgrn2_scan_kernel<NSP_>, dim3(R, H, zb), dim3(threads), smem, stream, (const float*)gates, state, cu_q, \
                            slot_ids, o32, H, dk, dv, DVB));                                                                  \
    break
  switch (NSP) {
    REC_GO(1);
    REC_GO(2);
    REC_GO(4);
    REC_GO(8);
    REC_GO(16);
    REC_GO(32);
  }
#undef REC_GO
  JLX_LAUNCH_CHECK("hgrn2_scan");
  const int rows = N * H, wpb = 8;
  JLX_DISPATCH_DTYPE(out_dtype, TO, {
    JLX_CUDA(jlx_launch_pdl(head_rms_norm_kernel<TO>, dim3((rows + wpb - 1) / wpb), dim3(wpb * 32), 0, stream, (const float*)o32, norm_w,
                            eps, (TO*)out, rows, dv));
  });
  JLX_LAUNCH_CHECK("head_rms_norm");
  return 0;
}
