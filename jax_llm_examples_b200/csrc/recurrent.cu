// Gated linear recurrences with a matrix state per head, in 32-bit, over the flattened batch of a step.
//
// HGRN2 form (the forget gate f is also the write gate 1 - f; keys do not exist):
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
// With SEG (a segment that did not start from the request's true state): cum = the product of the gates since the
// segment's start, and qd (if given) gets cum * q, with which the segment's outputs are corrected once its true start
// state is known.
template <bool SEG>
__device__ __forceinline__ void rec_token(const float* __restrict__ row, int dkp, int i0, int jl,
                                          float2 (&S)[REC_RT / 2][REC_CT], float (&acc)[REC_CT], float2 (&cum)[REC_RT / 2],
                                          float* __restrict__ qd, int qd_rows) {
  float2 f[REC_RT / 2], q[REC_RT / 2];
  float v[REC_CT];
#pragma unroll
  for (int a = 0; a < REC_RT / 2; a += 2) {
    *reinterpret_cast<float4*>(&f[a]) = *reinterpret_cast<const float4*>(row + i0 + 2 * a);
    *reinterpret_cast<float4*>(&q[a]) = *reinterpret_cast<const float4*>(row + dkp + i0 + 2 * a);
  }
  if (SEG) {
#pragma unroll
    for (int a = 0; a < REC_RT / 2; ++a) cum[a] = make_float2(cum[a].x * f[a].x, cum[a].y * f[a].y);
    if (qd) {
      if (qd_rows == REC_RT && (reinterpret_cast<uintptr_t>(qd) & 15) == 0) {
#pragma unroll
        for (int a = 0; a < REC_RT / 2; a += 2)
          *reinterpret_cast<float4*>(qd + 2 * a) = make_float4(cum[a].x * q[a].x, cum[a].y * q[a].y, cum[a + 1].x * q[a + 1].x, cum[a + 1].y * q[a + 1].y);
      } else {  // a slice that the head's rows end in, or rows that do not start on 16 bytes
#pragma unroll
        for (int a = 0; a < REC_RT / 2; ++a) {
          if (2 * a < qd_rows) qd[2 * a] = cum[a].x * q[a].x;
          if (2 * a + 1 < qd_rows) qd[2 * a + 1] = cum[a].y * q[a].y;
        }
      }
    }
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

// With `segs` (int32 [blocks.x, 4] = request, first row, end row, flags) a block serves a SEGMENT of a request's tokens
// instead of all of them.  flags bit 0: the segment starts from the request's carried state (else from zero); bit 1: the
// request has several segments, and the segment's end state goes to seg_state[segment] (else to the state slab).
template <int NSP, bool SEG>
__global__ void __launch_bounds__(512)
hgrn2_scan_kernel(const float* __restrict__ g, float* __restrict__ state, const int* __restrict__ cu_q,
                  const int* __restrict__ slot_ids, float* __restrict__ o32, int H, int dk, int dv, int DVB,
                  const int* __restrict__ segs, float* __restrict__ seg_state, float* __restrict__ seg_decay,
                  float* __restrict__ qd) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int dkp = NSP * REC_RT;         // dk padded to whole row slices
  const int rowlen = 2 * dkp + DVB;     // a token in shared memory: [f (dkp) | q (dkp) | v (DVB)]
  float* buf0 = smem;
  float* buf1 = smem + REC_TCH * rowlen;
  const int hd = blockIdx.y, col0 = blockIdx.z * DVB;
  const int NC = DVB / REC_CT;
  const int c = threadIdx.x / NSP, s = threadIdx.x % NSP;
  const bool live = c < NC;  // the block is rounded up to whole warps
  const int i0 = s * REC_RT, jl = live ? c * REC_CT : 0, j0 = col0 + jl;
  const int r = SEG ? segs[4 * blockIdx.x] : blockIdx.x;
  const int n0 = SEG ? segs[4 * blockIdx.x + 1] : cu_q[r], n1 = SEG ? segs[4 * blockIdx.x + 2] : cu_q[r + 1];
  const int flags = SEG ? segs[4 * blockIdx.x + 3] : 1;
  const bool from_state = flags & 1, to_scratch = flags & 2;
  const int HK = H * dk;
  const int C = 2 * HK + H * dv;
  float* S_g = state + (((size_t)slot_ids[r] * H + hd) * dk) * dv;
  float* S_out = to_scratch ? seg_state + (((size_t)blockIdx.x * H + hd) * dk) * dv : S_g;
  // the correction's inputs are written once per head: by the first column group of the first column slice
  const bool corr = SEG && !from_state;
  float* qd_row = (corr && live && c == 0 && blockIdx.z == 0 && i0 < dk) ? qd + hd * dk + i0 : nullptr;
  const int qd_rows = min(REC_RT, dk - i0);  // rows of this slice that the head has
  float2 cum[REC_RT / 2];
#pragma unroll
  for (int a = 0; a < REC_RT / 2; ++a) cum[a] = make_float2(1.f, 1.f);

  float2 S[REC_RT / 2][REC_CT];
  auto held = [&](int a, int k) { return live && i0 + a < dk && j0 + k < dv; };
#pragma unroll
  for (int a = 0; a < REC_RT / 2; ++a)
#pragma unroll
    for (int k = 0; k < REC_CT; ++k) {
      S[a][k].x = (from_state && held(2 * a, k)) ? S_g[(size_t)(i0 + 2 * a) * dv + j0 + k] : 0.f;
      S[a][k].y = (from_state && held(2 * a + 1, k)) ? S_g[(size_t)(i0 + 2 * a + 1) * dv + j0 + k] : 0.f;
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
      float* qdt = qd_row ? qd_row + (size_t)(cs + tt) * HK : nullptr;
      if (corr) {
        rec_token<true>(cur + tt * rowlen, dkp, i0, jl, S, a0, cum, qdt, qd_rows);
        rec_token<true>(cur + (tt + 1) * rowlen, dkp, i0, jl, S, a1, cum, qdt ? qdt + HK : nullptr, qd_rows);
        rec_token<true>(cur + (tt + 2) * rowlen, dkp, i0, jl, S, a2, cum, qdt ? qdt + 2 * HK : nullptr, qd_rows);
        rec_token<true>(cur + (tt + 3) * rowlen, dkp, i0, jl, S, a3, cum, qdt ? qdt + 3 * HK : nullptr, qd_rows);
      } else {
        rec_token<false>(cur + tt * rowlen, dkp, i0, jl, S, a0, cum, nullptr, 0);
        rec_token<false>(cur + (tt + 1) * rowlen, dkp, i0, jl, S, a1, cum, nullptr, 0);
        rec_token<false>(cur + (tt + 2) * rowlen, dkp, i0, jl, S, a2, cum, nullptr, 0);
        rec_token<false>(cur + (tt + 3) * rowlen, dkp, i0, jl, S, a3, cum, nullptr, 0);
      }
      emit(cs + tt, a0);
      emit(cs + tt + 1, a1);
      emit(cs + tt + 2, a2);
      emit(cs + tt + 3, a3);
    }
    for (; tt < cnt; ++tt) {
      float a0[REC_CT];
      if (corr) rec_token<true>(cur + tt * rowlen, dkp, i0, jl, S, a0, cum, qd_row ? qd_row + (size_t)(cs + tt) * HK : nullptr, qd_rows);
      else rec_token<false>(cur + tt * rowlen, dkp, i0, jl, S, a0, cum, nullptr, 0);
      emit(cs + tt, a0);
    }
    cp_async_wait_all();
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < REC_RT / 2; ++a)
#pragma unroll
    for (int k = 0; k < REC_CT; ++k) {
      if (held(2 * a, k)) S_out[(size_t)(i0 + 2 * a) * dv + j0 + k] = S[a][k].x;
      if (held(2 * a + 1, k)) S_out[(size_t)(i0 + 2 * a + 1) * dv + j0 + k] = S[a][k].y;
    }
  if (qd_row) {  // the product of the segment's gates, per state row
    float* d = seg_decay + (size_t)blockIdx.x * HK + hd * dk + i0;
#pragma unroll
    for (int a = 0; a < REC_RT / 2; ++a) {
      if (i0 + 2 * a < dk) d[2 * a] = cum[a].x;
      if (i0 + 2 * a + 1 < dk) d[2 * a + 1] = cum[a].y;
    }
  }
}

// The true states of a request that was scanned in several segments.  Segment 0 started from the carried state, so its
// end state is true; for k >= 1: start_k = end_(k-1), end_k = decay_k * start_k + (the segment's end state from zero).
// seg_state[k] is overwritten by start_k (what the correction needs); the last end goes to the state slab.
__global__ void hgrn2_chain_kernel(const int* __restrict__ segs, int n_seg, float* __restrict__ seg_state,
                                   const float* __restrict__ seg_decay, float* __restrict__ state,
                                   const int* __restrict__ slot_ids, int H, int dk, int dv) {
  JLX_TL(TL_OTHER);
  const int b = blockIdx.x, hd = blockIdx.y;
  const int flags = segs[4 * b + 3];
  if ((flags & 3) != 3) return;  // only the first segment of a request with several walks the chain
  const int r = segs[4 * b];
  const size_t per = (size_t)dk * dv;
  float* S_g = state + ((size_t)slot_ids[r] * H + hd) * per;
  {  // one state entry per thread: the chain's steps are dependent, its entries are not
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= dk * dv) return;
    const int i = e / dv;
    float t = seg_state[((size_t)b * H + hd) * per + e];
    for (int k = b + 1; k < n_seg && segs[4 * k] == r && !(segs[4 * k + 3] & 1); ++k) {
      float* at = seg_state + ((size_t)k * H + hd) * per + e;
      const float end_from_zero = *at;
      *at = t;
      t = fmaf(seg_decay[(size_t)k * H * dk + hd * dk + i], t, end_from_zero);
    }
    S_g[e] = t;
  }
}

// o[t, j] += sum_i start[i, j] * qd[t, i] for the tokens of the segments that started from zero.  One block: a segment's
// tile of 32 tokens, a head, 32 value columns; the sums run over i in ascending order.
#define COR_TOK 32
#define COR_COL 32
__global__ void __launch_bounds__(128)
hgrn2_correct_kernel(const int* __restrict__ segs, const float* __restrict__ seg_state, const float* __restrict__ qd,
                     float* __restrict__ o32, int H, int dk, int dv, int tiles_per_seg) {
  JLX_TL(TL_OTHER);
  extern __shared__ __align__(16) float smem[];
  float* Ts = smem;                 // [dk][COR_COL]
  float* Qs = smem + dk * COR_COL;  // [COR_TOK][dk + 1]
  const int b = blockIdx.x / tiles_per_seg, tile = blockIdx.x % tiles_per_seg;
  const int hd = blockIdx.y, col0 = blockIdx.z * COR_COL;
  if (segs[4 * b + 3] & 1) return;
  const int t0 = segs[4 * b + 1] + tile * COR_TOK, t1 = min(segs[4 * b + 2], t0 + COR_TOK);
  if (t0 >= t1) return;
  const float* T = seg_state + ((size_t)b * H + hd) * dk * dv;
  for (int e = threadIdx.x; e < dk * COR_COL; e += blockDim.x) {
    const int i = e / COR_COL, j = e % COR_COL;
    Ts[e] = col0 + j < dv ? T[(size_t)i * dv + col0 + j] : 0.f;
  }
  for (int e = threadIdx.x; e < COR_TOK * dk; e += blockDim.x) {
    const int u = e / dk, i = e - u * dk;
    Qs[u * (dk + 1) + i] = t0 + u < t1 ? qd[(size_t)(t0 + u) * H * dk + hd * dk + i] : 0.f;
  }
  __syncthreads();
  const int tx = threadIdx.x % COR_COL, ty = threadIdx.x / COR_COL;  // a column, a group of 8 tokens
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int i = 0; i < dk; ++i) {
    const float tv = Ts[i * COR_COL + tx];
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[u] = fmaf(Qs[(ty * 8 + u) * (dk + 1) + i], tv, acc[u]);
  }
  if (col0 + tx < dv)
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (t0 + ty * 8 + u < t1) o32[(size_t)(t0 + ty * 8 + u) * H * dv + hd * dv + col0 + tx] += acc[u];
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
                           const int* segs, int n_seg, int seg_tokens, float* seg_state, float* seg_decay, float* qd,
                           cudaStream_t stream) {
  JLX_REQUIRE(R >= 0 && N >= 0 && H > 0 && dk > 0 && dv > 0 && splits >= 1, "hgrn2_scan: bad sizes R=%d H=%d dk=%d dv=%d", R, H, dk, dv);
  JLX_REQUIRE(dk <= 32 * REC_RT, "hgrn2_scan: %d state rows per head are above the supported maximum %d", dk, 32 * REC_RT);
  JLX_REQUIRE(eps > 0.f, "hgrn2_scan: eps must be positive");
  JLX_REQUIRE(gates && o32, "hgrn2_scan: scratch is missing");
  JLX_REQUIRE(!segs || (n_seg >= R && seg_tokens >= COR_TOK && seg_state && seg_decay && qd), "hgrn2_scan: segments need their scratch");
  if (R == 0 || N == 0) return 0;
  const int nb = segs ? n_seg : R;  // blocks along x: segments, or requests
  JLX_CUDA(jlx_launch_pdl(hgrn2_gates_kernel, dim3(N), dim3(256), 0, stream, qfv, splits, split_stride, f_bias, lower, gates, H * dk, H * dv));
  JLX_LAUNCH_CHECK("hgrn2_gates");
  int NSP = 1;
  while (NSP * REC_RT < dk) NSP *= 2;
  // value columns per block: as many as a block of 512 threads takes, fewer while the grid would not fill the GPU
  int DVB = 4;
  while (DVB < dv && DVB < 64 && (DVB * 2 / REC_CT) * NSP <= 512) DVB *= 2;
  while (DVB > 16 && (long long)nb * H * ((dv + DVB - 1) / DVB) < 2 * sm_count) DVB /= 2;  // every slice reads the head's f and q again
  const int zb = (dv + DVB - 1) / DVB;
  JLX_REQUIRE(H <= 65535 && zb <= 65535, "hgrn2_scan: too many heads or column slices");
  const int threads = ((DVB / REC_CT) * NSP + 31) / 32 * 32;
  const int dkp = NSP * REC_RT;
  const size_t smem = sizeof(float) * (2 * (size_t)REC_TCH * (2 * dkp + DVB));
#define REC_GO(NSP_)                                                                                                        \
  case NSP_:                                                                                                                \
    if (segs) {                                                                                                             \
      if (smem > 48 * 1024)                                                                                                 \
        JLX_CUDA(cudaFuncSetAttribute(hgrn2_scan_kernel<NSP_, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      JLX_CUDA(jlx_launch_pdl(hgrn2_scan_kernel<NSP_, true>, dim3(nb, H, zb), dim3(threads), smem, stream, (const float*)gates, \
                              state, cu_q, slot_ids, o32, H, dk, dv, DVB, segs, seg_state, seg_decay, qd));                  \
    } else {                                                                                                                \
      if (smem > 48 * 1024)                                                                                                 \
        JLX_CUDA(cudaFuncSetAttribute(hgrn2_scan_kernel<NSP_, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      JLX_CUDA(jlx_launch_pdl(hgrn2_scan_kernel<NSP_, false>, dim3(nb, H, zb), dim3(threads), smem, stream, (const float*)gates, \
                              state, cu_q, slot_ids, o32, H, dk, dv, DVB, segs, seg_state, seg_decay, qd));                  \
    }                                                                                                                       \
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
  if (segs) {
    hgrn2_chain_kernel<<<dim3(n_seg, H, (dk * dv + 255) / 256), 256, 0, stream>>>(segs, n_seg, seg_state, seg_decay, state, slot_ids, H, dk, dv);
    JLX_LAUNCH_CHECK("hgrn2_chain");
    const int tiles = (seg_tokens + COR_TOK - 1) / COR_TOK;
    const size_t csm = sizeof(float) * ((size_t)dk * COR_COL + (size_t)COR_TOK * (dk + 1));
    if (csm > 48 * 1024) JLX_CUDA(cudaFuncSetAttribute(hgrn2_correct_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csm));
    hgrn2_correct_kernel<<<dim3(n_seg * tiles, H, (dv + COR_COL - 1) / COR_COL), 128, csm, stream>>>(segs, seg_state, qd, o32, H, dk, dv, tiles);
    JLX_LAUNCH_CHECK("hgrn2_correct");
  }
  const int rows = N * H, wpb = 8;
  JLX_DISPATCH_DTYPE(out_dtype, TO, {
    JLX_CUDA(jlx_launch_pdl(head_rms_norm_kernel<TO>, dim3((rows + wpb - 1) / wpb), dim3(wpb * 32), 0, stream, (const float*)o32, norm_w,
                            eps, (TO*)out, rows, dv));
  });
  JLX_LAUNCH_CHECK("head_rms_norm");
  return 0;
}
