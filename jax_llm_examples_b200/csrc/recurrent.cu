// Gated linear recurrences with a matrix state per head, in 32-bit, over the flattened batch of a step.
//
// HGRN2 form (the forget gate also says how much is written; there is no key):
//   f_t = lower + (1 - lower) * sigmoid(f_pre_t + f_bias)            per head and channel i < dk
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T                         S: [dk, dv] per request and head
//   o_t = S_t^T silu(q_pre_t)
//   out_t = norm_w * o_t / sqrt(mean(o_t^2) + eps)                    per head over dv
// The projected rows come as float32 [N, 2 H dk + H dv] = [q_pre | f_pre | v] (or split-K partials of them).
// The state lives in a float32 slab [slots, H, dk, dv]; a request's tokens are walked in order, whatever the
// step brings of them (a prompt portion or one decoded token), so the result does not depend on the cut.
//
// One block per (request, head).  Thread (j, s) keeps rows [s * rpt, (s + 1) * rpt) of column j of S in registers.
#include "common.cuh"

#define REC_MAX_RPT 32

template <typename TO>
__global__ void __launch_bounds__(512)
hgrn2_scan_kernel(const float* __restrict__ qfv, int splits, long long split_stride, const float* __restrict__ f_bias,
                  const float* __restrict__ lower, float* __restrict__ state, const int* __restrict__ cu_q,
                  const int* __restrict__ slot_ids, const float* __restrict__ norm_w, float eps, TO* __restrict__ out,
                  int H, int dk, int dv, int KS, int rpt) {
  JLX_TL(TL_OTHER);
  extern __shared__ float smem[];
  float* fs = smem;            // [dk] forget gate
  float* gs = fs + dk;         // [dk] 1 - forget gate
  float* qs = gs + dk;         // [dk] silu(q)
  float* vs = qs + dk;         // [dv]
  float* red = vs + dv;        // [KS][dv] partial outputs
  float* scratch = red + KS * dv;  // [33]
  const int r = blockIdx.x, hd = blockIdx.y;
  const bool live = threadIdx.x < dv * KS;  // the block is rounded up to whole warps
  const int j = live ? threadIdx.x % dv : 0, s = live ? threadIdx.x / dv : 0;
  const int i0 = s * rpt;
  const int n0 = cu_q[r], n1 = cu_q[r + 1];
  const int C = 2 * H * dk + H * dv;
  float* S_g = state + (((size_t)slot_ids[r] * H + hd) * dk) * dv;
  float S[REC_MAX_RPT];
#pragma unroll
  for (int ii = 0; ii < REC_MAX_RPT; ++ii) S[ii] = (live && ii < rpt && i0 + ii < dk) ? S_g[(size_t)(i0 + ii) * dv + j] : 0.f;
  const float nw = norm_w ? norm_w[j] : 1.f;

  for (int t = n0; t < n1; ++t) {
    const float* row = qfv + (size_t)t * C;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
      float qp = 0.f, fp = 0.f;
      for (int z = 0; z < splits; ++z) {
        qp += row[(size_t)z * split_stride + hd * dk + i];
        fp += row[(size_t)z * split_stride + H * dk + hd * dk + i];
      }
      fp += f_bias[hd * dk + i];
      const float lo = lower[hd * dk + i];
      const float f = lo + (1.f - lo) * (1.f / (1.f + expf(-fp)));
      fs[i] = f;
      gs[i] = 1.f - f;
      qs[i] = qp / (1.f + expf(-qp));
    }
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
      float v = 0.f;
      for (int z = 0; z < splits; ++z) v += row[(size_t)z * split_stride + 2 * H * dk + hd * dv + i];
      vs[i] = v;
    }
    __syncthreads();
    const float vj = vs[j];
    float acc = 0.f;
#pragma unroll
    for (int ii = 0; ii < REC_MAX_RPT; ++ii) {
      if (live && ii < rpt && i0 + ii < dk) {
        S[ii] = fmaf(fs[i0 + ii], S[ii], gs[i0 + ii] * vj);
        acc = fmaf(S[ii], qs[i0 + ii], acc);
      }
    }
    if (live) red[s * dv + j] = acc;
    __syncthreads();
    float o = 0.f;
    if (live && s == 0)
      for (int k = 0; k < KS; ++k) o += red[k * dv + j];
    const float ss = block_sum(live && s == 0 ? o * o : 0.f, scratch);  // syncs: fs/gs/qs/vs/red are free afterwards
    if (live && s == 0) out[(size_t)t * H * dv + hd * dv + j] = from_f32<TO>(o / sqrtf(ss / (float)dv + eps) * nw);
  }
#pragma unroll
  for (int ii = 0; ii < REC_MAX_RPT; ++ii)
    if (live && ii < rpt && i0 + ii < dk) S_g[(size_t)(i0 + ii) * dv + j] = S[ii];
}

JLX_API int jlx_hgrn2_scan(const float* qfv, int splits, long long split_stride, const float* f_bias, const float* lower,
                           float* state, const int* cu_q, const int* slot_ids, const float* norm_w, float eps, void* out,
                           int out_dtype, int R, int H, int dk, int dv, cudaStream_t stream) {
  JLX_REQUIRE(R >= 0 && H > 0 && dk > 0 && dv > 0 && splits >= 1, "hgrn2_scan: bad sizes R=%d H=%d dk=%d dv=%d", R, H, dk, dv);
  JLX_REQUIRE(dv <= 512, "hgrn2_scan: value size %d is above the supported maximum 512", dv);
  JLX_REQUIRE(eps > 0.f, "hgrn2_scan: eps must be positive");
  if (R == 0) return 0;
  // slices of the state's rows per column: enough that a thread keeps at most REC_MAX_RPT rows, and more while the
  // block stays small (a block of few threads walks its tokens no faster)
  int KS = 1;
  while (dv * KS * 2 <= 512 && ((dk + KS - 1) / KS > REC_MAX_RPT || (dv * KS < 256 && (dk + KS - 1) / KS > 4))) KS *= 2;
  const int rpt = (dk + KS - 1) / KS;
  JLX_REQUIRE(rpt <= REC_MAX_RPT, "hgrn2_scan: a state of %d x %d per head does not fit a block's registers", dk, dv);
  JLX_REQUIRE(H <= 65535, "hgrn2_scan: too many heads (%d)", H);
  const size_t smem = sizeof(float) * (3 * (size_t)dk + dv + (size_t)KS * dv + 33);
  JLX_DISPATCH_DTYPE(out_dtype, TO, {
    if (smem > 48 * 1024)
      JLX_CUDA(cudaFuncSetAttribute(hgrn2_scan_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    hgrn2_scan_kernel<TO><<<dim3(R, H), (dv * KS + 31) / 32 * 32, smem, stream>>>(qfv, splits, split_stride, f_bias, lower, state, cu_q, slot_ids,
                                                                  norm_w, eps, (TO*)out, H, dk, dv, KS, rpt);
  });
  JLX_LAUNCH_CHECK("hgrn2_scan");
  return 0;
}
