// y[M,N] = x[M,K] W[N,K]^T for a handful of rows: the single-token projections of a decode step
// (F.linear(x, qkvo_w[:3].flatten(0,1)) and F.linear(y, qkvo_w[3]) with x [B,1,dim], models/daisy/attention.py:119,201).
//
// HBM-bound on W: every weight row is read once per pass of up to 8 input rows.  A warp owns two weight rows at a
// time; each lane streams 16-byte pieces of them (all of a row's pieces are issued before the first is used), the
// matching pieces of the few x rows come through L1, and the 32 partial dot products of each (row, column) pair are
// folded with xor-shuffles.  bf16 in and out, fp32 accumulation.
#include "common.cuh"

namespace daisy {

constexpr int SK_WARPS = 4, SK_NR = 2, SK_MT = 8;

struct SkinnyParams {
  const __nv_bfloat16* x; int64_t ldx;
  const __nv_bfloat16* w; int64_t ldw;
  __nv_bfloat16* y; int64_t ldy;
  int M, N, K;
};

template <int MT>
__device__ __forceinline__ void skinny_pass(const SkinnyParams& p, int m0, int n0, int lane) {
  float acc[SK_NR][MT];
#pragma unroll
  for (int r = 0; r < SK_NR; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
  const __nv_bfloat16* w0 = p.w + (int64_t)n0 * p.ldw;
  const bool two = n0 + 1 < p.N;
  const __nv_bfloat16* w1 = w0 + (two ? p.ldw : 0);
#pragma unroll 4
  for (int k0 = lane * 8; k0 < p.K; k0 += 256) {
    const uint4 wa = ld_stream16(w0 + k0), wb = ld_stream16(w1 + k0);
    float fa[8], fb[8];
    unpack8(wa, fa);
    unpack8(wb, fb);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int mm = min(m0 + m, p.M - 1);                           // rows past M repeat the last one (never stored)
      float fx[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(p.x + (int64_t)mm * p.ldx + k0)), fx);
#pragma unroll
      for (int e = 0; e < 8; ++e) { acc[0][m] = fmaf(fa[e], fx[e], acc[0][m]); acc[1][m] = fmaf(fb[e], fx[e], acc[1][m]); }
    }
  }
#pragma unroll
  for (int r = 0; r < SK_NR; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && m0 + m < p.M && (r == 0 || two)) p.y[(int64_t)(m0 + m) * p.ldy + n0 + r] = __float2bfloat16_rn(v);
    }
}

__global__ void __launch_bounds__(32 * SK_WARPS) skinny_gemm_kernel(const SkinnyParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * SK_WARPS + warp) * SK_NR;
  if (n0 >= p.N) return;
  for (int m0 = 0; m0 < p.M; m0 += SK_MT) {
    const int left = p.M - m0;
    if (left == 1) skinny_pass<1>(p, m0, n0, lane);
    else if (left == 2) skinny_pass<2>(p, m0, n0, lane);
    else if (left <= 4) skinny_pass<4>(p, m0, n0, lane);
    else skinny_pass<SK_MT>(p, m0, n0, lane);
  }
}

}  // namespace daisy

using namespace daisy;

extern "C" int daisy_b200_gemm_skinny(const void* x, int64_t ldx, const void* w, int64_t ldw, void* y, int64_t ldy,
                                      int M, int N, int K, void* stream) {
  if (!x || !w || !y || M <= 0 || N <= 0 || K <= 0) return DAISY_EINVAL;
  if (M > 64 || (K & 7)) return DAISY_EUNSUPPORTED;
  if (!daisy_aligned16(x) || !daisy_aligned16(w) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K || ldy < N) return DAISY_EALIGN;
  SkinnyParams p{(const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, ldw, (__nv_bfloat16*)y, ldy, M, N, K};
  const int cols_per_block = SK_WARPS * SK_NR;
  skinny_gemm_kernel<<<(N + cols_per_block - 1) / cols_per_block, 32 * SK_WARPS, 0, (cudaStream_t)stream>>>(p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}
