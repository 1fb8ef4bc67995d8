// y[M,N] = x[M,K] W[N,K]^T for a handful of rows: the single-token projections of a decode step
// (F.linear(x, qkvo_w[:3].flatten(0,1)) and F.linear(y, qkvo_w[3]) with x [B,1,dim], models/daisy/attention.py:119,201).
//
// HBM-bound on W: every weight row is read once per pass of up to 8 input rows.  A warp owns two weight rows at a
// time; each lane streams 16-byte pieces of them (all of a row's pieces are issued before the first is used), the
// matching pieces of the few x rows come from a copy in shared memory, and the 32 partial dot products of each (row,
// column) pair are folded with xor-shuffles.  bf16 in and out, fp32 accumulation.
#include "common.cuh"

namespace daisy {

constexpr int SK_WARPS = 4, SK_NR = 2, SK_MT = 8;
constexpr size_t SK_SMEM_LIMIT = 160 * 1024;            // staged x rows
constexpr size_t SK_PREFETCH_LIMIT = 48u << 20;         // weights up to this size are hinted into L2 ahead of the wait

struct SkinnyParams {
  const __nv_bfloat16* x; int64_t ldx;
  const __nv_bfloat16* w; int64_t ldw;
  __nv_bfloat16* y; int64_t ldy;
  int M, N, K;
  int mt;                                                // x rows per pass (1, 2, 4 or 8): mt * K * 2 bytes of shared memory
  int prefetch;
};

// xs: the pass's x rows in shared memory, K elements each
template <int MT>
__device__ __forceinline__ void skinny_pass(const SkinnyParams& p, const __nv_bfloat16* xs, int rows, int m0, int n0, int lane) {
  float acc[SK_NR][MT];
#pragma unroll
  for (int r = 0; r < SK_NR; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
  const __nv_bfloat16* w0 = p.w + (int64_t)n0 * p.ldw;
  const bool two = n0 + 1 < p.N;
  const __nv_bfloat16* w1 = w0 + (two ? p.ldw : 0);
#pragma unroll 8
  for (int k0 = lane * 8; k0 < p.K; k0 += 256) {
    const uint4 wa = ld_stream16(w0 + k0), wb = ld_stream16(w1 + k0);
    float fa[8], fb[8];
    unpack8(wa, fa);
    unpack8(wb, fb);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int mm = min(m, rows - 1);                               // rows past M repeat the last one (never stored)
      float fx[8];
      unpack8(*reinterpret_cast<const uint4*>(xs + (size_t)mm * p.K + k0), fx);
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
      if (lane == 0 && m < rows && (r == 0 || two)) p.y[(int64_t)(m0 + m) * p.ldy + n0 + r] = __float2bfloat16_rn(v);
    }
}

// Launched as a dependent grid: before the wait it only asks L2 for the weight rows it owns (they do not depend on the
// preceding kernel; a hint is harmless even if they did), so in a chain of decode-step kernels the weights of this
// projection stream in while the previous kernel is still running.  x, which the previous kernel may have produced, is
// read after the wait, through L2, into shared memory.
__global__ void __launch_bounds__(32 * SK_WARPS) skinny_gemm_kernel(const SkinnyParams p) {
  extern __shared__ __align__(16) uint8_t sk_smem[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(sk_smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * SK_WARPS + warp) * SK_NR;
  if (p.prefetch && lane < SK_NR && n0 + lane < p.N) l2_prefetch_bulk(p.w + (int64_t)(n0 + lane) * p.ldw, (uint32_t)p.K * 2u);
  grid_dep_launch();
  grid_dep_wait();
  const int kv = p.K >> 3;                                           // 16-byte pieces per row
  for (int m0 = 0; m0 < p.M; m0 += p.mt) {
    const int rows = min(p.mt, p.M - m0);
    if (m0) __syncthreads();
    for (int idx = threadIdx.x; idx < rows * kv; idx += 32 * SK_WARPS) {
      const int r = idx / kv, c = idx - r * kv;
      reinterpret_cast<uint4*>(xs)[idx] = ld_cg16(p.x + (int64_t)(m0 + r) * p.ldx + c * 8);
    }
    __syncthreads();
    if (n0 >= p.N) continue;
    if (rows == 1) skinny_pass<1>(p, xs, rows, m0, n0, lane);
    else if (rows == 2) skinny_pass<2>(p, xs, rows, m0, n0, lane);
    else if (rows <= 4) skinny_pass<4>(p, xs, rows, m0, n0, lane);
    else skinny_pass<SK_MT>(p, xs, rows, m0, n0, lane);
  }
}

}  // namespace daisy

using namespace daisy;

extern "C" int daisy_b200_gemm_skinny(const void* x, int64_t ldx, const void* w, int64_t ldw, void* y, int64_t ldy,
                                      int M, int N, int K, void* stream) {
  if (!x || !w || !y || M <= 0 || N <= 0 || K <= 0) return DAISY_EINVAL;
  if (M > 64 || (K & 7)) return DAISY_EUNSUPPORTED;
  if (!daisy_aligned16(x) || !daisy_aligned16(w) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K || ldy < N) return DAISY_EALIGN;
  int mt = M > 4 ? SK_MT : (M > 2 ? 4 : M);
  while (mt > 1 && (size_t)mt * K * 2 > SK_SMEM_LIMIT) mt >>= 1;
  const size_t smem = (size_t)mt * K * 2;
  if (smem > SK_SMEM_LIMIT) return DAISY_EUNSUPPORTED;
  static bool attr[daisy_host::MAX_DEVICES] = {};                    // the attribute is per device
  const int dev = daisy_host::device_slot();
  if (dev < 0) return DAISY_ENODEV;
  if (!attr[dev]) {
    if (cudaFuncSetAttribute(skinny_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SK_SMEM_LIMIT) != cudaSuccess) {
      (void)cudaGetLastError();
      return DAISY_ECUDA;
    }
    attr[dev] = true;
  }
  SkinnyParams p{(const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, ldw, (__nv_bfloat16*)y, ldy, M, N, K, mt,
                 (size_t)N * K * 2 <= SK_PREFETCH_LIMIT ? 1 : 0};
  const int cols_per_block = SK_WARPS * SK_NR;
  if (daisy_host::launch_dependent(skinny_gemm_kernel, dim3((N + cols_per_block - 1) / cols_per_block), dim3(32 * SK_WARPS),
                                   smem, (cudaStream_t)stream, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return DAISY_ECUDA;
  }
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}
