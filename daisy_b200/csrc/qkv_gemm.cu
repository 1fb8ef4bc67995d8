// C[M,N] = X[M,K] W[N,K]^T on tcgen05 tensor cores, bf16 in, fp32 accumulation in TMEM, with the projection's
// element-wise tail as the epilogue.
//
// Two uses (the GEMMs either side of the attention core, models/daisy/attention.py:118-125 and :149):
//   EPI_QKV    W = qkvo_w[:3] flattened ([3*H*128, dim]): a 128-column output tile is one head of q, k or v of 128
//              tokens, so the weightless RMS norm over D and the half-rotation RoPE are per-thread work on the
//              accumulator row (thread = token = TMEM lane); q', k', v' leave as [B,T,H,D] bf16 and the separate
//              norm/RoPE pass over q, k, v (1.6 GB at B=8, T=8192, 16 heads) disappears.
//   EPI_PLAIN  bf16 store of C (the output projection).
//
// Persistent CTAs walk 128 x BN output tiles (n fastest, so concurrently running CTAs share X tiles and the
// whole W in L2).  Roles (192 threads): warps 0-3 epilogue, warp 4 TMA producer, warp 5 MMA issuer.  Both
// operands are K-major with 128-byte swizzle (64-element boxes), exactly the Q K^T operand form of the
// attention kernel; BN = 256 halves the shared-memory bytes read per flop against BN = 128 (the SS form of a
// 128 x 128 x 16 MMA reads 8 KB per 64 cycles, all the shared-memory pipe has).  Two accumulators in TMEM
// (2 x BN columns) let the epilogue of tile i run under the main loop of tile i + 1.
// PAIR form (N a multiple of 256): clusters of two CTAs on 256 x 256 tiles with cta_group::2 MMAs.  Each CTA loads its
// own 128 rows of X and its own 128 of the tile's 256 weight rows (plain per-CTA TMA loads), the pair's tensor cores
// read both weight halves, so the shared-memory fill and operand reads per flop drop by a third against the single-CTA
// 128 x 256 tile; rank 0 issues the MMAs, both CTAs run the epilogue on their own 128 accumulator rows.
// All mbarrier waits are bounded (abort flag, DAISY_ETIMEOUT through the status word), as everywhere else.
#include "common.cuh"
#include <cuda_fp16.h>

namespace daisy {

constexpr int GM = 128, GK = 64;
constexpr int G_THREADS = 192;
constexpr int G_A_BYTES = GM * GK * 2;                 // 16 KB
constexpr int G_STAGE_ROW = 256 + 16;                  // one staged output row (128 bf16) + pad: conflict-free 16-byte accesses
constexpr int G_STAGING = 4 * 16 * G_STAGE_ROW;        // per warp 16 rows at a time

template <int BN, bool PAIR> struct GemmCfg {
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;    // weight rows this CTA keeps per stage
  static constexpr int B_BYTES = B_ROWS * GK * 2;
  static constexpr int STAGE = G_A_BYTES + B_BYTES;
  static constexpr int NST = (BN == 256 && !PAIR) ? 4 : 6;
  static constexpr int SMEM = 1024 + NST * STAGE + G_STAGING + 256;
  static constexpr int TILE_M = PAIR ? 2 * GM : GM;
};

struct GemmParams {
  int M, N, K;
  int epi;                       // 0 plain, 1 qkv
  // plain
  __nv_bfloat16* c; int64_t ldc;
  // qkv
  __nv_bfloat16* out[3];         // q', k', v'  [M, H, 128]
  const float *cos, *sin;        // [T, 64]
  const __nv_bfloat16* ve;       // value embedding [M, H, 128] (row stride ve_ld elements) or null
  int64_t ve_ld;
  const float* ve_gate_logit;    // v' = g * norm(v) + (1 - g) * ve, g = sigmoid(*ve_gate_logit)
  int T, H;
  float eps;
  unsigned flags;
  int* status;
  // optional ring-cache side output: rows t >= ring_first of k' (ring[0]) and v' (ring[1]) also go to slot t % cap of
  // a [B,H,cap,128] ring with element strides (r_sb, r_sh, r_sr); bf16 or (ring_f16) float16 rows
  void* ring[2];
  int64_t r_sb, r_sh, r_sr;
  int cap, ring_first, ring_f16;
};

struct GemmBars {
  uint64_t full[6], empty[6];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int BN, bool PAIR>
__global__ void __launch_bounds__(G_THREADS, 1)
qkv_gemm_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const GemmParams p) {
  using Cfg = GemmCfg<BN, PAIR>;
  extern __shared__ uint8_t gemm_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint8_t* staging = smem + Cfg::NST * Cfg::STAGE;
  GemmBars* bars = reinterpret_cast<GemmBars*>(staging + G_STAGING);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + Cfg::TILE_M - 1) / Cfg::TILE_M, n_tiles = p.N / BN, kb_n = p.K / GK;
  const int tiles = m_tiles * n_tiles;
  // PAIR: the work item belongs to the cluster; rank 0 issues the MMAs, rank r owns rows r * 128 .. of the tile
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::NST; ++i) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->acc_full[i], 1); mbar_init(&bars->acc_empty[i], PAIR ? 256 : 128); }
    bars->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 5) {
    if (PAIR) { tmem_alloc_pair(&bars->tmem_base, 2 * BN); tmem_relinquish_pair(); }
    else { tmem_alloc(&bars->tmem_base, 2 * BN); tmem_relinquish(); }
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all();                        // the peer's barriers exist before anything arrives on them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tm_x); prefetch_tmap(&tm_w);
      uint32_t n = 0;
      bool ok = true;
      for (int tile = worker; tile < tiles && ok; tile += workers) {
        const int m0 = (tile / n_tiles) * Cfg::TILE_M + (int)rank * GM, n0 = (tile % n_tiles) * BN + (int)rank * Cfg::B_ROWS;
        for (int kb = 0; kb < kb_n; ++kb, ++n) {
          const int st = n % Cfg::NST;
          if (!mbar_wait(&bars->empty[st], ((n / Cfg::NST) & 1) ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
          uint8_t* dst = stages + st * Cfg::STAGE;
          if (PAIR) {
            // both CTAs' bytes are counted on rank 0's barrier, which the MMA issuer waits on
            const uint32_t full0 = mapa_shared(smem_u32(&bars->full[st]), 0);
            if (rank == 0) mbar_expect_tx(&bars->full[st], 2 * Cfg::STAGE);
            tma_load_3d_pair(dst, &tm_x, full0, kb * GK, m0, 0);
            tma_load_3d_pair(dst + G_A_BYTES, &tm_w, full0, kb * GK, n0, 0);
          } else {
            mbar_expect_tx(&bars->full[st], Cfg::STAGE);
            tma_load_3d(dst, &tm_x, &bars->full[st], kb * GK, m0, 0);
            tma_load_3d(dst + G_A_BYTES, &tm_w, &bars->full[st], kb * GK, n0, 0);
          }
        }
      }
    }
  } else if (warp == 5 && rank == 0) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t leader = elect_one() ? 1u : 0u;
    constexpr uint32_t idesc = umma_idesc_bf16(Cfg::TILE_M, BN, 0, 0);
    const uint64_t ad = umma_desc_sw128(smem_u32(stages), 16, 1024);
    const uint64_t bd = umma_desc_sw128(smem_u32(stages + G_A_BYTES), 16, 1024);
    const uint32_t a_lo0 = (uint32_t)ad, b_lo0 = (uint32_t)bd, hi = (uint32_t)(ad >> 32);
    uint32_t n = 0, it = 0;
    bool ok = true;
    for (int tile = worker; tile < tiles && ok; tile += workers, ++it) {
      const uint32_t buf = it & 1;
      if (!mbar_wait(&bars->acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag, p.status, 2)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * BN;
      for (int kb = 0; kb < kb_n; ++kb, ++n) {
        const int st = n % Cfg::NST;
        if (!mbar_wait(&bars->full[st], (n / Cfg::NST) & 1, abort_flag, p.status, 3)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_lo = a_lo0 + st * (Cfg::STAGE >> 4), b_lo = b_lo0 + st * (Cfg::STAGE >> 4);
#pragma unroll
        for (int k = 0; k < GK / 16; ++k) {
          if (PAIR) umma_ss_pair_p(leader, d_tmem, a_lo + k * 2, hi, b_lo + k * 2, hi, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          else umma_ss_lh_p(leader, d_tmem, a_lo + k * 2, hi, b_lo + k * 2, hi, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        if (PAIR) tc_commit_pair_p(leader, &bars->empty[st]);       // both CTAs' producers may refill the stage
        else tc_commit_p(leader, &bars->empty[st]);
      }
      if (ok) {
        if (PAIR) tc_commit_pair_p(leader, &bars->acc_full[buf]);
        else tc_commit_p(leader, &bars->acc_full[buf]);
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ epilogue: thread = output row
    const int row = warp * 32 + lane;
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    uint8_t* stg = staging + warp * 16 * G_STAGE_ROW;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = worker; tile < tiles && ok; tile += workers, ++it) {
      const uint32_t buf = it & 1;
      const int m0 = (tile / n_tiles) * Cfg::TILE_M + (int)rank * GM, n0 = (tile % n_tiles) * BN;
      const int m = m0 + row;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_full[buf], (it >> 1) & 1, abort_flag, p.status, 4));
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int half = 0; half < BN / 128; ++half) {
        uint32_t r[128];
        const uint32_t t0 = tmem_base + lane_off + buf * BN + half * 128;
        tmem_ld32(t0, r); tmem_ld32(t0 + 32, r + 32); tmem_ld32(t0 + 64, r + 64); tmem_ld32(t0 + 96, r + 96);
        tc_wait_ld();
        if (half == BN / 128 - 1) {                                // accumulator read out: the MMA warp may refill it
          tc_fence_before();
          if (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&bars->acc_empty[buf]), 0));   // the issuer waits for both CTAs
          else mbar_arrive(&bars->acc_empty[buf]);
        }
        __nv_bfloat16* dst_row;                                    // this thread's output row (128 bf16)
        uint8_t* ring_row = nullptr;
        if (p.epi == 1) {
          const int nh = (n0 + half * 128) >> 7;                   // head slot among 3 H
          const int which = nh / p.H, h = nh - which * p.H;
          const bool do_norm = (p.flags & (which == 0 ? DAISY_NORM_Q : which == 1 ? DAISY_NORM_K : DAISY_NORM_V)) != 0;
          if (do_norm) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 128; ++i) { const float x = __uint_as_float(r[i]); ss = fmaf(x, x, ss); }
            const float rs = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
#pragma unroll
            for (int i = 0; i < 128; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * rs);
          }
          if (which < 2 && (p.flags & DAISY_ROPE)) {
            const int pos = min(m, p.M - 1) % p.T;
            const float4* cr = reinterpret_cast<const float4*>(p.cos + (size_t)pos * 64);
            const float4* sr = reinterpret_cast<const float4*>(p.sin + (size_t)pos * 64);
#pragma unroll
            for (int i4 = 0; i4 < 16; ++i4) {
              const float4 c = cr[i4], s = sr[i4];
              const float cc[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = 4 * i4 + e;
                const float a = __uint_as_float(r[i]), b2 = __uint_as_float(r[i + 64]);
                r[i] = __float_as_uint(a * cc[e] + b2 * sn[e]);
                r[i + 64] = __float_as_uint(b2 * cc[e] - a * sn[e]);
              }
            }
          }
          if (which == 2 && p.ve) {                                // value-embedding gate on the normalised v
            const float gte = 1.0f / (1.0f + __expf(-*p.ve_gate_logit));
            const uint4* vr = reinterpret_cast<const uint4*>(p.ve + (size_t)min(m, p.M - 1) * p.ve_ld + h * 128);
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              float f[8];
              unpack8(vr[c], f);
#pragma unroll
              for (int e = 0; e < 8; ++e) r[8 * c + e] = __float_as_uint(gte * __uint_as_float(r[8 * c + e]) + (1.0f - gte) * f[e]);
            }
          }
          dst_row = p.out[which] + ((size_t)m * p.H + h) * 128;
          if (which >= 1 && p.ring[which - 1] && m < p.M) {        // this row's slot in the ring cache, if it is kept
            const int b = m / p.T, t = m - b * p.T;
            if (t >= p.ring_first)
              ring_row = reinterpret_cast<uint8_t*>(p.ring[which - 1]) + ((int64_t)b * p.r_sb + (int64_t)h * p.r_sh + (int64_t)(t % p.cap) * p.r_sr) * 2;
          }
        } else {
          dst_row = p.c + (size_t)m * p.ldc + n0 + half * 128;
        }
        // bf16 pack, then through the warp's staging rows so that each store instruction writes two whole rows
        uint4 ch[16];
#pragma unroll
        for (int c = 0; c < 16; ++c)
          ch[c] = make_uint4(pack_bf16(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1])),
                             pack_bf16(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3])),
                             pack_bf16(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5])),
                             pack_bf16(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7])));
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          if ((lane >> 4) == pass) {
#pragma unroll
            for (int c = 0; c < 16; ++c) *reinterpret_cast<uint4*>(stg + (lane & 15) * G_STAGE_ROW + c * 16) = ch[c];
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = 2 * i + (lane >> 4);                    // staged row, = warp row 16 pass + rr
            const uint4 val = *reinterpret_cast<const uint4*>(stg + rr * G_STAGE_ROW + (lane & 15) * 16);
            const int src_lane = 16 * pass + rr;
            // the row's global address lives in the lane that owns the row
            const unsigned long long base = __shfl_sync(0xffffffffu, (unsigned long long)reinterpret_cast<uintptr_t>(dst_row), src_lane);
            const int mm = __shfl_sync(0xffffffffu, m, src_lane);
            if (mm < p.M) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(base) + (lane & 15) * 16) = val;
            if (p.epi == 1 && p.ring[0]) {                         // warp-uniform: a ring is attached to this call
              const unsigned long long rb = __shfl_sync(0xffffffffu, (unsigned long long)reinterpret_cast<uintptr_t>(ring_row), src_lane);
              if (rb) {
                uint4 rv = val;
                if (p.ring_f16) {                                  // the ring keeps float16 rows
                  float f[8];
                  unpack8(val, f);
                  const __half2 h0 = __floats2half2_rn(f[0], f[1]), h1 = __floats2half2_rn(f[2], f[3]);
                  const __half2 h2 = __floats2half2_rn(f[4], f[5]), h3 = __floats2half2_rn(f[6], f[7]);
                  rv = make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                                  *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
                }
                *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(rb) + (lane & 15) * 16) = rv;
              }
            }
          }
          __syncwarp();
        }
      }
    }
  }

  tc_fence_before();
  if (PAIR) cluster_sync_all();                        // neither CTA leaves while the other may still read its operands
  else __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, 2 * BN);
    else tmem_dealloc(tmem_base, 2 * BN);
  }
}

}  // namespace daisy

using namespace daisy;

template <int BN, bool PAIR>
static int launch_gemm(const CUtensorMap& tx, const CUtensorMap& tw, const GemmParams& p, cudaStream_t st) {
  using Cfg = GemmCfg<BN, PAIR>;
  static_assert(Cfg::SMEM <= 232448, "over the 227 KB a CTA may use");
  static bool attr[daisy_host::MAX_DEVICES] = {};
  static int max_clusters[daisy_host::MAX_DEVICES] = {};
  const int dev = daisy_host::device_slot();
  if (dev < 0) return DAISY_ENODEV;
  const int sms = daisy_host::sm_count_cached();
  if (sms <= 0) return DAISY_ENODEV;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(G_THREADS); cfg.dynamicSmemBytes = Cfg::SMEM; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  if (PAIR) { cfg.attrs = at; cfg.numAttrs = 1; }
  if (!attr[dev]) {
    if (cudaFuncSetAttribute(qkv_gemm_kernel<BN, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) {
      (void)cudaGetLastError();
      return DAISY_ECUDA;
    }
    if (PAIR) {                                          // how many CTA pairs the device can hold at once
      cfg.gridDim = dim3((unsigned)(sms & ~1));
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, qkv_gemm_kernel<BN, PAIR>, &cfg) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return DAISY_ECUDA;
      }
      max_clusters[dev] = n;
    }
    attr[dev] = true;
  }
  const int64_t tiles = (int64_t)((p.M + Cfg::TILE_M - 1) / Cfg::TILE_M) * (p.N / BN);
  if (PAIR) {
    const int64_t pairs = tiles < max_clusters[dev] ? tiles : max_clusters[dev];
    cfg.gridDim = dim3((unsigned)(2 * pairs));
  } else {
    cfg.gridDim = dim3((unsigned)(tiles < sms ? tiles : sms));
  }
  if (cudaLaunchKernelEx(&cfg, qkv_gemm_kernel<BN, PAIR>, tx, tw, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return DAISY_ECUDA;
  }
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}

static int gemm_common(const void* x, int64_t ldx, const void* w, int64_t ldw, GemmParams& p, void* stream) {
  if (!x || !w || p.M <= 0 || p.N <= 0 || p.K <= 0) return DAISY_EINVAL;
  if (p.K % GK != 0 || p.N % 128 != 0) return DAISY_EUNSUPPORTED;
  if (!daisy_aligned16(x) || !daisy_aligned16(w) || (ldx & 7) || (ldw & 7) || ldx < p.K || ldw < p.K) return DAISY_EALIGN;
  const bool pair = p.N % 256 == 0 && p.M > GM;        // CTA pairs on 256 x 256 tiles; else one CTA per 128 x 128 tile
  CUtensorMap tx, tw;
  int rc;
  if ((rc = daisy_host::make_tmap_bf16_3d(&tx, x, p.K, p.M, 1, (uint64_t)ldx * 2, (uint64_t)ldx * 2 * p.M, GK, GM)) != DAISY_OK) return rc;
  if ((rc = daisy_host::make_tmap_bf16_3d(&tw, w, p.K, p.N, 1, (uint64_t)ldw * 2, (uint64_t)ldw * 2 * p.N, GK, 128)) != DAISY_OK) return rc;
  return pair ? launch_gemm<256, true>(tx, tw, p, (cudaStream_t)stream) : launch_gemm<128, false>(tx, tw, p, (cudaStream_t)stream);
}

extern "C" int daisy_b200_gemm_nt(const void* x, int64_t ldx, const void* w, int64_t ldw, void* c, int64_t ldc,
                                  int M, int N, int K, int* status_word, void* stream) {
  if (!c) return DAISY_EINVAL;
  if (!daisy_aligned16(c) || (ldc & 7) || ldc < N) return DAISY_EALIGN;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.epi = 0;
  p.c = (__nv_bfloat16*)c; p.ldc = ldc; p.status = status_word;
  return gemm_common(x, ldx, w, ldw, p, stream);
}

extern "C" int daisy_b200_qkv_gemm(const void* x, int64_t ldx, const void* w_qkv, int64_t ldw,
                                   const float* cos, const float* sin,
                                   void* q_out, void* k_out, void* v_out,
                                   const void* ve, int64_t ve_ld, const float* ve_gate_logit,
                                   int B, int T, int H, int D, int dim, float eps, unsigned flags,
                                   int* status_word, void* stream) {
  return daisy_b200_qkv_gemm_ring(x, ldx, w_qkv, ldw, cos, sin, q_out, k_out, v_out, ve, ve_ld, ve_gate_logit,
                                  nullptr, nullptr, 0, 0, 0, 0, 0, B, T, H, D, dim, eps, flags, status_word, stream);
}

extern "C" int daisy_b200_qkv_gemm_ring(const void* x, int64_t ldx, const void* w_qkv, int64_t ldw,
                                        const float* cos, const float* sin,
                                        void* q_out, void* k_out, void* v_out,
                                        const void* ve, int64_t ve_ld, const float* ve_gate_logit,
                                        void* ring_k, void* ring_v, int64_t r_sb, int64_t r_sh, int64_t r_sr,
                                        int cap, int ring_first,
                                        int B, int T, int H, int D, int dim, float eps, unsigned flags,
                                        int* status_word, void* stream) {
  if (!q_out || !k_out || !v_out || B <= 0 || T <= 0 || H <= 0) return DAISY_EINVAL;
  if (D != DAISY_HEAD_DIM) return DAISY_EUNSUPPORTED;
  if ((int64_t)B * T >= (int64_t)1 << 31) return DAISY_EUNSUPPORTED;
  if (flags & ~(DAISY_QKV_DEFAULT | DAISY_CACHE_FP16)) return DAISY_EINVAL;
  if ((ring_k == nullptr) != (ring_v == nullptr)) return DAISY_EINVAL;
  if (ring_k) {
    if (cap <= 0 || ring_first < 0 || T - ring_first > cap) return DAISY_EINVAL;          // the kept rows would alias in the ring
    if (!daisy_aligned16(ring_k) || !daisy_aligned16(ring_v) || ((r_sb | r_sh | r_sr) & 7)) return DAISY_EALIGN;
  }
  if ((flags & DAISY_ROPE) && (!cos || !sin)) return DAISY_EINVAL;
  if ((flags & DAISY_ROPE) && (!daisy_aligned16(cos) || !daisy_aligned16(sin))) return DAISY_EALIGN;
  if (!daisy_aligned16(q_out) || !daisy_aligned16(k_out) || !daisy_aligned16(v_out)) return DAISY_EALIGN;
  if (ve && (!ve_gate_logit || !daisy_aligned16(ve) || (ve_ld & 7) || ve_ld < (int64_t)H * D)) return ve_gate_logit ? DAISY_EALIGN : DAISY_EINVAL;
  GemmParams p{};
  p.ve = (const __nv_bfloat16*)ve; p.ve_ld = ve_ld; p.ve_gate_logit = ve_gate_logit;
  p.M = B * T; p.N = 3 * H * D; p.K = dim; p.epi = 1;
  p.out[0] = (__nv_bfloat16*)q_out; p.out[1] = (__nv_bfloat16*)k_out; p.out[2] = (__nv_bfloat16*)v_out;
  p.cos = cos; p.sin = sin; p.T = T; p.H = H; p.eps = eps; p.flags = flags & DAISY_QKV_DEFAULT; p.status = status_word;
  p.ring[0] = ring_k; p.ring[1] = ring_v; p.r_sb = r_sb; p.r_sh = r_sh; p.r_sr = r_sr;
  p.cap = cap; p.ring_first = ring_first; p.ring_f16 = (flags & DAISY_CACHE_FP16) ? 1 : 0;
  return gemm_common(x, ldx, w_qkv, ldw, p, stream);
}
