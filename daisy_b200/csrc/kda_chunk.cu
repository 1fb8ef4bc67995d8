// Kimi delta attention (KDA), chunked forward, chunk = 64, K = V = 128.
//
// Per head the recurrence  S <- diag(e^{g_t}) S;  u_t = beta_t (v_t - S^T k_t);  S <- S + k_t u_t^T;
// o_t = S^T (scale q_t)  is evaluated 64 tokens at a time.  With G_i the inclusive cumulative
// log-decay inside a chunk and S_0 the state entering it:
//     A_kk[i,j] = beta_i sum_c k_ic k_jc e^{G_ic-G_jc} (j < i)     A_qk[i,j] = scale sum_c q_ic k_jc e^{G_ic-G_jc} (j <= i)
//     T = (I + A_kk)^-1          W = T (beta k e^G)          U0 = T (beta v)
//     U = U0 - W S_0             O = (scale q e^G) S_0 + A_qk U          S_C = e^{G_C} S_0 + (k e^{G_C-G})^T U
// Two kernels:
//  * kda_intra_kernel  -- everything that does not depend on the state, all chunks in parallel, on tcgen05 tensor
//    cores: a persistent CTA per SM walks (batch, head, chunk) work items; 16 "element" warps turn the TMA-staged
//    inputs into fp16 operand images and issue the Gram products on them, 8 "solver" warps pull the Gram entries
//    out of TMEM and solve (I + A_kk) W = beta k e^G, (I + A_kk) U0 = beta v block by block with register-chained
//    mma.sync tiles -- two pipelines that overlap across consecutive chunks.  Per chunk it writes a record of fp16 operand images (rows padded so that fragment loads
//    are bank-conflict free): W^T, (scale q e^G)^T, (k e^{G_C-G})^T, U0^T as [128][72], A_qk as [64][72], e^{G_C}.
//  * kda_state_kernel  -- one CTA per (batch, head, V-slice), sequential over chunks: a producer warp
//    bulk-copies the images of chunk c+1.. into a shared-memory ring while the compute warps hold their
//    slice of S^T (16 V-rows x 128 K-columns per warp) in fp32 accumulator registers and chain the
//    three products through register-resident fragments (an accumulator tile pair is exactly the next
//    product's A fragment), so the state never leaves the register file between chunks.  With few (batch, head)
//    pairs per GPU two warps share a slice, each holding half of the K-columns.
// Tensor-core operands are fp16 (10-bit mantissa, every decay factor and operand here is <= O(1)):
// measured relative error of o against the fp32 token recurrence is ~4e-4, bf16 operands give ~3e-3.
#include <cuda_fp16.h>
#include "common.cuh"

namespace daisy {

constexpr int KC = 64;                 // chunk length
constexpr int KD = 128;                // K = V
constexpr int LDT = 72;                // padded row (halves) of a [. x 64] image
constexpr int IMG_T = KD * LDT * 2;    // one [128][72] fp16 image: 18432 bytes
// per-chunk record in the workspace (bytes)
constexpr int OFF_WT = 0;                              // W^T      [128][72] fp16
constexpr int OFF_QT = OFF_WT + IMG_T;                 // q~^T     [128][72] fp16   (scale q e^G)^T
constexpr int OFF_KT = OFF_QT + IMG_T;                 // k~^T     [128][72] fp16   (k e^{G_C-G})^T
constexpr int OFF_AQK = OFF_KT + IMG_T;                // A_qk     [64][72]  fp16
constexpr int OFF_D = OFF_AQK + KC * LDT * 2;          // e^{G_C}  [128]     fp32
constexpr int SHARED_BYTES = OFF_D + KD * 4;           // 65024: identical for every V-slice
constexpr int OFF_UT = SHARED_BYTES;                   // U0^T     [128][72] fp16
constexpr int REC_BYTES = OFF_UT + IMG_T;              // 83456
static_assert(SHARED_BYTES % 16 == 0 && REC_BYTES % 16 == 0, "bulk copies move 16-byte units");

// Four 8x8 fp16 matrices from shared memory: lanes 8m..8m+7 give the row addresses of matrix m (16 bytes per
// row); register m of lane l then holds elements (row l/4, columns 2(l%4), 2(l%4)+1) of matrix m -- the B
// fragment layout of mma.m16n8k16 when the rows are the n index and the columns the k index.
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* row_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(row_ptr)));
}
// The transposing form: register m of lane l holds elements (rows 2(l%4), 2(l%4)+1, column l/4) of matrix m --
// the same B fragment when the stored rows are the k index and the columns the n index.
__device__ __forceinline__ void ldmatrix_x4_t(uint32_t* r, const void* row_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(row_ptr)));
}

__device__ __forceinline__ void mma_f16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_h2(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void st_global16(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// =============================================================================================
// intra-chunk kernel
// =============================================================================================
//
// Gated Gram matrices without a single positive exponent.  e^{G_i - G_j} (i > j) is needed per channel inside the
// contraction over channels, so it must factor into a row term times a column term, and neither term may overflow
// whatever the gates are.  Pairs are split by the highest bit in which i and j differ ("level" s = 1, 2, .., 32):
// tokens fall into aligned groups of 2s, i lies in the upper half of its group, j in the lower half.  With r the
// last row of the lower half,  e^{G_i - G_j} = e^{G_i - G_r} * e^{G_r - G_j}:  the row factor is the product of the
// per-token decays d_t = e^{g_t} <= 1 from the start of the upper half up to i, the column factor their product from
// j + 1 to the end of the lower half.  Every factor is a running product of numbers <= 1 -- ONE exponential per
// input element, no cumulative sum, and underflow is the correct limit.  A level is then one plain product
//      [ k * f ; q * f ]  (128 x 128 channels)   x   (k * f)^T  (128 channels x 64)      f = the level's factor per token
// whose entries at (i upper, j lower, same group) are that level's Gram entries (everything else is ignored): six
// 128 x 64 x 128 tcgen05 products per chunk with fp16 operand images staged in shared memory and fp32
// accumulators in TMEM.  The prefix / suffix products are carried from one level to the next with one multiply per
// element; after the last level they are e^{G} and e^{G_C - G}, the decay factors of the state-pass operands.
struct KdaIntraParams {
  const float* beta;
  uint8_t* ws;
  int T, H, NC;            // NC = chunks per sequence
  int total;               // work items: B * H * NC
  float scale;
  int l2norm;
  int* status;
  // packed variable-length sequences (B = 1): chunk c of the packed row covers tokens chunk_tab[2c] .. + chunk_tab[2c+1]
  // (1..64 of them; chunks never straddle a sequence boundary); null: chunk c covers tokens 64 c ..
  const int* chunk_tab;
};

constexpr int KI_ELEM_WARPS = 16, KI_SOLVER_WARPS = 8;
constexpr int KI_ELEM_THREADS = 32 * KI_ELEM_WARPS;                         // 512
constexpr int KI_SOLVER_THREADS = 32 * KI_SOLVER_WARPS;                     // 256
// 24 warps = 6 per scheduler: 80 registers per thread
constexpr int KI_THREADS = KI_ELEM_THREADS + KI_SOLVER_THREADS;             // 768
constexpr int KI_IMG_BYTES = KD * KC * 2;                                   // one [128 channels][64 tokens] fp16 image: 16384
constexpr int KI_IN_BYTES = KC * KD * 4 + 2 * KC * KD * 2;                  // g + q + k tiles: 65536
constexpr int LDAKH = 72;
constexpr int KI_SETS = 2;              // operand image sets in flight; divides the six levels of a chunk

struct __align__(1024) KdaIntraSmem {
  uint8_t img[KI_SETS][2 * KI_IMG_BYTES];   // level operand images, a ring of sets of (k image, q image); 128-byte swizzle
  float g[KC][KD];                       // TMA destinations, plain rows
  __nv_bfloat16 q[KC][KD];
  __nv_bfloat16 k[KC][KD];
  __nv_bfloat16 v[KC][KD];
  __half xt[KD][LDT];                    // (k e^G)^T, fp16: right-hand side of the W solve
  float akk_t[4][16][16];                // beta * A_kk, the four diagonal 16 x 16 blocks in fp32, column-major ([j][i])
  __half akh[KC][LDAKH];                 //              the whole lower triangle as fp16 operands
  __half th[KC][LDT];                    // the inverses of the diagonal blocks of I + A_kk, row-major, fp16
  float tot[4][KD];                      // product of the decays of each 16-token segment
  float rq[2][KC], rk[2][KC], beta[2][KC], qkd[2][KC];   // per-token scalars, double-buffered by chunk parity
  float sbeta[KC];                       // the solver's own copy
  uint64_t in_full, v_full, x_full, x_empty;
  uint64_t img_full[KI_SETS], img_empty[KI_SETS], d_full[6], d_empty[6];
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(KdaIntraSmem) + 1024 <= 232448, "over the 227 KB a CTA may use");

// byte offset of (row, 16-byte chunk) inside a 128-byte-swizzled image whose rows are 128 bytes
__device__ __forceinline__ uint32_t sw128(int row, int chunk) {
  return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + (((chunk ^ row) & 7) << 4));
}

__device__ __forceinline__ void ki_coords(int w, int NC, int H, int& b, int& h, int& chunk) {
  chunk = w % NC;
  const int bh = w / NC;
  h = bh % H;
  b = bh / H;
}
// first token and number of tokens of a chunk
__device__ __forceinline__ void ki_chunk_span(const int* chunk_tab, int chunk, int T, int& t0, int& rows) {
  if (chunk_tab) { t0 = chunk_tab[2 * chunk]; rows = chunk_tab[2 * chunk + 1]; }
  else { t0 = chunk * KC; rows = min(KC, T - t0); }
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// One level's operand images (this thread's 16 tokens of channel c; kn / qn hold them as fp16 pairs) into the image
// set of the level's turn, then -- one warp per level, so that no warp falls far behind the others -- the level's
// Gram product once every element thread has delivered its share.
__device__ __forceinline__ void ki_emit_level(KdaIntraSmem& sm, const float (&f)[16], const uint32_t (&kn)[8], const uint32_t (&qn)[8],
                                              const bool write_q, const int c, const int seg, const int warp, const uint32_t leader,
                                              const uint32_t ci, uint32_t& n_img, bool& ok, const uint32_t tmem_base,
                                              const uint32_t g_lo0, const uint32_t g_hi, volatile int* abort_flag, int* status) {
  constexpr uint32_t idesc_g = umma_idesc_f16(128, KC, 1, 1);                   // A and B both token-contiguous (MN-major)
  const uint32_t set = n_img % KI_SETS, use = n_img / KI_SETS;
  uint32_t fh[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) fh[i] = pack_h2(f[2 * i], f[2 * i + 1]);
  if (use >= 1) ok = mbar_wait_long(&sm.img_empty[set], (use - 1) & 1, abort_flag, status, 2) && ok;
  uint8_t* kimg = sm.img[set];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const uint32_t off = sw128(c, 2 * seg + e);
    *reinterpret_cast<uint4*>(kimg + off) = make_uint4(hmul2_u32(kn[4 * e], fh[4 * e]), hmul2_u32(kn[4 * e + 1], fh[4 * e + 1]),
                                                       hmul2_u32(kn[4 * e + 2], fh[4 * e + 2]), hmul2_u32(kn[4 * e + 3], fh[4 * e + 3]));
    if (write_q)
      *reinterpret_cast<uint4*>(kimg + KI_IMG_BYTES + off) = make_uint4(hmul2_u32(qn[4 * e], fh[4 * e]), hmul2_u32(qn[4 * e + 1], fh[4 * e + 1]),
                                                                        hmul2_u32(qn[4 * e + 2], fh[4 * e + 2]), hmul2_u32(qn[4 * e + 3], fh[4 * e + 3]));
  }
  fence_proxy_async();
  mbar_arrive(&sm.img_full[set]);
  const int li = (int)(n_img % 6u);
  if (warp == li) {                                                             // level li's product is issued by element warp li
    ok = mbar_wait_long(&sm.img_full[set], use & 1, abort_flag, status, 4) && ok;
    if (ci >= 1) ok = mbar_wait_long(&sm.d_empty[li], (ci - 1) & 1, abort_flag, status, 5) && ok;
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const uint32_t lo = g_lo0 + set * ((2 * KI_IMG_BYTES) >> 4);
#pragma unroll
      for (int ks = 0; ks < KD / 16; ++ks)                                      // 16 channels = 16 rows of 128 bytes per step
        umma_ss_lh_p(leader, tmem_base + 64 * li, lo + ks * (2048 >> 4), g_hi, lo + ks * (2048 >> 4), g_hi, idesc_g, ks > 0 ? 1u : 0u);
    }
    tc_commit_p(leader, &sm.img_empty[set]);                                    // arrives at once when nothing was issued
    tc_commit_p(leader, &sm.d_full[li]);
  }
  ++n_img;
}

// Level S < 16: the factor of token i is pre[i] if bit S of i is set, else suf[i]; afterwards both products are carried
// from aligned blocks of S to blocks of 2 S (upper block: prefix times the lower block's total; lower block: suffix
// times the upper block's total).
template <int S, typename Emit>
__device__ __forceinline__ void ki_level_inreg(float (&pre)[16], float (&suf)[16], Emit& emit) {
  float f[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) f[i] = (i & S) ? pre[i] : suf[i];
  emit(f, true);
#pragma unroll
  for (int a = 0; a < 16; a += 2 * S) {
    const float tot_l = pre[a + S - 1], tot_u = pre[a + 2 * S - 1];
#pragma unroll
    for (int i = 0; i < S; ++i) { pre[a + S + i] *= tot_l; suf[a + i] *= tot_u; }
  }
}

__global__ void __launch_bounds__(KI_THREADS, 1)
kda_intra_kernel(const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const KdaIntraParams p) {
  extern __shared__ uint8_t kda_smem_raw[];
  KdaIntraSmem& sm = *reinterpret_cast<KdaIntraSmem*>((reinterpret_cast<uintptr_t>(kda_smem_raw) + 1023) & ~uintptr_t(1023));
  volatile int* abort_flag = &sm.abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    mbar_init(&sm.in_full, 1); mbar_init(&sm.v_full, 1);
    mbar_init(&sm.x_full, KI_ELEM_THREADS); mbar_init(&sm.x_empty, 1);
    for (int i = 0; i < KI_SETS; ++i) { mbar_init(&sm.img_full[i], KI_ELEM_THREADS); mbar_init(&sm.img_empty[i], 1); }
    for (int i = 0; i < 6; ++i) { mbar_init(&sm.d_full[i], 1); mbar_init(&sm.d_empty[i], KI_SOLVER_THREADS); }
    sm.abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 0) { tmem_alloc(&sm.tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;

  if (warp < KI_ELEM_WARPS) {
    // ================================================================== element warps
    const int c = tid & (KD - 1), seg = tid >> 7;          // this thread's channel and 16-token segment (warp-uniform)
    if (tid == 0 && (int)blockIdx.x < p.total) {
      int b, h, chunk, ft0, frows;
      ki_coords(blockIdx.x, p.NC, p.H, b, h, chunk);
      ki_chunk_span(p.chunk_tab, chunk, p.T, ft0, frows);
      prefetch_tmap(&tm_g); prefetch_tmap(&tm_q); prefetch_tmap(&tm_k);
      mbar_expect_tx(&sm.in_full, KI_IN_BYTES);
      tma_load_4d(&sm.g[0][0], &tm_g, &sm.in_full, 0, ft0, h, b);
      tma_load_4d(&sm.q[0][0], &tm_q, &sm.in_full, 0, ft0, h, b);
      tma_load_4d(&sm.k[0][0], &tm_k, &sm.in_full, 0, ft0, h, b);
    }
    // warps 0..5 double as the issuers of the six Gram products (warp li issues level li): after its own share of
    // the level's images the warp waits for everybody else's (all element warps do the same work in step, so the
    // wait is short) and issues the product
    const uint32_t leader = (warp < 6 && elect_one()) ? 1u : 0u;
    const uint64_t gd0 = umma_desc_sw128(smem_u32(sm.img[0]), KI_IMG_BYTES, 1024);
    const uint32_t g_lo0 = (uint32_t)gd0, g_hi = (uint32_t)(gd0 >> 32);
    uint32_t ci = 0, n_img = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < p.total; w += gridDim.x, ++ci) {
      int b, h, chunk;
      ki_coords(w, p.NC, p.H, b, h, chunk);
      const int par = ci & 1;
      int t0, rows;
      ki_chunk_span(p.chunk_tab, chunk, p.T, t0, rows);
      uint8_t* rec = p.ws + (size_t)w * REC_BYTES;
      ok = mbar_wait_long(&sm.in_full, ci & 1, abort_flag, p.status, 1) && ok;
      if (p.chunk_tab && rows < KC) {
        // a sequence's last chunk: the rows after it belong to the next sequence (the tile load only zero-fills past
        // the end of the tensor) -- blank them, so that they behave like padding: g = 0, k = q = 0 (beta = 0 below)
        for (int i = tid; i < (KC - rows) * (KD / 4); i += KI_ELEM_THREADS) {
          const int r = rows + i / (KD / 4), c4 = (i % (KD / 4)) * 4;
          *reinterpret_cast<float4*>(&sm.g[r][c4]) = make_float4(0.f, 0.f, 0.f, 0.f);
          *reinterpret_cast<uint2*>(&sm.q[r][c4]) = make_uint2(0u, 0u);
          *reinterpret_cast<uint2*>(&sm.k[r][c4]) = make_uint2(0u, 0u);
        }
        named_bar(1, KI_ELEM_THREADS);
      }

      // ---- per-token scalars: 8 threads per row, 16 channels each
      {
        const int r = tid >> 3, part = tid & 7;
        float qf[16], kf[16];
        unpack8(*reinterpret_cast<const uint4*>(&sm.q[r][16 * part]), qf);
        unpack8(*reinterpret_cast<const uint4*>(&sm.q[r][16 * part + 8]), qf + 8);
        unpack8(*reinterpret_cast<const uint4*>(&sm.k[r][16 * part]), kf);
        unpack8(*reinterpret_cast<const uint4*>(&sm.k[r][16 * part + 8]), kf + 8);
        float sq = 0.f, sk = 0.f, dqk = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) { sq = fmaf(qf[e], qf[e], sq); sk = fmaf(kf[e], kf[e], sk); dqk = fmaf(qf[e], kf[e], dqk); }
#pragma unroll
        for (int o = 1; o <= 4; o <<= 1) {
          sq += __shfl_xor_sync(0xffffffffu, sq, o);
          sk += __shfl_xor_sync(0xffffffffu, sk, o);
          dqk += __shfl_xor_sync(0xffffffffu, dqk, o);
        }
        if (part == 0) {
          const float a = p.l2norm ? rsqrtf(sq + 1e-6f) : 1.f, cc = p.l2norm ? rsqrtf(sk + 1e-6f) : 1.f;
          sm.rq[par][r] = a; sm.rk[par][r] = cc; sm.qkd[par][r] = a * cc * dqk;
        }
        if (tid < KC) sm.beta[par][tid] = (tid < rows) ? p.beta[((size_t)b * p.T + t0 + tid) * p.H + h] : 0.f;
      }
      if (named_bar_or(1, KI_ELEM_THREADS, !ok)) break;

      // ---- this thread's column of the chunk: 16 tokens of channel c
      float pre[16], suf[16];
      uint32_t kn[8], qn[8];                                                     // normalised k, q as fp16 pairs (tokens 2i, 2i + 1)
      {
        const int r0 = 16 * seg;
        float rkv[16], rqv[16];
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
          *reinterpret_cast<float4*>(&rkv[i]) = *reinterpret_cast<const float4*>(&sm.rk[par][r0 + i]);
          *reinterpret_cast<float4*>(&rqv[i]) = *reinterpret_cast<const float4*>(&sm.rq[par][r0 + i]);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          pre[i] = fast_exp2(sm.g[r0 + i][c] * 1.4426950408889634f);           // d_t = e^{g_t}
          suf[i] = 1.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          kn[i] = pack_h2(__bfloat162float(sm.k[r0 + 2 * i][c]) * rkv[2 * i], __bfloat162float(sm.k[r0 + 2 * i + 1][c]) * rkv[2 * i + 1]);
          qn[i] = pack_h2(__bfloat162float(sm.q[r0 + 2 * i][c]) * rqv[2 * i], __bfloat162float(sm.q[r0 + 2 * i + 1][c]) * rqv[2 * i + 1]);
        }
      }
      named_bar(1, KI_ELEM_THREADS);                                            // every read of the input tiles is done
      if (tid == 0 && w + (int)gridDim.x < p.total) {                           // next item's inputs land under this item's work
        int nb, nh, nchunk, nt0, nrows;
        ki_coords(w + gridDim.x, p.NC, p.H, nb, nh, nchunk);
        ki_chunk_span(p.chunk_tab, nchunk, p.T, nt0, nrows);
        mbar_expect_tx(&sm.in_full, KI_IN_BYTES);
        tma_load_4d(&sm.g[0][0], &tm_g, &sm.in_full, 0, nt0, nh, nb);
        tma_load_4d(&sm.q[0][0], &tm_q, &sm.in_full, 0, nt0, nh, nb);
        tma_load_4d(&sm.k[0][0], &tm_k, &sm.in_full, 0, nt0, nh, nb);
      }

      // ---- six levels.  At level s token t is "upper" iff bit s of t is set; its factor is pre (upper) or suf (lower):
      //      the inclusive prefix / exclusive suffix product of d inside the aligned s-block of t.
      auto emit = [&](const float (&f)[16], const bool write_q) {
        ki_emit_level(sm, f, kn, qn, write_q, c, seg, warp, leader, ci, n_img, ok, tmem_base, g_lo0, g_hi, abort_flag, p.status);
      };
      // s = 1, 2, 4, 8: inside the segment (rows of lower tokens in the q image are never read back)
      ki_level_inreg<1>(pre, suf, emit);
      ki_level_inreg<2>(pre, suf, emit);
      ki_level_inreg<4>(pre, suf, emit);
      ki_level_inreg<8>(pre, suf, emit);
      sm.tot[seg][c] = pre[15];
      if (named_bar_or(1, KI_ELEM_THREADS, !ok)) break;
      {                                                                         // s = 16: segments pair up
        const bool up = (seg & 1) != 0;
        float f[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] = up ? pre[i] : suf[i];
        emit(f, up);
        const float m = sm.tot[seg ^ 1][c];
        if (seg & 1) {
#pragma unroll
          for (int i = 0; i < 16; ++i) pre[i] *= m;
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) suf[i] *= m;
        }
      }
      {                                                                         // s = 32: halves of the chunk
        const bool up = (seg & 2) != 0;
        float f[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] = up ? pre[i] : suf[i];
        emit(f, up);
        const float m = (seg & 2) ? sm.tot[0][c] * sm.tot[1][c] : sm.tot[2][c] * sm.tot[3][c];
        if (seg & 2) {
#pragma unroll
          for (int i = 0; i < 16; ++i) pre[i] *= m;
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) suf[i] *= m;
        }
      }
      // ---- pre = e^{G}, suf = e^{G_C - G}: the state-pass operands
      if (ci >= 1) ok = mbar_wait_long(&sm.x_empty, (ci - 1) & 1, abort_flag, p.status, 3) && ok;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float x[8], qt[8], kt[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 kf = unpack_h2(kn[4 * e + i]), qf = unpack_h2(qn[4 * e + i]);
          const int t = 8 * e + 2 * i;
          x[2 * i] = kf.x * pre[t]; x[2 * i + 1] = kf.y * pre[t + 1];
          qt[2 * i] = qf.x * pre[t] * p.scale; qt[2 * i + 1] = qf.y * pre[t + 1] * p.scale;
          kt[2 * i] = kf.x * suf[t]; kt[2 * i + 1] = kf.y * suf[t + 1];
        }
        *reinterpret_cast<uint4*>(&sm.xt[c][16 * seg + 8 * e]) =
            make_uint4(pack_h2(x[0], x[1]), pack_h2(x[2], x[3]), pack_h2(x[4], x[5]), pack_h2(x[6], x[7]));
        const size_t goff = ((size_t)c * LDT + 16 * seg + 8 * e) * 2;
        st_global16(rec + OFF_QT + goff, pack_h2(qt[0], qt[1]), pack_h2(qt[2], qt[3]), pack_h2(qt[4], qt[5]), pack_h2(qt[6], qt[7]));
        st_global16(rec + OFF_KT + goff, pack_h2(kt[0], kt[1]), pack_h2(kt[2], kt[3]), pack_h2(kt[4], kt[5]), pack_h2(kt[6], kt[7]));
      }
      if (seg == 3) reinterpret_cast<float*>(rec + OFF_D)[c] = pre[15];         // e^{G_C}
      mbar_arrive(&sm.x_full);
    }
  } else {
    // ================================================================== solver warps
    // Two warps share each quarter of the TMEM lanes (warp % 4): rows 32 hb .. 32 hb + 31 of the k (quarters 0, 1) or
    // q (quarters 2, 3) products; `ch` splits a row's 32-column window into two halves of 16.
    const int ws = warp - KI_ELEM_WARPS, st = tid - KI_ELEM_THREADS;            // 0..7, 0..255
    const int g8 = lane >> 2, t4 = lane & 3;
    const int qt4 = ws & 3, ch = ws >> 2;
    const bool is_qk = qt4 >= 2;
    const int hb = qt4 & 1;
    const int row = 32 * hb + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(32 * qt4) << 16);
    if (st == 0 && (int)blockIdx.x < p.total) {
      int b, h, chunk, ft0, frows;
      ki_coords(blockIdx.x, p.NC, p.H, b, h, chunk);
      ki_chunk_span(p.chunk_tab, chunk, p.T, ft0, frows);
      prefetch_tmap(&tm_v);
      mbar_expect_tx(&sm.v_full, KI_IMG_BYTES);
      tma_load_4d(&sm.v[0][0], &tm_v, &sm.v_full, 0, ft0, h, b);
    }
    uint32_t ci = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < p.total; w += gridDim.x, ++ci) {
      const int par = ci & 1;
      uint8_t* rec = p.ws + (size_t)w * REC_BYTES;
      // ---- Gram entries out of TMEM.  acc[j] collects row `row`, column 32 hb + 16 ch + j, level by level: the
      //      entry of (row, column) lives in the level of the highest bit in which the two token indices differ.
      float acc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = 0.f;
      float my_beta = 0.f, my_qkd = 0.f;
#pragma unroll
      for (int li = 0; li < 6; ++li) {
        ok = __all_sync(0xffffffffu, mbar_wait_long(&sm.d_full[li], ci & 1, abort_flag, p.status, 6)) && ok;
        if (li == 0) {                                                          // the item's scalars are final once its first image exists
          if (st < KC) sm.sbeta[st] = sm.beta[par][st];
          my_beta = sm.beta[par][row]; my_qkd = sm.qkd[par][row];
        }
        tc_fence_after();
        uint32_t r[16];
        if (li < 5) {
          tmem_ld16(lane_base + 64 * li + 32 * hb + 16 * ch, r);
          tc_wait_ld();
          const uint32_t lx = (uint32_t)lane >> li;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (lx == (uint32_t)((((16 * ch + j) >> li)) ^ 1)) acc[j] = __uint_as_float(r[j]);
        } else if (hb == 1) {                                                   // s = 32: rows 32..63 against columns 0..31, all of them
          tmem_ld16(lane_base + 64 * 5 + 16 * ch, r);
          tc_wait_ld();
          const float sc = is_qk ? p.scale : my_beta;
          uint32_t pk[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) pk[j] = pack_h2(sc * __uint_as_float(r[2 * j]), sc * __uint_as_float(r[2 * j + 1]));
          if (is_qk) {
            uint8_t* dst = rec + OFF_AQK + ((size_t)row * LDT + 16 * ch) * 2;
            st_global16(dst, pk[0], pk[1], pk[2], pk[3]);
            st_global16(dst + 16, pk[4], pk[5], pk[6], pk[7]);
          } else {
            *reinterpret_cast<uint4*>(&sm.akh[row][16 * ch]) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            *reinterpret_cast<uint4*>(&sm.akh[row][16 * ch + 8]) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          }
        }
        tc_fence_before();
        mbar_arrive(&sm.d_empty[li]);
      }
      {
        const float sc = is_qk ? p.scale : my_beta;
        const int lj = lane - 16 * ch;                                          // this row's own column inside the 16 (if 0 <= lj < 16)
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = (j < lj) ? sc * acc[j] : 0.f;
        uint32_t pk[8];
        if (is_qk) {
#pragma unroll
          for (int j = 0; j < 16; ++j) if (j == lj) v[j] = p.scale * my_qkd;    // the diagonal: q_i . k_i, no decay
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) pk[j] = pack_h2(v[2 * j], v[2 * j + 1]);
        if (is_qk) {
          uint8_t* dst = rec + OFF_AQK + ((size_t)row * LDT + 32 * hb + 16 * ch) * 2;
          st_global16(dst, pk[0], pk[1], pk[2], pk[3]);
          st_global16(dst + 16, pk[4], pk[5], pk[6], pk[7]);
        } else {
          *reinterpret_cast<uint4*>(&sm.akh[row][32 * hb + 16 * ch]) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint4*>(&sm.akh[row][32 * hb + 16 * ch + 8]) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          if ((lane >> 4) == ch) {                                              // the row's diagonal 16 x 16 block, in fp32
            const int blk = row >> 4;
#pragma unroll
            for (int j = 0; j < 16; ++j) sm.akk_t[blk][j][row & 15] = v[j];
          }
        }
      }
      if (named_bar_or(2, KI_SOLVER_THREADS, !ok)) break;

      // ---- the four 16 x 16 diagonal blocks of I + A_kk inverted in fp32, one block per warp, lane = column: a column
      //      sweep (once t_j is final every later row takes its update at once), so the chain is 16 steps deep
      if (ws < 4 && lane < 16) {
        float t[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) t[i] = (i == lane) ? 1.f : 0.f;
#pragma unroll
        for (int j = 0; j < 15; ++j) {
          float a[16];
#pragma unroll
          for (int i4 = (j + 1) & ~3; i4 < 16; i4 += 4)
            *reinterpret_cast<float4*>(&a[i4]) = *reinterpret_cast<const float4*>(&sm.akk_t[ws][j][i4]);
#pragma unroll
          for (int i = j + 1; i < 16; ++i) t[i] = fmaf(-a[i], t[j], t[i]);
        }
        const int base = ws * 16;
#pragma unroll
        for (int i = 0; i < 16; ++i) sm.th[base + i][base + lane] = __float2half_rn(t[i]);   // t[i] = T[base + i][base + lane]
      }
      ok = mbar_wait_long(&sm.x_full, ci & 1, abort_flag, p.status, 7) && ok;   // (k e^G)^T is in place
      ok = mbar_wait_long(&sm.v_full, ci & 1, abort_flag, p.status, 8) && ok;   // and the v tile
      if (named_bar_or(2, KI_SOLVER_THREADS, !ok)) break;

      // ---- W and U0 by blocked forward substitution on the transposed systems
      //          W^T (I + A)^T = (diag(beta) k e^G)^T,      U0^T (I + A)^T = (diag(beta) v)^T
      //      A warp owns 32 of the 256 rows (channels of W^T: warps 0-3, value columns of U0^T: warps 4-7) for all
      //      four 16-token block columns I, so there is nothing to exchange between warps:
      //          Z_I = R_I - sum_{J<I} Z_J A_IJ^T,   then   Z_I <- Z_I T_II^T
      //      with every product an m16n8k16 tile whose fp32 accumulators, rounded to fp16, are the A fragment of
      //      the products that follow.  The two row tiles of a warp are independent chains issued side by side.
      {
        const bool is_w = ws < 4;
        uint8_t* dst = rec + (is_w ? OFF_WT : OFF_UT);
        uint32_t zf[2][3][4];                                                   // Z_J as fp16 A fragments: [row tile][J][4]
#pragma unroll
        for (int I = 0; I < 4; ++I) {
          float acc1[2][2][4];
#pragma unroll
          for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int nn = 0; nn < 2; ++nn) { acc1[m][nn][0] = acc1[m][nn][1] = acc1[m][nn][2] = acc1[m][nn][3] = 0.f; }
#pragma unroll
          for (int J = 0; J < I; ++J) {
#pragma unroll
            for (int nn = 0; nn < 2; ++nn) {
              const __half* arow = &sm.akh[I * 16 + nn * 8 + g8][J * 16 + 2 * t4];
              const uint32_t b0 = *reinterpret_cast<const uint32_t*>(arow), b1 = *reinterpret_cast<const uint32_t*>(arow + 8);
#pragma unroll
              for (int m = 0; m < 2; ++m) mma_f16(acc1[m][nn], zf[m][J], b0, b1);
            }
          }
          uint32_t a2[2][4];
#pragma unroll
          for (int nn = 0; nn < 2; ++nn) {
            const int tk = I * 16 + nn * 8 + 2 * t4;                            // this thread's two tokens of the tile
            const float2 bt = *reinterpret_cast<const float2*>(&sm.sbeta[tk]);
#pragma unroll
            for (int m = 0; m < 2; ++m) {
              const int r0 = 16 * (2 * (ws & 3) + m) + g8;                      // row inside this matrix: channel or value column
              float2 lo, hi;                                                    // right-hand side at rows r0 and r0 + 8
              if (is_w) {
                lo = unpack_h2(*reinterpret_cast<const uint32_t*>(&sm.xt[r0][tk]));
                hi = unpack_h2(*reinterpret_cast<const uint32_t*>(&sm.xt[r0 + 8][tk]));
              } else {
                lo = make_float2(__bfloat162float(sm.v[tk][r0]), __bfloat162float(sm.v[tk + 1][r0]));
                hi = make_float2(__bfloat162float(sm.v[tk][r0 + 8]), __bfloat162float(sm.v[tk + 1][r0 + 8]));
              }
              a2[m][2 * nn] = pack_h2(lo.x * bt.x - acc1[m][nn][0], lo.y * bt.y - acc1[m][nn][1]);
              a2[m][2 * nn + 1] = pack_h2(hi.x * bt.x - acc1[m][nn][2], hi.y * bt.y - acc1[m][nn][3]);
            }
          }
#pragma unroll
          for (int nn = 0; nn < 2; ++nn) {
            const __half* trow = &sm.th[I * 16 + nn * 8 + g8][I * 16 + 2 * t4];
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(trow), b1 = *reinterpret_cast<const uint32_t*>(trow + 8);
            const int tk = I * 16 + nn * 8 + 2 * t4;
#pragma unroll
            for (int m = 0; m < 2; ++m) {
              float acc2[4] = {0.f, 0.f, 0.f, 0.f};
              mma_f16(acc2, a2[m], b0, b1);
              const uint32_t z_lo = pack_h2(acc2[0], acc2[1]), z_hi = pack_h2(acc2[2], acc2[3]);
              if (I < 3) { zf[m][I][2 * nn] = z_lo; zf[m][I][2 * nn + 1] = z_hi; }
              const int r0 = 16 * (2 * (ws & 3) + m) + g8;
              *reinterpret_cast<uint32_t*>(dst + ((size_t)r0 * LDT + tk) * 2) = z_lo;
              *reinterpret_cast<uint32_t*>(dst + ((size_t)(r0 + 8) * LDT + tk) * 2) = z_hi;
            }
          }
        }
      }
      if (named_bar_or(2, KI_SOLVER_THREADS, !ok)) break;                      // every warp is done with the X image and the v tile
      if (st == 0) {
        mbar_arrive(&sm.x_empty);
        if (w + (int)gridDim.x < p.total) {
          int nb, nh, nchunk, nt0, nrows;
          ki_coords(w + gridDim.x, p.NC, p.H, nb, nh, nchunk);
          ki_chunk_span(p.chunk_tab, nchunk, p.T, nt0, nrows);
          mbar_expect_tx(&sm.v_full, KI_IMG_BYTES);
          tma_load_4d(&sm.v[0][0], &tm_v, &sm.v_full, 0, nt0, nh, nb);
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// =============================================================================================
// inter-chunk state kernel
// =============================================================================================
struct KdaStateParams {
  const uint8_t* ws;
  const float* h0;
  float* hT;
  void* o;
  int T, H, NC, out_fp32;
  int* status;
  // packed variable-length sequences (B = 1): blockIdx.y = sequence * H + head, the sequence's chunks are
  // seq_ptr[s] .. seq_ptr[s + 1] - 1 of the packed row's NC chunks, chunk_tab as in the intra kernel; null: dense
  const int* chunk_tab;
  const int* seq_ptr;
};


// NW V-slices of 16 rows per CTA, each owned by KS warps that split the K dimension of the state between them.
// KS = 1: a warp keeps its 16 V-rows x 128 K-columns of S^T in accumulator registers and chains everything through
// register fragments.  KS > 1 (few (batch, head) pairs per GPU, where the serial chain over the chunks -- 212
// dependent mma.sync per chunk and warp -- is all that is left): warp kq holds K-columns [128 kq / KS, 128 (kq+1) / KS);
// the two products that contract over K (S^T W^T and S^T q~^T) become partial sums that the slice's warps exchange
// through shared memory once per chunk (fragment order, double-buffered, one named barrier), after which every warp
// has the whole U^T, finishes the output for its own token tiles and updates its own K-columns of the state.
template <int NW, int KS, int NST>
struct KdaStateSmem {
  static constexpr int VS = 16 * NW;
  static constexpr int CW = NW * KS;                     // compute warps
  static constexpr int U_BYTES = VS * LDT * 2;
  static constexpr int STAGE = SHARED_BYTES + U_BYTES;
  static constexpr int O_LD = VS + 4;                    // floats; staging of one chunk of output
  static constexpr int XCH_WARP = 2 * 8 * 32 * 16;       // one warp's two partial accumulators: 8 tiles x 32 lanes x float4
  static constexpr int XCH = KS > 1 ? CW * XCH_WARP : 0;
  static constexpr int BYTES = NST * STAGE + KC * O_LD * 4 + XCH + 64;
};

template <int NW, int KS, int NST>
__global__ void __launch_bounds__(32 * (NW * KS + 1), 1) kda_state_kernel(const KdaStateParams p) {
  using L = KdaStateSmem<NW, KS, NST>;
  constexpr int KDA_NST = NST;                             // ring stages of chunk records
  constexpr int VS = L::VS, CW = L::CW;
  constexpr int NKT = 16 / KS;                             // this warp's 8-column tiles of the state
  constexpr int NKS = 8 / KS;                              // and its 16-deep steps of the contractions over K
  constexpr int TPW = 8 / KS;                              // token tiles whose output this warp finishes
  extern __shared__ __align__(128) uint8_t kda_smem_raw[];
  uint8_t* stages = kda_smem_raw;
  float* o_stage = reinterpret_cast<float*>(kda_smem_raw + KDA_NST * L::STAGE);
  float4* xch = reinterpret_cast<float4*>(kda_smem_raw + KDA_NST * L::STAGE + KC * L::O_LD * 4);
  uint64_t* full = reinterpret_cast<uint64_t*>(kda_smem_raw + KDA_NST * L::STAGE + KC * L::O_LD * 4 + L::XCH);
  uint64_t* empty = full + KDA_NST;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + KDA_NST);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g8 = lane >> 2, t4 = lane & 3;
  const int vsl = blockIdx.x, bh = blockIdx.y;              // bh also indexes h0 / hT
  const int h = bh % p.H;
  const int b = p.seq_ptr ? 0 : bh / p.H;
  const int c_begin = p.seq_ptr ? p.seq_ptr[bh / p.H] : 0, c_end = p.seq_ptr ? p.seq_ptr[bh / p.H + 1] : p.NC;
  const int v_base = vsl * VS;
  const uint8_t* recs = p.ws + ((size_t)(b * p.H + h) * p.NC + c_begin) * REC_BYTES;    // this sequence's first record
  const int n_chunks = c_end - c_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < KDA_NST; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CW); }
    *abort_flag = 0;
    mbar_init_fence();
  }
  __syncthreads();

  if (warp == CW) {
    // ------------------------------------------------------------ producer: bulk copies into the ring
    if (lane == 0) {
      for (int c = 0; c < n_chunks; ++c) {
        const int s = c % KDA_NST;
        if (!mbar_wait(&empty[s], ((c / KDA_NST) & 1) ^ 1, abort_flag, p.status, 1)) break;
        const uint8_t* rec = recs + (size_t)c * REC_BYTES;
        mbar_expect_tx(&full[s], L::STAGE);
        bulk_g2s(stages + s * L::STAGE, rec, SHARED_BYTES, &full[s]);
        bulk_g2s(stages + s * L::STAGE + SHARED_BYTES, rec + OFF_UT + (size_t)v_base * LDT * 2, L::U_BYTES, &full[s]);
      }
    }
    return;
  }

  // ------------------------------------------------------------ compute warps: 16 V rows, 128 / KS K columns each
  const int vs = warp / KS, kq = warp % KS;
  const int vr0 = vs * 16 + g8, vr1 = vr0 + 8;                     // rows inside the CTA's V range
  float st[NKT][4];                                                // S^T[v][k]: tile j -> k = 8 (kq NKT + j) + 2 t4 (+1)
#pragma unroll
  for (int j = 0; j < NKT; ++j) {
    if (p.h0) {
      const float* hp = p.h0 + (size_t)bh * KD * KD;
      const int k0 = (kq * NKT + j) * 8 + 2 * t4;
      st[j][0] = hp[(size_t)k0 * KD + v_base + vr0]; st[j][1] = hp[(size_t)(k0 + 1) * KD + v_base + vr0];
      st[j][2] = hp[(size_t)k0 * KD + v_base + vr1]; st[j][3] = hp[(size_t)(k0 + 1) * KD + v_base + vr1];
    } else {
      st[j][0] = st[j][1] = st[j][2] = st[j][3] = 0.f;
    }
  }

  for (int c = 0; c < n_chunks; ++c) {
    const int s = c % KDA_NST;
    const bool ok = __all_sync(0xffffffffu, mbar_wait(&full[s], (c / KDA_NST) & 1, abort_flag, p.status, 2));
    if (!ok) break;
    const uint8_t* sb = stages + s * L::STAGE;
    const __half* Wt = reinterpret_cast<const __half*>(sb + OFF_WT);
    const __half* Qt = reinterpret_cast<const __half*>(sb + OFF_QT);
    const __half* Kt = reinterpret_cast<const __half*>(sb + OFF_KT);
    const __half* Aq = reinterpret_cast<const __half*>(sb + OFF_AQK);
    const float* dv = reinterpret_cast<const float*>(sb + OFF_D);
    const __half* Ut = reinterpret_cast<const __half*>(sb + SHARED_BYTES);

    // (1) accU = S^T W^T   and   (2a) accO = S^T q~^T      [16 x 64 tokens each], over this warp's K columns
    float au[8][4], ao[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { au[nt][0] = au[nt][1] = au[nt][2] = au[nt][3] = 0.f; ao[nt][0] = ao[nt][1] = ao[nt][2] = ao[nt][3] = 0.f; }
#pragma unroll
    for (int ksl = 0; ksl < NKS; ++ksl) {
      const int ks = kq * NKS + ksl;
      uint32_t a[4];
      a[0] = pack_h2(st[2 * ksl][0], st[2 * ksl][1]); a[1] = pack_h2(st[2 * ksl][2], st[2 * ksl][3]);
      a[2] = pack_h2(st[2 * ksl + 1][0], st[2 * ksl + 1][1]); a[3] = pack_h2(st[2 * ksl + 1][2], st[2 * ksl + 1][3]);
      // B fragments of two token tiles per transposing ldmatrix.x4 from the channel-major images: matrix m =
      // (k half m & 1, token tile nt + (m >> 1)); its stored rows are channels, its columns tokens
      const int lrow = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), lcol = (lane >> 4) * 8;
#pragma unroll
      for (int nt = 0; nt < 8; nt += 2) {
        uint32_t bw[4], bq[4];
        ldmatrix_x4_t(bw, &Wt[lrow * LDT + nt * 8 + lcol]);
        ldmatrix_x4_t(bq, &Qt[lrow * LDT + nt * 8 + lcol]);
        mma_f16(au[nt], a, bw[0], bw[1]);
        mma_f16(ao[nt], a, bq[0], bq[1]);
        mma_f16(au[nt + 1], a, bw[2], bw[3]);
        mma_f16(ao[nt + 1], a, bq[2], bq[3]);
      }
    }
    if (KS > 1) {
      // exchange: every warp of the slice needs the whole accU; accO only for the token tiles it finishes.  The sums
      // run over the warps in a fixed order, so all of them hold the same bits.
      float4* mine = xch + (size_t)warp * (L::XCH_WARP / 16);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        mine[nt * 32 + lane] = make_float4(au[nt][0], au[nt][1], au[nt][2], au[nt][3]);
        mine[256 + nt * 32 + lane] = make_float4(ao[nt][0], ao[nt][1], ao[nt][2], ao[nt][3]);
      }
      named_bar(2 + vs, 32 * KS);
      const float4* slice = xch + (size_t)(vs * KS) * (L::XCH_WARP / 16);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float4 t = slice[nt * 32 + lane];
#pragma unroll
        for (int q = 1; q < KS; ++q) {
          const float4 u = slice[q * (L::XCH_WARP / 16) + nt * 32 + lane];
          t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        au[nt][0] = t.x; au[nt][1] = t.y; au[nt][2] = t.z; au[nt][3] = t.w;
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (nt / TPW != kq) continue;                                // compile-time tile index, warp-uniform test
        float4 t = slice[256 + nt * 32 + lane];
#pragma unroll
        for (int q = 1; q < KS; ++q) {
          const float4 u = slice[q * (L::XCH_WARP / 16) + 256 + nt * 32 + lane];
          t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        ao[nt][0] = t.x; ao[nt][1] = t.y; ao[nt][2] = t.z; ao[nt][3] = t.w;
      }
      named_bar(2 + vs, 32 * KS);                                    // everybody has read: the next chunk may overwrite
    }
    // U^T = U0^T - accU, as fp16 A fragments over the token axis
    uint32_t ua[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int tok = nt * 8 + 2 * t4;
      const float2 u0 = unpack_h2(*reinterpret_cast<const uint32_t*>(&Ut[vr0 * LDT + tok]));
      const float2 u1 = unpack_h2(*reinterpret_cast<const uint32_t*>(&Ut[vr1 * LDT + tok]));
      const uint32_t lo = pack_h2(u0.x - au[nt][0], u0.y - au[nt][1]);
      const uint32_t hi = pack_h2(u1.x - au[nt][2], u1.y - au[nt][3]);
      ua[nt >> 1][(nt & 1) * 2 + 0] = lo;
      ua[nt >> 1][(nt & 1) * 2 + 1] = hi;
    }
    // (2b) accO += U^T A_qk^T, for the token tiles this warp finishes
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const int lrow = (lane >> 4) * 8 + (lane & 7), lcol = ks * 16 + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int nt = 2 * ks; nt < 8; nt += 2) {                     // A_qk[i][j] = 0 for j > i: tiles below 2 ks are empty
        if (KS > 1 && nt / TPW != kq) continue;
        uint32_t ba[4];
        ldmatrix_x4(ba, &Aq[(nt * 8 + lrow) * LDT + lcol]);
        mma_f16(ao[nt], ua[ks], ba[0], ba[1]);
        mma_f16(ao[nt + 1], ua[ks], ba[2], ba[3]);
      }
    }
    // (3) S^T = S^T diag(e^{G_C}) + U^T k~, this warp's K columns
#pragma unroll
    for (int j = 0; j < NKT; ++j) {
      const float2 d2 = *reinterpret_cast<const float2*>(&dv[(kq * NKT + j) * 8 + 2 * t4]);
      st[j][0] *= d2.x; st[j][1] *= d2.y; st[j][2] *= d2.x; st[j][3] *= d2.y;
    }
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const int lrow = (lane >> 4) * 8 + (lane & 7), lcol = ks * 16 + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int j = 0; j < NKT; j += 2) {
        uint32_t bk[4];
        ldmatrix_x4(bk, &Kt[((kq * NKT + j) * 8 + lrow) * LDT + lcol]);
        mma_f16(st[j], ua[ks], bk[0], bk[1]);
        mma_f16(st[j + 1], ua[ks], bk[2], bk[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);                         // this warp is done with the stage

    // output: stage [token][v] in shared memory, then coalesced rows
    asm volatile("bar.sync 1, %0;" ::"n"(32 * CW) : "memory");    // previous chunk's copy-out finished
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      if (KS > 1 && nt / TPW != kq) continue;
      const int tok = nt * 8 + 2 * t4;
      o_stage[tok * L::O_LD + vr0] = ao[nt][0]; o_stage[(tok + 1) * L::O_LD + vr0] = ao[nt][1];
      o_stage[tok * L::O_LD + vr1] = ao[nt][2]; o_stage[(tok + 1) * L::O_LD + vr1] = ao[nt][3];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * CW) : "memory");
    int t0, rows;
    ki_chunk_span(p.chunk_tab, c_begin + c, p.T, t0, rows);
    for (int idx = threadIdx.x; idx < KC * (VS / 4); idx += 32 * CW) {
      const int tok = idx / (VS / 4), v4 = (idx % (VS / 4)) * 4;
      if (tok >= rows) continue;
      const float4 x = *reinterpret_cast<const float4*>(&o_stage[tok * L::O_LD + v4]);
      const size_t off = (((size_t)b * p.T + (size_t)t0 + tok) * p.H + h) * KD + v_base + v4;
      if (p.out_fp32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.o) + off) = x;
      } else {
        uint2 pk = make_uint2(pack_bf16(x.x, x.y), pack_bf16(x.z, x.w));
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.o) + off) = pk;
      }
    }
  }

  if (p.hT) {
    float* hp = p.hT + (size_t)bh * KD * KD;
#pragma unroll
    for (int j = 0; j < NKT; ++j) {
      const int k0 = (kq * NKT + j) * 8 + 2 * t4;
      hp[(size_t)k0 * KD + v_base + vr0] = st[j][0]; hp[(size_t)(k0 + 1) * KD + v_base + vr0] = st[j][1];
      hp[(size_t)k0 * KD + v_base + vr1] = st[j][2]; hp[(size_t)(k0 + 1) * KD + v_base + vr1] = st[j][3];
    }
  }
}

}  // namespace daisy

using namespace daisy;

extern "C" size_t daisy_b200_kda_workspace_bytes(int B, int T, int H, int K, int V) {
  if (B <= 0 || T <= 0 || H <= 0 || K != KD || V != KD) return 0;
  const size_t nc = (size_t)(T + KC - 1) / KC;
  return (size_t)B * H * nc * REC_BYTES;
}

template <int NW, int KS, int NST>
static int launch_state(const KdaStateParams& sp, int BH, cudaStream_t st) {
  using L = KdaStateSmem<NW, KS, NST>;
  static_assert(L::BYTES <= 232448, "over the 227 KB a CTA may use");
  static bool attr[daisy_host::MAX_DEVICES] = {};             // the attribute is per device
  const int dev = daisy_host::device_slot();
  if (dev < 0) return DAISY_ENODEV;
  if (!attr[dev]) {
    if (cudaFuncSetAttribute(kda_state_kernel<NW, KS, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES) != cudaSuccess) return DAISY_ECUDA;
    attr[dev] = true;
  }
  kda_state_kernel<NW, KS, NST><<<dim3(KD / L::VS, BH), 32 * (L::CW + 1), L::BYTES, st>>>(sp);
  return cudaGetLastError() == cudaSuccess ? DAISY_OK : DAISY_ECUDA;
}

// Shared launcher.  Dense: NC = ceil(T / 64) chunks per (batch, head) row, n_seq = B.  Packed variable-length (B = 1):
// chunk_tab [NC][2] and seq_ptr [n_seq + 1] (both in device memory) say which tokens each chunk covers and which
// chunks each sequence owns; h0 / hT are [n_seq, H, K, V].
static int kda_launch(const void* q, const void* k, const void* v, const float* g, const float* beta, const float* h0, void* o,
                      float* hT, int B, int T, int H, int K, int V, int chunk, float scale, unsigned flags,
                      void* workspace, size_t workspace_bytes, int NC, int n_seq, const int* chunk_tab, const int* seq_ptr,
                      int* status_word, void* stream) {
  if (!q || !k || !v || !g || !beta || !o || !workspace || B <= 0 || T <= 0 || H <= 0 || NC <= 0 || n_seq <= 0) return DAISY_EINVAL;
  if (K != KD || V != KD || chunk != KC) return DAISY_EUNSUPPORTED;
  if (B > 65535 || H > 65535 || (size_t)n_seq * H > 65535) return DAISY_EUNSUPPORTED;
  if (workspace_bytes < (size_t)B * H * NC * REC_BYTES) return DAISY_EWORKSPACE;
  if (!daisy_aligned16(q) || !daisy_aligned16(k) || !daisy_aligned16(v) || !daisy_aligned16(g) || !daisy_aligned16(o) ||
      !daisy_aligned16(workspace) || (h0 && !daisy_aligned16(h0)) || (hT && !daisy_aligned16(hT)))
    return DAISY_EALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  static bool attr[daisy_host::MAX_DEVICES] = {};             // the attribute is per device
  const int dev = daisy_host::device_slot();
  if (dev < 0) return DAISY_ENODEV;
  constexpr int intra_smem = (int)sizeof(KdaIntraSmem) + 1024;   // the kernel aligns its image buffers to 1 KB itself
  if (!attr[dev]) {
    if (cudaFuncSetAttribute(kda_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, intra_smem) != cudaSuccess) {
      (void)cudaGetLastError();
      return DAISY_ECUDA;
    }
    attr[dev] = true;
  }
  if ((int64_t)B * H * NC >= ((int64_t)1 << 31)) return DAISY_EUNSUPPORTED;
  CUtensorMap tg, tq, tk, tv;
  int trc;
  if ((trc = daisy_host::make_tmap_rows_bthd(&tg, g, 4, KD, T, H, B, KC)) != DAISY_OK) return trc;
  if ((trc = daisy_host::make_tmap_rows_bthd(&tq, q, 2, KD, T, H, B, KC)) != DAISY_OK) return trc;
  if ((trc = daisy_host::make_tmap_rows_bthd(&tk, k, 2, KD, T, H, B, KC)) != DAISY_OK) return trc;
  if ((trc = daisy_host::make_tmap_rows_bthd(&tv, v, 2, KD, T, H, B, KC)) != DAISY_OK) return trc;
  KdaIntraParams ip;
  ip.beta = beta; ip.ws = (uint8_t*)workspace;
  ip.T = T; ip.H = H; ip.NC = NC; ip.total = B * H * NC;
  ip.scale = scale > 0.f ? scale : 1.0f / sqrtf((float)K);
  ip.l2norm = (flags & DAISY_KDA_L2NORM_QK) ? 1 : 0;
  ip.status = status_word;
  ip.chunk_tab = chunk_tab;
  const int sms = daisy_host::sm_count_cached();
  if (sms <= 0) return DAISY_ENODEV;
  kda_intra_kernel<<<ip.total < sms ? ip.total : sms, KI_THREADS, intra_smem, st>>>(tg, tq, tk, tv, ip);
  DAISY_CHECK_LAUNCH();

  KdaStateParams sp;
  sp.ws = (const uint8_t*)workspace; sp.h0 = h0; sp.hT = hT; sp.o = o;
  sp.T = T; sp.H = H; sp.NC = NC; sp.out_fp32 = (flags & DAISY_KDA_OUT_FP32) ? 1 : 0;
  sp.status = status_word;
  sp.chunk_tab = chunk_tab; sp.seq_ptr = seq_ptr;
  const int BH = n_seq * H;
  // V-slices: 64 rows (4 warps) fill the machine when there are >= 48 (sequence, head) pairs; fewer take narrower slices
  int rc;
  if (BH * 2 >= 96) rc = launch_state<4, 1, 2>(sp, BH, st);
  else if (BH * 4 >= 96) rc = launch_state<2, 2, 2>(sp, BH, st);
  else rc = launch_state<1, 2, 3>(sp, BH, st);
  if (rc != DAISY_OK) { (void)cudaGetLastError(); return rc; }
  return DAISY_OK;
}

extern "C" int daisy_b200_kda_chunk_fwd(const void* q, const void* k, const void* v, const float* g,
                                        const float* beta, const float* h0, void* o, float* hT,
                                        int B, int T, int H, int K, int V, int chunk, float scale,
                                        unsigned flags, void* workspace, size_t workspace_bytes,
                                        int* status_word, void* stream) {
  if (T <= 0) return DAISY_EINVAL;
  return kda_launch(q, k, v, g, beta, h0, o, hT, B, T, H, K, V, chunk, scale, flags, workspace, workspace_bytes,
                    (T + KC - 1) / KC, B, nullptr, nullptr, status_word, stream);
}

extern "C" size_t daisy_b200_kda_varlen_workspace_bytes(int n_chunks, int H, int K, int V) {
  if (n_chunks <= 0 || H <= 0 || K != KD || V != KD) return 0;
  return (size_t)H * n_chunks * REC_BYTES;
}

extern "C" int daisy_b200_kda_chunk_fwd_varlen(const void* q, const void* k, const void* v, const float* g,
                                               const float* beta, const float* h0, void* o, float* hT,
                                               int T_total, int H, int K, int V, int chunk, float scale, unsigned flags,
                                               const int32_t* chunk_tab, int n_chunks, const int32_t* seq_ptr, int n_seq,
                                               void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
  if (!chunk_tab || !seq_ptr || n_chunks <= 0 || n_seq <= 0) return DAISY_EINVAL;
  if ((reinterpret_cast<uintptr_t>(chunk_tab) & 7) || (reinterpret_cast<uintptr_t>(seq_ptr) & 3)) return DAISY_EALIGN;
  return kda_launch(q, k, v, g, beta, h0, o, hT, 1, T_total, H, K, V, chunk, scale, flags, workspace, workspace_bytes,
                    n_chunks, n_seq, chunk_tab, seq_ptr, status_word, stream);
}
