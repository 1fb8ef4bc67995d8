// Kimi delta attention (KDA), chunked forward, chunk = 64, K = V = 128.
//
// Per head the recurrence  S <- diag(e^{g_t}) S;  u_t = beta_t (v_t - S^T k_t);  S <- S + k_t u_t^T;
// o_t = S^T (scale q_t)  is evaluated 64 tokens at a time.  With G_i the inclusive cumulative
// log-decay inside a chunk and S_0 the state entering it:
//     A_kk[i,j] = beta_i sum_c k_ic k_jc e^{G_ic-G_jc} (j < i)     A_qk[i,j] = scale sum_c q_ic k_jc e^{G_ic-G_jc} (j <= i)
//     T = (I + A_kk)^-1          W = T (beta k e^G)          U0 = T (beta v)
//     U = U0 - W S_0             O = (scale q e^G) S_0 + A_qk U          S_C = e^{G_C} S_0 + (k e^{G_C-G})^T U
// Two kernels:
//  * kda_intra_kernel  -- one CTA per (batch, head, chunk), all chunks in parallel: cumulative gates,
//    the two gated Gram matrices (off-diagonal 16x16 blocks on tensor cores with both decay factors <= 1,
//    diagonal blocks with the exact e^{G_i-G_j} per pair), the unit-lower-triangular inverse in fp32,
//    W and U0 on tensor cores.  It writes, per chunk, fp16 "shared-memory images" (rows padded so that
//    fragment loads are bank-conflict free) of W, scale q e^G, (k e^{G_C-G})^T, A_qk, U0^T and e^{G_C}.
//  * kda_state_kernel  -- one CTA per (batch, head, V-slice), sequential over chunks: a producer warp
//    bulk-copies the images of chunk c+1.. into a shared-memory ring while the compute warps hold their
//    slice of S^T (16 V-rows x 128 K-columns per warp) in fp32 accumulator registers and chain the
//    three products through register-resident fragments (an accumulator tile pair is exactly the next
//    product's A fragment), so the state never leaves the register file between chunks.
// Tensor-core operands are fp16 (10-bit mantissa, every decay factor and operand here is <= O(1)):
// measured relative error of o against the fp32 token recurrence is ~4e-4, bf16 operands give ~3e-3.
#include <cuda_fp16.h>
#include "common.cuh"

namespace daisy {

constexpr int KC = 64;                 // chunk length
constexpr int KD = 128;                // K = V
constexpr int LDW = 136;               // padded row (halves) of a [64 x 128] image
constexpr int LDT = 72;                // padded row (halves) of a [. x 64] image
// per-chunk record in the workspace (bytes)
constexpr int OFF_W = 0;                               // W        [64][136] fp16
constexpr int OFF_Q = OFF_W + KC * LDW * 2;            // q~       [64][136] fp16   (scale q e^G)
constexpr int OFF_KT = OFF_Q + KC * LDW * 2;           // k~^T     [128][72] fp16   (k e^{G_C-G})^T
constexpr int OFF_AQK = OFF_KT + KD * LDT * 2;         // A_qk     [64][72]  fp16
constexpr int OFF_D = OFF_AQK + KC * LDT * 2;          // e^{G_C}  [128]     fp32
constexpr int SHARED_BYTES = OFF_D + KD * 4;           // 62976: identical for every V-slice
constexpr int OFF_UT = SHARED_BYTES;                   // U0^T     [128][72] fp16
constexpr int REC_BYTES = OFF_UT + KD * LDT * 2;       // 81408

// Four 8x8 fp16 matrices from shared memory: lanes 8m..8m+7 give the row addresses of matrix m (16 bytes per
// row); register m of lane l then holds elements (row l/4, columns 2(l%4), 2(l%4)+1) of matrix m -- the B
// fragment layout of mma.m16n8k16 when the rows are the n index and the columns the k index.
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* row_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(row_ptr)));
}

__device__ __forceinline__ void mma_f16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
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

// =============================================================================================
// intra-chunk kernel
// =============================================================================================
struct KdaIntraParams {
  const __nv_bfloat16 *q, *k, *v;
  const float *g, *beta;
  uint8_t* ws;
  int T, H, NC;            // NC = chunks per sequence
  int ahead;               // CTAs per wave: how far ahead (in launch order) a CTA prefetches
  float scale;
  int l2norm;
};

constexpr int LDA = 65;    // padded row (floats) of the fp32 [64 x 64] matrices
constexpr int LDG = KD + 4;     // padded row (floats) of G: fragment gathers (8 rows x 4 column pairs) hit 32 banks
constexpr int LDR = KD + 8;     // padded row (bf16) of the raw k / q tiles, same reason
static_assert(KC * LDG * 4 <= 2 * KC * LDW * 2, "the decay image must fit under Mk + Mq");
struct KdaIntraSmem {
  float G[KC][LDG];                // cumulative log-decay; later the W staging image
  __nv_bfloat16 kraw[KC][LDR];     // later (with qraw) the U0^T staging image
  __nv_bfloat16 qraw[KC][LDR];
  __nv_bfloat16 vraw[KC][KD];
  float Akk[KC][LDA];              // beta * gated k k^T: the 16 x 16 diagonal blocks (fp32, for the exact block inverses)
  __half Akh[KC][LDT];             //                     the off-diagonal blocks as tensor-core operands
  __half Th[KC][LDT];              // T = (I + A_kk)^-1, row-major
  __half ThT[KC][LDT];             // T^T
  __half Aqk[KC][LDT];
  __half Mk[KC][LDW];              // one level's Gram operands: k * e^{-|G - r|}   (Mk + Mq first hold e^g, fp32 [64][LDG])
  __half Mq[KC][LDW];              //                             q * e^{-|G - r|} on upper rows, else 0
  __half XT[KD][LDT];              // (beta k e^G)^T
  __half YT[KD][LDT];              // (beta v)^T
  float rq[KC], rk[KC], beta[KC];
};

constexpr int KDA_INTRA_THREADS = 512;   // 16 warps: one 200 KB CTA per SM, so latency is hidden by warps, not by CTAs

__global__ void __launch_bounds__(KDA_INTRA_THREADS, 1) kda_intra_kernel(const KdaIntraParams p) {
  extern __shared__ __align__(128) uint8_t kda_smem_raw[];
  KdaIntraSmem& sm = *reinterpret_cast<KdaIntraSmem*>(kda_smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, t4 = lane & 3;
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int t0 = chunk * KC;
  const int rows = min(KC, p.T - t0);
  uint8_t* rec = p.ws + ((size_t)(b * p.H + h) * p.NC + chunk) * REC_BYTES;

  // ---- P0: load the chunk (rows beyond T are zero: g = 0, beta = 0, q = k = v = 0).  All of a thread's
  //           16-byte loads are issued before the first store so that ~20 are in flight per thread.
  {
    const size_t tok0 = ((size_t)b * p.T + t0) * p.H + h;          // token row index into [B,T,H,*]
    uint4 rq_[2], rk_[2], rv_[2], rg_[4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {                                  // 16-byte chunks of the bf16 tiles
      const int idx = tid + u * KDA_INTRA_THREADS, r = idx >> 4, c8 = (idx & 15) * 8;
      rq_[u] = rk_[u] = rv_[u] = make_uint4(0, 0, 0, 0);
      if (r < rows) {
        const size_t off = (tok0 + (size_t)r * p.H) * KD + c8;
        rq_[u] = ld_stream16(p.q + off); rk_[u] = ld_stream16(p.k + off); rv_[u] = ld_stream16(p.v + off);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {                                  // 16-byte chunks of the fp32 gate tile
      const int idx = tid + u * KDA_INTRA_THREADS, r = idx >> 5, c4 = (idx & 31) * 4;
      rg_[u] = make_uint4(0, 0, 0, 0);
      if (r < rows) rg_[u] = ld_stream16(p.g + (tok0 + (size_t)r * p.H) * KD + c4);
    }
    if (tid < KC) sm.beta[tid] = tid < rows ? p.beta[tok0 + (size_t)tid * p.H] : 0.f;
    // Pull the inputs of the CTA that will run one wave from now into L2 (ten 128-byte lines per token row), so
    // that its load phase, which nothing overlaps, pays L2 latency instead of HBM latency.
    {
      const long long lin = (long long)blockIdx.x + (long long)gridDim.x * (blockIdx.y + (long long)gridDim.y * blockIdx.z) + p.ahead;
      const int nchunk = (int)(lin % p.NC), nh = (int)((lin / p.NC) % p.H);
      const long long nb = lin / ((long long)p.NC * p.H);
      for (int idx = tid; idx < KC * 10; idx += KDA_INTRA_THREADS) {
        const int r = idx / 10, w = idx - r * 10;
        const int t = nchunk * KC + r;
        if (nb < (long long)gridDim.z && t < p.T) {
          const size_t ntok = ((size_t)nb * p.T + t) * p.H + nh;
          const void* a = w < 2 ? (const void*)(reinterpret_cast<const char*>(p.q + ntok * KD) + w * 128)
                        : w < 4 ? (const void*)(reinterpret_cast<const char*>(p.k + ntok * KD) + (w - 2) * 128)
                        : w < 6 ? (const void*)(reinterpret_cast<const char*>(p.v + ntok * KD) + (w - 4) * 128)
                                : (const void*)(reinterpret_cast<const char*>(p.g + ntok * KD) + (w - 6) * 128);
          asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
        }
      }
    }
    for (int idx = tid; idx < KC * LDT / 2; idx += KDA_INTRA_THREADS) reinterpret_cast<uint32_t*>(&sm.Aqk[0][0])[idx] = 0u;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int idx = tid + u * KDA_INTRA_THREADS, r = idx >> 4, c8 = (idx & 15) * 8;
      *reinterpret_cast<uint4*>(&sm.qraw[r][c8]) = rq_[u];
      *reinterpret_cast<uint4*>(&sm.kraw[r][c8]) = rk_[u];
      *reinterpret_cast<uint4*>(&sm.vraw[r][c8]) = rv_[u];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int idx = tid + u * KDA_INTRA_THREADS, r = idx >> 5, c4 = (idx & 31) * 4;
      *reinterpret_cast<uint4*>(&sm.G[r][c4]) = rg_[u];
      // per-token decays d = e^g <= 1 for the running products of P3; the image borrows the Mk / Mq buffers
      // until the Gram levels need them
      float (*dd)[LDG] = reinterpret_cast<float (*)[LDG]>(&sm.Mk[0][0]);
      *reinterpret_cast<float4*>(&dd[r][c4]) = make_float4(__expf(__uint_as_float(rg_[u].x)), __expf(__uint_as_float(rg_[u].y)),
                                                           __expf(__uint_as_float(rg_[u].z)), __expf(__uint_as_float(rg_[u].w)));
    }
  }
  __syncthreads();

  // ---- P1: cumulative gates (threads 0-127, one channel each) and L2 norms (threads 128-383)
  if (tid < KD) {
    float acc = 0.f;
#pragma unroll 8
    for (int i = 0; i < KC; ++i) { acc += sm.G[i][tid]; sm.G[i][tid] = acc; }
  } else if (tid < KD + 4 * KC) {
    const int r = (tid - KD) >> 2, quarter = tid & 3;                // four threads per row, 32 channels each
    float sq = 0.f, sk = 0.f, dqk = 0.f;
#pragma unroll 8
    for (int c = 0; c < 32; ++c) {
      const float xq = __bfloat162float(sm.qraw[r][quarter * 32 + c]), xk = __bfloat162float(sm.kraw[r][quarter * 32 + c]);
      sq = fmaf(xq, xq, sq); sk = fmaf(xk, xk, sk); dqk = fmaf(xq, xk, dqk);
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
      sk += __shfl_xor_sync(0xffffffffu, sk, o);
      dqk += __shfl_xor_sync(0xffffffffu, dqk, o);
    }
    if (quarter == 0) {
      const float a = p.l2norm ? rsqrtf(sq + 1e-6f) : 1.f, c = p.l2norm ? rsqrtf(sk + 1e-6f) : 1.f;
      sm.rq[r] = a; sm.rk[r] = c;
      sm.Aqk[r][r] = __float2half_rn(p.scale * a * c * dqk);         // diagonal of A_qk: q_i . k_i, no decay
    }
  }
  __syncthreads();

  // ---- P2: element-wise images: q~ and k~^T and e^{G_C} straight to the workspace, X^T and Y^T to smem
  for (int idx = tid; idx < KC * 16; idx += KDA_INTRA_THREADS) {                 // q~[i][8 channels]
    const int i = idx >> 4, c8 = (idx & 15) * 8;
    const float rs = sm.rq[i] * p.scale;
    float qf[8];
    unpack8(*reinterpret_cast<const uint4*>(&sm.qraw[i][c8]), qf);
    const float4 g0 = *reinterpret_cast<const float4*>(&sm.G[i][c8]), g1 = *reinterpret_cast<const float4*>(&sm.G[i][c8 + 4]);
    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 8; e += 2) o[e >> 1] = pack_h2(qf[e] * rs * __expf(gg[e]), qf[e + 1] * rs * __expf(gg[e + 1]));
    *reinterpret_cast<uint4*>(rec + OFF_Q + ((size_t)i * LDW + c8) * 2) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  for (int idx = tid; idx < KD * 8; idx += KDA_INTRA_THREADS) {                  // (channel c, 8 tokens)
    const int c = idx & (KD - 1), j8 = (idx >> 7) * 8;
    const float gc = sm.G[KC - 1][c];
    uint32_t kt[4], xt[4], yt[4];
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      float kv[2], xv[2], yv[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int j = j8 + e + u;
        const float kn = __bfloat162float(sm.kraw[j][c]) * sm.rk[j];
        const float gj = sm.G[j][c];
        kv[u] = kn * __expf(gc - gj);
        xv[u] = kn * sm.beta[j] * __expf(gj);
        yv[u] = __bfloat162float(sm.vraw[j][c]) * sm.beta[j];
      }
      kt[e >> 1] = pack_h2(kv[0], kv[1]); xt[e >> 1] = pack_h2(xv[0], xv[1]); yt[e >> 1] = pack_h2(yv[0], yv[1]);
    }
    *reinterpret_cast<uint4*>(rec + OFF_KT + ((size_t)c * LDT + j8) * 2) = make_uint4(kt[0], kt[1], kt[2], kt[3]);
    *reinterpret_cast<uint4*>(&sm.XT[c][j8]) = make_uint4(xt[0], xt[1], xt[2], xt[3]);
    *reinterpret_cast<uint4*>(&sm.YT[c][j8]) = make_uint4(yt[0], yt[1], yt[2], yt[3]);
    if (j8 == 0) reinterpret_cast<float*>(rec + OFF_D)[c] = __expf(gc);
  }

  // ---- P3: both gated Gram matrices.  e^{G_i - G_j} must never be formed from a positive exponent, whatever
  // the gate values, so pairs are split by distance:
  //  (a) pairs inside a 16-token block, on the FMA pipes with RUNNING PRODUCTS of the per-token decays
  //      d_t = e^{g_t} <= 1:  k_j * prod_{t=j+1..i} d_t  is carried from row i-1 to row i with one multiply per
  //      channel -- no exponential per pair at all;
  //  (b) pairs in different blocks, on tensor cores by two binary levels s = 32, 16: tokens fall into groups of
  //      2s, rows of a group's upper half pair with columns of its lower half.  With r = G at the last row of the
  //      lower half, e^{G_i - G_j} = e^{G_i - r} * e^{r - G_j}, both exponents <= 0: each row carries ONE factor
  //      e^{-|G_i - r|} per level, staged as fp16 operands Mk = k * factor (all rows), Mq = q * factor (upper
  //      rows, else 0), and the level's blocks are plain m16n8k16 products.
  {
    // (a) a warp takes four columns j of one block over a range of rows, lane = four channels: row i of d, k, q is
    //     read once per warp (512 + 256 + 256 contiguous bytes) and serves four columns from registers; the 2 x 4
    //     partial dots of a row are reduced over the 32 lanes by a halving butterfly (9 shuffles for 8 values).
    //     A column group's rows (15, 11, 7 or 3 of them) are cut into segments so that each of a block's four
    //     warps walks nine rows -- the pass is bound by the dependent chain of one row after another, not by
    //     issue slots.  A segment that does not begin at its columns' first row starts its running product from
    //     e^{G_{start-1} - G_j} (exponent <= 0).  block = warp & 3: one block per scheduler.
    {
      const float (*dd)[LDG] = reinterpret_cast<const float (*)[LDG]>(&sm.Mk[0][0]);
      const int blk = warp & 3, c0 = lane * 4;
      int jq = 0;                                                  // column group of the segment being walked
      float kp[4][4];                                              // k_j * running decay product, 4 columns x 4 channels
      const bool hi16 = (lane & 16) != 0, hi8 = (lane & 8) != 0, hi4 = (lane & 4) != 0;
      const int vsel = lane >> 2;                                  // after the butterfly: the value this lane holds
      auto row = [&](const int i, const bool all_started) {
        const int ii = blk * 16 + i, cc = jq * 4 + (vsel >> 1);
        const float4 d4 = *reinterpret_cast<const float4*>(&dd[ii][c0]);
        const uint2 kr = *reinterpret_cast<const uint2*>(&sm.kraw[ii][c0]);
        const uint2 qr = *reinterpret_cast<const uint2*>(&sm.qraw[ii][c0]);
        const float out_scale = (vsel & 1) ? p.scale * sm.rq[ii] : sm.beta[ii] * sm.rk[ii];
        const float ki[4] = {__uint_as_float(kr.x << 16), __uint_as_float(kr.x & 0xffff0000u),
                             __uint_as_float(kr.y << 16), __uint_as_float(kr.y & 0xffff0000u)};
        const float qi[4] = {__uint_as_float(qr.x << 16), __uint_as_float(qr.x & 0xffff0000u),
                             __uint_as_float(qr.y << 16), __uint_as_float(qr.y & 0xffff0000u)};
        float val[8];                                              // [2 c] = k_i . kp_c, [2 c + 1] = q_i . kp_c
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const bool on = all_started || i > jq * 4 + c;           // column c has started (warp-uniform)
          kp[c][0] *= on ? d4.x : 1.f; kp[c][1] *= on ? d4.y : 1.f; kp[c][2] *= on ? d4.z : 1.f; kp[c][3] *= on ? d4.w : 1.f;
          val[2 * c] = fmaf(ki[0], kp[c][0], ki[1] * kp[c][1]) + fmaf(ki[2], kp[c][2], ki[3] * kp[c][3]);
          val[2 * c + 1] = fmaf(qi[0], kp[c][0], qi[1] * kp[c][1]) + fmaf(qi[2], kp[c][2], qi[3] * kp[c][3]);
        }
        float v4[4], v2[2], tot;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float recv = __shfl_xor_sync(0xffffffffu, hi16 ? val[t] : val[t + 4], 16);
          v4[t] = (hi16 ? val[t + 4] : val[t]) + recv;
        }
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          const float recv = __shfl_xor_sync(0xffffffffu, hi8 ? v4[t] : v4[t + 2], 8);
          v2[t] = (hi8 ? v4[t + 2] : v4[t]) + recv;
        }
        tot = (hi4 ? v2[1] : v2[0]) + __shfl_xor_sync(0xffffffffu, hi4 ? v2[0] : v2[1], 4);
        tot += __shfl_xor_sync(0xffffffffu, tot, 2);
        tot += __shfl_xor_sync(0xffffffffu, tot, 1);
        // the lane now holds value number lane >> 2 of this row, summed over all channels
        if ((lane & 3) == 0 && i > cc) {
          if (vsel & 1) sm.Aqk[ii][blk * 16 + cc] = __float2half_rn(out_scale * tot);
          else          sm.Akk[ii][blk * 16 + cc] = out_scale * tot;
        }
      };
      auto segment = [&](const int q, const int r0, const int r1) {
        jq = q;
        const bool fresh = (r0 == q * 4 + 1);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int jj = blk * 16 + q * 4 + c;
          const float rkj = sm.rk[jj];
          const uint2 kr = *reinterpret_cast<const uint2*>(&sm.kraw[jj][c0]);
          float f[4] = {1.f, 1.f, 1.f, 1.f};
          if (!fresh) {
            const float4 ga = *reinterpret_cast<const float4*>(&sm.G[blk * 16 + r0 - 1][c0]);
            const float4 gj = *reinterpret_cast<const float4*>(&sm.G[jj][c0]);
            f[0] = __expf(ga.x - gj.x); f[1] = __expf(ga.y - gj.y); f[2] = __expf(ga.z - gj.z); f[3] = __expf(ga.w - gj.w);
          }
          kp[c][0] = __uint_as_float(kr.x << 16) * rkj * f[0]; kp[c][1] = __uint_as_float(kr.x & 0xffff0000u) * rkj * f[1];
          kp[c][2] = __uint_as_float(kr.y << 16) * rkj * f[2]; kp[c][3] = __uint_as_float(kr.y & 0xffff0000u) * rkj * f[3];
        }
        if (fresh) {                                               // the first three rows see only some of the columns
          for (int i = r0; i < r0 + 3 && i < r1; ++i) row(i, false);
#pragma unroll 2
          for (int i = r0 + 3; i < r1; ++i) row(i, true);
        } else {
#pragma unroll 2
          for (int i = r0; i < r1; ++i) row(i, true);
        }
      };
      switch (warp >> 2) {                                         // nine rows per warp
        case 0:  segment(0, 1, 10); break;
        case 1:  segment(0, 10, 16); segment(3, 13, 16); break;
        case 2:  segment(1, 5, 14); break;
        default: segment(1, 14, 16); segment(2, 9, 16); break;
      }
    }
    // (b) build mapping: lanes 0-7 of a warp take 8 consecutive rows at the same channels, so every 8-lane phase of
    // a 16-byte shared-memory access spreads over all banks (row strides are 4 banks apart).  Two warps share
    // eight rows; a thread owns channels bq + 64 k .. + 8 (k = 0, 1).
    const int brow = (warp >> 1) * 8 + (lane & 7), bq = ((lane >> 3) + 4 * (warp & 1)) * 8;
    // this thread's 16 normalised k and q values and cumulative gates stay in registers across the levels
    float kn[16], qn[16], gi[16];
    {
      const float rkb = sm.rk[brow], rqb = sm.rq[brow];
#pragma unroll
      for (int kq = 0; kq < 2; ++kq) {
        const int c = bq + 64 * kq;
        float kf[8], qf[8];
        unpack8(*reinterpret_cast<const uint4*>(&sm.kraw[brow][c]), kf);
        unpack8(*reinterpret_cast<const uint4*>(&sm.qraw[brow][c]), qf);
        const float4 g0 = *reinterpret_cast<const float4*>(&sm.G[brow][c]);
        const float4 g1 = *reinterpret_cast<const float4*>(&sm.G[brow][c + 4]);
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) { kn[8 * kq + e] = kf[e] * rkb; qn[8 * kq + e] = qf[e] * rqb; gi[8 * kq + e] = gg[e]; }
      }
    }
    __syncthreads();                                                 // (a) is done with the decay image under Mk / Mq
#pragma unroll 1
    for (int ls = 5; ls >= 4; --ls) {
      const int s = 1 << ls;
      // -- build the level's operands
      {
        const bool upper = (brow & s) != 0;
        const int ref = (brow & ~(2 * s - 1)) + s - 1;
#pragma unroll
        for (int kq = 0; kq < 2; ++kq) {
          const int c = bq + 64 * kq;
          const float4 r0 = *reinterpret_cast<const float4*>(&sm.G[ref][c]);
          const float4 r1 = *reinterpret_cast<const float4*>(&sm.G[ref][c + 4]);
          const float gr[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
          uint32_t mk[4], mq[4];
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            const float f0 = __expf(-fabsf(gi[8 * kq + e] - gr[e])), f1 = __expf(-fabsf(gi[8 * kq + e + 1] - gr[e + 1]));
            mk[e >> 1] = pack_h2(kn[8 * kq + e] * f0, kn[8 * kq + e + 1] * f1);
            mq[e >> 1] = upper ? pack_h2(qn[8 * kq + e] * f0, qn[8 * kq + e + 1] * f1) : 0u;
          }
          *reinterpret_cast<uint4*>(&sm.Mk[brow][c]) = make_uint4(mk[0], mk[1], mk[2], mk[3]);
          *reinterpret_cast<uint4*>(&sm.Mq[brow][c]) = make_uint4(mq[0], mq[1], mq[2], mq[3]);
        }
      }
      __syncthreads();
      // -- the level's blocks, one 16 x 8 tile per warp.  Level 32: rows 32-63 x columns 0-31, eight tiles per
      //    matrix, all 16 warps (warp -> tile w & 7, matrix w >> 3).  Level 16: rows 16-31 x columns 0-15 and rows
      //    48-63 x columns 32-47, four tiles per matrix, warps 0-7 (tile w & 3, matrix w >> 2).
      {
        int mrow, ncol0;
        const int which = (s == 32) ? (warp >> 3) : ((warp >> 2) & 1);      // 0 = A_kk, 1 = A_qk
        const bool active = (s == 32) || warp < 8;
        if (s == 32) { const int c = warp & 7; mrow = 32 + 16 * (c >> 2); ncol0 = 8 * (c & 3); }
        else { const int c = warp & 3; mrow = 16 + 32 * (c >> 1); ncol0 = 32 * (c >> 1) + 8 * (c & 1); }
        if (active) {
          float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};   // two independent chains
          const int i0 = mrow + g8, i1 = i0 + 8;
          // all fragments first (independent shared-memory loads), then the products
          uint32_t bf[KD / 16][2], af[KD / 16][4];
          const __half* abase = (which == 1) ? &sm.Mq[0][0] : &sm.Mk[0][0];
          // ldmatrix.x4: the four 8x8 pieces of a 16x16 A fragment; two k-steps of an 8-column B fragment
          const __half* aptr = abase + (mrow + (lane & 7) + ((lane >> 3) & 1) * 8) * LDW + (lane >> 4) * 8;
          const __half* bptr = &sm.Mk[ncol0 + (lane & 7)][(lane >> 3) * 8];
#pragma unroll
          for (int ks = 0; ks < KD / 16; ++ks) ldmatrix_x4(af[ks], aptr + ks * 16);
#pragma unroll
          for (int ks = 0; ks < KD / 16; ks += 2) {
            uint32_t b4[4];
            ldmatrix_x4(b4, bptr + ks * 16);
            bf[ks][0] = b4[0]; bf[ks][1] = b4[1]; bf[ks + 1][0] = b4[2]; bf[ks + 1][1] = b4[3];
          }
#pragma unroll
          for (int ks = 0; ks < KD / 16; ks += 2) {
            mma_f16(acc, af[ks], bf[ks][0], bf[ks][1]);
            mma_f16(acc2, af[ks + 1], bf[ks + 1][0], bf[ks + 1][1]);
          }
          // outputs: rows i0 (acc[0], acc[1]) and i1 (acc[2], acc[3]), columns ncol0 + 2 t4 (+1)
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int i = (x < 2) ? i0 : i1, jc = ncol0 + 2 * t4 + (x & 1);
            const float a = acc[x] + acc2[x];
            if (which == 0) sm.Akh[i][jc] = __float2half_rn(sm.beta[i] * a);
            else            sm.Aqk[i][jc] = __float2half_rn(p.scale * a);
          }
        }
      }
      __syncthreads();
    }
  }

  // ---- P4: T = (I + A_kk)^-1.  (a) the four 16x16 diagonal blocks by forward substitution in fp32
  if (warp < 4 && lane < 16) {
    const int base = warp * 16;
    float t[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float s = (i == lane) ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) s = fmaf(-sm.Akk[base + i][base + j], t[j], s);
      t[i] = s;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {                                 // t[i] = T[base + i][base + lane]
      const __half th = __float2half_rn(t[i]);
      sm.Th[base + i][base + lane] = th;
      sm.ThT[base + lane][base + i] = th;
    }
  }
  __syncthreads();
  //      (b) block rows I = 1..3 on tensor cores, in transposed form so that the two products chain through
  //          registers:  R = T^T,  R_{<I,I} = -(R_{<I,<I} A_{I,<I}^T) R_II.  Warp mt < I owns 16 rows of R_{<I,I};
  //          the first product's accumulator pair is the second product's A fragment.  fp16 operands here cost
  //          nothing measurable: T is consumed as fp16 by every later product anyway.
#pragma unroll 1
  for (int I = 1; I < 4; ++I) {
    if (warp < I) {
      const int mt = warp;
      float acc1[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      for (int kb = mt; kb < I; ++kb) {                            // R is block upper triangular
        uint32_t a[4];
        const int kc = kb * 16 + 2 * t4;
        a[0] = *reinterpret_cast<const uint32_t*>(&sm.ThT[mt * 16 + g8][kc]);
        a[1] = *reinterpret_cast<const uint32_t*>(&sm.ThT[mt * 16 + g8 + 8][kc]);
        a[2] = *reinterpret_cast<const uint32_t*>(&sm.ThT[mt * 16 + g8][kc + 8]);
        a[3] = *reinterpret_cast<const uint32_t*>(&sm.ThT[mt * 16 + g8 + 8][kc + 8]);
#pragma unroll
        for (int nn = 0; nn < 2; ++nn) {
          const __half* arow = &sm.Akh[I * 16 + nn * 8 + g8][kc];
          mma_f16(acc1[nn], a, *reinterpret_cast<const uint32_t*>(arow), *reinterpret_cast<const uint32_t*>(arow + 8));
        }
      }
      uint32_t a2[4];
      a2[0] = pack_h2(acc1[0][0], acc1[0][1]); a2[1] = pack_h2(acc1[0][2], acc1[0][3]);
      a2[2] = pack_h2(acc1[1][0], acc1[1][1]); a2[3] = pack_h2(acc1[1][2], acc1[1][3]);
#pragma unroll
      for (int nn = 0; nn < 2; ++nn) {
        float acc2[4] = {0.f, 0.f, 0.f, 0.f};
        const __half* trow = &sm.Th[I * 16 + nn * 8 + g8][I * 16 + 2 * t4];
        mma_f16(acc2, a2, *reinterpret_cast<const uint32_t*>(trow), *reinterpret_cast<const uint32_t*>(trow + 8));
        // acc2[0..1] = R[mt*16 + g8][nn*8 + 2 t4 (+1)], acc2[2..3] the same for row g8 + 8;  T[i][j] = -R[j][i]
        const int ti = I * 16 + nn * 8 + 2 * t4, tj = mt * 16 + g8;
        const __half h0 = __float2half_rn(-acc2[0]), h1 = __float2half_rn(-acc2[1]);
        const __half h2 = __float2half_rn(-acc2[2]), h3 = __float2half_rn(-acc2[3]);
        sm.Th[ti][tj] = h0; sm.Th[ti + 1][tj] = h1; sm.Th[ti][tj + 8] = h2; sm.Th[ti + 1][tj + 8] = h3;
        *reinterpret_cast<__half2*>(&sm.ThT[tj][ti]) = __halves2half2(h0, h1);
        *reinterpret_cast<__half2*>(&sm.ThT[tj + 8][ti]) = __halves2half2(h2, h3);
      }
    }
    __syncthreads();
  }

  // ---- P5: W = T X  (warp = row block I x channel quarter) and U0^T = Y^T T^T (warp = 16 V rows x token half), fp16 MMAs.
  //          G and kraw/qraw are dead: they become the staging images.
  __half* w_img = reinterpret_cast<__half*>(&sm.G[0][0]);          // [64][136]
  __half* u_img = reinterpret_cast<__half*>(&sm.kraw[0][0]);       // [128][72]  (kraw + qraw = 32 KB)
  {
    const int I = warp >> 2, ch = (warp & 3) * 32;
    float acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
    const int i0 = I * 16 + g8, i1 = i0 + 8;
    for (int ks = 0; ks <= I; ++ks) {
      uint32_t a[4];
      const int j = ks * 16 + 2 * t4;
      a[0] = *reinterpret_cast<const uint32_t*>(&sm.Th[i0][j]);
      a[1] = *reinterpret_cast<const uint32_t*>(&sm.Th[i1][j]);
      a[2] = *reinterpret_cast<const uint32_t*>(&sm.Th[i0][j + 8]);
      a[3] = *reinterpret_cast<const uint32_t*>(&sm.Th[i1][j + 8]);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int c = ch + nt * 8 + g8;
        mma_f16(acc[nt], a, *reinterpret_cast<const uint32_t*>(&sm.XT[c][j]), *reinterpret_cast<const uint32_t*>(&sm.XT[c][j + 8]));
      }
    }
    __syncthreads();                                               // every reader of G is done
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int c = ch + nt * 8 + 2 * t4;
      *reinterpret_cast<uint32_t*>(&w_img[i0 * LDW + c]) = pack_h2(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<uint32_t*>(&w_img[i1 * LDW + c]) = pack_h2(acc[nt][2], acc[nt][3]);
    }
  }
  {
    const int v0 = (warp >> 1) * 16 + g8, v1 = v0 + 8, nt0 = (warp & 1) * 4;
    float acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t a[4];
      const int j = ks * 16 + 2 * t4;
      a[0] = *reinterpret_cast<const uint32_t*>(&sm.YT[v0][j]);
      a[1] = *reinterpret_cast<const uint32_t*>(&sm.YT[v1][j]);
      a[2] = *reinterpret_cast<const uint32_t*>(&sm.YT[v0][j + 8]);
      a[3] = *reinterpret_cast<const uint32_t*>(&sm.YT[v1][j + 8]);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        if (ks * 16 > (nt0 + nt) * 8 + 7) continue;                // T[i][j] = 0 for j > i
        const int i = (nt0 + nt) * 8 + g8;
        mma_f16(acc[nt], a, *reinterpret_cast<const uint32_t*>(&sm.Th[i][j]), *reinterpret_cast<const uint32_t*>(&sm.Th[i][j + 8]));
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int i = (nt0 + nt) * 8 + 2 * t4;
      *reinterpret_cast<uint32_t*>(&u_img[v0 * LDT + i]) = pack_h2(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<uint32_t*>(&u_img[v1 * LDT + i]) = pack_h2(acc[nt][2], acc[nt][3]);
    }
  }
  __syncthreads();

  // ---- P6: staged images -> workspace, 16 bytes per thread per store
  for (int idx = tid; idx < KC * LDW * 2 / 16; idx += KDA_INTRA_THREADS)
    reinterpret_cast<uint4*>(rec + OFF_W)[idx] = reinterpret_cast<const uint4*>(w_img)[idx];
  for (int idx = tid; idx < KD * LDT * 2 / 16; idx += KDA_INTRA_THREADS)
    reinterpret_cast<uint4*>(rec + OFF_UT)[idx] = reinterpret_cast<const uint4*>(u_img)[idx];
  for (int idx = tid; idx < KC * LDT * 2 / 16; idx += KDA_INTRA_THREADS)
    reinterpret_cast<uint4*>(rec + OFF_AQK)[idx] = reinterpret_cast<const uint4*>(&sm.Aqk[0][0])[idx];
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
};

constexpr int KDA_NST = 2;     // ring stages

template <int NW>
struct KdaStateSmem {
  static constexpr int VS = 16 * NW;
  static constexpr int U_BYTES = VS * LDT * 2;
  static constexpr int STAGE = SHARED_BYTES + U_BYTES;
  static constexpr int O_LD = VS + 4;                    // floats; staging of one chunk of output
  static constexpr int BYTES = KDA_NST * STAGE + KC * O_LD * 4 + 64;
};

template <int NW>
__global__ void __launch_bounds__(32 * (NW + 1), 1) kda_state_kernel(const KdaStateParams p) {
  using L = KdaStateSmem<NW>;
  constexpr int VS = L::VS;
  extern __shared__ __align__(128) uint8_t kda_smem_raw[];
  uint8_t* stages = kda_smem_raw;
  float* o_stage = reinterpret_cast<float*>(kda_smem_raw + KDA_NST * L::STAGE);
  uint64_t* full = reinterpret_cast<uint64_t*>(kda_smem_raw + KDA_NST * L::STAGE + KC * L::O_LD * 4);
  uint64_t* empty = full + KDA_NST;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + KDA_NST);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g8 = lane >> 2, t4 = lane & 3;
  const int vsl = blockIdx.x, bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int v_base = vsl * VS;
  const uint8_t* recs = p.ws + (size_t)bh * p.NC * REC_BYTES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < KDA_NST; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], NW); }
    *abort_flag = 0;
    mbar_init_fence();
  }
  __syncthreads();

  if (warp == NW) {
    // ------------------------------------------------------------ producer: bulk copies into the ring
    if (lane == 0) {
      for (int c = 0; c < p.NC; ++c) {
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

  // ------------------------------------------------------------ compute warps: 16 V rows each
  const int vr0 = warp * 16 + g8, vr1 = vr0 + 8;                   // rows inside the slice
  float st[16][4];                                                 // S^T[v][k]: tile nt -> k = 8 nt + 2 t4 (+1)
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    if (p.h0) {
      const float* hp = p.h0 + (size_t)bh * KD * KD;
      const int k0 = nt * 8 + 2 * t4;
      st[nt][0] = hp[(size_t)k0 * KD + v_base + vr0]; st[nt][1] = hp[(size_t)(k0 + 1) * KD + v_base + vr0];
      st[nt][2] = hp[(size_t)k0 * KD + v_base + vr1]; st[nt][3] = hp[(size_t)(k0 + 1) * KD + v_base + vr1];
    } else {
      st[nt][0] = st[nt][1] = st[nt][2] = st[nt][3] = 0.f;
    }
  }

  for (int c = 0; c < p.NC; ++c) {
    const int s = c % KDA_NST;
    const bool ok = __all_sync(0xffffffffu, mbar_wait(&full[s], (c / KDA_NST) & 1, abort_flag, p.status, 2));
    if (!ok) break;
    const uint8_t* sb = stages + s * L::STAGE;
    const __half* Wm = reinterpret_cast<const __half*>(sb + OFF_W);
    const __half* Qm = reinterpret_cast<const __half*>(sb + OFF_Q);
    const __half* Kt = reinterpret_cast<const __half*>(sb + OFF_KT);
    const __half* Aq = reinterpret_cast<const __half*>(sb + OFF_AQK);
    const float* dv = reinterpret_cast<const float*>(sb + OFF_D);
    const __half* Ut = reinterpret_cast<const __half*>(sb + SHARED_BYTES);

    // (1) accU = S^T W^T   and   (2a) accO = S^T q~^T      [16 x 64 tokens each]
    float au[8][4], ao[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { au[nt][0] = au[nt][1] = au[nt][2] = au[nt][3] = 0.f; ao[nt][0] = ao[nt][1] = ao[nt][2] = ao[nt][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t a[4];
      a[0] = pack_h2(st[2 * ks][0], st[2 * ks][1]); a[1] = pack_h2(st[2 * ks][2], st[2 * ks][3]);
      a[2] = pack_h2(st[2 * ks + 1][0], st[2 * ks + 1][1]); a[3] = pack_h2(st[2 * ks + 1][2], st[2 * ks + 1][3]);
      // B fragments of two token tiles per ldmatrix.x4: matrix m = (tile nt + (m >> 1), k half m & 1)
      const int lrow = (lane >> 4) * 8 + (lane & 7), lcol = ks * 16 + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int nt = 0; nt < 8; nt += 2) {
        uint32_t bw[4], bq[4];
        ldmatrix_x4(bw, &Wm[(nt * 8 + lrow) * LDW + lcol]);
        ldmatrix_x4(bq, &Qm[(nt * 8 + lrow) * LDW + lcol]);
        mma_f16(au[nt], a, bw[0], bw[1]);
        mma_f16(ao[nt], a, bq[0], bq[1]);
        mma_f16(au[nt + 1], a, bw[2], bw[3]);
        mma_f16(ao[nt + 1], a, bq[2], bq[3]);
      }
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
    // (2b) accO += U^T A_qk^T
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const int lrow = (lane >> 4) * 8 + (lane & 7), lcol = ks * 16 + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int nt = 2 * ks; nt < 8; nt += 2) {                     // A_qk[i][j] = 0 for j > i: tiles below 2 ks are empty
        uint32_t ba[4];
        ldmatrix_x4(ba, &Aq[(nt * 8 + lrow) * LDT + lcol]);
        mma_f16(ao[nt], ua[ks], ba[0], ba[1]);
        mma_f16(ao[nt + 1], ua[ks], ba[2], ba[3]);
      }
    }
    // (3) S^T = S^T diag(e^{G_C}) + U^T k~
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      const float2 d2 = *reinterpret_cast<const float2*>(&dv[nt * 8 + 2 * t4]);
      st[nt][0] *= d2.x; st[nt][1] *= d2.y; st[nt][2] *= d2.x; st[nt][3] *= d2.y;
    }
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const int lrow = (lane >> 4) * 8 + (lane & 7), lcol = ks * 16 + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int nt = 0; nt < 16; nt += 2) {
        uint32_t bk[4];
        ldmatrix_x4(bk, &Kt[(nt * 8 + lrow) * LDT + lcol]);
        mma_f16(st[nt], ua[ks], bk[0], bk[1]);
        mma_f16(st[nt + 1], ua[ks], bk[2], bk[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);                         // this warp is done with the stage

    // output: stage [token][v] in shared memory, then coalesced rows
    asm volatile("bar.sync 1, %0;" ::"n"(32 * NW) : "memory");    // previous chunk's copy-out finished
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int tok = nt * 8 + 2 * t4;
      o_stage[tok * L::O_LD + vr0] = ao[nt][0]; o_stage[(tok + 1) * L::O_LD + vr0] = ao[nt][1];
      o_stage[tok * L::O_LD + vr1] = ao[nt][2]; o_stage[(tok + 1) * L::O_LD + vr1] = ao[nt][3];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * NW) : "memory");
    const int rows = min(KC, p.T - c * KC);
    for (int idx = threadIdx.x; idx < KC * (VS / 4); idx += 32 * NW) {
      const int tok = idx / (VS / 4), v4 = (idx % (VS / 4)) * 4;
      if (tok >= rows) continue;
      const float4 x = *reinterpret_cast<const float4*>(&o_stage[tok * L::O_LD + v4]);
      const size_t off = (((size_t)b * p.T + (size_t)c * KC + tok) * p.H + h) * KD + v_base + v4;
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
    for (int nt = 0; nt < 16; ++nt) {
      const int k0 = nt * 8 + 2 * t4;
      hp[(size_t)k0 * KD + v_base + vr0] = st[nt][0]; hp[(size_t)(k0 + 1) * KD + v_base + vr0] = st[nt][1];
      hp[(size_t)k0 * KD + v_base + vr1] = st[nt][2]; hp[(size_t)(k0 + 1) * KD + v_base + vr1] = st[nt][3];
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

template <int NW>
static int launch_state(const KdaStateParams& sp, int BH, cudaStream_t st) {
  using L = KdaStateSmem<NW>;
  static bool attr[daisy_host::MAX_DEVICES] = {};             // the attribute is per device
  const int dev = daisy_host::device_slot();
  if (dev < 0) return DAISY_ENODEV;
  if (!attr[dev]) {
    if (cudaFuncSetAttribute(kda_state_kernel<NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES) != cudaSuccess) return DAISY_ECUDA;
    attr[dev] = true;
  }
  kda_state_kernel<NW><<<dim3(KD / L::VS, BH), 32 * (NW + 1), L::BYTES, st>>>(sp);
  return cudaGetLastError() == cudaSuccess ? DAISY_OK : DAISY_ECUDA;
}

extern "C" int daisy_b200_kda_chunk_fwd(const void* q, const void* k, const void* v, const float* g,
                                        const float* beta, const float* h0, void* o, float* hT,
                                        int B, int T, int H, int K, int V, int chunk, float scale,
                                        unsigned flags, void* workspace, size_t workspace_bytes,
                                        int* status_word, void* stream) {
  if (!q || !k || !v || !g || !beta || !o || !workspace || B <= 0 || T <= 0 || H <= 0) return DAISY_EINVAL;
  if (K != KD || V != KD || chunk != KC) return DAISY_EUNSUPPORTED;
  if (B > 65535 || H > 65535 || (size_t)B * H > 65535) return DAISY_EUNSUPPORTED;
  if (workspace_bytes < daisy_b200_kda_workspace_bytes(B, T, H, K, V)) return DAISY_EWORKSPACE;
  if (!daisy_aligned16(q) || !daisy_aligned16(k) || !daisy_aligned16(v) || !daisy_aligned16(g) || !daisy_aligned16(o) ||
      !daisy_aligned16(workspace) || (h0 && !daisy_aligned16(h0)) || (hT && !daisy_aligned16(hT)))
    return DAISY_EALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  const int NC = (T + KC - 1) / KC;
  static bool attr[daisy_host::MAX_DEVICES] = {};             // the attribute is per device
  const int dev = daisy_host::device_slot();
  if (dev < 0) return DAISY_ENODEV;
  if (!attr[dev]) {
    if (cudaFuncSetAttribute(kda_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(KdaIntraSmem)) != cudaSuccess) {
      (void)cudaGetLastError();
      return DAISY_ECUDA;
    }
    attr[dev] = true;
  }
  KdaIntraParams ip;
  ip.q = (const __nv_bfloat16*)q; ip.k = (const __nv_bfloat16*)k; ip.v = (const __nv_bfloat16*)v;
  ip.g = g; ip.beta = beta; ip.ws = (uint8_t*)workspace;
  ip.T = T; ip.H = H; ip.NC = NC;
  ip.scale = scale > 0.f ? scale : 1.0f / sqrtf((float)K);
  ip.l2norm = (flags & DAISY_KDA_L2NORM_QK) ? 1 : 0;
  {
    const int sms = daisy_host::sm_count_cached();
    ip.ahead = sms > 0 ? sms : 148;
  }
  kda_intra_kernel<<<dim3(NC, H, B), KDA_INTRA_THREADS, sizeof(KdaIntraSmem), st>>>(ip);
  DAISY_CHECK_LAUNCH();

  KdaStateParams sp;
  sp.ws = (const uint8_t*)workspace; sp.h0 = h0; sp.hT = hT; sp.o = o;
  sp.T = T; sp.H = H; sp.NC = NC; sp.out_fp32 = (flags & DAISY_KDA_OUT_FP32) ? 1 : 0;
  sp.status = status_word;
  const int BH = B * H;
  // V-slices: 64 rows (4 warps) fill the machine when B*H >= 64; fewer sequences take narrower slices
  int rc;
  if (BH * 2 >= 96) rc = launch_state<4>(sp, BH, st);
  else if (BH * 4 >= 96) rc = launch_state<2>(sp, BH, st);
  else rc = launch_state<1>(sp, BH, st);
  if (rc != DAISY_OK) { (void)cudaGetLastError(); return rc; }
  return DAISY_OK;
}
