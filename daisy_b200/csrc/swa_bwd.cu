// Backward pass of the sliding-window causal softmax attention (the training form,
// models/daisy/attention.py:156-162 under autograd), on tcgen05 tensor cores.
//
// With Z = scale Q K^T (masked), P = softmax(Z), O = P V and the incoming gradient dO:
//     delta_q = sum_d dO[q,d] O[q,d]        dP = dO V^T        dZ = P o (dP - delta)
//     dV = P^T dO        dK = scale dZ^T Q        dQ = scale dZ K
// P is rebuilt from the forward's per-row log2 denominators: P[q,k] = 2^(Z[q,k] log2 e - lse2[q]).
//
// One kernel template, two launches, no atomics (bitwise deterministic):
//   MODE 0  key block stationary:  item = 128 keys of one (batch, head); K_j, V_j stay in shared memory, the query
//           blocks that can see them stream through (Q_i, dO_i).  Scores are formed TRANSPOSED,
//           S^T = K_j Q_i^T and dP^T = V_j dO_i^T (TMEM lane = key), so P^T and dZ^T, rounded to bf16 and written back
//           over them, are exactly the TMEM A operands of  dV += P^T dO_i  and  dK += dZ^T Q_i.
//   MODE 1  query block stationary:  item = 128 queries; Q_i, dO_i stay, the key blocks of the window stream
//           (K_j, V_j);  S = Q_i K_j^T, dP = dO_i V_j^T (TMEM lane = query),  dQ += dZ K_j.
// In both:  S = X0 Y0^T,  dP = X1 Y1^T  (X stationary, Y streamed),  acc1 += dZ Y0,  and MODE 0 also acc0 += P Y1.
// Roles (576 threads): warps 0-15 rebuild P / dZ -- four warpgroups, thread = TMEM lane, 32 of a tile's 128 columns
// each (every warpgroup writes its bf16 results over the first 16 columns of its OWN 32, so nobody overwrites
// columns somebody else still has to read) -- and write the results; warp 16 TMA producer, warp 17 MMA issuer.
// TMEM: S [0,128) dP [128,256) acc0 [256,384) acc1 [384,512).
// All mbarrier waits are bounded (abort flag, DAISY_ETIMEOUT through the status word).
#include "common.cuh"

namespace daisy {

constexpr int WB = 128;                                   // block of queries / keys
constexpr int W_TILE = WB * DAISY_HEAD_DIM * 2;           // 32768
constexpr int W_HALF = W_TILE / 2;
constexpr int W_NST = 2;                                  // stages of streamed (Y0, Y1) tile pairs
constexpr int BWD_THREADS = 576;
constexpr int BWD_WORKERS = 512;                          // threads of warps 0-15
constexpr int BWD_SMEM = 1024 + 2 * W_TILE + W_NST * 2 * W_TILE + 2 * 3 * WB * 4 + 256;
static_assert(BWD_SMEM <= 232448, "over the 227 KB a CTA may use");

struct BwdParams {
  const float* lse2;        // [B,H,T]
  const float* delta;       // [B,H,T]
  const int* doc_start;     // null or [.,T], batch stride doc_sb
  int64_t doc_sb;
  __nv_bfloat16 *d0, *d1;   // outputs: MODE 0: dV, dK; MODE 1: (unused), dQ -- [B,T,H,D] contiguous
  int T, H, B, window, window_blocks;
  float scale, scale_log2;
  int* status;
};

struct BwdBars {
  uint64_t x_full, x_empty, y_full[W_NST], y_empty[W_NST], s_full[2], p_full[2], acc_full, acc_empty;
  uint32_t tmem_base;
  int abort_flag;
};

// Streamed block range [lo, hi] of an item.
template <int MODE>
__device__ __forceinline__ void bwd_range(int blk, int nblk, int T, int window, int window_blocks, const int* doc_row, int& lo, int& hi) {
  if (MODE == 0) {                                         // key block blk: query blocks that can see it
    lo = blk;
    hi = nblk - 1;
    if (window_blocks > 0) hi = min(hi, blk + window_blocks - 1);
    else if (window > 0) hi = min(hi, (blk * WB + WB - 1 + window - 1) / WB);
  } else {                                                 // query block blk: key blocks inside its window
    hi = blk;
    int klo = 0;
    if (window_blocks > 0) klo = max(0, blk - window_blocks + 1) * WB;
    else if (window > 0) klo = max(0, blk * WB - window + 1);
    if (doc_row) klo = max(klo, min(doc_row[blk * WB], blk * WB));    // keys before the first row's document: invisible to all
    lo = klo / WB;
  }
}

template <int MODE>
__global__ void __launch_bounds__(BWD_THREADS, 1)
swa_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do, const BwdParams p) {
  extern __shared__ uint8_t bwd_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(bwd_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* x_tiles = smem;                                           // X0, X1
  uint8_t* y_tiles = smem + 2 * W_TILE;                              // per stage: Y0, Y1
  float* col_f = reinterpret_cast<float*>(y_tiles + W_NST * 2 * W_TILE);   // MODE 0: [2][lse2 | delta | doc_start][128]
  BwdBars* bars = reinterpret_cast<BwdBars*>(reinterpret_cast<uint8_t*>(col_f) + 2 * 3 * WB * 4);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = p.T, nblk = (T + WB - 1) / WB;
  // blocks whose range is cut short by the sequence's end (MODE 0: the last key blocks) or start (MODE 1: the first
  // query blocks) go last, longest first
  const int span = p.window_blocks > 0 ? p.window_blocks * WB : p.window;
  const BalancedWalk walk(nblk, p.H * p.B, span > 0 ? (span + WB - 1) / WB : nblk, MODE == 0);
  const CUtensorMap* tx0 = MODE == 0 ? &tm_k : &tm_q;
  const CUtensorMap* tx1 = MODE == 0 ? &tm_v : &tm_do;
  const CUtensorMap* ty0 = MODE == 0 ? &tm_q : &tm_k;
  const CUtensorMap* ty1 = MODE == 0 ? &tm_do : &tm_v;

  if (threadIdx.x == 0) {
    mbar_init(&bars->x_full, 1); mbar_init(&bars->x_empty, 1);
    for (int i = 0; i < W_NST; ++i) { mbar_init(&bars->y_full[i], 1); mbar_init(&bars->y_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->s_full[i], 1); mbar_init(&bars->p_full[i], BWD_WORKERS / 2); }
    mbar_init(&bars->acc_full, 1); mbar_init(&bars->acc_empty, BWD_WORKERS);
    bars->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 17) { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 16) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_do);
      uint32_t n = 0, it = 0;
      bool ok = true;
      for (int item; (item = walk.at((int)it)) >= 0 && ok; ++it) {
        const int blk = item % nblk, bh = item / nblk, h = bh % p.H, b = bh / p.H;
        int lo, hi;
        bwd_range<MODE>(blk, nblk, T, p.window, p.window_blocks, p.doc_start ? p.doc_start + b * p.doc_sb : nullptr, lo, hi);
        if (!mbar_wait(&bars->x_empty, (it & 1) ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
        mbar_expect_tx(&bars->x_full, 2 * W_TILE);
        tma_load_4d(x_tiles, tx0, &bars->x_full, 0, blk * WB, h, b);
        tma_load_4d(x_tiles + W_HALF, tx0, &bars->x_full, 64, blk * WB, h, b);
        tma_load_4d(x_tiles + W_TILE, tx1, &bars->x_full, 0, blk * WB, h, b);
        tma_load_4d(x_tiles + W_TILE + W_HALF, tx1, &bars->x_full, 64, blk * WB, h, b);
        for (int y = lo; y <= hi && ok; ++y, ++n) {
          const int st = n % W_NST;
          if (!mbar_wait(&bars->y_empty[st], ((n / W_NST) & 1) ^ 1, abort_flag, p.status, 2)) { ok = false; break; }
          uint8_t* dst = y_tiles + st * 2 * W_TILE;
          mbar_expect_tx(&bars->y_full[st], 2 * W_TILE);
          tma_load_4d(dst, ty0, &bars->y_full[st], 0, y * WB, h, b);
          tma_load_4d(dst + W_HALF, ty0, &bars->y_full[st], 64, y * WB, h, b);
          tma_load_4d(dst + W_TILE, ty1, &bars->y_full[st], 0, y * WB, h, b);
          tma_load_4d(dst + W_TILE + W_HALF, ty1, &bars->y_full[st], 64, y * WB, h, b);
        }
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------------ MMA issuer
    // The score tiles are formed and consumed in two halves of 64 streamed rows (= 64 TMEM columns), two worker
    // warpgroups each, and the halves are software-pipelined: while the warpgroups of a half rebuild its P / dZ, the tensor core
    // forms the other half's scores, accumulates the previous half's products and already forms the NEXT tile's
    // scores of a half as soon as that half's columns have been consumed:
    //   S0(y) S1(y) | wait P0(y): A0(y) S0(y+1) | wait P1(y): A1(y) S1(y+1) | wait P0(y+1): ...
    // (S = both score products of a half, A = both accumulating products).  tcgen05 MMAs of one thread execute in
    // order, so S_h(y+1) overwrites columns that A_h(y) has finished reading.
    const uint32_t leader = elect_one() ? 1u : 0u;
    constexpr uint32_t idesc_s = umma_idesc_bf16(WB, WB / 2, 0, 0);               // X Y_half^T: both K-major, 64 streamed rows
    constexpr uint32_t idesc_a = umma_idesc_bf16(WB, DAISY_HEAD_DIM, 0, 1);       // (P | dZ from TMEM) x Y: Y as an MN-major operand
    const uint64_t xd = umma_desc_sw128(smem_u32(x_tiles), 16, 1024);
    const uint64_t yd = umma_desc_sw128(smem_u32(y_tiles), 16, 1024);
    const uint64_t ymn = umma_desc_sw128(smem_u32(y_tiles), W_HALF, 1024);
    const uint32_t x_lo0 = (uint32_t)xd, y_lo0 = (uint32_t)yd, k_hi = (uint32_t)(xd >> 32);
    const uint32_t ymn_lo0 = (uint32_t)ymn, ymn_hi = (uint32_t)(ymn >> 32);
    const uint32_t s_t = tmem_base, dp_t = tmem_base + 128, a0_t = tmem_base + 256, a1_t = tmem_base + 384;
    uint32_t n = 0, it = 0;
    bool ok = true;
    // both score products of half hf of the tile in stage st
    auto scores = [&](int st, int hf) {
      const uint32_t y0 = y_lo0 + st * ((2 * W_TILE) >> 4) + hf * ((64 * 128) >> 4), y1 = y0 + (W_TILE >> 4);
#pragma unroll
      for (int k = 0; k < DAISY_HEAD_DIM / 16; ++k) {                            // S = X0 Y0^T
        const uint32_t off = ((k >> 2) * W_HALF + (k & 3) * 32) >> 4;
        umma_ss_lh_p(leader, s_t + 64 * hf, x_lo0 + off, k_hi, y0 + off, k_hi, idesc_s, k > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int k = 0; k < DAISY_HEAD_DIM / 16; ++k) {                            // dP = X1 Y1^T
        const uint32_t off = ((k >> 2) * W_HALF + (k & 3) * 32) >> 4;
        umma_ss_lh_p(leader, dp_t + 64 * hf, x_lo0 + (W_TILE >> 4) + off, k_hi, y1 + off, k_hi, idesc_s, k > 0 ? 1u : 0u);
      }
      tc_commit_p(leader, &bars->s_full[hf]);
    };
    // both accumulating products over the 64 streamed rows of half hf
    auto accumulate = [&](int st, int hf, uint32_t acc) {
      const uint32_t ymn0 = ymn_lo0 + st * ((2 * W_TILE) >> 4), ymn1 = ymn0 + (W_TILE >> 4);
      if (MODE == 0) {
#pragma unroll
        for (int k = 4 * hf; k < 4 * hf + 4; ++k)                               // acc0 += P Y1   (dV += P^T dO)
          umma_ts_lh_p(leader, a0_t, s_t + (k & 1) * 8 + (k >> 1) * 32, ymn1 + k * (2048 >> 4), ymn_hi, idesc_a, (acc || k > 4 * hf) ? 1u : 0u);
      }
#pragma unroll
      for (int k = 4 * hf; k < 4 * hf + 4; ++k)                                 // acc1 += dZ Y0  (dK += dZ^T Q | dQ += dZ K)
        umma_ts_lh_p(leader, a1_t, dp_t + (k & 1) * 8 + (k >> 1) * 32, ymn0 + k * (2048 >> 4), ymn_hi, idesc_a, (acc || k > 4 * hf) ? 1u : 0u);
    };
    for (int item; (item = walk.at((int)it)) >= 0 && ok; ++it) {
      const int blk = item % nblk, bh = item / nblk, b = bh / p.H;
      int lo, hi;
      bwd_range<MODE>(blk, nblk, T, p.window, p.window_blocks, p.doc_start ? p.doc_start + b * p.doc_sb : nullptr, lo, hi);
      if (!mbar_wait(&bars->x_full, it & 1, abort_flag, p.status, 3)) { ok = false; break; }
      // the item's first tile
      if (!mbar_wait(&bars->y_full[n % W_NST], (n / W_NST) & 1, abort_flag, p.status, 4)) { ok = false; break; }
      tc_fence_after();
      scores(n % W_NST, 0);
      scores(n % W_NST, 1);
      // its first accumulating products overwrite the accumulators: the workers have read out the previous item's
      if (!mbar_wait(&bars->acc_empty, (it & 1) ^ 1, abort_flag, p.status, 8)) { ok = false; break; }
      for (int y = lo; y <= hi && ok; ++y, ++n) {
        const int st = n % W_NST, st_next = (n + 1) % W_NST;
        const bool more = y < hi;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          if (!mbar_wait(&bars->p_full[hf], n & 1, abort_flag, p.status, 5)) { ok = false; break; }
          tc_fence_after();
          accumulate(st, hf, (y == lo && hf == 0) ? 0u : 1u);
          if (hf == 1) tc_commit_p(leader, &bars->y_empty[st]);
          if (more) {
            if (hf == 0) {
              if (!mbar_wait(&bars->y_full[st_next], ((n + 1) / W_NST) & 1, abort_flag, p.status, 4)) { ok = false; break; }
              tc_fence_after();
            }
            scores(st_next, hf);
          }
        }
        if (ok && y == hi) { tc_commit_p(leader, &bars->acc_full); tc_commit_p(leader, &bars->x_empty); }
      }
    }
  } else {
    // ------------------------------------------------------------------ P / dZ rebuild and epilogue: thread = TMEM lane
    const int grp = warp >> 2, quarter = warp & 3;                    // which 32 columns; which 32 TMEM lanes
    const int half = grp >> 1;                                        // the 64-column half whose barriers this warpgroup uses
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_t = tmem_base + lane_off + 32 * grp, dp_t = s_t + 128;        // this thread's 32 S and 32 dP columns
    const uint32_t a0_t = tmem_base + lane_off + 256 + 32 * grp, a1_t = a0_t + 128;    // and its 32 output columns of each accumulator
    const float c2 = p.scale_log2;
    uint32_t n = 0, it = 0;
    bool ok = true;
    for (int item; (item = walk.at((int)it)) >= 0 && ok; ++it) {
      const int blk = item % nblk, bh = item / nblk, h = bh % p.H, b = bh / p.H;
      const int* doc_row = p.doc_start ? p.doc_start + b * p.doc_sb : nullptr;
      int lo, hi;
      bwd_range<MODE>(blk, nblk, T, p.window, p.window_blocks, doc_row, lo, hi);
      const int64_t rowbase = ((int64_t)b * p.H + h) * T;
      const int xr = blk * WB + row;                                  // this lane's key (MODE 0) or query (MODE 1)
      float my_lse = 0.f, my_delta = 0.f;
      int my_doc = 0;
      if (MODE == 1 && xr < T) {
        my_lse = p.lse2[rowbase + xr]; my_delta = p.delta[rowbase + xr];
        my_doc = doc_row ? min(doc_row[xr], xr) : 0;
      }
      for (int y = lo; y <= hi; ++y, ++n) {
        float* cf = col_f + (n & 1) * 3 * WB;
        if (MODE == 0) {                                              // the streamed queries' scalars, shared by all lanes
          if (grp == 0) {
            const int q = y * WB + row;
            cf[row] = q < T ? p.lse2[rowbase + q] : 0.f;
            cf[WB + row] = q < T ? p.delta[rowbase + q] : 0.f;
            reinterpret_cast<int*>(cf)[2 * WB + row] = (doc_row && q < T) ? min(doc_row[q], q) : 0;
          }
          // the eight warps leave together: a warp that gave up still comes here, and everybody learns of it
          if (named_bar_or(1, BWD_WORKERS, !ok)) { ok = false; break; }
        }
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[half], n & 1, abort_flag, p.status, 6));
        if (!ok) { if (MODE == 0) continue; else break; }
        tc_fence_after();
        const int y0 = y * WB;
        // is every (lane, column) pair of this tile pair visible?
        bool full;
        if (MODE == 0) {
          full = (blk * WB + WB - 1 <= y0) && (y0 + WB - 1 < T) && (p.window_blocks > 0 || p.window <= 0 || y0 + WB - 1 - blk * WB < p.window) &&
                 (!doc_row || doc_row[min(y0 + WB - 1, T - 1)] <= blk * WB);
        } else {
          full = (y0 + WB - 1 <= blk * WB) && (p.window_blocks > 0 || p.window <= 0 || blk * WB + WB - 1 - y0 < p.window) &&
                 (!doc_row || doc_row[min(blk * WB + WB - 1, T - 1)] <= y0);
        }
        {                                                             // the results go back over the first 16 of the 32 columns
          uint32_t rs[32], rd[32];
          tmem_ld32(s_t, rs);
          tmem_ld32(dp_t, rd);
          tc_wait_ld();
          uint32_t pp[16], pz[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const int col0 = 32 * grp + i;
            float lse4[4], dl4[4];
            int doc4[4] = {0, 0, 0, 0};
            if (MODE == 0) {                                          // four columns' scalars per shared-memory load
              *reinterpret_cast<float4*>(lse4) = *reinterpret_cast<const float4*>(cf + col0);
              *reinterpret_cast<float4*>(dl4) = *reinterpret_cast<const float4*>(cf + WB + col0);
              if (!full) *reinterpret_cast<int4*>(doc4) = *reinterpret_cast<const int4*>(reinterpret_cast<const int*>(cf) + 2 * WB + col0);
            }
            float pv[4], zv[4];
            // two columns per packed instruction: x = S c2 - lse, then dZ = P (dP - delta)
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
              const float l0 = MODE == 0 ? lse4[e] : my_lse, l1 = MODE == 0 ? lse4[e + 1] : my_lse;
              const float d0 = MODE == 0 ? dl4[e] : my_delta, d1 = MODE == 0 ? dl4[e + 1] : my_delta;
              float x0, x1;
              unpack2f(ffma2(pack2f(__uint_as_float(rs[i + e]), __uint_as_float(rs[i + e + 1])), pack2f(c2, c2), pack2f(-l0, -l1)), x0, x1);
              float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              if (!full) {
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                  const int col = col0 + e + u;
                  bool vis;
                  if (MODE == 0) {
                    const int q = y0 + col, k = xr;
                    vis = (k <= q) && (q < T) && (p.window_blocks > 0 || p.window <= 0 || q - k < p.window) && (k >= doc4[e + u]);
                  } else {
                    const int q = xr, k = y0 + col;
                    vis = (k <= q) && (p.window_blocks > 0 || p.window <= 0 || q - k < p.window) && (k >= my_doc);
                  }
                  if (!vis) { if (u == 0) p0 = 0.f; else p1 = 0.f; }
                }
              }
              pv[e] = p0; pv[e + 1] = p1;
              unpack2f(fmul2(pack2f(p0, p1), fadd2(pack2f(__uint_as_float(rd[i + e]), __uint_as_float(rd[i + e + 1])), pack2f(-d0, -d1))),
                       zv[e], zv[e + 1]);
            }
            pp[i >> 1] = pack_bf16(pv[0], pv[1]); pp[(i >> 1) + 1] = pack_bf16(pv[2], pv[3]);
            pz[i >> 1] = pack_bf16(zv[0], zv[1]); pz[(i >> 1) + 1] = pack_bf16(zv[2], zv[3]);
          }
          if (MODE == 0) tmem_st16(s_t, pp);
          tmem_st16(dp_t, pz);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&bars->p_full[half]);
      }
      // ---- epilogue: the item's accumulators -> global rows (thread = row; 256 contiguous bytes each)
      if (ok) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_full, it & 1, abort_flag, p.status, 7));
      }
      if (ok) {
        tc_fence_after();
#pragma unroll 1
        for (int which = (MODE == 0 ? 0 : 1); which < 2; ++which) {
          __nv_bfloat16* dst = (which == 0 ? p.d0 : p.d1) + (((int64_t)b * T + xr) * p.H + h) * DAISY_HEAD_DIM + 32 * grp;
          const float sc = which == 0 ? 1.f : p.scale;
          {
            uint32_t r[32];
            tmem_ld32(which == 0 ? a0_t : a1_t, r);
            tc_wait_ld();
            if (xr < T) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 o;
                o.x = pack_bf16(__uint_as_float(r[i]) * sc, __uint_as_float(r[i + 1]) * sc);
                o.y = pack_bf16(__uint_as_float(r[i + 2]) * sc, __uint_as_float(r[i + 3]) * sc);
                o.z = pack_bf16(__uint_as_float(r[i + 4]) * sc, __uint_as_float(r[i + 5]) * sc);
                o.w = pack_bf16(__uint_as_float(r[i + 6]) * sc, __uint_as_float(r[i + 7]) * sc);
                *reinterpret_cast<uint4*>(dst + i) = o;
              }
            }
          }
        }
        // the next item's first accumulating products overwrite what was just read
        tc_fence_before();
      }
      mbar_arrive(&bars->acc_empty);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 17) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ---------------------------------------------------------------------------------------------
// delta[b,h,t] = sum_d dO[b,t,h,d] O[b,t,h,d]: eight lanes per 256-byte row.
struct DeltaParams {
  const __nv_bfloat16 *o, *d_o;
  int64_t o_sb, o_st, o_sh, g_sb, g_st, g_sh;
  float* delta;
  int B, T, H;
};

__global__ void __launch_bounds__(256) swa_bwd_delta_kernel(const DeltaParams p) {
  const int64_t rows = (int64_t)p.B * p.T * p.H;
  const int64_t r = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 3;
  const int sub = threadIdx.x & 7;
  const int64_t rc = r < rows ? r : rows - 1;
  const int h = (int)(rc % p.H);
  const int64_t bt = rc / p.H;
  const int t = (int)(bt % p.T), b = (int)(bt / p.T);
  const __nv_bfloat16* po = p.o + b * p.o_sb + t * p.o_st + h * p.o_sh + 16 * sub;
  const __nv_bfloat16* pg = p.d_o + b * p.g_sb + t * p.g_st + h * p.g_sh + 16 * sub;
  float acc = 0.f;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    float a[8], g[8];
    unpack8(ld_stream16(po + 8 * u), a);
    unpack8(ld_stream16(pg + 8 * u), g);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc = fmaf(a[e], g[e], acc);
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  if (sub == 0 && r < rows) p.delta[((int64_t)b * p.H + h) * p.T + t] = acc;
}

// ---------------------------------------------------------------------------------------------
// Backward of the q/k/v preparation y = rope(rms_norm(x)) (no RoPE for v), row-wise:
//     g_n = rope^T(g_y),   xh = x r,  r = rsqrt(mean(x^2) + eps),   g_x = r (g_n - xh mean(g_n xh))
// Eight lanes per row; lane `sub` owns elements [8 sub, 8 sub + 8) and [64 + 8 sub, ...), the two halves RoPE pairs.
struct PrepBwdTensor {
  const __nv_bfloat16* x;        // raw input, logical [B,T,H,D] strides
  int64_t sb, st, sh;
  const __nv_bfloat16* gy;       // gradient of the prepared tensor, [B,T,H,D] contiguous
  __nv_bfloat16* gx;             // gradient of the raw input, [B,T,H,D] contiguous
  int do_norm, do_rope;
};
struct PrepBwdParams {
  PrepBwdTensor t[3];
  const float *cos, *sin;
  int B, T, H;
  float eps;
};

__global__ void __launch_bounds__(256) qkv_prep_bwd_kernel(const PrepBwdParams p) {
  const PrepBwdTensor& ten = p.t[blockIdx.y];
  if (ten.x == nullptr) return;
  const int64_t rows = (int64_t)p.B * p.T * p.H;
  const int64_t r = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 3;
  const int sub = threadIdx.x & 7;
  const int64_t rc = r < rows ? r : rows - 1;
  const int h = (int)(rc % p.H);
  const int64_t bt = rc / p.H;
  const int t = (int)(bt % p.T), b = (int)(bt / p.T);
  const __nv_bfloat16* px = ten.x + b * ten.sb + t * ten.st + h * ten.sh + 8 * sub;
  const __nv_bfloat16* pg = ten.gy + rc * DAISY_HEAD_DIM + 8 * sub;
  float x1[8], x2[8], g1[8], g2[8];
  unpack8(ld_stream16(px), x1); unpack8(ld_stream16(px + 64), x2);
  unpack8(ld_stream16(pg), g1); unpack8(ld_stream16(pg + 64), g2);
  if (ten.do_rope) {                                               // transpose of the rotation
    const float* cr = p.cos + (int64_t)t * 64 + 8 * sub;
    const float* sr = p.sin + (int64_t)t * 64 + 8 * sub;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float c = cr[e], s = sr[e], a = g1[e], b2 = g2[e];
      g1[e] = a * c - b2 * s;
      g2[e] = a * s + b2 * c;
    }
  }
  if (ten.do_norm) {
    float ss = 0.f, gd = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) { ss += x1[e] * x1[e] + x2[e] * x2[e]; gd += g1[e] * x1[e] + g2[e] * x2[e]; }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) { ss += __shfl_xor_sync(0xffffffffu, ss, o); gd += __shfl_xor_sync(0xffffffffu, gd, o); }
    const float rr = rsqrtf(ss * (1.0f / DAISY_HEAD_DIM) + p.eps);
    const float m = gd * rr * rr * (1.0f / DAISY_HEAD_DIM);        // mean(g_n xh) r = sum(g_n x) r^2 / D
#pragma unroll
    for (int e = 0; e < 8; ++e) { g1[e] = rr * (g1[e] - x1[e] * m); g2[e] = rr * (g2[e] - x2[e] * m); }
  }
  if (r < rows) {
    __nv_bfloat16* dst = ten.gx + rc * DAISY_HEAD_DIM + 8 * sub;
    *reinterpret_cast<uint4*>(dst) = pack8(g1);
    *reinterpret_cast<uint4*>(dst + 64) = pack8(g2);
  }
}

}  // namespace daisy

using namespace daisy;

static int bwd_smem_attr() {
  static bool done[daisy_host::MAX_DEVICES] = {};
  const int dev = daisy_host::device_slot();
  if (dev < 0) return DAISY_ENODEV;
  if (done[dev]) return DAISY_OK;
  if (cudaFuncSetAttribute(swa_bwd_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess) return DAISY_ECUDA;
  if (cudaFuncSetAttribute(swa_bwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess) return DAISY_ECUDA;
  done[dev] = true;
  return DAISY_OK;
}

extern "C" size_t daisy_b200_swa_attend_bwd_workspace_bytes(int B, int T, int H) {
  if (B <= 0 || T <= 0 || H <= 0) return 0;
  return (size_t)B * T * H * sizeof(float);                        // delta
}

extern "C" int daisy_b200_swa_attend_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                         int64_t q_sb, int64_t q_st, int64_t q_sh,
                                         int64_t k_sb, int64_t k_st, int64_t k_sh,
                                         int64_t v_sb, int64_t v_st, int64_t v_sh,
                                         int64_t o_sb, int64_t o_st, int64_t o_sh,
                                         int64_t g_sb, int64_t g_st, int64_t g_sh,
                                         const float* lse2, void* dq, void* dk, void* dv,
                                         int B, int T, int H, int D, int window, float scale,
                                         const int32_t* doc_start, int64_t doc_sb, unsigned flags,
                                         void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
  if (!q || !k || !v || !o || !d_o || !lse2 || !dq || !dk || !dv || !workspace || B <= 0 || T <= 0 || H <= 0 || !(scale > 0.f)) return DAISY_EINVAL;
  if (D != DAISY_HEAD_DIM) return DAISY_EUNSUPPORTED;
  if (flags & ~DAISY_WINDOW_BLOCKS) return DAISY_EINVAL;
  if (workspace_bytes < daisy_b200_swa_attend_bwd_workspace_bytes(B, T, H)) return DAISY_EWORKSPACE;
  const void* ptrs[] = {q, k, v, o, d_o, dq, dk, dv, workspace};
  for (const void* x : ptrs) if (!daisy_aligned16(x)) return DAISY_EALIGN;
  if ((q_sb | q_st | q_sh | k_sb | k_st | k_sh | v_sb | v_st | v_sh | o_sb | o_st | o_sh | g_sb | g_st | g_sh) & 7) return DAISY_EALIGN;
  if (q_st <= 0 || k_st <= 0 || v_st <= 0 || g_st <= 0 || o_st <= 0) return DAISY_EINVAL;
  if ((H > 1 && (q_sh <= 0 || k_sh <= 0 || v_sh <= 0 || g_sh <= 0 || o_sh <= 0)) || (B > 1 && (q_sb <= 0 || k_sb <= 0 || v_sb <= 0 || g_sb <= 0 || o_sb <= 0)))
    return DAISY_EINVAL;
  if (doc_start && (doc_sb < 0 || (reinterpret_cast<uintptr_t>(doc_start) & 3))) return DAISY_EINVAL;
  if ((int64_t)B * T * H >= (int64_t)1 << 31) return DAISY_EUNSUPPORTED;
  if (const int arc = bwd_smem_attr(); arc != DAISY_OK) { (void)cudaGetLastError(); return arc; }
  cudaStream_t st = (cudaStream_t)stream;
  float* delta = (float*)workspace;
  {
    DeltaParams dp{(const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, o_sb, o_st, o_sh, g_sb, g_st, g_sh, delta, B, T, H};
    const int64_t rows = (int64_t)B * T * H;
    swa_bwd_delta_kernel<<<(unsigned)((rows * 8 + 255) / 256), 256, 0, st>>>(dp);
    DAISY_CHECK_LAUNCH();
  }
  CUtensorMap tq, tk, tv, tg;
  int rc;
  auto sb = [](int64_t s, int n) { return (uint64_t)(n == 1 ? 16 : s * 2); };
  if ((rc = daisy_host::make_tmap_bf16_dthb(&tq, q, D, T, H, B, q_st * 2, sb(q_sh, H), sb(q_sb, B), 64, WB)) != DAISY_OK) return rc;
  if ((rc = daisy_host::make_tmap_bf16_dthb(&tk, k, D, T, H, B, k_st * 2, sb(k_sh, H), sb(k_sb, B), 64, WB)) != DAISY_OK) return rc;
  if ((rc = daisy_host::make_tmap_bf16_dthb(&tv, v, D, T, H, B, v_st * 2, sb(v_sh, H), sb(v_sb, B), 64, WB)) != DAISY_OK) return rc;
  if ((rc = daisy_host::make_tmap_bf16_dthb(&tg, d_o, D, T, H, B, g_st * 2, sb(g_sh, H), sb(g_sb, B), 64, WB)) != DAISY_OK) return rc;
  BwdParams p;
  p.lse2 = lse2; p.delta = delta; p.doc_start = doc_start; p.doc_sb = doc_sb;
  p.T = T; p.H = H; p.B = B;
  const bool in_blocks = (flags & DAISY_WINDOW_BLOCKS) != 0;
  p.window = in_blocks ? 0 : window;
  p.window_blocks = (in_blocks && window > 0) ? window : 0;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_word;
  const int sms = daisy_host::sm_count_cached();
  if (sms <= 0) return DAISY_ENODEV;
  const int64_t items = (int64_t)((T + WB - 1) / WB) * H * B;
  const unsigned grid = (unsigned)(items < sms ? items : sms);
  p.d0 = (__nv_bfloat16*)dv; p.d1 = (__nv_bfloat16*)dk;
  swa_bwd_kernel<0><<<grid, BWD_THREADS, BWD_SMEM, st>>>(tq, tk, tv, tg, p);
  DAISY_CHECK_LAUNCH();
  p.d0 = nullptr; p.d1 = (__nv_bfloat16*)dq;
  swa_bwd_kernel<1><<<grid, BWD_THREADS, BWD_SMEM, st>>>(tq, tk, tv, tg, p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}

extern "C" int daisy_b200_qkv_prep_bwd(const void* q, const void* k, const void* v,
                                       int64_t q_sb, int64_t q_st, int64_t q_sh,
                                       int64_t k_sb, int64_t k_st, int64_t k_sh,
                                       int64_t v_sb, int64_t v_st, int64_t v_sh,
                                       const float* cos, const float* sin,
                                       const void* dq_p, const void* dk_p, const void* dv_p,
                                       void* dq, void* dk, void* dv,
                                       int B, int T, int H, int D, float eps, unsigned flags, void* stream) {
  if (B <= 0 || T <= 0 || H <= 0) return DAISY_EINVAL;
  if (D != DAISY_HEAD_DIM) return DAISY_EUNSUPPORTED;
  if (flags & ~DAISY_QKV_DEFAULT) return DAISY_EINVAL;
  if ((q == nullptr) != (dq == nullptr) || (q == nullptr) != (dq_p == nullptr) || (k == nullptr) != (dk == nullptr) ||
      (k == nullptr) != (dk_p == nullptr) || (v == nullptr) != (dv == nullptr) || (v == nullptr) != (dv_p == nullptr)) return DAISY_EINVAL;
  if (!q && !k && !v) return DAISY_EINVAL;
  if ((flags & DAISY_ROPE) && (!cos || !sin)) return DAISY_EINVAL;
  const void* ptrs[] = {q, k, v, dq_p, dk_p, dv_p, dq, dk, dv};
  for (const void* x : ptrs) if (x && !daisy_aligned16(x)) return DAISY_EALIGN;
  if ((q_sb | q_st | q_sh | k_sb | k_st | k_sh | v_sb | v_st | v_sh) & 7) return DAISY_EALIGN;
  if ((int64_t)B * T * H >= (int64_t)1 << 31) return DAISY_EUNSUPPORTED;
  PrepBwdParams p;
  p.t[0] = {(const __nv_bfloat16*)q, q_sb, q_st, q_sh, (const __nv_bfloat16*)dq_p, (__nv_bfloat16*)dq, (flags & DAISY_NORM_Q) ? 1 : 0, (flags & DAISY_ROPE) ? 1 : 0};
  p.t[1] = {(const __nv_bfloat16*)k, k_sb, k_st, k_sh, (const __nv_bfloat16*)dk_p, (__nv_bfloat16*)dk, (flags & DAISY_NORM_K) ? 1 : 0, (flags & DAISY_ROPE) ? 1 : 0};
  p.t[2] = {(const __nv_bfloat16*)v, v_sb, v_st, v_sh, (const __nv_bfloat16*)dv_p, (__nv_bfloat16*)dv, (flags & DAISY_NORM_V) ? 1 : 0, 0};
  p.cos = cos; p.sin = sin; p.B = B; p.T = T; p.H = H; p.eps = eps;
  const int64_t rows = (int64_t)B * T * H;
  dim3 grid((unsigned)((rows * 8 + 255) / 256), 3, 1);
  qkv_prep_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}
