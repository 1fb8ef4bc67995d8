// Sliding-window causal softmax attention, prefill form, on tcgen05 tensor cores.
//
// One CTA owns 256 consecutive query rows of one (batch, head): two 128-row streams that share
// every K/V tile.  Roles, general form (NSPLIT = 1, 320 threads):
//   warps 0-3   softmax of stream 0 (thread = query row = TMEM lane)
//   warps 4-7   softmax of stream 1
//   warp  8     TMA producer: Q tiles one item ahead, then K_j, V_j tiles into a ring of 32 KB buffers
//   warp  9     MMA issuer (one elected lane): S_s = Q_s K_j^T (smem x smem), O_s += P_s V_j (TMEM x smem)
// Bounded-logit form (NSPLIT = 2, 576 threads): warps 0-15 are two softmax warpgroups per stream, 64 key
// columns each; warp 16 producer, warp 17 issuer (see the comment above the kernel).
// TMEM (512 columns): S_0 [0,128) S_1 [128,256) O_0 [256,384) O_1 [384,512), fp32.  P_s (bf16,
// two keys per column) overwrites columns of S_s once they have been read.
// General form: softmax is online in the exp2 domain with a lazily refreshed reference maximum: the
// accumulator is rescaled only when the running maximum has grown by more than 8 (a factor 256), so most
// iterations touch O only through the tensor core.  KV tiles wholly outside the window, or wholly before
// the document of the block's first query, are never loaded; the partially visible tiles (causal diagonal,
// trailing window edge, a document boundary) go through one element-wise predicate.
// All mbarrier waits are bounded; a wait that runs out raises an abort flag that every role polls,
// the CTA drains to its teardown, frees TMEM and reports DAISY_ETIMEOUT through the status word.
#include "common.cuh"

namespace daisy {

constexpr int BM = 128;
constexpr int BN = 128;
#ifndef PREFILL_NSTAGE
#define PREFILL_NSTAGE 3
#endif
#ifndef PREFILL_NQBUF
#define PREFILL_NQBUF 2
#endif
constexpr int NSTAGE = PREFILL_NSTAGE; // K/V ring stages (32 KB each)
constexpr int NQBUF = PREFILL_NQBUF;   // Q double buffer: the next item's Q lands while this item computes
constexpr int TILE_BYTES = BM * DAISY_HEAD_DIM * 2;      // 32768
constexpr int HALF_BYTES = TILE_BYTES / 2;               // one [128 x 64] swizzled box
constexpr int PREFILL_THREADS = 320;          // one softmax warpgroup per stream
constexpr int PREFILL_THREADS_SPLIT = 576;    // two softmax warpgroups per stream (64 key columns each)
constexpr int SMEM_TILES = (2 * NQBUF + NSTAGE) * TILE_BYTES;
constexpr int PREFILL_SMEM = 1024 + SMEM_TILES + 256 + 2 * 128 * 4;   // alignment slack, tiles, barriers, row-sum exchange
static_assert(PREFILL_SMEM <= 232448, "over the 227 KB a CTA may use");
constexpr float NEG_BIG = -1.0e30f;
#ifndef POLY_MASK
#define POLY_MASK 4                        // pairs with (i & POLY_MASK) == POLY_MASK go to the polynomial: 4 = one in four
#endif
#ifndef POLY_HALF
#define POLY_HALF 0                      // 1: every second pair of exponentials by polynomial; 0: one pair in four
#endif

struct PrefillParams {
  __nv_bfloat16* out;
  int64_t o_sb, o_st, o_sh;
  int T, H, B, window;
  int window_blocks;       // > 0: block-granular window (key tile >= query tile - window_blocks + 1), window = 0
  float scale_log2;
  int* status;
  // document mask: doc_start[b * doc_sb + t] = first key position of the document token t belongs to (null: one
  // document).  Non-decreasing in t.
  const int* doc_start;
  int64_t doc_sb;
  // raw-Q mode: the kernel RMS-normalises and rotates the Q tile in shared memory before the first product
  const float* cos;
  const float* sin;
  float eps;
  int q_norm, q_rope;
  // optional: log2 of each row's softmax denominator in the kernel's exp2 domain, [B,H,T] float32:
  // P[q,k] = 2^(logit * log2(e) - lse2[q]).  What the backward pass rebuilds P from.
  float* lse2;
};

struct PrefillBarriers {
  uint64_t q_full[2][NQBUF];
  uint64_t q_empty[2][NQBUF];
  uint64_t q_ready[2][NQBUF];
  uint64_t kv_full[NSTAGE];
  uint64_t kv_empty[NSTAGE];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t o_full[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ bool key_visible(int q, int k, int window) {
  return (k <= q) && (window <= 0 || k > q - window);
}

// Geometry of one work item: 256 query rows (two streams) of one (batch, head).
struct ItemGeom {
  int b, h;
  int q0[2], jlo_s[2], jhi_s[2];
  bool valid[2];
  int jlo, jhi;
};
__device__ __forceinline__ ItemGeom item_geom(int item, int nq, int H, int T, int window,
                                              const int* doc_start = nullptr, int64_t doc_sb = 0, int window_blocks = 0) {
  ItemGeom g;
  const int qp = item % nq, bh = item / nq;
  g.h = bh % H; g.b = bh / H;
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    g.q0[s] = (qp * 2 + s) * BM;
    g.valid[s] = g.q0[s] < T;
    int klo = window > 0 ? max(0, g.q0[s] - window + 1) : 0;
    // block-granular window of the training form: whole key tiles, the nearest window_blocks of them
    if (window_blocks > 0) klo = max(0, g.q0[s] / BM - window_blocks + 1) * BN;
    // keys before the document of the stream's FIRST row are invisible to every row of the stream
    // (clamped to the row itself: a malformed table must not leave a stream without tiles)
    if (doc_start && g.valid[s]) klo = max(klo, min(doc_start[g.b * doc_sb + g.q0[s]], g.q0[s]));
    g.jlo_s[s] = g.valid[s] ? klo / BN : 1;
    g.jhi_s[s] = g.valid[s] ? min(g.q0[s] + BM - 1, T - 1) / BN : 0;
  }
  g.jlo = g.jlo_s[0];
  g.jhi = g.valid[1] ? g.jhi_s[1] : g.jhi_s[0];
  return g;
}

// Raw-Q mode: RMS norm over the row and half-rotation RoPE at position `qrow`, in place in the 128-byte-
// swizzled Q tile (thread = row; chunk c of row r sits at r*128 + ((c ^ r) & 7)*16 of box c >> 3).  Called by
// the 128 threads that own the rows of stream s, between two softmax tiles; signals q_ready.
__device__ __forceinline__ bool prepare_q_tile(PrefillBarriers* bars, uint8_t* q_tiles, int s, int row, uint32_t& n_qs,
                                               int qrow, const PrefillParams& p, volatile int* abort_flag) {
  const uint32_t qb = n_qs % NQBUF;
  if (!__all_sync(0xffffffffu, mbar_wait(&bars->q_full[s][qb], (n_qs / NQBUF) & 1, abort_flag, p.status, 12))) return false;
  ++n_qs;
  uint8_t* qt = q_tiles + (qb * 2 + s) * TILE_BYTES + row * 128;
  const int sw = row & 7;
  // two passes over the row in shared memory (sum of squares, then rotate) keep the live registers few
  float ss = 0.f;
#pragma unroll 4
  for (int c = 0; c < 16; ++c) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(qt + (c >> 3) * HALF_BYTES + (((c & 7) ^ sw) << 4)), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
  }
  const float rs = p.q_norm ? rsqrtf(ss * (1.0f / DAISY_HEAD_DIM) + p.eps) : 1.f;
  const int pos = min(qrow, p.T - 1);
  const float* cr = p.cos + (int64_t)pos * 64;
  const float* sr = p.sin + (int64_t)pos * 64;
#pragma unroll 2
  for (int c = 0; c < 8; ++c) {
    float x1[8], x2[8];
    unpack8(*reinterpret_cast<const uint4*>(qt + (((c & 7) ^ sw) << 4)), x1);
    unpack8(*reinterpret_cast<const uint4*>(qt + HALF_BYTES + (((c & 7) ^ sw) << 4)), x2);
    float cs[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f}, sn[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (p.q_rope) {
      const float4 c0 = *reinterpret_cast<const float4*>(cr + 8 * c), c1 = *reinterpret_cast<const float4*>(cr + 8 * c + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sr + 8 * c), s1 = *reinterpret_cast<const float4*>(sr + 8 * c + 4);
      cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
      sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
    float y1[8], y2[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float a = x1[e] * rs, b2 = x2[e] * rs;
      y1[e] = a * cs[e] + b2 * sn[e];
      y2[e] = b2 * cs[e] - a * sn[e];
    }
    *reinterpret_cast<uint4*>(qt + (((c & 7) ^ sw) << 4)) = pack8(y1);
    *reinterpret_cast<uint4*>(qt + HALF_BYTES + (((c & 7) ^ sw) << 4)) = pack8(y2);
  }
  fence_proxy_async();                                              // generic-proxy writes -> visible to the MMA's reads
  mbar_arrive(&bars->q_ready[s][qb]);
  return true;
}

// Persistent schedule: item = (batch*H + head) * nq + q-pair, walked in the balanced order of BalancedWalk (all
// q-pairs that see a full window first, (batch, head)-major; then the causal-ramp q-pairs, longest first).
__device__ __forceinline__ BalancedWalk prefill_walk(int nq, int BH, int window, int window_blocks) {
  const int span = window > 0 ? window : (window_blocks > 0 ? window_blocks * BN : 0);       // keys a full row sees
  return BalancedWalk(nq, BH, span > 0 ? (span + 2 * BM - 1) / (2 * BM) : nq, false);
}

// Barrier phases are kept as
// running counters per role, so the K/V ring, the Q buffers and the TMEM accumulators carry over from
// one item to the next: the producer prefetches the next item's Q and K while the softmax warps are
// still writing the previous item's output.
//
// NSPLIT = 2 (bounded logits only): each stream's S tile is shared by two warpgroups, 64 key columns each, so a
// tile's exponentials take half as long on the critical path  Q K^T -> softmax -> P V  of its stream.  With
// |logit * log2 e| <= 60 no reference maximum is needed at all (2^x stays far inside fp32 and bf16 range), so the
// two halves of a row never talk to each other until the epilogue adds their partial row sums.  Each half writes
// its P over the first 32 columns of its OWN 64 S columns (P_s = two 32-column pieces at S_s + 0 and S_s + 64).
template <bool QRAW, bool BOUNDED, int NSPLIT>
__global__ void __launch_bounds__(32 * (8 * NSPLIT + 2), 1)
swa_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_tiles = smem;
  uint8_t* kv_tiles = smem + 2 * NQBUF * TILE_BYTES;
  PrefillBarriers* bars = reinterpret_cast<PrefillBarriers*>(smem + SMEM_TILES);
  volatile int* abort_flag = &bars->abort_flag;

  static_assert(NSPLIT == 1 || (NSPLIT == 2 && BOUNDED), "the split softmax needs bounded logits");
  constexpr int TMA_WARP = 8 * NSPLIT, MMA_WARP = 8 * NSPLIT + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = p.T, window = p.window;
  const int nq = (T + 2 * BM - 1) / (2 * BM);
  const BalancedWalk walk = prefill_walk(nq, p.H * p.B, window, p.window_blocks);

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      for (int qb = 0; qb < NQBUF; ++qb) { mbar_init(&bars->q_full[s][qb], 1); mbar_init(&bars->q_empty[s][qb], 1); mbar_init(&bars->q_ready[s][qb], 128); }
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->p_full[s], 128 * NSPLIT);
      mbar_init(&bars->o_full[s], 1);
    }
    for (int i = 0; i < NSTAGE; ++i) { mbar_init(&bars->kv_full[i], 1); mbar_init(&bars->kv_empty[i], 1); }
    bars->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == TMA_WARP) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v);
      int n = 0;                         // K/V tiles loaded so far (ring position)
      uint32_t qn[2] = {0, 0};           // Q tiles loaded so far per stream
      bool ok = true;
      // Q tiles run one item ahead of the K/V stream (double buffer), so the softmax warps can prepare the
      // next item's Q while the current item is still computing.
      auto load_q = [&](int it_item) {
        const ItemGeom gq = item_geom(it_item, nq, p.H, T, window, p.doc_start, p.doc_sb, p.window_blocks);
        for (int s = 0; s < 2 && ok; ++s) {
          if (!gq.valid[s]) continue;
          const int qb = qn[s] % NQBUF;
          if (!mbar_wait(&bars->q_empty[s][qb], ((qn[s] / NQBUF) & 1) ^ 1, abort_flag, p.status, 9)) { ok = false; break; }
          ++qn[s];
          uint8_t* qdst = q_tiles + (qb * 2 + s) * TILE_BYTES;
          mbar_expect_tx(&bars->q_full[s][qb], TILE_BYTES);
          tma_load_4d(qdst, &tm_q, &bars->q_full[s][qb], 0, gq.q0[s], gq.h, gq.b);
          tma_load_4d(qdst + HALF_BYTES, &tm_q, &bars->q_full[s][qb], 64, gq.q0[s], gq.h, gq.b);
        }
      };
      if (walk.at(0) >= 0) load_q(walk.at(0));
      for (int rd = 0, item; (item = walk.at(rd)) >= 0 && ok; ++rd) {
        const ItemGeom g = item_geom(item, nq, p.H, T, window, p.doc_start, p.doc_sb, p.window_blocks);
        for (int j = g.jlo; j <= g.jhi && ok; ++j) {
          for (int kv = 0; kv < 2; ++kv, ++n) {
            const int stage = n % NSTAGE;
            const uint32_t ph = (n / NSTAGE) & 1;
            if (!mbar_wait(&bars->kv_empty[stage], ph ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
            uint8_t* dst = kv_tiles + stage * TILE_BYTES;
            const CUtensorMap* tm = kv ? &tm_v : &tm_k;
            mbar_expect_tx(&bars->kv_full[stage], TILE_BYTES);
            tma_load_4d(dst, tm, &bars->kv_full[stage], 0, j * BN, g.h, g.b);
            tma_load_4d(dst + HALF_BYTES, tm, &bars->kv_full[stage], 64, j * BN, g.h, g.b);
          }
          // next item's Q: after this item's first K/V tiles are on their way (its buffer was released when the
          // previous item issued its last Q K^T, which the ring has long passed by now)
          if (j == (NQBUF > 1 ? g.jlo : g.jhi) && walk.at(rd + 1) >= 0) load_q(walk.at(rd + 1));
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer (one thread)
    // Issue order per K/V tile j:  PV_0(j-1) QK_0(j) PV_1(j-1) QK_1(j).  While softmax 0 works on S_0(j) the
    // tensor core runs stream 1's pair and vice versa.  (Splitting the issue over one thread per stream was
    // measured slower: the two streams drift into phase and compete for the same softmax slots.)
    // The whole warp walks the loop (uniform control flow and descriptor arithmetic); the tcgen05 instructions
    // themselves are predicated on one elected lane.
    {
      const uint32_t leader = elect_one() ? 1u : 0u;
      constexpr uint32_t idesc_qk = umma_idesc_bf16(BM, BN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(BM, DAISY_HEAD_DIM, 0, 1);
      // descriptor halves: low = start address >> 4 | LBO field, high = SBO | version | swizzle (constant)
      const uint64_t qd = umma_desc_sw128(smem_u32(q_tiles), 16, 1024);        // K-major operands of Q K^T
      const uint64_t kd = umma_desc_sw128(smem_u32(kv_tiles), 16, 1024);
      const uint64_t vd = umma_desc_sw128(smem_u32(kv_tiles), HALF_BYTES, 1024);   // MN-major V of P V
      const uint32_t q_lo0 = (uint32_t)qd, k_lo0 = (uint32_t)kd, qk_hi = (uint32_t)(qd >> 32);
      const uint32_t v_lo0 = (uint32_t)vd, v_hi = (uint32_t)(vd >> 32);
      int n_base = 0;                    // ring position of this item's first K tile
      uint32_t n_pv[2] = {0, 0};         // P tiles consumed so far per stream (phase of p_full)
      uint32_t n_q[2] = {0, 0};          // Q tiles consumed so far per stream (phase of q_full)
      bool ok = true;
      for (int rd = 0, item; (item = walk.at(rd)) >= 0 && ok; ++rd) {
        const ItemGeom g = item_geom(item, nq, p.H, T, window, p.doc_start, p.doc_sb, p.window_blocks);
        for (int j = g.jlo; j <= g.jhi + 1 && ok; ++j) {
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            if (!g.valid[s]) continue;
            const uint32_t s_tmem = tmem_base + s * 128;
            const uint32_t o_tmem = tmem_base + 256 + s * 128;
            // O_s += P_s(j-1) V_{j-1}
            if (j - 1 >= g.jlo_s[s] && j - 1 <= g.jhi_s[s]) {
              const int n = n_base + 2 * (j - 1 - g.jlo) + 1;
              const int stage = n % NSTAGE;
              if (!mbar_wait(&bars->p_full[s], n_pv[s] & 1, abort_flag, p.status, 2)) { ok = false; break; }
              ++n_pv[s];
              const bool v_seen = (s == 1) && g.valid[0] && (j - 1 >= g.jlo_s[0]) && (j - 1 <= g.jhi_s[0]);   // stream 0 waited on V_{j-1}
              if (!v_seen && !mbar_wait(&bars->kv_full[stage], (n / NSTAGE) & 1, abort_flag, p.status, 3)) { ok = false; break; }
              tc_fence_after();
              const uint32_t v_lo = v_lo0 + stage * (TILE_BYTES >> 4);
              const bool first = (j - 1 == g.jlo_s[s]);             // first PV of the item overwrites O_s
              umma_ts_lh_p(leader, o_tmem, s_tmem, v_lo, v_hi, idesc_pv, first ? 0u : 1u);
#pragma unroll
              for (int k = 1; k < BN / 16; ++k)   // P columns: contiguous, or (split softmax) 32 at S_s and 32 at S_s + 64
                umma_ts_lh_p(leader, o_tmem, s_tmem + (NSPLIT == 2 ? (k & 3) * 8 + (k >> 2) * 64 : k * 8), v_lo + k * (2048 >> 4), v_hi, idesc_pv, 1u);
              const bool other_uses = (s == 0) && g.valid[1] && (j - 1 >= g.jlo_s[1]) && (j - 1 <= g.jhi_s[1]);
              if (!other_uses) tc_commit_p(leader, &bars->kv_empty[stage]);
              if (j - 1 == g.jhi_s[s]) tc_commit_p(leader, &bars->o_full[s]);
            }
            // S_s = Q_s K_j^T
            if (j >= g.jlo_s[s] && j <= g.jhi_s[s]) {
              const int n = n_base + 2 * (j - g.jlo);
              const int stage = n % NSTAGE;
              if (j == g.jlo_s[s]) {
                const uint32_t qb = n_q[s] % NQBUF;
                if (!mbar_wait(QRAW ? &bars->q_ready[s][qb] : &bars->q_full[s][qb], (n_q[s] / NQBUF) & 1, abort_flag, p.status, 4)) { ok = false; break; }
                ++n_q[s];
              }
              const bool k_seen = (s == 1) && g.valid[0] && (j >= g.jlo_s[0]) && (j <= g.jhi_s[0]);           // stream 0 waited on K_j
              if (!k_seen && !mbar_wait(&bars->kv_full[stage], (n / NSTAGE) & 1, abort_flag, p.status, 5)) { ok = false; break; }
              tc_fence_after();
              const uint32_t q_buf = (n_q[s] - 1) % NQBUF;              // the buffer this item's Q_s sits in
              const uint32_t q_lo = q_lo0 + (q_buf * 2 + s) * (TILE_BYTES >> 4);
              const uint32_t k_lo = k_lo0 + stage * (TILE_BYTES >> 4);
#pragma unroll
              for (int k = 0; k < DAISY_HEAD_DIM / 16; ++k) {
                const uint32_t off = ((k >> 2) * HALF_BYTES + (k & 3) * 32) >> 4;
                umma_ss_lh_p(leader, s_tmem, q_lo + off, qk_hi, k_lo + off, qk_hi, idesc_qk, k > 0 ? 1u : 0u);
              }
              tc_commit_p(leader, &bars->s_full[s]);
              if (j == g.jhi_s[s]) tc_commit_p(leader, &bars->q_empty[s][q_buf]);     // Q_s may be overwritten by the next item
              const bool other_uses = (s == 0) && g.valid[1] && (j >= g.jlo_s[1]) && (j <= g.jhi_s[1]);
              if (!other_uses) tc_commit_p(leader, &bars->kv_empty[stage]);
            }
          }
        }
        n_base += 2 * (g.jhi - g.jlo + 1);
      }
    }
  } else if constexpr (NSPLIT == 2) {
    // ------------------------------------------------------------------ split softmax + epilogue (bounded logits)
    const int grp = warp >> 2, quarter = warp & 3;
    const int s = grp & 1, half = grp >> 1;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_off + s * 128 + half * 64;          // this thread's 64 S columns; P over the first 32
    const uint32_t o_tmem = tmem_base + lane_off + 256 + s * 128 + half * 64;    // and its 64 output columns in the epilogue
    float* lsum = reinterpret_cast<float*>(smem + SMEM_TILES + 256) + s * 128 + row;   // one exchange slot per row
    const uint64_t c2p = pack2f(p.scale_log2, p.scale_log2);
    uint32_t n_s = 0, n_o = 0, n_qs = 0;
    bool ok = true;
    bool q_prepared = false;                                       // raw-Q mode: the lower half prepares the stream's Q rows
    for (int rd = 0, item; (item = walk.at(rd)) >= 0 && ok; ++rd) {
      const ItemGeom g = item_geom(item, nq, p.H, T, window, p.doc_start, p.doc_sb, p.window_blocks);
      if (!g.valid[s]) continue;
      const int q0 = g.q0[s];
      const int q_row = q0 + row;
      bool next_valid = false;
      int q_row_next = 0;
      if (QRAW && half == 0) {
        // a wait that ran out must not leave the item loop here: the stream's other half still comes to the two
        // named barriers below, which need all 256 threads -- skip the tile loop and the epilogue instead
        if (!q_prepared) ok = prepare_q_tile(bars, q_tiles, s, row, n_qs, q_row, p, abort_flag);
        q_prepared = false;
        const int item_next = walk.at(rd + 1);
        if (item_next >= 0) {
          const ItemGeom gn = item_geom(item_next, nq, p.H, T, window, p.doc_start, p.doc_sb, p.window_blocks);
          next_valid = gn.valid[s];
          q_row_next = gn.q0[s] + row;
        }
      }
      uint64_t sum_a = pack2f(0.f, 0.f), sum_b = sum_a;
      // first visible key of this row's document, and the latest such start among the stream's rows
      const int ds_row = p.doc_start ? min(p.doc_start[g.b * p.doc_sb + min(q_row, T - 1)], q_row) : 0;   // a row always sees itself
      const int ds_max = p.doc_start ? p.doc_start[g.b * p.doc_sb + min(q0 + BM - 1, T - 1)] : 0;
      for (int j = g.jlo_s[s]; ok && j <= g.jhi_s[s]; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[s], n_s & 1, abort_flag, p.status, 6));
        if (!ok) break;
        ++n_s;
        tc_fence_after();
        const int k0 = j * BN + half * 64;                            // key index of this thread's first column
        const bool full_tile = (j * BN + BN - 1 <= q0) && (window <= 0 || j * BN > q0 + BM - 1 - window) && ds_max <= j * BN;
        uint32_t r[64];
        tmem_ld32(s_tmem, r);
        tmem_ld32(s_tmem + 32, r + 32);
        tc_wait_ld();
        if (!full_tile) {
          const int hi = q_row - k0;                                   // column i is visible iff lo < i <= hi
          const int lo = max(window > 0 ? q_row - window - k0 : -1, ds_row - 1 - k0);
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (!(i > lo && i <= hi)) r[i] = 0xff800000u;              // -inf -> weight 0
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const uint64_t xa = fmul2(pack2f(__uint_as_float(r[32 * c + i]), __uint_as_float(r[32 * c + i + 1])), c2p);
            const uint64_t xb = fmul2(pack2f(__uint_as_float(r[32 * c + i + 2]), __uint_as_float(r[32 * c + i + 3])), c2p);
            float x0, x1, p2, p3;
            unpack2f(xa, x0, x1);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            uint64_t pb;
            if (POLY_HALF || (POLY_MASK && (i & POLY_MASK) == POLY_MASK)) {                           // a share of the pairs goes to the FMA pipes
              pb = exp2_poly2(xb);
              unpack2f(pb, p2, p3);
            } else {
              float x2, x3;
              unpack2f(xb, x2, x3);
              p2 = fast_exp2(x2); p3 = fast_exp2(x3);
              pb = pack2f(p2, p3);
            }
            sum_a = fadd2(sum_a, pack2f(p0, p1));
            sum_b = fadd2(sum_b, pb);
            pk[i >> 1] = pack_bf16(p0, p1);
            pk[(i >> 1) + 1] = pack_bf16(p2, p3);
          }
          tmem_st16(s_tmem + 16 * c, pk);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&bars->p_full[s]);
        if (QRAW && half == 0 && next_valid && !q_prepared && j == g.jlo_s[s] + 1) {   // next item's Q, inside this item
          ok = prepare_q_tile(bars, q_tiles, s, row, n_qs, q_row_next, p, abort_flag);
          if (!ok) break;
          q_prepared = true;
        }
      }
      float l;
      {
        float a0, a1, b0, b1;
        unpack2f(sum_a, a0, a1);
        unpack2f(sum_b, b0, b1);
        l = (a0 + a1) + (b0 + b1);
      }
      // the upper half publishes its partial sum, the lower half replaces it by the total (one slot per row)
      if (half == 1) *lsum = l;
      if (s == 0) asm volatile("bar.sync 1, 256;" ::: "memory");       // the 256 threads of this stream
      else        asm volatile("bar.sync 2, 256;" ::: "memory");
      if (half == 0) { l += *lsum; *lsum = l; }
      if (s == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
      else        asm volatile("bar.sync 2, 256;" ::: "memory");
      if (half == 1) l = *lsum;
      if (p.lse2 && half == 0 && q_row < T) p.lse2[((int64_t)g.b * p.H + g.h) * T + q_row] = __log2f(l);   // no reference maximum in this form
      if (ok) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full[s], n_o & 1, abort_flag, p.status, 7));
        ++n_o;
      }
      if (ok) {
        tc_fence_after();
        const float inv = 1.0f / l;
        uint32_t r[64];
        tmem_ld32(o_tmem, r);
        tmem_ld32(o_tmem + 32, r + 32);
        tc_wait_ld();
        // this thread's 64 normalised outputs as eight 16-byte chunks
        uint4 ch[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          ch[c].x = pack_bf16(__uint_as_float(r[8 * c]) * inv, __uint_as_float(r[8 * c + 1]) * inv);
          ch[c].y = pack_bf16(__uint_as_float(r[8 * c + 2]) * inv, __uint_as_float(r[8 * c + 3]) * inv);
          ch[c].z = pack_bf16(__uint_as_float(r[8 * c + 4]) * inv, __uint_as_float(r[8 * c + 5]) * inv);
          ch[c].w = pack_bf16(__uint_as_float(r[8 * c + 6]) * inv, __uint_as_float(r[8 * c + 7]) * inv);
        }
        // 8 x 8 transpose of chunks inside each group of eight lanes (three butterfly stages): afterwards lane l of
        // a group holds chunk l of the group's eight rows, so one store instruction writes four whole 128-byte
        // row segments instead of 32 scattered 16-byte pieces (rows are H*D*2 bytes apart in memory).
#pragma unroll
        for (int m = 4; m >= 1; m >>= 1) {
          const bool up = (lane & m) != 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (i & m) continue;
            const uint4 send = up ? ch[i] : ch[i | m];
            uint4 recv;
            recv.x = __shfl_xor_sync(0xffffffffu, send.x, m);
            recv.y = __shfl_xor_sync(0xffffffffu, send.y, m);
            recv.z = __shfl_xor_sync(0xffffffffu, send.z, m);
            recv.w = __shfl_xor_sync(0xffffffffu, send.w, m);
            if (up) ch[i] = recv; else ch[i | m] = recv;
          }
        }
        {
          const int l8 = lane & 7, row_g = q_row - l8;                   // first row of this lane's group
          __nv_bfloat16* dst = p.out + g.b * p.o_sb + (int64_t)row_g * p.o_st + g.h * p.o_sh + half * 64 + l8 * 8;
#pragma unroll
          for (int jr = 0; jr < 8; ++jr)
            if (row_g + jr < T) *reinterpret_cast<uint4*>(dst + (int64_t)jr * p.o_st) = ch[jr];
        }
        // the next item's first PV overwrites O_s only after every thread's P of that item has been signalled,
        // i.e. after these loads: program order is the guard
        tc_fence_before();
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int s = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_off + s * 128;
    const uint32_t o_tmem = tmem_base + lane_off + 256 + s * 128;
    const float c2 = p.scale_log2;
    uint32_t n_s = 0, n_o = 0, n_qs = 0; // S tiles / O tiles / Q tiles consumed so far (phases of s_full, o_full, q_full)
    bool ok = true;
    uint32_t r[128];
    bool q_prepared = false;
    auto prepare_q = [&](int qrow) -> bool { return prepare_q_tile(bars, q_tiles, s, row, n_qs, qrow, p, abort_flag); };
    for (int rd = 0, item; (item = walk.at(rd)) >= 0 && ok; ++rd) {
      const ItemGeom g = item_geom(item, nq, p.H, T, window, p.doc_start, p.doc_sb, p.window_blocks);
      if (!g.valid[s]) continue;
      const int q0 = g.q0[s];
      const int q_row = q0 + row;
      if (QRAW && !q_prepared) {
        ok = prepare_q(q_row);
        if (!ok) break;
      }
      q_prepared = false;
      // the next item's Q is prepared inside this item's loop (second iteration), in time these warps would
      // otherwise spend waiting for the tensor core
      const int item_next = walk.at(rd + 1);
      bool next_valid = false;
      int q_row_next = 0;
      if (QRAW && item_next >= 0) {
        const ItemGeom gn = item_geom(item_next, nq, p.H, T, window, p.doc_start, p.doc_sb, p.window_blocks);
        next_valid = gn.valid[s];
        q_row_next = gn.q0[s] + row;
      }
      float m_ref = NEG_BIG, l = 0.f, pend = 0.f;   // pend: how far the reference is known to lag (applied before the next P)
      const int ds_row = p.doc_start ? min(p.doc_start[g.b * p.doc_sb + min(q_row, T - 1)], q_row) : 0;   // a row always sees itself
      const int ds_max = p.doc_start ? p.doc_start[g.b * p.doc_sb + min(q0 + BM - 1, T - 1)] : 0;
      for (int j = g.jlo_s[s]; j <= g.jhi_s[s]; ++j) {
        const bool first = (j == g.jlo_s[s]);
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[s], n_s & 1, abort_flag, p.status, 6));
        if (!ok) break;
        ++n_s;
        tc_fence_after();
        const int k0 = j * BN;
        const bool full_tile = (k0 + BN - 1 <= q0) && (window <= 0 || k0 > q0 + BM - 1 - window) && ds_max <= k0;
        // whole S row into registers
        tmem_ld32(s_tmem, r);
        tmem_ld32(s_tmem + 32, r + 32);
        tmem_ld32(s_tmem + 64, r + 64);
        tmem_ld32(s_tmem + 96, r + 96);
        tc_wait_ld();
        if (!full_tile) {
          // column i of this tile is visible iff lo < i <= hi
          const int hi = q_row - k0;
          const int lo = max(window > 0 ? q_row - window - k0 : -1, ds_row - 1 - k0);
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (!(i > lo && i <= hi)) r[i] = 0xff800000u;              // -inf
        }
        // Reference maximum.  General inputs: row max of every tile first, accumulator rescaled lazily (only when
        // the maximum grew by more than 8).  BOUNDED inputs (RMS-normalised q and k, so |logit| <= scale*D and
        // 2^x cannot overflow whatever the reference): only an item's first tile pays for the max pass; later
        // tiles exponentiate against the current reference at once, the largest P of the row is tracked on the
        // side, and a reference that turned out stale by more than 2^8 is raised before the NEXT tile.
        float m_tgt = m_ref + pend;                                  // BOUNDED: reference the previous tile asked for
        const bool need_max = first || !BOUNDED || __any_sync(0xffffffffu, m_ref == NEG_BIG);   // warp-uniform
        if (need_max) {
          float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            m0 = fmax3(m0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
            m1 = fmax3(m1, __uint_as_float(r[32 + i]), __uint_as_float(r[33 + i]));
            m2 = fmax3(m2, __uint_as_float(r[64 + i]), __uint_as_float(r[65 + i]));
            m3 = fmax3(m3, __uint_as_float(r[96 + i]), __uint_as_float(r[97 + i]));
          }
          m_tgt = fmaxf(m_tgt, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * c2);
        }
        if (first) {
          m_ref = m_tgt;
        } else if (__any_sync(0xffffffffu, m_tgt - m_ref > 8.0f)) {
          const float alpha = fast_exp2(m_ref - m_tgt);              // 0 for rows that had seen nothing yet
          m_ref = m_tgt;
          l *= alpha;
          uint32_t t16[16];
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            tmem_ld16(o_tmem + 16 * c, t16);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) t16[i] = __float_as_uint(__uint_as_float(t16[i]) * alpha);
            tmem_st16(o_tmem + 16 * c, t16);
          }
        }
        pend = 0.f;
        // P = exp2(S * c2 - m_ref) as bf16 into TMEM over S; row sum in fp32
        const uint64_t c2p = pack2f(c2, c2), nm = pack2f(-m_ref, -m_ref);
        uint64_t sum_a = pack2f(0.f, 0.f), sum_b = sum_a;
        uint32_t pmax2 = 0u;                                         // running max of the packed bf16 P (both halves)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const uint64_t xa = ffma2(pack2f(__uint_as_float(r[32 * c + i]), __uint_as_float(r[32 * c + i + 1])), c2p, nm);
            const uint64_t xb = ffma2(pack2f(__uint_as_float(r[32 * c + i + 2]), __uint_as_float(r[32 * c + i + 3])), c2p, nm);
            float x0, x1, p2, p3;
            unpack2f(xa, x0, x1);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            uint64_t pb;
            if (POLY_HALF || (POLY_MASK && (i & POLY_MASK) == POLY_MASK)) {                       // a share of the pairs goes to the FMA pipes
              pb = exp2_poly2(xb);
              unpack2f(pb, p2, p3);
            } else {
              float x2, x3;
              unpack2f(xb, x2, x3);
              p2 = fast_exp2(x2); p3 = fast_exp2(x3);
              pb = pack2f(p2, p3);
            }
            sum_a = fadd2(sum_a, pack2f(p0, p1));
            sum_b = fadd2(sum_b, pb);
            pk[i >> 1] = pack_bf16(p0, p1);
            pk[(i >> 1) + 1] = pack_bf16(p2, p3);
            // P >= 0, so bf16 bit patterns order like unsigned integers
            if (BOUNDED) {
              const uint32_t a = pk[i >> 1], b2 = pk[(i >> 1) + 1];
              pmax2 = max(pmax2, max(max(a & 0xffff0000u, b2 & 0xffff0000u), max(a << 16, b2 << 16)));
            }
          }
          tmem_st16(s_tmem + 16 * c, pk);
        }
        float rowsum;
        {
          float a0, a1, b0, b1;
          unpack2f(sum_a, a0, a1);
          unpack2f(sum_b, b0, b1);
          rowsum = (a0 + a1) + (b0 + b1);
        }
        if (BOUNDED) {                                               // largest P = 2^(how far the reference lags)
          const float pmaxf = __uint_as_float(pmax2);
          pend = pmaxf > 256.f ? __log2f(pmaxf) : 0.f;
        }
        l += rowsum;
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&bars->p_full[s]);
        if (QRAW && next_valid && !q_prepared && j == g.jlo_s[s] + 1) {
          ok = prepare_q(q_row_next);
          if (!ok) break;
          q_prepared = true;
        }
      }
      if (ok) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full[s], n_o & 1, abort_flag, p.status, 7));
        ++n_o;
      }
      if (ok) {
        tc_fence_after();
        const float inv = 1.0f / l;
        if (p.lse2 && q_row < T) p.lse2[((int64_t)g.b * p.H + g.h) * T + q_row] = m_ref + __log2f(l);
        __nv_bfloat16* dst = p.out + g.b * p.o_sb + (int64_t)q_row * p.o_st + g.h * p.o_sh;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld32(o_tmem + 32 * c, r);
          tc_wait_ld();
          if (q_row < T) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
              o.y = pack_bf16(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
              o.z = pack_bf16(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
              o.w = pack_bf16(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + 32 * c + i) = o;
            }
          }
        }
        // the next item's first PV overwrites O_s only after this warp's P of that item has been signalled,
        // i.e. after these loads: program order of this warp is the guard
        tc_fence_before();
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// Tensor-core self-test: C[128,128] = A[128,K] x B in the three operand forms the kernel above uses.
struct SelftestParams { const __nv_bfloat16* a; float* c; int K, mode; int* status; };

__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                     const SelftestParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_tile = smem;
  uint8_t* b_tile = smem + TILE_BYTES;
  struct Bars { uint64_t full, done; uint32_t tmem_base; int abort_flag; };
  Bars* bars = reinterpret_cast<Bars*>(smem + 2 * TILE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // mode 3 is mode 0 with a transaction count that nothing completes: the bounded wait must give up, raise the
  // abort flag, report DAISY_ETIMEOUT and leave through the normal teardown
  const bool starve = (p.mode == 3);
  const int K = p.K, mode = starve ? 0 : p.mode;
  const int nhalf = K / 64;

  if (threadIdx.x == 0) {
    mbar_init(&bars->full, 1); mbar_init(&bars->done, 1); bars->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 0) { tmem_alloc(&bars->tmem_base, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
  const int row = warp * 32 + lane;
  // mode 0/1: A is [128 rows, K] in K-major boxes of 64 columns (128 rows each, 16 KB apart).
  // mode 0: B is [128 rows(N), K] the same way.  mode 1/2: B is [K rows, 128 cols(N)]: two boxes of
  // [K rows x 64 cols], K*128 bytes apart.
  const uint32_t b_half = (mode == 0) ? HALF_BYTES : (uint32_t)K * 128u;
  if (threadIdx.x == 0) {
    uint32_t bytes = (mode == 2 ? 0 : 128 * K * 2) + 128 * K * 2;
    mbar_expect_tx(&bars->full, bytes + (starve ? 16u : 0u));
    if (mode != 2)
      for (int hlf = 0; hlf < nhalf; ++hlf) tma_load_3d(a_tile + hlf * HALF_BYTES, &tm_a, &bars->full, 64 * hlf, 0, 0);
    if (mode == 0)
      for (int hlf = 0; hlf < nhalf; ++hlf) tma_load_3d(b_tile + hlf * HALF_BYTES, &tm_b, &bars->full, 64 * hlf, 0, 0);
    else
      for (int hlf = 0; hlf < 2; ++hlf) tma_load_3d(b_tile + hlf * b_half, &tm_b, &bars->full, 64 * hlf, 0, 0);
  }
  bool ok = true;
  if (mode == 2) {
    // A row -> TMEM columns [128, 128 + K/2) as packed bf16 pairs
    const uint32_t* arow = reinterpret_cast<const uint32_t*>(p.a + (int64_t)row * K);
    for (int c = 0; c < K / 32; ++c) {
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) pk[i] = arow[16 * c + i];
      tmem_st16(tmem_base + lane_off + 128 + 16 * c, pk);
    }
    tc_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    ok = mbar_wait(&bars->full, 0, &bars->abort_flag, p.status, 1);
    if (ok) {
      tc_fence_after();
      const uint32_t aa = smem_u32(a_tile), ba = smem_u32(b_tile);
      const uint32_t idesc = umma_idesc_bf16(128, 128, 0, mode == 0 ? 0 : 1);
      for (int k = 0; k < K / 16; ++k) {
        const uint32_t koff = (k >> 2) * HALF_BYTES + (k & 3) * 32;
        const uint64_t bdesc = (mode == 0) ? umma_desc_sw128(ba + koff, 16, 1024)
                                           : umma_desc_sw128(ba + k * 2048, b_half, 1024);
        if (mode == 2) umma_ts(tmem_base, tmem_base + 128 + 8 * k, bdesc, idesc, k > 0);
        else           umma_ss(tmem_base, umma_desc_sw128(aa + koff, 16, 1024), bdesc, idesc, k > 0);
      }
      tc_commit(&bars->done);
    }
  }
  ok = __all_sync(0xffffffffu, mbar_wait(&bars->done, 0, &bars->abort_flag, p.status, 2));
  if (ok) {
    tc_fence_after();
    uint32_t r[32];
    for (int c = 0; c < 4; ++c) {
      tmem_ld32(tmem_base + lane_off + 32 * c, r);
      tc_wait_ld();
      for (int i = 0; i < 32; ++i) p.c[row * 128 + 32 * c + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

}  // namespace daisy

using namespace daisy;

static int ensure_smem_attr() {
  static bool done[daisy_host::MAX_DEVICES] = {};             // the attribute is per device
  const int dev = daisy_host::device_slot();
  if (dev < 0) return DAISY_ENODEV;
  if (done[dev]) return DAISY_OK;
  if (cudaFuncSetAttribute(swa_prefill_kernel<false, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PREFILL_SMEM) != cudaSuccess) return DAISY_ECUDA;
  if (cudaFuncSetAttribute(swa_prefill_kernel<false, true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PREFILL_SMEM) != cudaSuccess) return DAISY_ECUDA;
  if (cudaFuncSetAttribute(swa_prefill_kernel<true, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PREFILL_SMEM) != cudaSuccess) return DAISY_ECUDA;
  if (cudaFuncSetAttribute(swa_prefill_kernel<true, true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PREFILL_SMEM) != cudaSuccess) return DAISY_ECUDA;
  if (cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 1024 + 2 * TILE_BYTES + 64) != cudaSuccess) return DAISY_ECUDA;
  done[dev] = true;
  return DAISY_OK;
}

// Shared launcher.  `qt` non-null: q is the RAW projection and the kernel normalises / rotates it on load.
struct QTransform { const float* cos; const float* sin; float eps; int norm, rope; };

static int launch_attend(const void* q, const void* k, const void* v,
                         int64_t q_sb, int64_t q_st, int64_t q_sh, int64_t k_sb, int64_t k_st, int64_t k_sh,
                         int64_t v_sb, int64_t v_st, int64_t v_sh,
                         void* out, int64_t o_sb, int64_t o_st, int64_t o_sh,
                         int B, int T, int H, int D, int window, float scale, const QTransform* qt, bool bounded_qk,
                         const int* doc_start, int64_t doc_sb, bool window_in_blocks, int* status_word, void* stream,
                         float* lse2 = nullptr) {
  if (!q || !k || !v || !out || B <= 0 || T <= 0 || H <= 0 || !(scale > 0.f)) return DAISY_EINVAL;
  if (D != DAISY_HEAD_DIM) return DAISY_EUNSUPPORTED;
  if (!daisy_aligned16(q) || !daisy_aligned16(k) || !daisy_aligned16(v) || !daisy_aligned16(out) || ((o_sb | o_st | o_sh) & 7) ||
      ((q_sb | q_st | q_sh | k_sb | k_st | k_sh | v_sb | v_st | v_sh) & 7))
    return DAISY_EALIGN;
  if (q_st <= 0 || k_st <= 0 || v_st <= 0 || q_sh < 0 || k_sh < 0 || v_sh < 0 || q_sb < 0 || k_sb < 0 || v_sb < 0) return DAISY_EINVAL;
  // a zero stride on a dimension longer than 1 is a broadcast (expanded) view, which the tile loads cannot express
  if ((H > 1 && (q_sh == 0 || k_sh == 0 || v_sh == 0)) || (B > 1 && (q_sb == 0 || k_sb == 0 || v_sb == 0))) return DAISY_EINVAL;
  if (qt && qt->rope && (!qt->cos || !qt->sin)) return DAISY_EINVAL;
  if (doc_start && (doc_sb < 0 || (reinterpret_cast<uintptr_t>(doc_start) & 3))) return DAISY_EINVAL;
  if (qt && qt->rope && (!daisy_aligned16(qt->cos) || !daisy_aligned16(qt->sin))) return DAISY_EALIGN;
  if (const int arc = ensure_smem_attr(); arc != DAISY_OK) { (void)cudaGetLastError(); return arc; }
  CUtensorMap tq, tk, tv;
  int rc;
  // a size-1 dimension may come with any stride; the encoder wants a non-zero multiple of 16 bytes
  auto sb = [](int64_t s, int n) { return (uint64_t)(n == 1 ? 16 : s * 2); };
  if ((rc = daisy_host::make_tmap_bf16_dthb(&tq, q, D, T, H, B, q_st * 2, sb(q_sh, H), sb(q_sb, B), 64, BM)) != DAISY_OK) return rc;
  if ((rc = daisy_host::make_tmap_bf16_dthb(&tk, k, D, T, H, B, k_st * 2, sb(k_sh, H), sb(k_sb, B), 64, BN)) != DAISY_OK) return rc;
  if ((rc = daisy_host::make_tmap_bf16_dthb(&tv, v, D, T, H, B, v_st * 2, sb(v_sh, H), sb(v_sb, B), 64, BN)) != DAISY_OK) return rc;
  PrefillParams p;
  p.out = (__nv_bfloat16*)out; p.o_sb = o_sb; p.o_st = o_st; p.o_sh = o_sh;
  p.T = T; p.H = H; p.B = B;
  p.window = window_in_blocks ? 0 : window;
  p.window_blocks = (window_in_blocks && window > 0) ? window : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_word;
  p.doc_start = doc_start; p.doc_sb = doc_sb;
  p.cos = qt ? qt->cos : nullptr; p.sin = qt ? qt->sin : nullptr;
  p.eps = qt ? qt->eps : 0.f; p.q_norm = qt ? qt->norm : 0; p.q_rope = qt ? qt->rope : 0;
  p.lse2 = lse2;
  const int64_t items = (int64_t)((T + 2 * BM - 1) / (2 * BM)) * H * B;
  if (items >= (int64_t)1 << 31) return DAISY_EUNSUPPORTED;
  const int sms = daisy_host::sm_count_cached();
  if (sms <= 0) return DAISY_ENODEV;
  dim3 grid((unsigned)(items < sms ? items : sms), 1, 1);
  const bool raw = qt && (qt->norm || qt->rope);
  // with RMS-normalised q and k every logit is bounded by scale * D: 2^(logit - reference) cannot overflow
  const bool bounded = bounded_qk && scale * 1.4426950408889634f * (float)D <= 60.f;
  cudaStream_t st = (cudaStream_t)stream;
  // bounded logits take the form with two softmax warpgroups per stream, everything else the general form
  if (raw && bounded)  swa_prefill_kernel<true, true, 2><<<grid, PREFILL_THREADS_SPLIT, PREFILL_SMEM, st>>>(tq, tk, tv, p);
  else if (raw)        swa_prefill_kernel<true, false, 1><<<grid, PREFILL_THREADS, PREFILL_SMEM, st>>>(tq, tk, tv, p);
  else if (bounded)    swa_prefill_kernel<false, true, 2><<<grid, PREFILL_THREADS_SPLIT, PREFILL_SMEM, st>>>(tq, tk, tv, p);
  else                 swa_prefill_kernel<false, false, 1><<<grid, PREFILL_THREADS, PREFILL_SMEM, st>>>(tq, tk, tv, p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}

extern "C" int daisy_b200_swa_attend(const void* q, const void* k, const void* v,
                                     int64_t q_sb, int64_t q_st, int64_t q_sh,
                                     int64_t k_sb, int64_t k_st, int64_t k_sh,
                                     int64_t v_sb, int64_t v_st, int64_t v_sh,
                                     void* out, int64_t o_sb, int64_t o_st, int64_t o_sh,
                                     int B, int T, int H, int D, int window, float scale,
                                     const int32_t* doc_start, int64_t doc_sb,
                                     unsigned flags, int* status_word, void* stream) {
  if (flags & ~(DAISY_BOUNDED_QK | DAISY_WINDOW_BLOCKS)) return DAISY_EINVAL;
  return launch_attend(q, k, v, q_sb, q_st, q_sh, k_sb, k_st, k_sh, v_sb, v_st, v_sh, out, o_sb, o_st, o_sh,
                       B, T, H, D, window, scale, nullptr, (flags & DAISY_BOUNDED_QK) != 0, doc_start, doc_sb,
                       (flags & DAISY_WINDOW_BLOCKS) != 0, status_word, stream);
}

extern "C" int daisy_b200_swa_attend_lse(const void* q, const void* k, const void* v,
                                         int64_t q_sb, int64_t q_st, int64_t q_sh,
                                         int64_t k_sb, int64_t k_st, int64_t k_sh,
                                         int64_t v_sb, int64_t v_st, int64_t v_sh,
                                         void* out, int64_t o_sb, int64_t o_st, int64_t o_sh, float* lse2,
                                         int B, int T, int H, int D, int window, float scale,
                                         const int32_t* doc_start, int64_t doc_sb,
                                         unsigned flags, int* status_word, void* stream) {
  if (flags & ~(DAISY_BOUNDED_QK | DAISY_WINDOW_BLOCKS)) return DAISY_EINVAL;
  if (!lse2 || (reinterpret_cast<uintptr_t>(lse2) & 3)) return DAISY_EINVAL;
  return launch_attend(q, k, v, q_sb, q_st, q_sh, k_sb, k_st, k_sh, v_sb, v_st, v_sh, out, o_sb, o_st, o_sh,
                       B, T, H, D, window, scale, nullptr, (flags & DAISY_BOUNDED_QK) != 0, doc_start, doc_sb,
                       (flags & DAISY_WINDOW_BLOCKS) != 0, status_word, stream, lse2);
}

static size_t align1k(size_t x) { return (x + 1023) & ~size_t(1023); }

extern "C" size_t daisy_b200_swa_prefill_workspace_bytes(int B, int T, int H, int D) {
  if (B <= 0 || T <= 0 || H <= 0 || D <= 0) return 0;
  return 3 * align1k((size_t)B * T * H * D * 2);       // slots: q', k', v' -- the latter two only when k_out/v_out are NULL
}

extern "C" int daisy_b200_swa_prefill_fwd(const void* q, const void* k, const void* v,
                                          int64_t q_sb, int64_t q_st, int64_t q_sh,
                                          int64_t k_sb, int64_t k_st, int64_t k_sh,
                                          int64_t v_sb, int64_t v_st, int64_t v_sh,
                                          const float* cos, const float* sin,
                                          void* out, int64_t o_sb, int64_t o_st, int64_t o_sh,
                                          void* k_out, void* v_out,
                                          int B, int T, int H, int D, int window, float scale, float eps,
                                          const int32_t* doc_start, int64_t doc_sb,
                                          unsigned flags, void* workspace, size_t workspace_bytes,
                                          int* status_word, void* stream) {
  if (!q || !k || !v || !out || !workspace || B <= 0 || T <= 0 || H <= 0) return DAISY_EINVAL;
  if (D != DAISY_HEAD_DIM) return DAISY_EUNSUPPORTED;
  if (workspace_bytes < daisy_b200_swa_prefill_workspace_bytes(B, T, H, D)) return DAISY_EWORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return DAISY_EALIGN;
  const size_t one = align1k((size_t)B * T * H * D * 2);
  char* ws = (char*)workspace;
  void* kp = k_out ? k_out : (void*)(ws + one);
  void* vp = v_out ? v_out : (void*)(ws + 2 * one);
  // K and V are prepared once (they are outputs anyway: the cache rows) and keep the [B,T,H,D] memory order
  // of the projections, a pure streaming pass.  Q is either prepared in the same pass (default) or, with
  // DAISY_Q_IN_KERNEL, consumed raw: the attention kernel then normalises and rotates each Q tile in shared
  // memory one item ahead of its use.  Measured on C2 the in-kernel form is slower (1.22 ms vs 1.18 ms per
  // step, 3.69 vs 3.45 ms at C4: the transform sits on the softmax warps, whose P the tensor pipe waits for),
  // so it is opt-in.
  const bool q_in_kernel = (flags & DAISY_Q_IN_KERNEL) != 0;
  const bool bounded_qk = (flags & DAISY_NORM_Q) && (flags & DAISY_NORM_K);
  void* qp = ws;
  const unsigned pf = (flags & DAISY_QKV_DEFAULT) | ((flags & DAISY_KV_BHTD) ? 0u : DAISY_OUT_BTHD);
  const int64_t HD = (int64_t)H * D, TD = (int64_t)T * D;
  int64_t sb_ = (int64_t)T * HD, st_ = HD, sh_ = D;
  if (flags & DAISY_KV_BHTD) { st_ = D; sh_ = TD; }
  QTransform qt{cos, sin, eps, (flags & DAISY_NORM_Q) ? 1 : 0, (flags & DAISY_ROPE) ? 1 : 0};

  // One batch slice [b0, b0 + nb): the streaming pass, then the attention over what it wrote.
  auto off = [](const void* base, int64_t elems) { return (const void*)((const char*)base + elems * 2); };
  auto prep = [&](int b0, int nb, void* s) {
    return daisy_b200_qkv_prep(q_in_kernel ? nullptr : off(q, b0 * q_sb), off(k, b0 * k_sb), off(v, b0 * v_sb),
                               q_sb, q_st, q_sh, k_sb, k_st, k_sh, v_sb, v_st, v_sh, cos, sin,
                               q_in_kernel ? nullptr : (void*)off(qp, b0 * sb_), (void*)off(kp, b0 * sb_), (void*)off(vp, b0 * sb_),
                               nullptr, 0, 0, 0, nullptr, nb, T, H, D, eps, pf, s);
  };
  auto attend = [&](int b0, int nb, void* s) {
    if (q_in_kernel)
      return launch_attend(off(q, b0 * q_sb), off(kp, b0 * sb_), off(vp, b0 * sb_), q_sb, q_st, q_sh, sb_, st_, sh_, sb_, st_, sh_,
                           (void*)off(out, b0 * o_sb), o_sb, o_st, o_sh, nb, T, H, D, window, scale, &qt, bounded_qk,
                           doc_start ? doc_start + b0 * doc_sb : nullptr, doc_sb, (flags & DAISY_WINDOW_BLOCKS) != 0, status_word, s);
    return launch_attend(off(qp, b0 * sb_), off(kp, b0 * sb_), off(vp, b0 * sb_), sb_, st_, sh_, sb_, st_, sh_, sb_, st_, sh_,
                         (void*)off(out, b0 * o_sb), o_sb, o_st, o_sh, nb, T, H, D, window, scale, nullptr, bounded_qk,
                         doc_start ? doc_start + b0 * doc_sb : nullptr, doc_sb, (flags & DAISY_WINDOW_BLOCKS) != 0, status_word, s);
  };

  // (Cutting the batch into slices so that the streaming pass over slice i+1 runs on a side stream underneath the
  // attention over slice i was measured at C2: 1.5 % with two slices, a loss with four -- both kernels already
  // run against the board's power limit -- so the two launches simply follow one another.)
  int rc = prep(0, B, stream);
  if (rc != DAISY_OK) return rc;
  return attend(0, B, stream);
}

extern "C" int daisy_b200_selftest_umma(const void* a, const void* b, float* c, int K, int mode,
                                        int* status_word, void* stream) {
  if (!a || !b || !c || (K != 64 && K != 128) || mode < 0 || mode > 3) return DAISY_EINVAL;
  if (const int arc = ensure_smem_attr(); arc != DAISY_OK) { (void)cudaGetLastError(); return arc; }
  CUtensorMap ta, tb;
  int rc;
  if ((rc = daisy_host::make_tmap_bf16_3d(&ta, a, K, 128, 1, (uint64_t)K * 2, (uint64_t)K * 256, 64, 128)) != DAISY_OK) return rc;
  if (mode == 0 || mode == 3) rc = daisy_host::make_tmap_bf16_3d(&tb, b, K, 128, 1, (uint64_t)K * 2, (uint64_t)K * 256, 64, 128);
  else           rc = daisy_host::make_tmap_bf16_3d(&tb, b, 128, K, 1, 256, (uint64_t)K * 256, 64, K);
  if (rc != DAISY_OK) return rc;
  SelftestParams p{(const __nv_bfloat16*)a, c, K, mode, status_word};
  umma_selftest_kernel<<<1, 128, 1024 + 2 * TILE_BYTES + 64, (cudaStream_t)stream>>>(ta, tb, p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}
