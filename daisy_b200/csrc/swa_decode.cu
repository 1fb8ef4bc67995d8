// Sliding-window decode step over a ring-buffer KV cache: split-KV partial pass + combine pass.
//
// HBM-bound: per (batch, head) the step reads r context rows of K and of V (256 bytes each) once.
// Pass 1 (grid = splits x H x B, 128 threads): each half-warp owns one 256-byte row per load
// instruction (16 bytes per lane, two adjacent rows per warp instruction -> 512 contiguous bytes),
// eight rows of K and of V are in flight per warp before any is consumed, the ring is indexed in
// place (slot = start + i, minus cap on wrap), scores are reduced with xor-shuffles inside the
// half-warp and folded into a running (max, sum, acc[128]) in the exp2 domain.  Pass 2 (grid = H x B)
// normalises/rotates the new token's q,k,v, merges the split partials with the new row's own score,
// writes the output and stores the new k,v row into the ring -- after every read of pass 1 has
// completed, so a window larger than the ring capacity still sees the row it is about to overwrite.
#include "rowops.cuh"
#include <cuda_fp16.h>

namespace daisy {

#define DEC_NEG (-1.0e30f)

// eight 16-bit cache values -> fp32: bf16 (the model dtype) or fp16 (the reference Generator's default cache
// dtype, inference/generate.py:62)
template <bool F16>
__device__ __forceinline__ void unpack8_cache(const uint4& u, float* f) {
  if (F16) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  } else {
    unpack8(u, f);
  }
}

struct DecodeParams {
  const __nv_bfloat16 *q, *k, *v;
  int64_t q_sb, q_sh, k_sb, k_sh, v_sb, v_sh;
  __nv_bfloat16 *kc, *vc;
  int64_t c_sb, c_sh, c_sr;
  int start_slot, r, cap, new_slot;
  const float *cos_row, *sin_row;
  __nv_bfloat16* out;
  int64_t o_sb, o_sh;
  __nv_bfloat16 *k_new_out, *v_new_out;
  int B, H;
  float qscale, eps;
  unsigned flags;
  float* ws_acc;   // [B,H,splits,128]
  float* ws_ml;    // [B,H,splits,2]
  int splits, rows_per_split;
  // position on the device (CUDA-graph replays): when t_dev is set, start_slot / r / new_slot / rows_per_split are
  // derived from *t_dev in the kernels, and cos_row / sin_row are the BASES of tables with table_rows rows
  const long long* t_dev;
  int window, table_rows;
  int* status;
  // single-launch form: the last split CTA of a (batch, head) to finish merges the partials itself; `tickets` holds
  // one counter per (batch, head), zero between calls
  int* tickets;
  // value-embedding gate on the new token's v (after the norm): v = g v + (1 - g) ve, g = sigmoid(*ve_gate)
  const __nv_bfloat16* ve;
  int64_t ve_sb, ve_sh;
  const float* ve_gate;
  int prefetch;    // single-launch form: hint the ring slice into L2 before waiting for the preceding kernel
};

// Row range and table rows of this step: the host's values, or derived from the device-side position.
struct DecodeGeom { int r, start_slot, new_slot, rows_per_split; const float *cos_row, *sin_row; };
template <bool DEV>
__device__ __forceinline__ DecodeGeom decode_geom(const DecodeParams& p) {
  DecodeGeom g{p.r, p.start_slot, p.new_slot, p.rows_per_split, p.cos_row, p.sin_row};
  if (DEV) {
    const long long t = *p.t_dev;
    long long r = t < p.cap ? t : p.cap;
    if (p.window > 0 && r > (long long)p.window - 1) r = p.window - 1;
    g.r = (int)r;
    g.start_slot = p.cap > 0 ? (int)((t - r) % p.cap) : 0;
    g.new_slot = p.cap > 0 ? (int)(t % p.cap) : 0;
    int rps = ((int)r + p.splits - 1) / p.splits;
    rps = (rps + 31) / 32 * 32;
    g.rows_per_split = rps ? rps : 32;
    long long pos = t;
    if (pos >= p.table_rows) {                                     // past the RoPE table: report, stay in bounds
      pos = p.table_rows - 1;
      if (p.status && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) p.status[0] = DAISY_EINVAL;
    }
    g.cos_row = p.cos_row + pos * (DAISY_HEAD_DIM / 2);
    g.sin_row = p.sin_row + pos * (DAISY_HEAD_DIM / 2);
  }
  return g;
}

template <bool DEV, bool F16>
__device__ __forceinline__ void decode_combine_body(const DecodeParams& p, const DecodeGeom& g, int h, int b, bool coherent);

// PIPE: issue the next iteration's loads before the current one's arithmetic (twice the registers).  It pays when a CTA
// has only a few iterations -- small batches, where the kernel is latency-bound -- and costs occupancy when the ring
// traffic is large enough to saturate HBM anyway.
template <bool DEV, bool F16, bool FUSED, bool PIPE = false>
__global__ void __launch_bounds__(128) swa_decode_partial_kernel(const DecodeParams p) {
  const int s = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, hw = lane >> 4, sub = lane & 15;

  if (FUSED) {
    // Launched as a dependent grid (see grid_dep_wait): while the projection that produces q, k, v still runs, ask L2
    // for this CTA's slice of the ring -- older tokens, which that projection does not touch.  Only a hint: the range
    // comes from a position that may be stale and is clamped to the ring; everything is read again after the wait.
    if (p.prefetch && threadIdx.x < 2) {
      const DecodeGeom g0 = decode_geom<DEV>(p);
      const int i0 = s * g0.rows_per_split, n = min(g0.r, i0 + g0.rows_per_split) - i0;
      if (n > 0 && n <= p.cap && g0.start_slot >= 0 && g0.start_slot < p.cap) {
        int s0 = g0.start_slot + i0;
        if (s0 >= p.cap) s0 -= p.cap;
        const int n1 = min(n, p.cap - s0);
        const __nv_bfloat16* base = (threadIdx.x ? p.vc : p.kc) + b * p.c_sb + h * p.c_sh;
        if (s0 >= 0 && s0 < p.cap) {
          l2_prefetch_bulk(base + (int64_t)s0 * p.c_sr, (uint32_t)(((int64_t)(n1 - 1) * p.c_sr + DAISY_HEAD_DIM) * 2));
          if (n > n1) l2_prefetch_bulk(base, (uint32_t)(((int64_t)(n - n1 - 1) * p.c_sr + DAISY_HEAD_DIM) * 2));
        }
      }
    }
    grid_dep_launch();
    grid_dep_wait();
  }
  const DecodeGeom g = decode_geom<DEV>(p);
  float qf[8];
  auto load_q = [&]() {
    unpack8(ld_cg16(p.q + b * p.q_sb + h * p.q_sh + 8 * sub), qf);
    norm_rope_row8(qf, sub, p.flags & DAISY_NORM_Q, p.flags & DAISY_ROPE, p.eps, g.cos_row, g.sin_row);
#pragma unroll
    for (int e = 0; e < 8; ++e) qf[e] *= p.qscale;
  };
  if (!PIPE) load_q();                                  // PIPE: after the first ring rows are on their way

  const int i0 = s * g.rows_per_split;
  const int i1 = min(g.r, i0 + g.rows_per_split);
  const __nv_bfloat16* kbase = p.kc + b * p.c_sb + h * p.c_sh + 8 * sub;
  const __nv_bfloat16* vbase = p.vc + b * p.c_sb + h * p.c_sh + 8 * sub;

  float m = DEC_NEG, l = 0.f, acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;

  // Rows come eight per warp iteration (four per half-warp).
  auto fetch = [&](int base, uint4* kk, uint4* vv, unsigned& valid) {
    valid = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = base + 2 * j + hw;
      const bool ok = row < i1;
      valid |= ok ? (1u << j) : 0u;
      int slot = g.start_slot + (ok ? row : i0);
      if (slot >= p.cap) slot -= p.cap;
      kk[j] = ld_stream16(kbase + (int64_t)slot * p.c_sr);
      vv[j] = ld_stream16(vbase + (int64_t)slot * p.c_sr);
    }
  };
  auto consume = [&](const uint4* kk, const uint4* vv, unsigned valid) {
    float sc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float kf[8];
      unpack8_cache<F16>(kk[j], kf);
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) d = fmaf(qf[e], kf[e], d);
      d = halfwarp_sum(d);
      sc[j] = (valid >> j) & 1u ? d : -INFINITY;
    }
    const float mn = fmaxf(fmaxf(m, fmaxf(sc[0], sc[1])), fmaxf(sc[2], sc[3]));
    const float alpha = fast_exp2(m - mn);
    float pj[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) pj[j] = fast_exp2(sc[j] - mn);
    l = l * alpha + (pj[0] + pj[1]) + (pj[2] + pj[3]);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= alpha;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float vf[8];
      unpack8_cache<F16>(vv[j], vf);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = fmaf(pj[j], vf[e], acc[e]);
    }
    m = mn;
  };
  if (!PIPE) {
    for (int base = i0 + warp * 8; base < i1; base += 32) {
      uint4 ka[4], va[4];
      unsigned oka;
      fetch(base, ka, va, oka);
      consume(ka, va, oka);
    }
  } else {
    uint4 ka[4], va[4], kb[4], vb[4];
    unsigned oka = 0, okb = 0;
    int base = i0 + warp * 8;
    if (base < i1) fetch(base, ka, va, oka);
    load_q();
    while (base < i1) {
      const bool more_b = base + 32 < i1;
      if (more_b) fetch(base + 32, kb, vb, okb);
      consume(ka, va, oka);
      if (!more_b) break;
      const bool more_a = base + 64 < i1;
      if (more_a) fetch(base + 64, ka, va, oka);
      consume(kb, vb, okb);
      if (!more_a) break;
      base += 64;
    }
  }

  // merge the two half-warps
  {
    const float om = __shfl_xor_sync(0xffffffffu, m, 16);
    const float ol = __shfl_xor_sync(0xffffffffu, l, 16);
    const float M = fmaxf(m, om);
    const float a = fast_exp2(m - M), c = fast_exp2(om - M);
    l = l * a + ol * c;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float oa = __shfl_xor_sync(0xffffffffu, acc[e], 16);
      acc[e] = acc[e] * a + oa * c;
    }
    m = M;
  }
  __shared__ float sm_m[4], sm_l[4];
  __shared__ __align__(16) float sm_acc[4][DAISY_HEAD_DIM];
  if (hw == 0) {
    *reinterpret_cast<float4*>(&sm_acc[warp][8 * sub]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(&sm_acc[warp][8 * sub + 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (sub == 0) { sm_m[warp] = m; sm_l[warp] = l; }
  }
  __syncthreads();
  const int d = threadIdx.x;
  const float M = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
  float a = 0.f, L = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const float f = fast_exp2(sm_m[w] - M);
    a = fmaf(f, sm_acc[w][d], a);
    L = fmaf(f, sm_l[w], L);
  }
  const int64_t slot = ((int64_t)b * p.H + h) * p.splits + s;
  p.ws_acc[slot * DAISY_HEAD_DIM + d] = a;
  if (d == 0) { p.ws_ml[slot * 2] = M; p.ws_ml[slot * 2 + 1] = L; }
  if (FUSED) {
    // ticket per (batch, head): whoever draws the last one knows every other split's partials are in memory (each
    // CTA fences its stores before drawing) and merges them; it also puts the counter back to zero for the next call
    __shared__ int last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      int* tk = p.tickets + b * p.H + h;
      const int drawn = atomicAdd(tk, 1);
      last = (drawn == p.splits - 1);
      if (last) *tk = 0;
    }
    __syncthreads();
    if (last) {
      __threadfence();
      decode_combine_body<DEV, F16>(p, g, h, b, true);
    }
  }
}

__device__ __forceinline__ float block128_sum(float x, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  __syncthreads();                                   // protect `red` from the previous use
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = x;
  __syncthreads();
  return (red[0] + red[1]) + (red[2] + red[3]);
}

__device__ __forceinline__ float block128_max(float x, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = x;
  __syncthreads();
  return fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
}

// Merge of the split partials with the new token (thread = head-dim element, 128 threads): normalises / rotates the
// new q, k, v, adds the new row's own score, writes the output row and stores the new k, v into the ring.
// `coherent`: the partials were written by other SMs during this same launch -- read them past the L1.
template <bool DEV, bool F16>
__device__ __forceinline__ void decode_combine_body(const DecodeParams& p, const DecodeGeom& g, int h, int b, bool coherent) {
  const int d = threadIdx.x;
  __shared__ float red[4];
  __shared__ float xq[DAISY_HEAD_DIM], xk[DAISY_HEAD_DIM];
  float q = __bfloat162float(p.q[b * p.q_sb + h * p.q_sh + d]);
  float k = __bfloat162float(p.k[b * p.k_sb + h * p.k_sh + d]);
  float v = __bfloat162float(p.v[b * p.v_sb + h * p.v_sh + d]);
  const float inv_d = 1.0f / DAISY_HEAD_DIM;
  if (p.flags & DAISY_NORM_Q) q *= rsqrtf(block128_sum(q * q, red) * inv_d + p.eps);
  if (p.flags & DAISY_NORM_K) k *= rsqrtf(block128_sum(k * k, red) * inv_d + p.eps);
  if (p.flags & DAISY_NORM_V) v *= rsqrtf(block128_sum(v * v, red) * inv_d + p.eps);
  if (p.ve) {
    const float gate = 1.0f / (1.0f + __expf(-*p.ve_gate));
    v = gate * v + (1.0f - gate) * __bfloat162float(p.ve[b * p.ve_sb + h * p.ve_sh + d]);
  }
  if (p.flags & DAISY_ROPE) {
    xq[d] = q; xk[d] = k;
    __syncthreads();
    const float c = g.cos_row[d & 63], sn = g.sin_row[d & 63];
    const float sgn = d < 64 ? 1.f : -1.f;
    q = q * c + sgn * xq[d ^ 64] * sn;
    k = k * c + sgn * xk[d ^ 64] * sn;
  }
  // the new row is used at the precision it will have in the cache
  const __nv_bfloat16 kb = __float2bfloat16_rn(k), vb = __float2bfloat16_rn(v);
  const __half kh = __float2half_rn(k), vh = __float2half_rn(v);
  k = F16 ? __half2float(kh) : __bfloat162float(kb);
  v = F16 ? __half2float(vh) : __bfloat162float(vb);
  const float s_self = block128_sum(q * p.qscale * k, red);

  const int64_t base = ((int64_t)b * p.H + h) * p.splits;
  auto ml = [&](int64_t i) { return coherent ? __ldcg(p.ws_ml + i) : p.ws_ml[i]; };
  auto part = [&](int64_t s) { return coherent ? __ldcg(p.ws_acc + (base + s) * DAISY_HEAD_DIM + d) : p.ws_acc[(base + s) * DAISY_HEAD_DIM + d]; };
  float num, den;
  if (p.splits <= 128) {
    // one round trip for all the (maximum, sum) pairs -- thread s takes split s -- and the partial rows in batches of
    // eight loads in flight: a serial walk over the splits costs a memory latency per split, which at batch 1
    // (31 splits) was a third of the whole step
    __shared__ float wgt[128];
    float m_s = DEC_NEG, l_s = 0.f;
    if (d < p.splits) { m_s = ml((base + d) * 2); l_s = ml((base + d) * 2 + 1); }
    const float M = fmaxf(block128_max(m_s, red), s_self);
    const float f_s = d < p.splits ? fast_exp2(m_s - M) : 0.f;
    wgt[d] = f_s;
    const float w = fast_exp2(s_self - M);
    den = block128_sum(f_s * l_s, red) + w;            // its barriers also publish wgt
    num = w * v;
    for (int s0 = 0; s0 < p.splits; s0 += 8) {
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = s0 + j < p.splits ? part(s0 + j) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) num = fmaf(s0 + j < p.splits ? wgt[s0 + j] : 0.f, a[j], num);
    }
  } else {
    float M = s_self;
    for (int s = 0; s < p.splits; ++s) M = fmaxf(M, ml((base + s) * 2));
    const float w = fast_exp2(s_self - M);
    num = w * v; den = w;
    for (int s = 0; s < p.splits; ++s) {
      const float f = fast_exp2(ml((base + s) * 2) - M);
      num = fmaf(f, part(s), num);
      den = fmaf(f, ml((base + s) * 2 + 1), den);
    }
  }
  p.out[b * p.o_sb + h * p.o_sh + d] = __float2bfloat16_rn(num / den);
  const int64_t row = ((int64_t)b * p.H + h) * DAISY_HEAD_DIM + d;
  if (p.k_new_out) p.k_new_out[row] = kb;
  if (p.v_new_out) p.v_new_out[row] = vb;
  if (p.flags & DAISY_WRITE_RING) {
    const int64_t at = b * p.c_sb + h * p.c_sh + (int64_t)g.new_slot * p.c_sr + d;
    if (F16) { reinterpret_cast<__half*>(p.kc)[at] = kh; reinterpret_cast<__half*>(p.vc)[at] = vh; }
    else     { p.kc[at] = kb; p.vc[at] = vb; }
  }
}

template <bool DEV, bool F16>
__global__ void __launch_bounds__(128) swa_decode_combine_kernel(const DecodeParams p) {
  decode_combine_body<DEV, F16>(p, decode_geom<DEV>(p), blockIdx.x, blockIdx.y, false);
}

}  // namespace daisy

using namespace daisy;

extern "C" int daisy_b200_swa_decode_splits(int B, int H, int ctx_rows, int sm_count) {
  if (B <= 0 || H <= 0 || ctx_rows <= 0) return 1;
  if (sm_count <= 0) sm_count = 148;
  const int64_t bh = (int64_t)B * H;
  const int64_t target = (int64_t)sm_count * 16;            // 16 CTAs of 128 threads fit on one SM
  int64_t splits = (target + bh - 1) / bh;
  const int64_t max_by_rows = ctx_rows >= 128 ? (ctx_rows + 127) / 128 : 1;   // about 4 loop trips per CTA at least
  if (splits > max_by_rows) splits = max_by_rows;
  if (splits > 64) splits = 64;
  if (splits < 1) splits = 1;
  // a split covers a whole number of 32-row iterations: drop the splits that rounding would leave without rows
  // (4095 rows in 31 splits are 160 rows each, i.e. 26 splits of five iterations and five idle ones; 32 splits are
  // 128 rows each, four iterations, nobody idle)
  const int64_t rps = ((ctx_rows + splits - 1) / splits + 31) / 32 * 32;
  splits = (ctx_rows + rps - 1) / rps;
  return (int)splits;
}

extern "C" size_t daisy_b200_swa_decode_workspace_bytes(int B, int H, int D, int splits) {
  if (B <= 0 || H <= 0 || D <= 0 || splits <= 0) return 0;
  return (size_t)B * H * splits * (D + 2) * sizeof(float);
}

extern "C" size_t daisy_b200_swa_decode_fused_workspace_bytes(int B, int H, int D, int splits) {
  const size_t base = daisy_b200_swa_decode_workspace_bytes(B, H, D, splits);
  if (!base) return 0;
  return base + (((size_t)B * H * sizeof(int)) + 15) / 16 * 16;       // + one ticket per (batch, head)
}

struct DecodeExtras { bool fused; const void* ve; int64_t ve_sb, ve_sh; const float* ve_gate; };

static int decode_launch(const void* q_new, const void* k_new, const void* v_new,
                         int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh, int64_t v_sb, int64_t v_sh,
                         void* kcache, void* vcache, int64_t c_sb, int64_t c_sh, int64_t c_sr,
                         int64_t t, const int64_t* t_dev, int table_rows, int cap, int window,
                         const float* cos_row, const float* sin_row,
                         void* out, int64_t o_sb, int64_t o_sh, void* k_new_out, void* v_new_out,
                         int B, int H, int D, float scale, float eps, unsigned flags,
                         void* workspace, size_t workspace_bytes, int splits, int* status_word, void* stream,
                         const DecodeExtras ex = DecodeExtras{false, nullptr, 0, 0, nullptr}) {
  const bool fused = ex.fused;
  if (!q_new || !k_new || !v_new || !out || B <= 0 || H <= 0 || t < 0 || cap < 0 || splits <= 0) return DAISY_EINVAL;
  if (D != DAISY_HEAD_DIM) return DAISY_EUNSUPPORTED;
  if (B > 65535 || H > 65535) return DAISY_EUNSUPPORTED;
  if ((flags & DAISY_ROPE) && (!cos_row || !sin_row)) return DAISY_EINVAL;
  if ((flags & DAISY_WRITE_RING) && cap == 0) return DAISY_EINVAL;
  if (t_dev && (table_rows <= 0 || (reinterpret_cast<uintptr_t>(t_dev) & 7))) return DAISY_EINVAL;
  // with the position on the device the host sizes the launch for the longest context it can meet
  int64_t r = t_dev ? cap : (t < cap ? t : cap);
  if (window > 0 && r > (int64_t)window - 1) r = window - 1;
  if ((r > 0 || (flags & DAISY_WRITE_RING)) && (!kcache || !vcache)) return DAISY_EINVAL;
  if (!workspace) return DAISY_EINVAL;
  if (workspace_bytes < (fused ? daisy_b200_swa_decode_fused_workspace_bytes(B, H, D, splits) : daisy_b200_swa_decode_workspace_bytes(B, H, D, splits)))
    return DAISY_EWORKSPACE;
  if (ex.ve && (!ex.ve_gate || (flags & DAISY_NORM_V) == 0 || !daisy_aligned16(ex.ve) || ((ex.ve_sb | ex.ve_sh) & 7))) return DAISY_EINVAL;
  if (!daisy_aligned16(q_new) || !daisy_aligned16(k_new) || !daisy_aligned16(v_new) || !daisy_aligned16(workspace) ||
      ((q_sb | q_sh | k_sb | k_sh | v_sb | v_sh) & 7))
    return DAISY_EALIGN;
  if (r > 0 && (!daisy_aligned16(kcache) || !daisy_aligned16(vcache) || ((c_sb | c_sh | c_sr) & 7))) return DAISY_EALIGN;
  if ((flags & DAISY_ROPE) && (!daisy_aligned16(cos_row) || !daisy_aligned16(sin_row))) return DAISY_EALIGN;

  DecodeParams p;
  p.q = (const __nv_bfloat16*)q_new; p.k = (const __nv_bfloat16*)k_new; p.v = (const __nv_bfloat16*)v_new;
  p.q_sb = q_sb; p.q_sh = q_sh; p.k_sb = k_sb; p.k_sh = k_sh; p.v_sb = v_sb; p.v_sh = v_sh;
  p.kc = (__nv_bfloat16*)kcache; p.vc = (__nv_bfloat16*)vcache;
  p.c_sb = c_sb; p.c_sh = c_sh; p.c_sr = c_sr;
  p.r = (int)r; p.cap = cap;
  p.start_slot = (cap > 0 && !t_dev) ? (int)((t - r) % cap) : 0;
  p.new_slot = (cap > 0 && !t_dev) ? (int)(t % cap) : 0;
  p.cos_row = cos_row; p.sin_row = sin_row;
  p.out = (__nv_bfloat16*)out; p.o_sb = o_sb; p.o_sh = o_sh;
  p.k_new_out = (__nv_bfloat16*)k_new_out; p.v_new_out = (__nv_bfloat16*)v_new_out;
  p.B = B; p.H = H;
  p.qscale = scale * 1.4426950408889634f;
  p.eps = eps; p.flags = flags;
  p.ws_acc = (float*)workspace;
  p.ws_ml = p.ws_acc + (size_t)B * H * splits * DAISY_HEAD_DIM;
  p.splits = splits;
  int rps = (int)((r + splits - 1) / splits);
  rps = (rps + 31) / 32 * 32;                                 // whole 32-row CTA iterations
  if (rps == 0) rps = 32;
  p.rows_per_split = rps;
  p.t_dev = (const long long*)t_dev; p.window = window; p.table_rows = table_rows; p.status = status_word;
  p.tickets = fused ? reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + daisy_b200_swa_decode_workspace_bytes(B, H, D, splits)) : nullptr;
  p.ve = (const __nv_bfloat16*)ex.ve; p.ve_sb = ex.ve_sb; p.ve_sh = ex.ve_sh; p.ve_gate = ex.ve_gate;
  // the ring slices of a small step fit L2 with room to spare; a large one would evict its own prefetches
  p.prefetch = (fused && (size_t)B * H * (size_t)r * DAISY_HEAD_DIM * 4 <= ((size_t)48 << 20)) ? 1 : 0;

  cudaStream_t st = (cudaStream_t)stream;
  const bool f16 = (flags & DAISY_CACHE_FP16) != 0;
  const dim3 g1(splits, H, B), g2(H, B);
  if (fused) {                                                     // one launch: the last split CTA of a (batch, head) merges
    using daisy_host::launch_dependent;
    cudaError_t le;
    const int variant = (t_dev ? 4 : 0) | (f16 ? 2 : 0) | (p.prefetch ? 1 : 0);   // small steps: pipelined loads as well
    switch (variant) {
      case 0: le = launch_dependent(swa_decode_partial_kernel<false, false, true, false>, g1, dim3(128), 0, st, p); break;
      case 1: le = launch_dependent(swa_decode_partial_kernel<false, false, true, true>, g1, dim3(128), 0, st, p); break;
      case 2: le = launch_dependent(swa_decode_partial_kernel<false, true, true, false>, g1, dim3(128), 0, st, p); break;
      case 3: le = launch_dependent(swa_decode_partial_kernel<false, true, true, true>, g1, dim3(128), 0, st, p); break;
      case 4: le = launch_dependent(swa_decode_partial_kernel<true, false, true, false>, g1, dim3(128), 0, st, p); break;
      case 5: le = launch_dependent(swa_decode_partial_kernel<true, false, true, true>, g1, dim3(128), 0, st, p); break;
      case 6: le = launch_dependent(swa_decode_partial_kernel<true, true, true, false>, g1, dim3(128), 0, st, p); break;
      default: le = launch_dependent(swa_decode_partial_kernel<true, true, true, true>, g1, dim3(128), 0, st, p); break;
    }
    if (le != cudaSuccess) { (void)cudaGetLastError(); return DAISY_ECUDA; }
    DAISY_CHECK_LAUNCH();
    return DAISY_OK;
  }
  if (t_dev) { if (f16) swa_decode_partial_kernel<true, true, false><<<g1, 128, 0, st>>>(p); else swa_decode_partial_kernel<true, false, false><<<g1, 128, 0, st>>>(p); }
  else       { if (f16) swa_decode_partial_kernel<false, true, false><<<g1, 128, 0, st>>>(p); else swa_decode_partial_kernel<false, false, false><<<g1, 128, 0, st>>>(p); }
  DAISY_CHECK_LAUNCH();
  if (t_dev) { if (f16) swa_decode_combine_kernel<true, true><<<g2, 128, 0, st>>>(p); else swa_decode_combine_kernel<true, false><<<g2, 128, 0, st>>>(p); }
  else       { if (f16) swa_decode_combine_kernel<false, true><<<g2, 128, 0, st>>>(p); else swa_decode_combine_kernel<false, false><<<g2, 128, 0, st>>>(p); }
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}

extern "C" int daisy_b200_swa_decode_step(const void* q_new, const void* k_new, const void* v_new,
                                          int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                                          int64_t v_sb, int64_t v_sh,
                                          void* kcache, void* vcache, int64_t c_sb, int64_t c_sh, int64_t c_sr,
                                          int64_t t, int cap, int window,
                                          const float* cos_row, const float* sin_row,
                                          void* out, int64_t o_sb, int64_t o_sh,
                                          void* k_new_out, void* v_new_out,
                                          int B, int H, int D, float scale, float eps, unsigned flags,
                                          void* workspace, size_t workspace_bytes, int splits,
                                          int* status_word, void* stream) {
  return decode_launch(q_new, k_new, v_new, q_sb, q_sh, k_sb, k_sh, v_sb, v_sh, kcache, vcache, c_sb, c_sh, c_sr,
                       t, nullptr, 0, cap, window, cos_row, sin_row, out, o_sb, o_sh, k_new_out, v_new_out,
                       B, H, D, scale, eps, flags, workspace, workspace_bytes, splits, status_word, stream);
}

extern "C" int daisy_b200_swa_decode_step_dev(const void* q_new, const void* k_new, const void* v_new,
                                              int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                                              int64_t v_sb, int64_t v_sh,
                                              void* kcache, void* vcache, int64_t c_sb, int64_t c_sh, int64_t c_sr,
                                              const int64_t* t_dev, int cap, int window,
                                              const float* cos_table, const float* sin_table, int table_rows,
                                              void* out, int64_t o_sb, int64_t o_sh,
                                              void* k_new_out, void* v_new_out,
                                              int B, int H, int D, float scale, float eps, unsigned flags,
                                              void* workspace, size_t workspace_bytes, int splits,
                                              int* status_word, void* stream) {
  if (!t_dev) return DAISY_EINVAL;
  return decode_launch(q_new, k_new, v_new, q_sb, q_sh, k_sb, k_sh, v_sb, v_sh, kcache, vcache, c_sb, c_sh, c_sr,
                       0, t_dev, table_rows, cap, window, cos_table, sin_table, out, o_sb, o_sh, k_new_out, v_new_out,
                       B, H, D, scale, eps, flags, workspace, workspace_bytes, splits, status_word, stream);
}

extern "C" int daisy_b200_swa_decode_step_fused(const void* q_new, const void* k_new, const void* v_new,
                                                int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                                                int64_t v_sb, int64_t v_sh,
                                                void* kcache, void* vcache, int64_t c_sb, int64_t c_sh, int64_t c_sr,
                                                int64_t t, const int64_t* t_dev, int cap, int window,
                                                const float* cos, const float* sin, int table_rows,
                                                void* out, int64_t o_sb, int64_t o_sh,
                                                void* k_new_out, void* v_new_out,
                                                const void* ve, int64_t ve_sb, int64_t ve_sh, const float* ve_gate_logit,
                                                int B, int H, int D, float scale, float eps, unsigned flags,
                                                void* workspace, size_t workspace_bytes, int splits,
                                                int* status_word, void* stream) {
  return decode_launch(q_new, k_new, v_new, q_sb, q_sh, k_sb, k_sh, v_sb, v_sh, kcache, vcache, c_sb, c_sh, c_sr,
                       t_dev ? 0 : t, t_dev, t_dev ? table_rows : 0, cap, window, cos, sin, out, o_sb, o_sh, k_new_out, v_new_out,
                       B, H, D, scale, eps, flags, workspace, workspace_bytes, splits, status_word, stream,
                       DecodeExtras{true, ve, ve_sb, ve_sh, ve_gate_logit});
}

// ---------------------------------------------------------------------------------------------
// Decode step for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at all: code running between cudaStreamBeginCapture and
// EndCapture of someone else's stream, plugins inside a serving process whose memory is owned entirely by
// a pool allocator that forbids driver allocations after start-up, or a C/Go/Rust embedding that only holds
// the q/k/v and cache pointers it was handed.  The split-KV decode needs a few MB of scratch for its
// per-split partial results; here that scratch is a fixed array inside the library image, so the caller
// passes inputs and outputs only.
//
// The array lives in every GPU context that loads the library until the process exits.  Its device address
// is looked up once per device (cudaGetSymbolAddress with that device current) on the first call made on
// that device; make that first call outside any stream capture.  All calls on a device share the one array:
// two calls whose kernels can overlap on the GPU (different streams, no ordering) race on it.  Nothing in it
// has to be zero at entry -- every partial slot a call reads is written by that same call first.
constexpr int DECODE_STATIC_SLOTS = 4096;                       // (batch x heads x splits) partials: 2.1 MB
static __device__ __align__(256) float g_decode_scratch[DECODE_STATIC_SLOTS * (DAISY_HEAD_DIM + 2)];

extern "C" size_t daisy_b200_swa_decode_static_capacity(void) { return (size_t)DECODE_STATIC_SLOTS; }

extern "C" int daisy_b200_swa_decode_step_static(const void* q_new, const void* k_new, const void* v_new,
                                                 int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                                                 int64_t v_sb, int64_t v_sh,
                                                 void* kcache, void* vcache, int64_t c_sb, int64_t c_sh, int64_t c_sr,
                                                 int64_t t, int cap, int window,
                                                 const float* cos_row, const float* sin_row,
                                                 void* out, int64_t o_sb, int64_t o_sh,
                                                 void* k_new_out, void* v_new_out,
                                                 int B, int H, int D, float scale, float eps, unsigned flags,
                                                 int splits, int* status_word, void* stream) {
  if (B <= 0 || H <= 0 || splits <= 0) return DAISY_EINVAL;
  if ((int64_t)B * H * splits > DECODE_STATIC_SLOTS) return DAISY_EWORKSPACE;   // beyond the built-in scratch
  constexpr int MAX_DEV = 64;
  static float* scratch_addr[MAX_DEV] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) { (void)cudaGetLastError(); return DAISY_ENODEV; }
  if (!scratch_addr[dev]) {
    // In host code the array's name is only a handle; the kernels need its address on THIS device.
    float* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, g_decode_scratch) != cudaSuccess || !ptr) { (void)cudaGetLastError(); return DAISY_ECUDA; }
    scratch_addr[dev] = ptr;
  }
  return daisy_b200_swa_decode_step(q_new, k_new, v_new, q_sb, q_sh, k_sb, k_sh, v_sb, v_sh, kcache, vcache, c_sb, c_sh, c_sr,
                                    t, cap, window, cos_row, sin_row, out, o_sb, o_sh, k_new_out, v_new_out, B, H, D, scale,
                                    eps, flags, scratch_addr[dev], sizeof(g_decode_scratch), splits, status_word, stream);
}
