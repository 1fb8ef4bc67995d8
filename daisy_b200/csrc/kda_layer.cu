// KDA layer, the two row-wise passes around the attention itself (both HBM-bound, one read and one write per
// element):
//   * the short causal depthwise convolution + SiLU on the q / k / v projections
//       y[t, c] = silu(bias[c] + sum_j w[c, j] * x[t - (W-1) + j, c]),   W <= 4,
//     with the last W inputs carried as a state [B, C, W] between calls (prefill -> decode steps);
//   * the gated RMS norm of the attention output over the head dimension.
#include "common.cuh"

namespace daisy {

constexpr int SC_MAX_W = 4;      // taps
constexpr int SC_ROWS = 32;      // output rows per CTA; the tile in shared memory holds 3 more in front (9 % re-read, L2 hits)
constexpr int SC_COLS = 512;     // channels per CTA: 1 KB of a row, 64 16-byte chunks
constexpr int SC_CH = 4;         // channels per thread in the arithmetic phase (8-byte shared-memory reads)
constexpr int SC_SLICES = 2;     // the 32 rows as two slices of 16 consecutive rows per thread
constexpr int SC_THREADS = SC_COLS / SC_CH * SC_SLICES;   // 256
constexpr int SC_TILE_ROWS = SC_ROWS + 3;
constexpr int SC_LOADS = (SC_TILE_ROWS * (SC_COLS / 8) + SC_THREADS - 1) / SC_THREADS;   // 16-byte loads per thread: 9

struct ShortConvParams {
  const __nv_bfloat16* x;        // [B, T, C], row stride x_st, batch stride x_sb (elements)
  const __nv_bfloat16* w;        // [C, W]
  const __nv_bfloat16* bias;     // [C] or null
  const __nv_bfloat16* s_in;     // [B, C, W] or null (zero history)
  __nv_bfloat16* s_out;          // [B, C, W] or null
  __nv_bfloat16* y;              // [B, T, C], strides y_st, y_sb
  long long x_sb, x_st, y_sb, y_st;
  int T, C, W, silu;
  const int2* tok;               // packed sequences (B = 1): per token (first token of its sequence, sequence index), else null;
                                 // s_in / s_out are then [n_seq, C, W]
};

__device__ __forceinline__ void unpack4(const uint2 u, float* f) {
  f[0] = bf16_lo(u.x); f[1] = bf16_hi(u.x); f[2] = bf16_lo(u.y); f[3] = bf16_hi(u.y);
}
// 1 / (1 + 2^(-a log2 e)): one multiply, one add and the two special-function instructions, nothing else
__device__ __forceinline__ float fast_sigmoid(float a) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + fast_exp2(a * -1.4426950408889634f)));
  return r;
}

// The 8 channels from c at time t < 0: the carried state, else zeros.
__device__ __forceinline__ uint4 conv_state_row(const ShortConvParams& p, int b, int t, int c) {
  float f[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] = 0.f;
  if (p.s_in && p.W + t >= 0) {
    const __nv_bfloat16* s = p.s_in + ((long long)b * p.C + c) * p.W + (p.W + t);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = __bfloat162float(s[e * p.W]);
  }
  return pack8(f);
}

// Phase 1: the CTA's tile of x (35 rows x 1 KB) goes to shared memory with coalesced 16-byte loads, all of a thread's
// loads in flight before the first is used.  Phase 2: thread = 4 channels x 16 consecutive rows, sliding the taps'
// window through registers, one 8-byte shared-memory read and one 8-byte store per row.
// Packed sequences: the window never crosses a sequence's first token -- the inputs before it are that sequence's
// carried state (or zeros), patched into the sliding registers at the first three rows of each sequence -- and the row
// that ends a sequence leaves that sequence's state.
template <bool SILU, bool VARLEN>
__global__ void __launch_bounds__(SC_THREADS) kda_short_conv_kernel(const ShortConvParams p) {
  __shared__ uint4 tile[SC_TILE_ROWS][SC_COLS / 8];
  const int cblk = blockIdx.x * SC_COLS;                           // channel blocks vary fastest, then time blocks:
  const int b = blockIdx.z;                                        // CTAs launched together walk the tensor front to back
  const int tblk = blockIdx.y * SC_ROWS;
  const int t_end = min(tblk + SC_ROWS, p.T);

  uint4 v[SC_LOADS];
  const __nv_bfloat16* xb = p.x + (long long)b * p.x_sb;
#pragma unroll
  for (int i = 0; i < SC_LOADS; ++i) {
    const int idx = i * SC_THREADS + threadIdx.x;
    const int r = idx / (SC_COLS / 8), c = cblk + (idx % (SC_COLS / 8)) * 8, t = tblk - 3 + r;
    v[i] = make_uint4(0, 0, 0, 0);
    if (r < SC_TILE_ROWS && c < p.C) {
      if (t >= 0) { if (t < t_end) v[i] = ld_stream16(xb + (long long)t * p.x_st + c); }
      else if (!VARLEN) v[i] = conv_state_row(p, b, t, c);
    }
  }
#pragma unroll
  for (int i = 0; i < SC_LOADS; ++i) {
    const int idx = i * SC_THREADS + threadIdx.x;
    if (idx < SC_TILE_ROWS * (SC_COLS / 8)) tile[idx / (SC_COLS / 8)][idx % (SC_COLS / 8)] = v[i];
  }

  const int cg = threadIdx.x % (SC_COLS / SC_CH), slice = threadIdx.x / (SC_COLS / SC_CH);
  const int c0 = cblk + cg * SC_CH;
  const bool have = c0 < p.C;
  // taps right-aligned in four slots: slot 3 multiplies the current row, slot 3-i the row i steps back
  float wt[SC_CH][SC_MAX_W], bs[SC_CH];
#pragma unroll
  for (int e = 0; e < SC_CH; ++e) {
    bs[e] = 0.f;
#pragma unroll
    for (int j = 0; j < SC_MAX_W; ++j) wt[e][j] = 0.f;
  }
  if (have) {
    if (p.W == 4) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {                                // 4 channels x 4 taps = 32 contiguous bytes
        float f[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(p.w + (long long)c0 * 4 + h * 8)), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) wt[h * 2 + i / 4][i % 4] = f[i];
      }
    } else {
#pragma unroll
      for (int e = 0; e < SC_CH; ++e)
#pragma unroll
        for (int j = 0; j < SC_MAX_W; ++j) {
          const int tap = j - (SC_MAX_W - p.W);
          if (tap >= 0) wt[e][j] = __bfloat162float(p.w[(long long)(c0 + e) * p.W + tap]);
        }
    }
    if (p.bias) {
#pragma unroll
      for (int e = 0; e < SC_CH; ++e) bs[e] = __bfloat162float(p.bias[c0 + e]);
    }
  }
  __syncthreads();
  if (!have) return;

  const uint2* col = reinterpret_cast<const uint2*>(&tile[0][0]) + cg;      // row stride: SC_COLS / 4 uint2
  constexpr int RS = SC_COLS / SC_CH;
  constexpr int PER = SC_ROWS / SC_SLICES;
  const int r0 = slice * PER;                                      // tile row of input t-3 for this slice's first output
  float h1[SC_CH], h2[SC_CH], h3[SC_CH];                           // rows t-1, t-2, t-3
  unpack4(col[(r0 + 0) * RS], h3); unpack4(col[(r0 + 1) * RS], h2); unpack4(col[(r0 + 2) * RS], h1);
  __nv_bfloat16* yr = p.y + (long long)b * p.y_sb + c0;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int t = tblk + r0 + i;
    float cur[SC_CH], o[SC_CH];
    unpack4(col[(r0 + 3 + i) * RS], cur);
    int2 tk = make_int2(0, 0);
    if (VARLEN && t < t_end) {
      tk = __ldg(p.tok + t);
      if (t - 3 < tk.x) {                                          // one of the three rows back lies before this sequence
        const __nv_bfloat16* s = p.s_in ? p.s_in + ((long long)tk.y * p.C + c0) * p.W : nullptr;
#pragma unroll
        for (int e = 0; e < SC_CH; ++e) {
          const int o1 = p.W + (t - 1 - tk.x), o2 = o1 - 1, o3 = o1 - 2;     // slot in the state of rows t-1, t-2, t-3
          if (t - 1 < tk.x) h1[e] = (s && o1 >= 0) ? __bfloat162float(s[e * p.W + o1]) : 0.f;
          if (t - 2 < tk.x) h2[e] = (s && o2 >= 0) ? __bfloat162float(s[e * p.W + o2]) : 0.f;
          if (t - 3 < tk.x) h3[e] = (s && o3 >= 0) ? __bfloat162float(s[e * p.W + o3]) : 0.f;
        }
      }
    }
    float old3[SC_CH];
#pragma unroll
    for (int e = 0; e < SC_CH; ++e) {
      float a = bs[e];
      a = fmaf(wt[e][0], h3[e], a);
      a = fmaf(wt[e][1], h2[e], a);
      a = fmaf(wt[e][2], h1[e], a);
      a = fmaf(wt[e][3], cur[e], a);
      o[e] = SILU ? a * fast_sigmoid(a) : a;
      old3[e] = h3[e];
      h3[e] = h2[e]; h2[e] = h1[e]; h1[e] = cur[e];
    }
    if (t < t_end)
      *reinterpret_cast<uint2*>(yr + (long long)t * p.y_st) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
    if (VARLEN && p.s_out && t < t_end && (t == p.T - 1 || __ldg(p.tok + t + 1).x == t + 1)) {
      __nv_bfloat16* s = p.s_out + ((long long)tk.y * p.C + c0) * p.W;         // the sequence ends here: rows t-W+1 .. t
#pragma unroll
      for (int e = 0; e < SC_CH; ++e) {
        const float last[4] = {old3[e], h3[e], h2[e], h1[e]};
        for (int j = 0; j < p.W; ++j) s[e * p.W + j] = __float2bfloat16_rn(last[4 - p.W + j]);
      }
    }
  }
  if (VARLEN) return;

  // the CTA that owns the last row leaves the state: the last W inputs, oldest first (tile row of input t: t - tblk + 3)
  if (p.s_out && t_end == p.T && slice == 0) {
    __nv_bfloat16* s = p.s_out + ((long long)b * p.C + c0) * p.W;
    for (int j = 0; j < p.W; ++j) {
      float f[SC_CH];
      unpack4(col[(p.T - p.W + j - tblk + 3) * RS], f);
#pragma unroll
      for (int e = 0; e < SC_CH; ++e) s[e * p.W + j] = __float2bfloat16_rn(f[e]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ gated norm
constexpr int ON_D = 128;        // head dimension: 16 lanes x 8 elements per row

struct OutNormParams {
  const void* o;                 // [rows, 128] bf16 or fp32
  const __nv_bfloat16* g;        // [rows, 128] gate pre-activation
  const __nv_bfloat16* w;        // [128] or null (ones)
  const __nv_bfloat16* gbias;    // [H, 128] or null: added to the gate (row r belongs to head r % H), rounded to bf16
  int H;
  __nv_bfloat16* y;              // [rows, 128]
  long long rows;
  float eps;
  int o_fp32, mode;
};

constexpr int ON_LPR = 8;        // lanes per row: elements [8 sub, 8 sub + 8) and [64 + 8 sub, 64 + 8 sub + 8)

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {       // one rounding per lane, like a bf16 tensor product
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Gate combination for eight elements -> four packed bf16 pairs.  The exp / reciprocal / conversion unit is what this
// kernel saturates first, so the two-factor mode rounds in pairs (one conversion per two values) and multiplies the
// rounded factors as packed bf16, which is exactly bf16(bf16(n g s) * bf16(s)).
template <int MODE>
__device__ __forceinline__ uint4 gate8(const float* n, const float* g) {
  uint32_t out[4];
#pragma unroll
  for (int e = 0; e < 8; e += 2) {
    const float s0 = fast_sigmoid(g[e]), s1 = fast_sigmoid(g[e + 1]);
    if (MODE == 0)      out[e / 2] = pack_bf16(n[e] * s0, n[e + 1] * s1);
    else if (MODE == 1) out[e / 2] = pack_bf16(n[e] * g[e] * s0, n[e + 1] * g[e + 1] * s1);
    else                out[e / 2] = mul_bf16x2(pack_bf16(n[e] * g[e] * s0, n[e + 1] * g[e + 1] * s1), pack_bf16(s0, s1));
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

// One pass per thread (one row per group of eight lanes), no loop: the block scheduler keeps the memory system fed.
template <int MODE, bool O32>
__global__ void __launch_bounds__(256) kda_out_norm_kernel(const OutNormParams p) {
  const int sub = threadIdx.x & (ON_LPR - 1);
  const long long row_raw = ((long long)blockIdx.x * 256 + threadIdx.x) / ON_LPR;
  const bool live = row_raw < p.rows;
  const long long row = live ? row_raw : p.rows - 1;               // past the end the last row is repeated: the
  float x1[8], x2[8], g1[8], g2[8];                                // shuffles below need whole warps
  if (O32) {
    const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.o) + row * ON_D + 8 * sub);
    const float4 a = src[0], b = src[1], c = src[16], d = src[17];
    x1[0] = a.x; x1[1] = a.y; x1[2] = a.z; x1[3] = a.w; x1[4] = b.x; x1[5] = b.y; x1[6] = b.z; x1[7] = b.w;
    x2[0] = c.x; x2[1] = c.y; x2[2] = c.z; x2[3] = c.w; x2[4] = d.x; x2[5] = d.y; x2[6] = d.z; x2[7] = d.w;
  } else {
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(p.o) + row * ON_D + 8 * sub;
    const uint4 a = ld_stream16(src), c = ld_stream16(src + 64);
    unpack8(a, x1); unpack8(c, x2);
  }
  {
    const uint4 a = ld_stream16(p.g + row * ON_D + 8 * sub), c = ld_stream16(p.g + row * ON_D + 64 + 8 * sub);
    unpack8(a, g1); unpack8(c, g2);
  }
  if (p.gbias) {                                                   // the bias of the gate's projection, as its Linear adds it
    const __nv_bfloat16* bsrc = p.gbias + (row % p.H) * ON_D + 8 * sub;
    float b1[8], b2[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(bsrc)), b1);
    unpack8(__ldg(reinterpret_cast<const uint4*>(bsrc + 64)), b2);
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      const uint32_t r1 = pack_bf16(g1[e] + b1[e], g1[e + 1] + b1[e + 1]), r2 = pack_bf16(g2[e] + b2[e], g2[e + 1] + b2[e + 1]);
      g1[e] = bf16_lo(r1); g1[e + 1] = bf16_hi(r1); g2[e] = bf16_lo(r2); g2[e + 1] = bf16_hi(r2);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += x1[e] * x1[e] + x2[e] * x2[e];
  ss += __shfl_xor_sync(0xffffffffu, ss, 4);
  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  const float rstd = rsqrtf(ss * (1.0f / ON_D) + p.eps);
  if (p.w) {
    float w1[8], w2[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(p.w + 8 * sub)), w1);
    unpack8(__ldg(reinterpret_cast<const uint4*>(p.w + 64 + 8 * sub)), w2);
#pragma unroll
    for (int e = 0; e < 8; ++e) { x1[e] *= rstd * w1[e]; x2[e] *= rstd * w2[e]; }
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) { x1[e] *= rstd; x2[e] *= rstd; }
  }
  if (live) {
    __nv_bfloat16* dst = p.y + row * ON_D + 8 * sub;
    *reinterpret_cast<uint4*>(dst) = gate8<MODE>(x1, g1);
    *reinterpret_cast<uint4*>(dst + 64) = gate8<MODE>(x2, g2);
  }
}

template <int MODE>
static void launch_out_norm(const OutNormParams& p, unsigned grid, cudaStream_t st) {
  if (p.o_fp32) kda_out_norm_kernel<MODE, true><<<grid, 256, 0, st>>>(p);
  else          kda_out_norm_kernel<MODE, false><<<grid, 256, 0, st>>>(p);
}

}  // namespace daisy

using namespace daisy;

extern "C" int daisy_b200_kda_short_conv(const void* x, int64_t x_sb, int64_t x_st, const void* w, const void* bias,
                                         const void* state_in, void* state_out, void* y, int64_t y_sb, int64_t y_st,
                                         int B, int T, int C, int W, unsigned flags, void* stream) {
  if (!x || !w || !y || B <= 0 || T <= 0 || C <= 0) return DAISY_EINVAL;
  if (W < 1 || W > SC_MAX_W || C % 8 != 0 || B > 65535 || (T + SC_ROWS - 1) / SC_ROWS > 65535) return DAISY_EUNSUPPORTED;
  if (flags & ~DAISY_KDA_CONV_SILU) return DAISY_EINVAL;
  if (!daisy_aligned16(x) || !daisy_aligned16(y) || !daisy_aligned16(w) || (bias && !daisy_aligned16(bias)) ||
      x_sb % 8 || x_st % 8 || y_sb % 8 || y_st % 8)
    return DAISY_EALIGN;
  // a state updated in place is read by the threads of the first rows and written by the CTA of the last: one CTA only
  if (state_in && state_in == state_out && T > SC_ROWS) return DAISY_EINVAL;
  ShortConvParams p;
  p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.bias = (const __nv_bfloat16*)bias;
  p.s_in = (const __nv_bfloat16*)state_in; p.s_out = (__nv_bfloat16*)state_out; p.y = (__nv_bfloat16*)y;
  p.x_sb = x_sb; p.x_st = x_st; p.y_sb = y_sb; p.y_st = y_st;
  p.T = T; p.C = C; p.W = W; p.silu = (flags & DAISY_KDA_CONV_SILU) ? 1 : 0;
  p.tok = nullptr;
  const dim3 grid((C + SC_COLS - 1) / SC_COLS, (T + SC_ROWS - 1) / SC_ROWS, B);
  if (p.silu) kda_short_conv_kernel<true, false><<<grid, SC_THREADS, 0, (cudaStream_t)stream>>>(p);
  else        kda_short_conv_kernel<false, false><<<grid, SC_THREADS, 0, (cudaStream_t)stream>>>(p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}

extern "C" int daisy_b200_kda_short_conv_varlen(const void* x, int64_t x_st, const void* w, const void* bias,
                                                const void* state_in, void* state_out, void* y, int64_t y_st,
                                                int T, int C, int W, const int32_t* tok_tab, unsigned flags, void* stream) {
  if (!x || !w || !y || !tok_tab || T <= 0 || C <= 0) return DAISY_EINVAL;
  if (W < 1 || W > SC_MAX_W || C % 8 != 0 || (T + SC_ROWS - 1) / SC_ROWS > 65535) return DAISY_EUNSUPPORTED;
  if (flags & ~DAISY_KDA_CONV_SILU) return DAISY_EINVAL;
  if (!daisy_aligned16(x) || !daisy_aligned16(y) || !daisy_aligned16(w) || (bias && !daisy_aligned16(bias)) ||
      x_st % 8 || y_st % 8 || (reinterpret_cast<uintptr_t>(tok_tab) & 7))
    return DAISY_EALIGN;
  if (state_in && state_in == state_out) return DAISY_EINVAL;     // sequences end in different CTAs
  ShortConvParams p;
  p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.bias = (const __nv_bfloat16*)bias;
  p.s_in = (const __nv_bfloat16*)state_in; p.s_out = (__nv_bfloat16*)state_out; p.y = (__nv_bfloat16*)y;
  p.x_sb = 0; p.x_st = x_st; p.y_sb = 0; p.y_st = y_st;
  p.T = T; p.C = C; p.W = W; p.silu = (flags & DAISY_KDA_CONV_SILU) ? 1 : 0;
  p.tok = reinterpret_cast<const int2*>(tok_tab);
  const dim3 grid((C + SC_COLS - 1) / SC_COLS, (T + SC_ROWS - 1) / SC_ROWS, 1);
  if (p.silu) kda_short_conv_kernel<true, true><<<grid, SC_THREADS, 0, (cudaStream_t)stream>>>(p);
  else        kda_short_conv_kernel<false, true><<<grid, SC_THREADS, 0, (cudaStream_t)stream>>>(p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}

extern "C" int daisy_b200_kda_out_norm(const void* o, int o_is_fp32, const void* gate, const void* gate_bias, int H,
                                       const void* weight, void* y, int64_t rows, int D, float eps, int mode,
                                       void* stream) {
  if (!o || !gate || !y || rows <= 0 || mode < 0 || mode > 2 || !(eps >= 0.f)) return DAISY_EINVAL;
  if (gate_bias && (H <= 0 || rows % H != 0)) return DAISY_EINVAL;
  if (D != ON_D) return DAISY_EUNSUPPORTED;
  if (!daisy_aligned16(o) || !daisy_aligned16(gate) || !daisy_aligned16(y) || (weight && !daisy_aligned16(weight)) ||
      (gate_bias && !daisy_aligned16(gate_bias)))
    return DAISY_EALIGN;
  OutNormParams p;
  p.o = o; p.g = (const __nv_bfloat16*)gate; p.w = (const __nv_bfloat16*)weight; p.y = (__nv_bfloat16*)y;
  p.gbias = (const __nv_bfloat16*)gate_bias; p.H = gate_bias ? H : 1;
  p.rows = rows; p.eps = eps; p.o_fp32 = o_is_fp32 ? 1 : 0; p.mode = mode;
  const long long rows_per_cta = 256 / ON_LPR;
  const long long want = (rows + rows_per_cta - 1) / rows_per_cta;
  if (want > 0x7fffffffLL) return DAISY_EUNSUPPORTED;
  const unsigned grid = (unsigned)want;
  if (mode == 0)      launch_out_norm<0>(p, grid, (cudaStream_t)stream);
  else if (mode == 1) launch_out_norm<1>(p, grid, (cudaStream_t)stream);
  else                launch_out_norm<2>(p, grid, (cudaStream_t)stream);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}
