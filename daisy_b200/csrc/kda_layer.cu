// KDA layer, the two row-wise passes around the attention itself (both HBM-bound, one read and one write per
// element):
//   * the short causal depthwise convolution + SiLU on the q / k / v projections
//       y[t, c] = silu(bias[c] + sum_j w[c, j] * x[t - (W-1) + j, c]),   W <= 4,
//     with the last W inputs carried as a state [B, C, W] between calls (prefill -> decode steps);
//   * the gated RMS norm of the attention output over the head dimension.
#include "common.cuh"

namespace daisy {

constexpr int SC_MAX_W = 4;      // taps
constexpr int SC_TT = 32;        // time steps per thread: the W-1 halo rows are re-read once per 32 rows
constexpr int SC_THREADS = 128;  // thread = 8 adjacent channels (one 16-byte access per row)

struct ShortConvParams {
  const __nv_bfloat16* x;        // [B, T, C], row stride x_st, batch stride x_sb (elements)
  const __nv_bfloat16* w;        // [C, W]
  const __nv_bfloat16* bias;     // [C] or null
  const __nv_bfloat16* s_in;     // [B, C, W] or null (zero history)
  __nv_bfloat16* s_out;          // [B, C, W] or null
  __nv_bfloat16* y;              // [B, T, C], strides y_st, y_sb
  long long x_sb, x_st, y_sb, y_st;
  int T, C, W, silu;
};

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Input at time t (may be negative: the carried state, else zero) for the 8 channels from c0.
__device__ __forceinline__ void conv_input_row(const ShortConvParams& p, int b, int t, int c0, float* f) {
  if (t >= 0) {
    unpack8(*reinterpret_cast<const uint4*>(p.x + (long long)b * p.x_sb + (long long)t * p.x_st + c0), f);
  } else if (p.s_in && p.W + t >= 0) {
    const __nv_bfloat16* s = p.s_in + ((long long)b * p.C + c0) * p.W + (p.W + t);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = __bfloat162float(s[e * p.W]);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = 0.f;
  }
}

__global__ void __launch_bounds__(SC_THREADS) kda_short_conv_kernel(const ShortConvParams p) {
  const int c0 = (blockIdx.z * SC_THREADS + threadIdx.x) * 8;
  if (c0 >= p.C) return;
  const int b = blockIdx.y;
  const int t0 = blockIdx.x * SC_TT;
  const int t1 = min(t0 + SC_TT, p.T);

  // taps right-aligned in four slots: slot 3 multiplies the current row, slot 3-i the row i steps back
  float wt[8][SC_MAX_W];
  if (p.W == 4) {
#pragma unroll
    for (int h = 0; h < 4; ++h) {                                  // 8 channels x 4 taps = 64 contiguous bytes
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(p.w + (long long)c0 * 4 + h * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) wt[h * 2 + i / 4][i % 4] = f[i];
    }
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
      for (int j = 0; j < SC_MAX_W; ++j) {
        const int tap = j - (SC_MAX_W - p.W);
        wt[e][j] = tap >= 0 ? __bfloat162float(p.w[(long long)(c0 + e) * p.W + tap]) : 0.f;
      }
  }
  float bs[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) bs[e] = 0.f;
  if (p.bias) unpack8(*reinterpret_cast<const uint4*>(p.bias + c0), bs);

  float h1[8], h2[8], h3[8];                                       // rows t-1, t-2, t-3
  conv_input_row(p, b, t0 - 1, c0, h1);
  conv_input_row(p, b, t0 - 2, c0, h2);
  conv_input_row(p, b, t0 - 3, c0, h3);

  const __nv_bfloat16* xr = p.x + (long long)b * p.x_sb + c0;
  __nv_bfloat16* yr = p.y + (long long)b * p.y_sb + c0;
  for (int t = t0; t < t1; t += 4) {
    uint4 raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)                                    // four independent 16-byte loads in flight
      raw[i] = (t + i < t1) ? *reinterpret_cast<const uint4*>(xr + (long long)(t + i) * p.x_st) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (t + i >= t1) break;
      float cur[8], o[8];
      unpack8(raw[i], cur);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float a = bs[e];
        a = fmaf(wt[e][0], h3[e], a);
        a = fmaf(wt[e][1], h2[e], a);
        a = fmaf(wt[e][2], h1[e], a);
        a = fmaf(wt[e][3], cur[e], a);
        o[e] = p.silu ? a / (1.f + __expf(-a)) : a;
        h3[e] = h2[e]; h2[e] = h1[e]; h1[e] = cur[e];
      }
      *reinterpret_cast<uint4*>(yr + (long long)(t + i) * p.y_st) =
          make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
    }
  }

  // the CTA that owns the last row leaves the state: the last W inputs, oldest first
  if (p.s_out && t1 == p.T) {
    float st[SC_MAX_W][8];
#pragma unroll
    for (int j = 0; j < SC_MAX_W; ++j)
      if (j < p.W) conv_input_row(p, b, p.T - p.W + j, c0, st[j]);
    __nv_bfloat16* s = p.s_out + ((long long)b * p.C + c0) * p.W;
#pragma unroll
    for (int j = 0; j < SC_MAX_W; ++j)
      if (j < p.W) {
#pragma unroll
        for (int e = 0; e < 8; ++e) s[e * p.W + j] = __float2bfloat16_rn(st[j][e]);
      }
  }
}

// ------------------------------------------------------------------------------------------------ gated norm
constexpr int ON_D = 128;        // head dimension: 16 lanes x 8 elements per row

struct OutNormParams {
  const void* o;                 // [rows, 128] bf16 or fp32
  const __nv_bfloat16* g;        // [rows, 128] gate pre-activation
  const __nv_bfloat16* w;        // [128] or null (ones)
  __nv_bfloat16* y;              // [rows, 128]
  long long rows;
  float eps;
  int o_fp32, mode;
};

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__global__ void __launch_bounds__(256) kda_out_norm_kernel(const OutNormParams p) {
  const int sub = threadIdx.x & 15;                                // lane within the row
  float wv[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) wv[e] = 1.f;
  if (p.w) unpack8(*reinterpret_cast<const uint4*>(p.w + sub * 8), wv);
  const long long stride = (long long)gridDim.x * 16;
  for (long long base = (long long)blockIdx.x * 16; base < p.rows; base += stride) {   // uniform per block: the
    const long long row_raw = base + (threadIdx.x >> 4);                                // shuffles below need whole warps
    const bool valid = row_raw < p.rows;
    const long long row = valid ? row_raw : p.rows - 1;
    float x[8], g[8];
    if (p.o_fp32) {
      const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.o) + row * ON_D + sub * 8);
      const float4 a = src[0], c = src[1];
      x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = c.x; x[5] = c.y; x[6] = c.z; x[7] = c.w;
    } else {
      unpack8(*reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.o) + row * ON_D + sub * 8), x);
    }
    unpack8(*reinterpret_cast<const uint4*>(p.g + row * ON_D + sub * 8), g);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(x[e], x[e], ss);
#pragma unroll
    for (int m = 8; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
    const float rstd = 1.0f / sqrtf(ss * (1.0f / ON_D) + p.eps);
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float n = x[e] * rstd * wv[e];
      const float sg = 1.f / (1.f + __expf(-g[e]));
      if (p.mode == 0)      o[e] = n * sg;                         // sigmoid gate
      else if (p.mode == 1) o[e] = n * g[e] * sg;                  // swish gate
      else                  o[e] = round_bf16(n * g[e] * sg) * round_bf16(sg);   // swish-gated norm (rounded), then x sigmoid
    }
    if (valid)
      *reinterpret_cast<uint4*>(p.y + row * ON_D + sub * 8) =
          make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
  }
}

}  // namespace daisy

using namespace daisy;

extern "C" int daisy_b200_kda_short_conv(const void* x, int64_t x_sb, int64_t x_st, const void* w, const void* bias,
                                         const void* state_in, void* state_out, void* y, int64_t y_sb, int64_t y_st,
                                         int B, int T, int C, int W, unsigned flags, void* stream) {
  if (!x || !w || !y || B <= 0 || T <= 0 || C <= 0) return DAISY_EINVAL;
  if (W < 1 || W > SC_MAX_W || C % 8 != 0 || B > 65535) return DAISY_EUNSUPPORTED;
  if (flags & ~DAISY_KDA_CONV_SILU) return DAISY_EINVAL;
  if (!daisy_aligned16(x) || !daisy_aligned16(y) || !daisy_aligned16(w) || (bias && !daisy_aligned16(bias)) ||
      x_sb % 8 || x_st % 8 || y_sb % 8 || y_st % 8)
    return DAISY_EALIGN;
  // a state updated in place is read by the first time block and written by the last: one block only
  if (state_in && state_in == state_out && T > SC_TT) return DAISY_EINVAL;
  ShortConvParams p;
  p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.bias = (const __nv_bfloat16*)bias;
  p.s_in = (const __nv_bfloat16*)state_in; p.s_out = (__nv_bfloat16*)state_out; p.y = (__nv_bfloat16*)y;
  p.x_sb = x_sb; p.x_st = x_st; p.y_sb = y_sb; p.y_st = y_st;
  p.T = T; p.C = C; p.W = W; p.silu = (flags & DAISY_KDA_CONV_SILU) ? 1 : 0;
  const int groups = C / 8;
  const dim3 grid((T + SC_TT - 1) / SC_TT, B, (groups + SC_THREADS - 1) / SC_THREADS);
  kda_short_conv_kernel<<<grid, SC_THREADS, 0, (cudaStream_t)stream>>>(p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}

extern "C" int daisy_b200_kda_out_norm(const void* o, int o_is_fp32, const void* gate, const void* weight, void* y,
                                       int64_t rows, int D, float eps, int mode, void* stream) {
  if (!o || !gate || !y || rows <= 0 || mode < 0 || mode > 2 || !(eps >= 0.f)) return DAISY_EINVAL;
  if (D != ON_D) return DAISY_EUNSUPPORTED;
  if (!daisy_aligned16(o) || !daisy_aligned16(gate) || !daisy_aligned16(y) || (weight && !daisy_aligned16(weight)))
    return DAISY_EALIGN;
  OutNormParams p;
  p.o = o; p.g = (const __nv_bfloat16*)gate; p.w = (const __nv_bfloat16*)weight; p.y = (__nv_bfloat16*)y;
  p.rows = rows; p.eps = eps; p.o_fp32 = o_is_fp32 ? 1 : 0; p.mode = mode;
  const long long want = (rows + 15) / 16;
  const unsigned grid = (unsigned)(want < 148LL * 16 ? want : 148LL * 16);
  kda_out_norm_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}
