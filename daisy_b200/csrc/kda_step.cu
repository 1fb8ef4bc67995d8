// KDA layer, the two small pieces either side of the chunked forward:
//   * the log-decay gate  y = -exp(A_log[h]) * softplus(g + bias)   (element-wise, HBM-bound)
//   * the token-by-token recurrence for short inputs (decode steps): the state S [K x V] of one (batch, head)
//     lives in registers of one CTA per 32 value columns, is read once, updated T times and written once.
#include "common.cuh"

namespace daisy {

constexpr int KS_K = 128;          // key / value head dimension
constexpr int KS_VS = 32;          // value columns per CTA
constexpr int KS_THREADS = 128;    // thread = (value column, quarter of the key axis)

// ------------------------------------------------------------------------------------------------ gate
struct KdaGateParams {
  const void* g;            // [rows, H*D] bf16 or fp32
  const float* a_log;       // [H]
  const float* bias;        // [H*D] or null
  float* out;               // [rows, H*D] fp32
  size_t n4;                // rows * H * D / 4
  int HD, D, in_bf16, round_bf16;
  float beta, threshold;
};

__global__ void __launch_bounds__(256) kda_gate_kernel(const KdaGateParams p) {
  const float inv_beta = 1.0f / p.beta;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.n4; i += (size_t)gridDim.x * blockDim.x) {
    const int col = (int)((i * 4) % (size_t)p.HD);                 // D is a multiple of 4: one head per group of four
    float x[4];
    if (p.in_bf16) {
      const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.g) + i * 4);
      x[0] = __uint_as_float(raw.x << 16); x[1] = __uint_as_float(raw.x & 0xffff0000u);
      x[2] = __uint_as_float(raw.y << 16); x[3] = __uint_as_float(raw.y & 0xffff0000u);
    } else {
      const float4 raw = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.g) + i * 4);
      x[0] = raw.x; x[1] = raw.y; x[2] = raw.z; x[3] = raw.w;
    }
    if (p.bias) {
      const float4 bb = *reinterpret_cast<const float4*>(p.bias + col);
      x[0] += bb.x; x[1] += bb.y; x[2] += bb.z; x[3] += bb.w;
    }
    const float a = -expf(p.a_log[col / p.D]);
    float y[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float bx = x[e] * p.beta;
      const float sp = bx > p.threshold ? x[e] : log1pf(expf(bx)) * inv_beta;
      y[e] = a * sp;
      if (p.round_bf16) y[e] = __bfloat162float(__float2bfloat16_rn(y[e]));
    }
    *reinterpret_cast<float4*>(p.out + i * 4) = make_float4(y[0], y[1], y[2], y[3]);
  }
}

// The same gate, eight elements per thread and one pass per thread (no loop), for D % 8 == 0.  The element-wise
// arithmetic, not DRAM, bounds the version above (precise expf + log1pf: 0.4 of the copy bandwidth), so softplus is
// evaluated as  max(z, 0) + log1p(u),  u = exp(-|z|) in (0, 1]  with one ex2.approx and a degree-9 polynomial for
// log1p(u) / u  (Chebyshev interpolant on [0, 1]; 1.6e-7 relative in fp32 arithmetic).
__device__ __forceinline__ float log1p_unit(float u) {
  float r = -0.0031760570127516985f;
  r = fmaf(r, u, 0.019542528316378593f);
  r = fmaf(r, u, -0.05637361481785774f);
  r = fmaf(r, u, 0.10543623566627502f);
  r = fmaf(r, u, -0.1526966691017151f);
  r = fmaf(r, u, 0.1966327428817749f);
  r = fmaf(r, u, -0.24951615929603577f);
  r = fmaf(r, u, 0.33329710364341736f);
  r = fmaf(r, u, -0.49999892711639404f);
  r = fmaf(r, u, 1.0f);
  return r * u;
}

template <bool IN_BF16, bool ROUND>
__global__ void __launch_bounds__(256) kda_gate8_kernel(const KdaGateParams p) {
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;         // group of eight elements
  if (i >= p.n4 / 2) return;
  const int col = (int)((i * 8) % (size_t)p.HD);                   // D % 8 == 0: one head per group
  float x[8];
  if (IN_BF16) {
    unpack8(ld_stream16(reinterpret_cast<const __nv_bfloat16*>(p.g) + i * 8), x);
  } else {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.g) + i * 8);
    const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.g) + i * 8 + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
  if (p.bias) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p.bias + col));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + col + 4));
    x[0] += a.x; x[1] += a.y; x[2] += a.z; x[3] += a.w; x[4] += b.x; x[5] += b.y; x[6] += b.z; x[7] += b.w;
  }
  const float a = -expf(__ldg(p.a_log + col / p.D));
  const float inv_beta = 1.0f / p.beta;
  float y[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float z = x[e] * p.beta;
    const float u = fast_exp2(fabsf(z) * -1.4426950408889634f);
    const float sp = z > p.threshold ? x[e] : (fmaxf(z, 0.f) + log1p_unit(u)) * inv_beta;
    y[e] = a * sp;
    if (ROUND) y[e] = __uint_as_float(pack_bf16(0.f, y[e]) & 0xffff0000u);
  }
  float4* dst = reinterpret_cast<float4*>(p.out + i * 8);
  dst[0] = make_float4(y[0], y[1], y[2], y[3]);
  dst[1] = make_float4(y[4], y[5], y[6], y[7]);
}

// ------------------------------------------------------------------------------------------------ recurrence
struct KdaStepParams {
  const __nv_bfloat16 *q, *k, *v;   // [B,T,H,128]
  const float *g, *beta;            // [B,T,H,128], [B,T,H]
  const float* h0;                  // [B,H,128,128] or null (zero state)
  float* hT;                        // [B,H,128,128] or null; may alias h0
  void* o;                          // [B,T,H,128] bf16 or fp32
  int T, H, out_fp32, l2norm;
  float scale;
};

__global__ void __launch_bounds__(KS_THREADS) kda_recurrent_kernel(const KdaStepParams p) {
  __shared__ float s_k[KS_K], s_q[KS_K], s_d[KS_K];
  __shared__ float s_red[4][KS_VS];
  __shared__ float s_nrm[2][4];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int vcol = blockIdx.x * KS_VS + lane;                      // this thread's value column
  const int h = blockIdx.y, b = blockIdx.z;
  const int k0 = warp * 32;                                        // and its 32 keys
  const size_t bh = (size_t)b * p.H + h;

  float S[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) S[i] = p.h0 ? p.h0[(bh * KS_K + k0 + i) * KS_K + vcol] : 0.f;

  for (int t = 0; t < p.T; ++t) {
    const size_t row = ((size_t)b * p.T + t) * p.H + h;
    // stage this token: thread = channel
    const float kf = __bfloat162float(p.k[row * KS_K + tid]);
    const float qf = __bfloat162float(p.q[row * KS_K + tid]);
    float sk = kf * kf, sq = qf * qf;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) { sk += __shfl_xor_sync(0xffffffffu, sk, o); sq += __shfl_xor_sync(0xffffffffu, sq, o); }
    if (lane == 0) { s_nrm[0][warp] = sk; s_nrm[1][warp] = sq; }
    __syncthreads();                                               // also: every reader of the previous token's stage is done
    const float rk = p.l2norm ? rsqrtf(s_nrm[0][0] + s_nrm[0][1] + s_nrm[0][2] + s_nrm[0][3] + 1e-6f) : 1.f;
    const float rq = p.l2norm ? rsqrtf(s_nrm[1][0] + s_nrm[1][1] + s_nrm[1][2] + s_nrm[1][3] + 1e-6f) : 1.f;
    s_k[tid] = kf * rk;
    s_q[tid] = qf * rq * p.scale;
    s_d[tid] = __expf(p.g[row * KS_K + tid]);
    const float vt = __bfloat162float(p.v[row * KS_K + vcol]);
    const float bt = p.beta[row];
    __syncthreads();
    // S <- diag(e^g) S ;  partial (S^T k)[v]
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) { S[i] *= s_d[k0 + i]; dot = fmaf(S[i], s_k[k0 + i], dot); }
    s_red[warp][lane] = dot;
    __syncthreads();
    const float u = bt * (vt - (s_red[0][lane] + s_red[1][lane] + s_red[2][lane] + s_red[3][lane]));
    __syncthreads();                                               // s_red is reused below
    // S <- S + k u^T ;  partial (S^T q)[v]
    float od = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) { S[i] = fmaf(s_k[k0 + i], u, S[i]); od = fmaf(S[i], s_q[k0 + i], od); }
    s_red[warp][lane] = od;
    __syncthreads();
    if (warp == 0) {
      const float ov = s_red[0][lane] + s_red[1][lane] + s_red[2][lane] + s_red[3][lane];
      if (p.out_fp32) reinterpret_cast<float*>(p.o)[row * KS_K + vcol] = ov;
      else            reinterpret_cast<__nv_bfloat16*>(p.o)[row * KS_K + vcol] = __float2bfloat16_rn(ov);
    }
  }
  if (p.hT) {
#pragma unroll
    for (int i = 0; i < 32; ++i) p.hT[(bh * KS_K + k0 + i) * KS_K + vcol] = S[i];
  }
}

}  // namespace daisy

using namespace daisy;

extern "C" int daisy_b200_kda_gate(const void* g, int g_is_bf16, const float* a_log, const float* bias, float* out,
                                   int64_t rows, int H, int D, float beta, float threshold, unsigned flags,
                                   void* stream) {
  if (!g || !a_log || !out || rows <= 0 || H <= 0 || D <= 0 || !(beta > 0.f)) return DAISY_EINVAL;
  if (D % 4 != 0) return DAISY_EUNSUPPORTED;
  if (flags & ~DAISY_KDA_GATE_ROUND_BF16) return DAISY_EINVAL;
  if (!daisy_aligned16(g) || !daisy_aligned16(out) || (bias && !daisy_aligned16(bias))) return DAISY_EALIGN;
  KdaGateParams p;
  p.g = g; p.a_log = a_log; p.bias = bias; p.out = out;
  p.n4 = (size_t)rows * H * D / 4;
  p.HD = H * D; p.D = D; p.in_bf16 = g_is_bf16 ? 1 : 0; p.round_bf16 = (flags & DAISY_KDA_GATE_ROUND_BF16) ? 1 : 0;
  p.beta = beta; p.threshold = threshold;
  if (D % 8 == 0 && (p.n4 / 2 + 255) / 256 <= 0x7fffffffULL) {
    const unsigned grid8 = (unsigned)((p.n4 / 2 + 255) / 256);
    cudaStream_t st = (cudaStream_t)stream;
    if (p.in_bf16) { if (p.round_bf16) kda_gate8_kernel<true, true><<<grid8, 256, 0, st>>>(p);
                     else              kda_gate8_kernel<true, false><<<grid8, 256, 0, st>>>(p); }
    else           { if (p.round_bf16) kda_gate8_kernel<false, true><<<grid8, 256, 0, st>>>(p);
                     else              kda_gate8_kernel<false, false><<<grid8, 256, 0, st>>>(p); }
    DAISY_CHECK_LAUNCH();
    return DAISY_OK;
  }
  const size_t want = (p.n4 + 255) / 256;
  const unsigned grid = (unsigned)(want < 148u * 16u ? want : 148u * 16u);
  kda_gate_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}

extern "C" int daisy_b200_kda_recurrent_fwd(const void* q, const void* k, const void* v, const float* g,
                                            const float* beta, const float* h0, void* o, float* hT,
                                            int B, int T, int H, int K, int V, float scale, unsigned flags,
                                            void* stream) {
  if (!q || !k || !v || !g || !beta || !o || B <= 0 || T <= 0 || H <= 0) return DAISY_EINVAL;
  if (K != KS_K || V != KS_K) return DAISY_EUNSUPPORTED;
  if (B > 65535 || H > 65535) return DAISY_EUNSUPPORTED;
  if (flags & ~(DAISY_KDA_L2NORM_QK | DAISY_KDA_OUT_FP32)) return DAISY_EINVAL;
  KdaStepParams p;
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
  p.g = g; p.beta = beta; p.h0 = h0; p.hT = hT; p.o = o;
  p.T = T; p.H = H; p.out_fp32 = (flags & DAISY_KDA_OUT_FP32) ? 1 : 0; p.l2norm = (flags & DAISY_KDA_L2NORM_QK) ? 1 : 0;
  p.scale = scale > 0.f ? scale : 1.0f / sqrtf((float)K);
  kda_recurrent_kernel<<<dim3(KS_K / KS_VS, H, B), KS_THREADS, 0, (cudaStream_t)stream>>>(p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}
