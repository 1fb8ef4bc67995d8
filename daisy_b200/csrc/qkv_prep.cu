// q/k/v preparation (RMS norm + RoPE + [B,T,H,D] -> [B,H,T,D]) and ring-buffer row copies.
// Both are pure HBM streaming kernels: eight lanes per 256-byte row, 2 x 16 bytes per lane.
#include "rowops.cuh"

namespace daisy {

struct PrepTensor {
  const __nv_bfloat16* in;
  __nv_bfloat16* out;
  int64_t sb, st, sh;
  int do_norm, do_rope;
  // value-embedding gate (v only): out = g * x + (1 - g) * mix, g = sigmoid(*gate_logit), after the norm
  const __nv_bfloat16* mix;
  int64_t mix_sb, mix_st, mix_sh;
  const float* gate_logit;
};
struct PrepParams {
  PrepTensor t[3];
  const float* cos;
  const float* sin;
  int B, T, H;
  float eps;
  int out_bthd;
};

#ifndef PREP_ROWS_N
#define PREP_ROWS_N 2
#endif
constexpr int PREP_ROWS = PREP_ROWS_N;   // rows per lane group: independent loads in flight per lane
constexpr int PREP_LPR = 8;              // lanes per 256-byte row: 16 bytes of each half of the row per lane

// Lane `sub` of a group of eight owns elements [8 sub, 8 sub + 8) and [64 + 8 sub, 64 + 8 sub + 8) of a row: the
// two halves RoPE pairs together, so the rotation needs no shuffle and two float4 of cos and of sin.
template <bool MIX>
__global__ void __launch_bounds__(256) qkv_prep_kernel(const PrepParams p) {
  const PrepTensor& ten = p.t[blockIdx.y];
  if (ten.in == nullptr) return;
  const int lane = threadIdx.x & 31, sub = lane & (PREP_LPR - 1);
  // 32-bit row arithmetic (the host refuses B*T*H >= 2^31): one division pair per thread, then increments
  const uint32_t rows = (uint32_t)p.B * p.T * p.H;
  const uint32_t row0 = ((blockIdx.x * 256u + threadIdx.x) / PREP_LPR) * PREP_ROWS;
  uint4 lo[PREP_ROWS], hi[PREP_ROWS], mlo[MIX ? PREP_ROWS : 1], mhi[MIX ? PREP_ROWS : 1];
  int hh[PREP_ROWS], tt[PREP_ROWS], bb[PREP_ROWS];
  bool live[PREP_ROWS];
  const uint32_t fast = p.out_bthd ? (uint32_t)p.H : (uint32_t)p.T;   // extent of the fastest row index
  const uint32_t mid = p.out_bthd ? (uint32_t)p.T : (uint32_t)p.H;
  const uint32_t rc = min(row0, rows - 1);
  uint32_t i_fast = rc % fast, rest = rc / fast;
  uint32_t i_mid = rest % mid, i_b = rest / mid;
#pragma unroll
  for (int u = 0; u < PREP_ROWS; ++u) {
    live[u] = row0 + u < rows;
    // rows numbered (b, t, h) when the output keeps [B,T,H,D] (both streams contiguous), else (b, h, t)
    hh[u] = p.out_bthd ? (int)i_fast : (int)i_mid;
    tt[u] = p.out_bthd ? (int)i_mid : (int)i_fast;
    bb[u] = (int)i_b;
    if (row0 + u + 1 < rows) {                     // advance; past the end the last row is repeated
      if (++i_fast == fast) { i_fast = 0; if (++i_mid == mid) { i_mid = 0; ++i_b; } }
    }
    const __nv_bfloat16* src = ten.in + bb[u] * ten.sb + tt[u] * ten.st + hh[u] * ten.sh + 8 * sub;
    lo[u] = ld_stream16(src);
    hi[u] = ld_stream16(src + 64);
    if (MIX && ten.mix) {
      const __nv_bfloat16* ms = ten.mix + bb[u] * ten.mix_sb + tt[u] * ten.mix_st + hh[u] * ten.mix_sh + 8 * sub;
      mlo[MIX ? u : 0] = ld_stream16(ms);
      mhi[MIX ? u : 0] = ld_stream16(ms + 64);
    }
  }
  const float gate = (MIX && ten.mix) ? 1.0f / (1.0f + __expf(-*ten.gate_logit)) : 1.0f;
#pragma unroll
  for (int u = 0; u < PREP_ROWS; ++u) {
    float x1[8], x2[8];
    unpack8(lo[u], x1);
    unpack8(hi[u], x2);
    if (ten.do_norm) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += x1[e] * x1[e] + x2[e] * x2[e];
      ss += __shfl_xor_sync(0xffffffffu, ss, 4);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      const float r = rsqrtf(ss * (1.0f / DAISY_HEAD_DIM) + p.eps);
#pragma unroll
      for (int e = 0; e < 8; ++e) { x1[e] *= r; x2[e] *= r; }
    }
    if (ten.do_rope) {
      const float* cr = p.cos + (int64_t)tt[u] * 64 + 8 * sub;
      const float* sr = p.sin + (int64_t)tt[u] * 64 + 8 * sub;
      const float4 c0 = *reinterpret_cast<const float4*>(cr), c1 = *reinterpret_cast<const float4*>(cr + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sr), s1 = *reinterpret_cast<const float4*>(sr + 4);
      const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float a = x1[e], b2 = x2[e];
        x1[e] = a * c[e] + b2 * s[e];
        x2[e] = b2 * c[e] - a * s[e];
      }
    }
    if (MIX && ten.mix) {
      float m1[8], m2[8];
      unpack8(mlo[MIX ? u : 0], m1);
      unpack8(mhi[MIX ? u : 0], m2);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        x1[e] = gate * x1[e] + (1.0f - gate) * m1[e];
        x2[e] = gate * x2[e] + (1.0f - gate) * m2[e];
      }
    }
    if (live[u]) {
      const int64_t orow = p.out_bthd ? ((int64_t)bb[u] * p.T + tt[u]) * p.H + hh[u]
                                      : ((int64_t)bb[u] * p.H + hh[u]) * p.T + tt[u];
      __nv_bfloat16* dst = ten.out + orow * DAISY_HEAD_DIM + 8 * sub;
      *reinterpret_cast<uint4*>(dst) = pack8(x1);
      *reinterpret_cast<uint4*>(dst + 64) = pack8(x2);
    }
  }
}

struct RingCopyParams {
  char* ring; char* lin;
  int64_t r_sb, r_sh, r_sr, l_sb, l_sh, l_sr;   // in bytes
  int B, H, cap, n, row_bytes, to_ring;
  int64_t first_pos;
};

__global__ void __launch_bounds__(256) ring_copy_kernel(const RingCopyParams p) {
  const int chunks = p.row_bytes >> 4;                       // 16-byte chunks per row
  const int64_t total = (int64_t)p.B * p.H * p.n * chunks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % chunks);
    int64_t r = i / chunks;
    const int row = (int)(r % p.n); r /= p.n;
    const int h = (int)(r % p.H);
    const int b = (int)(r / p.H);
    const int slot = (int)((p.first_pos + row) % p.cap);
    char* a = p.ring + b * p.r_sb + h * p.r_sh + (int64_t)slot * p.r_sr + 16 * c;
    char* l = p.lin + b * p.l_sb + h * p.l_sh + (int64_t)row * p.l_sr + 16 * c;
    if (p.to_ring) *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(l);
    else           *reinterpret_cast<uint4*>(l) = *reinterpret_cast<const uint4*>(a);
  }
}

}  // namespace daisy

using namespace daisy;

static int check_in(const void* p, int64_t sb, int64_t st, int64_t sh) {
  if (!p) return DAISY_OK;
  if (!daisy_aligned16(p) || (sb & 7) || (st & 7) || (sh & 7)) return DAISY_EALIGN;
  return DAISY_OK;
}

extern "C" int daisy_b200_qkv_prep(const void* q, const void* k, const void* v,
                                   int64_t q_sb, int64_t q_st, int64_t q_sh,
                                   int64_t k_sb, int64_t k_st, int64_t k_sh,
                                   int64_t v_sb, int64_t v_st, int64_t v_sh,
                                   const float* cos, const float* sin,
                                   void* q_out, void* k_out, void* v_out,
                                   const void* ve, int64_t ve_sb, int64_t ve_st, int64_t ve_sh, const float* ve_gate_logit,
                                   int B, int T, int H, int D, float eps, unsigned flags, void* stream) {
  if (B <= 0 || T <= 0 || H <= 0) return DAISY_EINVAL;
  if (D != DAISY_HEAD_DIM) return DAISY_EUNSUPPORTED;
  if ((int64_t)B * T * H >= (int64_t)1 << 31) return DAISY_EUNSUPPORTED;
  if ((q == nullptr) != (q_out == nullptr) || (k == nullptr) != (k_out == nullptr) || (v == nullptr) != (v_out == nullptr))
    return DAISY_EINVAL;
  if (!q && !k && !v) return DAISY_EINVAL;
  if ((flags & DAISY_ROPE) && (!cos || !sin)) return DAISY_EINVAL;
  if (ve && (!v || !ve_gate_logit)) return DAISY_EINVAL;
  int rc;
  if ((rc = check_in(ve, ve_sb, ve_st, ve_sh))) return rc;
  if ((rc = check_in(q, q_sb, q_st, q_sh)) || (rc = check_in(k, k_sb, k_st, k_sh)) || (rc = check_in(v, v_sb, v_st, v_sh))) return rc;
  if (!daisy_aligned16(q_out) || !daisy_aligned16(k_out) || !daisy_aligned16(v_out)) return DAISY_EALIGN;
  if ((flags & DAISY_ROPE) && (!daisy_aligned16(cos) || !daisy_aligned16(sin))) return DAISY_EALIGN;
  PrepParams p;
  p.t[0] = {(const __nv_bfloat16*)q, (__nv_bfloat16*)q_out, q_sb, q_st, q_sh, (flags & DAISY_NORM_Q) ? 1 : 0, (flags & DAISY_ROPE) ? 1 : 0, nullptr, 0, 0, 0, nullptr};
  p.t[1] = {(const __nv_bfloat16*)k, (__nv_bfloat16*)k_out, k_sb, k_st, k_sh, (flags & DAISY_NORM_K) ? 1 : 0, (flags & DAISY_ROPE) ? 1 : 0, nullptr, 0, 0, 0, nullptr};
  p.t[2] = {(const __nv_bfloat16*)v, (__nv_bfloat16*)v_out, v_sb, v_st, v_sh, (flags & DAISY_NORM_V) ? 1 : 0, 0,
            (const __nv_bfloat16*)ve, ve_sb, ve_st, ve_sh, ve_gate_logit};
  p.cos = cos; p.sin = sin; p.B = B; p.T = T; p.H = H; p.eps = eps;
  p.out_bthd = (flags & DAISY_OUT_BTHD) ? 1 : 0;
  const int64_t rows = (int64_t)B * T * H;
  const int64_t rows_per_block = (256 / PREP_LPR) * PREP_ROWS;
  dim3 grid((unsigned)((rows + rows_per_block - 1) / rows_per_block), 3, 1);
  if (ve) qkv_prep_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  else    qkv_prep_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}

extern "C" int daisy_b200_ring_copy_rows(void* ring, int64_t r_sb, int64_t r_sh, int64_t r_sr,
                                         void* lin, int64_t l_sb, int64_t l_sh, int64_t l_sr,
                                         int B, int H, int D, int cap, int64_t first_pos, int n,
                                         int elem_bytes, int to_ring, void* stream) {
  if (!ring || !lin || B <= 0 || H <= 0 || D <= 0 || cap <= 0 || n < 0 || first_pos < 0) return DAISY_EINVAL;
  if (elem_bytes != 2 && elem_bytes != 4) return DAISY_EINVAL;
  if (n > cap) return DAISY_EINVAL;                          // rows would alias in the ring
  if (n == 0) return DAISY_OK;
  const int64_t e = elem_bytes;
  if (((int64_t)D * e) & 15) return DAISY_EALIGN;
  if (!daisy_aligned16(ring) || !daisy_aligned16(lin)) return DAISY_EALIGN;
  const int64_t s[6] = {r_sb * e, r_sh * e, r_sr * e, l_sb * e, l_sh * e, l_sr * e};
  for (int i = 0; i < 6; ++i) if (s[i] & 15) return DAISY_EALIGN;
  RingCopyParams p{(char*)ring, (char*)lin, s[0], s[1], s[2], s[3], s[4], s[5], B, H, cap, n, (int)(D * e), to_ring, first_pos};
  const int64_t total = (int64_t)B * H * n * (p.row_bytes >> 4);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  ring_copy_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p);
  DAISY_CHECK_LAUNCH();
  return DAISY_OK;
}
