// Library-level entry points and host helpers shared by the kernels' launchers.
#include "common.cuh"

extern "C" int daisy_b200_version(void) { return DAISY_B200_VERSION; }

extern "C" const char* daisy_b200_strerror(int code) {
  switch (code) {
    case DAISY_OK: return "ok";
    case DAISY_EINVAL: return "invalid argument";
    case DAISY_EUNSUPPORTED: return "unsupported shape (head_dim must be 128; KDA needs K=V=128, chunk=64)";
    case DAISY_EALIGN: return "pointer or stride not 16-byte aligned";
    case DAISY_EWORKSPACE: return "workspace too small";
    case DAISY_ECUDA: return "CUDA call failed";
    case DAISY_ETIMEOUT: return "device-side bounded wait ran out";
    case DAISY_ENODEV: return "no sm_100 CUDA device";
    default: return "unknown daisy_b200 status";
  }
}

extern "C" int daisy_b200_sm_count(void) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
  return n;
}

namespace daisy_host {

int device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
  return (dev >= 0 && dev < MAX_DEVICES) ? dev : -1;
}

int sm_count_cached() {
  static int sms[MAX_DEVICES] = {};
  const int d = device_slot();
  if (d < 0) return 0;
  if (sms[d] <= 0) sms[d] = daisy_b200_sm_count();
  return sms[d];
}

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

int make_tmap_bf16_3d(CUtensorMap* m, const void* base, uint64_t n0, uint64_t n1, uint64_t n2,
                      uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return DAISY_ECUDA;
  cuuint64_t dims[3] = {n0, n1, n2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DAISY_OK : DAISY_ECUDA;
}

int make_tmap_bf16_dthb(CUtensorMap* m, const void* base, uint64_t D, uint64_t T, uint64_t H, uint64_t B,
                        uint64_t st_bytes, uint64_t sh_bytes, uint64_t sb_bytes, uint32_t b0, uint32_t b1) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return DAISY_ECUDA;
  cuuint64_t dims[4] = {D, T, H, B};
  cuuint64_t strides[3] = {st_bytes, sh_bytes, sb_bytes};
  cuuint32_t box[4] = {b0, b1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DAISY_OK : DAISY_ECUDA;
}

int make_tmap_rows_bthd(CUtensorMap* m, const void* base, int elem_bytes, uint64_t D, uint64_t T, uint64_t H, uint64_t B,
                        uint32_t rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return DAISY_ECUDA;
  const uint64_t e = (uint64_t)elem_bytes;
  cuuint64_t dims[4] = {D, T, H, B};
  cuuint64_t strides[3] = {H * D * e, D * e, T * H * D * e};
  cuuint32_t box[4] = {(cuuint32_t)D, rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DAISY_OK : DAISY_ECUDA;
}

}  // namespace daisy_host
