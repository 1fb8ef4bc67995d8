// Kimi delta attention, chunked forward (placeholder host entry until the kernels land).
#include "common.cuh"

extern "C" size_t daisy_b200_kda_workspace_bytes(int B, int T, int H, int K, int V) {
  (void)B; (void)T; (void)H; (void)K; (void)V;
  return 0;
}

extern "C" int daisy_b200_kda_chunk_fwd(const void* q, const void* k, const void* v, const float* g,
                                        const float* beta, const float* h0, void* o, float* hT,
                                        int B, int T, int H, int K, int V, int chunk, float scale,
                                        unsigned flags, void* workspace, size_t workspace_bytes,
                                        int* status_word, void* stream) {
  (void)q; (void)k; (void)v; (void)g; (void)beta; (void)h0; (void)o; (void)hT; (void)B; (void)T; (void)H;
  (void)K; (void)V; (void)chunk; (void)scale; (void)flags; (void)workspace; (void)workspace_bytes;
  (void)status_word; (void)stream;
  return DAISY_EUNSUPPORTED;
}
