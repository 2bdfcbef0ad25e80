// Attention entry points (placeholder until the kernels land).
#include "common.cuh"
using namespace mgb;
MGB_EXPORT int mograd_b200_flash_attn_fwd(const void*, const void*, const void*, const void*, void*, float*, int64_t,
                                          int64_t, int64_t, int64_t, float, int, int, int, void*) {
  return fail(MGB_EUNSUPPORTED, "flash_attn_fwd: not built yet");
}
MGB_EXPORT size_t mograd_b200_flash_attn_bwd_workspace_bytes(int64_t, int64_t, int64_t, int64_t, int) { return 0; }
MGB_EXPORT int mograd_b200_flash_attn_bwd(const void*, const void*, const void*, const void*, const void*, const void*,
                                          const float*, void*, void*, void*, int64_t, int64_t, int64_t, int64_t, float,
                                          int, int, int, void*, size_t, void*) {
  return fail(MGB_EUNSUPPORTED, "flash_attn_bwd: not built yet");
}
