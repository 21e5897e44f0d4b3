// tcgen05 grouped expert GEMMs (placeholder while the kernels are brought up).
#include "moe_kernels.h"
namespace xkb {
bool int4_tc_supported(int, int64_t, int64_t, int64_t, int, int, int) { return false; }
int int4_tc_block(int64_t, int) { return 16; }
int64_t int4_tc_workspace_bytes(int64_t, int64_t, int64_t, int) { return 256; }
int launch_int4_tc(const void*, const int32_t*, const void*, const Routing&, const float*, float*,
                   int64_t, int64_t, int, int, int, void*, cudaStream_t) {
  return fail(XKB_ERR_ARG, "tcgen05 INT4 path not built");
}
bool mxfp4_tc_supported(int, int64_t, int64_t, int64_t, int, int) { return false; }
int mxfp4_tc_block(int64_t, int) { return 16; }
int64_t mxfp4_tc_workspace_bytes(int64_t, int64_t, int64_t, int) { return 256; }
int launch_mxfp4_tc(const void*, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*,
                    const void*, const void*, const Routing&, const float*, __nv_bfloat16*, float*,
                    int64_t, int64_t, int, int, float, int, void*, cudaStream_t) {
  return fail(XKB_ERR_ARG, "tcgen05 MXFP4 path not built");
}
}  // namespace xkb
