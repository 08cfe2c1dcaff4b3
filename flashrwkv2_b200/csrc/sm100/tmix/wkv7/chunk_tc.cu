// placeholder until the tensor-core kernel lands
#include "../../common.cuh"
namespace frwkv {
size_t chunk_tc_workspace_bytes(int, int, int) { return 0; }
int launch_chunk_tc(const int32_t*, const int32_t*, const int32_t*, float*, const void*, const void*, const void*,
                    const void*, const void*, const void*, const void*, void*, float*, int, int, int, int, int, float,
                    int, void*, size_t, int32_t*, cudaStream_t) {
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_prefill: tensor-core chunk kernel not built");
}
}  // namespace frwkv
