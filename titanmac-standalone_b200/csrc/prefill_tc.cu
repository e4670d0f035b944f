// placeholder until the tensor-core kernel lands
#include "tmw_common.cuh"
namespace tmw {
bool prefill_tc_supports(const tmw_prefill_desc&, const void*, const void*, const void*, const void*) { return false; }
int launch_prefill_tc(const tmw_prefill_desc&, const void*, const void*, const void*, void*, cudaStream_t) {
    return TMW_ERR_UNSUPPORTED;
}
}  // namespace tmw
