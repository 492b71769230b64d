#include "dst_common.cuh"
namespace dst {
bool decode_supports(const GemmArgs&) { return false; }
int launch_decode(const GemmArgs&, cudaStream_t) { return DST_ERR_UNSUPPORTED; }
}  // namespace dst
