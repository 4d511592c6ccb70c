#include "kivi_common.cuh"
namespace kivi {
bool decode_mma_supports(const Geom&, int) { return false; }
cudaError_t launch_decode_mma(const DecodeParams&, cudaStream_t) { return cudaErrorNotSupported; }
}
