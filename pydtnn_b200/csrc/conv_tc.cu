// Tensor-core engine (tcgen05 / TMEM / TMA). Placeholder until the kernels land: reports no
// supported shape, so AUTO always selects the FMA engine and ENGINE_TENSOR returns UNSUPPORTED.
#include "b2c_common.cuh"
namespace b2c {
bool tc_supported(const Geo&, int) { return false; }
size_t tc_workspace_bytes(const Geo&, int) { return 0; }
int tc_fprop(const Geo&, const void*, const void*, const void*, const b2c_bn_params*, int, void*, void*, size_t, cudaStream_t) { return B2C_ERR_UNSUPPORTED; }
int tc_dgrad(const Geo&, const void*, const void*, void*, void*, size_t, cudaStream_t) { return B2C_ERR_UNSUPPORTED; }
int tc_wgrad(const Geo&, const void*, const void*, void*, void*, void*, size_t, cudaStream_t) { return B2C_ERR_UNSUPPORTED; }
}  // namespace b2c
