// Shape of the decoder network (the reference's MlpDesc, src/MlpDesc.h): four layers,
// 48 -> 64 -> 48 -> 32 -> 16, shared by the weight staging, the container loader and the quantiser.
#pragma once

namespace ntcb
{

constexpr int kMlpLayers = 4;
constexpr int kLayerInputs[kMlpLayers] = {48, 64, 48, 32};
constexpr int kLayerOutputs[kMlpLayers] = {64, 48, 32, 16};
constexpr int kNetworkColumns = 64 + 48 + 32 + 16;                    // outputs of all layers
constexpr int kNetworkWeights = 48 * 64 + 64 * 48 + 48 * 32 + 32 * 16; // weights of all layers

// The same as functions, for device code (a constexpr array cannot be indexed dynamically there).
#ifdef __CUDACC__
__host__ __device__
#endif
constexpr int LayerInputs(int layer)
{
    return layer == 0 ? 48 : layer == 1 ? 64 : layer == 2 ? 48 : 32;
}
#ifdef __CUDACC__
__host__ __device__
#endif
constexpr int LayerOutputs(int layer)
{
    return layer == 0 ? 64 : layer == 1 ? 48 : layer == 2 ? 32 : 16;
}

} // namespace ntcb
