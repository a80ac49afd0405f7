// TEST INFRASTRUCTURE ONLY (never linked into the product library).
//
// A plain-C driver around two internal functions of the UNMODIFIED reference library, built from
// the reference's own sources by build_ref.sh: the producers that a compression session runs last
// (src/TextureSet.cpp:1589-1633) and that have no entry point of their own in the public API:
//   ntc::cuda::PackLatents       src/Quantizer.h:48, src/Quantizer.cu:529-541
//   ntc::cuda::QuantizeNetwork   src/Quantizer.h:28, src/Quantizer.cu:305-323
// The driver moves data between plain arrays and the layouts those functions expect (the fp16
// weights live in the reference's MMA-fragment order, addressed through its own
// tin::host::HMatrixB::get_packed_offset); it restates none of their arithmetic.

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <vector>

#include "ChannelInfo.h"
#include "MlpDesc.h"
#include "Quantizer.h"
#include "WeightLayout.h"
#include "tin/tin_matrix_host.h"

namespace ntc::cuda
{
void SetChannelInfos(const ChannelInfo* data, int count); // src/Regression.h:26, src/Regression.cu:49-52
}

namespace
{
thread_local char g_producerError[512];

int Fail(char const* where, cudaError_t error)
{
    std::snprintf(g_producerError, sizeof g_producerError, "%s: %s", where, cudaGetErrorString(error));
    return -1;
}
} // namespace

extern "C"
{

char const* ntcref_producers_last_error()
{
    return g_producerError;
}

// Host arrays in, host array out; `latents` holds `latentCount` fp16 values in the reference's
// quantised-latent layout, `packed` receives width * height * numLayers words.
int ntcref_pack_latents(int width, int height, int numLayers, size_t latentStride, const uint16_t* latents,
    size_t latentCount, uint16_t* packed)
{
    g_producerError[0] = 0;
    const size_t words = size_t(width) * size_t(height) * size_t(numLayers);
    half* deviceLatents = nullptr;
    uint16_t* devicePacked = nullptr;
    cudaError_t error = cudaMalloc(&deviceLatents, latentCount * sizeof(uint16_t));
    if (error == cudaSuccess)
        error = cudaMalloc(&devicePacked, words * sizeof(uint16_t));
    if (error == cudaSuccess)
        error = cudaMemcpy(deviceLatents, latents, latentCount * sizeof(uint16_t), cudaMemcpyHostToDevice);
    if (error == cudaSuccess)
    {
        ntc::cuda::PackLatents(width, height, numLayers, latentStride, deviceLatents, devicePacked);
        error = cudaDeviceSynchronize();
    }
    if (error == cudaSuccess)
        error = cudaMemcpy(packed, devicePacked, words * sizeof(uint16_t), cudaMemcpyDeviceToHost);
    cudaFree(deviceLatents);
    cudaFree(devicePacked);
    return error == cudaSuccess ? 0 : Fail("ntcref_pack_latents", error);
}

// `weights`: fp16 bits, per layer outputs x inputs values with the inputs of one output together;
// `biases`: 160 fp16 values; `outputScale` / `outputBias`: 16 floats each (optimal-to-linear).
// `blob` receives the GenericInt8 or GenericFP8 blob (`blobBytes` must equal the layout's size),
// `roundedWeights` the reference's fp16 copy after quantisation, in the order of `weights`.
int ntcref_quantize_network(const uint16_t* weights, const uint16_t* biases, const float* outputScale,
    const float* outputBias, int useFP8, uint8_t* blob, size_t blobBytes, uint16_t* roundedWeights)
{
    g_producerError[0] = 0;
    ntc::WeightLayout fp16Layout, quantizedLayout;
    ntc::MakeFP16WeightLayout(fp16Layout);
    if (!ntc::MakeQuantizedWeightLayout(nullptr,
            useFP8 ? ntc::InferenceWeightType::GenericFP8 : ntc::InferenceWeightType::GenericInt8, quantizedLayout))
    {
        std::snprintf(g_producerError, sizeof g_producerError, "MakeQuantizedWeightLayout failed");
        return -2;
    }
    if (quantizedLayout.bufferSize != blobBytes)
    {
        std::snprintf(g_producerError, sizeof g_producerError, "blob is %zu bytes in the reference's layout, caller gave %zu",
            quantizedLayout.bufferSize, blobBytes);
        return -3;
    }

    // plain order -> the reference's fragment order
    std::vector<uint16_t> packedHalves(fp16Layout.bufferSize / sizeof(uint16_t), 0);
    size_t plainOffset = 0, biasOffset = 0;
    for (int layer = 0; layer < NTC_MLP_LAYERS; ++layer)
    {
        const int rows = ntc::MlpDesc::GetLayerInputChannels(layer), cols = ntc::MlpDesc::GetLayerOutputChannels(layer);
        tin::host::HMatrixB matrix(rows, cols);
        uint16_t* layerHalves = packedHalves.data() + fp16Layout.weights[layer].offset / sizeof(uint16_t);
        for (int col = 0; col < cols; ++col)
            for (int row = 0; row < rows; row += 2)
            {
                const uint32_t pairIndex = matrix.get_packed_offset(row, col);
                layerHalves[pairIndex * 2 + 0] = weights[plainOffset + size_t(col) * rows + row];
                layerHalves[pairIndex * 2 + 1] = weights[plainOffset + size_t(col) * rows + row + 1];
            }
        uint16_t* layerBiases = packedHalves.data() + fp16Layout.biases[layer].offset / sizeof(uint16_t);
        for (int col = 0; col < cols; ++col)
            layerBiases[col] = biases[biasOffset + col];
        plainOffset += size_t(rows) * cols;
        biasOffset += cols;
    }

    ChannelInfo channelInfos[NTC_MAX_CHANNELS];
    for (int c = 0; c < NTC_MAX_CHANNELS; ++c)
    {
        channelInfos[c].optimalToLinearScale = outputScale[c];
        channelInfos[c].optimalToLinearBias = outputBias[c];
    }
    ntc::cuda::SetChannelInfos(channelInfos, NTC_MAX_CHANNELS);

    half* deviceHalves = nullptr;
    int8_t* deviceBlob = nullptr;
    cudaError_t error = cudaMalloc(&deviceHalves, fp16Layout.bufferSize);
    if (error == cudaSuccess)
        error = cudaMalloc(&deviceBlob, blobBytes);
    if (error == cudaSuccess)
        error = cudaMemset(deviceBlob, 0, blobBytes);
    if (error == cudaSuccess)
        error = cudaMemcpy(deviceHalves, packedHalves.data(), fp16Layout.bufferSize, cudaMemcpyHostToDevice);
    if (error == cudaSuccess)
    {
        ntc::cuda::QuantizeNetwork(fp16Layout, quantizedLayout, deviceHalves, deviceBlob, useFP8 != 0);
        error = cudaDeviceSynchronize();
    }
    if (error == cudaSuccess)
        error = cudaMemcpy(blob, deviceBlob, blobBytes, cudaMemcpyDeviceToHost);
    if (error == cudaSuccess)
        error = cudaMemcpy(packedHalves.data(), deviceHalves, fp16Layout.bufferSize, cudaMemcpyDeviceToHost);
    cudaFree(deviceHalves);
    cudaFree(deviceBlob);
    if (error != cudaSuccess)
        return Fail("ntcref_quantize_network", error);

    // fragment order -> plain order
    plainOffset = 0;
    for (int layer = 0; layer < NTC_MLP_LAYERS && roundedWeights; ++layer)
    {
        const int rows = ntc::MlpDesc::GetLayerInputChannels(layer), cols = ntc::MlpDesc::GetLayerOutputChannels(layer);
        tin::host::HMatrixB matrix(rows, cols);
        const uint16_t* layerHalves = packedHalves.data() + fp16Layout.weights[layer].offset / sizeof(uint16_t);
        for (int col = 0; col < cols; ++col)
            for (int row = 0; row < rows; row += 2)
            {
                const uint32_t pairIndex = matrix.get_packed_offset(row, col);
                roundedWeights[plainOffset + size_t(col) * rows + row] = layerHalves[pairIndex * 2 + 0];
                roundedWeights[plainOffset + size_t(col) * rows + row + 1] = layerHalves[pairIndex * 2 + 1];
            }
        plainOffset += size_t(rows) * cols;
    }
    return 0;
}

} // extern "C"
