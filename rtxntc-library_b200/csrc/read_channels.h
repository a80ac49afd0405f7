// The conversion kernels behind ReadChannels: decoded fp16 channels to the client's pixels (1:1 and
// with the reference's bilinear resize).  Implemented in read_channels.cu.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "output_convert.cuh"

namespace ntcb
{

// One thread per destination pixel; grid and block cover the destination.
cudaError_t LaunchReadChannels(dim3 grid, dim3 block, cudaStream_t stream, const __half* src, int layout, int width, int height,
    int channels, int firstChannel, int numChannels, const OutputConversion& conversion, uint8_t* dst, size_t pixelStride,
    size_t rowPitch);
cudaError_t LaunchResizeChannels(dim3 grid, dim3 block, cudaStream_t stream, const __half* src, int layout, int srcWidth,
    int srcHeight, int channels, int firstChannel, int numChannels, const OutputConversion& conversion, uint8_t* dst, int dstWidth,
    int dstHeight, size_t pixelStride, size_t rowPitch);

// Plain FLOAT16 read-out: linear to linear, no dithering.
OutputConversion Float16Conversion(size_t pixelStride);

} // namespace ntcb
