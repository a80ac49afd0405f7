// ReadChannels on the device: decoded fp16 channels of one mip to the client's pixels.  The kernels
// follow the reference's CopyImageKernel (src/ImageProcessing.cu:24-71, 220-266); the arithmetic of a
// component is in output_convert.cuh.  Also the two entry points of the C ABI that work on texels
// the caller holds: ntcb_convert_channels and ntcb_read_channels_to_host_noalloc.

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>

#include "container.h"
#include "decode_kernel.h"
#include "error.h"
#include "ntcb.h"
#include "read_channels.h"

namespace ntcb
{
namespace
{

// Converts `numChannels` channels of one decoded mip into a pixel-interleaved destination with
// arbitrary strides: the 1:1 case of the reference's CopyImageKernel (src/ImageProcessing.cu:220-266)
// with the decoded fp16 texels as source.  One thread per texel.
template <int kFormat, bool kLinear>
__global__ void ReadChannelsKernelT(const __half* __restrict__ src, int layout, int width, int height, int channels,
    int firstChannel, int numChannels, OutputConversion conversion, uint8_t* __restrict__ dst, size_t pixelStride,
    size_t rowPitch)
{
    // the format and "every colour space is Linear" are compile-time here: the per-component work of
    // the common requests is a multiply and a rounding, not a chain of run-time switches
    conversion.format = kFormat;
    if (kLinear)
        conversion.srcSpaces = conversion.dstSpaces = 0u;
    const int x = blockIdx.x * blockDim.x + threadIdx.x;
    const int y = blockIdx.y * blockDim.y + threadIdx.y;
    if (x >= width || y >= height)
        return;
    uint8_t* out = dst + size_t(y) * rowPitch + size_t(x) * pixelStride;
    const uint32_t seed = conversion.dither ? DitherSeed(uint32_t(x) + uint32_t(y) * uint32_t(width)) : 0u;
    constexpr int componentBytes = kFormat == kFormatUnorm8 ? 1 : (kFormat == kFormatUnorm16 || kFormat == kFormatFloat16) ? 2 : 4;
    // Channel pairs (even channel, even channel count) are aligned 32-bit words in both layouts.
    const bool pairs = !(firstChannel & 1) && !(channels & 1);
    const size_t texel = layout == kLayoutPlanarPairs ? size_t(y) * width * channels + size_t(x) * 2
                                                       : (size_t(y) * width + x) * channels;
    // The pixel is assembled in registers and stored as whole words when everything is 4-byte
    // aligned (one- and two-byte stores per component otherwise): the kernel moves bytes, nothing else.
    const int pixelBytes = conversion.dstChannels * componentBytes;
    const bool wordStores = !(pixelBytes & 3) && !(pixelStride & 3) && !(rowPitch & 3) && !(reinterpret_cast<uintptr_t>(dst) & 3);
    uint32_t words[kMaxChannels] = {};
    uint32_t pairBits = 0;
#pragma unroll
    for (int c = 0; c < kMaxChannels; ++c)
    {
        if (c >= conversion.dstChannels)
            break;
        const float dither = conversion.dither ? DitherDraw(seed, uint32_t(c) + 1u) : 0.f;
        uint32_t bits;
        if (c < numChannels)
        {
            const int channel = firstChannel + c;
            uint32_t halfBits;
            if (pairs)
            {
                if (!(c & 1))
                {
                    const size_t index = layout == kLayoutPlanarPairs ? texel + size_t(channel) * width : texel + size_t(channel);
                    pairBits = c + 1 < numChannels ? *reinterpret_cast<const uint32_t*>(src + index)
                                                   : uint32_t(__half_as_ushort(src[index]));
                }
                halfBits = (c & 1) ? pairBits >> 16 : pairBits & 0xffffu;
            }
            else
            {
                const size_t index = layout == kLayoutPlanarPairs ? texel + size_t(channel & ~1) * width + (channel & 1)
                                                                   : texel + size_t(channel);
                halfBits = __half_as_ushort(src[index]);
            }
            bits = ConvertComponent(conversion, c, __ushort_as_half(static_cast<unsigned short>(halfBits)), dither);
        }
        else
            bits = DefaultComponent(conversion, c, dither);
        if (!wordStores)
        {
            if (componentBytes == 1)
                out[c] = uint8_t(bits);
            else if (componentBytes == 2)
                reinterpret_cast<uint16_t*>(out)[c] = uint16_t(bits);
            else
                reinterpret_cast<uint32_t*>(out)[c] = bits;
        }
        else if (componentBytes == 1)
            words[c >> 2] |= (bits & 0xffu) << (8 * (c & 3));
        else if (componentBytes == 2)
            words[c >> 1] |= (bits & 0xffffu) << (16 * (c & 1));
        else
            words[c] = bits;
    }
    if (wordStores)
    {
        const int count = pixelBytes >> 2;
        uint32_t* out32 = reinterpret_cast<uint32_t*>(out);
        if (!(count & 3) && !(pixelStride & 15) && !(rowPitch & 15) && !(reinterpret_cast<uintptr_t>(dst) & 15))
        {
#pragma unroll
            for (int w = 0; w < kMaxChannels; w += 4)
                if (w < count)
                    reinterpret_cast<uint4*>(out32)[w >> 2] = make_uint4(words[w], words[w + 1], words[w + 2], words[w + 3]);
        }
        else
        {
#pragma unroll
            for (int w = 0; w < kMaxChannels; ++w)
                if (w < count)
                    out32[w] = words[w];
        }
    }
}

} // namespace

// Launches the instantiation for the request's format.
cudaError_t LaunchReadChannels(dim3 grid, dim3 block, cudaStream_t stream, const __half* src, int layout, int width, int height,
    int channels, int firstChannel, int numChannels, const OutputConversion& conversion, uint8_t* dst, size_t pixelStride,
    size_t rowPitch)
{
    const bool linear = conversion.srcSpaces == 0u && conversion.dstSpaces == 0u;
#define NTCB_READ_CHANNELS_CASE(format)                                                                                  \
    case format:                                                                                                         \
        if (linear)                                                                                                      \
            ReadChannelsKernelT<format, true><<<grid, block, 0, stream>>>(src, layout, width, height, channels, firstChannel, \
                numChannels, conversion, dst, pixelStride, rowPitch);                                                    \
        else                                                                                                             \
            ReadChannelsKernelT<format, false><<<grid, block, 0, stream>>>(src, layout, width, height, channels, firstChannel, \
                numChannels, conversion, dst, pixelStride, rowPitch);                                                    \
        break;
    switch (conversion.format)
    {
        NTCB_READ_CHANNELS_CASE(kFormatUnorm8)
        NTCB_READ_CHANNELS_CASE(kFormatUnorm16)
        NTCB_READ_CHANNELS_CASE(kFormatFloat16)
        NTCB_READ_CHANNELS_CASE(kFormatFloat32)
        NTCB_READ_CHANNELS_CASE(kFormatUint32)
    default:
        return cudaErrorInvalidValue;
    }
#undef NTCB_READ_CHANNELS_CASE
    return cudaGetLastError();
}

namespace
{

// The resizing case of CopyImageKernel (src/ImageProcessing.cu:24-71, 220-266): each output pixel is a
// bilinear blend of up to four source texels, each taken out of its stored colour space first; taps
// of zero weight are not read.  The reference is built with --use_fast_math, so its division is the
// approximate one and its multiply-adds are fused; both are spelled out here.
__global__ void ResizeChannelsKernel(const __half* __restrict__ src, int layout, int srcWidth, int srcHeight, int channels,
    int firstChannel, int numChannels, OutputConversion conversion, uint8_t* __restrict__ dst, int dstWidth, int dstHeight,
    size_t pixelStride, size_t rowPitch)
{
    const int x = blockIdx.x * blockDim.x + threadIdx.x;
    const int y = blockIdx.y * blockDim.y + threadIdx.y;
    if (x >= dstWidth || y >= dstHeight)
        return;
    const float u = ApproxDivide(AddFtz(float(x), 0.5f), float(dstWidth));
    const float v = ApproxDivide(AddFtz(float(y), 0.5f), float(dstHeight));
    const float px = fmaxf(0.f, fminf(AddFtz(float(srcWidth), -1.f), FmaFtz(u, float(srcWidth), -0.5f)));
    const float py = fmaxf(0.f, fminf(AddFtz(float(srcHeight), -1.f), FmaFtz(v, float(srcHeight), -0.5f)));
    const int sx = int(__float2uint_rd(px)), sy = int(__float2uint_rd(py));
    const float fx = AddFtz(px, -floorf(px)), fy = AddFtz(py, -floorf(py));
    const float gx = AddFtz(1.f, -fx), gy = AddFtz(1.f, -fy);
    const float weights[4] = {MulFtz(gx, gy), MulFtz(fx, gy), MulFtz(gx, fy), MulFtz(fx, fy)};

    uint8_t* out = dst + size_t(y) * rowPitch + size_t(x) * pixelStride;
    const uint32_t seed = conversion.dither ? DitherSeed(uint32_t(x) + uint32_t(y) * uint32_t(dstWidth)) : 0u;
    const int componentBytes = BytesPerComponent(conversion.format);
    for (int c = 0; c < conversion.dstChannels; ++c)
    {
        const float dither = conversion.dither ? DitherDraw(seed, uint32_t(c) + 1u) : 0.f;
        float value;
        if (c < numChannels)
        {
            const int channel = firstChannel + c;
            const int srcSpace = (conversion.srcSpaces >> (2 * c)) & 3;
            float taps[4];
#pragma unroll
            for (int t = 0; t < 4; ++t)
            {
                taps[t] = 0.f;
                if (weights[t] > 0.f)
                {
                    const int tx = sx + (t & 1), ty = sy + (t >> 1);
                    const size_t index = layout == kLayoutPlanarPairs
                        ? size_t(ty) * srcWidth * channels + size_t(channel & ~1) * srcWidth + size_t(tx) * 2 + (channel & 1)
                        : (size_t(ty) * srcWidth + tx) * channels + channel;
                    taps[t] = DecodeColorSpace(srcSpace, __half2float(src[index]));
                }
            }
            // a*w0 + b*w1 + c*w2 + d*w3 as the reference build contracts it: the second product is the
            // one that stays a plain multiplication
            value = FmaFtz(taps[3], weights[3], FmaFtz(taps[2], weights[2], FmaFtz(taps[0], weights[0], MulFtz(taps[1], weights[1]))));
            value = EncodeColorSpace((conversion.dstSpaces >> (2 * c)) & 3, value);
        }
        else
            value = c == 3 ? 1.f : 0.f;
        const uint32_t bits = QuantizeComponent(conversion.format, value, dither);
        if (componentBytes == 1)
            out[c] = uint8_t(bits);
        else if (componentBytes == 2)
            reinterpret_cast<uint16_t*>(out)[c] = uint16_t(bits);
        else
            reinterpret_cast<uint32_t*>(out)[c] = bits;
    }
}

} // namespace

cudaError_t LaunchResizeChannels(dim3 grid, dim3 block, cudaStream_t stream, const __half* src, int layout, int srcWidth,
    int srcHeight, int channels, int firstChannel, int numChannels, const OutputConversion& conversion, uint8_t* dst, int dstWidth,
    int dstHeight, size_t pixelStride, size_t rowPitch)
{
    ResizeChannelsKernel<<<grid, block, 0, stream>>>(src, layout, srcWidth, srcHeight, channels, firstChannel, numChannels, conversion,
        dst, dstWidth, dstHeight, pixelStride, rowPitch);
    return cudaGetLastError();
}

OutputConversion Float16Conversion(size_t pixelStride)
{
    OutputConversion conversion{};
    conversion.format = kFormatFloat16;
    conversion.dstChannels = int(std::min<size_t>(pixelStride / 2, size_t(kMaxChannels)));
    return conversion;
}

namespace
{

// Staging area of ntcb_read_channels_to_host_noalloc: part of the library image, so every GPU
// that loads the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_noAllocStaging[NTCB_NOALLOC_STAGING_BYTES];

// Device address of g_noAllocStaging on the current device.  In host code the array's name is
// only a handle for the runtime, not a pointer a kernel can use: the address has to be asked for,
// once per device, with that device current.
int NoAllocStagingAddress(unsigned char** outPointer)
{
    // one slot per device; relaxed atomics: two threads that make their first call together both ask
    // the runtime and store the same address
    static std::atomic<unsigned char*> cache[64];
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess)
        return CudaFailure("cudaGetDevice", err);
    if (device < 0 || device >= 64)
    {
        SetError("CUDA device index %d is out of the supported range.", device);
        return NTCB_ERR_CUDA;
    }
    unsigned char* pointer = cache[device].load(std::memory_order_relaxed);
    if (!pointer)
    {
        void* address = nullptr;
        err = cudaGetSymbolAddress(&address, g_noAllocStaging);
        if (err != cudaSuccess)
            return CudaFailure("cudaGetSymbolAddress", err);
        pointer = static_cast<unsigned char*>(address);
        cache[device].store(pointer, std::memory_order_relaxed);
    }
    *outPointer = pointer;
    return NTCB_OK;
}

} // namespace
} // namespace ntcb

extern "C"
{

int ntcb_read_channels_to_host_noalloc(const void* deviceMip, int layout, int width, int height, int channels,
    int firstChannel, int numChannels, void* hostDestination, size_t pixelStride, size_t rowPitch, void* stream)
{
    using namespace ntcb;
    if (!deviceMip || !hostDestination)
    {
        SetError("deviceMip and hostDestination must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (reinterpret_cast<uintptr_t>(deviceMip) & 3)
    {
        // the gather kernel reads channel pairs as 32-bit words
        SetError("deviceMip must be 4-byte aligned.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if ((layout != NTCB_LAYOUT_PLANAR_PAIRS && layout != NTCB_LAYOUT_INTERLEAVED) || width < 1 || height < 1 ||
        channels < 2 || channels > 16 || (channels & 1))
    {
        SetError("Invalid layout (%d), size (%dx%d) or channel count (%d).", layout, width, height, channels);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (firstChannel < 0 || firstChannel >= channels || numChannels < 1 || numChannels > channels - firstChannel)
    {
        SetError("For the provided firstChannel (%d), numChannels (%d) must be between 1 and %d.", firstChannel, numChannels,
            channels - firstChannel);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (pixelStride < size_t(numChannels) * 2 || rowPitch < pixelStride * size_t(width) || (pixelStride & 1) || (rowPitch & 1))
    {
        SetError("pixelStride (%zu) must hold numChannels fp16 values and rowPitch (%zu) a row of pixels; both must be even.",
            pixelStride, rowPitch);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const size_t bytes = size_t(height) * rowPitch;
    if (bytes > size_t(NTCB_NOALLOC_STAGING_BYTES))
    {
        SetError("The request needs %zu bytes of staging, more than the %zu bytes this entry point owns; read fewer rows "
                 "or channels per call, or use ntcb_texture_set_read_channels.",
            bytes, size_t(NTCB_NOALLOC_STAGING_BYTES));
        return NTCB_ERR_OUT_OF_RANGE;
    }
    unsigned char* staging = nullptr;
    int status = NoAllocStagingAddress(&staging);
    if (status != NTCB_OK)
        return status;
    cudaStream_t cudaStream = static_cast<cudaStream_t>(stream);
    cudaError_t err;
    if (rowPitch > pixelStride * size_t(width) || pixelStride > size_t(numChannels) * 2)
    {
        // the array keeps what the previous call left there: the gaps the kernel does not write must
        // read as zeros
        err = cudaMemsetAsync(staging, 0, bytes, cudaStream);
        if (err != cudaSuccess)
            return CudaFailure("cudaMemsetAsync (staging)", err);
    }
    dim3 block(32, 8);
    dim3 grid((width + block.x - 1) / block.x, (height + block.y - 1) / block.y);
    err = LaunchReadChannels(grid, block, cudaStream, static_cast<const __half*>(deviceMip), layout, width, height, channels,
        firstChannel, numChannels, Float16Conversion(pixelStride), staging, pixelStride, rowPitch);
    if (err != cudaSuccess)
        return CudaFailure("ReadChannelsKernel launch", err);
    CountLaunch();
    err = cudaMemcpyAsync(hostDestination, staging, bytes, cudaMemcpyDeviceToHost, cudaStream);
    if (err != cudaSuccess)
        return CudaFailure("cudaMemcpyAsync (staging)", err);
    err = cudaStreamSynchronize(cudaStream);
    if (err != cudaSuccess)
        return CudaFailure("cudaStreamSynchronize", err);
    ClearError();
    return NTCB_OK;
}

int ntcb_convert_channels(const NtcbConvertParams* params, void* stream)
{
    using namespace ntcb;
    if (!params || !params->deviceMip || !params->deviceDestination)
    {
        SetError("ntcb_convert_channels: params, deviceMip and deviceDestination must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if ((params->layout != NTCB_LAYOUT_PLANAR_PAIRS && params->layout != NTCB_LAYOUT_INTERLEAVED) || params->width < 1 ||
        params->height < 1 || params->channels < 2 || params->channels > NTCB_MAX_CHANNELS || (params->channels & 1))
    {
        SetError("Invalid layout (%d), size (%dx%d) or channel count (%d).", params->layout, params->width, params->height,
            params->channels);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    OutputConversion conversion;
    int status = MakeOutputConversion(params->conversion, params->channels, conversion);
    if (status != NTCB_OK)
        return status;
    if (params->dstWidth < 0 || params->dstHeight < 0 || (params->dstWidth == 0) != (params->dstHeight == 0))
    {
        SetError("dstWidth (%d) and dstHeight (%d) must both be positive, or both 0 for the mip's size.", params->dstWidth,
            params->dstHeight);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    const int dstWidth = params->dstWidth ? params->dstWidth : params->width;
    const int dstHeight = params->dstHeight ? params->dstHeight : params->height;
    const size_t componentBytes = size_t(BytesPerComponent(conversion.format));
    if (params->pixelStride < size_t(conversion.dstChannels) * componentBytes ||
        params->rowPitch < params->pixelStride * size_t(dstWidth) || params->pixelStride % componentBytes ||
        params->rowPitch % componentBytes || reinterpret_cast<uintptr_t>(params->deviceDestination) % componentBytes ||
        (reinterpret_cast<uintptr_t>(params->deviceMip) & 3))
    {
        SetError("pixelStride (%zu) must hold %d components of %zu bytes and rowPitch (%zu) a row of pixels; strides and "
                 "the destination must be multiples of the component size, deviceMip 4-byte aligned.",
            params->pixelStride, conversion.dstChannels, componentBytes, params->rowPitch);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    dim3 block(32, 8);
    dim3 grid((dstWidth + block.x - 1) / block.x, (dstHeight + block.y - 1) / block.y);
    const __half* source = static_cast<const __half*>(params->deviceMip);
    uint8_t* destination = static_cast<uint8_t*>(params->deviceDestination);
    const cudaStream_t cudaStream = static_cast<cudaStream_t>(stream);
    const bool resized = dstWidth != params->width || dstHeight != params->height;
    cudaError_t err = resized
        ? LaunchResizeChannels(grid, block, cudaStream, source, params->layout, params->width, params->height, params->channels,
              params->conversion.firstChannel, params->conversion.numChannels, conversion, destination, dstWidth, dstHeight,
              params->pixelStride, params->rowPitch)
        : LaunchReadChannels(grid, block, cudaStream, source, params->layout, params->width, params->height, params->channels,
              params->conversion.firstChannel, params->conversion.numChannels, conversion, destination, params->pixelStride,
              params->rowPitch);
    if (err != cudaSuccess)
        return CudaFailure("ReadChannelsKernel launch", err);
    CountLaunch();
    ClearError();
    return NTCB_OK;
}

} // extern "C"
