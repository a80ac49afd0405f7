// BC4 / BC5 encoding of decoded texels: the "decompress on load, then block-compress" step that the
// reference runs as compute shaders through a graphics API (IContext::MakeBlockCompressionComputePass,
// src/Context.cpp:630-779; src/shaders/CompressBC4.hlsl, CompressBC5.hlsl and BC4_CompressFast in
// src/shaders/BlockCompressCommon.hlsli:510-796), here as a CUDA kernel on the decode output.
//
// The encoder follows the shader's algorithm: quantise the 16 values to 8 bits; start from endpoints
// pulled 1/34 of the range inwards (pinned to 0 / 255 when the block touches them); alternate
// nearest-palette index assignment with a least-squares refit of the endpoints, at most eight times,
// while the squared error falls; do the same for the six-interpolant mode (explicit 0 and 255);
// keep the better of the two.  One thread per 4x4 block, as in the shader.
//
// Arithmetic notes.  The refits use binary32 in the shader's order of operations, written with
// explicit round-to-nearest multiplies and adds so that nothing is fused; `round` is HLSL's round
// (half to even); a NaN or infinity from a singular refit goes through clamp as in the shader
// (max(NaN, 0) = 0).  Squared errors are sums of at most 16 integers below 2^16, exact in binary32,
// so they are kept as integers here.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "error.h"
#include "ntcb.h"

namespace ntcb
{
namespace
{

struct Bc4Block
{
    uint32_t alpha0, alpha1; // 8-bit endpoints (the shader masks what it stores to 8 bits)
    uint64_t indices;        // 3 bits per pixel, pixel 0 in the lowest bits
};

__device__ __forceinline__ uint32_t IndexOf(const Bc4Block& block, int pixel)
{
    return uint32_t(block.indices >> (3 * pixel)) & 7u;
}

// The eight palette entries two endpoints stand for (BC4_EvaluatePalette, :563-603).
__device__ __forceinline__ void Palette(uint32_t a0, uint32_t a1, uint32_t (&palette)[8])
{
    palette[0] = a0;
    palette[1] = a1;
    if (a0 > a1)
    {
#pragma unroll
        for (uint32_t k = 1; k <= 6; ++k)
            palette[k + 1] = ((7 - k) * a0 + k * a1 + 3) / 7;
    }
    else
    {
#pragma unroll
        for (uint32_t k = 1; k <= 4; ++k)
            palette[k + 1] = ((5 - k) * a0 + k * a1 + 2) / 5;
        palette[6] = 0;
        palette[7] = 255;
    }
}

// Nearest palette entry per pixel, the first one on ties; returns the block's squared error
// (BC4_ComputeAlphaIndices, :605-632).
__device__ uint32_t AssignIndices(const uint32_t (&values)[16], Bc4Block& block)
{
    uint32_t palette[8];
    Palette(block.alpha0, block.alpha1, palette);
    uint64_t indices = 0;
    uint32_t total = 0;
#pragma unroll
    for (int pixel = 0; pixel < 16; ++pixel)
    {
        int best = 0x7fffffff;
        uint32_t bestIndex = 0;
#pragma unroll
        for (uint32_t p = 0; p < 8; ++p)
        {
            const int difference = int(values[pixel]) - int(palette[p]);
            const int distance = difference * difference;
            if (distance < best)
            {
                best = distance;
                bestIndex = p;
            }
        }
        total += uint32_t(best);
        indices |= uint64_t(bestIndex) << (3 * pixel);
    }
    block.indices = indices;
    return total;
}

// Weight of endpoint 0 in each palette entry: 1 - index for the endpoints, (8 - index) / 7 or
// (6 - index) / 5 for the interpolants, the quotients rounded to binary32 as a division at run time
// would round them.
__constant__ float kWeightEight[8] = {1.f, 0.f, 6.f / 7.f, 5.f / 7.f, 4.f / 7.f, 3.f / 7.f, 2.f / 7.f, 1.f / 7.f};
__constant__ float kWeightSix[8] = {1.f, 0.f, 4.f / 5.f, 3.f / 5.f, 2.f / 5.f, 1.f / 5.f, 0.f, 0.f};

struct RefitSums
{
    float alpha2 = 0.f, beta2 = 0.f, alphaBeta = 0.f, alphaX = 0.f, betaX = 0.f;

    __device__ __forceinline__ void Add(float alpha, float value)
    {
        const float beta = __fsub_rn(1.f, alpha);
        alpha2 = __fadd_rn(alpha2, __fmul_rn(alpha, alpha));
        beta2 = __fadd_rn(beta2, __fmul_rn(beta, beta));
        alphaBeta = __fadd_rn(alphaBeta, __fmul_rn(alpha, beta));
        alphaX = __fadd_rn(alphaX, __fmul_rn(alpha, value));
        betaX = __fadd_rn(betaX, __fmul_rn(beta, value));
    }
    __device__ __forceinline__ float Determinant() const
    {
        return __fsub_rn(__fmul_rn(alpha2, beta2), __fmul_rn(alphaBeta, alphaBeta));
    }
    __device__ __forceinline__ float NumeratorA() const
    {
        return __fsub_rn(__fmul_rn(alphaX, beta2), __fmul_rn(betaX, alphaBeta));
    }
    __device__ __forceinline__ float NumeratorB() const
    {
        return __fsub_rn(__fmul_rn(betaX, alpha2), __fmul_rn(alphaX, alphaBeta));
    }
};

__device__ __forceinline__ uint32_t RoundToByte(float x)
{
    return uint32_t(rintf(fminf(fmaxf(x, 0.f), 255.f)));
}

// Least-squares endpoints for the current indices, eight-interpolant mode (BC4_OptimizeAlpha8, :634-670).
__device__ void RefitEight(const uint32_t (&values)[16], Bc4Block& block, bool zeroAlpha1, bool oneAlpha0)
{
    RefitSums sums;
#pragma unroll
    for (int pixel = 0; pixel < 16; ++pixel)
    {
        const uint32_t index = IndexOf(block, pixel);
        sums.Add(kWeightEight[index], float(values[pixel]));
    }
    const float factor = __fdiv_rn(1.f, sums.Determinant());
    uint32_t a0 = oneAlpha0 ? 255u : RoundToByte(__fmul_rn(sums.NumeratorA(), factor));
    uint32_t a1 = zeroAlpha1 ? 0u : RoundToByte(__fmul_rn(sums.NumeratorB(), factor));
    if (a0 < a1)
    {
        const uint32_t t = a0;
        a0 = a1;
        a1 = t;
    }
    block.alpha0 = a0;
    block.alpha1 = a1;
}

// The same for the six-interpolant mode; pixels on the explicit 0 / 255 entries do not take part
// (BC4_OptimizeAlpha6, :672-708).
__device__ void RefitSix(const uint32_t (&values)[16], Bc4Block& block)
{
    RefitSums sums;
#pragma unroll
    for (int pixel = 0; pixel < 16; ++pixel)
    {
        const uint32_t index = IndexOf(block, pixel);
        if (index >= 6)
            continue;
        sums.Add(kWeightSix[index], float(values[pixel]));
    }
    const float determinant = sums.Determinant();
    if (determinant == 0.f)
        return;
    block.alpha0 = RoundToByte(__fdiv_rn(sums.NumeratorA(), determinant));
    block.alpha1 = RoundToByte(__fdiv_rn(sums.NumeratorB(), determinant));
}

// Alternates refit and index assignment while the error falls (the two loops of BC4_CompressFast, :741-794).
template <bool kSix>
__device__ void Refine(const uint32_t (&values)[16], Bc4Block& block, Bc4Block& best, uint32_t& bestError, bool zeroAlpha1,
    bool oneAlpha0)
{
    for (int pass = 0; pass < 8; ++pass)
    {
        if (kSix)
            RefitSix(values, block);
        else
            RefitEight(values, block, zeroAlpha1, oneAlpha0);
        const uint32_t error = AssignIndices(values, block);
        if (error >= bestError)
            break;
        const bool settled = block.indices == best.indices;
        best = block;
        if (settled)
            break;
        bestError = error;
    }
}

__device__ uint2 EncodeBc4(const float (&pixels)[16])
{
    uint32_t values[16];
    uint32_t low = 255, high = 0, lowInside = 255, highInside = 0;
#pragma unroll
    for (int pixel = 0; pixel < 16; ++pixel)
    {
        // saturate() sends NaN to 0
        const float saturated = pixels[pixel] != pixels[pixel] ? 0.f : fminf(fmaxf(pixels[pixel], 0.f), 1.f);
        const uint32_t v = uint32_t(rintf(__fmul_rn(saturated, 255.f)));
        values[pixel] = v;
        low = min(low, v);
        high = max(high, v);
        if (v != 0)
            lowInside = min(lowInside, v);
        if (v != 255)
            highInside = max(highInside, v);
    }
    const bool zeroAlpha1 = low == 0, oneAlpha0 = high == 255;

    Bc4Block block;
    block.alpha0 = oneAlpha0 ? 255u : (high - (high - low) / 34u) & 0xffu;
    block.alpha1 = zeroAlpha1 ? 0u : (low + (high - low) / 34u) & 0xffu;
    uint32_t bestError = AssignIndices(values, block);
    Bc4Block best = block;
    Refine<false>(values, block, best, bestError, zeroAlpha1, oneAlpha0);

    // six interpolants between the extremes that are not 0 or 255; unsigned wrap-around when the
    // block holds nothing else, as in the shader
    const uint32_t inset = (highInside - lowInside) / 34u;
    block.alpha0 = (lowInside + inset) & 0xffu;
    block.alpha1 = (highInside - inset) & 0xffu;
    uint32_t bestErrorSix = AssignIndices(values, block);
    Bc4Block bestSix = block;
    Refine<true>(values, block, bestSix, bestErrorSix, false, false);

    if (bestErrorSix < bestError)
        best = bestSix;
    const uint64_t bits = uint64_t(best.alpha0) | (uint64_t(best.alpha1) << 8) | (best.indices << 16);
    return make_uint2(uint32_t(bits), uint32_t(bits >> 32));
}

struct BlockCompressArguments
{
    const __half* texels;
    int layout, width, height, channels, firstChannel;
    int srcLeft, srcTop, widthInBlocks, heightInBlocks, formatChannels;
    uint8_t* blocks;
    size_t rowPitch;
};

// A texel outside the mip reads as 0, as an out-of-range texture load does.
__device__ __forceinline__ float LoadChannel(const BlockCompressArguments& args, int x, int y, int channel)
{
    if (x >= args.width || y >= args.height)
        return 0.f;
    const size_t w = size_t(args.width), c = size_t(args.channels);
    const size_t index = args.layout == NTCB_LAYOUT_INTERLEAVED
        ? (size_t(y) * w + size_t(x)) * c + size_t(channel)
        : size_t(y) * w * c + size_t(channel & ~1) * w + 2 * size_t(x) + size_t(channel & 1);
    return __half2float(args.texels[index]);
}

// One thread per 4x4 block and channel: BC5 is two BC4 blocks side by side, encoded by two threads
// (blockIdx.z = the channel), which keeps one copy of the encoder's code and its register count.
__global__ void __launch_bounds__(128) BlockCompressKernel(const BlockCompressArguments args)
{
    const int blockX = blockIdx.x * 16 + (threadIdx.x & 15); // thread groups of 16 x 8 blocks, as the shader's
    const int blockY = blockIdx.y * 8 + (threadIdx.x >> 4);
    const int c = blockIdx.z;
    if (blockX >= args.widthInBlocks || blockY >= args.heightInBlocks)
        return;
    float pixels[16];
#pragma unroll
    for (int pixel = 0; pixel < 16; ++pixel)
        pixels[pixel] = LoadChannel(args, args.srcLeft + blockX * 4 + (pixel & 3), args.srcTop + blockY * 4 + (pixel >> 2),
            args.firstChannel + c);
    uint8_t* destination = args.blocks + size_t(blockY) * args.rowPitch + size_t(blockX) * (8 * args.formatChannels);
    reinterpret_cast<uint2*>(destination)[c] = EncodeBc4(pixels);
}

} // namespace
} // namespace ntcb

using namespace ntcb;

extern "C" int ntcb_block_compress(const NtcbBlockCompressParams* params, void* stream)
{
    if (!params || !params->deviceMip || !params->deviceBlocks)
    {
        SetError("ntcb_block_compress: params, deviceMip and deviceBlocks must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (params->format != NTCB_BLOCK_FORMAT_BC4 && params->format != NTCB_BLOCK_FORMAT_BC5)
    {
        SetError("dstFormat (%d) is not supported: BC4 (%d) and BC5 (%d) are.", params->format, NTCB_BLOCK_FORMAT_BC4,
            NTCB_BLOCK_FORMAT_BC5);
        return params->format >= 1 && params->format <= 7 ? NTCB_ERR_UNSUPPORTED : NTCB_ERR_OUT_OF_RANGE;
    }
    const int formatChannels = params->format == NTCB_BLOCK_FORMAT_BC4 ? 1 : 2;
    const size_t blockBytes = 8u * formatChannels;
    if (params->layout != NTCB_LAYOUT_PLANAR_PAIRS && params->layout != NTCB_LAYOUT_INTERLEAVED)
    {
        SetError("ntcb_block_compress: unknown layout %d.", params->layout);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (params->width <= 0 || params->height <= 0 || params->channels <= 0 || params->channels > NTCB_MAX_CHANNELS
        || (params->layout == NTCB_LAYOUT_PLANAR_PAIRS && (params->channels & 1)))
    {
        SetError("ntcb_block_compress: width (%d) and height (%d) must be > 0 and channels (%d) between 1 and %d (even for the "
                 "planar-pair layout).", params->width, params->height, params->channels, NTCB_MAX_CHANNELS);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (params->firstChannel < 0 || params->firstChannel + formatChannels > params->channels)
    {
        SetError("firstChannel (%d) must be between 0 and %d for a format of %d channel(s).", params->firstChannel,
            params->channels - formatChannels, formatChannels);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (params->srcLeft < 0 || params->srcTop < 0 || params->widthInBlocks <= 0 || params->heightInBlocks <= 0)
    {
        SetError("srcLeft (%d) and srcTop (%d) must be >= 0; widthInBlocks (%d) and heightInBlocks (%d) must be > 0",
            params->srcLeft, params->srcTop, params->widthInBlocks, params->heightInBlocks);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (params->rowPitch < size_t(params->widthInBlocks) * blockBytes || params->rowPitch % blockBytes != 0
        || reinterpret_cast<uintptr_t>(params->deviceBlocks) % blockBytes != 0)
    {
        SetError("ntcb_block_compress: rowPitch (%zu) must be a multiple of the block size (%zu) and hold %d blocks; "
                 "deviceBlocks must be aligned to the block size.", params->rowPitch, blockBytes, params->widthInBlocks);
        return NTCB_ERR_INVALID_ARGUMENT;
    }

    BlockCompressArguments args;
    args.texels = static_cast<const __half*>(params->deviceMip);
    args.layout = params->layout;
    args.width = params->width;
    args.height = params->height;
    args.channels = params->channels;
    args.firstChannel = params->firstChannel;
    args.srcLeft = params->srcLeft;
    args.srcTop = params->srcTop;
    args.widthInBlocks = params->widthInBlocks;
    args.heightInBlocks = params->heightInBlocks;
    args.formatChannels = formatChannels;
    args.blocks = static_cast<uint8_t*>(params->deviceBlocks);
    args.rowPitch = params->rowPitch;

    const dim3 grid(unsigned(params->widthInBlocks + 15) / 16, unsigned(params->heightInBlocks + 7) / 8, unsigned(formatChannels));
    BlockCompressKernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(args);
    CountLaunch();
    const cudaError_t error = cudaGetLastError();
    if (error != cudaSuccess)
        return CudaFailure("BlockCompressKernel", error);
    ClearError();
    return NTCB_OK;
}
