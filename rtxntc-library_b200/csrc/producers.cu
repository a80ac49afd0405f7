// The two small encoder-side producers of the data the decode kernels consume: 4-bit latent words
// from quantised fp16 latents, and the GenericInt8 / GenericFP8 network blobs from fp16 weights.
// They replace cuda::PackLatents (src/Quantizer.cu:497-541) and cuda::QuantizeNetwork
// (src/Quantizer.cu:90-325), which the reference runs at the end of a compression session
// (src/TextureSet.cpp:1589-1633).
//
// The reference is built with --use_fast_math (src/CMakeLists.txt:33): its float divisions are the
// approximate hardware form and everything flushes denormals.  The same forms are spelled out here
// so that the results do not depend on this library's compiler flags.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "error.h"
#include "network_shape.h"
#include "ntcb.h"
#include "output_convert.cuh"

namespace ntcb
{
namespace
{

// ---------------------------------------------------------------------------------------------
// Latent packing

// QuantizeValue(value, 4) of src/Quantizer.cu:481-487: clamp to [0, 1] (std::min(1.f, NaN) is 1, so NaN
// packs as 15), divide by the step fl(1/15), round half away from zero.
//
// For an fp16 value v the product 15 v is exact in binary32 and lies at least 2^-16 away from every
// rounding tie, except v = 0.5 (15 v = 7.5), where the reference's quotient 0.5 / fl(1/15) falls
// just below the tie and rounds to 7.  Hence code = floor(v * m + 0.5) with m = 15 - 2^-20: the
// shortfall (at most 1e-6) moves nothing across an integer but sends 7.5 to 7.  The floor and the
// conversion to an integer are folded into the same fused multiply-add: adding 2^22 + 0.5 with
// rounding towards minus infinity leaves floor-to-halves of v * m + 0.5 in the low mantissa bits
// (units of 0.5 in [2^22, 2^23)), so bits 1-4 of the result are the code.  Two half-precision
// min / max clamp a pair (they return the other operand for NaN), then one conversion, one
// multiply-add, one shift and one logic operation per code - the first version (approximate
// division, roundf, a float-to-integer conversion: 14 instructions per code) was bound by
// instruction issue, not by memory.
__device__ __forceinline__ uint32_t CodeBits(float clamped)
{
    return __float_as_uint(__fmaf_rd(clamped, 14.99999905f, 4194304.5f));
}

__device__ __forceinline__ __half2 AsHalf2Bits(uint32_t bits)
{
    return *reinterpret_cast<const __half2*>(&bits);
}

__device__ __forceinline__ uint32_t LatentWord(__half2 first, __half2 second)
{
    const __half2 zero = __float2half2_rn(0.f), one = __float2half2_rn(1.f);
    const float2 a = __half22float2(__hmax2(__hmin2(first, one), zero));
    const float2 b = __half22float2(__hmax2(__hmin2(second, one), zero));
    return ((CodeBits(a.x) >> 1) & 0xfu) | ((CodeBits(a.y) << 3) & 0xf0u) | ((CodeBits(b.x) << 7) & 0xf00u)
         | ((CodeBits(b.y) << 11) & 0xf000u);
}

// One thread per latent texel and layer; any width, stride and alignment.
__global__ void PackLatentsKernel(const __half* __restrict__ latents, uint64_t texels, int layers, uint64_t latentStride,
    uint16_t* __restrict__ packed)
{
    const uint64_t total = texels * uint64_t(layers);
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x)
    {
        const uint64_t layer = i / texels, texel = i - layer * texels;
        const __half* src = latents + layer * latentStride * 2 + texel * 2;
        const __half2 first = __halves2half2(src[0], src[1]);
        const __half2 second = __halves2half2(src[latentStride], src[latentStride + 1]);
        packed[i] = uint16_t(LatentWord(first, second));
    }
}

// Eight texels per thread: two 32-byte reads, one 16-byte store.  Needs texels and latentStride to
// be multiples of 8 and both pointers 16-byte aligned.
__global__ void PackLatentsWideKernel(const uint4* __restrict__ latents, uint64_t texelGroups, int layers,
    uint64_t strideVectors, uint4* __restrict__ packed)
{
    const uint64_t total = texelGroups * uint64_t(layers);
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x)
    {
        const uint64_t layer = i / texelGroups, group = i - layer * texelGroups;
        const uint4* src = latents + layer * strideVectors * 2 + group * 2; // 8 texels x 2 halves = 2 vectors
        const uint4 a0 = __ldcs(src), a1 = __ldcs(src + 1);
        const uint4 b0 = __ldcs(src + strideVectors), b1 = __ldcs(src + strideVectors + 1);
        const uint32_t a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const uint32_t b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        uint32_t words[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
        {
            const uint32_t lo = LatentWord(AsHalf2Bits(a[2 * k]), AsHalf2Bits(b[2 * k]));
            const uint32_t hi = LatentWord(AsHalf2Bits(a[2 * k + 1]), AsHalf2Bits(b[2 * k + 1]));
            words[k] = lo | (hi << 16);
        }
        __stcs(packed + i, make_uint4(words[0], words[1], words[2], words[3]));
    }
}

// ---------------------------------------------------------------------------------------------
// Network quantisation

constexpr int kLayers = kMlpLayers;
constexpr int kColumns = kNetworkColumns;
constexpr int kWeights = kNetworkWeights;

struct QuantizeArguments
{
    const __half* weights; // per layer: outputs x inputs, one output's inputs together (the blob's order)
    const __half* biases;  // kColumns values, the layers one after another
    uint8_t* blob;
    __half* rounded;       // optional: the weights as the decoder will see them, same order as `weights`
    float outputScale[16], outputBias[16];
    int fp8;
};

// roundf: half away from zero, exact.
__device__ __forceinline__ float RoundAway(float x)
{
    return roundf(x);
}

// One output column quantised to int8 with a per-column scale and an integer bias
// (QuantizeColumnInt8, src/Quantizer.cu:90-208).
__device__ void QuantizeColumnInt8(int layer, int column, const __half* weights, float bias, int8_t* codes, __half* rounded,
    float* scaleOut, int32_t* biasOut, float outputScale, float outputBias)
{
    const int rows = LayerInputs(layer);
    float low = 3.402823466e+38f, high = 1.175494351e-38f; // the reference's starting values
    for (int r = 0; r < rows; ++r)
    {
        const float w = __half2float(weights[r]);
        low = fminf(low, w);
        high = fmaxf(high, w);
    }
    const float limit = fmaxf(fabsf(high), fabsf(low));
    float inverseLimit;
    asm("rcp.rn.ftz.f32 %0, %1;" : "=f"(inverseLimit) : "f"(limit));

    const float scale = 127.5f, inverseScale = 1.f / 127.5f;
    const float ratio = ApproxDivide(scale, limit); // the odd rows use scale / limit, the even ones scale * (1 / limit)
    int sum = 0;
    for (int r = 0; r < rows; ++r)
    {
        const float w = __half2float(weights[r]);
        float q = (r & 1) ? RoundAway(MulFtz(w, ratio)) : RoundAway(MulFtz(MulFtz(w, scale), inverseLimit));
        q = fmaxf(fminf(q, 127.f), -127.f);
        codes[r] = int8_t(q);
        sum += int(q);
        if (rounded)
            rounded[r] = __float2half_rn(MulFtz(MulFtz(q, limit), inverseScale));
    }

    float layerScale = MulFtz(limit, inverseScale);
    float layerBias = bias;
    if (layer == 0)
        layerScale = ApproxDivide(layerScale, 127.5f); // tin::InputQuant::scale
    else
    {
        const float activationStep = 3.1875f / 255.f; // tin::ActHGELUClamp::step
        const int activationBias = -113;             // tin::ActHGELUClamp::bias
        layerScale = MulFtz(layerScale, activationStep);
        layerBias = FmaFtz(-float(sum * activationBias), layerScale, layerBias);
        if (layer == kLayers - 1)
        {
            layerScale = MulFtz(layerScale, outputScale);
            layerBias = FmaFtz(layerBias, outputScale, outputBias);
        }
    }

    // (output * scale + bias) becomes ((output + integer bias) * scale); a zero scale (a constant
    // image channel) is replaced by 2^-16 with zero weights.
    int integerBias;
    if (layerScale == 0.f)
    {
        layerScale = 1.f / 65536.f;
        integerBias = int(RoundAway(MulFtz(layerBias, 65536.f)));
        for (int r = 0; r < rows; ++r)
            codes[r] = 0;
    }
    else
        integerBias = int(RoundAway(ApproxDivide(layerBias, layerScale)));
    *scaleOut = layerScale;
    *biasOut = integerBias;
}

// One output column rounded to e4m3; the bias stays fp16 (QuantizeColumnFP8, src/Quantizer.cu:210-252).
__device__ void QuantizeColumnFp8(int rows, const __half* weights, uint8_t* codes, __half* rounded)
{
    for (int r = 0; r < rows; r += 2)
    {
        const __half2 pair = __halves2half2(weights[r], weights[r + 1]);
        const __nv_fp8x2_e4m3 q(pair);
        codes[r] = uint8_t(q.__x & 0xff);
        codes[r + 1] = uint8_t(q.__x >> 8);
        if (rounded)
        {
            const __half2 back = __half2(q);
            rounded[r] = __low2half(back);
            rounded[r + 1] = __high2half(back);
        }
    }
}

// One thread per output column, the columns of all layers one after another: a single CTA.
__global__ void __launch_bounds__(kColumns) QuantizeNetworkKernel(const QuantizeArguments args)
{
    int column = threadIdx.x, layer = 0, weightOffset = 0, columnOffset = 0;
    while (column >= LayerOutputs(layer))
    {
        column -= LayerOutputs(layer);
        columnOffset += LayerOutputs(layer);
        weightOffset += LayerInputs(layer) * LayerOutputs(layer);
        ++layer;
    }
    const int rows = LayerInputs(layer);
    const __half* weights = args.weights + weightOffset + column * rows;
    __half* rounded = args.rounded ? args.rounded + weightOffset + column * rows : nullptr;
    uint8_t* codes = args.blob + weightOffset + column * rows;
    const __half bias = args.biases[columnOffset + column];

    if (!args.fp8)
    {
        // weights, then the scales of all layers, then the integer biases (src/WeightLayout.cpp:184-255)
        float* scales = reinterpret_cast<float*>(args.blob + kWeights) + columnOffset + column;
        int32_t* biases = reinterpret_cast<int32_t*>(args.blob + kWeights + 4 * kColumns) + columnOffset + column;
        QuantizeColumnInt8(layer, column, weights, __half2float(bias), reinterpret_cast<int8_t*>(codes), rounded, scales, biases,
            args.outputScale[column & 15], args.outputBias[column & 15]);
    }
    else if (layer < kLayers - 1)
    {
        // weights, then the fp16 biases of layers 0-2, then the output layer's scales and integer biases
        QuantizeColumnFp8(rows, weights, codes, rounded);
        reinterpret_cast<__half*>(args.blob + kWeights)[columnOffset + column] = bias;
    }
    else
    {
        uint8_t* tail = args.blob + kWeights + 2 * (kColumns - 16);
        QuantizeColumnInt8(layer, column, weights, __half2float(bias), reinterpret_cast<int8_t*>(codes), rounded,
            reinterpret_cast<float*>(tail) + column, reinterpret_cast<int32_t*>(tail + 64) + column,
            args.outputScale[column], args.outputBias[column]);
    }
}

// ---------------------------------------------------------------------------------------------
// Latents re-laid for inference on sample: pixel-major, the layers of a pixel side by side
// ---------------------------------------------------------------------------------------------

constexpr int kMaxGrids = 2 * NTCB_MAX_MIPS;

struct InterleaveArguments
{
    const uint16_t* planar;
    uint16_t* interleaved;
    int numGrids, numLayers, slot;                // slot: elements per pixel in the copy (1, 2 or 4)
    unsigned long long firstPixel[kMaxGrids + 1]; // running pixel count: grid g owns [firstPixel[g], firstPixel[g + 1])
    unsigned long long offset[kMaxGrids];         // element offset of the grid in the planar buffer
    unsigned long long plane[kMaxGrids];          // elements between the layers of the planar grid
};

// One thread per latent pixel: reads its layers from the planes (coalesced over the warp, layer by layer) and
// writes its slot (contiguous over the warp); the fourth element of a three-layer slot is zero.
__global__ void InterleaveLatentsKernel(const __grid_constant__ InterleaveArguments args)
{
    const unsigned long long total = args.firstPixel[args.numGrids];
    for (unsigned long long index = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; index < total;
         index += (unsigned long long)gridDim.x * blockDim.x)
    {
        int grid = 0;
        while (grid + 1 < args.numGrids && index >= args.firstPixel[grid + 1])
            ++grid;
        const unsigned long long pixel = index - args.firstPixel[grid];
        const uint16_t* source = args.planar + args.offset[grid] + pixel;
        uint16_t* target = args.interleaved + args.offset[grid] / args.numLayers * args.slot + pixel * (unsigned long long)args.slot;
        for (int layer = 0; layer < args.slot; ++layer)
            target[layer] = layer < args.numLayers ? __ldg(source + (unsigned long long)layer * args.plane[grid]) : uint16_t(0);
    }
}

} // namespace
} // namespace ntcb

using namespace ntcb;

extern "C" int ntcb_pack_latents(const void* latents, int width, int height, int numLayers, size_t latentStride,
    void* packed, void* stream)
{
    if (!latents || !packed)
    {
        SetError("ntcb_pack_latents: latents and packed must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (width <= 0 || height <= 0 || numLayers <= 0)
    {
        SetError("ntcb_pack_latents: width (%d), height (%d) and numLayers (%d) must be positive.", width, height, numLayers);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    const uint64_t texels = uint64_t(width) * uint64_t(height);
    if (latentStride < texels * 2)
    {
        SetError("ntcb_pack_latents: latentStride (%zu) must be at least 2 * width * height (%llu).", latentStride,
            static_cast<unsigned long long>(texels * 2));
        return NTCB_ERR_OUT_OF_RANGE;
    }
    int device = 0, sms = 0;
    cudaError_t error = cudaGetDevice(&device);
    if (error == cudaSuccess)
        error = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (error != cudaSuccess)
        return CudaFailure("cudaDeviceGetAttribute", error);

    const cudaStream_t cudaStream = static_cast<cudaStream_t>(stream);
    const int threads = 256;
    const bool wide = texels % 8 == 0 && latentStride % 8 == 0 && reinterpret_cast<uintptr_t>(latents) % 16 == 0
                   && reinterpret_cast<uintptr_t>(packed) % 16 == 0;
    const uint64_t items = (wide ? texels / 8 : texels) * uint64_t(numLayers);
    const uint64_t wanted = (items + threads - 1) / threads;
    // Whole waves of 8 CTAs of 256 threads per SM; eight waves, each CTA striding over the items,
    // measured 6 % faster than a single resident wave (the tail of a wave overlaps the next one).
    const uint64_t resident = uint64_t(sms) * 8 * 8;
    const unsigned grid = unsigned(wanted < resident ? wanted : resident);
    if (wide)
        PackLatentsWideKernel<<<grid, threads, 0, cudaStream>>>(static_cast<const uint4*>(latents), texels / 8, numLayers,
            latentStride / 8, static_cast<uint4*>(packed));
    else
        PackLatentsKernel<<<grid, threads, 0, cudaStream>>>(static_cast<const __half*>(latents), texels, numLayers, latentStride,
            static_cast<uint16_t*>(packed));
    CountLaunch();
    error = cudaGetLastError();
    if (error != cudaSuccess)
        return CudaFailure("PackLatentsKernel", error);
    ClearError();
    return NTCB_OK;
}

extern "C" int ntcb_interleave_latents(const uint16_t* latents, uint16_t* interleaved, const NtcbMipDesc* mips, int numMips,
    int numFeatures, void* stream)
{
    if (!latents || !interleaved || !mips || latents == interleaved)
    {
        SetError("ntcb_interleave_latents: latents, interleaved (another buffer) and mips must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (numMips < 1 || numMips > NTCB_MAX_MIPS || numFeatures < 4 || numFeatures > 16 || (numFeatures & 3))
    {
        SetError("ntcb_interleave_latents: invalid mip count (%d) or feature count (%d).", numMips, numFeatures);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (reinterpret_cast<uintptr_t>(interleaved) & 7)
    {
        SetError("ntcb_interleave_latents: interleaved must be 8-byte aligned.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    InterleaveArguments args{};
    args.planar = latents;
    args.interleaved = interleaved;
    args.numLayers = numFeatures / 4;
    args.slot = args.numLayers == 3 ? 4 : args.numLayers;
    // the colour mips of a neural mip share its grids: each distinct grid once
    auto addGrid = [&](uint64_t offset, uint64_t plane, int width, int height) -> int {
        const uint64_t pixels = uint64_t(width) * uint64_t(height);
        if (width < 1 || height < 1 || plane < pixels)
        {
            SetError("ntcb_interleave_latents: a grid of %d x %d pixels with %llu elements between its layers.", width, height,
                static_cast<unsigned long long>(plane));
            return NTCB_ERR_INVALID_ARGUMENT;
        }
        if (offset % uint64_t(args.numLayers))
        {
            SetError("ntcb_interleave_latents: the offset of a grid (%llu) is not a multiple of the layer count (%d).",
                static_cast<unsigned long long>(offset), args.numLayers);
            return NTCB_ERR_INVALID_ARGUMENT;
        }
        for (int g = 0; g < args.numGrids; ++g)
            if (args.offset[g] == offset)
                return NTCB_OK;
        args.offset[args.numGrids] = offset;
        args.plane[args.numGrids] = plane;
        args.firstPixel[args.numGrids + 1] = args.firstPixel[args.numGrids] + pixels;
        ++args.numGrids;
        return NTCB_OK;
    };
    for (int m = 0; m < numMips; ++m)
    {
        int status = addGrid(mips[m].hiOffset, mips[m].hiPlane, mips[m].hiWidth, mips[m].hiHeight);
        if (status == NTCB_OK)
            status = addGrid(mips[m].loOffset, mips[m].loPlane, mips[m].loWidth, mips[m].loHeight);
        if (status != NTCB_OK)
            return status;
    }
    int device = 0, sms = 0;
    cudaError_t error = cudaGetDevice(&device);
    if (error == cudaSuccess)
        error = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (error != cudaSuccess)
        return CudaFailure("cudaDeviceGetAttribute", error);
    const int threads = 256;
    const uint64_t wanted = (args.firstPixel[args.numGrids] + threads - 1) / threads;
    const uint64_t resident = uint64_t(sms) * 8 * 4;
    const unsigned grid = unsigned(wanted < resident ? wanted : resident);
    InterleaveLatentsKernel<<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(args);
    CountLaunch();
    error = cudaGetLastError();
    if (error != cudaSuccess)
        return CudaFailure("InterleaveLatentsKernel", error);
    ClearError();
    return NTCB_OK;
}

extern "C" int ntcb_quantize_network(const NtcbQuantizeNetworkParams* params, void* stream)
{
    if (!params || !params->weights || !params->biases || !params->blob)
    {
        SetError("ntcb_quantize_network: params, weights, biases and blob must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (params->weightMode != NTCB_WEIGHTS_INT8 && params->weightMode != NTCB_WEIGHTS_FP8)
    {
        SetError("ntcb_quantize_network: unknown weight mode %d.", params->weightMode);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    QuantizeArguments args;
    args.weights = static_cast<const __half*>(params->weights);
    args.biases = static_cast<const __half*>(params->biases);
    args.blob = static_cast<uint8_t*>(params->blob);
    args.rounded = static_cast<__half*>(params->roundedWeights);
    args.fp8 = params->weightMode == NTCB_WEIGHTS_FP8;
    for (int c = 0; c < 16; ++c)
    {
        args.outputScale[c] = params->outputScale ? params->outputScale[c] : 1.f;
        args.outputBias[c] = params->outputBias ? params->outputBias[c] : 0.f;
    }
    QuantizeNetworkKernel<<<1, kColumns, 0, static_cast<cudaStream_t>(stream)>>>(args);
    CountLaunch();
    const cudaError_t error = cudaGetLastError();
    if (error != cudaSuccess)
        return CudaFailure("QuantizeNetworkKernel", error);
    ClearError();
    return NTCB_OK;
}
