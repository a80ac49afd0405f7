// BC7 encoding of decoded texels: the CUDA form of the reference's src/shaders/CompressBC7.hlsl, the
// compute pass IContext::MakeBlockCompressionComputePass describes for BlockCompressedFormat::BC7
// (src/Context.cpp:630-779).  Two kernels, as the shader is built twice:
//
//  * with a mode buffer (USE_MODE_BUFFER, the run-time path): 9 bits per block say which mode and
//    partition (for modes 4 / 5: rotation and index selector) the block had when the texture was
//    compressed offline (ntc::MakeBC7ModeBuffer, src/PublicFunctions.cpp:488-556); the encoder only
//    fits endpoints and indices for that one configuration.  The threads of a CTA are re-ordered by
//    mode through shared memory so that a warp runs one mode (CompressBC7.hlsl:1446-1493);
//  * without: every mode is tried - 64 partitions of modes 0 / 2, 1 / 3 and 7 by estimated error, the
//    best one of each encoded, modes 4 / 5 under the four channel rotations, mode 6 - and the block
//    with the smallest squared error of its reconstruction kept (ties: the later mode).
//
// This file is compiled with --fmad=false: the encoder's arithmetic is binary32 in the shader's order
// of operations with nothing fused, divisions and `round` (half to even) IEEE; min / max / saturate
// return the other operand when one is a NaN, as the HLSL intrinsics do.  The input is the decode
// kernel's fp16 output (either layout), staged per CTA in shared memory as four halves per texel,
// texel i of block slot t at word i * 256 + t, so the loops over the texels stay rolled.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>
#include <string.h>

#include "block_compress.h"
#include "error.h"
#include "ntcb.h"

namespace ntcb
{
namespace
{

constexpr int kGroupWidth = 32;  // blocks per CTA, x
constexpr int kGroupHeight = 8;  // and y
constexpr int kThreads = kGroupWidth * kGroupHeight;
constexpr uint32_t kAllPixels = 0xffffu;

// The partition tables of the BC7 format (Khronos data format specification, BPTC: tables P2, P3 and
// the anchor tables A2, A3a, A3b), as pixel masks.  Two subsets: the mask of subset 1 (subset 0 is the
// rest; pixel 0 is always in subset 0).  Three subsets: subset 1 in the low half, subset 2 in the high
// half.  Anchors: bits 0-3 the anchor of subset 1 of a two-subset partition, bits 4-7 and 8-11 those of
// subsets 1 and 2 of a three-subset partition.
__constant__ uint16_t kPartition2[64] = {
    0xcccc, 0x8888, 0xeeee, 0xecc8, 0xc880, 0xfeec, 0xfec8, 0xec80, 0xc800, 0xffec, 0xfe80, 0xe800, 0xffe8, 0xff00, 0xfff0, 0xf000,
    0xf710, 0x008e, 0x7100, 0x08ce, 0x008c, 0x7310, 0x3100, 0x8cce, 0x088c, 0x3110, 0x6666, 0x366c, 0x17e8, 0x0ff0, 0x718e, 0x399c,
    0xaaaa, 0xf0f0, 0x5a5a, 0x33cc, 0x3c3c, 0x55aa, 0x9696, 0xa55a, 0x73ce, 0x13c8, 0x324c, 0x3bdc, 0x6996, 0xc33c, 0x9966, 0x0660,
    0x0272, 0x04e4, 0x4e40, 0x2720, 0xc936, 0x936c, 0x39c6, 0x639c, 0x9336, 0x9cc6, 0x817e, 0xe718, 0xccf0, 0x0fcc, 0x7744, 0xee22,
};
__constant__ uint32_t kPartition3[64] = {
    0xf60008ccu, 0x73008cc8u, 0x3310cc80u, 0x00ceec00u, 0xcc003300u, 0xcc0000ccu, 0x00ccff00u, 0x3300ccccu,
    0xf0000f00u, 0xf0000ff0u, 0xff0000f0u, 0x88884444u, 0x88886666u, 0xcccc2222u, 0xec80136cu, 0x7310008cu,
    0xc80036c8u, 0x310008ceu, 0xccc03330u, 0x0cccf000u, 0xee0000eeu, 0x77008888u, 0xcc0022c0u, 0x33004430u,
    0x00cc0c22u, 0xfc880344u, 0x06606996u, 0x66009960u, 0xc88c0330u, 0xf9000066u, 0x0cc0c22cu, 0x73108c00u,
    0xec801300u, 0x08cec400u, 0xec80004cu, 0x44442222u, 0x0f0000f0u, 0x49242492u, 0x42942942u, 0x0c30c30cu,
    0x03c0c03cu, 0xff0000aau, 0x5500aa00u, 0xcccc3030u, 0x0c0cc0c0u, 0x66669090u, 0x0ff0a00au, 0x5550aaa0u,
    0xf0000aaau, 0x0e0ee0e0u, 0x88887070u, 0x99906660u, 0xe00e0ee0u, 0x88880770u, 0xf0000666u, 0x99006600u,
    0xff000066u, 0xc00c0cc0u, 0xcccc0330u, 0x90006000u, 0x08088080u, 0xeeee1010u, 0xfff0000au, 0x731008ceu,
};
__constant__ uint16_t kAnchors[64] = {
    0xf3f, 0x83f, 0x8ff, 0x3ff, 0xf8f, 0xf3f, 0x3ff, 0x8ff, 0xf8f, 0xf8f, 0xf6f, 0xf6f, 0xf6f, 0xf5f, 0xf3f, 0x83f,
    0xf3f, 0x832, 0xf88, 0x3f2, 0xf32, 0x838, 0xf68, 0x8af, 0x352, 0xf88, 0x682, 0xa62, 0xf88, 0xf58, 0xaf2, 0x8f2,
    0xf8f, 0x3ff, 0xf36, 0xa58, 0xa62, 0x8a8, 0x98f, 0xaff, 0x6f2, 0xf38, 0x8f2, 0xf52, 0x3f2, 0x6ff, 0x6ff, 0x8f6,
    0xf36, 0x3f2, 0xf56, 0xf58, 0xf5f, 0xf8f, 0xf52, 0xfa2, 0xf5f, 0xfaf, 0xf8f, 0xfdf, 0x3ff, 0xfc2, 0xf32, 0x83f,
};

// The subsets of a partition: pixel masks and anchor pixels (the pixel whose index loses its top bit).
struct Subsets
{
    uint32_t mask[3];
    int anchor[3];
};

__device__ __forceinline__ Subsets TwoSubsets(int partition)
{
    const uint32_t second = kPartition2[partition];
    return {{~second & kAllPixels, second, 0u}, {0, int(kAnchors[partition] & 15), 0}};
}

__device__ __forceinline__ Subsets ThreeSubsets(int partition)
{
    const uint32_t packed = kPartition3[partition];
    const uint32_t second = packed & kAllPixels, third = packed >> 16;
    const uint32_t anchors = kAnchors[partition];
    return {{~(second | third) & kAllPixels, second, third}, {0, int((anchors >> 4) & 15), int((anchors >> 8) & 15)}};
}

// ---- vectors of 1, 3 or 4 components -----------------------------------------------------------------
template <int C>
struct Vec
{
    float v[C];
};

template <int C>
__device__ __forceinline__ Vec<C> Splat(float s)
{
    Vec<C> r;
#pragma unroll
    for (int c = 0; c < C; ++c)
        r.v[c] = s;
    return r;
}

#define NTCB_VEC_BINARY(name, expression)                                      \
    template <int C>                                                           \
    __device__ __forceinline__ Vec<C> name(const Vec<C>& a, const Vec<C>& b)   \
    {                                                                          \
        Vec<C> r;                                                              \
        _Pragma("unroll") for (int c = 0; c < C; ++c) r.v[c] = (expression);   \
        return r;                                                              \
    }
NTCB_VEC_BINARY(operator+, a.v[c] + b.v[c])
NTCB_VEC_BINARY(operator-, a.v[c] - b.v[c])
NTCB_VEC_BINARY(Min, fminf(a.v[c], b.v[c]))
NTCB_VEC_BINARY(Max, fmaxf(a.v[c], b.v[c]))
#undef NTCB_VEC_BINARY

template <int C>
__device__ __forceinline__ Vec<C> operator*(const Vec<C>& a, float s)
{
    Vec<C> r;
#pragma unroll
    for (int c = 0; c < C; ++c)
        r.v[c] = a.v[c] * s;
    return r;
}

// x*x + y*y + z*z (+ w*w), summed left to right
template <int C>
__device__ __forceinline__ float Dot(const Vec<C>& a, const Vec<C>& b)
{
    float sum = a.v[0] * b.v[0];
#pragma unroll
    for (int c = 1; c < C; ++c)
        sum = sum + a.v[c] * b.v[c];
    return sum;
}

__device__ __forceinline__ float Saturate(float v)
{
    return fminf(fmaxf(v, 0.f), 1.f); // NaN -> 0
}

// ---- the texels of a block ------------------------------------------------------------------------------
// rotation: which channel is the scalar one of a dual-plane mode (0: alpha, 1: red, 2: green, 3: blue, the
// other one of the pair taking alpha's place); the vector part is the first three components.
struct Pixels
{
    const uint2* base; // texel i at base[i * kThreads]
    int rotation;
};

template <int C>
__device__ __forceinline__ Vec<C> Pixel(const Pixels& pixels, int i)
{
    const uint2 raw = pixels.base[i * kThreads];
    const float2 rg = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 ba = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    float r = rg.x, g = rg.y, b = ba.x, a = ba.y;
    if (pixels.rotation == 1)
    {
        const float t = r;
        r = a;
        a = t;
    }
    else if (pixels.rotation == 2)
    {
        const float t = g;
        g = a;
        a = t;
    }
    else if (pixels.rotation == 3)
    {
        const float t = b;
        b = a;
        a = t;
    }
    Vec<C> result;
    if (C == 1)
        result.v[0] = a;
    else
    {
        result.v[0] = r;
        result.v[C > 1 ? 1 : 0] = g;
        result.v[C > 2 ? 2 : 0] = b;
        if (C == 4)
            result.v[C - 1] = a;
    }
    return result;
}

// ---- the encoder's building blocks (CompressBC7.hlsl:144-527) ----------------------------------------
__device__ __forceinline__ int Quantize(float value, int bits)
{
    const float scale = float((1u << bits) - 1u);
    return int(rintf(Saturate(value) * scale));
}

__device__ __forceinline__ int ExpandTo8Bits(int q, int bits)
{
    return (q << (8 - bits)) | (q >> (2 * bits - 8));
}

template <int C>
__device__ __forceinline__ void MinMax(const Pixels& pixels, uint32_t mask, Vec<C>& mins, Vec<C>& maxs)
{
    mins = Splat<C>(FLT_MAX);
    maxs = Splat<C>(-FLT_MAX);
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        if ((mask >> i) & 1u)
        {
            const Vec<C> p = Pixel<C>(pixels, i);
            mins = Min(mins, p);
            maxs = Max(maxs, p);
        }
}

// Two rounds of least squares on the endpoints for the indices the current endpoints give
// (BC7_OptimizeEndpoints, :188-244); endpoint components at exactly 0 or 1 stay.
template <int C>
__device__ void OptimizeEndpoints(const Pixels& pixels, uint32_t mask, Vec<C>& ep0, Vec<C>& ep1, int indexBits)
{
#pragma unroll 1
    for (int iteration = 0; iteration < 2; ++iteration)
    {
        const Vec<C> axis = ep1 - ep0;
        float mul = Dot(axis, axis);
        if (mul > 0.0f)
            mul = 1.0f / mul;
        const float scale = float((1u << indexBits) - 1u);
        const float inverseScale = 1.0f / scale;
        float alpha2 = 0.f, beta2 = 0.f, alphaBeta = 0.f;
        Vec<C> alphaX = Splat<C>(0.f), betaX = Splat<C>(0.f);
#pragma unroll 1
        for (int i = 0; i < 16; ++i)
            if ((mask >> i) & 1u)
            {
                const Vec<C> color = Pixel<C>(pixels, i);
                const float index = Saturate(Dot(color - ep0, axis) * mul);
                const float beta = rintf(index * scale) * inverseScale;
                const float alpha = 1.0f - beta;
                alpha2 += alpha * alpha;
                beta2 += beta * beta;
                alphaBeta += alpha * beta;
                alphaX = alphaX + color * alpha;
                betaX = betaX + color * beta;
            }
        const float denominator = alpha2 * beta2 - alphaBeta * alphaBeta;
        if (!(fabsf(denominator) > 0.0001f))
            break;
        const float factor = 1.0f / denominator;
#pragma unroll
        for (int c = 0; c < C; ++c)
        {
            const float a = Saturate((alphaX.v[c] * beta2 - betaX.v[c] * alphaBeta) * factor);
            const float b = Saturate((betaX.v[c] * alpha2 - alphaX.v[c] * alphaBeta) * factor);
            if (!(ep0.v[c] == 0.0f || ep0.v[c] == 1.0f))
                ep0.v[c] = a;
            if (!(ep1.v[c] == 0.0f || ep1.v[c] == 1.0f))
                ep1.v[c] = b;
        }
    }
}

// Min / max endpoints put every component's low value in ep0; where two components run against each
// other over the subset, one of them is swapped (BC7_SwapEndpointComponents_RGB / _RGBA, :248-345): the
// first component with an extent is the reference, the later ones follow the sign of their covariance with it.
template <int C>
__device__ void SwapEndpointComponents(const Pixels& pixels, uint32_t mask, Vec<C>& ep0, Vec<C>& ep1)
{
    Vec<C> sum = Splat<C>(0.f);
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        if ((mask >> i) & 1u)
            sum = sum + Pixel<C>(pixels, i);
    const float count = float(__popc(mask));
    Vec<C> center;
#pragma unroll
    for (int c = 0; c < C; ++c)
        center.v[c] = sum.v[c] / count;
    float covariance[C][C];
#pragma unroll
    for (int a = 0; a < C; ++a)
#pragma unroll
        for (int b = 0; b < C; ++b)
            covariance[a][b] = 0.f;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        if ((mask >> i) & 1u)
        {
            const Vec<C> p = Pixel<C>(pixels, i) - center;
#pragma unroll
            for (int a = 0; a < C; ++a)
#pragma unroll
                for (int b = a + 1; b < C; ++b)
                    covariance[a][b] += p.v[a] * p.v[b];
        }
    bool done = false;
#pragma unroll
    for (int a = 0; a + 1 < C; ++a)
        if (!done && ep0.v[a] != ep1.v[a])
        {
            done = true;
#pragma unroll
            for (int b = a + 1; b < C; ++b)
                if (covariance[a][b] < 0.f)
                {
                    const float t = ep0.v[b];
                    ep0.v[b] = ep1.v[b];
                    ep1.v[b] = t;
                }
        }
}

// Squared error of the subset against the line between two unquantised endpoints, with the indices
// rounded to `indexBits` but not clamped (BC7_EstimateError, :347-377).
template <int C>
__device__ float EstimateError(const Pixels& pixels, uint32_t mask, const Vec<C>& ep0, const Vec<C>& ep1, int indexBits)
{
    const Vec<C> axis = ep1 - ep0;
    float mul = Dot(axis, axis);
    if (mul > 0.0f)
        mul = 1.0f / mul;
    const float maxIndex = float((1u << indexBits) - 1u);
    const float indexScale = 1.f / maxIndex;
    float error = 0.f;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        if ((mask >> i) & 1u)
        {
            const Vec<C> p = Pixel<C>(pixels, i) - ep0;
            float index = Dot(p, axis) * mul;
            index = rintf(index * maxIndex) * indexScale;
            const Vec<C> difference = axis * index - p;
            error += Dot(difference, difference);
        }
    return error;
}

// Indices of a subset's pixels, 4 bits per pixel in `indices`; true when the anchor's top bit was set and
// all of the subset's indices were therefore inverted - the caller then swaps the endpoints
// (BC7_CalculateIndices, :441-489; the anchor-0 form :493-527 gives the same indices).
template <int C>
__device__ bool CalculateIndices(const Pixels& pixels, uint32_t mask, int anchor, int indexBits, int endpointBits,
    const int (&q0)[C], const int (&q1)[C], uint64_t& indices)
{
    Vec<C> ep0, axis;
#pragma unroll
    for (int c = 0; c < C; ++c)
    {
        ep0.v[c] = float(ExpandTo8Bits(q0[c], endpointBits)) / 255.0f;
        axis.v[c] = float(ExpandTo8Bits(q1[c], endpointBits)) / 255.0f - ep0.v[c];
    }
    float mul = Dot(axis, axis);
    if (mul > 0.0f)
        mul = 1.0f / mul;
    uint64_t subsetIndices = 0, subsetMask = 0;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        if ((mask >> i) & 1u)
        {
            const float index = Dot(Pixel<C>(pixels, i) - ep0, axis) * mul;
            subsetIndices |= uint64_t(Quantize(index, indexBits)) << (4 * i);
            subsetMask |= uint64_t((1u << indexBits) - 1u) << (4 * i);
        }
    const bool flip = ((subsetIndices >> (4 * anchor)) >> (indexBits - 1)) & 1u;
    if (flip)
        subsetIndices ^= subsetMask;
    indices = (indices & ~subsetMask) | subsetIndices;
    return flip;
}

// Squared error of the subset as a decoder reconstructs it (BC7_ComputeError, :379-412).
template <int C>
__device__ float ComputeError(const Pixels& pixels, uint64_t indices, uint32_t mask, const int (&q0)[C], const int (&q1)[C],
    int indexBits, int endpointBits)
{
    int e0[C], e1[C];
#pragma unroll
    for (int c = 0; c < C; ++c)
    {
        e0[c] = ExpandTo8Bits(q0[c], endpointBits);
        e1[c] = ExpandTo8Bits(q1[c], endpointBits);
    }
    const float maxIndex = float((1u << indexBits) - 1u);
    const float indexScale = 64.f / maxIndex;
    float error = 0.f;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        if ((mask >> i) & 1u)
        {
            const int weight = int(rintf(float(int(indices >> (4 * i)) & 15) * indexScale)); // 0..64
            const Vec<C> p = Pixel<C>(pixels, i);
            Vec<C> difference;
#pragma unroll
            for (int c = 0; c < C; ++c)
                difference.v[c] = float((e0[c] * (64 - weight) + e1[c] * weight + 32) >> 6) / 255.0f - p.v[c];
            error += Dot(difference, difference);
        }
    return error;
}

// ---- the 128 bits of a block ------------------------------------------------------------------------------
struct BlockBits
{
    uint64_t low = 0, high = 0;
    int offset = 0;

    __device__ __forceinline__ void Put(int length, uint32_t value)
    {
        const uint64_t bits = value & ((1u << length) - 1u);
        if (offset < 64)
        {
            low |= bits << offset;
            if (offset + length > 64)
                high |= bits >> (64 - offset);
        }
        else
            high |= bits << (offset - 64);
        offset += length;
    }
    __device__ __forceinline__ uint4 Words() const
    {
        return make_uint4(uint32_t(low), uint32_t(low >> 32), uint32_t(high), uint32_t(high >> 32));
    }
};

// ---- modes 0-3, 6, 7: one colour plane, one to three subsets ------------------------------------------
template <int kMode>
struct ModeTraits;
// subsets, components, index bits, endpoint bits (with the p-bit), p-bits: 0 none, 1 one per endpoint, 2 one per subset
#define NTCB_BC7_MODE(mode, subsets, components, indexBits, endpointBits, pBits, partitionBits)                          \
    template <>                                                                                                           \
    struct ModeTraits<mode>                                                                                               \
    {                                                                                                                     \
        static constexpr int kSubsets = subsets, kComponents = components, kIndexBits = indexBits, kEndpointBits = endpointBits, \
                             kPBits = pBits, kPartitionBits = partitionBits;                                              \
    };
NTCB_BC7_MODE(0, 3, 3, 3, 5, 1, 4)
NTCB_BC7_MODE(1, 2, 3, 3, 7, 2, 6)
NTCB_BC7_MODE(2, 3, 3, 2, 5, 0, 6)
NTCB_BC7_MODE(3, 2, 3, 2, 8, 1, 6)
NTCB_BC7_MODE(6, 1, 4, 4, 8, 1, 0)
NTCB_BC7_MODE(7, 2, 4, 2, 6, 1, 6)
#undef NTCB_BC7_MODE

// Refines the endpoints found for a partition, quantises them, assigns indices and, when the block is no
// worse than the best one so far, encodes it (BC7_Mode0_Finalize ... BC7_Mode3_Finalize, BC7_Mode6_Compress,
// the second half of BC7_Mode7_Compress).  With a mode buffer there is nothing to compare: the error stays 0.
template <int kMode, bool kSingleMode>
__device__ void FinalizeMode(const Pixels& pixels, int partition, const Subsets& subsets,
    const Vec<ModeTraits<kMode>::kComponents>* endpoints, float& currentError, uint4& currentBlock)
{
    using Traits = ModeTraits<kMode>;
    constexpr int C = Traits::kComponents, kSubsets = Traits::kSubsets, kIndexBits = Traits::kIndexBits,
                  kEndpointBits = Traits::kEndpointBits;
    Vec<C> ep[2 * kSubsets];
#pragma unroll
    for (int i = 0; i < 2 * kSubsets; ++i)
        ep[i] = endpoints[i];
#pragma unroll
    for (int s = 0; s < kSubsets; ++s)
        OptimizeEndpoints<C>(pixels, subsets.mask[s], ep[2 * s], ep[2 * s + 1], kIndexBits);

    int q[2 * kSubsets][C];
#pragma unroll
    for (int i = 0; i < 2 * kSubsets; ++i)
#pragma unroll
        for (int c = 0; c < C; ++c)
            q[i][c] = Quantize(ep[i].v[c], kEndpointBits);
    if (Traits::kPBits == 1 && C == 3)
    {
        // the p-bit of an endpoint: what most of its components end in (BC7_RGB_QuantizeEndpoint, :414-423)
#pragma unroll
        for (int i = 0; i < 2 * kSubsets; ++i)
        {
            const int bit = (q[i][0] & 1) + (q[i][1] & 1) + (q[i][2] & 1) >= 2 ? 1 : 0;
#pragma unroll
            for (int c = 0; c < C; ++c)
                q[i][c] = (q[i][c] & 0xFE) | bit;
        }
    }
    else if (Traits::kPBits == 1)
    {
        // with alpha: 0 stays 0 and 1 stays 1 (BC7_RGBA_QuantizeEndpoint, :439-455)
#pragma unroll
        for (int i = 0; i < 2 * kSubsets; ++i)
        {
            const bool majorityOdd = (q[i][0] & 1) + (q[i][1] & 1) + (q[i][2] & 1) + (q[i][C - 1] & 1) >= 2;
            const bool alphaZero = q[i][C - 1] == 0;
            const bool alphaOne = ep[i].v[C - 1] == 1.0f;
            const int bit = ((majorityOdd && !alphaZero) || alphaOne) ? 1 : 0;
#pragma unroll
            for (int c = 0; c < C; ++c)
                q[i][c] = (q[i][c] & 0xFE) | bit;
        }
    }
    else if (Traits::kPBits == 2)
    {
        // one p-bit for both endpoints of a subset (BC7_RGB_QuantizeEndpoints_SharedLSB, :426-436)
#pragma unroll
        for (int s = 0; s < kSubsets; ++s)
        {
            int odd = 0;
#pragma unroll
            for (int c = 0; c < C; ++c)
                odd += (q[2 * s][c] & 1) + (q[2 * s + 1][c] & 1);
            const int bit = odd >= 4 ? 1 : 0;
#pragma unroll
            for (int c = 0; c < C; ++c)
            {
                q[2 * s][c] = (q[2 * s][c] & 0xFE) | bit;
                q[2 * s + 1][c] = (q[2 * s + 1][c] & 0xFE) | bit;
            }
        }
    }

    uint64_t indices = 0;
    float error = 0.f;
#pragma unroll
    for (int s = 0; s < kSubsets; ++s)
    {
        if (CalculateIndices<C>(pixels, subsets.mask[s], subsets.anchor[s], kIndexBits, kEndpointBits, q[2 * s], q[2 * s + 1], indices))
        {
#pragma unroll
            for (int c = 0; c < C; ++c)
            {
                const int t = q[2 * s][c];
                q[2 * s][c] = q[2 * s + 1][c];
                q[2 * s + 1][c] = t;
            }
        }
        if (!kSingleMode)
        {
            const float subsetError = ComputeError<C>(pixels, indices, subsets.mask[s], q[2 * s], q[2 * s + 1], kIndexBits, kEndpointBits);
            error = s == 0 ? subsetError : error + subsetError;
        }
    }
    if (error > currentError)
        return;

    BlockBits bits;
    bits.Put(kMode + 1, 1u << kMode);
    if (Traits::kPartitionBits)
        bits.Put(Traits::kPartitionBits, uint32_t(partition));
    constexpr int kStoredBits = Traits::kPBits ? kEndpointBits - 1 : kEndpointBits;
#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
        for (int i = 0; i < 2 * kSubsets; ++i)
            bits.Put(kStoredBits, uint32_t(q[i][c]) >> (Traits::kPBits ? 1 : 0));
    if (Traits::kPBits == 1)
    {
#pragma unroll
        for (int i = 0; i < 2 * kSubsets; ++i)
            bits.Put(1, uint32_t(q[i][0]));
    }
    else if (Traits::kPBits == 2)
    {
#pragma unroll
        for (int s = 0; s < kSubsets; ++s)
            bits.Put(1, uint32_t(q[2 * s][0]));
    }
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
    {
        const bool anchor = i == 0 || (kSubsets > 1 && i == subsets.anchor[1]) || (kSubsets > 2 && i == subsets.anchor[2]);
        bits.Put(anchor ? kIndexBits - 1 : kIndexBits, uint32_t(indices >> (4 * i)) & 15u);
    }
    currentError = error;
    currentBlock = bits.Words();
}

// The endpoints a partition starts from: per subset the extremes of each component, components swapped
// where they run against each other (not for mode 7: the shader leaves that out).
template <int C, int kSubsets, bool kSwap>
__device__ __forceinline__ void StartingEndpoints(const Pixels& pixels, const Subsets& subsets, Vec<C>* ep)
{
#pragma unroll
    for (int s = 0; s < kSubsets; ++s)
    {
        MinMax<C>(pixels, subsets.mask[s], ep[2 * s], ep[2 * s + 1]);
        if (kSwap)
            SwapEndpointComponents<C>(pixels, subsets.mask[s], ep[2 * s], ep[2 * s + 1]);
    }
}

// The partition of `kSubsets` subsets with the smallest estimated error (the first one on ties) and its
// starting endpoints (the loops of BC7_Mode0_2_Compress :724-775, BC7_Mode1_3_Compress :930-979,
// BC7_Mode7_Compress :1296-1335).
template <int C, int kSubsets, bool kSwap>
__device__ int SearchPartitions(const Pixels& pixels, int searchIndexBits, Vec<C>* bestEndpoints)
{
    int best = 0;
    float bestError = FLT_MAX;
#pragma unroll 1
    for (int partition = 0; partition < 64; ++partition)
    {
        const Subsets subsets = kSubsets == 3 ? ThreeSubsets(partition) : TwoSubsets(partition);
        Vec<C> ep[2 * kSubsets];
        StartingEndpoints<C, kSubsets, kSwap>(pixels, subsets, ep);
        float error = 0.f;
#pragma unroll
        for (int s = 0; s < kSubsets; ++s)
        {
            const float subsetError = EstimateError<C>(pixels, subsets.mask[s], ep[2 * s], ep[2 * s + 1], searchIndexBits);
            error = s == 0 ? subsetError : error + subsetError;
        }
        if (error < bestError)
        {
            best = partition;
            bestError = error;
#pragma unroll
            for (int i = 0; i < 2 * kSubsets; ++i)
                bestEndpoints[i] = ep[i];
        }
    }
    return best;
}

// ---- modes 4 and 5: a colour plane and a scalar plane with indices of their own ----------------------
// mode 4: 5-bit colours, 6-bit scalar, 2- and 3-bit indices (kSelector: the colours get the 3-bit ones);
// mode 5: 7-bit colours, 8-bit scalar, 2-bit indices for both.  (BC7_Mode4_Compress_Internal :982-1069,
// BC7_Mode5_Compress_Internal :1071-1147.)
template <int kMode, bool kSelector, bool kSingleMode>
__device__ void EncodeDualPlane(const Pixels& pixels, float& currentError, uint4& currentBlock)
{
    constexpr int kColorIndexBits = kMode == 5 ? 2 : kSelector ? 3 : 2;
    constexpr int kScalarIndexBits = kMode == 5 ? 2 : kSelector ? 2 : 3;
    constexpr int kColorBits = kMode == 5 ? 7 : 5, kScalarBits = kMode == 5 ? 8 : 6;

    Vec<1> s0, s1;
    MinMax<1>(pixels, kAllPixels, s0, s1);
    OptimizeEndpoints<1>(pixels, kAllPixels, s0, s1, kScalarIndexBits);
    Vec<3> c0, c1;
    MinMax<3>(pixels, kAllPixels, c0, c1);
    SwapEndpointComponents<3>(pixels, kAllPixels, c0, c1);
    OptimizeEndpoints<3>(pixels, kAllPixels, c0, c1, kColorIndexBits);

    int q0[3], q1[3], a0[1], a1[1];
#pragma unroll
    for (int c = 0; c < 3; ++c)
    {
        q0[c] = Quantize(c0.v[c], kColorBits);
        q1[c] = Quantize(c1.v[c], kColorBits);
    }
    a0[0] = Quantize(s0.v[0], kScalarBits);
    a1[0] = Quantize(s1.v[0], kScalarBits);

    uint64_t colorIndices = 0, scalarIndices = 0;
    float error = 0.f;
    if (CalculateIndices<3>(pixels, kAllPixels, 0, kColorIndexBits, kColorBits, q0, q1, colorIndices))
    {
#pragma unroll
        for (int c = 0; c < 3; ++c)
        {
            const int t = q0[c];
            q0[c] = q1[c];
            q1[c] = t;
        }
    }
    if (!kSingleMode)
        error = ComputeError<3>(pixels, colorIndices, kAllPixels, q0, q1, kColorIndexBits, kColorBits);
    if (CalculateIndices<1>(pixels, kAllPixels, 0, kScalarIndexBits, kScalarBits, a0, a1, scalarIndices))
    {
        const int t = a0[0];
        a0[0] = a1[0];
        a1[0] = t;
    }
    if (!kSingleMode)
        error += ComputeError<1>(pixels, scalarIndices, kAllPixels, a0, a1, kScalarIndexBits, kScalarBits);
    if (error > currentError)
        return;

    BlockBits bits;
    bits.Put(kMode + 1, 1u << kMode);
    bits.Put(2, uint32_t(pixels.rotation));
    if (kMode == 4)
        bits.Put(1, kSelector ? 1u : 0u);
#pragma unroll
    for (int c = 0; c < 3; ++c)
    {
        bits.Put(kColorBits, uint32_t(q0[c]));
        bits.Put(kColorBits, uint32_t(q1[c]));
    }
    bits.Put(kScalarBits, uint32_t(a0[0]));
    bits.Put(kScalarBits, uint32_t(a1[0]));
    // mode 4 stores its 2-bit indices first, whichever plane they belong to; mode 5 colours, then scalar
    const bool scalarFirst = kMode == 4 && kSelector;
    const uint64_t first = scalarFirst ? scalarIndices : colorIndices, second = scalarFirst ? colorIndices : scalarIndices;
    const int firstBits = scalarFirst ? kScalarIndexBits : kColorIndexBits, secondBits = scalarFirst ? kColorIndexBits : kScalarIndexBits;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        bits.Put(i == 0 ? firstBits - 1 : firstBits, uint32_t(first >> (4 * i)) & 15u);
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        bits.Put(i == 0 ? secondBits - 1 : secondBits, uint32_t(second >> (4 * i)) & 15u);
    currentError = error;
    currentBlock = bits.Words();
}

// ---- the kernel -----------------------------------------------------------------------------------------
struct Bc7Arguments
{
    BlockCompressArguments base;
    int numChannels;            // channels that feed the block: red, green, blue, alpha; missing ones read 0, alpha 1
    const uint32_t* modeBuffer; // null: full search
    uint32_t modeBufferByteOffset, modeMapWidthInBlocks, modeMapHeightInBlocks;
    int modeMapOffsetX, modeMapOffsetY;
};

// The block a wrong or missing mode-buffer entry produces: four 2x2 squares, black, red, green, blue
// (CompressBC7.hlsl:1537-1545).
__device__ __forceinline__ uint4 MissingModeBlock()
{
    return make_uint4(0x00f80004u, 0x0001f000u, 0x3ff0001fu, 0x1f9e0000u);
}

// Mode and partition of a block from the 9-bit entries of a mode buffer (LoadModeAndPartition, :1409-1444,
// including the way it forms the word address: the byte offset is added before the mask is applied).
__device__ __forceinline__ bool LoadModeAndPartition(const Bc7Arguments& args, int blockX, int blockY, uint32_t& mode, uint32_t& partition)
{
    const uint32_t x = uint32_t(blockX + args.modeMapOffsetX), y = uint32_t(blockY + args.modeMapOffsetY);
    if (x >= args.modeMapWidthInBlocks || y >= args.modeMapHeightInBlocks)
        return false;
    const uint32_t firstBit = (y * args.modeMapWidthInBlocks + x) * 9u;
    const uint32_t wordOffset = (args.modeBufferByteOffset + (firstBit >> 3)) & ~3u;
    const uint32_t bitOffset = firstBit & 31u;
    const uint32_t low = args.modeBuffer[wordOffset >> 2];
    uint32_t entry = low >> bitOffset;
    if (bitOffset + 9u > 32u)
        entry |= args.modeBuffer[(wordOffset >> 2) + 1] << (32u - bitOffset);
    entry &= 0x1ffu;
    if (entry == 0u)
        return false; // reserved: nothing was stored for this block
    if (entry == 0x1bfu)
        entry = 0u; // mode 0, partition 0 (stored as the otherwise impossible mode 6, partition 63)
    mode = (entry >> 6) & 7u;
    partition = entry & 0x3fu;
    return true;
}

// One block: with a mode buffer the one configuration it names, otherwise the best of all
// (CompressBC7.hlsl main(), :1548-1587).  texels: the block's texel i at texels[i * kThreads].
template <bool kSingleMode>
__device__ uint4 EncodeBlock(const uint2* texels, uint32_t mode, uint32_t partition)
{
    Pixels pixels;
    pixels.base = texels;
    pixels.rotation = 0;
    float error = FLT_MAX;
    uint4 block = make_uint4(0u, 0u, 0u, 0u);

    if (kSingleMode)
    {
        switch (mode)
        {
        case 0:
        case 2:
        {
            const Subsets subsets = ThreeSubsets(int(partition));
            Vec<3> ep[6];
            StartingEndpoints<3, 3, true>(pixels, subsets, ep);
            if (mode == 0)
                FinalizeMode<0, true>(pixels, int(partition), subsets, ep, error, block);
            else
                FinalizeMode<2, true>(pixels, int(partition), subsets, ep, error, block);
            break;
        }
        case 1:
        case 3:
        {
            const Subsets subsets = TwoSubsets(int(partition));
            Vec<3> ep[4];
            StartingEndpoints<3, 2, true>(pixels, subsets, ep);
            if (mode == 1)
                FinalizeMode<1, true>(pixels, int(partition), subsets, ep, error, block);
            else
                FinalizeMode<3, true>(pixels, int(partition), subsets, ep, error, block);
            break;
        }
        case 4:
        case 5:
            // the partition field of these modes: rotation in bits 0-1, mode 4's index selector in bit 2
            pixels.rotation = int(partition & 3u);
            if (mode == 5)
                EncodeDualPlane<5, false, true>(pixels, error, block);
            else if (partition & 4u)
                EncodeDualPlane<4, true, true>(pixels, error, block);
            else
                EncodeDualPlane<4, false, true>(pixels, error, block);
            break;
        case 6:
        {
            const Subsets subsets = {{kAllPixels, 0u, 0u}, {0, 0, 0}};
            Vec<4> ep[2];
            StartingEndpoints<4, 1, true>(pixels, subsets, ep);
            FinalizeMode<6, true>(pixels, 0, subsets, ep, error, block);
            break;
        }
        default:
        {
            const Subsets subsets = TwoSubsets(int(partition));
            Vec<4> ep[4];
            StartingEndpoints<4, 2, false>(pixels, subsets, ep);
            FinalizeMode<7, true>(pixels, int(partition), subsets, ep, error, block);
            break;
        }
        }
    }
    else
    {
        // the three-component modes cannot hold alpha: only for blocks without a texel of alpha < 1
        bool opaque = true;
#pragma unroll 1
        for (int i = 0; i < 16; ++i)
            if (Pixel<4>(pixels, i).v[3] < 1.0f)
                opaque = false;
        if (opaque)
        {
            {
                Vec<3> ep[6];
                const int best = SearchPartitions<3, 3, true>(pixels, 3, ep);
                const Subsets subsets = ThreeSubsets(best);
                if (best < 16)
                    FinalizeMode<0, false>(pixels, best, subsets, ep, error, block);
                FinalizeMode<2, false>(pixels, best, subsets, ep, error, block);
            }
            {
                Vec<3> ep[4];
                const int best = SearchPartitions<3, 2, true>(pixels, 3, ep);
                const Subsets subsets = TwoSubsets(best);
                FinalizeMode<1, false>(pixels, best, subsets, ep, error, block);
                FinalizeMode<3, false>(pixels, best, subsets, ep, error, block);
            }
        }
#pragma unroll 1
        for (int rotation = 0; rotation < 4; ++rotation)
        {
            pixels.rotation = rotation;
            EncodeDualPlane<4, false, false>(pixels, error, block);
            EncodeDualPlane<4, true, false>(pixels, error, block);
            EncodeDualPlane<5, false, false>(pixels, error, block);
        }
        pixels.rotation = 0;
        {
            const Subsets subsets = {{kAllPixels, 0u, 0u}, {0, 0, 0}};
            Vec<4> ep[2];
            StartingEndpoints<4, 1, true>(pixels, subsets, ep);
            FinalizeMode<6, false>(pixels, 0, subsets, ep, error, block);
        }
        {
            Vec<4> ep[4];
            const int best = SearchPartitions<4, 2, false>(pixels, 2, ep);
            FinalizeMode<7, false>(pixels, best, TwoSubsets(best), ep, error, block);
        }
    }
    return block;
}

template <bool kSingleMode>
__global__ void __launch_bounds__(kThreads) Bc7Kernel(const Bc7Arguments args)
{
    __shared__ uint2 staged[16 * kThreads];
    __shared__ uint32_t binCount[2 * kThreads + 1]; // blocks per (mode, partition) pair, then where each pair's blocks start
    __shared__ uint32_t warpTotal[kThreads / 32];
    __shared__ uint32_t order[kThreads];

    const int tid = threadIdx.x;
    if (kSingleMode)
    {
        binCount[tid] = 0;
        binCount[tid + kThreads] = 0;
        if (tid == 0)
            binCount[2 * kThreads] = 0;
    }
    // The CTA's 128 x 32 texels, neighbouring threads on neighbouring texels of a row, handed to the slot of
    // their block through shared memory; red-green and blue-alpha as two 32-bit words.
    const bool pairs = !(args.base.firstChannel & 1) && !(args.base.channels & 1);
#pragma unroll 1
    for (int k = 0; k < 16; ++k)
    {
        const int p = k * kThreads + tid;
        const int localX = p & (4 * kGroupWidth - 1), localY = p / (4 * kGroupWidth);
        const int x = args.base.srcLeft + blockIdx.x * (4 * kGroupWidth) + localX, y = args.base.srcTop + blockIdx.y * (4 * kGroupHeight) + localY;
        uint32_t redGreen = 0u, blueAlpha = 0u; // outside the mip every component reads 0
        if (x < args.base.width && y < args.base.height)
        {
            const int first = args.base.firstChannel, count = args.numChannels;
            if (pairs)
            {
                redGreen = count >= 2 ? LoadPair(args.base, x, y, first) : uint32_t(__half_as_ushort(LoadHalf(args.base, x, y, first)));
                blueAlpha = count == 4 ? LoadPair(args.base, x, y, first + 2)
                          : (count == 3 ? uint32_t(__half_as_ushort(LoadHalf(args.base, x, y, first + 2))) : 0u) | 0x3c000000u;
            }
            else
            {
                uint32_t c[4] = {0u, 0u, 0u, 0x3c00u};
#pragma unroll
                for (int channel = 0; channel < 4; ++channel)
                    if (channel < count)
                        c[channel] = __half_as_ushort(LoadHalf(args.base, x, y, first + channel));
                redGreen = c[0] | (c[1] << 16);
                blueAlpha = c[2] | (c[3] << 16);
            }
        }
        const int owner = (localY >> 2) * kGroupWidth + (localX >> 2), texel = (localY & 3) * 4 + (localX & 3);
        staged[texel * kThreads + owner] = make_uint2(redGreen, blueAlpha);
    }

    int slot = tid;
    uint32_t mode = 0, partition = 0;
    bool active;
    {
        const int blockX = blockIdx.x * kGroupWidth + (tid & (kGroupWidth - 1));
        const int blockY = blockIdx.y * kGroupHeight + tid / kGroupWidth;
        active = blockX < args.base.widthInBlocks && blockY < args.base.heightInBlocks;
        if (kSingleMode)
        {
            if (active && !LoadModeAndPartition(args, blockX, blockY, mode, partition))
            {
                reinterpret_cast<uint4*>(args.base.blocks + size_t(blockY) * args.base.rowPitch)[blockX] = MissingModeBlock();
                active = false;
            }
            // Threads trade blocks so that those of one mode AND partition sit next to each other: a warp then
            // runs one encoder, and its lanes loop over the same subsets (sorted by mode alone, as the shader
            // does, half of the lanes idle in the pixel loops: 16 active lanes per instruction).  A counting
            // sort over the 512 (mode, partition) pairs, blocks without work last.
            __syncthreads();
            const uint32_t key = active ? (mode << 6 | partition) : 512u;
            const uint32_t rank = atomicAdd(&binCount[key], 1u);
            __syncthreads();
            {
                // exclusive prefix sum of the bins: two per thread, scanned within the warp, then over the warps
                const uint32_t first = binCount[2 * tid], second = binCount[2 * tid + 1], pair = first + second;
                uint32_t inclusive = pair;
#pragma unroll
                for (int delta = 1; delta < 32; delta *= 2)
                {
                    const uint32_t below = __shfl_up_sync(0xFFFFFFFFu, inclusive, delta);
                    if ((tid & 31) >= delta)
                        inclusive += below;
                }
                if ((tid & 31) == 31)
                    warpTotal[tid >> 5] = inclusive;
                __syncthreads();
                uint32_t start = inclusive - pair;
                for (int w = 0; w < (tid >> 5); ++w)
                    start += warpTotal[w];
                binCount[2 * tid] = start;
                binCount[2 * tid + 1] = start + first;
                if (tid == kThreads - 1)
                    binCount[512] = start + pair;
            }
            __syncthreads();
            order[binCount[key] + rank] = uint32_t(tid) | (partition << 16) | ((active ? mode : 8u) << 24);
            __syncthreads();
            const uint32_t task = order[tid];
            slot = int(task & 0xffffu);
            partition = (task >> 16) & 0x3fu;
            mode = task >> 24;
            active = mode < 8u;
        }
        else
            __syncthreads();
    }
    if (!active)
        return;

    const uint4 block = EncodeBlock<kSingleMode>(staged + slot, mode, partition);
    const int blockX = blockIdx.x * kGroupWidth + (slot & (kGroupWidth - 1));
    const int blockY = blockIdx.y * kGroupHeight + slot / kGroupWidth;
    reinterpret_cast<uint4*>(args.base.blocks + size_t(blockY) * args.base.rowPitch)[blockX] = block;
}

} // namespace

int LaunchBlockCompressBc7(const NtcbBlockCompressParams& params, const BlockCompressArguments& base, cudaStream_t stream)
{
    Bc7Arguments args;
    args.base = base;
    args.numChannels = base.formatChannels;
    args.modeBuffer = static_cast<const uint32_t*>(params.deviceModeBuffer);
    args.modeBufferByteOffset = params.modeBufferByteOffset;
    args.modeMapWidthInBlocks = params.modeMapWidthInBlocks;
    args.modeMapHeightInBlocks = params.modeMapHeightInBlocks;
    args.modeMapOffsetX = params.modeMapOffsetX;
    args.modeMapOffsetY = params.modeMapOffsetY;
    if (args.modeBuffer)
    {
        if (args.modeMapWidthInBlocks == 0 || args.modeMapHeightInBlocks == 0)
        {
            SetError("modeMapWidthInBlocks and modeMapHeightInBlocks must be non-zero when a mode buffer is given.");
            return NTCB_ERR_INVALID_ARGUMENT;
        }
        if (reinterpret_cast<uintptr_t>(params.deviceModeBuffer) % 4 != 0)
        {
            SetError("deviceModeBuffer must be aligned to 4 bytes.");
            return NTCB_ERR_INVALID_ARGUMENT;
        }
    }
    const dim3 grid(unsigned(base.widthInBlocks + kGroupWidth - 1) / kGroupWidth, unsigned(base.heightInBlocks + kGroupHeight - 1) / kGroupHeight);
    if (args.modeBuffer)
        Bc7Kernel<true><<<grid, kThreads, 0, stream>>>(args);
    else
        Bc7Kernel<false><<<grid, kThreads, 0, stream>>>(args);
    CountLaunch();
    const cudaError_t error = cudaGetLastError();
    if (error != cudaSuccess)
        return CudaFailure("Bc7Kernel", error);
    ClearError();
    return NTCB_OK;
}

} // namespace ntcb

using namespace ntcb;

// ntc::GetBC7ModeBufferSize (src/PublicFunctions.cpp:470-474).
extern "C" size_t ntcb_bc7_mode_buffer_size(int widthInBlocks, int heightInBlocks)
{
    if (widthInBlocks <= 0 || heightInBlocks <= 0)
        return 0;
    const size_t blocks = size_t(widthInBlocks) * size_t(heightInBlocks);
    return ((blocks * 9 + 31) >> 5) << 2;
}

// ntc::MakeBC7ModeBuffer (src/PublicFunctions.cpp:488-556): same checks, same layout; the buffer is cleared first.
extern "C" int ntcb_make_bc7_mode_buffer(int widthInBlocks, int heightInBlocks, const void* blockData, size_t blockDataSize,
    size_t rowPitch, void* modeBuffer, size_t modeBufferSize)
{
    if (!blockData)
    {
        SetError("blockData is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (!modeBuffer)
    {
        SetError("modeBuffer is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (widthInBlocks <= 0 || heightInBlocks <= 0)
    {
        SetError("widthInBlocks (%d) and heightInBlocks (%d) must be > 0.", widthInBlocks, heightInBlocks);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    const size_t bytesPerBlock = 16;
    const size_t expectedRowPitch = size_t(widthInBlocks) * bytesPerBlock;
    if (rowPitch < expectedRowPitch || rowPitch % bytesPerBlock != 0)
    {
        SetError("Invalid rowPitch (%zu), must be at least %zu and a multiple of %zu.", rowPitch, expectedRowPitch, bytesPerBlock);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const size_t expectedSize = size_t(heightInBlocks) * rowPitch;
    if (blockDataSize < expectedSize)
    {
        SetError("Size of BC7 block data (%zu bytes) does not match the expected size (%zu bytes).", blockDataSize, expectedSize);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const size_t expectedModeBufferSize = ntcb_bc7_mode_buffer_size(widthInBlocks, heightInBlocks);
    if (modeBufferSize < expectedModeBufferSize)
    {
        SetError("Size of BC7 mode buffer (%zu bytes) is smaller than the expected size (%zu bytes).", modeBufferSize, expectedModeBufferSize);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const uint8_t* blocks = static_cast<const uint8_t*>(blockData);
    uint8_t* entries = static_cast<uint8_t*>(modeBuffer);
    memset(entries, 0, expectedModeBufferSize);
    static const uint32_t partitionMask[8] = {15, 63, 63, 63, 7, 3, 0, 63};
    for (int row = 0; row < heightInBlocks; ++row)
        for (int column = 0; column < widthInBlocks; ++column)
        {
            uint32_t firstWord;
            memcpy(&firstWord, blocks + size_t(row) * rowPitch + size_t(column) * bytesPerBlock, 4);
            // the mode is the position of the lowest set bit of the block; what follows it selects the partition
            // (modes 4 and 5: rotation and index selector)
            uint32_t mode = 0;
            while (mode < 7 && !((firstWord >> mode) & 1u))
                ++mode;
            const uint32_t partition = (firstWord >> (mode + 1)) & partitionMask[mode];
            uint32_t entry = (mode << 6) | partition;
            if (entry == 0)
                entry = 0x1bf; // 0 means "no entry": mode 0, partition 0 is stored as mode 6, partition 63
            const size_t bitAddress = (size_t(row) * size_t(widthInBlocks) + size_t(column)) * 9;
            const size_t byteOffset = bitAddress / 8;
            const uint32_t bitOffset = uint32_t(bitAddress & 7);
            entries[byteOffset] |= uint8_t(entry << bitOffset);
            entries[byteOffset + 1] |= uint8_t(entry >> (8 - bitOffset));
        }
    ClearError();
    return NTCB_OK;
}
