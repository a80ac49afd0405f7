// BC1 - BC5 encoding of decoded texels: the "decompress on load, then block-compress" step that the
// reference runs as compute shaders through a graphics API (IContext::MakeBlockCompressionComputePass,
// src/Context.cpp:630-779; src/shaders/CompressBC1-5.hlsl, src/shaders/BlockCompressCommon.hlsli),
// here as CUDA kernels on the decode output.  First part: BC4 / BC5 (BC4_CompressFast, :510-796);
// second part: the BC1 colour block and the formats built on it.
//
// The BC4 encoder follows the shader's algorithm: quantise the 16 values to 8 bits; start from endpoints
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

#include <mutex>

#include "block_compress.h"
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

// The sixteen 8-bit values of a block, packed: the loops over the texels stay rolled (a dynamic
// shift instead of a register array), which keeps the encoder's code a few hundred instructions.
// Fully unrolled, the kernel spent most of its issue slots waiting for instructions (ncu: stall
// "no_instruction" 3.7 per issue).
struct BlockValues
{
    uint64_t low = 0, high = 0; // texels 0-7 and 8-15, one byte each

    __device__ __forceinline__ void Set(int pixel, uint32_t value)
    {
        if (pixel < 8)
            low |= uint64_t(value) << (8 * pixel);
        else
            high |= uint64_t(value) << (8 * (pixel - 8));
    }
    __device__ __forceinline__ uint32_t operator[](int pixel) const
    {
        return uint32_t((pixel < 8 ? low : high) >> (8 * (pixel & 7))) & 0xffu;
    }
};

// Nearest palette entry per pixel, the first one on ties; returns the block's squared error
// (BC4_ComputeAlphaIndices, :605-632).
__device__ uint32_t AssignIndices(const BlockValues& values, Bc4Block& block)
{
    uint32_t palette[8];
    Palette(block.alpha0, block.alpha1, palette);
    uint64_t indices = 0;
    uint32_t total = 0;
#pragma unroll 1
    for (int pixel = 0; pixel < 16; ++pixel)
    {
        int best = 0x7fffffff;
        uint32_t bestIndex = 0;
        const uint32_t value = values[pixel];
#pragma unroll
        for (uint32_t p = 0; p < 8; ++p)
        {
            const int difference = int(value) - int(palette[p]);
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
__device__ void RefitEight(const BlockValues& values, Bc4Block& block, bool zeroAlpha1, bool oneAlpha0)
{
    RefitSums sums;
#pragma unroll 1
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
__device__ void RefitSix(const BlockValues& values, Bc4Block& block)
{
    RefitSums sums;
#pragma unroll 1
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
__device__ void Refine(const BlockValues& values, Bc4Block& block, Bc4Block& best, uint32_t& bestError, bool zeroAlpha1,
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
    BlockValues values;
    uint32_t low = 255, high = 0, lowInside = 255, highInside = 0;
#pragma unroll
    for (int pixel = 0; pixel < 16; ++pixel)
    {
        // saturate() sends NaN to 0
        const float saturated = pixels[pixel] != pixels[pixel] ? 0.f : fminf(fmaxf(pixels[pixel], 0.f), 1.f);
        const uint32_t v = uint32_t(rintf(__fmul_rn(saturated, 255.f)));
        values.Set(pixel, v);
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
    {
        const int x = args.srcLeft + blockX * 4 + (pixel & 3), y = args.srcTop + blockY * 4 + (pixel >> 2);
        // a negative channel: the constant 1 inside the mip (the alpha of texels that carry none)
        pixels[pixel] = args.firstChannel >= 0 ? LoadChannel(args, x, y, args.firstChannel + c)
                                               : (x < args.width && y < args.height ? 1.f : 0.f);
    }
    uint8_t* destination = args.blocks + size_t(blockY) * args.rowPitch + size_t(blockX) * (8 * args.formatChannels);
    reinterpret_cast<uint2*>(destination)[c] = EncodeBc4(pixels);
}

// ---------------------------------------------------------------------------------------------
// BC1 colour blocks (BlockCompressCommon.hlsli:82-493), alone (BC1, with punch-through alpha) or
// beside an alpha block (BC2: 4-bit alpha, BC3: a BC4 block)

// Single-colour match tables: for an 8-bit value, the pair of 5- or 6-bit endpoints (low byte: the
// one weighted 2/3, high byte: the one weighted 1/3) whose interpolant comes closest, with a small
// penalty on the distance between the endpoints.  Filled by FillMatchTable below.
__constant__ uint16_t kMatch5[256];
__constant__ uint16_t kMatch6[256];

struct Rgb
{
    float r, g, b;
};

struct Texel
{
    Rgb rgb;
    float a;
};

__device__ __forceinline__ float Mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float Add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float Sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float Saturate(float x) { return x != x ? 0.f : fminf(fmaxf(x, 0.f), 1.f); }

__device__ __forceinline__ Rgb Sub(Rgb a, Rgb b) { return {Sub(a.r, b.r), Sub(a.g, b.g), Sub(a.b, b.b)}; }
__device__ __forceinline__ Rgb Add(Rgb a, Rgb b) { return {Add(a.r, b.r), Add(a.g, b.g), Add(a.b, b.b)}; }
__device__ __forceinline__ Rgb Scale(Rgb a, float s) { return {Mul(a.r, s), Mul(a.g, s), Mul(a.b, s)}; }
__device__ __forceinline__ Rgb Saturate(Rgb a) { return {Saturate(a.r), Saturate(a.g), Saturate(a.b)}; }
__device__ __forceinline__ float Dot(Rgb a, Rgb b) { return Add(Add(Mul(a.r, b.r), Mul(a.g, b.g)), Mul(a.b, b.b)); }
__device__ __forceinline__ float Distance(Rgb a, Rgb b) { const Rgb d = Sub(a, b); return Dot(d, d); }
// lerp(x, y, s) = x + s * (y - x)
__device__ __forceinline__ Rgb Lerp(Rgb x, Rgb y, float s) { return Add(x, Scale(Sub(y, x), s)); }
__device__ __forceinline__ float Dot4(const Texel& t)
{
    return Add(Add(Add(Mul(t.rgb.r, t.rgb.r), Mul(t.rgb.g, t.rgb.g)), Mul(t.rgb.b, t.rgb.b)), Mul(t.a, t.a));
}

__device__ __forceinline__ Rgb Expand565(uint32_t w)
{
    return {__fdiv_rn(float((w >> 11) & 0x1f), 31.f), __fdiv_rn(float((w >> 5) & 0x3f), 63.f), __fdiv_rn(float(w & 0x1f), 31.f)};
}

__device__ __forceinline__ Rgb RoundTo565(Rgb v, uint32_t& w)
{
    const uint32_t x = uint32_t(rintf(Mul(Saturate(v.r), 31.f)));
    const uint32_t y = uint32_t(rintf(Mul(Saturate(v.g), 63.f)));
    const uint32_t z = uint32_t(rintf(Mul(Saturate(v.b), 31.f)));
    w = (x << 11) | (y << 5) | z;
    return Expand565(w);
}

// The smallest of four distances, the pairs (0, 1) and (2, 3) compared first (BC1_SelectBestIndex).
__device__ __forceinline__ uint32_t SelectIndex(float d0, float d1, float d2, float d3, float& error)
{
    if (fminf(d0, d1) < fminf(d2, d3))
    {
        error = d0 < d1 ? d0 : d1;
        return d0 < d1 ? 0u : 1u;
    }
    error = d2 < d3 ? d2 : d3;
    return d2 < d3 ? 2u : 3u;
}

struct Palette4
{
    Rgb c0, c1, c2, c3;
    __device__ Palette4(Rgb maxColor, Rgb minColor)
        : c0(maxColor), c1(minColor), c2(Lerp(maxColor, minColor, 1.0f / 3.0f)), c3(Lerp(maxColor, minColor, 2.0f / 3.0f))
    {
    }
    __device__ __forceinline__ uint32_t Index(const Texel& t, float& error) const // BC1_ComputeIndex4
    {
        const float transparency = Sub(1.f, t.a);
        const float alphaDistance = Mul(transparency, transparency);
        return SelectIndex(Add(Distance(c0, t.rgb), alphaDistance), Add(Distance(c1, t.rgb), alphaDistance),
            Add(Distance(c2, t.rgb), alphaDistance), Add(Distance(c3, t.rgb), alphaDistance), error);
    }
};

struct Palette3
{
    Rgb c0, c1, c2;
    float alphaThreshold;
    __device__ Palette3(Rgb maxColor, Rgb minColor, float threshold)
        : c0(maxColor), c1(minColor), c2(Lerp(maxColor, minColor, 0.5f)), alphaThreshold(threshold)
    {
    }
    __device__ __forceinline__ uint32_t Index(const Texel& t, float& error) const // BC1_ComputeIndex3
    {
        if (t.a <= alphaThreshold)
        {
            error = 0.f;
            return 3u;
        }
        const float transparency = Sub(1.f, t.a);
        const float alphaDistance = Mul(transparency, transparency);
        return SelectIndex(Add(Distance(c0, t.rgb), alphaDistance), Add(Distance(c1, t.rgb), alphaDistance),
            Add(Distance(c2, t.rgb), alphaDistance), Dot4(t), error);
    }
};

// Extremes of the block per component, with the green and blue ends swapped where they run against
// the reference axis (negative covariance), then pulled inwards by `insetDivisor`-th of the extent.
struct Extremes
{
    Rgb low{1.f, 1.f, 1.f}, high{0.f, 0.f, 0.f}, sums{0.f, 0.f, 0.f};

    __device__ __forceinline__ void Include(Rgb c)
    {
        sums = Add(sums, c);
        low = {fminf(low.r, c.r), fminf(low.g, c.g), fminf(low.b, c.b)};
        high = {fmaxf(high.r, c.r), fmaxf(high.g, c.g), fmaxf(high.b, c.b)};
    }
};

struct Covariance
{
    float rg = 0.f, rb = 0.f, gb = 0.f;
    __device__ __forceinline__ void Include(Rgb c, Rgb center)
    {
        const Rgb d = Sub(c, center);
        rg = Add(rg, Mul(d.r, d.g));
        rb = Add(rb, Mul(d.r, d.b));
        gb = Add(gb, Mul(d.g, d.b));
    }
};

__device__ __forceinline__ void Swap(float& a, float& b)
{
    const float t = a;
    a = b;
    b = t;
}

__device__ __forceinline__ void OrientAndInset(Extremes& e, const Covariance& cov, float insetDivisor)
{
    if (e.low.r != e.high.r)
    {
        if (cov.rg < 0.f) Swap(e.low.g, e.high.g);
        if (cov.rb < 0.f) Swap(e.low.b, e.high.b);
    }
    else if (e.low.g != e.high.g)
    {
        if (cov.gb < 0.f) Swap(e.low.b, e.high.b);
    }
    const Rgb extent = Sub(e.high, e.low);
    const Rgb inset = {__fdiv_rn(extent.r, insetDivisor), __fdiv_rn(extent.g, insetDivisor), __fdiv_rn(extent.b, insetDivisor)};
    e.high = Saturate(Sub(e.high, inset));
    e.low = Saturate(Add(e.low, inset));
}

struct ColorRefit
{
    float alpha2 = 0.f, beta2 = 0.f, alphaBeta = 0.f;
    Rgb alphaX{0.f, 0.f, 0.f}, betaX{0.f, 0.f, 0.f};

    __device__ __forceinline__ void Include(float beta, Rgb c)
    {
        const float alpha = Sub(1.f, beta);
        alpha2 = Add(alpha2, Mul(alpha, alpha));
        beta2 = Add(beta2, Mul(beta, beta));
        alphaBeta = Add(alphaBeta, Mul(alpha, beta));
        alphaX = Add(alphaX, Scale(c, alpha));
        betaX = Add(betaX, Scale(c, beta));
    }
    // The least-squares endpoints, when the system is well conditioned.
    __device__ __forceinline__ bool Solve(Rgb& a, Rgb& b) const
    {
        const float denominator = Sub(Mul(alpha2, beta2), Mul(alphaBeta, alphaBeta));
        if (!(fabsf(denominator) > 0.0001f))
            return false;
        const float factor = __fdiv_rn(1.f, denominator);
        a = Scale(Sub(Scale(alphaX, beta2), Scale(betaX, alphaBeta)), factor);
        b = Scale(Sub(Scale(betaX, alpha2), Scale(alphaX, alphaBeta)), factor);
        return true;
    }
};

// A component already at 0 or 1 stays there; the others take the refitted value.
__device__ __forceinline__ float KeepExtreme(float current, float refitted)
{
    return (current == 0.f || current == 1.f) ? current : Saturate(refitted);
}
__device__ __forceinline__ Rgb KeepExtremes(Rgb current, Rgb refitted)
{
    return {KeepExtreme(current.r, refitted.r), KeepExtreme(current.g, refitted.g), KeepExtreme(current.b, refitted.b)};
}

// The sixteen texels of a block, staged in shared memory as four halves each (the input is fp16, so
// nothing is lost), texel i of thread t at word i * 128 + t: conflict-free to read, and indexable, so
// the loops over the texels stay rolled.  Held in registers (64 of them) with every loop unrolled, the
// BC1 kernel needed 158 registers and waited for instructions.
struct BlockTexels
{
    const uint2* base;
    bool opaque; // alpha reads as 1

    __device__ __forceinline__ Texel operator[](int i) const
    {
        const uint2 raw = base[i * 128];
        const float2 rg = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        const float2 ba = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
        return {{rg.x, rg.y, ba.x}, opaque ? 1.f : ba.y};
    }
    __device__ __forceinline__ float Alpha(int i) const
    {
        return __high2float(*reinterpret_cast<const __half2*>(&base[i * 128].y));
    }
};

// The whole block as one colour, through the match tables (BC1_EncodeSingleColor, :205-247).
__device__ uint2 EncodeSingleColor(const BlockTexels& texels, float& blockError)
{
    Rgb sum{0.f, 0.f, 0.f};
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        sum = Add(sum, texels[i].rgb);
    const Rgb average = {__fdiv_rn(sum.r, 16.f), __fdiv_rn(sum.g, 16.f), __fdiv_rn(sum.b, 16.f)};
    // the shader indexes its tables with these values unclamped; they are clamped to the tables here
    const int r = min(max(int(rintf(Mul(average.r, 255.f))), 0), 255);
    const int g = min(max(int(rintf(Mul(average.g, 255.f))), 0), 255);
    const int b = min(max(int(rintf(Mul(average.b, 255.f))), 0), 255);
    const uint32_t mr = kMatch5[r], mg = kMatch6[g], mb = kMatch5[b];
    const uint32_t color0 = ((mr & 0x1f) << 11) | ((mg & 0x3f) << 5) | (mb & 0x1f);
    const uint32_t color1 = (((mr >> 8) & 0x1f) << 11) | (((mg >> 8) & 0x3f) << 5) | ((mb >> 8) & 0x1f);
    uint2 result;
    if (color0 < color1)
        result = make_uint2((color0 << 16) | color1, 0xffffffffu);
    else
        result = make_uint2((color1 << 16) | color0, 0xaaaaaaaau);
    const Rgb encoded = Lerp(Expand565(color0), Expand565(color1), 1.0f / 3.0f);
    blockError = 0.f;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
    {
        const Texel texel = texels[i];
        const Texel difference = {Sub(texel.rgb, encoded), Sub(texel.a, 1.f)};
        blockError = Add(blockError, Dot4(difference));
    }
    return result;
}

// Four-colour mode: endpoints from the extremes, refined by least squares (BC1_CompressFast, :249-376).
__device__ uint2 EncodeFourColors(const BlockTexels& texels, float& blockError)
{
    Extremes extremes;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        extremes.Include(texels[i].rgb);
    const Rgb center = {__fdiv_rn(extremes.sums.r, 16.f), __fdiv_rn(extremes.sums.g, 16.f), __fdiv_rn(extremes.sums.b, 16.f)};
    Covariance covariance;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        covariance.Include(texels[i].rgb, center);
    OrientAndInset(extremes, covariance, 16.f);
    Rgb maxColor = extremes.high, minColor = extremes.low;

    uint32_t color0 = 0, color1 = 0;
    for (int pass = 0; pass < 4; ++pass)
    {
        const Palette4 palette(maxColor, minColor);
        ColorRefit refit;
#pragma unroll 1
        for (int i = 0; i < 16; ++i)
        {
            float ignored;
            const Texel texel = texels[i];
            const uint32_t index = palette.Index(texel, ignored);
            float beta = float(index & 1u);
            if (index & 2u)
                beta = __fdiv_rn(Add(1.f, beta), 3.0f);
            refit.Include(beta, texel.rgb);
        }
        Rgb a, b;
        if (refit.Solve(a, b))
        {
            minColor = KeepExtremes(minColor, b);
            maxColor = KeepExtremes(maxColor, a);
        }
        uint32_t newColor0, newColor1;
        maxColor = RoundTo565(maxColor, newColor0);
        minColor = RoundTo565(minColor, newColor1);
        if (newColor0 == color0 && newColor1 == color1)
            break;
        color0 = newColor0;
        color1 = newColor1;
    }

    // color0 must exceed color1, or the block would decode in the three-colour mode
    if (color0 == color1)
    {
        if (color0 == 0)
        {
            color0 = 1;
            maxColor = Expand565(color0);
        }
        else
        {
            color1 = color0 - 1;
            minColor = Expand565(color1);
        }
    }
    else if (color0 < color1)
    {
        const Rgb t = maxColor;
        maxColor = minColor;
        minColor = t;
        const uint32_t c = color0;
        color0 = color1;
        color1 = c;
    }

    const Palette4 palette(maxColor, minColor);
    uint32_t indices = 0;
    blockError = 0.f;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
    {
        float pixelError;
        indices |= palette.Index(texels[i], pixelError) << (2 * i);
        blockError = Add(blockError, pixelError);
    }
    return make_uint2((color1 << 16) | color0, indices);
}

// Three colours and transparent black: one refit, transparent texels left out (BC1a_CompressFast, :378-493).
__device__ uint2 EncodeThreeColors(const BlockTexels& texels, float alphaThreshold, float& blockError)
{
    Extremes extremes;
    int opaque = 0;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
    {
        const Texel texel = texels[i];
        if (!(texel.a <= alphaThreshold))
        {
            extremes.Include(texel.rgb);
            ++opaque;
        }
    }
    const float count = float(opaque);
    const Rgb center = opaque > 0 ? Rgb{__fdiv_rn(extremes.sums.r, count), __fdiv_rn(extremes.sums.g, count), __fdiv_rn(extremes.sums.b, count)}
                                  : Rgb{0.f, 0.f, 0.f};
    Covariance covariance;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
    {
        const Texel texel = texels[i];
        if (!(texel.a <= alphaThreshold))
            covariance.Include(texel.rgb, center);
    }
    OrientAndInset(extremes, covariance, count);
    Rgb maxColor = extremes.high, minColor = extremes.low;

    ColorRefit refit;
    {
        const Palette3 palette(maxColor, minColor, alphaThreshold);
#pragma unroll 1
        for (int i = 0; i < 16; ++i)
        {
            float ignored;
            const Texel texel = texels[i];
            const uint32_t index = palette.Index(texel, ignored);
            if (index != 3u)
                refit.Include((index & 2u) ? 0.5f : float(index & 1u), texel.rgb);
        }
    }
    Rgb a, b;
    if (refit.Solve(a, b))
    {
        // as in the shader: the low end takes the solution of the high end's weights and vice versa
        minColor = KeepExtremes(minColor, a);
        maxColor = KeepExtremes(maxColor, b);
    }
    uint32_t color0, color1;
    maxColor = RoundTo565(maxColor, color0);
    minColor = RoundTo565(minColor, color1);
    if (color0 > color1)
    {
        const Rgb t = maxColor;
        maxColor = minColor;
        minColor = t;
        const uint32_t c = color0;
        color0 = color1;
        color1 = c;
    }
    const Palette3 palette(maxColor, minColor, alphaThreshold);
    uint32_t indices = 0;
    blockError = 0.f;
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
    {
        float pixelError;
        const Texel texel = texels[i];
        const uint32_t index = palette.Index(texel, pixelError);
        indices |= index << (2 * i);
        if (index != 3u || !(texel.a <= alphaThreshold))
            blockError = Add(blockError, pixelError);
    }
    return make_uint2((color1 << 16) | color0, indices);
}

// BC2's alpha: 4 bits per texel (BC2_EncodeAlpha, :495-508).
__device__ uint2 EncodeAlpha4(const BlockTexels& texels)
{
    uint2 block = make_uint2(0u, 0u);
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
    {
        const uint32_t value = uint32_t(rintf(Mul(Saturate(texels.Alpha(i)), 15.f)));
        if (i < 8)
            block.x |= value << (4 * i);
        else
            block.y |= value << (4 * (i - 8));
    }
    return block;
}

struct ColorCompressArguments
{
    BlockCompressArguments base;
    int numChannels; // channels that feed the block: red, green, blue, alpha; the missing ones read 0, alpha 1
    float alphaThreshold;
};

// CompressBC1.hlsl / CompressBC2.hlsl / CompressBC3.hlsl main().
template <int kFormat>
__global__ void __launch_bounds__(128) ColorBlockCompressKernel(const ColorCompressArguments args)
{
    __shared__ uint2 staged[16 * 128];
    // The CTA's 64 x 32 texels are loaded with neighbouring threads on neighbouring texels of a row
    // (coalesced) and handed to the thread that owns their block through shared memory.
    // an even first channel of an even channel count: channel pairs are aligned 32-bit words in both layouts
    const bool pairs = !(args.base.firstChannel & 1) && !(args.base.channels & 1);
#pragma unroll 1
    for (int k = 0; k < 16; ++k)
    {
        const int p = k * 128 + threadIdx.x;
        const int localX = p & 63, localY = p >> 6;
        const int x = args.base.srcLeft + blockIdx.x * 64 + localX, y = args.base.srcTop + blockIdx.y * 32 + localY;
        const bool inside = x < args.base.width && y < args.base.height;
        // red-green and blue-alpha as two 32-bit words; missing channels read 0, alpha 1 (0x3c00)
        uint32_t redGreen = 0u, blueAlpha = 0u;
        if (inside)
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
        const int owner = (localY >> 2) * 16 + (localX >> 2), texel = (localY & 3) * 4 + (localX & 3);
        staged[texel * 128 + owner] = make_uint2(redGreen, blueAlpha);
    }
    __syncthreads();
    const int blockX = blockIdx.x * 16 + (threadIdx.x & 15);
    const int blockY = blockIdx.y * 8 + (threadIdx.x >> 4);
    if (blockX >= args.base.widthInBlocks || blockY >= args.base.heightInBlocks)
        return;
    BlockTexels texels;
    texels.base = staged + threadIdx.x;
    texels.opaque = kFormat != NTCB_BLOCK_FORMAT_BC1; // BC2 / BC3 colour blocks ignore alpha

    float bestError;
    uint2 best;
    if (kFormat == NTCB_BLOCK_FORMAT_BC1)
    {
        // BC1a_TransparentBlock: everything transparent; the error is what the opaque texels lose
        bestError = 0.f;
#pragma unroll 1
        for (int i = 0; i < 16; ++i)
        {
            const Texel texel = texels[i];
            if (!(texel.a <= args.alphaThreshold))
                bestError = Add(bestError, Dot4(texel));
        }
        best = make_uint2(0u, 0xffffffffu);
        float error;
        const uint2 single = EncodeSingleColor(texels, error);
        if (error < bestError)
        {
            bestError = error;
            best = single;
        }
    }
    else
        best = EncodeSingleColor(texels, bestError);
    {
        float error;
        const uint2 four = EncodeFourColors(texels, error);
        if (error < bestError)
        {
            bestError = error;
            best = four;
        }
    }
    uint8_t* destination = args.base.blocks + size_t(blockY) * args.base.rowPitch;
    if (kFormat == NTCB_BLOCK_FORMAT_BC1)
    {
        float error;
        const uint2 three = EncodeThreeColors(texels, args.alphaThreshold, error);
        if (error < bestError)
            best = three;
        reinterpret_cast<uint2*>(destination)[blockX] = best;
    }
    else if (kFormat == NTCB_BLOCK_FORMAT_BC2)
    {
        const uint2 alpha = EncodeAlpha4(texels);
        reinterpret_cast<uint4*>(destination)[blockX] = make_uint4(alpha.x, alpha.y, best.x, best.y);
    }
    else // BC3: the alpha half is a BC4 block, written afterwards by BlockCompressKernel in a launch of its own
        reinterpret_cast<uint4*>(destination)[blockX] = make_uint4(0u, 0u, best.x, best.y);
}

// Entry i: the endpoint pair (mx | mn << 8) that minimises 1000 * |(2 * e(mx) + e(mn)) / 3 - i| +
// 14 * |e(mx) - e(mn)| over all pairs, mn in the outer loop, the first minimum kept; e() widens an
// endpoint to 8 bits by bit replication and the division is an integer one.  (The single-colour
// match of the public-domain DXT encoders; the weight of the spread term is the one that
// reproduces the tables in BlockCompressCommon.hlsli:40-80.)
void FillMatchTable(int bits, uint16_t (&table)[256])
{
    const int size = 1 << bits;
    int expanded[64];
    for (int c = 0; c < size; ++c)
        expanded[c] = (c << (8 - bits)) | (c >> (2 * bits - 8));
    for (int i = 0; i < 256; ++i)
    {
        int best = 1 << 30;
        for (int mn = 0; mn < size; ++mn)
            for (int mx = 0; mx < size; ++mx)
            {
                const int miss = (2 * expanded[mx] + expanded[mn]) / 3 - i;
                const int spread = expanded[mx] - expanded[mn];
                const int cost = 1000 * (miss < 0 ? -miss : miss) + 14 * (spread < 0 ? -spread : spread);
                if (cost < best)
                {
                    best = cost;
                    table[i] = uint16_t(mx | (mn << 8));
                }
            }
    }
}

std::mutex g_matchTableMutex;
uint64_t g_matchTableDevices = 0; // bit d: device d holds the tables

int UploadMatchTables()
{
    int device = 0;
    cudaError_t error = cudaGetDevice(&device);
    if (error != cudaSuccess)
        return CudaFailure("cudaGetDevice", error);
    std::lock_guard<std::mutex> lock(g_matchTableMutex);
    if (device < 64 && (g_matchTableDevices >> device) & 1)
        return NTCB_OK;
    static uint16_t match5[256], match6[256];
    static bool filled = false;
    if (!filled)
    {
        FillMatchTable(5, match5);
        FillMatchTable(6, match6);
        filled = true;
    }
    error = cudaMemcpyToSymbol(kMatch5, match5, sizeof match5);
    if (error == cudaSuccess)
        error = cudaMemcpyToSymbol(kMatch6, match6, sizeof match6);
    if (error != cudaSuccess)
        return CudaFailure("cudaMemcpyToSymbol", error);
    if (device < 64)
        g_matchTableDevices |= uint64_t(1) << device;
    return NTCB_OK;
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
    const int format = params->format;
    if (format < NTCB_BLOCK_FORMAT_BC1 || format > NTCB_BLOCK_FORMAT_BC7 || format == 6)
    {
        SetError("dstFormat (%d) is not supported: BC1 to BC5 (%d to %d) and BC7 (%d) are.", format, NTCB_BLOCK_FORMAT_BC1,
            NTCB_BLOCK_FORMAT_BC5, NTCB_BLOCK_FORMAT_BC7);
        return format == 6 ? NTCB_ERR_UNSUPPORTED : NTCB_ERR_OUT_OF_RANGE;
    }
    if (format != NTCB_BLOCK_FORMAT_BC7 && params->deviceModeBuffer)
    {
        SetError("Mode buffer can only be used with BC7 compression");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const bool color = format <= NTCB_BLOCK_FORMAT_BC3 || format == NTCB_BLOCK_FORMAT_BC7;
    // channels that feed a block: fixed for BC4 / BC5; red, green, blue[, alpha] for the colour formats
    const int natural = format == NTCB_BLOCK_FORMAT_BC4 ? 1 : format == NTCB_BLOCK_FORMAT_BC5 ? 2 : format == NTCB_BLOCK_FORMAT_BC1 ? 3 : 4;
    const int formatChannels = params->numChannels == 0 ? natural : params->numChannels;
    if (color ? (formatChannels < 1 || formatChannels > 4) : formatChannels != natural)
    {
        SetError("numChannels (%d) must be %s for this format.", params->numChannels, color ? "between 1 and 4, or 0" : "0");
        return NTCB_ERR_OUT_OF_RANGE;
    }
    const size_t blockBytes = (format == NTCB_BLOCK_FORMAT_BC1 || format == NTCB_BLOCK_FORMAT_BC4) ? 8u : 16u;
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

    const cudaStream_t cudaStream = static_cast<cudaStream_t>(stream);
    if (format == NTCB_BLOCK_FORMAT_BC7)
        return LaunchBlockCompressBc7(*params, args, cudaStream);
    const dim3 grid(unsigned(params->widthInBlocks + 15) / 16, unsigned(params->heightInBlocks + 7) / 8, color ? 1u : unsigned(formatChannels));
    if (!color)
        BlockCompressKernel<<<grid, 128, 0, cudaStream>>>(args);
    else
    {
        const int status = UploadMatchTables();
        if (status != NTCB_OK)
            return status;
        ColorCompressArguments colorArgs;
        colorArgs.base = args;
        colorArgs.numChannels = formatChannels;
        colorArgs.alphaThreshold = params->alphaThreshold;
        if (format == NTCB_BLOCK_FORMAT_BC1)
            ColorBlockCompressKernel<NTCB_BLOCK_FORMAT_BC1><<<grid, 128, 0, cudaStream>>>(colorArgs);
        else if (format == NTCB_BLOCK_FORMAT_BC2)
            ColorBlockCompressKernel<NTCB_BLOCK_FORMAT_BC2><<<grid, 128, 0, cudaStream>>>(colorArgs);
        else
        {
            // colour halves by the colour kernel, alpha halves by the BC4 kernel: two lean kernels instead
            // of one with both encoders inlined (158 registers; 1.56 ms against 1.1 ms on a 4096^2 mip)
            ColorBlockCompressKernel<NTCB_BLOCK_FORMAT_BC3><<<grid, 128, 0, cudaStream>>>(colorArgs);
            CountLaunch();
            BlockCompressArguments alphaArgs = args;
            alphaArgs.firstChannel = formatChannels == 4 ? args.firstChannel + 3 : -1;
            alphaArgs.formatChannels = 2; // 16-byte blocks, the alpha block first
            BlockCompressKernel<<<grid, 128, 0, cudaStream>>>(alphaArgs);
        }
    }
    CountLaunch();
    const cudaError_t error = cudaGetLastError();
    if (error != cudaSuccess)
        return CudaFailure("BlockCompressKernel", error);
    ClearError();
    return NTCB_OK;
}
