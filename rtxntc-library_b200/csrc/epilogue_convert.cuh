// The converting epilogue of the decode kernels: the thread's decoded channels (eight binary16
// pairs) become the pixel in the client's channel format and are stored.  `Context` is the
// kernel's per-thread tile context: `out` is the address of the thread's pixel, `outStepWords` the
// pixel's linear index in its mip (the dither seed), `rowChunk` the thread's 16-byte slot in chunk 0
// of its half's A operand (chunks are 2048 bytes apart).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "kernel_parts.cuh"
#include "output_convert.cuh"

namespace ntcb
{
namespace
{

// Stores `bytes` bytes of a pixel held in `words` (little endian) at `pixel`, whose address and
// size are both multiples of the widest store used.
template <int kMaxWords>
__device__ __forceinline__ void StorePixel(unsigned char* pixel, const uint32_t (&words)[kMaxWords], int bytes)
{
    if ((bytes & 15) == 0 && kMaxWords >= 4)
    {
#pragma unroll
        for (int w = 0; w + 3 < kMaxWords; w += 4)
            if (w * 4 < bytes)
                *reinterpret_cast<uint4*>(pixel + w * 4) = make_uint4(words[w], words[w + 1], words[w + 2], words[w + 3]);
    }
    else if ((bytes & 7) == 0 && kMaxWords >= 2)
    {
#pragma unroll
        for (int w = 0; w + 1 < kMaxWords; w += 2)
            if (w * 4 < bytes)
                *reinterpret_cast<uint2*>(pixel + w * 4) = make_uint2(words[w], words[w + 1]);
    }
    else if ((bytes & 3) == 0)
    {
#pragma unroll
        for (int w = 0; w < kMaxWords; ++w)
            if (w * 4 < bytes)
                *reinterpret_cast<uint32_t*>(pixel + w * 4) = words[w];
    }
    else if ((bytes & 1) == 0)
    {
#pragma unroll
        for (int h = 0; h < kMaxWords * 2; ++h)
            if (h * 2 < bytes)
                *reinterpret_cast<uint16_t*>(pixel + h * 2) = uint16_t(words[h >> 1] >> (16 * (h & 1)));
    }
    else
    {
#pragma unroll
        for (int b = 0; b < kMaxWords * 4; ++b)
            if (b < bytes)
                pixel[b] = (unsigned char)(words[b >> 2] >> (8 * (b & 3)));
    }
}

// Converting epilogue for one channel format: pairs[j] holds the requested channels 2j and 2j + 1
// as (scrubbed) binary16; the pixel goes to ctx.out.  What ITextureSet::ReadChannels would produce
// from the stored texels (src/TextureSet.cpp:915-985, src/ImageProcessing.cu:220-266).
template <int kFormat, typename Context>
__device__ __forceinline__ void ConvertPixel(const OutputConversion& conversion, int numChannels, const Context& ctx,
    const uint32_t (&pairs)[8])
{
    constexpr int kBytes = kFormat == kFormatUnorm8 ? 1 : (kFormat == kFormatUnorm16 || kFormat == kFormatFloat16) ? 2 : 4;
    constexpr int kPerWord = 4 / kBytes;
    constexpr int kMaxWords = 16 / kPerWord;
    const int components = conversion.dstChannels;
    uint32_t words[kMaxWords];
#pragma unroll
    for (int w = 0; w < kMaxWords; ++w)
        words[w] = 0;

    const bool plain = (conversion.srcSpaces | conversion.dstSpaces) == 0 && !conversion.dither;
    if (kFormat == kFormatUnorm8 && plain)
    {
        // Linear, undithered UNORM8: round(clamp(v) * 255).  The product of a binary16 value and 255 is
        // exact in binary32 and its only tie inside [0, 255] is 127.5 (v = 0.5), which rounds to 128
        // both to nearest-even and away from zero, so adding 1.5 * 2^23 leaves the reference's
        // roundf() result in the low byte.  (Decoded texels are finite: the epilogue scrubs Inf / NaN.)
        const __half2 one = __float2half2_rn(1.f);
#pragma unroll
        for (int j = 0; j < 8; ++j)
        {
            if (2 * j < components)
            {
                const float2 v = __half22float2(__hmul2_sat(AsHalf2(pairs[j]), one));
                uint32_t lo = __float_as_uint(__fmaf_rn(v.x, 255.f, 12582912.f));
                uint32_t hi = __float_as_uint(__fmaf_rn(v.y, 255.f, 12582912.f));
                // components past the requested channels: 0, component 3: 255
                if (2 * j >= numChannels) lo = (2 * j == 3) ? 255u : 0u;
                if (2 * j + 1 >= numChannels) hi = (2 * j + 1 == 3) ? 255u : 0u;
                if (2 * j + 1 >= components) hi = 0u;
                // byte 0 of each holds the code; an odd pair lands in the upper half of its word
                words[j >> 1] = (j & 1) ? __byte_perm(words[j >> 1], __byte_perm(lo, hi, 0x0040), 0x5410)
                                        : (__byte_perm(lo, hi, 0x0040) & 0xFFFFu);
            }
        }
    }
    else if (plain)
    {
        // linear and undithered in another format: no colour-space branches, no generator
#pragma unroll
        for (int c = 0; c < 16; ++c)
        {
            if (c < components)
            {
                const __half2 pair = AsHalf2(pairs[c >> 1]);
                float value = __half2float((c & 1) ? __high2half(pair) : __low2half(pair));
                if (c >= numChannels)
                    value = c == 3 ? 1.f : 0.f;
                words[c / kPerWord] |= QuantizeComponent(kFormat, value, 0.f) << (8 * kBytes * (c % kPerWord));
            }
        }
    }
    else
    {
        const uint32_t seed = conversion.dither ? DitherSeed(ctx.outStepWords) : 0u;
#pragma unroll
        for (int c = 0; c < 16; ++c)
        {
            if (c < components)
            {
                const float dither = conversion.dither ? DitherDraw(seed, uint32_t(c) + 1u) : 0.f;
                const __half2 pair = AsHalf2(pairs[c >> 1]);
                const __half texel = (c & 1) ? __high2half(pair) : __low2half(pair);
                uint32_t component;
                if (c < numChannels)
                {
                    float value = __half2float(texel);
                    const int srcSpace = (conversion.srcSpaces >> (2 * c)) & 3;
                    const int dstSpace = (conversion.dstSpaces >> (2 * c)) & 3;
                    if (srcSpace | dstSpace)
                        value = EncodeColorSpace(dstSpace, DecodeColorSpace(srcSpace, value));
                    component = QuantizeComponent(kFormat, value, dither);
                }
                else
                    component = QuantizeComponent(kFormat, c == 3 ? 1.f : 0.f, dither);
                words[c / kPerWord] |= component << (8 * kBytes * (c % kPerWord));
            }
        }
    }
    StorePixel<kMaxWords>(reinterpret_cast<unsigned char*>(ctx.out), words, components * kBytes);
}

// Converting epilogue: the thread's (scrubbed) fp16 channel pairs -> the pixel in the client's
// format, stored at ctx.out.
template <typename Context>
__device__ __forceinline__ void StoreConverted(const OutputConversion& conversion, int firstChannel, int numChannels,
    const Context& ctx, uint32_t (&bits)[8])
{
    if (firstChannel != 0)
    {
        // Re-base the channels so that the first requested one sits in bits[0]: park them in the
        // thread's own slots of the A operand, which the tensor core has finished reading (layer 3's
        // MMA has completed), and read them back from the shifted position.
        uint4* slot = ctx.rowChunk;
        slot[0] = make_uint4(bits[0], bits[1], bits[2], bits[3]);
        slot[128] = make_uint4(bits[4], bits[5], bits[6], bits[7]);
        const unsigned char* parked = reinterpret_cast<const unsigned char*>(slot);
#pragma unroll
        for (int j = 0; j < 8; ++j)
        {
            const int c0 = firstChannel + 2 * j, c1 = c0 + 1;
            const uint32_t lo = c0 < 16 ? *reinterpret_cast<const uint16_t*>(parked + (c0 >> 3) * 2048 + (c0 & 7) * 2) : 0u;
            const uint32_t hi = c1 < 16 ? *reinterpret_cast<const uint16_t*>(parked + (c1 >> 3) * 2048 + (c1 & 7) * 2) : 0u;
            bits[j] = lo | (hi << 16);
        }
    }
    switch (conversion.format)
    {
    case kFormatUnorm8: ConvertPixel<kFormatUnorm8>(conversion, numChannels, ctx, bits); break;
    case kFormatUnorm16: ConvertPixel<kFormatUnorm16>(conversion, numChannels, ctx, bits); break;
    case kFormatFloat16: ConvertPixel<kFormatFloat16>(conversion, numChannels, ctx, bits); break;
    case kFormatFloat32: ConvertPixel<kFormatFloat32>(conversion, numChannels, ctx, bits); break;
    default: ConvertPixel<kFormatUint32>(conversion, numChannels, ctx, bits); break;
    }
}

} // namespace
} // namespace ntcb
