// Conversion of decoded fp16 channels to the client's channel format: colour-space transfer
// functions, dithering, quantisation.  Shared by the ReadChannels kernel (texture_set.cu) and the
// decode kernel's converting epilogue (decode_kernel.cu).
//
// The arithmetic follows the reference's CopyImageKernel (src/ImageProcessing.cu:86-164, 220-266)
// and its helpers (src/CudaUtils.h:63-184).  The reference is built with --use_fast_math
// (src/CMakeLists.txt:33): its powf / logf / expf / sqrtf and its divisions are the approximate
// hardware forms, flushing denormals.  They are spelled out here as PTX so that the results do not
// depend on this library's own compiler flags.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace ntcb
{

// ntc::ChannelFormat (include/libntc/ntc.h:227-236)
constexpr int kFormatUnorm8 = 1;
constexpr int kFormatUnorm16 = 2;
constexpr int kFormatFloat16 = 3;
constexpr int kFormatFloat32 = 4;
constexpr int kFormatUint32 = 5;

// ntc::ColorSpace (include/libntc/ntc.h:251-256)
constexpr int kSpaceLinear = 0;
constexpr int kSpaceSrgb = 1;
constexpr int kSpaceHlg = 2;

// How decoded channels become output components.  Colour spaces are packed two bits per channel:
// `srcSpaces` holds the stored colour space of the requested channels (index 0 = the first
// requested channel), `dstSpaces` the colour space each one is encoded to.
struct OutputConversion
{
    int format;       // kFormat*
    int dstChannels;  // components written per pixel; those past the requested channels get 0 (component 3: 1)
    int dither;       // nonzero: add a hash-based offset in [-0.5, 0.5) code units before rounding
    uint32_t srcSpaces, dstSpaces;
};

__host__ __device__ inline int BytesPerComponent(int format)
{
    return format == kFormatUnorm8 ? 1 : (format == kFormatUnorm16 || format == kFormatFloat16) ? 2
         : (format == kFormatFloat32 || format == kFormatUint32) ? 4 : 0;
}

__device__ __forceinline__ float ApproxLog2(float x)
{
    float r;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ float ApproxExp2(float x)
{
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ float ApproxSqrt(float x)
{
    float r;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ float ApproxDivide(float a, float b)
{
    float r;
    asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

__device__ __forceinline__ float MulFtz(float a, float b)
{
    float r;
    asm("mul.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

__device__ __forceinline__ float AddFtz(float a, float b)
{
    float r;
    asm("add.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

__device__ __forceinline__ float FmaFtz(float a, float b, float c)
{
    float r;
    asm("fma.rn.ftz.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// powf under fast math: 2^(y * log2 x)
__device__ __forceinline__ float ApproxPow(float x, float y)
{
    return ApproxExp2(MulFtz(y, ApproxLog2(x)));
}

// src/CudaUtils.h:92-108
__device__ __forceinline__ float SrgbEncode(float linear)
{
    return (linear <= 0.0031308f) ? MulFtz(linear, 12.92f) : FmaFtz(1.055f, ApproxPow(linear, 1.0f / 2.4f), -0.055f);
}

__device__ __forceinline__ float SrgbDecode(float encoded)
{
    return (encoded <= 0.04045f) ? ApproxDivide(encoded, 12.92f)
                                 : ApproxPow(ApproxDivide(AddFtz(encoded, 0.055f), 1.055f), 2.4f);
}

// src/CudaUtils.h:63-89
__device__ __forceinline__ float HlgEncode(float e)
{
    constexpr float a = 0.17883277f, b = 0.28466892f, c = 0.55991073f;
    const float sign = (e < 0.f) ? -1.f : 1.f;
    e = fabsf(e);
    return (e < 1.f) ? MulFtz(MulFtz(0.5f, ApproxSqrt(e)), sign)
                     : MulFtz(FmaFtz(a, MulFtz(ApproxLog2(AddFtz(e, -b)), 0.693147182f), c), sign);
}

__device__ __forceinline__ float HlgDecode(float h)
{
    constexpr float a = 0.17883277f, b = 0.28466892f, c = 0.55991073f;
    const float sign = (h < 0.f) ? -1.f : 1.f;
    h = fabsf(h);
    return (h < 0.5f) ? MulFtz(MulFtz(MulFtz(4.f, h), h), sign)
                      : MulFtz(AddFtz(ApproxExp2(MulFtz(ApproxDivide(AddFtz(h, -c), a), 1.44269502f)), b), sign);
}

__device__ __forceinline__ float DecodeColorSpace(int space, float value) // src/ImageProcessing.cu:86-98
{
    return space == kSpaceSrgb ? SrgbDecode(value) : space == kSpaceHlg ? HlgDecode(value) : value;
}

__device__ __forceinline__ float EncodeColorSpace(int space, float value) // src/ImageProcessing.cu:100-112
{
    return space == kSpaceSrgb ? SrgbEncode(value) : space == kSpaceHlg ? HlgEncode(value) : value;
}

// Per-pixel generator of the dither offsets (src/CudaUtils.h:111-184): the seed is a Jenkins hash
// of the pixel's linear index, each draw one Murmur3 round keyed by the draw counter (from 1).
__device__ __forceinline__ uint32_t DitherSeed(uint32_t linearIndex)
{
    uint32_t a = linearIndex;
    a = (a + 0x7ed55d16u) + (a << 12);
    a = (a ^ 0xc761c23cu) ^ (a >> 19);
    a = (a + 0x165667b1u) + (a << 5);
    a = (a + 0xd3a2646cu) ^ (a << 9);
    a = (a + 0xfd7046c5u) + (a << 3);
    a = (a ^ 0xb55a4f09u) ^ (a >> 16);
    return a;
}

// Draw number `index` (1, 2, ...) as a float in [-0.5, 0.5).
__device__ __forceinline__ float DitherDraw(uint32_t seed, uint32_t index)
{
    uint32_t k = index * 0xcc9e2d51u;
    k = __funnelshift_l(k, k, 15) * 0x1b873593u;
    uint32_t hash = seed ^ k;
    hash = __funnelshift_l(hash, hash, 13) * 5u + 0xe6546b64u;
    hash ^= 4u;
    hash ^= hash >> 16;
    hash *= 0x85ebca6bu;
    hash ^= hash >> 13;
    hash *= 0xc2b2ae35u;
    hash ^= hash >> 16;
    return AddFtz(AddFtz(__uint_as_float((hash & 0x7fffffu) | 0x3f800000u), -1.f), -0.5f);
}

// max(0, min(limit, roundf(x))) as an integer, for limit < 2^23.  roundf (half away from zero)
// equals floor(x + 0.5) computed in binary32 for every x >= 0 except the largest float below 0.5,
// where the sum rounds up to 1; negative x and NaN give 0 here (the reference's std::min / std::max
// give `limit` for NaN, which only a NaN texel could produce: decoded texels are scrubbed).
__device__ __forceinline__ uint32_t RoundToCode(float x, float limit)
{
    float shifted = AddFtz(x, 0.5f);
    if (x == 0.49999997f)
        shifted = 0.f;
    return __float2uint_rd(fminf(shifted, limit + 0.5f));
}

// The quantising half of WriteImageChannel (src/ImageProcessing.cu:139-164) after the colour-space
// encode: the component's bit pattern in the low BytesPerComponent(format) bytes of the result.
__device__ __forceinline__ uint32_t QuantizeComponent(int format, float value, float dither)
{
    switch (format)
    {
    case kFormatUnorm8:
        value = AddFtz(value, ApproxDivide(dither, 255.f));
        return RoundToCode(MulFtz(value, 255.f), 255.f);
    case kFormatUnorm16:
        value = AddFtz(value, ApproxDivide(dither, 65535.f));
        return RoundToCode(MulFtz(value, 65535.f), 65535.f);
    case kFormatFloat16:
        return uint32_t(__half_as_ushort(__float2half_rn(fmaxf(-65504.f, fminf(65504.f, value)))));
    case kFormatFloat32:
        return __float_as_uint(value);
    case kFormatUint32:
        return __float2uint_rz(fmaxf(value, 0.f));
    default:
        return 0;
    }
}

// One output component from one decoded fp16 value.
__device__ __forceinline__ uint32_t ConvertComponent(const OutputConversion& conversion, int channel, __half texel, float dither)
{
    const int srcSpace = (conversion.srcSpaces >> (2 * channel)) & 3;
    const int dstSpace = (conversion.dstSpaces >> (2 * channel)) & 3;
    float value = DecodeColorSpace(srcSpace, __half2float(texel));
    value = EncodeColorSpace(dstSpace, value);
    return QuantizeComponent(conversion.format, value, dither);
}

// Components past the requested channels: 0, or 1 for component 3 (alpha), linear
// (src/ImageProcessing.cu:166-170).
__device__ __forceinline__ uint32_t DefaultComponent(const OutputConversion& conversion, int component, float dither)
{
    return QuantizeComponent(conversion.format, component == 3 ? 1.f : 0.f, dither);
}

} // namespace ntcb
