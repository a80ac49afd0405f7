// Input stage of the decode kernels whose A operand holds 8-bit codes (int8 or e4m3): per-tile
// lookup tables, staging of the latent footprint, the bilinear gather, and the thread's 64-byte row
// of the A operand.  `Shared` is the kernel's shared-memory structure (members tables,
// footprintHi, footprintLo, latentTable), `Context` its per-thread tile context (members x, y,
// rowChunk).
#pragma once

#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "decode_kernel.h"
#include "kernel_parts.cuh"

namespace ntcb
{
namespace
{

// The decode kernels are compiled for a fixed number of latent layers (kLayers = 2, 3 or 4: 8, 12 or
// 16 features, the shapes the reference's presets use) and once for any number (kLayers = 0): with
// the count known the layer loops unroll without predicated-off iterations and the footprint
// stride is a constant - 5 % fewer instructions on the benchmark set.
template <int kLayers>
__device__ __forceinline__ int NumLayers(const KernelParams& params)
{
    return kLayers ? kLayers : params.numLayers;
}

template <int kLayers>
__device__ __forceinline__ int StrideBytes(const KernelMip& mip)
{
    return kLayers ? (kLayers == 1 ? 8 : kLayers <= 3 ? 24 : 40) : mip.strideBytes;
}

// Quantises a pair of network inputs.  Int8: floor(x * 127.5 - 0.5) clamped to +-127
// (src/tin/tin_mlp.h:25-31), returned as the low bytes of the two 16-bit lanes.  FP8: round to
// nearest even e4m3, saturating (src/tin/tin_activation.h:44-48), returned as two packed bytes.
template <bool kFp8>
__device__ __forceinline__ uint32_t QuantizeInputPair(__half2 x)
{
    if (kFp8)
    {
        return uint32_t(__nv_cvt_halfraw2_to_fp8x2(static_cast<__half2_raw>(x), __NV_SATFINITE, __NV_E4M3));
    }
    else
    {
        __half2 y = __hfma2(x, __float2half2_rn(127.5f), __float2half2_rn(-0.5f));
        y = h2floor(y);
        y = __hmax2(__hmin2(y, __float2half2_rn(127.f)), __float2half2_rn(-127.f));
        // integer-valued: adding 1536 puts the two's-complement code in the low byte of each lane
        return AsU32(__hadd2_rn(y, __float2half2_rn(1536.f)));
    }
}

// Two quantised pairs -> four operand bytes.
template <bool kFp8>
__device__ __forceinline__ uint32_t PackCodes(uint32_t pair0, uint32_t pair1)
{
    if (kFp8)
    {
        // pair0 | pair1 << 16 (both are 16-bit values) as an integer multiply-add: it runs on the FMA
        // pipe, leaving the busier ALU pipe to the conversions and min/max
        uint32_t packed;
        asm("mad.lo.u32 %0, %1, 65536, %2;" : "=r"(packed) : "r"(pair1), "r"(pair0));
        return packed;
    }
    return __byte_perm(pair0, pair1, 0x6420);
}

// One latent pixel layer (four 4-bit features, the low 16 bits of each p) of one grid -> four quantised inputs.
// Blend order as the reference build evaluates it: fma(l11,w3, fma(l10,w2, fma(l00,w0, l01*w1))).
template <bool kFp8>
__device__ __forceinline__ uint32_t BlendLayer(uint32_t p00, uint32_t p01, uint32_t p10, uint32_t p11, const GridTaps& taps,
    const uint32_t* __restrict__ lut)
{
    uint32_t pairs[2];
#pragma unroll
    for (int j = 0; j < 2; ++j)
    {
        __half2 l00 = AsHalf2(lut[(p00 >> (8 * j)) & 0xFF]), l01 = AsHalf2(lut[(p01 >> (8 * j)) & 0xFF]);
        __half2 l10 = AsHalf2(lut[(p10 >> (8 * j)) & 0xFF]), l11 = AsHalf2(lut[(p11 >> (8 * j)) & 0xFF]);
        __half2 d = __hmul2_rn(l01, taps.w01);
        d = __hfma2(l00, taps.w00, d);
        d = __hfma2(l10, taps.w10, d);
        d = __hfma2(l11, taps.w11, d);
        d = __hfma2(d, __float2half2_rn(2.f), __float2half2_rn(-1.f));
        pairs[j] = QuantizeInputPair<kFp8>(d);
    }
    return PackCodes<kFp8>(pairs[0], pairs[1]);
}

// ... with the taps read from one layer's plane in global memory.
template <bool kFp8>
__device__ __forceinline__ uint32_t SampleLayer(const uint16_t* __restrict__ plane, const GridTaps& taps,
    const uint32_t* __restrict__ lut)
{
    uint32_t p00 = __ldg(plane + taps.o00), p01 = __ldg(plane + taps.o01);
    uint32_t p10 = __ldg(plane + taps.o10), p11 = __ldg(plane + taps.o11);
    return BlendLayer<kFp8>(p00, p01, p10, p11, taps, lut);
}

// Both grids of a texel from the pixel-major copy of the latents (ntcb_interleave_latents): latent pixel p of a
// grid is ONE aligned word at grid + p * slot holding its layers side by side - 8 bytes for three or four layers,
// 4 for two, 2 for one.  `blend(grid, layer, p00, p01, p10, p11)` receives layer l of the four taps in the low 16
// bits of its arguments.  Inference on sample, whose taps are scattered, is bound by the rate at which the L1
// serves scattered words: a tap costs it one request instead of one per layer, and the eight requests of a query
// are all in flight before the first is needed.
template <typename Blend>
__device__ __forceinline__ void SampleInterleaved(const uint16_t* __restrict__ hi, const uint16_t* __restrict__ lo, int numLayers,
    const GridTaps& hiTaps, const GridTaps& loTaps, Blend&& blend)
{
    if (numLayers >= 3)
    {
        const uint2* wideHi = reinterpret_cast<const uint2*>(hi);
        const uint2* wideLo = reinterpret_cast<const uint2*>(lo);
        const uint2 h00 = __ldg(wideHi + hiTaps.o00), h01 = __ldg(wideHi + hiTaps.o01);
        const uint2 h10 = __ldg(wideHi + hiTaps.o10), h11 = __ldg(wideHi + hiTaps.o11);
        const uint2 l00 = __ldg(wideLo + loTaps.o00), l01 = __ldg(wideLo + loTaps.o01);
        const uint2 l10 = __ldg(wideLo + loTaps.o10), l11 = __ldg(wideLo + loTaps.o11);
        blend(0, 0, h00.x, h01.x, h10.x, h11.x);
        blend(0, 1, h00.x >> 16, h01.x >> 16, h10.x >> 16, h11.x >> 16);
        blend(0, 2, h00.y, h01.y, h10.y, h11.y);
        if (numLayers == 4)
            blend(0, 3, h00.y >> 16, h01.y >> 16, h10.y >> 16, h11.y >> 16);
        blend(1, 0, l00.x, l01.x, l10.x, l11.x);
        blend(1, 1, l00.x >> 16, l01.x >> 16, l10.x >> 16, l11.x >> 16);
        blend(1, 2, l00.y, l01.y, l10.y, l11.y);
        if (numLayers == 4)
            blend(1, 3, l00.y >> 16, l01.y >> 16, l10.y >> 16, l11.y >> 16);
    }
    else if (numLayers == 2)
    {
        const uint32_t* wideHi = reinterpret_cast<const uint32_t*>(hi);
        const uint32_t* wideLo = reinterpret_cast<const uint32_t*>(lo);
        const uint32_t h00 = __ldg(wideHi + hiTaps.o00), h01 = __ldg(wideHi + hiTaps.o01);
        const uint32_t h10 = __ldg(wideHi + hiTaps.o10), h11 = __ldg(wideHi + hiTaps.o11);
        const uint32_t l00 = __ldg(wideLo + loTaps.o00), l01 = __ldg(wideLo + loTaps.o01);
        const uint32_t l10 = __ldg(wideLo + loTaps.o10), l11 = __ldg(wideLo + loTaps.o11);
        blend(0, 0, h00, h01, h10, h11);
        blend(0, 1, h00 >> 16, h01 >> 16, h10 >> 16, h11 >> 16);
        blend(1, 0, l00, l01, l10, l11);
        blend(1, 1, l00 >> 16, l01 >> 16, l10 >> 16, l11 >> 16);
    }
    else
    {
        blend(0, 0, __ldg(hi + hiTaps.o00), __ldg(hi + hiTaps.o01), __ldg(hi + hiTaps.o10), __ldg(hi + hiTaps.o11));
        blend(1, 0, __ldg(lo + loTaps.o00), __ldg(lo + loTaps.o01), __ldg(lo + loTaps.o10), __ldg(lo + loTaps.o11));
    }
}

// Per-tile lookup tables of the bilinear taps: tap position and weights are separable in x and y, so
// they are computed once per tile column / row instead of once per texel.  Shared by every decode
// kernel.
struct __align__(16) TapTables
{
    // per grid (0 = high-res, 1 = low-res) and tile column: byte offset of the left tap inside a footprint row, dx, 1 - dx
    int4 colTap[2][kTileWidth];
    // per grid and tile row: byte offset of the upper tap's footprint row, dy, 1 - dy, bytes per footprint row
    int4 rowTap[2][kTileHeight];
    // per grid: footprint width and height in latent pixels, pixel count, and the multiplier that divides a
    // pixel index by the width (p / width == (p * magic) >> 20 for p < 2048)
    int4 footprint[2];
    // per grid: the footprint origin (tap of the first column / row) of the tile the tables were built for, and that tile's origin
    int4 origin[2];
};

// Tap tables plus the positional encoding as operand bytes (kernels whose A operand holds 8-bit codes).
struct __align__(16) TileTables
{
    TapTables taps;
    // positional-encoding operand bytes: x = {X0 w0, X1 w0, X0 w1, X1 w1}, y = {X0 w2, X1 w2, 0, 0}
    uint2 colEnc[kTileWidth];
    uint2 rowEnc[kTileHeight];
    uint32_t lodWord;  // operand bytes of inputs 44..47: lod, lod, 0, 0
    uint32_t pad[3];
};

// Builds the tile's tap tables and stages the latent footprint of both grids in shared memory
// (nibbles unpacked to binary16 once per latent pixel instead of once per texel and tap).
// Even warps work on the high-res grid, odd warps on the low-res grid; the 128 threads of a grid
// share its footprint pixels.
// (Tried and dropped, both slower although they execute fewer instructions: two warps staging the
// footprints while the others go on - the tile then waits for those two; and requesting the latents
// before the wait for layer 0 and unpacking them after it.)
//
// `tablesValid`: the tables already hold this tile's values.  In a mip whose sizes and grid sizes
// are powers of two (KernelMip::invariant) every tile that lies wholly inside the mip has the same
// tap offsets and fractions relative to its own footprint - all the arithmetic is exact - so the
// tables are built for the first such tile and only the footprint is staged for the others.
template <bool kReferenceDivision, int kLayers = 0>
__device__ __forceinline__ void PrepareTaps(const KernelParams& params, const KernelMip& mip, TapTables& taps,
    uint8_t* footprintHi, uint8_t* footprintLo, const uint32_t* latentTable, int tileX0, int tileY0, int lane, int warp,
    bool tablesValid)
{
    const int grid = warp & 1;
    const int gw = grid ? mip.loWidth : mip.hiWidth;
    const int gh = grid ? mip.loHeight : mip.hiHeight;
    const int stride = StrideBytes<kLayers>(mip);

    int fx0, fy0, footW, count;
    uint32_t magic;
    if (tablesValid)
    {
        // only the footprint's origin depends on the tile, and it moves by whole latent pixels per tile step
        const int4 footprint = taps.footprint[grid];
        // a warp whose first footprint pixel lies beyond the footprint has nothing to stage (with a grid at a
        // quarter of the mip's resolution a footprint has 40 pixels: two of the grid's four warps)
        if (32 * (warp >> 1) >= footprint.z)
            return;
        const int4 origin = taps.origin[grid];
        fx0 = origin.x + ((tileX0 - origin.z) >> 5) * (grid ? mip.loStepX : mip.hiStepX);
        fy0 = origin.y + ((tileY0 - origin.w) >> 3) * (grid ? mip.loStepY : mip.hiStepY);
        footW = footprint.x;
        count = footprint.z;
        magic = uint32_t(footprint.w);
    }
    else
    {
        int xb, yb;
        float dx, dy;
        AxisTap<kReferenceDivision>(min(tileX0 + lane, mip.width - 1), mip.width, mip.invWidth, gw, xb, dx);
        AxisTap<kReferenceDivision>(min(tileY0 + (lane & (kTileHeight - 1)), mip.rowEnd - 1), mip.height, mip.invHeight, gh, yb, dy);
        fx0 = __shfl_sync(0xFFFFFFFFu, xb, 0);
        fy0 = __shfl_sync(0xFFFFFFFFu, yb, 0);
        footW = __shfl_sync(0xFFFFFFFFu, xb, 31) - fx0 + 2;
        const int footH = __shfl_sync(0xFFFFFFFFu, yb, kTileHeight - 1) - fy0 + 2;
        count = footW * footH;
        // the IEEE quotient of 2^20 / footW floors exactly
        magic = uint32_t(__float2int_rd(__fdiv_rn(1048576.f, float(footW)))) + 1;
        if (warp < 2)
        {
            taps.colTap[grid][lane] = make_int4((xb - fx0) * stride, __float_as_int(dx), __float_as_int(__fsub_rn(1.f, dx)), 0);
            if (lane < kTileHeight)
                taps.rowTap[grid][lane] =
                    make_int4((yb - fy0) * footW * stride, __float_as_int(dy), __float_as_int(__fsub_rn(1.f, dy)), footW * stride);
            if (lane == 0)
            {
                taps.footprint[grid] = make_int4(footW, footH, count, int(magic));
                taps.origin[grid] = make_int4(fx0, fy0, tileX0, tileY0);
            }
        }
    }

    if (mip.staged)
    {
        // footprint pixel p = fy * footW + fx, handed out over the 128 threads that share this grid
        // (tried: one footprint row per warp - no division, but more warps with a few active lanes each:
        // 5 % more instructions and 6 % slower; prefetching the next tile's latents into L1 a tile ahead: 5 % slower)
        const uint16_t* plane0 = params.latents + (grid ? mip.loOffset : mip.hiOffset);
        const uint32_t planePixels = uint32_t(grid ? mip.loPlane : mip.hiPlane);
        uint8_t* foot = grid ? footprintLo : footprintHi;
        for (int p = lane + 32 * (warp >> 1); p < count; p += kThreadsPerCta / 2)
        {
            const int fy = int((uint32_t(p) * magic) >> 20);
            const int fx = p - fy * footW;
            // wrap addressing (src/FeatureGridDevice.h:51-57); the footprint spans [-1, size]
            int gx = fx0 + fx, gy = fy0 + fy;
            gx += gx < 0 ? gw : 0;
            gx -= gx >= gw ? gw : 0;
            gy += gy < 0 ? gh : 0;
            gy -= gy >= gh ? gh : 0;
            const uint32_t first = uint32_t(gy) * uint32_t(gw) + uint32_t(gx);
            uint2* dst = reinterpret_cast<uint2*>(foot + p * stride);
#pragma unroll
            for (int layer = 0; layer < 4; ++layer)
            {
                if (layer < NumLayers<kLayers>(params))
                {
                    const uint32_t pixel = __ldg(plane0 + (first + uint32_t(layer) * planePixels));
                    dst[layer] = make_uint2(latentTable[pixel & 0xFF], latentTable[pixel >> 8]);
                }
            }
        }
    }
}

// The tile's tables (taps and positional encoding as operand bytes) and its staged footprints.
template <bool kFp8, bool kReferenceDivision, int kLayers = 0, typename Shared>
__device__ __forceinline__ void PrepareTile(const KernelParams& params, const KernelMip& mip, Shared& shared,
    int tileX0, int tileY0, int lane, int warp, bool tablesValid)
{
    if (!tablesValid && warp >= 2 && warp < 4)
    {
        // positional encoding (src/RegressionKernels.h:59-85): warp 2 the x part per column, warp 3
        // the y part per row, quantised exactly as the per-texel inputs would be
        const bool rows = warp == 3;
        const int coordinate = rows ? min(tileY0 + (lane & (kTileHeight - 1)), mip.rowEnd - 1) : min(tileX0 + lane, mip.width - 1);
        float f = __fmul_rn(float(coordinate), mip.positionScale);
        uint32_t q[3];
#pragma unroll
        for (int wave = 0; wave < 3; ++wave)
        {
            const float e0 = __fmaf_rn(Frac(f), 2.f, -1.f);
            const float e1 = __fmaf_rn(Frac(__fadd_rn(f, 0.25f)), 2.f, -1.f);
            q[wave] = QuantizeInputPair<kFp8>(__floats2half2_rn(e0, e1));
            f = __fmul_rn(f, 2.f);
        }
        const uint2 enc = make_uint2(PackCodes<kFp8>(q[0], q[1]), PackCodes<kFp8>(q[2], 0));
        if (!rows)
            shared.tables.colEnc[lane] = enc;
        else if (lane < kTileHeight)
            shared.tables.rowEnc[lane] = enc;
        if (rows && lane == kTileHeight)
            shared.tables.lodWord = PackCodes<kFp8>(QuantizeInputPair<kFp8>(__float2half2_rn(mip.positionLod)),
                                                   QuantizeInputPair<kFp8>(__float2half2_rn(0.f)));
    }
    PrepareTaps<kReferenceDivision, kLayers>(params, mip, shared.tables.taps, shared.footprintHi, shared.footprintLo, shared.latentTable,
        tileX0, tileY0, lane, warp, tablesValid);
}

// Whether the tables built for one tile of `mip` serve the tile at (tileX0, tileY0) too, and whether
// tables built for that tile may be kept for later ones: the tile lies wholly inside the decoded rows
// of a mip with invariant tables.
__device__ __forceinline__ bool TileKeepsTables(const KernelMip& mip, int tileX0, int tileY0)
{
    return mip.invariant && tileX0 + kTileWidth <= mip.width && tileY0 + kTileHeight <= mip.rowEnd;
}

// Four quantised inputs of one latent layer from the four staged taps.
// Blend order as the reference build evaluates it: fma(l11,w3, fma(l10,w2, fma(l00,w0, l01*w1))).
template <bool kFp8>
__device__ __forceinline__ uint32_t BlendLayer(uint2 l00, uint2 l01, uint2 l10, uint2 l11, __half2 w00, __half2 w01,
    __half2 w10, __half2 w11)
{
    const __half2 two = __float2half2_rn(2.f), minusOne = __float2half2_rn(-1.f);
    __half2 a = __hmul2_rn(AsHalf2(l01.x), w01);
    __half2 b = __hmul2_rn(AsHalf2(l01.y), w01);
    a = __hfma2(AsHalf2(l00.x), w00, a);
    b = __hfma2(AsHalf2(l00.y), w00, b);
    a = __hfma2(AsHalf2(l10.x), w10, a);
    b = __hfma2(AsHalf2(l10.y), w10, b);
    a = __hfma2(AsHalf2(l11.x), w11, a);
    b = __hfma2(AsHalf2(l11.y), w11, b);
    a = __hfma2(a, two, minusOne);
    b = __hfma2(b, two, minusOne);
    return PackCodes<kFp8>(QuantizeInputPair<kFp8>(a), QuantizeInputPair<kFp8>(b));
}

// Inputs 0..15 or 16..31 of one texel from the staged footprint of one grid.
template <bool kFp8, int kLayers = 0, typename Shared>
__device__ __forceinline__ void GatherGrid(const KernelParams& params, const KernelMip& mip, const Shared& shared,
    int grid, int lane, int tileRow, uint32_t* words)
{
    const int4 col = shared.tables.taps.colTap[grid][lane];
    const int4 row = shared.tables.taps.rowTap[grid][tileRow];
    const float dx = __int_as_float(col.y), dxn = __int_as_float(col.z);
    const float dy = __int_as_float(row.y), dyn = __int_as_float(row.z);
    // src/FeatureGridDevice.h:46-49
    const float f00 = __fmul_rn(dxn, dyn), f01 = __fmul_rn(dx, dyn), f10 = __fmul_rn(dxn, dy), f11 = __fmul_rn(dx, dy);
    const __half2 w00 = __floats2half2_rn(f00, f00), w01 = __floats2half2_rn(f01, f01);
    const __half2 w10 = __floats2half2_rn(f10, f10), w11 = __floats2half2_rn(f11, f11);

    const int stride = StrideBytes<kLayers>(mip);
    const uint8_t* tap00 = (grid ? shared.footprintLo : shared.footprintHi) + (col.x + row.x);
    const uint8_t* tap10 = tap00 + row.w;
#pragma unroll
    for (int layer = 0; layer < 4; ++layer)
    {
        if (layer < NumLayers<kLayers>(params))
        {
            const uint2 l00 = *reinterpret_cast<const uint2*>(tap00 + layer * 8);
            const uint2 l01 = *reinterpret_cast<const uint2*>(tap00 + stride + layer * 8);
            const uint2 l10 = *reinterpret_cast<const uint2*>(tap10 + layer * 8);
            const uint2 l11 = *reinterpret_cast<const uint2*>(tap10 + stride + layer * 8);
            words[layer] = BlendLayer<kFp8>(l00, l01, l10, l11, w00, w01, w10, w11);
        }
    }
}

// Inputs 0..31 of one texel with the taps read straight from global memory (`interleaved`: from the pixel-major
// copy ntcb_interleave_latents makes instead of the file's planes; the mip's offsets then refer to that copy).
template <bool kFp8, bool kReferenceDivision>
__device__ __forceinline__ void SampleGridsDirect(const uint16_t* __restrict__ latents, int numLayers, const KernelMip& mip,
    int x, int y, const uint32_t* __restrict__ latentTable, uint32_t* words, bool interleaved = false)
{
    // src/Inference.cu:52-53
    const float u = TexelCoordinate<kReferenceDivision>(x, mip.width, mip.invWidth);
    const float v = TexelCoordinate<kReferenceDivision>(y, mip.height, mip.invHeight);
    GridTaps taps;
    SetupTaps(u, v, mip.hiWidth, mip.hiHeight, taps);
    const uint16_t* hi = latents + mip.hiOffset;
    if (interleaved)
    {
        GridTaps lowTaps;
        SetupTaps(u, v, mip.loWidth, mip.loHeight, lowTaps);
        SampleInterleaved(hi, latents + mip.loOffset, numLayers, taps, lowTaps,
            [&](int grid, int layer, uint32_t p00, uint32_t p01, uint32_t p10, uint32_t p11) {
                words[4 * grid + layer] = BlendLayer<kFp8>(p00, p01, p10, p11, grid ? lowTaps : taps, latentTable);
            });
        return;
    }
#pragma unroll
    for (int layer = 0; layer < 4; ++layer)
        if (layer < numLayers)
            words[layer] = SampleLayer<kFp8>(hi + size_t(layer) * mip.hiPlane, taps, latentTable);
    SetupTaps(u, v, mip.loWidth, mip.loHeight, taps);
    const uint16_t* lo = latents + mip.loOffset;
#pragma unroll
    for (int layer = 0; layer < 4; ++layer)
        if (layer < numLayers)
            words[4 + layer] = SampleLayer<kFp8>(lo + size_t(layer) * mip.loPlane, taps, latentTable);
}

// The 48 network inputs of one texel -> its 64-byte row of the A operand (K-major core matrices:
// 16-byte chunk j of row r lives at j * 2048 + r * 16).
template <bool kFp8, bool kReferenceDivision, int kLayers = 0, typename Shared, typename Context>
__device__ __forceinline__ void BuildInputs(const KernelParams& params, const KernelMip& mip, const Shared& shared,
    const Context& ctx, int lane, int tileRow)
{
    uint32_t words[16];
    const uint32_t zeroWord = PackCodes<kFp8>(QuantizeInputPair<kFp8>(__float2half2_rn(0.f)),
                                              QuantizeInputPair<kFp8>(__float2half2_rn(0.f)));
#pragma unroll
    for (int i = 0; i < 8; ++i)
        words[i] = zeroWord; // unused feature slots hold quantised zeros (src/Inference.cu:49)
    // K padding: zeros for e4m3 operands; for int8 operands the constant inputs of the bias slots
    const uint32_t slotFill = kFp8 ? 0u : kBiasSlotValue * 0x01010101u;
    words[12] = words[13] = words[14] = slotFill;
    words[15] = kFp8 ? 0u : ((slotFill & 0x00FFFFFFu) | 0x01000000u);

    if (mip.staged)
    {
        GatherGrid<kFp8, kLayers>(params, mip, shared, 0, lane, tileRow, words);
        GatherGrid<kFp8, kLayers>(params, mip, shared, 1, lane, tileRow, words + 4);
    }
    else
    {
        // footprint too large to stage (strong minification): read the taps from global memory;
        // threads past the right / bottom edge compute a clamped texel and store nothing
        SampleGridsDirect<kFp8, kReferenceDivision>(params.latents, NumLayers<kLayers>(params), mip, min(ctx.x, mip.width - 1), min(ctx.y, mip.rowEnd - 1),
            shared.latentTable, words);
    }

    // positional encoding: interleave the column's x bytes with the row's y bytes
    const uint2 cx = shared.tables.colEnc[lane];
    const uint2 ry = shared.tables.rowEnc[tileRow];
    words[8] = __byte_perm(cx.x, ry.x, 0x5140);
    words[9] = __byte_perm(cx.x, ry.x, 0x7362);
    words[10] = __byte_perm(cx.y, ry.y, 0x5140);
    words[11] = shared.tables.lodWord;

#pragma unroll
    for (int chunk = 0; chunk < 4; ++chunk)
        ctx.rowChunk[chunk * 128] = make_uint4(words[4 * chunk], words[4 * chunk + 1], words[4 * chunk + 2], words[4 * chunk + 3]);
}

} // namespace
} // namespace ntcb
