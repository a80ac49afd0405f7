// NTC decode kernel for sm_100a with the REFERENCE'S numerics: binary16 weights, binary16
// activations and binary16 accumulators that are rounded once per 16 products, as LibNTC's own CUDA
// decoder computes (src/Inference.cu:46-136, src/tin/tin_mlp.h:22-89, src/tin/tin_mma.h:126-163).
//
// tcgen05.mma kind::f16 with a binary16 accumulator format (K = 16 per instruction) rounds exactly
// like the legacy wmma m16n16k16 path the reference is built on, so this kernel reproduces the
// reference's output bit for bit while keeping the structure of the exact-accumulation kernel in
// decode_kernel.cu: a 32x8 texel tile per CTA of 256 threads (thread = texel), two 128-row GEMM
// chains per tile, weights resident in shared memory, accumulators in tensor memory.
//
// What differs from decode_kernel.cu:
//   * the A operand holds binary16 values (the de-quantised network inputs / activations), up to 128
//     bytes per row.  Layer 0 reads it from shared memory, written by the threads in K-major
//     core-matrix order (16-byte chunk j, 8 halves, of row r at j * 2048 + r * 16); layers 2 and 3 read
//     it from tensor memory, where the activation step stores it (columns 32.. of the chain's 64,
//     beside those layers' accumulators); layer 1 reads its first two K steps from shared memory and
//     its last two from the 16 tensor-memory columns its 48 accumulators leave free;
//   * between the layers of a tile the two chains do not wait for each other (LayerBarrier,
//     kernel_parts.cuh);
//   * each layer starts with a "bias step": an MMA whose A operand has constant rows - a unit vector -
//     and whose B operand holds the bias in the column the unit vector picks, which sets the
//     accumulators to the binary16 bias exactly; the K = 16 steps of the layer then accumulate onto it.
//     (Int8 networks: ONE 64 x 8 matrix of biases, column l for layer l, and the rows e_l as one 8-row
//     core matrix that every row group reads - descriptor stride 0; FP8 networks: an N x 16 matrix per
//     layer with the bias in column 0 and 128 rows (1, 0, ..., 0).);
//   * the accumulators come back as binary16 (tcgen05.ld ... pack::16b: two per register), ready for
//     the packed-half activation; there is no scale, no integer bias, no conversion;
//   * activations are re-quantised and immediately de-quantised (e4m3, or the int8 grid k * 0.0125),
//     as the reference does (src/tin/tin_activation.h:44-48, 94-99).
//
// Every wait on an mbarrier is bounded, as in decode_kernel.cu.
//
// Two kernels live here.  DecodeKernelRef (first part of the file) keeps every operand in binary16
// and serves Int8 networks.  DecodeKernelRefFp8 (second part) serves FP8 networks with 8-bit operands
// for layers 0-2 (those of layers 1-3 in tensor memory) and produces the same bits; since ntcb_stage_network_reference lays an FP8
// network out for it, the binary16 kernel's templates are only instantiated with kFp8 = false
// (their kFp8 = true paths describe what the FP8 kernel replaces: e4m3 round trips in binary16).

#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstddef>

#include "decode_kernel.h"
#include "kernel_parts.cuh"
#include "input_stage.cuh"
#include "output_convert.cuh"
#include "epilogue_convert.cuh"

// Profiling aid: NTCB_ABLATE (a bit mask, 0 in the product build; 512: no tile walk, every tile at the place of the CTA's
// first; 1024: no barrier before a layer's products - only together with 16) removes one phase of
// DecodeKernelRefFp8 at a time so that its share of the kernel's instructions and time can be
// measured as a difference (`make ablations` builds one library per mask; their output is wrong by
// construction).  1: the per-tile tables and footprint staging after the first tile; 2: the latent
// gather and blend (constants are stored instead); 64: the tap tables are rebuilt for every tile; 4: the activation arithmetic of layers 0-2 (the
// raw accumulator words are stored); 8: the global stores of the epilogue; 16: the tensor-core work
// (no MMA issue, no wait for it); 32: the tensor-memory loads; 128: the proxy fence before each layer's
// barrier; 256: a plain barrier instead of the one that also agrees on giving up.
#ifndef NTCB_ABLATE
#define NTCB_ABLATE 0
#endif

namespace ntcb
{
namespace
{

constexpr int kAblate = NTCB_ABLATE;
// FP8 networks: the A operand of layers 1-3 lives in tensor memory, not in shared memory.  A layer's 64-byte
// input row is 16 of the 32-bit columns of its thread's own TMEM lane; layers 1-3 have at most 48 outputs,
// so their accumulators leave columns 48..63 of the chain's 64 free for it.  (Layer 0 has 64 outputs: its
// operand, the gathered inputs, stays in shared memory.)  The activations are stored with tcgen05.st, the
// products read them with the A-in-tensor-memory form of tcgen05.mma: no shared-memory stores, no proxy
// fence, and no operand reads from shared memory by the tensor core for three of the four layers (3 %).
constexpr bool kTmemOperand = true;
constexpr uint32_t kOperandColumn = 48;


// D[tmem] (+)= A[smem] * B[smem]^T, M = 128, K = 16 binary16 operands, binary16 accumulators.
__device__ __forceinline__ void UmmaF16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t instr, uint32_t accumulate,
    uint32_t enabled = 1)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(tmemD),
        "l"(descA), "l"(descB), "r"(instr), "r"(accumulate), "r"(enabled)
        : "memory");
}

// Instruction descriptor: dense, K-major A and B in binary16 (format 0), binary16 accumulators
// (format 0), M = 128; bits 17-22: N >> 3; bits 24-28: M >> 4.
__host__ __device__ constexpr uint32_t MakeInstrDescriptorF16(int n)
{
    return (uint32_t(n >> 3) << 17) | (uint32_t(128 >> 4) << 24);
}

// 32 consecutive binary16 accumulators of this thread's TMEM lane, two per register (an
// accumulator occupies the low half of a 32-bit TMEM cell; pack::16b joins adjacent columns).
__device__ __forceinline__ void TmemLoadPacked16(uint32_t address, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.pack::16b.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(address)
        : "memory");
}

// 16 consecutive binary16 accumulators, two per register.
__device__ __forceinline__ void TmemLoadPacked8(uint32_t address, uint32_t (&r)[8])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.pack::16b.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(address)
        : "memory");
}

// ---------------------------------------------------------------------------------------------
// Quantisers (value in, de-quantised value out)
// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ __half2 RoundTripE4m3(__half2 x)
{
    // src/tin/tin_activation.h:44-48: round to nearest even e4m3, saturating, and back to binary16
    const __nv_fp8x2_storage_t codes = __nv_cvt_halfraw2_to_fp8x2(static_cast<__half2_raw>(x), __NV_SATFINITE, __NV_E4M3);
    return __half2(__nv_cvt_fp8x2_to_halfraw2(codes, __NV_E4M3));
}

// A pair of network inputs as the first layer sees them.  Int8: floor(x * 127.5 - 0.5) clamped to
// +-127, times 1 / 127.5 (src/tin/tin_mlp.h:22-37).  FP8: rounded to e4m3.
template <bool kFp8>
__device__ __forceinline__ __half2 QuantizeInputRef(__half2 x)
{
    if (kFp8)
        return RoundTripE4m3(x);
    __half2 y = __hfma2(x, __float2half2_rn(127.5f), __float2half2_rn(-0.5f));
    y = h2floor(y);
    y = __hmax2(__hmin2(y, __float2half2_rn(127.f)), __float2half2_rn(-127.f));
    return __hmul2_rn(y, __float2half2_rn(1.f / 127.5f));
}

// Clamped HGELU in binary16 (src/tin/tin_activation.h:88-92) followed by the quantiser of the next
// layer's inputs: e4m3, or the int8 grid rint(y * 80) * 0.0125 (src/tin/tin_activation.h:94-99).
template <bool kToFp8>
__device__ __forceinline__ uint32_t ActivateRef(uint32_t bits)
{
    const __half2 x = AsHalf2(bits);
    const __half2 third = __float2half2_rn(1 / 3.f);
    const __half2 t = __hfma2_sat(third, x, __float2half2_rn(0.5f));
    const __half2 m = __hmin2(x, __float2half2_rn(3.f));
    const __half2 y = __hmul2_rn(m, t);
    if (kToFp8)
        return AsU32(RoundTripE4m3(y));
    const __half2 p = __hmul2_rn(y, __float2half2_rn(80.f));
    // rint(p), p in [-15, 240]: the binary16 spacing is 1 in [1024, 2048)
    __half2 r = __hadd2_rn(p, __float2half2_rn(1536.f));
    r = __hadd2_rn(r, __float2half2_rn(-1536.f));
    return AsU32(__hmul2_rn(r, __float2half2_rn(3.1875f / 255.f)));
}

// ---------------------------------------------------------------------------------------------
// Shared memory
// ---------------------------------------------------------------------------------------------

// Per-tile lookup tables: the taps (shared with the other kernels) and the positional encoding as
// quantised binary16 pairs.
struct __align__(16) RefTileTables
{
    TapTables taps;
    // positional encoding: word w = (wave w phase 0, wave w phase 0.25)
    uint4 colEnc[kTileWidth];
    uint4 rowEnc[kRefTileHeight];
    uint32_t lodPair;   // (lod, lod)
    uint32_t zeroPair;  // (quantised 0, quantised 0)
    uint32_t pad[2];
};

struct __align__(128) RefSharedStorage
{
    uint8_t network[kRefInt8NetworkBytes];                 // binary16 weights and the matrix of biases
    alignas(128) uint8_t operandA[kRefChains * kRefOperandBytes]; // A operands of layers 0 and 1 (its first half), one per chain
    // Constant A operands of the bias steps: four core matrices (8 rows x 8 halves) whose rows are the unit
    // vectors e_0 .. e_3, and one of zeros (the second 8-wide half of every step).  A stride offset of 0 in
    // the descriptor makes all sixteen 8-row groups of the 128-row operand read the same core matrix.
    alignas(128) uint8_t onesRegion[5 * 128];
    uint32_t latentTable[256];
    uint64_t barrier[kRefChains]; // MMA completion, per chain: a chain's threads go on as soon as their accumulators are ready
    uint64_t loadBarrier;  // arrival of the network image
    uint32_t tmemBase;
    // what inference on sample does not use comes last: its launches ask for the bytes before `tables` only
    alignas(128) RefTileTables tables;
    uint8_t footprintHi[kRefFootprintHiBytes];
    uint8_t footprintLo[kRefInt8FootprintLoBytes];
};

struct RefTileContext
{
    int tid;
    uint32_t tmemBase, tmemLane, operandA, networkBase, biasRegion;
    uint32_t barrierBase; // shared address of the chains' MMA-completion mbarriers
    uint32_t barrier;     // ... of this thread's chain
    uint4* rowChunk; // this thread's 16-byte slot in chunk 0 of its half's A operand
    int tile, x, y;
    uint32_t* out;
    uint32_t outStepWords;
    int storeBytes; // widest store the texel may go out with (KernelMip::storeBytes)
};

// ---------------------------------------------------------------------------------------------
// Inputs
// ---------------------------------------------------------------------------------------------

// Builds the tile's lookup tables and stages the latent footprint of both grids in shared memory
// (`tablesValid`: the tables already hold this tile's values, see PrepareTaps).
template <bool kFp8, int kLayers = 0>
__device__ __forceinline__ void PrepareTileRef(const KernelParams& params, const KernelMip& mip, RefSharedStorage& shared,
    int tileX0, int tileY0, int lane, int warp, bool tablesValid)
{
    static_assert(kRefTileHeight == kTileHeight && kRefThreadsPerCta == kThreadsPerCta, "the tap tables assume the common tile");
    if (!tablesValid && warp >= 2 && warp < 4)
    {
        // positional encoding (src/RegressionKernels.h:59-85): warp 2 the x part per column, warp 3
        // the y part per row, quantised exactly as the per-texel inputs would be
        const bool rows = warp == 3;
        const int coordinate = rows ? min(tileY0 + (lane & (kRefTileHeight - 1)), mip.rowEnd - 1) : min(tileX0 + lane, mip.width - 1);
        float f = __fmul_rn(float(coordinate), mip.positionScale);
        uint32_t q[3];
#pragma unroll
        for (int wave = 0; wave < 3; ++wave)
        {
            const float e0 = __fmaf_rn(Frac(f), 2.f, -1.f);
            const float e1 = __fmaf_rn(Frac(__fadd_rn(f, 0.25f)), 2.f, -1.f);
            q[wave] = AsU32(QuantizeInputRef<kFp8>(__floats2half2_rn(e0, e1)));
            f = __fmul_rn(f, 2.f);
        }
        if (!rows)
            shared.tables.colEnc[lane] = make_uint4(q[0], q[1], q[2], 0);
        else if (lane < kRefTileHeight)
            shared.tables.rowEnc[lane] = make_uint4(q[0], q[1], q[2], 0);
        if (rows && lane == kRefTileHeight)
        {
            shared.tables.lodPair = AsU32(QuantizeInputRef<kFp8>(__float2half2_rn(mip.positionLod)));
            shared.tables.zeroPair = AsU32(QuantizeInputRef<kFp8>(__float2half2_rn(0.f)));
        }
    }
    PrepareTaps<true, kLayers>(params, mip, shared.tables.taps, shared.footprintHi, shared.footprintLo, shared.latentTable, tileX0,
        tileY0, lane, warp, tablesValid);
}

// Four inputs of one latent layer from the four taps, as two binary16 pairs.
// Blend order as the reference build evaluates it: fma(l11,w3, fma(l10,w2, fma(l00,w0, l01*w1))).
template <bool kFp8>
__device__ __forceinline__ void BlendLayerRef(uint2 l00, uint2 l01, uint2 l10, uint2 l11, __half2 w00, __half2 w01,
    __half2 w10, __half2 w11, uint32_t* words)
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
    words[0] = AsU32(QuantizeInputRef<kFp8>(a));
    words[1] = AsU32(QuantizeInputRef<kFp8>(b));
}

// Inputs 0..15 or 16..31 of one texel (eight binary16 pairs) from the staged footprint of one grid.
template <bool kFp8, int kLayers = 0>
__device__ __forceinline__ void GatherGridRef(const KernelParams& params, const KernelMip& mip, const RefSharedStorage& shared,
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
            BlendLayerRef<kFp8>(l00, l01, l10, l11, w00, w01, w10, w11, words + 2 * layer);
        }
    }
}

// One latent layer of one grid (the low 16 bits of each p are the tap's four features) -> two pairs of inputs.
template <bool kFp8>
__device__ __forceinline__ void BlendPixelsRef(uint32_t p00, uint32_t p01, uint32_t p10, uint32_t p11, const GridTaps& taps,
    const uint32_t* __restrict__ lut, uint32_t* words)
{
#pragma unroll
    for (int j = 0; j < 2; ++j)
    {
        const __half2 l00 = AsHalf2(lut[(p00 >> (8 * j)) & 0xFF]), l01 = AsHalf2(lut[(p01 >> (8 * j)) & 0xFF]);
        const __half2 l10 = AsHalf2(lut[(p10 >> (8 * j)) & 0xFF]), l11 = AsHalf2(lut[(p11 >> (8 * j)) & 0xFF]);
        __half2 d = __hmul2_rn(l01, taps.w01);
        d = __hfma2(l00, taps.w00, d);
        d = __hfma2(l10, taps.w10, d);
        d = __hfma2(l11, taps.w11, d);
        d = __hfma2(d, __float2half2_rn(2.f), __float2half2_rn(-1.f));
        words[j] = AsU32(QuantizeInputRef<kFp8>(d));
    }
}

// ... with the taps read straight from the layer's plane in global memory.
template <bool kFp8>
__device__ __forceinline__ void SampleLayerRef(const uint16_t* __restrict__ plane, const GridTaps& taps,
    const uint32_t* __restrict__ lut, uint32_t* words)
{
    const uint32_t p00 = __ldg(plane + taps.o00), p01 = __ldg(plane + taps.o01);
    const uint32_t p10 = __ldg(plane + taps.o10), p11 = __ldg(plane + taps.o11);
    BlendPixelsRef<kFp8>(p00, p01, p10, p11, taps, lut, words);
}

// The 48 network inputs of one texel as 24 binary16 pairs -> its 96-byte row of the A operand.
template <bool kFp8, int kLayers = 0>
__device__ __forceinline__ void BuildInputsRef(const KernelParams& params, const KernelMip& mip, const RefSharedStorage& shared,
    const RefTileContext& ctx, int lane, int tileRow)
{
    uint32_t words[24];
    const uint32_t zeroPair = shared.tables.zeroPair;
#pragma unroll
    for (int i = 0; i < 16; ++i)
        words[i] = zeroPair; // unused feature slots hold quantised zeros (src/Inference.cu:49)

    if (mip.staged)
    {
        GatherGridRef<kFp8, kLayers>(params, mip, shared, 0, lane, tileRow, words);
        GatherGridRef<kFp8, kLayers>(params, mip, shared, 1, lane, tileRow, words + 8);
    }
    else
    {
        // footprint too large to stage: read the taps from global memory; threads past the right /
        // bottom edge compute a clamped texel and store nothing
        const int x = min(ctx.x, mip.width - 1), y = min(ctx.y, mip.rowEnd - 1);
        const float u = TexelCoordinate<true>(x, mip.width, mip.invWidth);
        const float v = TexelCoordinate<true>(y, mip.height, mip.invHeight);
        GridTaps taps;
        SetupTaps(u, v, mip.hiWidth, mip.hiHeight, taps);
        const uint16_t* hi = params.latents + mip.hiOffset;
#pragma unroll
        for (int layer = 0; layer < 4; ++layer)
            if (layer < NumLayers<kLayers>(params))
                SampleLayerRef<kFp8>(hi + size_t(layer) * mip.hiPlane, taps, shared.latentTable, words + 2 * layer);
        SetupTaps(u, v, mip.loWidth, mip.loHeight, taps);
        const uint16_t* lo = params.latents + mip.loOffset;
#pragma unroll
        for (int layer = 0; layer < 4; ++layer)
            if (layer < NumLayers<kLayers>(params))
                SampleLayerRef<kFp8>(lo + size_t(layer) * mip.loPlane, taps, shared.latentTable, words + 8 + 2 * layer);
    }

    // positional encoding: per wave the inputs (x phase 0, y phase 0, x phase 0.25, y phase 0.25)
    const uint4 cx = shared.tables.colEnc[lane];
    const uint4 ry = shared.tables.rowEnc[tileRow];
    words[16] = __byte_perm(cx.x, ry.x, 0x5410);
    words[17] = __byte_perm(cx.x, ry.x, 0x7632);
    words[18] = __byte_perm(cx.y, ry.y, 0x5410);
    words[19] = __byte_perm(cx.y, ry.y, 0x7632);
    words[20] = __byte_perm(cx.z, ry.z, 0x5410);
    words[21] = __byte_perm(cx.z, ry.z, 0x7632);
    words[22] = shared.tables.lodPair;
    words[23] = zeroPair;

#pragma unroll
    for (int chunk = 0; chunk < 6; ++chunk)
        ctx.rowChunk[chunk * 128] = make_uint4(words[4 * chunk], words[4 * chunk + 1], words[4 * chunk + 2], words[4 * chunk + 3]);
}

// ---------------------------------------------------------------------------------------------
// Layers
// ---------------------------------------------------------------------------------------------

// Int8 networks (binary16 operands): where a layer's inputs live.  A chain has 64 tensor-memory columns; a column
// holds one accumulator or two operand halves, so K step s (16 halves) of an operand in tensor memory is
// columns 32 + 8 s .. 32 + 8 s + 7.  Layers 2 and 3 (48 and 32 inputs beside 32 and 16 accumulators) have all
// their K steps there; layer 1 (64 inputs beside 48 accumulators) its last two, columns 48..63, and the first
// two in shared memory; layer 0's 48 inputs are all in shared memory (its 64 accumulators fill the chain).
constexpr uint32_t kRefOperandColumn = 32;
template <int kLayer>
constexpr int kRefFirstTmemStep = kLayer == 0 ? 99 : kLayer == 1 ? 2 : 0;
template <int kLayer>
constexpr bool kRefOperandInTmem = kRefFirstTmemStep<kLayer> == 0;      // nothing of it in shared memory
template <int kLayer>
constexpr bool kRefOperandInShared = kRefFirstTmemStep<kLayer> != 0;    // some of it in shared memory

__device__ __forceinline__ void UmmaF16FromTmem(uint32_t tmemD, uint32_t tmemA, uint64_t descB, uint32_t instr, uint32_t accumulate,
    uint32_t enabled)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}" ::"r"(tmemD),
        "r"(tmemA), "l"(descB), "r"(instr), "r"(accumulate), "r"(enabled)
        : "memory");
}

// First half of a layer for the current tile: barrier (LayerBarrier) and MMA issue - of both chains by warp 4
// after a CTA-wide barrier, of its own chain by the chain's first warp after a chain-local one.  Returns
// nonzero (uniformly over the threads that met in the barrier) when some thread gave up on a wait.
template <int kLayer, int kChainLocal = TileLayerBarrier<kLayer>()>
__device__ __forceinline__ int IssueLayerRef(const RefTileContext& ctx, int failed)
{
    constexpr int kN = kLayer == 0 ? 64 : kLayer == 1 ? 48 : kLayer == 2 ? 32 : 16;
    constexpr int kK = kLayer == 0 ? 48 : kLayer == 1 ? 64 : kLayer == 2 ? 48 : 32;
    constexpr int kWeightOffset =
        kLayer == 0 ? kRefWeightOffset0 : kLayer == 1 ? kRefWeightOffset1 : kLayer == 2 ? kRefWeightOffset2 : kRefWeightOffset3;

    // Makes the A operand written before this call visible to the tensor core, orders every
    // thread's TMEM reads of the previous layer before the accumulators are overwritten, and agrees
    // on whether any thread gave up waiting.
    if (kRefFirstTmemStep<kLayer> < kK / 16)
        TmemStoreWait(); // (part of) the operand went to tensor memory
    if (kRefOperandInShared<kLayer>)
        FenceProxyAsyncShared();
    TcgenFenceBeforeSync();
    if (LayerBarrier<kChainLocal>(ctx.tid, failed))
        return 1;

    // The whole issuing warp runs the descriptor arithmetic on values that are visibly the same in every
    // lane; one elected lane hands the work to the tensor core (see IssueLayerRefFp8).
    const int warpIndex = ctx.tid >> 5;
    if (kChainLocal ? (warpIndex & 3) == 0 : warpIndex == kIssuingWarp)
    {
        TcgenFenceAfterSync();
        constexpr uint32_t instr = MakeInstrDescriptorF16(kN);
        const uint32_t networkBase = __shfl_sync(0xFFFFFFFFu, ctx.networkBase, 0);
        const uint32_t tmemBase = __shfl_sync(0xFFFFFFFFu, ctx.tmemBase, 0);
        const uint32_t barrierBase = __shfl_sync(0xFFFFFFFFu, ctx.barrierBase, 0);
        // the four base descriptors are built once, every operand is then a constant offset (in 16-byte
        // units) added to the address field
        const uint64_t operandBase = MakeSmemDescriptor(__shfl_sync(0xFFFFFFFFu, ctx.operandA, 0), 2048, 128);
        // rows e_kLayer (every 8-row group reads the same core matrix: stride 0), then the core matrix of zeros
        const uint64_t onesBase = MakeSmemDescriptor(__shfl_sync(0xFFFFFFFFu, ctx.biasRegion, 0) + kLayer * 128, (4 - kLayer) * 128, 0);
        const uint64_t weightBase = MakeSmemDescriptor(networkBase + kWeightOffset, kN * 16, 128);
        // the matrix of biases, read twice (leading offset 0): its second copy meets the zeros
        const uint64_t biasBase = MakeSmemDescriptor(networkBase + kRefInt8BiasOffset, 0, 128);
        const uint32_t elected = ElectOne();
        const int ownChain = __shfl_sync(0xFFFFFFFFu, warpIndex >> 2, 0);
#pragma unroll
        for (int half = 0; half < kRefChains; ++half)
        {
            if (kChainLocal && half != ownChain)
                continue;
            const uint32_t accumulators = tmemBase + half * kTmemColumnsPerHalf;
            // accumulators := bias (rows e_l times the matrix whose column l is the layer's bias: exact)
            UmmaF16(accumulators, onesBase, biasBase, instr, 0, elected);
#pragma unroll
            for (int kStep = 0; kStep < kK / 16; ++kStep)
            {
                // one K step = two 16-byte core matrices; A: 2048 bytes apart, B: kN*16 bytes apart
                const uint64_t descA = operandBase + uint64_t((half * kRefOperandBytes + kStep * 2 * 2048) >> 4);
                const uint64_t descB = weightBase + uint64_t((kStep * 2 * kN * 16) >> 4);
                if (kStep >= kRefFirstTmemStep<kLayer>)
                    UmmaF16FromTmem(accumulators, accumulators + kRefOperandColumn + uint32_t(kStep) * 8u, descB, instr, 1, elected);
                else
                    UmmaF16(accumulators, descA, descB, instr, 1, elected);
            }
            // arrives once everything issued so far has completed: this chain's accumulators are ready
            if (elected)
                UmmaCommit(barrierBase + half * 8);
        }
    }
    return 0;
}

// Second half of a layer: waits for the MMA, then applies the activation and writes the next
// layer's A operand (layers 0-2) or stores the texel (layer 3).
template <bool kFp8, int kLayer, bool kConvert, typename Params>
__device__ __forceinline__ void ConsumeLayerRef(const Params& params, const RefTileContext& ctx, uint32_t& phase, int& failed)
{
    constexpr int kN = kLayer == 0 ? 64 : kLayer == 1 ? 48 : kLayer == 2 ? 32 : 16;

    if (!MbarrierWaitBounded(ctx.barrier, phase))
    {
        failed = 1;
        ReportTimeout(params.status, uint32_t(ctx.tile), uint32_t(kLayer));
    }
    phase ^= 1;
    TcgenFenceAfterSync();

    if (kLayer < 3)
    {
        constexpr bool kNextFp8 = kFp8 && kLayer < 2; // layer 2 always re-quantises to the int8 grid
        uint4* rowChunk = ctx.rowChunk;
        // all accumulators of the row are requested before the first wait, so that the round trips to
        // tensor memory overlap: 64 -> two loads of 32, 48 -> 32 + 16, 32 -> one load
        uint32_t low[16], high[16];
        TmemLoadPacked16(ctx.tmemLane, low);
        if (kN == 64)
            TmemLoadPacked16(ctx.tmemLane + 32, high);
        else if (kN == 48)
        {
            uint32_t (&tail)[8] = reinterpret_cast<uint32_t (&)[8]>(high);
            TmemLoadPacked8(ctx.tmemLane + 32, tail);
        }
        TmemLoadWait();
        // chunk c (8 halves, half a K step) of the next layer's operand row: to shared memory, or to tensor-memory
        // columns 32 + 4 c ..
        auto storeChunk = [&](int c, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
            if (c >= 2 * kRefFirstTmemStep<kLayer + 1>)
                TmemStore4(ctx.tmemLane + kRefOperandColumn + 4u * uint32_t(c), w0, w1, w2, w3);
            else
                rowChunk[c * 128] = make_uint4(w0, w1, w2, w3);
        };
#pragma unroll
        for (int c = 0; c < 4; ++c)
            storeChunk(c, ActivateRef<kNextFp8>(low[4 * c]), ActivateRef<kNextFp8>(low[4 * c + 1]),
                       ActivateRef<kNextFp8>(low[4 * c + 2]), ActivateRef<kNextFp8>(low[4 * c + 3]));
#pragma unroll
        for (int c = 0; c < (kN - 32) / 8; ++c)
            storeChunk(4 + c, ActivateRef<kNextFp8>(high[4 * c]), ActivateRef<kNextFp8>(high[4 * c + 1]),
                       ActivateRef<kNextFp8>(high[4 * c + 2]), ActivateRef<kNextFp8>(high[4 * c + 3]));
    }
    else
    {
        // output (src/Inference.cu:121-135): the accumulators are the channels
        uint32_t bits[8];
        TmemLoadPacked8(ctx.tmemLane, bits);
        TmemLoadWait();
        const int channelPairs = params.channels >> 1;
        ScrubSpecials(bits, channelPairs);
        if constexpr (kConvert)
        {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (j >= channelPairs)
                    bits[j] = 0;
            if (ctx.out)
                StoreConverted(params.conversion, params.firstChannel, params.numChannels, ctx, bits);
        }
        else if (ctx.out)
            StoreTexel(ctx.out, ctx.outStepWords, ctx.storeBytes, bits, channelPairs);
    }
}

template <bool kFp8, int kLayer, bool kConvert, int kChainLocal = TileLayerBarrier<kLayer>(), typename Params>
__device__ __forceinline__ int RunLayerRef(const Params& params, const RefTileContext& ctx, uint32_t& phase, int& failed)
{
    if (IssueLayerRef<kLayer, kChainLocal>(ctx, failed))
        return 1;
    ConsumeLayerRef<kFp8, kLayer, kConvert>(params, ctx, phase, failed);
    return 0;
}

// One-time setup of a CTA: the network image arrives by one TMA bulk copy while the threads fill
// the constant tables, set up the barriers and allocate tensor memory.  Returns nonzero in every
// thread that gave up waiting for the image (status words written).
__device__ __forceinline__ int SetupCtaRef(RefSharedStorage& shared, const uint8_t* network, uint32_t* status, uint32_t loadWaitPolls, int tid, int warp)
{
    // src/Quantizer.cu:490-495: value = float(nibble) * (1.f / 15.f), stored as binary16
    for (int i = tid; i < 256; i += kRefThreadsPerCta)
    {
        __half lo = __float2half_rn(__fmul_rn(float(i & 15), 1.f / 15.f));
        __half hi = __float2half_rn(__fmul_rn(float(i >> 4), 1.f / 15.f));
        shared.latentTable[i] = AsU32(__halves2half2(lo, hi));
    }
    // constant A operands of the bias steps: core matrix l (8 rows of 16 bytes) has 1.0 as half l of every row,
    // core matrix 4 is zero
    for (int i = tid; i < 5 * 8; i += kRefThreadsPerCta)
    {
        const int unit = i >> 3;
        reinterpret_cast<uint4*>(shared.onesRegion)[i] =
            make_uint4(unit == 0 ? 0x00003C00u : unit == 1 ? 0x3C000000u : 0u, unit == 2 ? 0x00003C00u : unit == 3 ? 0x3C000000u : 0u, 0u, 0u);
    }
    const uint32_t loadBarrier = SharedAddress(&shared.loadBarrier);
    if (tid == 0)
    {
        for (int chain = 0; chain < kRefChains; ++chain)
            MbarrierInit(SharedAddress(&shared.barrier[chain]), 1);
        MbarrierInit(loadBarrier, 1);
        FenceBarrierInit();
        MbarrierArriveExpectTx(loadBarrier, kRefInt8NetworkBytes);
        BulkCopyToShared(SharedAddress(shared.network), network, kRefInt8NetworkBytes, loadBarrier);
    }
    if (warp == 0)
        TmemAlloc(SharedAddress(&shared.tmemBase), kRefTmemColumns);
    FenceProxyAsyncShared(); // the bias region is read by the tensor core (async proxy)
    TcgenFenceBeforeSync();
    __syncthreads();
    TcgenFenceAfterSync();
    int failed = 0;
    if (!MbarrierWaitBounded(loadBarrier, 0, loadWaitPolls))
    {
        failed = 1;
        ReportTimeout(status, 0xFFFFFFFFu, 0xFFFFFFFFu); // no tile: the network image did not arrive
    }
    return failed;
}

// End of a CTA: agrees on whether anything went wrong, gives work in flight one more bounded chance
// to drain, and releases the tensor memory.
__device__ __forceinline__ void TeardownCtaRef(RefSharedStorage& shared, const RefTileContext& ctx, uint32_t phase, int failed,
    int tid, int warp)
{
    TcgenFenceBeforeSync();
    const int aborted = __syncthreads_or(failed);
    if (aborted && tid == 0)
    {
        for (int chain = 0; chain < kRefChains; ++chain)
            (void)MbarrierWaitBounded(ctx.barrierBase + chain * 8, phase ^ 1);
        (void)MbarrierWaitBounded(SharedAddress(&shared.loadBarrier), 0);
    }
    __syncthreads();
    if (warp == 0)
        TmemFree(ctx.tmemBase, kRefTmemColumns);
}

// ---------------------------------------------------------------------------------------------
// The kernels
// ---------------------------------------------------------------------------------------------

template <bool kFp8, bool kConvert, int kLayers>
__global__ void __launch_bounds__(kRefThreadsPerCta, kCtasPerSmRef) DecodeKernelRef(const __grid_constant__ KernelParams params)
{
    extern __shared__ __align__(128) unsigned char dynamicShared[];
    RefSharedStorage& shared = *reinterpret_cast<RefSharedStorage*>(dynamicShared);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;      // = the thread's row of the tile
    const int half = warp >> 2;     // the 128-row chain of this thread: rows 4 * half .. + 3 of the tile

    int failed = SetupCtaRef(shared, params.network, params.status, params.loadWaitPolls, tid, warp); // this thread gave up on a wait
    const uint32_t tmemBase = shared.tmemBase;
    uint32_t phase = 0;
    int aborted = 0;  // some thread of the CTA gave up (uniform: comes out of a barrier)

    RefTileContext ctx;
    ctx.tid = tid;
    ctx.tmemBase = tmemBase;
    // a warp may only touch the TMEM lanes 32 * (warp % 4) .. + 31
    ctx.tmemLane = tmemBase + half * kTmemColumnsPerHalf + (uint32_t((warp & 3) * 32) << 16);
    ctx.barrierBase = SharedAddress(&shared.barrier[0]);
    ctx.barrier = ctx.barrierBase + half * 8;
    ctx.operandA = SharedAddress(shared.operandA);
    ctx.rowChunk = reinterpret_cast<uint4*>(shared.operandA + half * kRefOperandBytes) + (tid & 127);
    ctx.networkBase = SharedAddress(shared.network);
    ctx.biasRegion = SharedAddress(shared.onesRegion);

    struct TilePlace
    {
        int mipIndex, tileX0, tileY0;
    };
    auto locate = [&](int tile, int fromMip) {
        TilePlace place;
        place.mipIndex = fromMip;
        while (place.mipIndex + 1 < params.numMips && tile >= params.mips[place.mipIndex + 1].firstTile)
            ++place.mipIndex;
        const KernelMip& mip = params.mips[place.mipIndex];
        const int local = tile - mip.firstTile;
        const int tileY = mip.tilesX == 1 ? local : int(__umulhi(uint32_t(local), mip.tilesXMagic));
        place.tileX0 = (local - tileY * mip.tilesX) * kTileWidth;
        place.tileY0 = mip.rowBegin + tileY * kRefTileHeight;
        return place;
    };

    int tile = blockIdx.x;
    TilePlace place{0, 0, 0};
    int tablesMip = -1; // mip whose tap / encoding tables are in shared memory and valid for every inner tile of it
    if (tile < params.totalTiles)
    {
        place = locate(tile, 0);
        PrepareTileRef<kFp8, kLayers>(params, params.mips[place.mipIndex], shared, place.tileX0, place.tileY0, lane, warp, false);
        tablesMip = TileKeepsTables(params.mips[place.mipIndex], place.tileX0, place.tileY0) ? place.mipIndex : -1;
        __syncthreads();
    }
    while (tile < params.totalTiles)
    {
        const KernelMip& mip = params.mips[place.mipIndex];
        ctx.tile = tile;
        ctx.x = place.tileX0 + lane;
        ctx.y = place.tileY0 + warp;
        BuildInputsRef<kFp8, kLayers>(params, mip, shared, ctx, lane, warp);

        // layer 0; while the tensor core works on it, prepare the NEXT tile (its tables and
        // footprints replace this tile's, which nobody reads after the barrier inside IssueLayerRef)
        aborted = IssueLayerRef<0>(ctx, failed);
        if (aborted)
            break;
        const int nextTile = tile + int(gridDim.x);
        if (nextTile < params.totalTiles)
        {
            place = locate(nextTile, place.mipIndex);
            // the tables of the previous tile serve this one too when both lie inside the same mip with invariant tables
            const bool keepsTables = TileKeepsTables(params.mips[place.mipIndex], place.tileX0, place.tileY0);
            PrepareTileRef<kFp8, kLayers>(params, params.mips[place.mipIndex], shared, place.tileX0, place.tileY0, lane, warp, keepsTables && place.mipIndex == tablesMip);
            tablesMip = keepsTables ? place.mipIndex : -1;
        }
        ConsumeLayerRef<kFp8, 0, false>(params, ctx, phase, failed);

        aborted = RunLayerRef<kFp8, 1, false>(params, ctx, phase, failed);
        if (!aborted) aborted = RunLayerRef<kFp8, 2, false>(params, ctx, phase, failed);
        if (aborted)
            break;
        {
            // where the texel goes (worked out only now: nothing of it has to stay in registers through the
            // layers); the element index inside a mip fits 32 bits (checked on the host)
            const bool planar = params.outputLayout == kLayoutPlanarPairs;
            const uint32_t first = planar ? uint32_t(ctx.y) * uint32_t(mip.width) * uint32_t(params.channels) + 2u * uint32_t(ctx.x)
                                          : (uint32_t(ctx.y) * uint32_t(mip.width) + uint32_t(ctx.x)) * uint32_t(params.channels);
            const bool inside = ctx.x < mip.width && ctx.y < mip.rowEnd;
            if constexpr (kConvert)
            {
                // pixels of dstChannels components, rows without padding; outOffset counts components
                const uint32_t pixelIndex = uint32_t(ctx.y) * uint32_t(mip.width) + uint32_t(ctx.x);
                const size_t component = size_t(mip.outOffset) + size_t(pixelIndex) * size_t(params.conversion.dstChannels);
                unsigned char* bytes = reinterpret_cast<unsigned char*>(params.out) + component * BytesPerComponent(params.conversion.format);
                ctx.out = inside ? reinterpret_cast<uint32_t*>(bytes) : nullptr;
                ctx.outStepWords = pixelIndex;
            }
            else
            {
                ctx.out = inside ? reinterpret_cast<uint32_t*>(params.out + mip.outOffset + first) : nullptr;
                ctx.outStepWords = planar ? uint32_t(mip.width) : 1u;
                ctx.storeBytes = mip.storeBytes;
            }
        }
        aborted = RunLayerRef<kFp8, 3, kConvert>(params, ctx, phase, failed);
        if (aborted)
            break;
        tile = nextTile;
    }

    TeardownCtaRef(shared, ctx, phase, failed, tid, warp);
}

// Inference on sample with the reference's numerics: one thread per query (u, v, lod) -> the texel
// (mip = clamp(floor(lod)), x = min(floor(u * W), W - 1), y likewise) is evaluated exactly as the
// decode kernel evaluates it; the taps are read straight from global memory.
template <bool kFp8>
__global__ void __launch_bounds__(kRefThreadsPerCta, kCtasPerSmRefSample) SampleKernelRef(const __grid_constant__ SampleParams params)
{
    extern __shared__ __align__(128) unsigned char dynamicShared[];
    RefSharedStorage& shared = *reinterpret_cast<RefSharedStorage*>(dynamicShared);
    __shared__ KernelMip mipTable[16];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int half = warp >> 2;

    // the mip descriptions are indexed per thread: a copy in shared memory (visible after the barrier inside SetupCtaRef)
    if (tid < params.numMips)
        mipTable[tid] = params.mips[tid];
    int failed = SetupCtaRef(shared, params.network, params.status, params.loadWaitPolls, tid, warp);
    int aborted = 0;
    uint32_t phase = 0;

    RefTileContext ctx;
    ctx.tid = tid;
    ctx.tmemBase = shared.tmemBase;
    ctx.tmemLane = ctx.tmemBase + half * kTmemColumnsPerHalf + (uint32_t((warp & 3) * 32) << 16);
    ctx.barrierBase = SharedAddress(&shared.barrier[0]);
    ctx.barrier = ctx.barrierBase + half * 8;
    ctx.operandA = SharedAddress(shared.operandA);
    ctx.rowChunk = reinterpret_cast<uint4*>(shared.operandA + half * kRefOperandBytes) + (tid & 127);
    ctx.networkBase = SharedAddress(shared.network);
    ctx.biasRegion = SharedAddress(shared.onesRegion);
    ctx.outStepWords = 1;
    ctx.storeBytes = 4;

    const uint32_t zeroPair = AsU32(QuantizeInputRef<kFp8>(__float2half2_rn(0.f)));
    const unsigned long long tiles = (params.numQueries + kRefThreadsPerCta - 1) / kRefThreadsPerCta;
    // a tile's queries are requested one tile ahead: their latency passes under the previous tile's layers
    float nextU = 0.f, nextV = 0.f, nextLod = 0.f;
    auto requestQuery = [&](unsigned long long ofTile) {
        if (ofTile < tiles)
        {
            const unsigned long long q = min(ofTile * kRefThreadsPerCta + tid, params.numQueries - 1);
            nextU = __ldg(params.queries + 3 * q);
            nextV = __ldg(params.queries + 3 * q + 1);
            nextLod = __ldg(params.queries + 3 * q + 2);
        }
    };
    requestQuery(blockIdx.x);
    for (unsigned long long tile = blockIdx.x; tile < tiles; tile += gridDim.x)
    {
        const unsigned long long query = tile * kRefThreadsPerCta + tid;
        const bool valid = query < params.numQueries;
        const float u = nextU, v = nextV, lod = nextLod;
        requestQuery(tile + gridDim.x);
        const int mipIndex = max(0, min(params.numMips - 1, int(floorf(lod))));
        const KernelMip& mip = mipTable[mipIndex];
        const int x = max(0, min(mip.width - 1, int(floorf(__fmul_rn(u, float(mip.width))))));
        const int y = max(0, min(mip.height - 1, int(floorf(__fmul_rn(v, float(mip.height))))));
        ctx.tile = int(tile);
        ctx.x = x;
        ctx.y = y;
        ctx.out = valid ? reinterpret_cast<uint32_t*>(params.out + query * params.channels) : nullptr;

        {
            uint32_t words[24];
#pragma unroll
            for (int i = 0; i < 16; ++i)
                words[i] = zeroPair; // unused feature slots hold quantised zeros (src/Inference.cu:49)
            // src/Inference.cu:52-53
            const float su = TexelCoordinate<true>(x, mip.width, mip.invWidth);
            const float sv = TexelCoordinate<true>(y, mip.height, mip.invHeight);
            GridTaps taps;
            SetupTaps(su, sv, mip.hiWidth, mip.hiHeight, taps);
            const uint16_t* hi = params.latents + mip.hiOffset;
            const uint16_t* lo = params.latents + mip.loOffset;
            if (params.interleaved)
            {
                GridTaps lowTaps;
                SetupTaps(su, sv, mip.loWidth, mip.loHeight, lowTaps);
                SampleInterleaved(hi, lo, params.numLayers, taps, lowTaps,
                    [&](int grid, int layer, uint32_t p00, uint32_t p01, uint32_t p10, uint32_t p11) {
                        BlendPixelsRef<kFp8>(p00, p01, p10, p11, grid ? lowTaps : taps, shared.latentTable, words + 8 * grid + 2 * layer);
                    });
            }
            else
            {
#pragma unroll
                for (int layer = 0; layer < 4; ++layer)
                    if (layer < params.numLayers)
                        SampleLayerRef<kFp8>(hi + size_t(layer) * mip.hiPlane, taps, shared.latentTable, words + 2 * layer);
                SetupTaps(su, sv, mip.loWidth, mip.loHeight, taps);
#pragma unroll
                for (int layer = 0; layer < 4; ++layer)
                    if (layer < params.numLayers)
                        SampleLayerRef<kFp8>(lo + size_t(layer) * mip.loPlane, taps, shared.latentTable, words + 8 + 2 * layer);
            }
            // src/RegressionKernels.h:59-85: per wave the inputs (x phase 0, y phase 0, x phase 0.25, y phase 0.25)
            float xf = __fmul_rn(float(x), mip.positionScale);
            float yf = __fmul_rn(float(y), mip.positionScale);
#pragma unroll
            for (int wave = 0; wave < 3; ++wave)
            {
                const float ex = __fmaf_rn(Frac(xf), 2.f, -1.f), ey = __fmaf_rn(Frac(yf), 2.f, -1.f);
                const float ez = __fmaf_rn(Frac(__fadd_rn(xf, 0.25f)), 2.f, -1.f);
                const float ew = __fmaf_rn(Frac(__fadd_rn(yf, 0.25f)), 2.f, -1.f);
                words[16 + 2 * wave] = AsU32(QuantizeInputRef<kFp8>(__floats2half2_rn(ex, ey)));
                words[17 + 2 * wave] = AsU32(QuantizeInputRef<kFp8>(__floats2half2_rn(ez, ew)));
                xf = __fmul_rn(xf, 2.f);
                yf = __fmul_rn(yf, 2.f);
            }
            words[22] = AsU32(QuantizeInputRef<kFp8>(__float2half2_rn(mip.positionLod)));
            words[23] = zeroPair;
#pragma unroll
            for (int chunk = 0; chunk < 6; ++chunk)
                ctx.rowChunk[chunk * 128] = make_uint4(words[4 * chunk], words[4 * chunk + 1], words[4 * chunk + 2], words[4 * chunk + 3]);
        }

        // nothing is shared between the chains of a query tile: each runs at its own pace
        aborted = RunLayerRef<kFp8, 0, false, 2>(params, ctx, phase, failed);
        if (!aborted) aborted = RunLayerRef<kFp8, 1, false, 2>(params, ctx, phase, failed);
        if (!aborted) aborted = RunLayerRef<kFp8, 2, false, 2>(params, ctx, phase, failed);
        if (!aborted) aborted = RunLayerRef<kFp8, 3, false, 2>(params, ctx, phase, failed);
        if (aborted)
            break;
    }
    TeardownCtaRef(shared, ctx, phase, failed, tid, warp);
}

// =============================================================================================
// FP8 networks: the same arithmetic with 8-bit operands
// =============================================================================================
//
// In an FP8 network the inputs of layers 0-2 and their weights are e4m3 numbers, which binary16
// holds exactly, so the products the reference forms are the same whether the operands are stored
// as binary16 or as e4m3 bytes.  What has to be preserved is the rounding rhythm: one rounding of
// the binary16 accumulator per 16 products.  tcgen05.mma kind::f8f6f4 takes 32 products per
// instruction, so every 32-wide K chunk is issued twice, against two copies of the weights of
// which one has columns 16-31 zeroed and the other columns 0-15: each instruction adds 16 real
// products (and 16 exact zeros) to the accumulator and rounds once - bit for bit what the binary16
// path does (checked on the GPU against wmma on 1.2 M accumulators before this kernel was written).
// The A operand shrinks to 64 bytes per row, which lets four CTAs share an SM.  Layer 3 (int8-grid
// activations, weights rebuilt from int8) stays on the binary16 path; its 32 inputs fit the same
// 64-byte rows.

struct __align__(128) RefFp8SharedStorage
{
    uint8_t network[kRefNetworkBytes];                  // layers 0-2: split e4m3 weight copies; layer 3 and bias steps: binary16
    alignas(128) uint8_t operandA[2 * kOperandBytes];   // A operands (top half, bottom half): 128 rows x 64 bytes each
    alignas(128) uint8_t biasRegion[128 * 32];          // constant binary16 A operand of the bias step: rows (1, 0 x 15)
    uint32_t latentTable[256];
    uint64_t barrier[kRefChains]; // MMA completion, per chain
    uint64_t loadBarrier;         // arrival of the network image
    uint32_t tmemBase;
    // what inference on sample does not use comes last: its launches ask for the bytes before `tables` only
    // (with the whole structure a sample kernel's static table of mips would cost it the fourth CTA per SM)
    alignas(128) TileTables tables;
    uint8_t footprintHi[kRefFootprintHiBytes];
    uint8_t footprintLo[kRefFootprintLoBytes];
};

// D[tmem] (+)= A[smem] * B[smem]^T, M = 128, K = 32 e4m3 operands, binary16 accumulators.
__device__ __forceinline__ void UmmaE4m3F16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t instr, uint32_t accumulate,
    uint32_t enabled = 1)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(tmemD),
        "l"(descA), "l"(descB), "r"(instr), "r"(accumulate), "r"(enabled)
        : "memory");
}

// The same two products with the A operand in tensor memory (lane = row, four 8-bit or two 16-bit K values per column).
__device__ __forceinline__ void UmmaE4m3F16FromTmem(uint32_t tmemD, uint32_t tmemA, uint64_t descB, uint32_t instr, uint32_t accumulate,
    uint32_t enabled)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t"
        "}" ::"r"(tmemD),
        "r"(tmemA), "l"(descB), "r"(instr), "r"(accumulate), "r"(enabled)
        : "memory");
}

// What the matrix products of a layer address, the same for every tile: descriptors of the operand regions
// (those of chain 1 lie kOperandBytes further) and the accumulator columns.
struct ChainBases
{
    uint64_t operand, ones, weight, bias;
    uint32_t accumulators, barrierBase;
};

template <int kLayer>
__device__ __forceinline__ ChainBases MakeChainBases(const RefTileContext& ctx)
{
    constexpr int kN = kLayer == 0 ? 64 : kLayer == 1 ? 48 : kLayer == 2 ? 32 : 16;
    constexpr int kWeightOffset =
        kLayer == 0 ? kRefWeightOffset0 : kLayer == 1 ? kRefWeightOffset1 : kLayer == 2 ? kRefWeightOffset2 : kRefWeightOffset3;
    constexpr int kBiasOffset =
        kLayer == 0 ? kRefBiasOffset0 : kLayer == 1 ? kRefBiasOffset1 : kLayer == 2 ? kRefBiasOffset2 : kRefBiasOffset3;
    ChainBases bases;
    // The issuing thread is the critical path of the layer: the four base descriptors are built
    // once, every operand is then a constant offset (in 16-byte units) added to the address field.
    bases.operand = MakeSmemDescriptor(ctx.operandA, 2048, 128);
    bases.ones = MakeSmemDescriptor(ctx.biasRegion, 2048, 128);
    bases.weight = MakeSmemDescriptor(ctx.networkBase + kWeightOffset, kN * 16, 128);
    bases.bias = MakeSmemDescriptor(ctx.networkBase + kBiasOffset, kN * 16, 128);
    bases.accumulators = ctx.tmemBase;
    bases.barrierBase = ctx.barrierBase;
    return bases;
}

// The matrix products of one layer for one chain of the tile, issued by the calling thread.
template <int kLayer>
__device__ __forceinline__ void IssueChainRefFp8(const ChainBases& bases, int half, uint32_t enabled)
{
    constexpr int kN = kLayer == 0 ? 64 : kLayer == 1 ? 48 : kLayer == 2 ? 32 : 16;
    constexpr int kK = kLayer == 0 ? 48 : kLayer == 1 ? 64 : kLayer == 2 ? 48 : 32;
    // both descriptors: binary16 accumulators, operand formats 0 (binary16 for kind::f16, e4m3 for kind::f8f6f4)
    constexpr uint32_t instr = MakeInstrDescriptorF16(kN);
    const uint64_t operandBase = bases.operand + uint64_t(uint32_t(half) * uint32_t(kOperandBytes >> 4));
    const uint32_t accumulators = bases.accumulators + half * kTmemColumnsPerHalf;
    // accumulators := bias (binary16 step: rows (1, 0, ...) times the bias column: exact)
    UmmaF16(accumulators, bases.ones, bases.bias, instr, 0, enabled);
#pragma unroll
    for (int step = 0; step < kK / 16; ++step)
    {
        if (kLayer < 3)
        {
            // 16 products of the 32-wide chunk step / 2: weight copy `step` has the other 16 columns zeroed
            const uint64_t descA = operandBase + uint64_t(((step / 2) * 2 * 2048) >> 4);
            const uint64_t descB = bases.weight + uint64_t((step * kN * 32) >> 4);
            if (kTmemOperand && kLayer > 0)
                UmmaE4m3F16FromTmem(accumulators, accumulators + kOperandColumn + uint32_t(step / 2) * 8u, descB, instr, 1, enabled);
            else
                UmmaE4m3F16(accumulators, descA, descB, instr, 1, enabled);
        }
        else
        {
            // binary16 operands: one K step = two core matrices of 8 halves
            const uint64_t descA = operandBase + uint64_t((step * 2 * 2048) >> 4);
            const uint64_t descB = bases.weight + uint64_t((step * 2 * kN * 16) >> 4);
            if (kTmemOperand)
                UmmaF16FromTmem(accumulators, accumulators + kOperandColumn + uint32_t(step) * 8u, descB, instr, 1, enabled);
            else
                UmmaF16(accumulators, descA, descB, instr, 1, enabled);
        }
    }
    // arrives once everything issued so far has completed: this chain's accumulators are ready
    if (enabled)
        UmmaCommit(bases.barrierBase + half * 8);
}

template <int kLayer>
__device__ __forceinline__ void IssueChainRefFp8(const RefTileContext& ctx, int half, uint32_t enabled)
{
    IssueChainRefFp8<kLayer>(MakeChainBases<kLayer>(ctx), half, enabled);
}

// The issuing warp's view of the context: values the compiler can see are the same in every lane.
__device__ __forceinline__ RefTileContext UniformContext(const RefTileContext& ctx)
{
    RefTileContext uniform = ctx;
    uniform.operandA = __shfl_sync(0xFFFFFFFFu, ctx.operandA, 0);
    uniform.biasRegion = __shfl_sync(0xFFFFFFFFu, ctx.biasRegion, 0);
    uniform.networkBase = __shfl_sync(0xFFFFFFFFu, ctx.networkBase, 0);
    uniform.tmemBase = __shfl_sync(0xFFFFFFFFu, ctx.tmemBase, 0);
    uniform.barrierBase = __shfl_sync(0xFFFFFFFFu, ctx.barrierBase, 0);
    return uniform;
}

// First half of a layer: hands the A operand written before this call to the tensor core.  Returns
// nonzero (uniformly over the CTA) when some thread gave up on a wait.
// (Tried and dropped: letting the two chains run apart between tiles - each chain with its own
// issuing thread waiting on an mbarrier its 128 threads arrive on - was 4 % slower than this
// CTA-wide barrier with one issuing thread.)
template <int kLayer, int kChainLocal = TileLayerBarrier<kLayer>()>
__device__ __forceinline__ int IssueLayerRefFp8(const RefTileContext& ctx, int failed)
{
    // Makes the A operand visible to the tensor core (async proxy), orders this thread's reads of the
    // previous layer's accumulators before they are overwritten, and agrees on giving up.
    // (The proxy fence is executed by every thread that wrote the operand, before the barrier: the
    // documented pattern.  A single fence in the issuing warp after the barrier passed every parity test
    // and was 2 % faster - the fence costs each thread about 200 cycles - but is not what the
    // programming guide shows, so it was not adopted.)
    if (kTmemOperand && kLayer > 0)
        TmemStoreWait(); // the operand went to tensor memory: nothing the async proxy reads was written
    else if (!(kAblate & 128))
        FenceProxyAsyncShared();
    TcgenFenceBeforeSync();
    if (kAblate & 1024)
        ;
    else if (kAblate & 256)
        __syncthreads();
    else if (LayerBarrier<kChainLocal>(ctx.tid, failed))
        return 1;
    // The whole issuing warp runs the descriptor arithmetic, on values the compiler can see are the same
    // in every lane (hence the shuffles), and one elected lane hands the work to the tensor core: issued
    // from a single thread inside a divergent branch the same code cost 85 instructions per texel more.
    // (Tried: building the descriptors before the barrier - 3 % slower.)
    const int warpIndex = ctx.tid >> 5;
    // (after a CTA-wide barrier one warp issues both chains: each chain's first warp issuing its own was 1 % slower)
    constexpr bool kOwnChainOnly = kChainLocal != 0;
    if ((kOwnChainOnly ? (warpIndex & 3) == 0 : warpIndex == kIssuingWarp) && !(kAblate & 16))
    {
        TcgenFenceAfterSync();
        const ChainBases bases = MakeChainBases<kLayer>(UniformContext(ctx));
        const uint32_t elected = ElectOne();
        if (kOwnChainOnly)
            IssueChainRefFp8<kLayer>(bases, __shfl_sync(0xFFFFFFFFu, warpIndex >> 2, 0), elected);
        else
        {
#pragma unroll
            for (int half = 0; half < kRefChains; ++half)
                IssueChainRefFp8<kLayer>(bases, half, elected);
        }
    }
    return 0;
}

// Clamped HGELU in binary16 and the e4m3 code of the result: two codes in the low 16 bits.
__device__ __forceinline__ uint32_t ActivateToE4m3(uint32_t bits)
{
    const __half2 x = AsHalf2(bits);
    const __half2 third = __float2half2_rn(1 / 3.f);
    const __half2 t = __hfma2_sat(third, x, __float2half2_rn(0.5f));
    const __half2 m = __hmin2(x, __float2half2_rn(3.f));
    const __half2 y = __hmul2_rn(m, t);
    return uint32_t(__nv_cvt_halfraw2_to_fp8x2(static_cast<__half2_raw>(y), __NV_SATFINITE, __NV_E4M3));
}

template <int kLayer, bool kConvert, typename Params>
__device__ __forceinline__ void ConsumeLayerRefFp8(const Params& params, const RefTileContext& ctx, uint32_t& phase, int& failed)
{
    constexpr int kN = kLayer == 0 ? 64 : kLayer == 1 ? 48 : kLayer == 2 ? 32 : 16;

    // (Every warp polls the barrier itself.  Tried and dropped: one polling warp per chain with the other
    // three blocked in a named barrier executes 1.5 % fewer instructions but wakes the chain later, 4.5 %
    // slower; an issuing thread per chain instead of one for both, 7 % slower; polls without a suspend-time
    // hint, the same speed.)
    if (!(kAblate & 16) && !MbarrierWaitBounded(ctx.barrier, phase))
    {
        failed = 1;
        ReportTimeout(params.status, uint32_t(ctx.tile), uint32_t(kLayer));
    }
    phase ^= 1;
    TcgenFenceAfterSync();

    if ((kAblate & 4) && kLayer < 3)
    {
        // profiling variant: the accumulator words go to the operand as they are
        uint4* rowChunk = ctx.rowChunk;
        uint32_t low[16];
        if (!(kAblate & 32))
        {
            TmemLoadPacked16(ctx.tmemLane, low);
            TmemLoadWait();
        }
        else
        {
#pragma unroll
            for (int i = 0; i < 16; ++i)
                low[i] = uint32_t(ctx.tile + i);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
        {
            if (kTmemOperand)
                TmemStore4(ctx.tmemLane + kOperandColumn + 4u * uint32_t(c), low[4 * c], low[4 * c + 1], low[4 * c + 2], low[4 * c + 3]);
            else
                rowChunk[c * 128] = make_uint4(low[4 * c], low[4 * c + 1], low[4 * c + 2], low[4 * c + 3]);
        }
        return;
    }

    if (kLayer < 2)
    {
        // e4m3 codes for the next layer: 16 per 16-byte chunk
        uint4* rowChunk = ctx.rowChunk;
        uint32_t low[16], high[16];
        if (!(kAblate & 32))
        {
            TmemLoadPacked16(ctx.tmemLane, low);
            if (kN == 64)
                TmemLoadPacked16(ctx.tmemLane + 32, high);
            else
            {
                uint32_t (&tail)[8] = reinterpret_cast<uint32_t (&)[8]>(high);
                TmemLoadPacked8(ctx.tmemLane + 32, tail);
            }
            TmemLoadWait();
        }
        else
        {
#pragma unroll
            for (int i = 0; i < 16; ++i)
                low[i] = high[i] = uint32_t(ctx.tile * 3 + i) & 0x3FFF3FFFu;
        }
        // chunk c of the next layer's operand row: to shared memory, or to tensor memory columns 48 + 4 c ..
        auto storeChunk = [&](int c, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
            if (kTmemOperand)
                TmemStore4(ctx.tmemLane + kOperandColumn + 4u * uint32_t(c), w0, w1, w2, w3);
            else
                rowChunk[c * 128] = make_uint4(w0, w1, w2, w3);
        };
#pragma unroll
        for (int c = 0; c < 2; ++c)
            storeChunk(c,
                PackCodes<true>(ActivateToE4m3(low[8 * c]), ActivateToE4m3(low[8 * c + 1])),
                PackCodes<true>(ActivateToE4m3(low[8 * c + 2]), ActivateToE4m3(low[8 * c + 3])),
                PackCodes<true>(ActivateToE4m3(low[8 * c + 4]), ActivateToE4m3(low[8 * c + 5])),
                PackCodes<true>(ActivateToE4m3(low[8 * c + 6]), ActivateToE4m3(low[8 * c + 7])));
#pragma unroll
        for (int c = 0; c < (kN - 32) / 16; ++c)
            storeChunk(2 + c,
                PackCodes<true>(ActivateToE4m3(high[8 * c]), ActivateToE4m3(high[8 * c + 1])),
                PackCodes<true>(ActivateToE4m3(high[8 * c + 2]), ActivateToE4m3(high[8 * c + 3])),
                PackCodes<true>(ActivateToE4m3(high[8 * c + 4]), ActivateToE4m3(high[8 * c + 5])),
                PackCodes<true>(ActivateToE4m3(high[8 * c + 6]), ActivateToE4m3(high[8 * c + 7])));
        if (kLayer == 1)
            storeChunk(3, 0, 0, 0, 0); // layer 2 has 48 inputs: the rest of its second chunk must be zeros
    }
    else if (kLayer == 2)
    {
        // layer 3 runs on the binary16 path: its inputs are the int8 grid values rint(y * 80) * 0.0125
        uint4* rowChunk = ctx.rowChunk;
        uint32_t acc[16];
        if (!(kAblate & 32))
        {
            TmemLoadPacked16(ctx.tmemLane, acc);
            TmemLoadWait();
        }
        else
        {
#pragma unroll
            for (int i = 0; i < 16; ++i)
                acc[i] = uint32_t(ctx.tile * 5 + i) & 0x3FFF3FFFu;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
        {
            const uint32_t w0 = ActivateRef<false>(acc[4 * c]), w1 = ActivateRef<false>(acc[4 * c + 1]);
            const uint32_t w2 = ActivateRef<false>(acc[4 * c + 2]), w3 = ActivateRef<false>(acc[4 * c + 3]);
            if (kTmemOperand)
                TmemStore4(ctx.tmemLane + kOperandColumn + 4u * uint32_t(c), w0, w1, w2, w3);
            else
                rowChunk[c * 128] = make_uint4(w0, w1, w2, w3);
        }
    }
    else
    {
        // output (src/Inference.cu:121-135): the accumulators are the channels
        uint32_t bits[8];
        if (!(kAblate & 32))
        {
            TmemLoadPacked8(ctx.tmemLane, bits);
            TmemLoadWait();
        }
        else
        {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                bits[i] = uint32_t(ctx.tile * 7 + i) & 0x3FFF3FFFu;
        }
        const int channelPairs = params.channels >> 1;
        ScrubSpecials(bits, channelPairs);
        if constexpr (kConvert)
        {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (j >= channelPairs)
                    bits[j] = 0;
            if (ctx.out)
                StoreConverted(params.conversion, params.firstChannel, params.numChannels, ctx, bits);
        }
        else if (ctx.out)
        {
            if (kAblate & 8)
            {
                // profiling variant: keep the values alive without storing them (the condition never holds)
                uint32_t all = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    all ^= bits[j];
                if (all == 0x12345679u && ctx.tile < 0)
                    ctx.out[0] = all;
            }
            else
                StoreTexel(ctx.out, ctx.outStepWords, ctx.storeBytes, bits, channelPairs);
        }
    }
}

template <int kLayer, bool kConvert, int kChainLocal = TileLayerBarrier<kLayer>(), typename Params>
__device__ __forceinline__ int RunLayerRefFp8(const Params& params, const RefTileContext& ctx, uint32_t& phase, int& failed)
{
    if (IssueLayerRefFp8<kLayer, kChainLocal>(ctx, failed))
        return 1;
    ConsumeLayerRefFp8<kLayer, kConvert>(params, ctx, phase, failed);
    return 0;
}

// Setup and teardown as for the binary16 kernel, on the FP8 kernel's shared-memory structure.
__device__ __forceinline__ int SetupCtaRefFp8(RefFp8SharedStorage& shared, const uint8_t* network, uint32_t* status, uint32_t loadWaitPolls, int tid, int warp)
{
    for (int i = tid; i < 256; i += kThreadsPerCta)
    {
        __half lo = __float2half_rn(__fmul_rn(float(i & 15), 1.f / 15.f));
        __half hi = __float2half_rn(__fmul_rn(float(i >> 4), 1.f / 15.f));
        shared.latentTable[i] = AsU32(__halves2half2(lo, hi));
    }
    for (int i = tid; i < 128 * 32 / 16; i += kThreadsPerCta)
        reinterpret_cast<uint4*>(shared.biasRegion)[i] = make_uint4(i < 128 ? 0x00003C00u : 0u, 0u, 0u, 0u);
    const uint32_t loadBarrier = SharedAddress(&shared.loadBarrier);
    if (tid == 0)
    {
        for (int chain = 0; chain < kRefChains; ++chain)
            MbarrierInit(SharedAddress(&shared.barrier[chain]), 1);
        MbarrierInit(loadBarrier, 1);
        FenceBarrierInit();
        MbarrierArriveExpectTx(loadBarrier, kRefNetworkBytes);
        BulkCopyToShared(SharedAddress(shared.network), network, kRefNetworkBytes, loadBarrier);
    }
    if (warp == 0)
        TmemAlloc(SharedAddress(&shared.tmemBase), kTmemColumns);
    FenceProxyAsyncShared();
    TcgenFenceBeforeSync();
    __syncthreads();
    TcgenFenceAfterSync();
    int failed = 0;
    if (!MbarrierWaitBounded(loadBarrier, 0, loadWaitPolls))
    {
        failed = 1;
        ReportTimeout(status, 0xFFFFFFFFu, 0xFFFFFFFFu); // no tile: the network image did not arrive
    }
    return failed;
}

__device__ __forceinline__ void TeardownCtaRefFp8(RefFp8SharedStorage& shared, const RefTileContext& ctx, uint32_t phase, int failed,
    int tid, int warp)
{
    TcgenFenceBeforeSync();
    const int aborted = __syncthreads_or(failed);
    if (aborted && tid == 0)
    {
        for (int chain = 0; chain < kRefChains; ++chain)
            (void)MbarrierWaitBounded(ctx.barrierBase + chain * 8, phase ^ 1);
        (void)MbarrierWaitBounded(SharedAddress(&shared.loadBarrier), 0);
    }
    __syncthreads();
    if (warp == 0)
        TmemFree(ctx.tmemBase, kTmemColumns);
}

template <bool kConvert, int kLayers>
__global__ void __launch_bounds__(kThreadsPerCta, kCtasPerSmRefFp8) DecodeKernelRefFp8(const __grid_constant__ KernelParams params)
{
    extern __shared__ __align__(128) unsigned char dynamicShared[];
    RefFp8SharedStorage& shared = *reinterpret_cast<RefFp8SharedStorage*>(dynamicShared);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;      // = the thread's row of the tile
    const int half = warp >> 2;     // the 128-row chain of this thread

    int failed = SetupCtaRefFp8(shared, params.network, params.status, params.loadWaitPolls, tid, warp);
    uint32_t phase = 0;
    int aborted = 0;

    RefTileContext ctx;
    ctx.tid = tid;
    ctx.tmemBase = shared.tmemBase;
    ctx.tmemLane = ctx.tmemBase + half * kTmemColumnsPerHalf + (uint32_t((warp & 3) * 32) << 16);
    ctx.barrierBase = SharedAddress(&shared.barrier[0]);
    ctx.barrier = ctx.barrierBase + half * 8;
    ctx.operandA = SharedAddress(shared.operandA);
    ctx.rowChunk = reinterpret_cast<uint4*>(shared.operandA + half * kOperandBytes) + (tid & 127);
    ctx.networkBase = SharedAddress(shared.network);
    ctx.biasRegion = SharedAddress(shared.biasRegion);

    struct TilePlace
    {
        int mipIndex, tileX0, tileY0;
    };
    auto locate = [&](int tile, int fromMip) {
        TilePlace place;
        place.mipIndex = fromMip;
        while (place.mipIndex + 1 < params.numMips && tile >= params.mips[place.mipIndex + 1].firstTile)
            ++place.mipIndex;
        const KernelMip& mip = params.mips[place.mipIndex];
        const int local = tile - mip.firstTile;
        const int tileY = mip.tilesX == 1 ? local : int(__umulhi(uint32_t(local), mip.tilesXMagic));
        place.tileX0 = (local - tileY * mip.tilesX) * kTileWidth;
        place.tileY0 = mip.rowBegin + tileY * kTileHeight;
        return place;
    };

    int tile = blockIdx.x;
    TilePlace place{0, 0, 0};
    int tablesMip = -1; // mip whose tap / encoding tables are in shared memory and valid for every inner tile of it
    if (tile < params.totalTiles)
    {
        place = locate(tile, 0);
        PrepareTile<true, true, kLayers>(params, params.mips[place.mipIndex], shared, place.tileX0, place.tileY0, lane, warp, false);
        tablesMip = TileKeepsTables(params.mips[place.mipIndex], place.tileX0, place.tileY0) ? place.mipIndex : -1;
        __syncthreads();
    }
    while (tile < params.totalTiles)
    {
        const KernelMip& mip = params.mips[place.mipIndex];
        ctx.tile = tile;
        ctx.x = place.tileX0 + lane;
        ctx.y = place.tileY0 + warp;
        // the e4m3 input stage is the one of the exact-accumulation kernel (64-byte rows of codes)
        if (kAblate & 2)
        {
            const uint32_t filler = uint32_t(tile) & 0x3F3F3F3Fu;
#pragma unroll
            for (int chunk = 0; chunk < 4; ++chunk)
                ctx.rowChunk[chunk * 128] = make_uint4(filler, filler + chunk, filler, filler);
        }
        else
            BuildInputs<true, true, kLayers>(params, mip, shared, ctx, lane, warp);

        aborted = IssueLayerRefFp8<0>(ctx, failed);
        if (aborted)
            break;
        const int nextTile = tile + int(gridDim.x);
        if (nextTile < params.totalTiles)
        {
            if (!(kAblate & 512))
                place = locate(nextTile, place.mipIndex);
            // the tables of the previous tile serve this one too when both lie inside the same mip with invariant tables
            const bool keepsTables = (kAblate & 512) ? true : TileKeepsTables(params.mips[place.mipIndex], place.tileX0, place.tileY0);
            if (!(kAblate & 1))
                PrepareTile<true, true, kLayers>(params, params.mips[place.mipIndex], shared, place.tileX0, place.tileY0, lane, warp,
                    keepsTables && place.mipIndex == tablesMip && !(kAblate & 64));
            tablesMip = keepsTables ? place.mipIndex : -1;
        }
        ConsumeLayerRefFp8<0, false>(params, ctx, phase, failed);

        aborted = RunLayerRefFp8<1, false>(params, ctx, phase, failed);
        if (!aborted) aborted = RunLayerRefFp8<2, false>(params, ctx, phase, failed);
        if (aborted)
            break;
        {
            // where the texel goes (worked out only now: nothing of it has to stay in registers through the layers)
            const bool planar = params.outputLayout == kLayoutPlanarPairs;
            const uint32_t first = planar ? uint32_t(ctx.y) * uint32_t(mip.width) * uint32_t(params.channels) + 2u * uint32_t(ctx.x)
                                          : (uint32_t(ctx.y) * uint32_t(mip.width) + uint32_t(ctx.x)) * uint32_t(params.channels);
            const bool inside = ctx.x < mip.width && ctx.y < mip.rowEnd;
            if constexpr (kConvert)
            {
                const uint32_t pixelIndex = uint32_t(ctx.y) * uint32_t(mip.width) + uint32_t(ctx.x);
                const size_t component = size_t(mip.outOffset) + size_t(pixelIndex) * size_t(params.conversion.dstChannels);
                unsigned char* bytes = reinterpret_cast<unsigned char*>(params.out) + component * BytesPerComponent(params.conversion.format);
                ctx.out = inside ? reinterpret_cast<uint32_t*>(bytes) : nullptr;
                ctx.outStepWords = pixelIndex;
            }
            else
            {
                ctx.out = inside ? reinterpret_cast<uint32_t*>(params.out + mip.outOffset + first) : nullptr;
                ctx.outStepWords = planar ? uint32_t(mip.width) : 1u;
                ctx.storeBytes = mip.storeBytes;
            }
        }
        aborted = RunLayerRefFp8<3, kConvert>(params, ctx, phase, failed);
        if (aborted)
            break;
        tile = nextTile;
    }
    TeardownCtaRefFp8(shared, ctx, phase, failed, tid, warp);
}

// Inference on sample for FP8 networks (8-bit operands): one thread per query, taps read straight
// from global memory.
__global__ void __launch_bounds__(kThreadsPerCta, kCtasPerSmRefFp8) SampleKernelRefFp8(const __grid_constant__ SampleParams params)
{
    extern __shared__ __align__(128) unsigned char dynamicShared[];
    RefFp8SharedStorage& shared = *reinterpret_cast<RefFp8SharedStorage*>(dynamicShared);
    __shared__ KernelMip mipTable[16];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int half = warp >> 2;

    if (tid < params.numMips)
        mipTable[tid] = params.mips[tid];
    int failed = SetupCtaRefFp8(shared, params.network, params.status, params.loadWaitPolls, tid, warp);
    int aborted = 0;
    uint32_t phase = 0;

    RefTileContext ctx;
    ctx.tid = tid;
    ctx.tmemBase = shared.tmemBase;
    ctx.tmemLane = ctx.tmemBase + half * kTmemColumnsPerHalf + (uint32_t((warp & 3) * 32) << 16);
    ctx.barrierBase = SharedAddress(&shared.barrier[0]);
    ctx.barrier = ctx.barrierBase + half * 8;
    ctx.operandA = SharedAddress(shared.operandA);
    ctx.rowChunk = reinterpret_cast<uint4*>(shared.operandA + half * kOperandBytes) + (tid & 127);
    ctx.networkBase = SharedAddress(shared.network);
    ctx.biasRegion = SharedAddress(shared.biasRegion);
    ctx.outStepWords = 1;
    ctx.storeBytes = 4;

    const unsigned long long tiles = (params.numQueries + kThreadsPerCta - 1) / kThreadsPerCta;
    // a tile's queries are requested one tile ahead: their latency passes under the previous tile's layers
    float nextU = 0.f, nextV = 0.f, nextLod = 0.f;
    auto requestQuery = [&](unsigned long long ofTile) {
        if (ofTile < tiles)
        {
            const unsigned long long q = min(ofTile * kThreadsPerCta + tid, params.numQueries - 1);
            nextU = __ldg(params.queries + 3 * q);
            nextV = __ldg(params.queries + 3 * q + 1);
            nextLod = __ldg(params.queries + 3 * q + 2);
        }
    };
    requestQuery(blockIdx.x);
    for (unsigned long long tile = blockIdx.x; tile < tiles; tile += gridDim.x)
    {
        const unsigned long long query = tile * kThreadsPerCta + tid;
        const bool valid = query < params.numQueries;
        const float u = nextU, v = nextV, lod = nextLod;
        requestQuery(tile + gridDim.x);
        const int mipIndex = max(0, min(params.numMips - 1, int(floorf(lod))));
        const KernelMip& mip = mipTable[mipIndex];
        const int x = max(0, min(mip.width - 1, int(floorf(__fmul_rn(u, float(mip.width))))));
        const int y = max(0, min(mip.height - 1, int(floorf(__fmul_rn(v, float(mip.height))))));
        ctx.tile = int(tile);
        ctx.x = x;
        ctx.y = y;
        ctx.out = valid ? reinterpret_cast<uint32_t*>(params.out + query * params.channels) : nullptr;

        {
            uint32_t words[16];
            const uint32_t zeroWord = PackCodes<true>(QuantizeInputPair<true>(__float2half2_rn(0.f)),
                                                      QuantizeInputPair<true>(__float2half2_rn(0.f)));
#pragma unroll
            for (int i = 0; i < 8; ++i)
                words[i] = zeroWord; // unused feature slots hold quantised zeros (src/Inference.cu:49)
#pragma unroll
            for (int i = 12; i < 16; ++i)
                words[i] = 0;        // K padding
            SampleGridsDirect<true, true>(params.latents, params.numLayers, mip, x, y, shared.latentTable, words, params.interleaved != 0);
            // src/RegressionKernels.h:59-85
            float xf = __fmul_rn(float(x), mip.positionScale);
            float yf = __fmul_rn(float(y), mip.positionScale);
#pragma unroll
            for (int wave = 0; wave < 3; ++wave)
            {
                const float ex = __fmaf_rn(Frac(xf), 2.f, -1.f), ey = __fmaf_rn(Frac(yf), 2.f, -1.f);
                const float ez = __fmaf_rn(Frac(__fadd_rn(xf, 0.25f)), 2.f, -1.f);
                const float ew = __fmaf_rn(Frac(__fadd_rn(yf, 0.25f)), 2.f, -1.f);
                words[8 + wave] = PackCodes<true>(QuantizeInputPair<true>(__floats2half2_rn(ex, ey)),
                                                  QuantizeInputPair<true>(__floats2half2_rn(ez, ew)));
                xf = __fmul_rn(xf, 2.f);
                yf = __fmul_rn(yf, 2.f);
            }
            words[11] = PackCodes<true>(QuantizeInputPair<true>(__float2half2_rn(mip.positionLod)),
                                        QuantizeInputPair<true>(__float2half2_rn(0.f)));
#pragma unroll
            for (int chunk = 0; chunk < 4; ++chunk)
                ctx.rowChunk[chunk * 128] = make_uint4(words[4 * chunk], words[4 * chunk + 1], words[4 * chunk + 2], words[4 * chunk + 3]);
        }

        // nothing is shared between the chains of a query tile: each runs at its own pace
        aborted = RunLayerRefFp8<0, false, 2>(params, ctx, phase, failed);
        if (!aborted) aborted = RunLayerRefFp8<1, false, 2>(params, ctx, phase, failed);
        if (!aborted) aborted = RunLayerRefFp8<2, false, 2>(params, ctx, phase, failed);
        if (!aborted) aborted = RunLayerRefFp8<3, false, 2>(params, ctx, phase, failed);
        if (aborted)
            break;
    }
    TeardownCtaRefFp8(shared, ctx, phase, failed, tid, warp);
}

} // namespace

// One kernel, set up for its dynamic shared memory on first use per device (`done`: one bit per device).
template <typename Kernel>
cudaError_t LaunchRefKernel(Kernel kernel, std::atomic<unsigned long long>& done, size_t sharedBytes, int threads,
    const KernelParams& params, int ctas, cudaStream_t stream)
{
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess)
        return err;
    const unsigned long long bit = 1ull << (device & 63);
    if (!(done.load(std::memory_order_acquire) & bit))
    {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sharedBytes));
        if (err != cudaSuccess)
            return err;
        done.fetch_or(bit, std::memory_order_release);
    }
    kernel<<<ctas, threads, sharedBytes, stream>>>(params);
    return cudaGetLastError();
}

cudaError_t LaunchDecodeRef(const KernelParams& params, bool fp8, int ctas, cudaStream_t stream)
{
    // kernels compiled for 2, 3 or 4 latent layers and one for any number, each with and without the
    // converting epilogue
    static std::atomic<unsigned long long> done[2][2][5];
    const int layers = params.numLayers < 2 || params.numLayers > 4 ? 0 : params.numLayers;
    const int convert = params.convert ? 1 : 0;
    if (fp8)
    {
        // FP8 networks take the kernel with 8-bit operands (same bits, four CTAs per SM)
        const size_t bytes = sizeof(RefFp8SharedStorage);
        std::atomic<unsigned long long>& flag = done[1][convert][layers];
        if (convert)
            switch (layers)
            {
            case 2: return LaunchRefKernel(DecodeKernelRefFp8<true, 2>, flag, bytes, kThreadsPerCta, params, ctas, stream);
            case 3: return LaunchRefKernel(DecodeKernelRefFp8<true, 3>, flag, bytes, kThreadsPerCta, params, ctas, stream);
            case 4: return LaunchRefKernel(DecodeKernelRefFp8<true, 4>, flag, bytes, kThreadsPerCta, params, ctas, stream);
            default: return LaunchRefKernel(DecodeKernelRefFp8<true, 0>, flag, bytes, kThreadsPerCta, params, ctas, stream);
            }
        switch (layers)
        {
        case 2: return LaunchRefKernel(DecodeKernelRefFp8<false, 2>, flag, bytes, kThreadsPerCta, params, ctas, stream);
        case 3: return LaunchRefKernel(DecodeKernelRefFp8<false, 3>, flag, bytes, kThreadsPerCta, params, ctas, stream);
        case 4: return LaunchRefKernel(DecodeKernelRefFp8<false, 4>, flag, bytes, kThreadsPerCta, params, ctas, stream);
        default: return LaunchRefKernel(DecodeKernelRefFp8<false, 0>, flag, bytes, kThreadsPerCta, params, ctas, stream);
        }
    }
    const size_t bytes = sizeof(RefSharedStorage);
    std::atomic<unsigned long long>& flag = done[0][convert][layers];
    if (convert)
        switch (layers)
        {
        case 2: return LaunchRefKernel(DecodeKernelRef<false, true, 2>, flag, bytes, kRefThreadsPerCta, params, ctas, stream);
        case 3: return LaunchRefKernel(DecodeKernelRef<false, true, 3>, flag, bytes, kRefThreadsPerCta, params, ctas, stream);
        case 4: return LaunchRefKernel(DecodeKernelRef<false, true, 4>, flag, bytes, kRefThreadsPerCta, params, ctas, stream);
        default: return LaunchRefKernel(DecodeKernelRef<false, true, 0>, flag, bytes, kRefThreadsPerCta, params, ctas, stream);
        }
    switch (layers)
    {
    case 2: return LaunchRefKernel(DecodeKernelRef<false, false, 2>, flag, bytes, kRefThreadsPerCta, params, ctas, stream);
    case 3: return LaunchRefKernel(DecodeKernelRef<false, false, 3>, flag, bytes, kRefThreadsPerCta, params, ctas, stream);
    case 4: return LaunchRefKernel(DecodeKernelRef<false, false, 4>, flag, bytes, kRefThreadsPerCta, params, ctas, stream);
    default: return LaunchRefKernel(DecodeKernelRef<false, false, 0>, flag, bytes, kRefThreadsPerCta, params, ctas, stream);
    }
}

cudaError_t LaunchSampleRef(const SampleParams& params, bool fp8, int ctas, cudaStream_t stream)
{
    static std::atomic<unsigned long long> done[2];
    auto launch = [&](auto kernel, std::atomic<unsigned long long>& doneMask) -> cudaError_t {
        int device = 0;
        cudaError_t err = cudaGetDevice(&device);
        if (err != cudaSuccess)
            return err;
        const unsigned long long bit = 1ull << (device & 63);
        if (!(doneMask.load(std::memory_order_acquire) & bit))
        {
            err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(offsetof(RefSharedStorage, tables)));
            if (err != cudaSuccess)
                return err;
            doneMask.fetch_or(bit, std::memory_order_release);
        }
        kernel<<<ctas, kRefThreadsPerCta, offsetof(RefSharedStorage, tables), stream>>>(params);
        return cudaGetLastError();
    };
    if (fp8)
    {
        int device = 0;
        cudaError_t err = cudaGetDevice(&device);
        if (err != cudaSuccess)
            return err;
        const unsigned long long bit = 1ull << (device & 63);
        if (!(done[1].load(std::memory_order_acquire) & bit))
        {
            err = cudaFuncSetAttribute(SampleKernelRefFp8, cudaFuncAttributeMaxDynamicSharedMemorySize, int(offsetof(RefFp8SharedStorage, tables)));
            if (err != cudaSuccess)
                return err;
            done[1].fetch_or(bit, std::memory_order_release);
        }
        SampleKernelRefFp8<<<ctas, kThreadsPerCta, offsetof(RefFp8SharedStorage, tables), stream>>>(params);
        return cudaGetLastError();
    }
    return launch(SampleKernelRef<false>, done[0]);
}

} // namespace ntcb
