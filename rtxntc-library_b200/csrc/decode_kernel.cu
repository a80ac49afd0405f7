// NTC decode kernel for sm_100a: one launch decodes every listed colour mip of a texture set.
//
// Work decomposition.  A tile is 32x8 texels; one CTA of 256 threads owns one tile at a time
// (thread = texel) and walks the tile list of the whole mip chain with a grid stride.  The tile is
// two 128-row GEMM chains (rows 0-3 and rows 4-7 of the tile; a thread's texel is one row of its
// half's 128x{64,48,32,16} chain and one TMEM lane), issued together.  Several CTAs are resident
// per SM, so the SIMT phases of one tile overlap the tensor-core phases of the others.
//
// Per tile:
//   1. every thread samples the two latent grids for its texel (packed BGRA4 pixels, nibble ->
//      binary16 through a 256-entry shared-memory table, bilinear blend in binary16), appends the
//      positional encoding and quantises the 48 inputs to int8 codes or e4m3, and writes its 64-byte
//      row of the A operand straight into the tensor core's K-major core-matrix order (a 16-byte
//      chunk per store, consecutive threads hit consecutive chunks: conflict-free);
//   2. one thread issues tcgen05.mma (kind::i8 or kind::f8f6f4, M=128, N=64/48/32/16, K=32 per
//      instruction) against the weights resident in shared memory; accumulators live in TMEM;
//   3. after the commit arrives on the mbarrier every thread pulls its row of accumulators with
//      tcgen05.ld, applies bias/scale and the clamped HGELU in packed binary16, re-quantises and
//      writes the next layer's A operand over the previous one - with FP8 weights into tensor memory
//      (tcgen05.st; the next product takes A from there), with Int8 weights into shared memory;
//   4. after the fourth layer the epilogue scales, converts to fp16 and stores.
//
// Arithmetic contract (what the CPU checker restates): everything outside the matrix products is
// done operation by operation as the reference CUDA kernel does it (src/FeatureGridDevice.h:33-98,
// src/RegressionKernels.h:59-85, src/tin/tin_mlp.h:22-37, src/tin/tin_activation.h:88-104); the
// matrix products accumulate exactly (int32, or fp32 for e4m3 operands) instead of in binary16.
//
// Every wait on the mbarrier is bounded; on expiry the CTA records an error in the status words,
// skips the remaining tiles, releases its TMEM columns and exits.

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

namespace ntcb
{
namespace
{

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------

// D[tmem] (+)= A[smem] * B[smem]^T, M = 128, K = 32 bytes of 8-bit operands.
template <bool kFp8>
__device__ __forceinline__ void Umma(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t instr, uint32_t accumulate)
{
    if (kFp8)
    {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
            "}" ::"r"(tmemD),
            "l"(descA), "l"(descB), "r"(instr), "r"(accumulate)
            : "memory");
    }
    else
    {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
            "}" ::"r"(tmemD),
            "l"(descA), "l"(descB), "r"(instr), "r"(accumulate)
            : "memory");
    }
}

// The same with the A operand in tensor memory: 8 columns (32 bytes per lane) starting at `tmemA`.
template <bool kFp8>
__device__ __forceinline__ void UmmaFromTmem(uint32_t tmemD, uint32_t tmemA, uint64_t descB, uint32_t instr, uint32_t accumulate)
{
    if (kFp8)
    {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t"
            "}" ::"r"(tmemD),
            "r"(tmemA), "l"(descB), "r"(instr), "r"(accumulate)
            : "memory");
    }
    else
    {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t"
            "}" ::"r"(tmemD),
            "r"(tmemA), "l"(descB), "r"(instr), "r"(accumulate)
            : "memory");
    }
}

// FP8 networks keep the A operands of layers 1-3 in tensor memory: the activation codes of a row (at most
// 64 bytes) go to columns [0,16) of the row's lane, and the accumulators of those layers start at column
// 16 (48 + 16 = 64 columns per chain).  Layer 0 reads its operand from shared memory and accumulates into
// columns [0,64); its consumer has loaded columns [0,32) before it stores the first codes to [0,8), and
// [32,64) before it stores to [8,16).  Int8 networks have the bias K step's operand in shared memory
// and 65 - 80 operand bytes per row: they keep every operand there.
template <bool kFp8, int kLayer>
constexpr bool kOperandInTmem = kFp8 && kLayer >= 1;
template <bool kFp8, int kLayer>
constexpr uint32_t kAccumulatorColumn = kOperandInTmem<kFp8, kLayer> ? 16u : 0u;

// Instruction descriptor: dense, K-major A and B, M = 128.
__host__ __device__ constexpr uint32_t MakeInstrDescriptor(bool fp8, int n)
{
    // bits 4-5: accumulator format (1 = f32, 2 = s32); bits 7-9 / 10-12: A / B format
    // (f8f6f4: 0 = e4m3; i8: 1 = signed); bits 17-22: N >> 3; bits 24-28: M >> 4.
    return (fp8 ? (1u << 4) : (2u << 4)) | (fp8 ? 0u : (1u << 7) | (1u << 10)) | (uint32_t(n >> 3) << 17) |
           (uint32_t(128 >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// Small arithmetic helpers
// ---------------------------------------------------------------------------------------------

// Clamped HGELU in binary16 (src/tin/tin_activation.h:88-92) followed by re-quantisation:
// e4m3 when `toFp8`, otherwise the int8 code rint(y * 80) - 113 (src/tin/tin_activation.h:94-99,
// the -113 offset is folded into the next layer's stored bias, src/Quantizer.cu:176-181).
// y * 80 lies in [-15, 240], so 113 is the only offset that fits int8; being odd, it cannot be
// merged into the even magic addend without changing how ties round.
template <bool kToFp8>
__device__ __forceinline__ uint32_t ActivatePair(__half2 x)
{
    const __half2 third = __float2half2_rn(1 / 3.f);
    __half2 t = __hfma2_sat(third, x, __float2half2_rn(0.5f));
    __half2 m = __hmin2(x, __float2half2_rn(3.f));
    __half2 y = __hmul2_rn(m, t);
    if (kToFp8)
    {
        return uint32_t(__nv_cvt_halfraw2_to_fp8x2(static_cast<__half2_raw>(y), __NV_SATFINITE, __NV_E4M3));
    }
    else
    {
        __half2 p = __hmul2_rn(y, __float2half2_rn(80.f));
        __half2 r = __hadd2_rn(p, __float2half2_rn(1536.f)); // rint(p): ulp is 1 in [1024, 2048)
        r = __hadd2_rn(r, __float2half2_rn(-113.f));         // exact
        return AsU32(r);
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------

struct __align__(128) SharedStorage
{
    uint8_t network[kStagedNetworkBytes]; // weights in core-matrix order, scales, biases
    // the tensor core reads operands as 128-byte core matrices: keep them on 128-byte lines
    alignas(128) uint8_t operandA[2 * kOperandBytes];  // A operands of the current layer (top half, bottom half), core-matrix order
    alignas(128) uint8_t biasRegion[kBiasRegionBytes]; // constant A operand of the bias K step of the int8 layers
    uint32_t latentTable[256];            // byte (two nibbles) -> two binary16 latent values
    uint64_t barrier;                     // MMA completion
    uint64_t loadBarrier;                 // arrival of the network image (bulk copy)
    uint32_t tmemBase;
    // What inference on sample does not use comes last: its launches ask for the bytes before `tables` only.
    // (With the whole structure, a sample kernel's own static shared memory - its table of mips - puts four CTAs
    // above an SM's 228 KB: three were resident and the fourth quarter of the grid ran alone afterwards.)
    alignas(128) TileTables tables;
    uint8_t footprintHi[kFootprintHiBytes]; // unpacked latents of the tile's footprint in the high-res grid
    uint8_t footprintLo[kFootprintLoBytes]; // ... and in the low-res grid
};


struct TileContext
{
    int tid;
    uint32_t tmemBase; // TMEM address of the CTA's accumulators: columns [0,64) top half, [64,128) bottom half
    uint32_t tmemLane; // ... of this thread's half at this thread's lane
    uint32_t barrier;  // shared address of the MMA-completion mbarrier
    uint32_t operandA; // shared address of the A operands (top half, then bottom half)
    uint4* rowChunk;   // this thread's 16-byte slot in chunk 0 of its half's A operand
    uint32_t networkBase;
    uint32_t biasRegion; // shared address of the constant A operand of the bias K step
    int tile, x, y;
    uint32_t* out;          // where this thread's first channel pair goes (nullptr: store nothing); with a
                            // converting epilogue: the address of the thread's pixel in the client's format
    uint32_t outStepWords;  // 32-bit words between consecutive channel pairs; with a converting epilogue:
                            // the pixel's linear index in its mip (the dither seed)
};

// First half of a layer of the MLP for the CTA's current tile: barrier and MMA issue (both halves
// of the tile).  Returns nonzero (uniformly over the CTA) when some thread gave up on a wait.
// (The default kernels' issue path - descriptors built warp-uniformly, an elected lane, one completion
// barrier per chain, chain-local barriers between layers - was tried here too: no gain with FP8 weights,
// 3.5 % slower with Int8 weights, where it spills under the 64-register cap.)
template <bool kFp8, int kLayer>
__device__ __forceinline__ int IssueLayer(const TileContext& ctx, int failed)
{
    constexpr int kN = kLayer == 0 ? 64 : kLayer == 1 ? 48 : kLayer == 2 ? 32 : 16;
    constexpr int kK = kLayer == 3 ? 32 : 64;
    constexpr int kWeightOffset =
        kLayer == 0 ? kWeightOffset0 : kLayer == 1 ? kWeightOffset1 : kLayer == 2 ? kWeightOffset2 : kWeightOffset3;
    constexpr bool kLayerFp8 = kFp8 && kLayer < 3;
    constexpr bool kBiasStep = !kFp8 && kLayer != 0; // Int8 mode: one more K step, the bias slots

    // Makes the A operand written before this call visible to the tensor core, orders every
    // thread's TMEM reads of the previous layer before the accumulators are overwritten, and agrees
    // on whether any thread gave up waiting.
    if (kOperandInTmem<kFp8, kLayer>)
        TmemStoreWait();
    else
        FenceProxyAsyncShared();
    TcgenFenceBeforeSync();
    if (__syncthreads_or(failed))
        return 1;

    if (ctx.tid == 0)
    {
        TcgenFenceAfterSync();
        constexpr uint32_t instr = MakeInstrDescriptor(kLayerFp8, kN);
#pragma unroll
        for (int half = 0; half < 2; ++half)
        {
#pragma unroll
            for (int kStep = 0; kStep < kK / 32; ++kStep)
            {
                // one K step = two 16-byte core matrices; A: 2048 bytes apart, B: kN*16 bytes apart
                uint64_t descA = MakeSmemDescriptor(ctx.operandA + half * kOperandBytes + kStep * 2 * 2048, 2048, 128);
                uint64_t descB = MakeSmemDescriptor(ctx.networkBase + kWeightOffset + kStep * 2 * kN * 16, kN * 16, 128);
                if (kOperandInTmem<kFp8, kLayer>)
                    UmmaFromTmem<kLayerFp8>(ctx.tmemBase + half * kTmemColumnsPerHalf + kAccumulatorColumn<kFp8, kLayer>,
                        ctx.tmemBase + half * kTmemColumnsPerHalf + kStep * 8, descB, instr, kStep != 0);
                else
                    Umma<kLayerFp8>(ctx.tmemBase + half * kTmemColumnsPerHalf, descA, descB, instr, kStep != 0);
            }
            if (kBiasStep)
            {
                uint64_t descA = MakeSmemDescriptor(ctx.biasRegion, 2048, 128);
                uint64_t descB = MakeSmemDescriptor(ctx.networkBase + kWeightOffset + (kK / 32) * 2 * kN * 16, kN * 16, 128);
                Umma<kLayerFp8>(ctx.tmemBase + half * kTmemColumnsPerHalf, descA, descB, instr, 1);
            }
        }
        UmmaCommit(ctx.barrier);
    }
    return 0;
}

// Second half of a layer: waits for the MMA, then applies the activation and writes the next
// layer's A operand (layers 0-2) or runs the output epilogue (layer 3).
template <bool kFp8, int kLayer, bool kConvert, bool kBiasTable, typename Params>
__device__ __forceinline__ void ConsumeLayerImpl(const Params& params, const SharedStorage& shared,
    const TileContext& ctx, uint32_t& phase, int& failed)
{
    uint32_t* const status = params.status;
    const int channels = params.channels;
    constexpr int kN = kLayer == 0 ? 64 : kLayer == 1 ? 48 : kLayer == 2 ? 32 : 16;
    constexpr bool kLayerFp8 = kFp8 && kLayer < 3;

    if (!MbarrierWaitBounded(ctx.barrier, phase))
    {
        failed = 1;
        ReportTimeout(status, uint32_t(ctx.tile), uint32_t(kLayer));
    }
    phase ^= 1;
    TcgenFenceAfterSync();

    const float* scale = reinterpret_cast<const float*>(shared.network + kScaleOffset) + kLayer * 64;
    const int32_t* biasI = reinterpret_cast<const int32_t*>(shared.network + kBiasOffset) + kLayer * 64;
    const __half2* biasH = reinterpret_cast<const __half2*>(shared.network + kBiasOffset + kLayer * 256);

    if (kLayer < 3)
    {
        constexpr bool kNextFp8 = kFp8 && kLayer < 2; // layer 2 always re-quantises to int8
        uint4* rowChunk = ctx.rowChunk;
        // 32 accumulator columns at a time keeps the register footprint small
#pragma unroll
        for (int part = 0; part < (kN + 31) / 32; ++part)
        {
            constexpr int kChunksTotal = kN / 16;
            const int firstChunk = part * 2;
            uint32_t acc[2][16];
#pragma unroll
            for (int c = 0; c < 2; ++c)
                if (firstChunk + c < kChunksTotal)
                    TmemLoad16(ctx.tmemLane + kAccumulatorColumn<kFp8, kLayer> + (firstChunk + c) * 16, acc[c]);
            TmemLoadWait();
#pragma unroll
            for (int c = 0; c < 2; ++c)
            {
                if (firstChunk + c < kChunksTotal)
                {
                    uint32_t pairs[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                    {
                        const int colIndex = (firstChunk + c) * 16 + 2 * j;
                        __half2 xh;
                        if (kLayerFp8)
                        {
                            xh = __floats2half2_rn(__uint_as_float(acc[c][2 * j]), __uint_as_float(acc[c][2 * j + 1]));
                            xh = __hadd2_rn(xh, biasH[colIndex >> 1]);
                        }
                        else
                        {
                            // include/libntc/shaders/Inference.hlsli:146-165: float(acc + bias) * scale
                            float f0 = __fmul_rn(float(int32_t(acc[c][2 * j]) + (kBiasTable ? biasI[colIndex] : 0)), scale[colIndex]);
                            float f1 = __fmul_rn(float(int32_t(acc[c][2 * j + 1]) + (kBiasTable ? biasI[colIndex + 1] : 0)), scale[colIndex + 1]);
                            xh = __floats2half2_rn(f0, f1);
                        }
                        pairs[j] = ActivatePair<kNextFp8>(xh);
                    }
                    const uint4 codes =
                        make_uint4(PackCodes<kNextFp8>(pairs[0], pairs[1]), PackCodes<kNextFp8>(pairs[2], pairs[3]),
                                   PackCodes<kNextFp8>(pairs[4], pairs[5]), PackCodes<kNextFp8>(pairs[6], pairs[7]));
                    if (kFp8)
                        TmemStore4(ctx.tmemLane + (firstChunk + c) * 4, codes.x, codes.y, codes.z, codes.w);
                    else
                        rowChunk[(firstChunk + c) * 128] = codes;
                }
            }
        }
        if (kLayer == 1)
        {
            // layer 2 has 48 inputs, K is padded to 64: zeros (e4m3) or the bias slots' inputs (int8)
            const uint32_t fill = kFp8 ? 0u : kBiasSlotValue * 0x01010101u;
            if (kFp8)
                TmemStore4(ctx.tmemLane + 12, 0u, 0u, 0u, 0u);
            else
                rowChunk[3 * 128] = make_uint4(fill, fill, fill, (fill & 0x00FFFFFFu) | 0x01000000u);
        }
    }
    else
    {
        // output epilogue (src/Inference.cu:121-135)
        uint32_t acc[16];
        TmemLoad16(ctx.tmemLane + kAccumulatorColumn<kFp8, kLayer>, acc);
        TmemLoadWait();
        const int channelPairs = channels >> 1;
        uint32_t bits[8];
        uint32_t special = 0; // bit 15 / 31 set when a value has an all-ones exponent
#pragma unroll
        for (int j = 0; j < 8; ++j)
        {
            if (j < channelPairs)
            {
                float f0 = __fmul_rn(float(int32_t(acc[2 * j]) + (kBiasTable ? biasI[2 * j] : 0)), scale[2 * j]);
                float f1 = __fmul_rn(float(int32_t(acc[2 * j + 1]) + (kBiasTable ? biasI[2 * j + 1] : 0)), scale[2 * j + 1]);
                bits[j] = AsU32(__floats2half2_rn(f0, f1));
                special |= (bits[j] & 0x7C007C00u) + 0x04000400u;
            }
        }
        if (special & 0x80008000u)
        {
            // Inf / NaN -> 0 (src/CudaUtils.h:30-35); rare, so kept off the common path
#pragma unroll
            for (int j = 0; j < 8; ++j)
            {
                if (j < channelPairs)
                {
                    if ((bits[j] & 0x7C00u) == 0x7C00u) bits[j] &= 0xFFFF0000u;
                    if ((bits[j] & 0x7C000000u) == 0x7C000000u) bits[j] &= 0x0000FFFFu;
                }
            }
        }
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
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (j < channelPairs)
                    ctx.out[j * ctx.outStepWords] = bits[j];
        }
    }
}

// Second half of a layer.  An int8 layer's bias is part of the accumulator already (bias slots of
// the matrix product) unless the staged network says that it has to come from the table.
template <bool kFp8, int kLayer, bool kConvert, typename Params>
__device__ __forceinline__ void ConsumeLayer(const Params& params, const SharedStorage& shared,
    const TileContext& ctx, uint32_t& phase, int& failed)
{
    // (FP8 mode has a single int8 layer of 16 outputs: it keeps the table)
    if (kFp8 || (*reinterpret_cast<const uint32_t*>(shared.network + kFlagsOffset) & kFlagBiasTable))
        ConsumeLayerImpl<kFp8, kLayer, kConvert, true>(params, shared, ctx, phase, failed);
    else
        ConsumeLayerImpl<kFp8, kLayer, kConvert, false>(params, shared, ctx, phase, failed);
}

template <bool kFp8, int kLayer, bool kConvert, typename Params>
__device__ __forceinline__ int RunLayer(const Params& params, const SharedStorage& shared,
    const TileContext& ctx, uint32_t& phase, int& failed)
{
    if (IssueLayer<kFp8, kLayer>(ctx, failed))
        return 1;
    ConsumeLayer<kFp8, kLayer, kConvert>(params, shared, ctx, phase, failed);
    return 0;
}

// One-time setup of a CTA: the network image arrives by one TMA bulk copy while the threads fill
// the constant tables, set up the barriers and allocate tensor memory.  Returns nonzero, uniformly
// over the CTA, when some thread gave up waiting for the image (status words written, one more
// bounded wait for the copy done, tensor memory released): the caller returns at once.
__device__ __forceinline__ int SetupCta(SharedStorage& shared, const uint8_t* network, uint32_t* status, uint32_t loadWaitPolls, int tid, int warp)
{
    // src/Quantizer.cu:490-495: value = float(nibble) * (1.f / 15.f), stored as binary16
    for (int i = tid; i < 256; i += kThreadsPerCta)
    {
        __half lo = __float2half_rn(__fmul_rn(float(i & 15), 1.f / 15.f));
        __half hi = __float2half_rn(__fmul_rn(float(i >> 4), 1.f / 15.f));
        shared.latentTable[i] = AsU32(__halves2half2(lo, hi));
    }
    // constant inputs of the bias K step: 31 slots of kBiasSlotValue and a last slot of 1 per row
    for (int i = tid; i < kBiasRegionBytes / 16; i += kThreadsPerCta)
    {
        const uint32_t fill = kBiasSlotValue * 0x01010101u;
        reinterpret_cast<uint4*>(shared.biasRegion)[i] =
            make_uint4(fill, fill, fill, i < 128 ? fill : ((fill & 0x00FFFFFFu) | 0x01000000u));
    }
    const uint32_t loadBarrier = SharedAddress(&shared.loadBarrier);
    if (tid == 0)
    {
        MbarrierInit(SharedAddress(&shared.barrier), 1);
        MbarrierInit(loadBarrier, 1);
        FenceBarrierInit();
        MbarrierArriveExpectTx(loadBarrier, kStagedNetworkBytes);
        BulkCopyToShared(SharedAddress(shared.network), network, kStagedNetworkBytes, loadBarrier);
    }
    if (warp == 0)
        TmemAlloc(SharedAddress(&shared.tmemBase), kTmemColumns);
    FenceProxyAsyncShared(); // the bias region is read by the tensor core (async proxy)
    TcgenFenceBeforeSync();
    __syncthreads();         // also publishes the barriers' initialisation
    TcgenFenceAfterSync();
    int failed = 0;
    if (!MbarrierWaitBounded(loadBarrier, 0, loadWaitPolls))
    {
        failed = 1;
        ReportTimeout(status, 0xFFFFFFFFu, 0xFFFFFFFFu); // no tile: the network image did not arrive
    }
    if (__syncthreads_or(failed))
    {
        if (tid == 0)
            (void)MbarrierWaitBounded(loadBarrier, 0);
        __syncthreads();
        if (warp == 0)
            TmemFree(shared.tmemBase, kTmemColumns);
        return 1;
    }
    return 0;
}

template <bool kFp8, bool kConvert>
__global__ void __launch_bounds__(kThreadsPerCta, kConvert ? kCtasPerSmConverting : kFp8 ? kCtasPerSmFp8 : kCtasPerSmInt8)
    DecodeKernel(const __grid_constant__ KernelParams params)
{
    // more than the 48 KB a kernel may declare statically: passed as dynamic shared memory at launch
    extern __shared__ __align__(128) unsigned char dynamicShared[];
    SharedStorage& shared = *reinterpret_cast<SharedStorage*>(dynamicShared);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;      // = the thread's row of the tile
    const int half = warp >> 2;     // 0: rows 0-3 of the tile, 1: rows 4-7

    if (SetupCta(shared, params.network, params.status, params.loadWaitPolls, tid, warp))
        return;
    int failed = 0;   // this thread gave up on a wait
    const uint32_t tmemBase = shared.tmemBase;
    uint32_t phase = 0;
    int aborted = 0;  // some thread of the CTA did (uniform: comes out of a barrier)

    TileContext ctx;
    ctx.tid = tid;
    ctx.tmemBase = tmemBase;
    // a warp may only touch the TMEM lanes 32 * (warp % 4) .. + 31
    ctx.tmemLane = tmemBase + half * kTmemColumnsPerHalf + (uint32_t((warp & 3) * 32) << 16);
    ctx.barrier = SharedAddress(&shared.barrier);
    ctx.operandA = SharedAddress(shared.operandA);
    ctx.rowChunk = reinterpret_cast<uint4*>(shared.operandA + half * kOperandBytes) + (tid & 127);
    ctx.networkBase = SharedAddress(shared.network);
    ctx.biasRegion = SharedAddress(shared.biasRegion);

    // Position of a tile in its mip.
    struct TilePlace
    {
        int mipIndex, tileX0, tileY0;
    };
    auto locate = [&](int tile, int fromMip) {
        // tiles are visited in increasing order, so the search resumes at the current mip
        TilePlace place;
        place.mipIndex = fromMip;
        while (place.mipIndex + 1 < params.numMips && tile >= params.mips[place.mipIndex + 1].firstTile)
            ++place.mipIndex;
        const KernelMip& mip = params.mips[place.mipIndex];
        const int local = tile - mip.firstTile;
        // local / tilesX through a precomputed reciprocal (exact while local * tilesX < 2^32)
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
        // ---- tables and latent footprints of the first tile -----------------------------------
        place = locate(tile, 0);
        PrepareTile<kFp8, false>(params, params.mips[place.mipIndex], shared, place.tileX0, place.tileY0, lane, warp, false);
        tablesMip = TileKeepsTables(params.mips[place.mipIndex], place.tileX0, place.tileY0) ? place.mipIndex : -1;
        __syncthreads();
    }
    while (tile < params.totalTiles)
    {
        const KernelMip& mip = params.mips[place.mipIndex];
        ctx.tile = tile;
        ctx.x = place.tileX0 + lane;
        ctx.y = place.tileY0 + warp;
        {
            // element index inside the mip fits 32 bits (8192^2 texels x 16 channels is 2^30)
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
                ctx.outStepWords = planar ? uint32_t(mip.width) : 1u; // channel pairs are 2 * width or 2 elements apart
            }
        }

        // ---- 1. this tile's network inputs -> A operand (the last MMA that read the A operand has
        //         completed: every thread waited for it) -------------------------------------------
        BuildInputs<kFp8, false>(params, mip, shared, ctx, lane, warp);

        // ---- 2. layer 0; while the tensor core works on it, prepare the NEXT tile: its tables and
        //         footprints replace this tile's, which nobody reads after the barrier inside
        //         IssueLayer, and the global-memory latency of the footprint hides behind the MMA ----
        aborted = IssueLayer<kFp8, 0>(ctx, failed);
        if (aborted)
            break;
        const int nextTile = tile + int(gridDim.x);
        if (nextTile < params.totalTiles)
        {
            place = locate(nextTile, place.mipIndex);
            // the tables of the previous tile serve this one too when both lie inside the same mip with invariant tables
            const bool keepsTables = TileKeepsTables(params.mips[place.mipIndex], place.tileX0, place.tileY0);
            PrepareTile<kFp8, false>(params, params.mips[place.mipIndex], shared, place.tileX0, place.tileY0, lane, warp, keepsTables && place.mipIndex == tablesMip);
            tablesMip = keepsTables ? place.mipIndex : -1;
        }
        ConsumeLayer<kFp8, 0, false>(params, shared, ctx, phase, failed);

        // ---- 3./4. layers 1-3 (their barriers also order the next tile's tables before its use) ---
        aborted = RunLayer<kFp8, 1, false>(params, shared, ctx, phase, failed);
        if (!aborted) aborted = RunLayer<kFp8, 2, false>(params, shared, ctx, phase, failed);
        if (!aborted) aborted = RunLayer<kFp8, 3, kConvert>(params, shared, ctx, phase, failed);
        if (aborted)
            break;
        tile = nextTile;
    }

    // ---- teardown -------------------------------------------------------------------------
    TcgenFenceBeforeSync();
    aborted = __syncthreads_or(failed);
    if (aborted && tid == 0)
        (void)MbarrierWaitBounded(ctx.barrier, phase ^ 1); // one more bounded chance for work in flight to drain
    __syncthreads();
    if (warp == 0)
        TmemFree(tmemBase, kTmemColumns);
}

// Inference on sample: one thread per query (u, v, lod) -> the texel (mip = clamp(floor(lod)),
// x = min(floor(u * W), W - 1), y likewise) is evaluated exactly as the decode kernel evaluates it
// (the reference's NtcSampleTextureSet takes an integer texel and mip and runs the same network,
// include/libntc/shaders/Inference.hlsli:282-357).  Queries are incoherent, so the taps are read
// straight from global memory; a tile is 256 consecutive queries, i.e. two 128-row GEMM chains.
template <bool kFp8>
__global__ void __launch_bounds__(kThreadsPerCta, kFp8 ? kCtasPerSmFp8 : kCtasPerSmInt8) SampleKernel(const __grid_constant__ SampleParams params)
{
    // more than the 48 KB a kernel may declare statically: passed as dynamic shared memory at launch
    extern __shared__ __align__(128) unsigned char dynamicShared[];
    SharedStorage& shared = *reinterpret_cast<SharedStorage*>(dynamicShared);
    __shared__ KernelMip mipTable[16];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int half = warp >> 2;

    // the mip descriptions are indexed per thread: a copy in shared memory (visible after the barrier inside SetupCta)
    if (tid < params.numMips)
        mipTable[tid] = params.mips[tid];
    if (SetupCta(shared, params.network, params.status, params.loadWaitPolls, tid, warp))
        return;
    int failed = 0, aborted = 0;
    const uint32_t tmemBase = shared.tmemBase;
    uint32_t phase = 0;

    TileContext ctx;
    ctx.tid = tid;
    ctx.tmemBase = tmemBase;
    ctx.tmemLane = tmemBase + half * kTmemColumnsPerHalf + (uint32_t((warp & 3) * 32) << 16);
    ctx.barrier = SharedAddress(&shared.barrier);
    ctx.operandA = SharedAddress(shared.operandA);
    ctx.rowChunk = reinterpret_cast<uint4*>(shared.operandA + half * kOperandBytes) + (tid & 127);
    ctx.networkBase = SharedAddress(shared.network);
    ctx.biasRegion = SharedAddress(shared.biasRegion);
    ctx.outStepWords = 1;

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
            const uint32_t zeroWord = PackCodes<kFp8>(QuantizeInputPair<kFp8>(__float2half2_rn(0.f)),
                                                      QuantizeInputPair<kFp8>(__float2half2_rn(0.f)));
#pragma unroll
            for (int i = 0; i < 8; ++i)
                words[i] = zeroWord;
            // K padding: zeros (e4m3) or the constant inputs of the bias slots (int8)
            const uint32_t slotFill = kFp8 ? 0u : kBiasSlotValue * 0x01010101u;
            words[12] = words[13] = words[14] = slotFill;
            words[15] = kFp8 ? 0u : ((slotFill & 0x00FFFFFFu) | 0x01000000u);
            SampleGridsDirect<kFp8, false>(params.latents, params.numLayers, mip, x, y, shared.latentTable, words, params.interleaved != 0);
            // src/RegressionKernels.h:59-85
            float xf = __fmul_rn(float(x), mip.positionScale);
            float yf = __fmul_rn(float(y), mip.positionScale);
#pragma unroll
            for (int wave = 0; wave < 3; ++wave)
            {
                const float ex = __fmaf_rn(Frac(xf), 2.f, -1.f), ey = __fmaf_rn(Frac(yf), 2.f, -1.f);
                const float ez = __fmaf_rn(Frac(__fadd_rn(xf, 0.25f)), 2.f, -1.f);
                const float ew = __fmaf_rn(Frac(__fadd_rn(yf, 0.25f)), 2.f, -1.f);
                words[8 + wave] = PackCodes<kFp8>(QuantizeInputPair<kFp8>(__floats2half2_rn(ex, ey)),
                                                   QuantizeInputPair<kFp8>(__floats2half2_rn(ez, ew)));
                xf = __fmul_rn(xf, 2.f);
                yf = __fmul_rn(yf, 2.f);
            }
            words[11] = PackCodes<kFp8>(QuantizeInputPair<kFp8>(__float2half2_rn(mip.positionLod)),
                                        QuantizeInputPair<kFp8>(__float2half2_rn(0.f)));
#pragma unroll
            for (int chunk = 0; chunk < 4; ++chunk)
                ctx.rowChunk[chunk * 128] = make_uint4(words[4 * chunk], words[4 * chunk + 1], words[4 * chunk + 2], words[4 * chunk + 3]);
        }

        aborted = RunLayer<kFp8, 0, false>(params, shared, ctx, phase, failed);
        if (!aborted) aborted = RunLayer<kFp8, 1, false>(params, shared, ctx, phase, failed);
        if (!aborted) aborted = RunLayer<kFp8, 2, false>(params, shared, ctx, phase, failed);
        if (!aborted) aborted = RunLayer<kFp8, 3, false>(params, shared, ctx, phase, failed);
        if (aborted)
            break;
    }

    TcgenFenceBeforeSync();
    aborted = __syncthreads_or(failed);
    if (aborted && tid == 0)
        (void)MbarrierWaitBounded(ctx.barrier, phase ^ 1);
    __syncthreads();
    if (warp == 0)
        TmemFree(tmemBase, kTmemColumns);
}



// Lets `kernel` use sizeof(SharedStorage) bytes of dynamic shared memory on the current device
// (needed once per device and kernel; remembered per device).
template <typename Kernel>
cudaError_t AllowSharedStorage(Kernel kernel, std::atomic<unsigned long long>& doneMask)
{
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess)
        return err;
    const unsigned long long bit = 1ull << (device & 63);
    if (doneMask.load(std::memory_order_acquire) & bit)
        return cudaSuccess;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(SharedStorage)));
    if (err == cudaSuccess)
        doneMask.fetch_or(bit, std::memory_order_release);
    return err;
}

template <typename Kernel, typename Params>
cudaError_t LaunchWithSharedStorage(Kernel kernel, std::atomic<unsigned long long>& doneMask, const Params& params, int ctas,
    cudaStream_t stream, size_t bytes = sizeof(SharedStorage))
{
    cudaError_t err = AllowSharedStorage(kernel, doneMask);
    if (err != cudaSuccess)
        return err;
    kernel<<<ctas, kThreadsPerCta, bytes, stream>>>(params);
    return cudaGetLastError();
}

} // namespace

cudaError_t LaunchSample(const SampleParams& params, bool fp8, int ctas, cudaStream_t stream)
{
    static std::atomic<unsigned long long> done[2];
    const size_t bytes = offsetof(SharedStorage, tables); // the tables and footprints are not used
    return fp8 ? LaunchWithSharedStorage(SampleKernel<true>, done[1], params, ctas, stream, bytes)
               : LaunchWithSharedStorage(SampleKernel<false>, done[0], params, ctas, stream, bytes);
}

cudaError_t LaunchDecode(const KernelParams& params, bool fp8, int ctas, cudaStream_t stream)
{
    static std::atomic<unsigned long long> done[4];
    if (params.convert)
        return fp8 ? LaunchWithSharedStorage(DecodeKernel<true, true>, done[3], params, ctas, stream)
                   : LaunchWithSharedStorage(DecodeKernel<false, true>, done[2], params, ctas, stream);
    return fp8 ? LaunchWithSharedStorage(DecodeKernel<true, false>, done[1], params, ctas, stream)
               : LaunchWithSharedStorage(DecodeKernel<false, false>, done[0], params, ctas, stream);
}

} // namespace ntcb
