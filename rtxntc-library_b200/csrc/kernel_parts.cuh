// Building blocks shared by the decode kernels (decode_kernel.cu: exact accumulation;
// decode_kernel_ref.cu: the reference's binary16 accumulation): PTX wrappers for mbarriers, tensor
// memory and the TMA bulk copy, the shared-memory matrix descriptor, and the bilinear tap setup.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "decode_kernel.h"

namespace ntcb
{
namespace
{

__device__ __forceinline__ uint32_t SharedAddress(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void MbarrierInit(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// One arrival (release at CTA scope: what this thread wrote before, and what it observed, is visible to a
// thread that sees the phase complete).
__device__ __forceinline__ void MbarrierArrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void FenceBarrierInit()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// One poll of a barrier phase.  The instruction may suspend the thread until the phase completes
// or `kWaitHintNanoseconds` have passed, whichever comes first (measured: the same speed as polls
// without the hint).
__device__ __forceinline__ bool MbarrierTryWait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kWaitHintNanoseconds)
        : "memory");
    return done != 0;
}

// Announces `bytes` of asynchronous copies that will complete on the barrier, and arrives on it.
__device__ __forceinline__ void MbarrierArriveExpectTx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// TMA bulk copy global -> shared memory of this CTA (addresses and size multiples of 16 bytes);
// completion is signalled on the barrier.
__device__ __forceinline__ void BulkCopyToShared(uint32_t dstShared, const void* srcGlobal, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dstShared), "l"(srcGlobal), "r"(bytes), "r"(bar)
                 : "memory");
}

// Bounded wait: returns false when the barrier did not complete within `limit` polls.
__device__ __forceinline__ bool MbarrierWaitBounded(uint32_t bar, uint32_t parity, uint32_t limit = kSpinLimit)
{
    for (uint32_t spin = 0; spin < limit; ++spin)
    {
        if (MbarrierTryWait(bar, parity))
            return true;
    }
    return false;
}

// Records an expired wait in the status words.  The first thread of the grid to report claims word 0
// and alone writes the tile and layer, so the three words always describe one and the same wait.
__device__ __noinline__ void ReportTimeout(uint32_t* status, uint32_t tile, uint32_t layer)
{
    if (atomicCAS(&status[0], 0u, kStatusBarrierTimeout) == 0u)
    {
        status[1] = tile;
        status[2] = layer;
    }
}

__device__ __forceinline__ void FenceProxyAsyncShared()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void TcgenFenceBeforeSync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void TcgenFenceAfterSync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void TmemAlloc(uint32_t sharedSlot, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sharedSlot), "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void TmemFree(uint32_t address, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

__device__ __forceinline__ void UmmaCommit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 16 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void TmemLoad16(uint32_t address, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(address)
        : "memory");
}

// Four consecutive 32-bit columns of this thread's TMEM lane, written.
__device__ __forceinline__ void TmemStore4(uint32_t address, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}

__device__ __forceinline__ void TmemStoreWait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void TmemLoadWait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, K-major, no swizzle: 8x16-byte core matrices; `leadingBytes`
// separates core matrices along K, `strideBytes` separates 8-row groups along M/N.
__device__ __forceinline__ uint64_t MakeSmemDescriptor(uint32_t sharedAddress, uint32_t leadingBytes, uint32_t strideBytes)
{
    uint64_t desc = 0;
    desc |= uint64_t((sharedAddress & 0x3FFFF) >> 4);
    desc |= uint64_t((leadingBytes >> 4) & 0x3FFF) << 16;
    desc |= uint64_t((strideBytes >> 4) & 0x3FFF) << 32;
    desc |= uint64_t(1) << 46; // descriptor version of this architecture
    return desc;               // base offset 0, layout type 0 (no swizzle)
}

__device__ __forceinline__ uint32_t AsU32(__half2 v)
{
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ __half2 AsHalf2(uint32_t v)
{
    return *reinterpret_cast<__half2*>(&v);
}

// Inf / NaN -> 0 in the channel pairs of one texel (src/Inference.cu:125-126, src/CudaUtils.h:30-35).
// A binary16 value times zero is a zero unless the value is an infinity or a NaN, so one fused
// multiply-add per pair into a common sum detects whether anything has to be done at all.
__device__ __forceinline__ void ScrubSpecials(uint32_t (&bits)[8], int channelPairs)
{
    __half2 sum = __float2half2_rn(0.f);
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if (j < channelPairs)
            sum = __hfma2(AsHalf2(bits[j]), __float2half2_rn(0.f), sum);
    if (AsU32(sum) & 0x7FFF7FFFu)
    {
        // rare, so kept off the common path
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
}

// Stores the channel pairs of one texel.  Pixel-interleaved layout: the pairs are consecutive words
// and go out as 16-, 8- or 4-byte stores, whatever `vectorBytes` (the alignment every texel of the
// mip has) allows; planar-pair layout: `stepWords` words apart, one word each.
__device__ __forceinline__ void StoreTexel(uint32_t* out, uint32_t stepWords, int vectorBytes, const uint32_t (&bits)[8],
    int channelPairs)
{
    if (vectorBytes == 16)
    {
#pragma unroll
        for (int j = 0; j < 8; j += 4)
            if (j < channelPairs)
                *reinterpret_cast<uint4*>(out + j) = make_uint4(bits[j], bits[j + 1], bits[j + 2], bits[j + 3]);
    }
    else if (vectorBytes == 8)
    {
#pragma unroll
        for (int j = 0; j < 8; j += 2)
            if (j < channelPairs)
                *reinterpret_cast<uint2*>(out + j) = make_uint2(bits[j], bits[j + 1]);
    }
    else
    {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (j < channelPairs)
                out[j * stepWords] = bits[j];
    }
}

struct GridTaps
{
    int o00, o01, o10, o11;
    __half2 w00, w01, w10, w11;
};

// Bilinear footprint of one texel in one latent grid (src/FeatureGridDevice.h:33-58).
__device__ __forceinline__ void SetupTaps(float u, float v, int w, int h, GridTaps& taps)
{
    float px = __fmaf_rn(u, float(w), -0.5f);
    float py = __fmaf_rn(v, float(h), -0.5f);
    float xbf = floorf(px), ybf = floorf(py);
    float dx = __fsub_rn(px, xbf), dy = __fsub_rn(py, ybf);
    float dxn = __fsub_rn(1.f, dx), dyn = __fsub_rn(1.f, dy);
    int xb = int(xbf), yb = int(ybf);
    // wrap addressing; the sample position is < size - 0.5, so only -1 needs folding
    int x0 = xb < 0 ? xb + w : xb;
    int y0 = yb < 0 ? yb + h : yb;
    int x1 = (x0 + 1 == w) ? 0 : x0 + 1;
    int y1 = (y0 + 1 == h) ? 0 : y0 + 1;
    taps.o00 = y0 * w + x0;
    taps.o01 = y0 * w + x1;
    taps.o10 = y1 * w + x0;
    taps.o11 = y1 * w + x1;
    taps.w00 = __half2half2(__float2half_rn(__fmul_rn(dxn, dyn)));
    taps.w01 = __half2half2(__float2half_rn(__fmul_rn(dx, dyn)));
    taps.w10 = __half2half2(__float2half_rn(__fmul_rn(dxn, dy)));
    taps.w11 = __half2half2(__float2half_rn(__fmul_rn(dx, dy)));
}

__device__ __forceinline__ float Frac(float t)
{
    return __fsub_rn(t, floorf(t));
}

// Normalised sample coordinate of a texel, (texel + 0.5) / extent (src/Inference.cu:52-53).  The
// reference is built with --use_fast_math, so its division is the approximate one
// (div.approx.ftz.f32: the operand times the hardware's reciprocal approximation, which for extents
// that are not powers of two can differ from the correctly rounded reciprocal in the last bit, and
// with it - rarely - a bilinear weight).  The reference-numerics kernels issue the same instruction;
// the exact-accumulation kernels keep the multiplication by the correctly rounded reciprocal that
// their CPU restatement uses.
template <bool kReferenceDivision>
__device__ __forceinline__ float TexelCoordinate(int texel, int extent, float invExtent)
{
    const float centre = __fadd_rn(float(texel), 0.5f);
    if (kReferenceDivision)
    {
        float u;
        asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(u) : "f"(centre), "f"(float(extent)));
        return u;
    }
    return __fmul_rn(centre, invExtent);
}

// One axis of the bilinear footprint (src/FeatureGridDevice.h:35-45): base tap index (before
// wrapping) and the fractional offset of a texel coordinate in a latent grid of `size` pixels.
template <bool kReferenceDivision>
__device__ __forceinline__ void AxisTap(int texel, int extent, float invExtent, int size, int& base, float& frac)
{
    const float u = TexelCoordinate<kReferenceDivision>(texel, extent, invExtent);
    const float p = __fmaf_rn(u, float(size), -0.5f);
    const float b = floorf(p);
    base = int(b);
    frac = __fsub_rn(p, b);
}

// Nonzero in exactly one lane of the (converged) warp.
__device__ __forceinline__ uint32_t ElectOne()
{
    uint32_t elected;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(elected));
    return elected;
}

// The barrier before a layer's matrix products.  The operand rows of a chain are written by the chain's
// own 128 threads, and only they read the chain's accumulators, so between two layers of the same tile a
// chain needs nobody else: kChainLocal = 1 makes its threads meet in a named barrier of their own (1 or 2)
// and go on without the other chain - 3.3 % faster on the benchmark workload than the CTA-wide barrier for
// every layer.  Giving up is then agreed on at the CTA-wide barriers that remain (kChainLocal = 0: layers 0
// and 3 of the decode kernels, where all eight warps share the tile's tables), or, with kChainLocal = 2,
// among the chain's threads (inference on sample, where nothing is shared).  Returns nonzero when the
// caller is to give up.
template <int kChainLocal>
__device__ __forceinline__ int LayerBarrier(int tid, int failed)
{
    if (kChainLocal == 0)
        return __syncthreads_or(failed);
    const int half = tid >> 7;
    if (kChainLocal == 1)
    {
        if (half)
            asm volatile("bar.sync 2, 128;" ::: "memory");
        else
            asm volatile("bar.sync 1, 128;" ::: "memory");
        return 0;
    }
    uint32_t any;
    if (half)
        asm volatile(
            "{\n\t"
            ".reg .pred p, q;\n\t"
            "setp.ne.b32 q, %1, 0;\n\t"
            "bar.red.or.pred p, 2, 128, q;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(any)
            : "r"(failed)
            : "memory");
    else
        asm volatile(
            "{\n\t"
            ".reg .pred p, q;\n\t"
            "setp.ne.b32 q, %1, 0;\n\t"
            "bar.red.or.pred p, 1, 128, q;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(any)
            : "r"(failed)
            : "memory");
    return int(any);
}

// Which barrier a layer of the tile decoders takes: see LayerBarrier.
template <int kLayer>
constexpr int TileLayerBarrier()
{
    return (kLayer == 1 || kLayer == 2) ? 1 : 0;
}

} // namespace
} // namespace ntcb
