// What the block-compression kernels share: the description of the source mip and of the block
// rectangle, and the texel loads (block_compress.cu: BC1 - BC5; block_compress_bc7.cu: BC7).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "ntcb.h"

namespace ntcb
{

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

__device__ __forceinline__ __half LoadHalf(const BlockCompressArguments& args, int x, int y, int channel)
{
    const size_t w = size_t(args.width), c = size_t(args.channels);
    const size_t index = args.layout == NTCB_LAYOUT_INTERLEAVED
        ? (size_t(y) * w + size_t(x)) * c + size_t(channel)
        : size_t(y) * w * c + size_t(channel & ~1) * w + 2 * size_t(x) + size_t(channel & 1);
    return args.texels[index];
}

// Channels `channel` (even) and `channel + 1` of one texel as one word; needs an even channel count.
__device__ __forceinline__ uint32_t LoadPair(const BlockCompressArguments& args, int x, int y, int channel)
{
    const size_t w = size_t(args.width), c = size_t(args.channels);
    const size_t index = args.layout == NTCB_LAYOUT_INTERLEAVED ? (size_t(y) * w + size_t(x)) * c + size_t(channel)
                                                                 : size_t(y) * w * c + size_t(channel) * w + 2 * size_t(x);
    return *reinterpret_cast<const uint32_t*>(args.texels + index);
}

// The BC7 half of ntcb_block_compress (block_compress_bc7.cu); `params` has passed the checks common to all formats.
int LaunchBlockCompressBc7(const NtcbBlockCompressParams& params, const BlockCompressArguments& args, cudaStream_t stream);

} // namespace ntcb
