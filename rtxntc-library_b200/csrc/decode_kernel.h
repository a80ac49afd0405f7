// Internal interface between the C ABI (ntcb.cu) and the sm_100a decode kernel (decode_kernel.cu).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "output_convert.cuh"

struct NtcbOutputConversion; // include/ntcb.h

namespace ntcb
{

constexpr int kTileWidth = 32;
constexpr int kTileHeight = 8;      // a tile is two 32x4 halves, each a 128-row GEMM chain
constexpr int kThreadsPerCta = kTileWidth * kTileHeight; // one thread per texel of a tile
constexpr int kOperandBytes = 128 * 64; // A operand of one half: 128 rows x 64 bytes
constexpr int kCtasPerSmInt8 = 4;  // resident CTAs per SM the two kernel variants are compiled for
constexpr int kCtasPerSmFp8 = 4;
constexpr int kCtasPerSmConverting = 4; // ... and the variants with a converting epilogue (either weight mode)
constexpr int kTmemColumnsPerHalf = 64;    // widest accumulator (layer 0: 64 outputs)
constexpr int kTmemColumns = 2 * kTmemColumnsPerHalf;
constexpr uint32_t kSpinLimit = 1u << 20;  // mbarrier polls before a wait is declared expired (about two seconds)
constexpr uint32_t kWaitHintNanoseconds = 2000; // how long one poll may suspend the thread
constexpr int kFootprintHiBytes = 11264;   // shared memory for a tile's unpacked footprint in the high-res grid
constexpr int kFootprintLoBytes = 4096;    // ... and in the low-res grid (half the resolution)

// Image of the network in shared memory (produced on the host by ntcb_stage_network).
// Weight matrix of layer l: N_l rows (outputs) x K_l bytes (inputs, padded to a multiple of 32) in
// K-major core-matrix order: byte (n, k) lives at (k / 16) * (N_l * 16) + n * 16 + (k % 16).
//
// Int8 layers carry their int32 bias inside the matrix product: the A operand holds constant
// inputs (kBiasSlotValue; 1 in the last slot of each K step) in K slots past the real inputs, and
// the weight rows hold a decomposition of the bias over those slots, so that sum(weights * inputs)
// already includes it.  Layers 0 and 2 have 16 such slots in the padding of their 48 inputs;
// layers 1, 2 and 3 get one more K step of 32 slots whose A operand is a constant region of shared
// memory.  When a bias does not fit, the whole network falls back to the bias table
// (kFlagBiasTable).  The FP8 network, whose only int8 layer is the 16-output last one, always uses
// the table.
constexpr int kWeightOffset0 = 0;      // 64 x 64
constexpr int kWeightOffset1 = 4096;   // 48 x 96 (64 inputs + 32 bias slots)
constexpr int kWeightOffset2 = 8704;   // 32 x 96 (48 inputs + 16 + 32 bias slots)
constexpr int kWeightOffset3 = 11776;  // 16 x 64 (32 inputs + 32 bias slots)
constexpr int kScaleOffset = 12800;    // float[4][64]
constexpr int kBiasOffset = 13824;     // per layer 256 bytes: int32[64] (int8 layers) or half[64] (e4m3 layers)
constexpr int kFlagsOffset = 14848;    // uint32[4]: word 0 = kFlag* bits
constexpr int kStagedNetworkBytes = 14864;
constexpr uint32_t kFlagBiasTable = 1; // int8 layers add their bias from the table (the bias slots hold zero weights)
constexpr int kBiasSlotValue = 127;
constexpr int kBiasRegionBytes = 128 * 32; // constant A operand of the extra K step: 128 rows x 32 slots

// Image of the network for the reference-numerics kernels (produced by ntcb_stage_network_reference).
// Int8 networks, and layer 3 of FP8 networks: binary16 weights as the reference's CUDA path rebuilds
// them from the file
// (src/Quantizer.cu:325-408), K-major core matrices of 8 halves (element (n, k) of layer l at
// (k / 8) * (N_l * 16) + n * 16 + (k % 8) * 2), followed per layer by the operand of the "bias
// step": an N_l x 16 matrix whose column 0 is the binary16 bias.  Multiplied by a constant A operand
// whose rows are (1, 0, ..., 0), it sets the accumulators to the bias exactly, as the reference
// initialises its accumulator fragments (src/tin/tin_mlp.h:71-89).  Layers 0-2 of FP8 networks keep
// their e4m3 bytes: one N_l x 32 byte matrix per 16-wide K step, the step's 16 weights at their place
// inside the 32-wide chunk and zeros in the other half (same offsets and sizes as the binary16
// matrices they replace).
// The image of an INT8 network is shorter: after the four weight matrices it has ONE 64 x 8 matrix of
// halves, 16 bytes per row n, whose column l is the bias of output n of layer l (kRefInt8BiasOffset).
// The bias step of layer l multiplies it by rows that are the unit vector e_l, which picks column l;
// the descriptor's leading offset of 0 makes the step's second 8-wide half read the same matrix, which
// the zeros in the second half of the e_l rows cancel.
constexpr int kRefWeightOffset0 = 0;       // 64 x 48 halves
constexpr int kRefWeightOffset1 = 6144;    // 48 x 64
constexpr int kRefWeightOffset2 = 12288;   // 32 x 48
constexpr int kRefWeightOffset3 = 15360;   // 16 x 32
constexpr int kRefBiasOffset0 = 16384;     // 64 x 16 halves
constexpr int kRefBiasOffset1 = 18432;     // 48 x 16
constexpr int kRefBiasOffset2 = 19968;     // 32 x 16
constexpr int kRefBiasOffset3 = 20992;     // 16 x 16
constexpr int kRefNetworkBytes = 21504;     // size of the image, both kinds (an Int8 network's ends early)
constexpr int kRefInt8BiasOffset = 16384;   // Int8 networks: 64 rows x 8 halves, column l = bias of layer l
constexpr int kRefInt8NetworkBytes = 17408; // ... what the Int8 kernels copy to shared memory
// A operand of one 128-row GEMM chain of the Int8 kernels in shared memory: 128 rows x 48 halves.  Layer 0
// has 48 inputs; of layer 1's 64 the first 32 are here, the other 32 in tensor memory, like all of
// layers 2 and 3.
constexpr int kRefOperandBytes = 128 * 96;
// Tile of the reference-numerics kernel: kRefChains 128-row chains (32 x 4 texels each) per CTA.
// Two chains (32x8 texels, 256 threads) at three CTAs per SM measured faster than four chains
// (32x16, 512 threads) at two.
constexpr int kRefChains = 2;
constexpr int kRefTileHeight = 4 * kRefChains;
constexpr int kRefThreadsPerCta = 128 * kRefChains;
constexpr int kRefTmemColumns = kRefChains * kTmemColumnsPerHalf;
constexpr int kRefFootprintHiBytes = 8192;  // the binary16 operands leave less room for the high-res footprint
constexpr int kRefFootprintLoBytes = 4096;
// The Int8 kernels, whose binary16 operands take more room, have less for the low-res footprint: enough for
// what fits into the high-res one (the low-res grid has half the resolution: at a grid-to-mip ratio of 1/2
// a tile's footprint is 18 x 6 pixels of 24 bytes).
constexpr int kRefInt8FootprintLoBytes = 2816;
// The warp that issues the matrix products of both chains of a tile after a CTA-wide barrier, chain 0 first:
// the first warp of chain 1.  It then waits for chain 1, whose products finish last anyway; a warp of chain 0
// would start on its own chain's results late by the time it takes to issue chain 1's (2 %).  (After a
// chain-local barrier each chain's first warp issues its own.)
constexpr int kIssuingWarp = 4;
constexpr int kCtasPerSmRef = 4;       // Int8 networks: 56 KB of shared memory and 64 registers, like the FP8 kernels
constexpr int kCtasPerSmRefFp8 = 4; // FP8 networks: 8-bit operands halve the A buffers
constexpr int kCtasPerSmRefSample = 4; // inference on sample, Int8 networks (its launches leave the footprints out)

constexpr uint32_t kStatusBarrierTimeout = 1;

constexpr int kLayoutPlanarPairs = 0;
constexpr int kLayoutInterleaved = 1;

struct KernelMip
{
    int width, height;
    int rowBegin, rowEnd;
    int hiWidth, hiHeight, loWidth, loHeight;
    unsigned long long hiOffset, loOffset, hiPlane, loPlane;
    unsigned long long outOffset;
    float invWidth, invHeight;
    float positionScale, positionLod;
    int firstTile, tilesX;
    unsigned tilesXMagic; // ceil(2^32 / tilesX) for tilesX > 1: local / tilesX == umulhi(local, magic) while local * tilesX < 2^32
    int staged;      // the tile footprints of both grids fit into shared memory
    int strideBytes; // bytes per staged latent pixel: 8 per layer, padded to an odd multiple of 8 (8, 24, 24, 40) so that
                     // the 8-byte reads of neighbouring pixels fall into different shared-memory banks
    int storeBytes;  // widest store (4, 8 or 16 bytes) the fp16 texels of this mip may go out with: the interleaved
                     // layout with a texel size and a mip address that are multiples of it; 4 otherwise
    int invariant;   // every size involved is a power of two: the tap and positional-encoding tables of a tile do not
                     // depend on which tile of the mip it is (see PrepareTaps)
    int hiStepX, hiStepY, loStepX, loStepY; // invariant mips: latent pixels of each grid per tile step in x and y
};

struct KernelParams
{
    const uint16_t* latents;
    const uint8_t* network;
    __half* out;
    uint32_t* status;
    int numMips;
    int numLayers;
    int channels;
    int outputLayout;
    int totalTiles;
    uint32_t loadWaitPolls; // polls a CTA spends waiting for the network image before it gives up (kSpinLimit by default)
    // converting epilogue (convert != 0): `out` receives pixels in the client's format instead of fp16 texels
    int convert;
    int firstChannel, numChannels; // channels the converted pixel starts with
    OutputConversion conversion;
    KernelMip mips[16];
};

struct SampleParams
{
    const uint16_t* latents;
    const uint8_t* network;
    const float* queries; // [numQueries][3]: u, v, lod
    __half* out;          // [numQueries][channels]
    uint32_t* status;
    unsigned long long numQueries;
    int numMips;
    int numLayers;
    int channels;
    uint32_t loadWaitPolls; // as in KernelParams
    // Nonzero: `latents` is the pixel-major copy ntcb_interleave_latents makes - the layers of a latent pixel side
    // by side in a slot of 1, 2 or 4 elements (three layers are padded to four) - and hiOffset / loOffset of the
    // mips are element offsets into THAT buffer.
    int interleaved;
    KernelMip mips[16];
};

// Alignment the converting epilogue needs for the first pixel of a mip: it stores a pixel of
// `pixelBytes` bytes with the widest vector store that divides its size (16, 8, 4, 2 or 1 bytes),
// and consecutive pixels are `pixelBytes` apart.
inline size_t ConvertedPixelAlignment(size_t pixelBytes)
{
    return !(pixelBytes & 15) ? 16 : !(pixelBytes & 7) ? 8 : !(pixelBytes & 3) ? 4 : !(pixelBytes & 1) ? 2 : 1;
}

// Checks a client's conversion request (NtcbOutputConversion of the C ABI) against a texture set of
// `channels` channels and packs it for the kernels; returns an NtcbStatus.
int MakeOutputConversion(const ::NtcbOutputConversion& request, int channels, OutputConversion& out);

cudaError_t LaunchDecode(const KernelParams& params, bool fp8, int ctas, cudaStream_t stream);
// The reference-numerics kernel (decode_kernel_ref.cu): params.network is a kRefNetworkBytes image.
cudaError_t LaunchDecodeRef(const KernelParams& params, bool fp8, int ctas, cudaStream_t stream);
cudaError_t LaunchSampleRef(const SampleParams& params, bool fp8, int ctas, cudaStream_t stream);
cudaError_t LaunchSample(const SampleParams& params, bool fp8, int ctas, cudaStream_t stream);

} // namespace ntcb
