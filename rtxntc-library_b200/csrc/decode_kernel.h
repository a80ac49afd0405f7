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
constexpr uint32_t kSpinLimit = 1u << 22;  // mbarrier polls before a wait is declared expired
constexpr int kFootprintHiBytes = 11264;   // shared memory for a tile's unpacked footprint in the high-res grid
constexpr int kFootprintLoBytes = 4096;    // ... and in the low-res grid (half the resolution)

// Image of the network in shared memory (produced on the host by ntcb_stage_network).
// Weight matrix of layer l: N_l rows (outputs) x K_l bytes (inputs, padded to a multiple of 32) in
// K-major core-matrix order: byte (n, k) lives at (k / 16) * (N_l * 16) + n * 16 + (k % 16).
constexpr int kWeightOffset0 = 0;     // 64 x 64
constexpr int kWeightOffset1 = 4096;  // 48 x 64
constexpr int kWeightOffset2 = 7168;  // 32 x 64
constexpr int kWeightOffset3 = 9216;  // 16 x 32
constexpr int kScaleOffset = 9728;    // float[4][64]
constexpr int kBiasOffset = 10752;    // per layer 256 bytes: int32[64] (int8 layers) or half[64] (e4m3 layers)
constexpr int kStagedNetworkBytes = 11776;

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
    int strideShift; // log2 of the bytes per staged latent pixel (8 bytes per layer, rounded up to a power of two)
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
    KernelMip mips[16];
};

// Checks a client's conversion request (NtcbOutputConversion of the C ABI) against a texture set of
// `channels` channels and packs it for the kernels; returns an NtcbStatus.
int MakeOutputConversion(const ::NtcbOutputConversion& request, int channels, OutputConversion& out);

cudaError_t LaunchDecode(const KernelParams& params, bool fp8, int ctas, cudaStream_t stream);
cudaError_t LaunchSample(const SampleParams& params, bool fp8, int ctas, cudaStream_t stream);

} // namespace ntcb
