// ntcb_host.h - C++ host interface of the B200-native NTC decoder.
//
// The classes mirror, for the decompression path only, the reference's public host interface
// (include/libntc/ntc.h): the same method names, argument meaning and error convention, so code
// written against ntc::IContext / ntc::ITextureSet ports by changing the namespace.  Every method
// is a thin layer over the C ABI in ntcb.h (which is what foreign-language bindings use).
//
//   ntc::CreateContext / DestroyContext                 -> ntcb::CreateContext / DestroyContext
//   IContext::CreateCompressedTextureSetFromMemory/File -> same names
//   IContext::DestroyTextureSet                         -> same name
//   ITextureSet::GetDesc / GetLatentShape               -> same names
//   ITextureSet::Decompress(stats, useInt8Weights)      -> same name, same default (FP8 weights)
//   ITextureSet::ReadChannels(params)                   -> same name (every ChannelFormat, colour spaces, dithering)
//   IContext::MakeBlockCompressionComputePass + dispatch -> ITextureSet::BlockCompress / BlockCompressTexture (BC1 - BC5, BC7; CUDA)
// tests/cpp/host_example.cpp is a complete client.
//
// Status values are the NtcbStatus codes of ntcb.h; ntcb::GetLastErrorMessage() returns the
// thread-local message of the last failing call, like ntc::GetLastErrorMessage().
#pragma once

#include "ntcb.h"

namespace ntcb
{

using Status = int; // NtcbStatus

struct TextureSetDesc // ntc::TextureSetDesc, include/libntc/ntc.h:158-177
{
    int width = 0, height = 0, channels = 0, mips = 1;
};

struct LatentShape // ntc::LatentShape, include/libntc/ntc.h:131-156
{
    int gridSizeScale = 4, numFeatures = 16;
};

struct ContextParameters // ntc::ContextParameters, include/libntc/ntc.h:1278-1305 (CUDA part)
{
    int cudaDevice = 0;
};

using TextureSetFeatures = NtcbTextureSetFeatures;
using DecompressionStats = NtcbDecompressionStats;
using ReadChannelsParameters = NtcbReadChannelsParams;

class ITextureSet
{
public:
    virtual TextureSetDesc const& GetDesc() const = 0;
    virtual LatentShape const& GetLatentShape() const = 0;
    // ITextureSetMetadata::GetTextureCount / GetTexture: a named channel range with its intended formats
    virtual int GetTextureCount() const = 0;
    virtual Status GetTexture(int index, NtcbTextureDesc& outTexture) const = 0;
    virtual Status Decompress(DecompressionStats* pOutStats, bool useInt8Weights = false) = 0;
    // rowRanges: [mips][2] = {rowBegin, rowEnd} per mip (tile-row sharding); NULL = whole mips
    virtual Status DecompressRows(const int32_t* rowRanges, DecompressionStats* pOutStats, bool useInt8Weights = false) = 0;
    // Decompress and ReadChannels of every mip fused into one kernel launch: `destination` (host or
    // device) receives the mips one after the other, each as rows of pixels of conversion.components
    // values of conversion.channelFormat without padding; the fp16 texels are not stored.
    // conversion.srcColorSpaces is ignored (the container's channel colour spaces apply).
    virtual Status DecompressConverted(DecompressionStats* pOutStats, bool useInt8Weights,
        NtcbOutputConversion const& conversion, int addressSpace, void* destination, size_t destinationBytes) = 0;
    virtual Status ReadChannels(ReadChannelsParameters const& params) = 0;
    virtual Status GetDeviceMip(int mipLevel, void** outPointer, size_t* outBytes) = 0;
    // One decoded mip to BC1 - BC5 or BC7 blocks in device memory (see ntcb_block_compress), queued on the
    // set's stream: the whole mip, (width + 3) / 4 blocks per row, rowPitch bytes between rows of blocks.
    virtual Status BlockCompress(int mipLevel, int firstChannel, int numChannels, int format, float alphaThreshold,
        void* deviceBlocks, size_t rowPitch) = 0;
    // ITextureMetadata::GetBC7ModeBuffer / MakeAndStoreBC7ModeBuffer (include/libntc/ntc.h:436-449) for texture
    // `textureIndex`: the mode bitmap stored in the file for a mip level (host memory owned by the set; null
    // and 0 when there is none), or made from BC7 blocks of exactly that mip's size in blocks.
    virtual Status GetBC7ModeBuffer(int textureIndex, int mipLevel, void const** outData, size_t* outSize) const = 0;
    virtual Status MakeAndStoreBC7ModeBuffer(int textureIndex, int mipLevel, int widthInBlocks, int heightInBlocks,
        void const* blockData, size_t blockDataSize, size_t rowPitch) = 0;
    // One mip of one texture of the set to the block format its header names (BC1 - BC5, BC7), with its
    // channel range; BC7 takes the texture's stored mode buffer of that mip when it has one
    // (BlockCompressionModeBufferSource::TextureSet), else searches every mode.
    virtual Status BlockCompressTexture(int textureIndex, int mipLevel, float alphaThreshold, void* deviceBlocks,
        size_t rowPitch) = 0;
    // ITextureSet::LoadFromMemory: another compressed set of the same dimensions and latent shape into this
    // one's buffers (FileIncompatible otherwise, and nothing changes); the texels must be decompressed again.
    virtual Status LoadFromMemory(void const* pData, size_t size) = 0;
    // Inference on sample (the reference offers it to shaders only: NtcSampleTextureSet,
    // include/libntc/shaders/Inference.hlsli:282-357, fed by IContext::MakeInferenceData).  `deviceQueries`: numQueries
    // x (u, v, lod) floats, `deviceOut`: numQueries x channels binary16 values, both in the memory of the set's
    // device; query q selects a texel as ntcb_sample describes and receives the bits Decompress would write there.
    // The compressed data is uploaded when the device copy is not current (first use, LoadFromMemory), its
    // pixel-major copy is made then too; the call waits for the answers.
    virtual Status Sample(float const* deviceQueries, uint64_t numQueries, void* deviceOut, bool useInt8Weights) = 0;
    virtual Status Synchronize() = 0;
    virtual ~ITextureSet() = default;
};

class IContext
{
public:
    virtual Status CreateCompressedTextureSetFromMemory(void const* pData, size_t size, TextureSetFeatures const& features,
        ITextureSet** pOutTextureSet) const = 0;
    virtual Status CreateCompressedTextureSetFromFile(char const* fileName, TextureSetFeatures const& features,
        ITextureSet** pOutTextureSet) const = 0;
    virtual void DestroyTextureSet(ITextureSet* textureSet) const = 0;
    virtual ~IContext() = default;
};

Status CreateContext(IContext** pOutContext, ContextParameters const& params);
void DestroyContext(IContext* context);
inline const char* GetLastErrorMessage() { return ntcb_last_error(); }
inline const char* StatusToString(Status status) { return ntcb_status_string(status); }

} // namespace ntcb
