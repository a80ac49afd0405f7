// Reader of NTC containers ("NTEX" header + JSON document + binary chunk) for the decode path, and
// the texture-set geometry the decoder needs.  Host only.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace ntcb
{

constexpr int kMaxMips = 16;
constexpr int kMaxChannels = 16;
constexpr int kMaxNeuralMips = 8;
constexpr size_t kInt8BlobBytes = 9472;
constexpr size_t kFp8BlobBytes = 8608;

// Geometry of a texture set; the rules are the reference's
// (src/FeatureGridMath.cpp:47-76, src/FeatureGridHost.cpp:27-52, src/TextureSet.cpp:88-101,450-463).
struct SetGeometry
{
    int width = 0, height = 0, channels = 0, mips = 0; // channels rounded up to even
    int gridSizeScale = 0, numFeatures = 0;
    int numLayers = 0, numNeuralMips = 0;
    int latentWidth[kMaxNeuralMips] = {}, latentHeight[kMaxNeuralMips] = {};
    uint64_t latentPixelOffset[kMaxNeuralMips + 1] = {}; // per-layer pixels, cumulative
    int mipWidth[kMaxMips] = {}, mipHeight[kMaxMips] = {}, neuralLod[kMaxMips] = {};
    float positionScale[kMaxMips] = {}, positionLod[kMaxMips] = {};
    uint64_t mipTexelOffset[kMaxMips + 1] = {};

    uint64_t TotalLatentPixels() const { return latentPixelOffset[numNeuralMips]; }
    uint64_t TotalTexels() const { return mipTexelOffset[mips]; }
};

int LodToNeuralLod(int lod, int gridSizeScale, int neuralLods);
int GridDimension(int imageDimension, int neuralLod, int gridSizeScale);

// Fills `out` from the description; returns an NtcbStatus (OutOfRange for invalid descriptions,
// with the reference's messages).
int MakeGeometry(int width, int height, int channels, int mips, int gridSizeScale, int numFeatures, SetGeometry& out);

// One texture of the set: a named range of channels with the formats its author intended for it
// (json::Texture, src/JsonFileFormat.h:124-139; defaults as TextureSetMetadata::LoadMetadataFromStream
// applies them, src/TextureSetMetadata.cpp:460-468).
struct LoadedTexture
{
    std::string name;
    int firstChannel = 0, numChannels = 0;
    int channelFormat = 1;         // ntc::ChannelFormat, default UNORM8
    int blockCompressedFormat = 0; // ntc::BlockCompressedFormat, default None
    int rgbColorSpace = 0, alphaColorSpace = 0; // ntc::ColorSpace, default Linear
    // BC7 mode bitmaps stored with the texture (json::Texture::bcModeBuffers), one per mip level, empty where
    // the file has none (TextureMetadata::SetBC7ModeBufferFootprint / LoadBC7ModeBuffers,
    // src/TextureMetadata.cpp:154-224)
    std::vector<std::vector<uint8_t>> modeBuffers;
    std::vector<uint8_t> modeBufferCompressed; // per mip: 1 = stored with GDeflate compression, which is not read
    std::vector<uint64_t> modeBufferOffset, modeBufferStoredSize; // per mip: where the file keeps it (0, 0: nowhere)
};

struct LoadedSet
{
    SetGeometry geometry;
    // BGRA4 latent pixels in device order: for each neural mip, for each layer, rows of pixels
    std::vector<uint16_t> latents;
    std::vector<uint8_t> int8Blob; // GenericInt8, empty when the file has no Int8 network
    std::vector<uint8_t> fp8Blob;  // GenericFP8, empty when the file has no FloatE4M3 network
    int channelColorSpaces[kMaxChannels] = {}; // ntc::ColorSpace each channel is stored in (0 Linear, 1 sRGB, 2 HLG)
    std::vector<LoadedTexture> textures;
};

// Parses a container held in memory.  Returns an NtcbStatus and sets the thread-local error
// message; mirrors the checks of TextureSetMetadata::LoadFileHeadersFromStream
// (src/TextureSetMetadata.cpp:1210-1264), LoadMetadataFromStream (:434-581), LoadWeightsFromStream
// (:676-784) and TextureSet::LoadFromStreamPostHeader (src/TextureSet.cpp:154-294).
int LoadContainer(const void* data, size_t size, LoadedSet& out);

} // namespace ntcb
