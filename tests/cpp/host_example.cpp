// A client of the C++ host interface (include/ntcb_host.h), written the way a client of the
// reference's ntc::IContext / ntc::ITextureSet is written: create a context, load a container,
// decompress, read mip 0 back as fp16, block-compress one channel as BC4 on the device.
// Prints "texels <FNV-1a of the fp16 bytes> bc4 <FNV-1a of the blocks>"; the test compares the
// digests with what the Python binding produces for the same container.
//
// usage: host_example <container file>     exit code 2: no usable GPU (message on stderr)
#include "ntcb_host.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <vector>

static uint64_t Fnv1a(const void* data, size_t bytes)
{
    uint64_t hash = 1469598103934665603ull;
    const unsigned char* p = static_cast<const unsigned char*>(data);
    for (size_t i = 0; i < bytes; ++i)
        hash = (hash ^ p[i]) * 1099511628211ull;
    return hash;
}

#define CHECK(call)                                                                        \
    do                                                                                     \
    {                                                                                      \
        const ntcb::Status checkedStatus = (call);                                         \
        if (checkedStatus != NTCB_OK)                                                      \
        {                                                                                  \
            std::fprintf(stderr, "%s: %s (%s)\n", #call, ntcb::StatusToString(checkedStatus), \
                ntcb::GetLastErrorMessage());                                              \
            return 1;                                                                      \
        }                                                                                  \
    } while (0)

int main(int argc, char** argv)
{
    if (argc < 2)
    {
        std::fprintf(stderr, "usage: host_example <container file>\n");
        return 1;
    }
    ntcb::ContextParameters contextParams;
    contextParams.cudaDevice = 0;
    ntcb::IContext* context = nullptr;
    const ntcb::Status created = ntcb::CreateContext(&context, contextParams);
    if (created != NTCB_OK)
    {
        std::fprintf(stderr, "CreateContext: %s (%s)\n", ntcb::StatusToString(created), ntcb::GetLastErrorMessage());
        return 2;
    }

    ntcb::TextureSetFeatures features = {};
    features.outputLayout = NTCB_LAYOUT_INTERLEAVED;
    features.numerics = NTCB_NUMERICS_REFERENCE;
    ntcb::ITextureSet* textureSet = nullptr;
    CHECK(context->CreateCompressedTextureSetFromFile(argv[1], features, &textureSet));
    const ntcb::TextureSetDesc& desc = textureSet->GetDesc();

    // the texture headers: which channels form which texture, and the formats their author intended
    for (int i = 0; i < textureSet->GetTextureCount(); ++i)
    {
        NtcbTextureDesc texture;
        CHECK(textureSet->GetTexture(i, texture));
        std::printf("texture %d: %s channels %d+%d bc %d\n", i, texture.name, texture.firstChannel, texture.numChannels,
            texture.blockCompressedFormat);
    }

    ntcb::DecompressionStats stats = {};
    CHECK(textureSet->Decompress(&stats, /*useInt8Weights*/ false));

    std::vector<uint16_t> texels(size_t(desc.width) * desc.height * desc.channels);
    ntcb::ReadChannelsParameters read = {};
    read.mipLevel = 0;
    read.firstChannel = 0;
    read.numChannels = desc.channels;
    read.addressSpace = NTCB_ADDRESS_SPACE_HOST;
    read.pOutData = texels.data();
    read.width = desc.width;
    read.height = desc.height;
    read.channelFormat = NTCB_CHANNEL_FORMAT_FLOAT16;
    read.pixelStride = size_t(desc.channels) * 2;
    read.rowPitch = read.pixelStride * desc.width;
    CHECK(textureSet->ReadChannels(read));

    const int blocksX = (desc.width + 3) / 4, blocksY = (desc.height + 3) / 4;
    std::vector<unsigned char> blocks(size_t(blocksX) * blocksY * 8);
    void* deviceBlocks = nullptr;
    if (cudaMalloc(&deviceBlocks, blocks.size()) != cudaSuccess)
        return 1;
    CHECK(textureSet->BlockCompress(0, /*firstChannel*/ 0, /*numChannels*/ 0, NTCB_BLOCK_FORMAT_BC4, 0.f, deviceBlocks,
        size_t(blocksX) * 8));
    CHECK(textureSet->Synchronize());
    if (cudaMemcpy(blocks.data(), deviceBlocks, blocks.size(), cudaMemcpyDeviceToHost) != cudaSuccess)
        return 1;
    cudaFree(deviceBlocks);

    // the texture whose header names BC7, by its stored mode bitmap when the file carries one
    // (ITextureMetadata::GetBC7ModeBuffer + BlockCompressionModeBufferSource::TextureSet)
    std::vector<unsigned char> blocks7(size_t(blocksX) * blocksY * 16);
    void const* modes = nullptr;
    size_t modeBytes = 0;
    CHECK(textureSet->GetBC7ModeBuffer(1, 0, &modes, &modeBytes));
    void* deviceBlocks7 = nullptr;
    if (cudaMalloc(&deviceBlocks7, blocks7.size()) != cudaSuccess)
        return 1;
    CHECK(textureSet->BlockCompressTexture(1, 0, 1.f / 255.f, deviceBlocks7, size_t(blocksX) * 16));
    CHECK(textureSet->Synchronize());
    if (cudaMemcpy(blocks7.data(), deviceBlocks7, blocks7.size(), cudaMemcpyDeviceToHost) != cudaSuccess)
        return 1;
    cudaFree(deviceBlocks7);

    // ITextureSet::LoadFromMemory: the same file again into the same buffers; the decode must not change
    std::vector<unsigned char> file;
    if (std::FILE* handle = std::fopen(argv[1], "rb"))
    {
        unsigned char chunk[4096];
        size_t got;
        while ((got = std::fread(chunk, 1, sizeof chunk, handle)) > 0)
            file.insert(file.end(), chunk, chunk + got);
        std::fclose(handle);
    }
    CHECK(textureSet->LoadFromMemory(file.data(), file.size()));
    CHECK(textureSet->Decompress(nullptr, /*useInt8Weights*/ false));
    std::vector<uint16_t> again(texels.size());
    read.pOutData = again.data();
    CHECK(textureSet->ReadChannels(read));
    // ITextureSet::Sample: one query at the centre of every texel of mip 0, in row order, must give mip 0 back
    const size_t numQueries = size_t(desc.width) * desc.height;
    std::vector<float> queries(numQueries * 3);
    for (int y = 0; y < desc.height; ++y)
        for (int x = 0; x < desc.width; ++x)
        {
            float* query = &queries[(size_t(y) * desc.width + x) * 3];
            query[0] = (float(x) + 0.5f) / float(desc.width);
            query[1] = (float(y) + 0.5f) / float(desc.height);
            query[2] = 0.25f;
        }
    float* deviceQueries = nullptr;
    void* deviceAnswers = nullptr;
    if (cudaMalloc(&deviceQueries, queries.size() * sizeof(float)) != cudaSuccess ||
        cudaMalloc(&deviceAnswers, texels.size() * 2) != cudaSuccess ||
        cudaMemcpy(deviceQueries, queries.data(), queries.size() * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess)
        return 1;
    CHECK(textureSet->Sample(deviceQueries, numQueries, deviceAnswers, /*useInt8Weights*/ false));
    std::vector<uint16_t> answers(texels.size());
    if (cudaMemcpy(answers.data(), deviceAnswers, answers.size() * 2, cudaMemcpyDeviceToHost) != cudaSuccess)
        return 1;
    cudaFree(deviceQueries);
    cudaFree(deviceAnswers);

    std::printf("bc7 %016llx mode_bytes %zu reloaded %s sampled %s\n", static_cast<unsigned long long>(Fnv1a(blocks7.data(), blocks7.size())),
        modeBytes, again == texels ? "same" : "DIFFERENT", answers == texels ? "same" : "DIFFERENT");

    std::printf("texels %016llx bc4 %016llx size %dx%dx%d mips %d gpu_ms %.4f\n",
        static_cast<unsigned long long>(Fnv1a(texels.data(), texels.size() * 2)),
        static_cast<unsigned long long>(Fnv1a(blocks.data(), blocks.size())), desc.width, desc.height, desc.channels, desc.mips,
        stats.gpuTimeMilliseconds);
    context->DestroyTextureSet(textureSet);
    ntcb::DestroyContext(context);
    return 0;
}
