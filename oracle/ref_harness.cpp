// TEST INFRASTRUCTURE ONLY (never linked into the product library).
//
// A plain-C driver around the UNMODIFIED reference library (LibNTC built from its own sources by
// build_ref.sh).  It lets the parity tests and the benchmark's reference arm run the reference's
// own CUDA decompression through the reference's own public API:
//   ntc::CreateContext                              include/libntc/ntc.h:1330
//   IContext::CreateCompressedTextureSetFromMemory  include/libntc/ntc.h:1171
//   ITextureSet::Decompress                         include/libntc/ntc.h:933
//   ITextureSet::ReadChannels                       include/libntc/ntc.h:902
// Nothing here re-implements any part of the decoder.

#include <libntc/ntc.h>
#include <cstdio>
#include <cstring>
#include <new>

namespace
{
struct RefHandle
{
    ntc::IContext* context = nullptr;
    ntc::ITextureSet* textureSet = nullptr;
};

thread_local char g_error[1200];

void SetError(char const* where, ntc::Status status)
{
    std::snprintf(g_error, sizeof g_error, "%s: %s (%s)", where, ntc::StatusToString(status),
        ntc::GetLastErrorMessage());
}
} // namespace

extern "C"
{

char const* ntcref_last_error()
{
    return g_error;
}

// Creates a reference context on `device` and loads a compressed texture set from an NTC
// container held in host memory.  `stagingBytesPerPixel` sizes the reference's staging buffer and
// bounds the widest ReadChannels call (channels * 2 for fp16).  Returns 0 on success.
int ntcref_open(void const* fileData, size_t fileSize, int device, int stagingBytesPerPixel, void** outHandle)
{
    g_error[0] = 0;
    *outHandle = nullptr;
    RefHandle* handle = new (std::nothrow) RefHandle();
    if (!handle)
        return -1;

    ntc::ContextParameters contextParams;
    contextParams.cudaDevice = device;
    contextParams.graphicsApi = ntc::GraphicsAPI::None;
    contextParams.enableCooperativeVector = false;
    ntc::Status status = ntc::CreateContext(&handle->context, contextParams);
    if (status != ntc::Status::Ok)
    {
        SetError("CreateContext", status);
        if (handle->context)
            ntc::DestroyContext(handle->context);
        delete handle;
        return int(status);
    }

    ntc::TextureSetFeatures features;
    features.stagingBytesPerPixel = stagingBytesPerPixel;
    features.enableCompression = false;
    features.separateRefOutData = false;
    status = handle->context->CreateCompressedTextureSetFromMemory(fileData, fileSize, features,
        &handle->textureSet);
    if (status != ntc::Status::Ok)
    {
        SetError("CreateCompressedTextureSetFromMemory", status);
        ntc::DestroyContext(handle->context);
        delete handle;
        return int(status);
    }

    *outHandle = handle;
    return 0;
}

// Metadata-only load (works without a GPU): parses the container through the reference's own
// loader and reports what it understood.  Used to validate the synthetic container writer.
// out[0..7] = width, height, channels, mips, gridSizeScale, numFeatures, latent mip count, valid mask
int ntcref_probe_metadata(void const* fileData, size_t fileSize, int* out)
{
    g_error[0] = 0;
    ntc::ContextParameters contextParams;
    contextParams.cudaDevice = ntc::DisableCudaDevice;
    contextParams.enableCooperativeVector = false;
    ntc::IContext* context = nullptr;
    ntc::Status status = ntc::CreateContext(&context, contextParams);
    if (!context)
    {
        SetError("CreateContext", status);
        return int(status);
    }
    ntc::IStream* stream = nullptr;
    status = context->OpenReadOnlyMemory(fileData, fileSize, &stream);
    if (status != ntc::Status::Ok)
    {
        SetError("OpenReadOnlyMemory", status);
        ntc::DestroyContext(context);
        return int(status);
    }
    ntc::ITextureSetMetadata* metadata = nullptr;
    status = context->CreateTextureSetMetadataFromStream(stream, &metadata);
    if (status != ntc::Status::Ok)
    {
        SetError("CreateTextureSetMetadataFromStream", status);
        context->CloseMemory(stream);
        ntc::DestroyContext(context);
        return int(status);
    }
    ntc::TextureSetDesc const& desc = metadata->GetDesc();
    ntc::LatentShape const& shape = metadata->GetLatentShape();
    out[0] = desc.width;
    out[1] = desc.height;
    out[2] = desc.channels;
    out[3] = desc.mips;
    out[4] = shape.gridSizeScale;
    out[5] = shape.numFeatures;
    out[6] = metadata->GetLatentTextureDesc().mipLevels;
    out[7] = int(metadata->GetValidChannelMask());
    context->DestroyTextureSetMetadata(metadata);
    context->CloseMemory(stream);
    ntc::DestroyContext(context);
    return 0;
}

// Metadata-only: where the reference's loader finds the BC7 mode bitmap of a texture's mip level
// (ITextureMetadata::GetBC7ModeBufferFootprint).  out[0..2] = offset in the stream, stored size, compression type.
int ntcref_probe_mode_buffer_footprint(void const* fileData, size_t fileSize, int textureIndex, int mipLevel, uint64_t* out)
{
    g_error[0] = 0;
    ntc::ContextParameters contextParams;
    contextParams.cudaDevice = ntc::DisableCudaDevice;
    contextParams.enableCooperativeVector = false;
    ntc::IContext* context = nullptr;
    ntc::Status status = ntc::CreateContext(&context, contextParams);
    if (!context)
    {
        SetError("CreateContext", status);
        return int(status);
    }
    ntc::IStream* stream = nullptr;
    status = context->OpenReadOnlyMemory(fileData, fileSize, &stream);
    if (status != ntc::Status::Ok)
    {
        SetError("OpenReadOnlyMemory", status);
        ntc::DestroyContext(context);
        return int(status);
    }
    ntc::ITextureSetMetadata* metadata = nullptr;
    status = context->CreateTextureSetMetadataFromStream(stream, &metadata);
    if (status != ntc::Status::Ok)
    {
        SetError("CreateTextureSetMetadataFromStream", status);
        context->CloseMemory(stream);
        ntc::DestroyContext(context);
        return int(status);
    }
    int result = 0;
    if (textureIndex < 0 || textureIndex >= metadata->GetTextureCount())
        result = int(ntc::Status::OutOfRange);
    else
    {
        ntc::BufferFootprint const footprint = metadata->GetTexture(textureIndex)->GetBC7ModeBufferFootprint(mipLevel);
        out[0] = footprint.rangeInStream.offset;
        out[1] = footprint.rangeInStream.size;
        out[2] = uint64_t(footprint.compressionType);
    }
    context->DestroyTextureSetMetadata(metadata);
    context->CloseMemory(stream);
    ntc::DestroyContext(context);
    return result;
}

// Runs the reference's CUDA decompression of every mip.  `gpuMilliseconds` receives the
// reference's own timing of its mip loop (DecompressionStats::gpuTimeMilliseconds).
int ntcref_decompress(void* opaque, int useInt8Weights, float* gpuMilliseconds)
{
    g_error[0] = 0;
    RefHandle* handle = static_cast<RefHandle*>(opaque);
    ntc::DecompressionStats stats;
    ntc::Status status = handle->textureSet->Decompress(&stats, useInt8Weights != 0);
    if (status != ntc::Status::Ok)
    {
        SetError("Decompress", status);
        return int(status);
    }
    if (gpuMilliseconds)
        *gpuMilliseconds = stats.gpuTimeMilliseconds;
    return 0;
}

// Copies `numChannels` decoded fp16 channels of one mip, interleaved per pixel
// ([y][x][channel], row pitch = width * numChannels * 2 bytes), into host (toDevice == 0) or
// device (toDevice != 0) memory.
int ntcref_read_mip(void* opaque, int mipLevel, int firstChannel, int numChannels, int width, int height,
    void* destination, int toDevice)
{
    g_error[0] = 0;
    RefHandle* handle = static_cast<RefHandle*>(opaque);
    ntc::ReadChannelsParameters params;
    params.page = ntc::TextureDataPage::Output;
    params.mipLevel = mipLevel;
    params.firstChannel = firstChannel;
    params.numChannels = numChannels;
    params.pOutData = static_cast<unsigned char*>(destination);
    params.addressSpace = toDevice ? ntc::AddressSpace::Device : ntc::AddressSpace::Host;
    params.width = width;
    params.height = height;
    params.pixelStride = size_t(numChannels) * 2;
    params.rowPitch = size_t(width) * size_t(numChannels) * 2;
    params.channelFormat = ntc::ChannelFormat::FLOAT16;
    params.dstColorSpaces = nullptr;
    params.useDithering = false;
    ntc::Status status = handle->textureSet->ReadChannels(params);
    if (status != ntc::Status::Ok)
    {
        SetError("ReadChannels", status);
        return int(status);
    }
    return 0;
}

// The general form of ITextureSet::ReadChannels on the decoded page: any channel format
// (ntc::ChannelFormat value), strides, destination colour spaces (ntc::ColorSpace values, one per
// channel, or NULL for Linear) and dithering; host destination.
int ntcref_read_channels(void* opaque, int mipLevel, int firstChannel, int numChannels, int width, int height,
    int channelFormat, size_t pixelStride, size_t rowPitch, const int* dstColorSpaces, int useDithering, void* destination)
{
    g_error[0] = 0;
    RefHandle* handle = static_cast<RefHandle*>(opaque);
    ntc::ColorSpace spaces[NTC_MAX_CHANNELS] = {};
    for (int i = 0; i < numChannels && i < NTC_MAX_CHANNELS && dstColorSpaces; ++i)
        spaces[i] = ntc::ColorSpace(dstColorSpaces[i]);
    ntc::ReadChannelsParameters params;
    params.page = ntc::TextureDataPage::Output;
    params.mipLevel = mipLevel;
    params.firstChannel = firstChannel;
    params.numChannels = numChannels;
    params.pOutData = static_cast<unsigned char*>(destination);
    params.addressSpace = ntc::AddressSpace::Host;
    params.width = width;
    params.height = height;
    params.pixelStride = pixelStride;
    params.rowPitch = rowPitch;
    params.channelFormat = ntc::ChannelFormat(channelFormat);
    params.dstColorSpaces = dstColorSpaces ? spaces : nullptr;
    params.useDithering = useDithering != 0;
    ntc::Status status = handle->textureSet->ReadChannels(params);
    if (status != ntc::Status::Ok)
    {
        SetError("ReadChannels", status);
        return int(status);
    }
    return 0;
}

void ntcref_close(void* opaque)
{
    RefHandle* handle = static_cast<RefHandle*>(opaque);
    if (!handle)
        return;
    if (handle->textureSet)
        handle->context->DestroyTextureSet(handle->textureSet);
    if (handle->context)
        ntc::DestroyContext(handle->context);
    delete handle;
}

// ntc::GetBC7ModeBufferSize / ntc::MakeBC7ModeBuffer (host functions; the mode buffer must arrive zeroed, as
// the reference's own caller hands it over: src/TextureMetadata.cpp:125-129).
size_t ntcref_bc7_mode_buffer_size(int widthInBlocks, int heightInBlocks)
{
    return ntc::GetBC7ModeBufferSize(widthInBlocks, heightInBlocks);
}

int ntcref_make_bc7_mode_buffer(int widthInBlocks, int heightInBlocks, void const* blockData, size_t blockDataSize,
    size_t rowPitch, void* modeBuffer, size_t modeBufferSize)
{
    ntc::Status const status = ntc::MakeBC7ModeBuffer(widthInBlocks, heightInBlocks, blockData, blockDataSize, rowPitch,
        modeBuffer, modeBufferSize);
    if (status != ntc::Status::Ok)
        SetError("MakeBC7ModeBuffer", status);
    return int(status);
}

} // extern "C"
