// Host objects of the decoder: a context bound to one CUDA device and texture sets that own the
// device buffers of one compressed set (packed latents, the two staged networks, the decoded
// texels).  They implement the C++ interface of include/ntcb_host.h and the texture-set level of
// the C ABI in include/ntcb.h, following the reference's host driver for this path
// (src/PublicFunctions.cpp:62-162, src/Context.cpp:295-366, src/TextureSet.cpp:81-152, 154-294,
// 915-985, 1664-1897).

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include "container.h"
#include "decode_kernel.h"
#include "error.h"
#include "ntcb.h"
#include "ntcb_host.h"
#include "output_convert.cuh"
#include "read_channels.h"

namespace ntcb
{
namespace
{

// Sets and restores the calling thread's current device around an API call, like the reference's
// CudaDeviceGuard (src/CudaDeviceGuard.cpp:21-61).
class DeviceGuard
{
public:
    explicit DeviceGuard(int device)
    {
        m_ok = cudaGetDevice(&m_previous) == cudaSuccess;
        if (m_ok && m_previous != device)
        {
            cudaError_t err = cudaSetDevice(device);
            if (err != cudaSuccess)
            {
                CudaFailure("cudaSetDevice", err);
                m_ok = false;
            }
            else
                m_switched = true;
        }
        else if (!m_ok)
            SetError("Call to cudaGetDevice failed.");
    }
    ~DeviceGuard()
    {
        if (m_switched)
            cudaSetDevice(m_previous);
    }
    bool Success() const { return m_ok; }

private:
    int m_previous = 0;
    bool m_ok = false, m_switched = false;
};

class Context;

class TextureSet final : public ITextureSet
{
public:
    TextureSet(const Context* context, int device, cudaStream_t stream) : m_context(context), m_device(device), m_stream(stream) {}
    ~TextureSet() override { Release(); }

    Status Initialize(LoadedSet&& loaded, const TextureSetFeatures& features);
    void Release();

    TextureSetDesc const& GetDesc() const override { return m_desc; }
    LatentShape const& GetLatentShape() const override { return m_latentShape; }
    Status Decompress(DecompressionStats* pOutStats, bool useInt8Weights) override
    {
        return DecompressRows(nullptr, pOutStats, useInt8Weights);
    }
    Status DecompressRows(const int32_t* rowRanges, DecompressionStats* pOutStats, bool useInt8Weights) override;
    Status DecompressConverted(DecompressionStats* pOutStats, bool useInt8Weights, NtcbOutputConversion const& conversion,
        int addressSpace, void* destination, size_t destinationBytes) override;
    Status ReadChannels(ReadChannelsParameters const& params) override;
    int GetTextureCount() const override { return int(m_textures.size()); }
    Status GetTexture(int index, NtcbTextureDesc& outTexture) const override;
    Status GetDeviceMip(int mipLevel, void** outPointer, size_t* outBytes) override;
    Status BlockCompress(int mipLevel, int firstChannel, int numChannels, int format, float alphaThreshold,
        void* deviceBlocks, size_t rowPitch) override;
    Status GetBC7ModeBuffer(int textureIndex, int mipLevel, void const** outData, size_t* outSize) const override;
    Status MakeAndStoreBC7ModeBuffer(int textureIndex, int mipLevel, int widthInBlocks, int heightInBlocks,
        void const* blockData, size_t blockDataSize, size_t rowPitch) override;
    Status BlockCompressTexture(int textureIndex, int mipLevel, float alphaThreshold, void* deviceBlocks, size_t rowPitch) override;
    Status LoadFromMemory(void const* pData, size_t size) override;
    Status Sample(float const* deviceQueries, uint64_t numQueries, void* deviceOut, bool useInt8Weights) override;
    Status Synchronize() override;

    const SetGeometry& Geometry() const { return m_geometry; }

private:
    Status CheckKernelStatus();
    Status CheckTextureAndMip(int textureIndex, int mipLevel) const;
    Status FillUpload(const LoadedSet& loaded);
    Status GrowStaging(size_t bytes);
    Status CopyBands(const uint8_t* deviceMip0, uint8_t* host, size_t rowBytes);
    Status DecodeInto(const int32_t* rowRanges, DecompressionStats* pOutStats, bool useInt8Weights,
        const NtcbOutputConversion* conversion, void* deviceOut);

    const Context* m_context;
    int m_device;
    cudaStream_t m_stream;
    SetGeometry m_geometry;
    TextureSetDesc m_desc;
    LatentShape m_latentShape;
    int m_layout = NTCB_LAYOUT_INTERLEAVED;
    int m_numerics = NTCB_NUMERICS_EXACT;
    size_t m_networkBytes = 0; // size of one staged network image (depends on the numerics)
    bool m_hasInt8 = false, m_hasFp8 = false;

    // pinned host image of everything Decompress uploads: latents, then the two staged networks
    uint8_t* m_hostUpload = nullptr;
    uint8_t* m_deviceUpload = nullptr;
    size_t m_uploadBytes = 0, m_latentBytes = 0;
    __half* m_texels = nullptr;
    size_t m_texelBytes = 0;
    uint32_t* m_status = nullptr;
    uint32_t* m_hostStatus = nullptr; // pinned
    int m_channelColorSpaces[kMaxChannels] = {}; // ntc::ColorSpace each channel is stored in (from the container)
    std::vector<LoadedTexture> m_textures;
    std::vector<std::vector<void*>> m_deviceModeBuffers; // [texture][mip]: device copies of the BC7 mode bitmaps, made on first use
    uint8_t* m_staging = nullptr;     // grown on demand by ReadChannels to host with padded strides
    size_t m_stagingBytes = 0;
    // Inference on sample keeps the compressed data resident: whether m_deviceUpload holds what m_hostUpload holds
    // (as far as the work queued on m_stream is concerned), and the pixel-major copy of the latents made from it
    bool m_deviceCurrent = false, m_pixelMajorCurrent = false;
    uint16_t* m_pixelMajor = nullptr;
    cudaEvent_t m_eventStart = nullptr, m_eventStop = nullptr;
    bool m_decoded = false;

    // A whole-set decode of a large set is issued as kBands launches over row bands of mip 0 plus one
    // for the other mips, so that a host read of mip 0 can start copying the first band while the
    // rest is still being decoded (the read-back, not the decode, bounds Decompress + ReadChannels).
    static constexpr int kBands = 4;
    static constexpr int kBandMinRows = 512;
    cudaStream_t m_copyStream = nullptr;
    cudaEvent_t m_bandEvents[kBands + 1] = {}; // [b]: band b of mip 0 decoded; [kBands]: everything decoded
    int m_bandEnd[kBands] = {};                // last row + 1 of each band
    int m_bandCount = 0;                       // 0: the last decode was a single launch
};

class Context final : public IContext
{
public:
    explicit Context(int device) : m_device(device) {}
    ~Context() override
    {
        if (m_stream)
        {
            DeviceGuard guard(m_device);
            cudaStreamDestroy(m_stream);
        }
    }

    Status Initialize()
    {
        int count = 0;
        cudaError_t err = cudaGetDeviceCount(&count);
        if (err != cudaSuccess)
            return CudaFailure("cudaGetDeviceCount", err);
        if (m_device < 0 || m_device >= count)
        {
            SetError("CUDA device %d does not exist (%d devices are visible).", m_device, count);
            return NTCB_ERR_CUDA;
        }
        int major = 0;
        err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, m_device);
        if (err != cudaSuccess)
            return CudaFailure("cudaDeviceGetAttribute", err);
        if (major != 10)
        {
            SetError("CUDA device %d has compute capability %d.x; the decoder needs 10.x (tcgen05, tensor memory).", m_device,
                major);
            return NTCB_ERR_CUDA;
        }
        DeviceGuard guard(m_device);
        if (!guard.Success())
            return NTCB_ERR_CUDA;
        err = cudaStreamCreateWithFlags(&m_stream, cudaStreamNonBlocking);
        if (err != cudaSuccess)
            return CudaFailure("cudaStreamCreateWithFlags", err);
        ClearError();
        return NTCB_OK;
    }

    Status CreateCompressedTextureSetFromMemory(void const* pData, size_t size, TextureSetFeatures const& features,
        ITextureSet** pOutTextureSet) const override
    {
        if (!pOutTextureSet)
        {
            SetError("pOutTextureSet is NULL.");
            return NTCB_ERR_INVALID_ARGUMENT;
        }
        *pOutTextureSet = nullptr;
        LoadedSet loaded;
        Status status = LoadContainer(pData, size, loaded);
        if (status != NTCB_OK)
            return status;
        DeviceGuard guard(m_device);
        if (!guard.Success())
            return NTCB_ERR_CUDA;
        TextureSet* set = new (std::nothrow) TextureSet(this, m_device, m_stream);
        if (!set)
        {
            SetError("Out of host memory.");
            return NTCB_ERR_OUT_OF_MEMORY;
        }
        status = set->Initialize(std::move(loaded), features);
        if (status != NTCB_OK)
        {
            delete set;
            return status;
        }
        *pOutTextureSet = set;
        ClearError();
        return NTCB_OK;
    }

    Status CreateCompressedTextureSetFromFile(char const* fileName, TextureSetFeatures const& features,
        ITextureSet** pOutTextureSet) const override
    {
        if (!fileName)
        {
            SetError("fileName is NULL.");
            return NTCB_ERR_INVALID_ARGUMENT;
        }
        FILE* file = fopen(fileName, "rb");
        if (!file)
        {
            SetError("Cannot open file '%s'.", fileName);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        std::vector<uint8_t> data;
        bool ok = fseek(file, 0, SEEK_END) == 0;
        long length = ok ? ftell(file) : -1;
        ok = ok && length >= 0 && fseek(file, 0, SEEK_SET) == 0;
        if (ok)
        {
            data.resize(size_t(length));
            ok = fread(data.data(), 1, data.size(), file) == data.size();
        }
        fclose(file);
        if (!ok)
        {
            SetError("Cannot read file '%s'.", fileName);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        return CreateCompressedTextureSetFromMemory(data.data(), data.size(), features, pOutTextureSet);
    }

    void DestroyTextureSet(ITextureSet* textureSet) const override
    {
        if (!textureSet)
            return;
        DeviceGuard guard(m_device);
        delete textureSet;
    }

private:
    int m_device;
    cudaStream_t m_stream = nullptr;
};

Status TextureSet::Initialize(LoadedSet&& loaded, const TextureSetFeatures& features)
{
    m_geometry = loaded.geometry;
    m_desc.width = m_geometry.width;
    m_desc.height = m_geometry.height;
    m_desc.channels = m_geometry.channels;
    m_desc.mips = m_geometry.mips;
    m_latentShape.gridSizeScale = m_geometry.gridSizeScale;
    m_latentShape.numFeatures = m_geometry.numFeatures;
    if (features.outputLayout != NTCB_LAYOUT_PLANAR_PAIRS && features.outputLayout != NTCB_LAYOUT_INTERLEAVED)
    {
        SetError("Unknown output layout %d.", features.outputLayout);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    m_layout = features.outputLayout;
    if (features.numerics != NTCB_NUMERICS_EXACT && features.numerics != NTCB_NUMERICS_REFERENCE)
    {
        SetError("Unknown numerics %d.", features.numerics);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    m_numerics = features.numerics;
    m_networkBytes = m_numerics == NTCB_NUMERICS_REFERENCE ? size_t(kRefNetworkBytes) : size_t(kStagedNetworkBytes);

    // upload image: latents (padded to 16 bytes), then the Int8 and the FP8 network images
    m_latentBytes = (loaded.latents.size() * 2 + 15) & ~size_t(15);
    m_uploadBytes = m_latentBytes + 2 * m_networkBytes;
    cudaError_t err = cudaHostAlloc(reinterpret_cast<void**>(&m_hostUpload), m_uploadBytes, cudaHostAllocDefault);
    if (err != cudaSuccess)
    {
        SetError("Failed to allocate %zu bytes of pinned host memory for the compressed data.", m_uploadBytes);
        return NTCB_ERR_OUT_OF_MEMORY;
    }
    Status filled = FillUpload(loaded);
    if (filled != NTCB_OK)
        return filled;

    err = cudaMalloc(reinterpret_cast<void**>(&m_deviceUpload), m_uploadBytes);
    if (err != cudaSuccess)
    {
        SetError("Failed to allocate %zu bytes of device memory for the compressed data.", m_uploadBytes);
        return NTCB_ERR_OUT_OF_MEMORY;
    }
    m_texelBytes = size_t(m_geometry.TotalTexels()) * m_geometry.channels * sizeof(__half);
    err = cudaMalloc(reinterpret_cast<void**>(&m_texels), m_texelBytes);
    if (err != cudaSuccess)
    {
        SetError("Failed to allocate %zu bytes of device memory for the decoded texture data.", m_texelBytes);
        return NTCB_ERR_OUT_OF_MEMORY;
    }
    err = cudaMalloc(reinterpret_cast<void**>(&m_status), NTCB_STATUS_WORDS * sizeof(uint32_t));
    if (err == cudaSuccess)
        err = cudaHostAlloc(reinterpret_cast<void**>(&m_hostStatus), NTCB_STATUS_WORDS * sizeof(uint32_t), cudaHostAllocDefault);
    if (err != cudaSuccess)
    {
        SetError("Failed to allocate the status words.");
        return NTCB_ERR_OUT_OF_MEMORY;
    }
    err = cudaEventCreate(&m_eventStart);
    if (err == cudaSuccess)
        err = cudaEventCreate(&m_eventStop);
    for (int b = 0; b <= kBands && err == cudaSuccess; ++b)
        err = cudaEventCreateWithFlags(&m_bandEvents[b], cudaEventDisableTiming);
    if (err != cudaSuccess)
        return CudaFailure("cudaEventCreate", err);
    err = cudaStreamCreateWithFlags(&m_copyStream, cudaStreamNonBlocking);
    if (err != cudaSuccess)
        return CudaFailure("cudaStreamCreateWithFlags", err);
    return NTCB_OK;
}

// What a container brings besides its shape: latents and staged networks into the pinned upload image,
// channel colour spaces, texture headers with their BC7 mode bitmaps.
Status TextureSet::FillUpload(const LoadedSet& loaded)
{
    for (int c = 0; c < kMaxChannels; ++c)
        m_channelColorSpaces[c] = loaded.channelColorSpaces[c];
    for (std::vector<void*>& perMip : m_deviceModeBuffers)
        for (void*& copy : perMip)
        {
            if (copy) cudaFree(copy);
            copy = nullptr;
        }
    m_textures = loaded.textures;
    m_deviceModeBuffers.assign(m_textures.size(), std::vector<void*>(size_t(m_geometry.mips), nullptr));
    m_hasInt8 = !loaded.int8Blob.empty();
    m_hasFp8 = !loaded.fp8Blob.empty();
    memset(m_hostUpload, 0, m_uploadBytes);
    memcpy(m_hostUpload, loaded.latents.data(), loaded.latents.size() * 2);
    auto stage = m_numerics == NTCB_NUMERICS_REFERENCE ? ntcb_stage_network_reference : ntcb_stage_network;
    if (m_hasInt8)
    {
        Status status = stage(loaded.int8Blob.data(), loaded.int8Blob.size(), NTCB_WEIGHTS_INT8, m_hostUpload + m_latentBytes);
        if (status != NTCB_OK)
            return status;
    }
    if (m_hasFp8)
    {
        Status status = stage(loaded.fp8Blob.data(), loaded.fp8Blob.size(), NTCB_WEIGHTS_FP8,
            m_hostUpload + m_latentBytes + m_networkBytes);
        if (status != NTCB_OK)
            return status;
    }
    return NTCB_OK;
}

// ITextureSet::LoadFromMemory (include/libntc/ntc.h:869-881): another compressed set of the same dimensions
// into this one's buffers.
Status TextureSet::LoadFromMemory(void const* pData, size_t size)
{
    LoadedSet loaded;
    Status status = LoadContainer(pData, size, loaded);
    if (status != NTCB_OK)
        return status;
    const SetGeometry& theirs = loaded.geometry;
    if (theirs.width != m_geometry.width || theirs.height != m_geometry.height || theirs.channels != m_geometry.channels
        || theirs.mips != m_geometry.mips || theirs.gridSizeScale != m_geometry.gridSizeScale || theirs.numFeatures != m_geometry.numFeatures)
    {
        SetError("The file holds a %dx%d set of %d channels and %d mips with latent shape {%d, %d}; this texture set is %dx%d, %d "
                 "channels, %d mips, {%d, %d}.", theirs.width, theirs.height, theirs.channels, theirs.mips, theirs.gridSizeScale,
            theirs.numFeatures, m_geometry.width, m_geometry.height, m_geometry.channels, m_geometry.mips, m_geometry.gridSizeScale,
            m_geometry.numFeatures);
        return NTCB_ERR_FILE_INCOMPATIBLE;
    }
    DeviceGuard guard(m_device);
    if (!guard.Success())
        return NTCB_ERR_CUDA;
    // uploads from the pinned image that are still queued must have read it
    cudaError_t err = cudaStreamSynchronize(m_stream);
    if (err != cudaSuccess)
        return CudaFailure("cudaStreamSynchronize", err);
    m_decoded = false;
    m_deviceCurrent = m_pixelMajorCurrent = false;
    status = FillUpload(loaded);
    if (status != NTCB_OK)
        return status;
    ClearError();
    return NTCB_OK;
}

void TextureSet::Release()
{
    if (m_stream)
        cudaStreamSynchronize(m_stream);
    if (m_copyStream)
    {
        cudaStreamSynchronize(m_copyStream);
        cudaStreamDestroy(m_copyStream);
        m_copyStream = nullptr;
    }
    for (cudaEvent_t& event : m_bandEvents)
    {
        if (event) cudaEventDestroy(event);
        event = nullptr;
    }
    if (m_eventStart) cudaEventDestroy(m_eventStart);
    if (m_eventStop) cudaEventDestroy(m_eventStop);
    for (std::vector<void*>& perMip : m_deviceModeBuffers)
        for (void*& copy : perMip)
        {
            if (copy) cudaFree(copy);
            copy = nullptr;
        }
    if (m_staging) cudaFree(m_staging);
    if (m_pixelMajor) cudaFree(m_pixelMajor);
    m_pixelMajor = nullptr;
    m_deviceCurrent = m_pixelMajorCurrent = false;
    if (m_status) cudaFree(m_status);
    if (m_hostStatus) cudaFreeHost(m_hostStatus);
    if (m_texels) cudaFree(m_texels);
    if (m_deviceUpload) cudaFree(m_deviceUpload);
    if (m_hostUpload) cudaFreeHost(m_hostUpload);
    m_eventStart = m_eventStop = nullptr;
    m_staging = nullptr;
    m_status = nullptr;
    m_hostStatus = nullptr;
    m_texels = nullptr;
    m_deviceUpload = nullptr;
    m_hostUpload = nullptr;
}

Status TextureSet::CheckKernelStatus()
{
    if (m_hostStatus[0] != 0)
    {
        SetError("A bounded wait inside the decode kernel expired (code %u, tile %u, layer %u).", m_hostStatus[0],
            m_hostStatus[1], m_hostStatus[2]);
        return NTCB_ERR_DEVICE_TIMEOUT;
    }
    return NTCB_OK;
}

Status TextureSet::DecompressRows(const int32_t* rowRanges, DecompressionStats* pOutStats, bool useInt8Weights)
{
    Status status = DecodeInto(rowRanges, pOutStats, useInt8Weights, nullptr, m_texels);
    if (status == NTCB_OK)
        m_decoded = true;
    return status;
}

Status TextureSet::DecompressConverted(DecompressionStats* pOutStats, bool useInt8Weights,
    NtcbOutputConversion const& requested, int addressSpace, void* destination, size_t destinationBytes)
{
    if (!destination)
    {
        SetError("destination is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (addressSpace != NTCB_ADDRESS_SPACE_HOST && addressSpace != NTCB_ADDRESS_SPACE_DEVICE)
    {
        SetError("Unknown address space %d.", addressSpace);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    // the colour space each channel is stored in comes from the container, as in ReadChannels
    NtcbOutputConversion conversion = requested;
    OutputConversion packed;
    Status status = MakeOutputConversion(conversion, m_geometry.channels, packed);
    if (status != NTCB_OK)
        return status;
    for (int c = 0; c < conversion.numChannels; ++c)
        conversion.srcColorSpaces[c] = uint8_t(m_channelColorSpaces[conversion.firstChannel + c]);
    const size_t pixelBytes = size_t(conversion.components) * size_t(BytesPerComponent(conversion.channelFormat));
    const size_t bytes = size_t(m_geometry.TotalTexels()) * pixelBytes;
    if (destinationBytes < bytes)
    {
        SetError("The destination holds %zu bytes, the converted mip chain needs %zu.", destinationBytes, bytes);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    const bool toHost = addressSpace == NTCB_ADDRESS_SPACE_HOST;
    // every mip starts a whole number of pixels into the destination, so the pixel stores are as
    // aligned as the destination itself
    const size_t alignment = std::max<size_t>(4, ConvertedPixelAlignment(pixelBytes));
    if (!toHost && (reinterpret_cast<uintptr_t>(destination) % alignment))
    {
        SetError("A device destination for pixels of %zu bytes must be %zu-byte aligned.", pixelBytes, alignment);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    DeviceGuard guard(m_device);
    if (!guard.Success())
        return NTCB_ERR_CUDA;
    void* target = destination;
    if (toHost)
    {
        status = GrowStaging(bytes);
        if (status != NTCB_OK)
            return status;
        target = m_staging;
    }
    status = DecodeInto(nullptr, pOutStats, useInt8Weights, &conversion, target);
    if (status != NTCB_OK)
        return status;
    cudaError_t err;
    if (toHost && m_bandCount > 0)
    {
        // mip 0 band by band while the rest is decoded, then the other mips
        const size_t rowBytes = size_t(m_geometry.mipWidth[0]) * pixelBytes;
        const size_t mip0Bytes = rowBytes * size_t(m_geometry.mipHeight[0]);
        status = CopyBands(m_staging, static_cast<uint8_t*>(destination), rowBytes);
        if (status != NTCB_OK)
            return status;
        if (bytes > mip0Bytes)
        {
            err = cudaMemcpyAsync(static_cast<uint8_t*>(destination) + mip0Bytes, m_staging + mip0Bytes, bytes - mip0Bytes,
                cudaMemcpyDeviceToHost, m_stream);
            if (err != cudaSuccess)
                return CudaFailure("cudaMemcpyAsync (converted texels)", err);
        }
    }
    else if (toHost)
    {
        err = cudaMemcpyAsync(destination, m_staging, bytes, cudaMemcpyDeviceToHost, m_stream);
        if (err != cudaSuccess)
            return CudaFailure("cudaMemcpyAsync (converted texels)", err);
    }
    err = cudaStreamSynchronize(m_stream);
    if (err != cudaSuccess)
        return CudaFailure("cudaStreamSynchronize", err);
    status = CheckKernelStatus();
    if (status != NTCB_OK)
        return status;
    ClearError();
    return NTCB_OK;
}

// Device-to-host copy of mip 0 (rows of `rowBytes` bytes, no padding) band by band as the bands of
// the last decode complete; returns when the copy stream has drained.
Status TextureSet::CopyBands(const uint8_t* deviceMip0, uint8_t* host, size_t rowBytes)
{
    int begin = 0;
    for (int b = 0; b < m_bandCount; ++b)
    {
        const int end = m_bandEnd[b];
        if (end > begin)
        {
            cudaError_t err = cudaStreamWaitEvent(m_copyStream, m_bandEvents[b], 0);
            if (err == cudaSuccess)
                err = cudaMemcpyAsync(host + size_t(begin) * rowBytes, deviceMip0 + size_t(begin) * rowBytes,
                    size_t(end - begin) * rowBytes, cudaMemcpyDeviceToHost, m_copyStream);
            if (err != cudaSuccess)
                return CudaFailure("cudaMemcpyAsync (band)", err);
        }
        begin = end;
    }
    cudaError_t err = cudaStreamSynchronize(m_copyStream);
    if (err != cudaSuccess)
        return CudaFailure("cudaStreamSynchronize (copy stream)", err);
    return NTCB_OK;
}

Status TextureSet::GrowStaging(size_t bytes)
{
    if (m_stagingBytes >= bytes)
        return NTCB_OK;
    cudaStreamSynchronize(m_stream);
    if (m_staging)
        cudaFree(m_staging);
    m_staging = nullptr;
    m_stagingBytes = 0;
    cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&m_staging), bytes);
    if (err != cudaSuccess)
    {
        SetError("Failed to allocate %zu bytes of device memory for the staging buffer.", bytes);
        return NTCB_ERR_OUT_OF_MEMORY;
    }
    m_stagingBytes = bytes;
    return NTCB_OK;
}

// One decode launch of all mips (or of a row range per mip) into `deviceOut`: fp16 texels in the
// set's layout, or converted pixels (mip after mip, rows without padding) when `conversion` is set.
Status TextureSet::DecodeInto(const int32_t* rowRanges, DecompressionStats* pOutStats, bool useInt8Weights,
    const NtcbOutputConversion* conversion, void* deviceOut)
{
    if (useInt8Weights ? !m_hasInt8 : !m_hasFp8)
    {
        SetError("The texture set has no %s network; it cannot be decompressed with these weights.",
            useInt8Weights ? "Int8" : "FP8");
        return NTCB_ERR_INVALID_STATE;
    }
    if (pOutStats)
        memset(pOutStats, 0, sizeof *pOutStats);
    DeviceGuard guard(m_device);
    if (!guard.Success())
        return NTCB_ERR_CUDA;

    // upload the encoded latents and the network weights, as the reference does on every
    // Decompress of a loaded set (src/TextureSet.cpp:1691-1757)
    cudaError_t err = cudaMemcpyAsync(m_deviceUpload, m_hostUpload, m_uploadBytes, cudaMemcpyHostToDevice, m_stream);
    if (err != cudaSuccess)
        return CudaFailure("cudaMemcpyAsync (compressed data)", err);
    m_deviceCurrent = true;
    err = cudaMemsetAsync(m_status, 0, NTCB_STATUS_WORDS * sizeof(uint32_t), m_stream);
    if (err != cudaSuccess)
        return CudaFailure("cudaMemsetAsync (status)", err);

    NtcbDecodeParams params{};
    params.latents = reinterpret_cast<const uint16_t*>(m_deviceUpload);
    params.network = m_deviceUpload + m_latentBytes + (useInt8Weights ? 0 : m_networkBytes);
    params.numerics = m_numerics;
    params.out = deviceOut;
    params.conversion = conversion;
    params.status = m_status;
    params.numMips = m_geometry.mips;
    params.numFeatures = m_geometry.numFeatures;
    params.channels = m_geometry.channels;
    params.weightMode = useInt8Weights ? NTCB_WEIGHTS_INT8 : NTCB_WEIGHTS_FP8;
    params.outputLayout = m_layout;
    for (int mip = 0; mip < m_geometry.mips; ++mip)
    {
        // the per-mip parameters TextureSet::Decompress fills (src/TextureSet.cpp:1806-1829)
        const int lod = m_geometry.neuralLod[mip];
        NtcbMipDesc& d = params.mips[mip];
        d.width = m_geometry.mipWidth[mip];
        d.height = m_geometry.mipHeight[mip];
        d.hiWidth = m_geometry.latentWidth[lod];
        d.hiHeight = m_geometry.latentHeight[lod];
        d.loWidth = m_geometry.latentWidth[lod + 1];
        d.loHeight = m_geometry.latentHeight[lod + 1];
        d.hiOffset = m_geometry.latentPixelOffset[lod] * m_geometry.numLayers;
        d.loOffset = m_geometry.latentPixelOffset[lod + 1] * m_geometry.numLayers;
        d.hiPlane = uint64_t(d.hiWidth) * d.hiHeight;
        d.loPlane = uint64_t(d.loWidth) * d.loHeight;
        d.positionScale = m_geometry.positionScale[mip];
        d.positionLod = m_geometry.positionLod[mip];
        d.outOffset = m_geometry.mipTexelOffset[mip] * uint64_t(conversion ? conversion->components : m_geometry.channels);
        d.rowBegin = rowRanges ? rowRanges[2 * mip] : 0;
        d.rowEnd = rowRanges ? rowRanges[2 * mip + 1] : d.height;
        if (d.rowBegin < 0 || d.rowEnd > d.height || d.rowBegin > d.rowEnd)
        {
            SetError("Row range [%d, %d) of mip %d is outside the mip (height %d).", d.rowBegin, d.rowEnd, mip, d.height);
            return NTCB_ERR_OUT_OF_RANGE;
        }
    }

    if (pOutStats)
    {
        err = cudaEventRecord(m_eventStart, m_stream);
        if (err != cudaSuccess)
            return CudaFailure("cudaEventRecord (1)", err);
    }
    Status status = NTCB_OK;
    m_bandCount = 0;
    const int height0 = m_geometry.mipHeight[0];
    if (!rowRanges && height0 >= kBandMinRows)
    {
        // row bands of mip 0 (whole tile rows), then the other mips
        const int bandRows = ((height0 + kBands - 1) / kBands + 15) & ~15;
        NtcbDecodeParams part = params;
        for (int mip = 1; mip < m_geometry.mips; ++mip)
            part.mips[mip].rowBegin = part.mips[mip].rowEnd = 0;
        for (int b = 0; b < kBands && status == NTCB_OK; ++b)
        {
            part.mips[0].rowBegin = std::min(height0, b * bandRows);
            part.mips[0].rowEnd = std::min(height0, (b + 1) * bandRows);
            m_bandEnd[b] = part.mips[0].rowEnd;
            status = ntcb_decode(&part, m_stream);
            if (status == NTCB_OK && cudaEventRecord(m_bandEvents[b], m_stream) != cudaSuccess)
                status = CudaFailure("cudaEventRecord (band)", cudaGetLastError());
        }
        if (status == NTCB_OK)
        {
            part = params;
            part.mips[0].rowBegin = part.mips[0].rowEnd = 0;
            status = ntcb_decode(&part, m_stream);
            if (status == NTCB_OK && cudaEventRecord(m_bandEvents[kBands], m_stream) != cudaSuccess)
                status = CudaFailure("cudaEventRecord (band)", cudaGetLastError());
        }
        if (status == NTCB_OK)
            m_bandCount = kBands;
    }
    else
        status = ntcb_decode(&params, m_stream);
    if (status != NTCB_OK)
        return status;
    if (pOutStats)
    {
        err = cudaEventRecord(m_eventStop, m_stream);
        if (err != cudaSuccess)
            return CudaFailure("cudaEventRecord (2)", err);
    }
    err = cudaMemcpyAsync(m_hostStatus, m_status, NTCB_STATUS_WORDS * sizeof(uint32_t), cudaMemcpyDeviceToHost, m_stream);
    if (err != cudaSuccess)
        return CudaFailure("cudaMemcpyAsync (status)", err);
    if (pOutStats)
    {
        err = cudaStreamSynchronize(m_stream);
        if (err != cudaSuccess)
            return CudaFailure("cudaStreamSynchronize", err);
        cudaEventElapsedTime(&pOutStats->gpuTimeMilliseconds, m_eventStart, m_eventStop);
        status = CheckKernelStatus();
        if (status != NTCB_OK)
            return status;
    }
    ClearError();
    return NTCB_OK;
}

Status TextureSet::Sample(float const* deviceQueries, uint64_t numQueries, void* deviceOut, bool useInt8Weights)
{
    if (useInt8Weights ? !m_hasInt8 : !m_hasFp8)
    {
        SetError("The texture set has no %s network; it cannot be sampled with these weights.", useInt8Weights ? "Int8" : "FP8");
        return NTCB_ERR_INVALID_STATE;
    }
    if (numQueries == 0)
    {
        ClearError();
        return NTCB_OK;
    }
    if (!deviceQueries || !deviceOut)
    {
        SetError("deviceQueries and deviceOut must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    DeviceGuard guard(m_device);
    if (!guard.Success())
        return NTCB_ERR_CUDA;

    cudaError_t err = cudaSuccess;
    if (!m_deviceCurrent)
    {
        err = cudaMemcpyAsync(m_deviceUpload, m_hostUpload, m_uploadBytes, cudaMemcpyHostToDevice, m_stream);
        if (err != cudaSuccess)
            return CudaFailure("cudaMemcpyAsync (compressed data)", err);
        m_deviceCurrent = true;
        m_pixelMajorCurrent = false;
    }
    NtcbSampleParams params{};
    params.numMips = m_geometry.mips;
    params.numFeatures = m_geometry.numFeatures;
    for (int mip = 0; mip < m_geometry.mips; ++mip)
    {
        // the per-mip parameters TextureSet::Decompress fills (src/TextureSet.cpp:1806-1829)
        const int lod = m_geometry.neuralLod[mip];
        NtcbMipDesc& d = params.mips[mip];
        d.width = m_geometry.mipWidth[mip];
        d.height = m_geometry.mipHeight[mip];
        d.hiWidth = m_geometry.latentWidth[lod];
        d.hiHeight = m_geometry.latentHeight[lod];
        d.loWidth = m_geometry.latentWidth[lod + 1];
        d.loHeight = m_geometry.latentHeight[lod + 1];
        d.hiOffset = m_geometry.latentPixelOffset[lod] * m_geometry.numLayers;
        d.loOffset = m_geometry.latentPixelOffset[lod + 1] * m_geometry.numLayers;
        d.hiPlane = uint64_t(d.hiWidth) * d.hiHeight;
        d.loPlane = uint64_t(d.loWidth) * d.loHeight;
        d.positionScale = m_geometry.positionScale[mip];
        d.positionLod = m_geometry.positionLod[mip];
        d.rowEnd = d.height;
    }
    if (!m_pixelMajorCurrent)
    {
        // the pixel-major copy of the latents: slots of 1, 2 or 4 elements per latent pixel
        const size_t slot = m_geometry.numLayers == 3 ? 4 : size_t(m_geometry.numLayers);
        if (!m_pixelMajor)
        {
            const size_t layers = size_t(m_geometry.numLayers), elements = m_latentBytes / 2;
            err = cudaMalloc(&m_pixelMajor, (elements + layers - 1) / layers * slot * 2);
            if (err != cudaSuccess)
            {
                m_pixelMajor = nullptr;
                CudaFailure("cudaMalloc (pixel-major latents)", err);
                return NTCB_ERR_OUT_OF_MEMORY;
            }
        }
        Status status = ntcb_interleave_latents(reinterpret_cast<const uint16_t*>(m_deviceUpload), m_pixelMajor, params.mips,
            m_geometry.mips, m_geometry.numFeatures, m_stream);
        if (status != NTCB_OK)
            return status;
        m_pixelMajorCurrent = true;
    }
    err = cudaMemsetAsync(m_status, 0, NTCB_STATUS_WORDS * sizeof(uint32_t), m_stream);
    if (err != cudaSuccess)
        return CudaFailure("cudaMemsetAsync (status)", err);
    params.latents = m_pixelMajor;
    params.latentLayout = NTCB_LATENTS_INTERLEAVED;
    params.network = m_deviceUpload + m_latentBytes + (useInt8Weights ? 0 : m_networkBytes);
    params.queries = deviceQueries;
    params.out = deviceOut;
    params.status = m_status;
    params.numQueries = numQueries;
    params.channels = m_geometry.channels;
    params.weightMode = useInt8Weights ? NTCB_WEIGHTS_INT8 : NTCB_WEIGHTS_FP8;
    params.numerics = m_numerics;
    Status status = ntcb_sample(&params, m_stream);
    if (status != NTCB_OK)
        return status;
    err = cudaMemcpyAsync(m_hostStatus, m_status, NTCB_STATUS_WORDS * sizeof(uint32_t), cudaMemcpyDeviceToHost, m_stream);
    if (err != cudaSuccess)
        return CudaFailure("cudaMemcpyAsync (status)", err);
    err = cudaStreamSynchronize(m_stream);
    if (err != cudaSuccess)
        return CudaFailure("cudaStreamSynchronize", err);
    status = CheckKernelStatus();
    if (status != NTCB_OK)
        return status;
    ClearError();
    return NTCB_OK;
}

Status TextureSet::ReadChannels(ReadChannelsParameters const& params)
{
    if (!params.pOutData)
    {
        SetError("pOutData is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    // argument checks of ValidateReadWriteChannelsArgs (src/TextureSet.cpp:1899-1956)
    if (params.mipLevel < 0 || params.mipLevel >= m_geometry.mips)
    {
        SetError("mipLevel (%d) must be between 0 and %d.", params.mipLevel, m_geometry.mips - 1);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (params.firstChannel < 0 || params.firstChannel >= m_geometry.channels)
    {
        SetError("firstChannel (%d) must be between 0 and %d.", params.firstChannel, m_geometry.channels - 1);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (params.numChannels < 1 || params.numChannels > m_geometry.channels - params.firstChannel)
    {
        SetError("For the provided firstChannel (%d), numChannels (%d) must be between 1 and %d.", params.firstChannel,
            params.numChannels, m_geometry.channels - params.firstChannel);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    // the mip's own size, and the size asked for: a different one means a bilinear resize, as in the reference
    const int mipWidth = m_geometry.mipWidth[params.mipLevel], mipHeight = m_geometry.mipHeight[params.mipLevel];
    if (params.width <= 0 || params.height <= 0)
    {
        SetError("width (%d) and height (%d) must be positive.", params.width, params.height);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    const int width = params.width, height = params.height;
    const bool resized = width != mipWidth || height != mipHeight;
    const size_t componentBytes = size_t(BytesPerComponent(params.channelFormat));
    if (componentBytes == 0)
    {
        SetError("Unknown channel format %d.", params.channelFormat);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (params.pixelStride < componentBytes || params.rowPitch < params.pixelStride * size_t(width) ||
        params.pixelStride % componentBytes || params.rowPitch % componentBytes ||
        (params.addressSpace == NTCB_ADDRESS_SPACE_DEVICE && reinterpret_cast<uintptr_t>(params.pOutData) % componentBytes))
    {
        SetError("pixelStride (%zu) must hold at least one %zu-byte component and rowPitch (%zu) a row of pixels; both, and a "
                 "device destination, must be multiples of the component size.",
            params.pixelStride, componentBytes, params.rowPitch);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    OutputConversion conversion{};
    conversion.format = params.channelFormat;
    conversion.dstChannels = int(std::min<size_t>(params.pixelStride / componentBytes, size_t(kMaxChannels))); // src/TextureSet.cpp:957
    conversion.dither = params.useDithering != 0;
    for (int c = 0; c < params.numChannels; ++c)
    {
        const int dstSpace = params.dstColorSpaces ? params.dstColorSpaces[c] : NTCB_COLOR_SPACE_LINEAR;
        if (dstSpace < NTCB_COLOR_SPACE_LINEAR || dstSpace > NTCB_COLOR_SPACE_HLG)
        {
            SetError("dstColorSpaces[%d] (%d) is not a known color space.", c, dstSpace);
            return NTCB_ERR_INVALID_ARGUMENT;
        }
        conversion.srcSpaces |= uint32_t(m_channelColorSpaces[params.firstChannel + c]) << (2 * c);
        conversion.dstSpaces |= uint32_t(dstSpace) << (2 * c);
    }
    const bool plainCopy = params.channelFormat == NTCB_CHANNEL_FORMAT_FLOAT16 && conversion.srcSpaces == conversion.dstSpaces;
    if (params.addressSpace != NTCB_ADDRESS_SPACE_HOST && params.addressSpace != NTCB_ADDRESS_SPACE_DEVICE)
    {
        SetError("Unknown address space %d.", params.addressSpace);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (!m_decoded)
    {
        SetError("The texture set has not been decompressed yet.");
        return NTCB_ERR_INVALID_STATE;
    }
    DeviceGuard guard(m_device);
    if (!guard.Success())
        return NTCB_ERR_CUDA;

    const __half* mipData = m_texels + m_geometry.mipTexelOffset[params.mipLevel] * m_geometry.channels;
    const size_t bytes = size_t(height) * params.rowPitch;
    const bool toHost = params.addressSpace == NTCB_ADDRESS_SPACE_HOST;
    const bool direct = !resized && plainCopy && m_layout == NTCB_LAYOUT_INTERLEAVED && params.firstChannel == 0 &&
                        params.numChannels == m_geometry.channels && params.pixelStride == size_t(m_geometry.channels) * 2 &&
                        params.rowPitch == params.pixelStride * size_t(width);
    cudaError_t err;
    if (direct && toHost && params.mipLevel == 0 && m_bandCount > 0)
    {
        // the request is the internal layout and the decode ran in row bands: every band is copied as
        // soon as it is decoded, on a stream of its own
        Status copied = CopyBands(reinterpret_cast<const uint8_t*>(mipData), static_cast<uint8_t*>(params.pOutData), params.rowPitch);
        if (copied != NTCB_OK)
            return copied;
    }
    else if (direct)
    {
        // the request is the internal layout: one copy, no conversion pass
        err = cudaMemcpyAsync(params.pOutData, mipData, bytes, toHost ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice,
            m_stream);
        if (err != cudaSuccess)
            return CudaFailure("cudaMemcpyAsync (texels)", err);
    }
    else
    {
        uint8_t* target = static_cast<uint8_t*>(params.pOutData);
        if (toHost)
        {
            Status grown = GrowStaging(bytes);
            if (grown != NTCB_OK)
                return grown;
            target = m_staging;
            if (params.rowPitch > params.pixelStride * size_t(width) ||
                params.pixelStride > size_t(conversion.dstChannels) * componentBytes)
            {
                // gaps are not written by the kernel: hand back zeros there, as the reference does
                err = cudaMemsetAsync(m_staging, 0, bytes, m_stream);
                if (err != cudaSuccess)
                    return CudaFailure("cudaMemsetAsync (staging)", err);
            }
        }
        dim3 block(32, 8);
        dim3 grid((width + block.x - 1) / block.x, (height + block.y - 1) / block.y);
        if (resized)
            err = LaunchResizeChannels(grid, block, m_stream, mipData, m_layout, mipWidth, mipHeight, m_geometry.channels,
                params.firstChannel, params.numChannels, conversion, target, width, height, params.pixelStride, params.rowPitch);
        else
            err = LaunchReadChannels(grid, block, m_stream, mipData, m_layout, width, height, m_geometry.channels,
                params.firstChannel, params.numChannels, conversion, target, params.pixelStride, params.rowPitch);
        if (err != cudaSuccess)
            return CudaFailure("ReadChannelsKernel launch", err);
        CountLaunch();
        if (toHost)
        {
            err = cudaMemcpyAsync(params.pOutData, m_staging, bytes, cudaMemcpyDeviceToHost, m_stream);
            if (err != cudaSuccess)
                return CudaFailure("cudaMemcpyAsync (staging)", err);
        }
    }
    err = cudaStreamSynchronize(m_stream);
    if (err != cudaSuccess)
        return CudaFailure("cudaStreamSynchronize", err);
    Status status = CheckKernelStatus();
    if (status != NTCB_OK)
        return status;
    ClearError();
    return NTCB_OK;
}

// Texture `index` of `textures` as the C structure; OutOfRange past the end.
Status FillTextureDesc(const std::vector<LoadedTexture>& textures, int index, NtcbTextureDesc* out)
{
    if (index < 0 || index >= int(textures.size()) || !out)
    {
        SetError("Texture index (%d) must be between 0 and %d and the output must not be NULL.", index, int(textures.size()) - 1);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    const LoadedTexture& texture = textures[size_t(index)];
    memset(out, 0, sizeof *out);
    snprintf(out->name, sizeof out->name, "%s", texture.name.c_str());
    out->firstChannel = texture.firstChannel;
    out->numChannels = texture.numChannels;
    out->channelFormat = texture.channelFormat;
    out->blockCompressedFormat = texture.blockCompressedFormat;
    out->rgbColorSpace = texture.rgbColorSpace;
    out->alphaColorSpace = texture.alphaColorSpace;
    ClearError();
    return NTCB_OK;
}

Status TextureSet::GetTexture(int index, NtcbTextureDesc& outTexture) const
{
    return FillTextureDesc(m_textures, index, &outTexture);
}

Status TextureSet::GetDeviceMip(int mipLevel, void** outPointer, size_t* outBytes)
{
    if (mipLevel < 0 || mipLevel >= m_geometry.mips || !outPointer || !outBytes)
    {
        SetError("mipLevel (%d) must be between 0 and %d and the output pointers must not be NULL.", mipLevel,
            m_geometry.mips - 1);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    *outPointer = m_texels + m_geometry.mipTexelOffset[mipLevel] * m_geometry.channels;
    *outBytes = size_t(m_geometry.mipWidth[mipLevel]) * m_geometry.mipHeight[mipLevel] * m_geometry.channels * sizeof(__half);
    ClearError();
    return NTCB_OK;
}

Status TextureSet::BlockCompress(int mipLevel, int firstChannel, int numChannels, int format, float alphaThreshold,
    void* deviceBlocks, size_t rowPitch)
{
    if (!m_decoded)
    {
        SetError("BlockCompress needs decoded texels: call Decompress first.");
        return NTCB_ERR_INVALID_STATE;
    }
    if (mipLevel < 0 || mipLevel >= m_geometry.mips)
    {
        SetError("mipLevel (%d) must be between 0 and %d.", mipLevel, m_geometry.mips - 1);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    DeviceGuard guard(m_device);
    if (!guard.Success())
        return NTCB_ERR_CUDA;
    NtcbBlockCompressParams params = {};
    params.deviceMip = m_texels + m_geometry.mipTexelOffset[mipLevel] * m_geometry.channels;
    params.layout = m_layout;
    params.width = m_geometry.mipWidth[mipLevel];
    params.height = m_geometry.mipHeight[mipLevel];
    params.channels = m_geometry.channels;
    params.firstChannel = firstChannel;
    params.numChannels = numChannels;
    params.format = format;
    params.alphaThreshold = alphaThreshold;
    params.widthInBlocks = (params.width + 3) / 4;
    params.heightInBlocks = (params.height + 3) / 4;
    params.deviceBlocks = deviceBlocks;
    params.rowPitch = rowPitch;
    return ntcb_block_compress(&params, m_stream);
}

Status TextureSet::CheckTextureAndMip(int textureIndex, int mipLevel) const
{
    if (textureIndex < 0 || textureIndex >= int(m_textures.size()))
    {
        SetError("textureIndex (%d) must be between 0 and %d.", textureIndex, int(m_textures.size()) - 1);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (mipLevel < 0 || mipLevel >= m_geometry.mips)
    {
        SetError("mipLevel (%d) must be between 0 and %d.", mipLevel, m_geometry.mips - 1);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    return NTCB_OK;
}

Status TextureSet::GetBC7ModeBuffer(int textureIndex, int mipLevel, void const** outData, size_t* outSize) const
{
    if (outData)
        *outData = nullptr;
    if (outSize)
        *outSize = 0;
    const Status status = CheckTextureAndMip(textureIndex, mipLevel);
    if (status != NTCB_OK)
        return status;
    const LoadedTexture& texture = m_textures[size_t(textureIndex)];
    if (texture.modeBufferCompressed[size_t(mipLevel)])
    {
        SetError("The BC7 mode buffer of texture %d, mip level %d is stored with GDeflate compression, which this decoder does not read.",
            textureIndex, mipLevel);
        return NTCB_ERR_UNSUPPORTED;
    }
    const std::vector<uint8_t>& data = texture.modeBuffers[size_t(mipLevel)];
    if (!data.empty())
    {
        if (outData)
            *outData = data.data();
        if (outSize)
            *outSize = data.size();
    }
    ClearError();
    return NTCB_OK;
}

Status TextureSet::MakeAndStoreBC7ModeBuffer(int textureIndex, int mipLevel, int widthInBlocks, int heightInBlocks,
    void const* blockData, size_t blockDataSize, size_t rowPitch)
{
    const Status status = CheckTextureAndMip(textureIndex, mipLevel);
    if (status != NTCB_OK)
        return status;
    const int mipWidthInBlocks = (m_geometry.mipWidth[mipLevel] + 3) / 4, mipHeightInBlocks = (m_geometry.mipHeight[mipLevel] + 3) / 4;
    if (widthInBlocks != mipWidthInBlocks || heightInBlocks != mipHeightInBlocks)
    {
        SetError("Provided widthInBlocks (%d) and heightInBlocks (%d) do not match the expected dimensions (%d x %d) for mip level %d.",
            widthInBlocks, heightInBlocks, mipWidthInBlocks, mipHeightInBlocks, mipLevel);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    LoadedTexture& texture = m_textures[size_t(textureIndex)];
    std::vector<uint8_t> data(ntcb_bc7_mode_buffer_size(widthInBlocks, heightInBlocks));
    const Status made = ntcb_make_bc7_mode_buffer(widthInBlocks, heightInBlocks, blockData, blockDataSize, rowPitch, data.data(), data.size());
    if (made != NTCB_OK)
        return made;
    // a device copy of the bitmap this one replaces may still be read by work queued on the stream
    void*& deviceCopy = m_deviceModeBuffers[size_t(textureIndex)][size_t(mipLevel)];
    if (deviceCopy)
    {
        DeviceGuard guard(m_device);
        if (!guard.Success())
            return NTCB_ERR_CUDA;
        cudaError_t err = cudaStreamSynchronize(m_stream);
        if (err == cudaSuccess)
            err = cudaFree(deviceCopy);
        if (err != cudaSuccess)
            return CudaFailure("cudaFree", err);
        deviceCopy = nullptr;
    }
    texture.modeBuffers[size_t(mipLevel)] = std::move(data);
    texture.modeBufferCompressed[size_t(mipLevel)] = 0;
    return NTCB_OK;
}

Status TextureSet::BlockCompressTexture(int textureIndex, int mipLevel, float alphaThreshold, void* deviceBlocks, size_t rowPitch)
{
    if (!m_decoded)
    {
        SetError("BlockCompress needs decoded texels: call Decompress first.");
        return NTCB_ERR_INVALID_STATE;
    }
    const Status status = CheckTextureAndMip(textureIndex, mipLevel);
    if (status != NTCB_OK)
        return status;
    const LoadedTexture& texture = m_textures[size_t(textureIndex)];
    const int format = texture.blockCompressedFormat;
    if (format == 0)
    {
        SetError("Texture %d ('%s') names no block-compressed format.", textureIndex, texture.name.c_str());
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    DeviceGuard guard(m_device);
    if (!guard.Success())
        return NTCB_ERR_CUDA;
    NtcbBlockCompressParams params = {};
    params.deviceMip = m_texels + m_geometry.mipTexelOffset[mipLevel] * m_geometry.channels;
    params.layout = m_layout;
    params.width = m_geometry.mipWidth[mipLevel];
    params.height = m_geometry.mipHeight[mipLevel];
    params.channels = m_geometry.channels;
    params.firstChannel = texture.firstChannel;
    params.format = format;
    params.alphaThreshold = alphaThreshold;
    params.widthInBlocks = (params.width + 3) / 4;
    params.heightInBlocks = (params.height + 3) / 4;
    params.deviceBlocks = deviceBlocks;
    params.rowPitch = rowPitch;
    // BC4 / BC5 take their one or two channels; the colour formats what the texture has, up to four
    params.numChannels = (format == NTCB_BLOCK_FORMAT_BC4 || format == NTCB_BLOCK_FORMAT_BC5) ? 0 : (texture.numChannels < 4 ? texture.numChannels : 4);
    if (format == NTCB_BLOCK_FORMAT_BC7)
    {
        if (texture.modeBufferCompressed[size_t(mipLevel)])
        {
            SetError("The BC7 mode buffer of texture %d, mip level %d is stored with GDeflate compression, which this decoder does not read.",
                textureIndex, mipLevel);
            return NTCB_ERR_UNSUPPORTED;
        }
        const std::vector<uint8_t>& modes = texture.modeBuffers[size_t(mipLevel)];
        if (!modes.empty())
        {
            const size_t needed = ntcb_bc7_mode_buffer_size(params.widthInBlocks, params.heightInBlocks);
            if (modes.size() < needed)
            {
                SetError("The BC7 mode buffer of texture %d, mip level %d holds %zu bytes, %zu are needed.", textureIndex, mipLevel,
                    modes.size(), needed);
                return NTCB_ERR_FILE_UNRECOGNIZED;
            }
            void*& deviceCopy = m_deviceModeBuffers[size_t(textureIndex)][size_t(mipLevel)];
            if (!deviceCopy)
            {
                // the kernel reads whole 32-bit words: the copy is padded to a multiple of four bytes
                const size_t bytes = (modes.size() + 3) & ~size_t(3);
                cudaError_t err = cudaMalloc(&deviceCopy, bytes);
                if (err == cudaSuccess)
                    err = cudaMemsetAsync(deviceCopy, 0, bytes, m_stream);
                if (err == cudaSuccess)
                    err = cudaMemcpyAsync(deviceCopy, modes.data(), modes.size(), cudaMemcpyHostToDevice, m_stream);
                if (err != cudaSuccess)
                {
                    if (deviceCopy)
                        cudaFree(deviceCopy);
                    deviceCopy = nullptr;
                    return CudaFailure("BC7 mode buffer upload", err);
                }
            }
            params.deviceModeBuffer = deviceCopy;
            params.modeMapWidthInBlocks = uint32_t(params.widthInBlocks);
            params.modeMapHeightInBlocks = uint32_t(params.heightInBlocks);
        }
    }
    return ntcb_block_compress(&params, m_stream);
}

Status TextureSet::Synchronize()
{
    DeviceGuard guard(m_device);
    if (!guard.Success())
        return NTCB_ERR_CUDA;
    cudaError_t err = cudaStreamSynchronize(m_stream);
    if (err != cudaSuccess)
        return CudaFailure("cudaStreamSynchronize", err);
    if (m_decoded)
    {
        Status status = CheckKernelStatus();
        if (status != NTCB_OK)
            return status;
    }
    ClearError();
    return NTCB_OK;
}

} // namespace

Status CreateContext(IContext** pOutContext, ContextParameters const& params)
{
    if (!pOutContext)
    {
        SetError("pOutContext is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    *pOutContext = nullptr;
    Context* context = new (std::nothrow) Context(params.cudaDevice);
    if (!context)
    {
        SetError("Out of host memory.");
        return NTCB_ERR_OUT_OF_MEMORY;
    }
    Status status = context->Initialize();
    if (status != NTCB_OK)
    {
        delete context;
        return status;
    }
    *pOutContext = context;
    return NTCB_OK;
}

void DestroyContext(IContext* context)
{
    delete context;
}

} // namespace ntcb

// ---------------------------------------------------------------------------------------------
// C ABI wrappers
// ---------------------------------------------------------------------------------------------

struct NtcbContext
{
    ntcb::IContext* impl;
};

struct NtcbTextureSet
{
    ntcb::ITextureSet* impl;
    const ntcb::IContext* owner;
};

extern "C"
{

static void FillDesc(const ntcb::SetGeometry& geo, NtcbTextureSetDesc* outDesc)
{
    outDesc->width = geo.width;
    outDesc->height = geo.height;
    outDesc->channels = geo.channels;
    outDesc->mips = geo.mips;
    outDesc->gridSizeScale = geo.gridSizeScale;
    outDesc->numFeatures = geo.numFeatures;
    outDesc->numNeuralMips = geo.numNeuralMips;
    outDesc->numLayers = geo.numLayers;
    outDesc->totalTexels = geo.TotalTexels();
}

int ntcb_probe_container(const void* data, size_t size, NtcbTextureSetDesc* outDesc)
{
    if (!outDesc)
    {
        ntcb::SetError("outDesc is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    ntcb::LoadedSet loaded;
    int status = ntcb::Guarded(__func__, [&]() { return ntcb::LoadContainer(data, size, loaded); });
    if (status != NTCB_OK)
        return status;
    FillDesc(loaded.geometry, outDesc);
    return NTCB_OK;
}

int ntcb_probe_container_texture(const void* data, size_t size, int index, NtcbTextureDesc* outTexture, int* outCount)
{
    ntcb::LoadedSet loaded;
    int status = ntcb::Guarded(__func__, [&]() { return ntcb::LoadContainer(data, size, loaded); });
    if (status != NTCB_OK)
        return status;
    if (outCount)
        *outCount = int(loaded.textures.size());
    return ntcb::FillTextureDesc(loaded.textures, index, outTexture);
}

int ntcb_probe_container_bc7_mode_buffer(const void* data, size_t size, int textureIndex, int mipLevel, uint64_t* outOffset,
    uint64_t* outStoredSize, int* outCompressed)
{
    if (outOffset)
        *outOffset = 0;
    if (outStoredSize)
        *outStoredSize = 0;
    if (outCompressed)
        *outCompressed = 0;
    ntcb::LoadedSet loaded;
    int status = ntcb::Guarded(__func__, [&]() { return ntcb::LoadContainer(data, size, loaded); });
    if (status != NTCB_OK)
        return status;
    if (textureIndex < 0 || textureIndex >= int(loaded.textures.size()))
    {
        ntcb::SetError("textureIndex (%d) must be between 0 and %d.", textureIndex, int(loaded.textures.size()) - 1);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    const ntcb::LoadedTexture& texture = loaded.textures[size_t(textureIndex)];
    if (mipLevel < 0 || mipLevel >= int(texture.modeBufferOffset.size()))
    {
        ntcb::SetError("mipLevel (%d) must be between 0 and %d.", mipLevel, int(texture.modeBufferOffset.size()) - 1);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (outOffset)
        *outOffset = texture.modeBufferOffset[size_t(mipLevel)];
    if (outStoredSize)
        *outStoredSize = texture.modeBufferStoredSize[size_t(mipLevel)];
    if (outCompressed)
        *outCompressed = texture.modeBufferCompressed[size_t(mipLevel)];
    ntcb::ClearError();
    return NTCB_OK;
}

int ntcb_context_create(int cudaDevice, NtcbContext** outContext)
{
    if (!outContext)
    {
        ntcb::SetError("outContext is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    *outContext = nullptr;
    ntcb::ContextParameters params;
    params.cudaDevice = cudaDevice;
    ntcb::IContext* impl = nullptr;
    int status = ntcb::Guarded(__func__, [&]() { return ntcb::CreateContext(&impl, params); });
    if (status != NTCB_OK)
        return status;
    *outContext = new (std::nothrow) NtcbContext{impl};
    if (!*outContext)
    {
        ntcb::DestroyContext(impl);
        ntcb::SetError("ntcb_context_create: out of host memory.");
        return NTCB_ERR_OUT_OF_MEMORY;
    }
    return NTCB_OK;
}

void ntcb_context_destroy(NtcbContext* context)
{
    if (!context)
        return;
    ntcb::DestroyContext(context->impl);
    delete context;
}

static int WrapTextureSet(NtcbContext* context, ntcb::ITextureSet* impl, NtcbTextureSet** outTextureSet)
{
    *outTextureSet = new (std::nothrow) NtcbTextureSet{impl, context->impl};
    if (!*outTextureSet)
    {
        context->impl->DestroyTextureSet(impl);
        ntcb::SetError("out of host memory.");
        return NTCB_ERR_OUT_OF_MEMORY;
    }
    return NTCB_OK;
}

int ntcb_texture_set_create_from_memory(NtcbContext* context, const void* data, size_t size,
    const NtcbTextureSetFeatures* features, NtcbTextureSet** outTextureSet)
{
    if (!context || !outTextureSet)
    {
        ntcb::SetError("context and outTextureSet must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    *outTextureSet = nullptr;
    NtcbTextureSetFeatures defaults{NTCB_LAYOUT_INTERLEAVED, 0};
    ntcb::ITextureSet* impl = nullptr;
    int status = ntcb::Guarded(__func__, [&]() { return context->impl->CreateCompressedTextureSetFromMemory(data, size, features ? *features : defaults, &impl); });
    if (status != NTCB_OK)
        return status;
    return WrapTextureSet(context, impl, outTextureSet);
}

int ntcb_texture_set_load_from_memory(NtcbTextureSet* textureSet, const void* data, size_t size)
{
    if (!textureSet)
    {
        ntcb::SetError("textureSet is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->LoadFromMemory(data, size); });
}

int ntcb_texture_set_create_from_file(NtcbContext* context, const char* fileName, const NtcbTextureSetFeatures* features,
    NtcbTextureSet** outTextureSet)
{
    if (!context || !outTextureSet)
    {
        ntcb::SetError("context and outTextureSet must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    *outTextureSet = nullptr;
    NtcbTextureSetFeatures defaults{NTCB_LAYOUT_INTERLEAVED, 0};
    ntcb::ITextureSet* impl = nullptr;
    int status = ntcb::Guarded(__func__, [&]() { return context->impl->CreateCompressedTextureSetFromFile(fileName, features ? *features : defaults, &impl); });
    if (status != NTCB_OK)
        return status;
    return WrapTextureSet(context, impl, outTextureSet);
}

void ntcb_texture_set_destroy(NtcbTextureSet* textureSet)
{
    if (!textureSet)
        return;
    textureSet->owner->DestroyTextureSet(textureSet->impl);
    delete textureSet;
}

int ntcb_texture_set_get_desc(const NtcbTextureSet* textureSet, NtcbTextureSetDesc* outDesc)
{
    if (!textureSet || !outDesc)
    {
        ntcb::SetError("textureSet and outDesc must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    FillDesc(static_cast<const ntcb::TextureSet*>(textureSet->impl)->Geometry(), outDesc);
    return NTCB_OK;
}

int ntcb_texture_set_decompress(NtcbTextureSet* textureSet, NtcbDecompressionStats* stats, int useInt8Weights)
{
    if (!textureSet)
    {
        ntcb::SetError("textureSet is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->Decompress(stats, useInt8Weights != 0); });
}

int ntcb_texture_set_decompress_rows(NtcbTextureSet* textureSet, const int32_t* rowRanges, NtcbDecompressionStats* stats,
    int useInt8Weights)
{
    if (!textureSet)
    {
        ntcb::SetError("textureSet is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->DecompressRows(rowRanges, stats, useInt8Weights != 0); });
}

int ntcb_texture_set_decompress_converted(NtcbTextureSet* textureSet, NtcbDecompressionStats* stats, int useInt8Weights,
    const NtcbOutputConversion* conversion, int addressSpace, void* destination, size_t destinationBytes)
{
    if (!textureSet || !conversion)
    {
        ntcb::SetError("textureSet and conversion must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->DecompressConverted(stats, useInt8Weights != 0, *conversion, addressSpace, destination,
        destinationBytes); });
}

int ntcb_texture_set_read_channels(NtcbTextureSet* textureSet, const NtcbReadChannelsParams* params)
{
    if (!textureSet || !params)
    {
        ntcb::SetError("textureSet and params must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->ReadChannels(*params); });
}

int ntcb_texture_set_device_mip(NtcbTextureSet* textureSet, int mipLevel, void** outPointer, size_t* outBytes)
{
    if (!textureSet)
    {
        ntcb::SetError("textureSet is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->GetDeviceMip(mipLevel, outPointer, outBytes); });
}

int ntcb_texture_set_block_compress(NtcbTextureSet* textureSet, int mipLevel, int firstChannel, int numChannels, int format,
    float alphaThreshold, void* deviceBlocks, size_t rowPitch)
{
    if (!textureSet)
    {
        ntcb::SetError("textureSet is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->BlockCompress(mipLevel, firstChannel, numChannels, format, alphaThreshold, deviceBlocks, rowPitch); });
}

int ntcb_texture_set_get_bc7_mode_buffer(NtcbTextureSet* textureSet, int textureIndex, int mipLevel, const void** outData,
    size_t* outSize)
{
    if (!textureSet)
    {
        ntcb::SetError("textureSet is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->GetBC7ModeBuffer(textureIndex, mipLevel, outData, outSize); });
}

int ntcb_texture_set_make_and_store_bc7_mode_buffer(NtcbTextureSet* textureSet, int textureIndex, int mipLevel, int widthInBlocks,
    int heightInBlocks, const void* blockData, size_t blockDataSize, size_t rowPitch)
{
    if (!textureSet)
    {
        ntcb::SetError("textureSet is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->MakeAndStoreBC7ModeBuffer(textureIndex, mipLevel, widthInBlocks, heightInBlocks, blockData, blockDataSize,
        rowPitch); });
}

int ntcb_texture_set_block_compress_texture(NtcbTextureSet* textureSet, int textureIndex, int mipLevel, float alphaThreshold,
    void* deviceBlocks, size_t rowPitch)
{
    if (!textureSet)
    {
        ntcb::SetError("textureSet is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->BlockCompressTexture(textureIndex, mipLevel, alphaThreshold, deviceBlocks, rowPitch); });
}

int ntcb_texture_set_get_texture(NtcbTextureSet* textureSet, int index, NtcbTextureDesc* outTexture, int* outCount)
{
    if (!textureSet)
    {
        ntcb::SetError("textureSet is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (outCount)
        *outCount = textureSet->impl->GetTextureCount();
    NtcbTextureDesc scratch;
    return textureSet->impl->GetTexture(index, outTexture ? *outTexture : scratch);
}

int ntcb_texture_set_sample(NtcbTextureSet* textureSet, const float* deviceQueries, uint64_t numQueries, void* deviceOut,
    int useInt8Weights)
{
    if (!textureSet)
    {
        ntcb::SetError("textureSet is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->Sample(deviceQueries, numQueries, deviceOut, useInt8Weights != 0); });
}

int ntcb_texture_set_synchronize(NtcbTextureSet* textureSet)
{
    if (!textureSet)
    {
        ntcb::SetError("textureSet is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ntcb::Guarded(__func__, [&]() { return textureSet->impl->Synchronize(); });
}

} // extern "C"
