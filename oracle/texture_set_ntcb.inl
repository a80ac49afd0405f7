// TEST INFRASTRUCTURE ONLY (never linked into the product library).
//
// The integration a LibNTC maintainer would make to put libntcb200.so behind the existing
// ntc::IContext / ntc::ITextureSet entry points, made real: this file is appended to a COPY of the
// reference's src/TextureSet.cpp by oracle/patch_texture_set.py (which also adds the declaration of
// the member function below to a copy of src/TextureSet.h and routes TextureSet::Decompress to it),
// and the result is built into oracle/_ref/libntc_ref_ntcb.so by `oracle/build_ref.sh --with-ntcb`.
// Everything else in that library is the unmodified reference: context creation, the container
// loader, ReadChannels and its CopyImage kernel.
//
// What it replaces inside TextureSet::Decompress (src/TextureSet.cpp:1664-1897) for a set loaded
// from a file: the latent unpacking and weight conversion of the prologue (:1691-1757) and the
// per-mip cuda::Inference loop (:1782-1864) become one weight staging and one ntcb_decode launch
// into the reference's own texture-data buffer, in the reference's own layout.

#include <ntcb.h>

#include <map>
#include <mutex>

namespace ntc
{

namespace
{
struct NtcbDeviceState
{
    uint8_t* networks = nullptr; // two staged network images (Int8, FP8)
    uint32_t* status = nullptr;  // NTCB_STATUS_WORDS words
};
std::mutex g_ntcbMutex;
std::map<const void*, NtcbDeviceState> g_ntcbState; // per texture set; lives as long as the process (test infrastructure)
}

Status TextureSet::DecompressThroughNtcb(DecompressionStats* pOutStats, bool useInt8Weights)
{
    if (pOutStats)
        memset(pOutStats, 0, sizeof(DecompressionStats));

    CudaDeviceGuard cudaGuard(m_context);
    if (!cudaGuard.Success())
        return Status::CudaError;

    // Upload the encoded latents, as the stock code does on every Decompress (:1695); they are
    // consumed as they are, so the unpacked fp16 copy is never produced.
    cudaError_t err = m_featureGrid.GetEncodedPixelsArray().CopyToDevice();
    if (err != cudaSuccess)
    {
        SetCudaErrorMessage("cudaMemcpy (QuantizedLatents)", err);
        return Status::CudaError;
    }

    NtcbDeviceState state;
    {
        std::lock_guard<std::mutex> lock(g_ntcbMutex);
        NtcbDeviceState& slot = g_ntcbState[this];
        if (!slot.networks)
        {
            err = cudaMalloc(reinterpret_cast<void**>(&slot.networks), 2 * NTCB_STAGED_REFERENCE_NETWORK_BYTES);
            if (err == cudaSuccess)
                err = cudaMalloc(reinterpret_cast<void**>(&slot.status), NTCB_STATUS_WORDS * sizeof(uint32_t));
            if (err != cudaSuccess)
            {
                SetCudaErrorMessage("cudaMalloc (staged networks)", err);
                return Status::OutOfMemory;
            }
        }
        state = slot;
    }

    // The weights: staged from the row-major blobs the loader keeps on the host (:207-231), in place
    // of ConvertNetworkFromQuantizedToFp16 (:1732-1755); uploaded on every call like the stock code.
    static thread_local uint8_t staged[2][NTCB_STAGED_REFERENCE_NETWORK_BYTES];
    if (ntcb_stage_network_reference(m_mlpDataInt8.HostPtr(), NTCB_INT8_BLOB_BYTES, NTCB_WEIGHTS_INT8, staged[0]) != NTCB_OK ||
        ntcb_stage_network_reference(m_mlpDataFP8.HostPtr(), NTCB_FP8_BLOB_BYTES, NTCB_WEIGHTS_FP8, staged[1]) != NTCB_OK)
    {
        SetErrorMessage("%s", ntcb_last_error());
        return Status::InternalError;
    }
    err = cudaMemcpy(state.networks, staged, sizeof staged, cudaMemcpyHostToDevice);
    if (err == cudaSuccess)
        err = cudaMemset(state.status, 0, NTCB_STATUS_WORDS * sizeof(uint32_t));
    if (err != cudaSuccess)
    {
        SetCudaErrorMessage("cudaMemcpy (staged networks)", err);
        return Status::CudaError;
    }

    half* const textureDataOut = m_textureDataOut.DevicePtr() ? m_textureDataOut.DevicePtr() : m_textureData.DevicePtr();
    uint16_t const* const latents = m_featureGrid.GetEncodedPixelsDevicePtr(0);

    NtcbDecodeParams p = {};
    p.latents = latents;
    p.network = state.networks + (useInt8Weights ? 0 : NTCB_STAGED_REFERENCE_NETWORK_BYTES);
    p.out = textureDataOut;
    p.status = state.status;
    p.numMips = m_desc.mips;
    p.numFeatures = m_latentShape.numFeatures;
    p.channels = m_desc.channels;
    p.weightMode = useInt8Weights ? NTCB_WEIGHTS_INT8 : NTCB_WEIGHTS_FP8;
    p.outputLayout = NTCB_LAYOUT_PLANAR_PAIRS; // the reference's internal layout: ReadChannels / CopyImage keep working
    p.numerics = NTCB_NUMERICS_REFERENCE;      // the bits cuda::Inference produces
    for (int mipLevel = 0; mipLevel < m_desc.mips; ++mipLevel)
    {
        int const neuralLod = ColorMipToNeuralLod(mipLevel);
        LatentImageDesc const& latentImage = m_latentImages[neuralLod];
        ColorMipDesc const& colorMip = m_colorMips[mipLevel];
        NtcbMipDesc& d = p.mips[mipLevel];
        d.width = std::max(m_desc.width >> mipLevel, 1);
        d.height = std::max(m_desc.height >> mipLevel, 1);
        d.hiWidth = latentImage.width;
        d.hiHeight = latentImage.height;
        d.loWidth = std::max(latentImage.width >> 1, 1);
        d.loHeight = std::max(latentImage.height >> 1, 1);
        d.hiPlane = uint64_t(d.hiWidth) * uint64_t(d.hiHeight);
        d.loPlane = uint64_t(d.loWidth) * uint64_t(d.loHeight);
        d.hiOffset = uint64_t(m_featureGrid.GetEncodedPixelsDevicePtr(neuralLod) - latents);
        d.loOffset = uint64_t(m_featureGrid.GetEncodedPixelsDevicePtr(neuralLod + 1) - latents);
        d.positionScale = colorMip.positionScale;
        d.positionLod = colorMip.positionLod;
        d.outOffset = m_textureMipOffsets[mipLevel] * uint64_t(m_desc.channels);
        d.rowBegin = 0;
        d.rowEnd = d.height;
    }

    if (pOutStats)
    {
        err = cudaEventRecord(m_eventStart);
        if (err != cudaSuccess)
        {
            SetCudaErrorMessage("cudaEventRecord (1)", err);
            return Status::CudaError;
        }
    }

    if (ntcb_decode(&p, /* stream = */ nullptr) != NTCB_OK) // the legacy default stream, which the reference uses everywhere
    {
        SetErrorMessage("%s", ntcb_last_error());
        return Status::CudaError;
    }

    if (pOutStats)
    {
        err = cudaEventRecord(m_eventStop);
        if (err == cudaSuccess)
            err = cudaEventSynchronize(m_eventStop);
        if (err != cudaSuccess)
        {
            SetCudaErrorMessage("cudaEventRecord / cudaEventSynchronize (2)", err);
            return Status::CudaError;
        }
        cudaEventElapsedTime(&pOutStats->gpuTimeMilliseconds, m_eventStart, m_eventStop);
        uint32_t words[NTCB_STATUS_WORDS] = {};
        cudaMemcpy(words, state.status, sizeof words, cudaMemcpyDeviceToHost);
        if (words[0] != 0)
        {
            SetErrorMessage("A bounded wait inside the decode kernel expired (tile %u, layer %u).", words[1], words[2]);
            return Status::CudaError;
        }
    }

    ClearErrorMessage();
    return Status::Ok;
}

} // namespace ntc
