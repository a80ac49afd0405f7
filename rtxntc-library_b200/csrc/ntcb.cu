// C ABI of the decoder: argument checking, weight staging and the kernel launch.
// The declarations and the reference interfaces they stand in for are in include/ntcb.h.

#include "ntcb.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cmath>

#include "decode_kernel.h"
#include "error.h"
#include "network_shape.h"

namespace ntcb
{

thread_local char g_lastError[1024] = "";
std::atomic<uint64_t> g_launchCount{0};
std::atomic<uint32_t> g_networkWaitPolls{kSpinLimit}; // see ntcb_debug_set_network_wait_polls

void SetError(const char* format, ...)
{
    va_list args;
    va_start(args, format);
    vsnprintf(g_lastError, sizeof g_lastError, format, args);
    va_end(args);
}

void ClearError()
{
    g_lastError[0] = 0;
}

int CudaFailure(const char* call, cudaError_t error)
{
    // same wording as the reference's SetCudaErrorMessage (src/Errors.cpp:43-46)
    SetError("Call to %s failed, error code = %s.", call, cudaGetErrorName(error));
    return NTCB_ERR_CUDA;
}

void CountLaunch()
{
    g_launchCount.fetch_add(1, std::memory_order_relaxed);
}

namespace
{

constexpr int kBiasSlots[4] = {16, 32, 48, 32};    // K slots that carry the bias of an int8 layer
constexpr int kWeightOffsets[4] = {kWeightOffset0, kWeightOffset1, kWeightOffset2, kWeightOffset3};
constexpr int kRefWeightOffsets[4] = {kRefWeightOffset0, kRefWeightOffset1, kRefWeightOffset2, kRefWeightOffset3};
constexpr int kRefBiasOffsets[4] = {kRefBiasOffset0, kRefBiasOffset1, kRefBiasOffset2, kRefBiasOffset3};

// `pairedOutput`: the launch stores fp16 channel pairs as 32-bit words, so a mip must start on one.
bool ValidMip(const NtcbMipDesc& m, bool pairedOutput)
{
    return !(m.width < 1 || m.height < 1 || m.hiWidth < 1 || m.hiHeight < 1 || m.loWidth < 1 || m.loHeight < 1 ||
             m.rowBegin < 0 || m.rowEnd > m.height || m.rowBegin > m.rowEnd || (pairedOutput && (m.outOffset & 1)) ||
             m.hiPlane < uint64_t(m.hiWidth) * m.hiHeight || m.loPlane < uint64_t(m.loWidth) * m.loHeight ||
             // the kernels index the pixels of a grid's layers with 32 bits
             m.hiPlane > 0x3FFFFFFFull || m.loPlane > 0x3FFFFFFFull);
}

// The kernel's view of one mip (everything but its place in the tile list).
void FillKernelMip(const NtcbMipDesc& m, int layers, KernelMip& km, int footprintHiBytes = kFootprintHiBytes,
    int footprintLoBytes = kFootprintLoBytes, int tileHeight = kTileHeight)
{
    km.width = m.width;
    km.height = m.height;
    km.rowBegin = m.rowBegin;
    km.rowEnd = m.rowEnd;
    km.hiWidth = m.hiWidth;
    km.hiHeight = m.hiHeight;
    km.loWidth = m.loWidth;
    km.loHeight = m.loHeight;
    km.hiOffset = m.hiOffset;
    km.loOffset = m.loOffset;
    km.hiPlane = m.hiPlane;
    km.loPlane = m.loPlane;
    km.outOffset = m.outOffset;
    km.invWidth = 1.0f / float(m.width);
    km.invHeight = 1.0f / float(m.height);
    km.positionScale = m.positionScale;
    km.positionLod = m.positionLod;
    // Largest footprint a tile can have in each grid: the tap index of the last column (row) minus
    // that of the first is at most floor(31 (7) * grid / mip) + 1, plus the second tap.
    km.strideBytes = layers == 1 ? 8 : layers <= 3 ? 24 : 40;
    const long long hiCapacity = footprintHiBytes / km.strideBytes, loCapacity = footprintLoBytes / km.strideBytes;
    auto footprint = [](int grid, int mip, int span) { return (long long)((long long)span * grid / mip) + 3; };
    const long long hiPixels = footprint(m.hiWidth, m.width, kTileWidth - 1) * footprint(m.hiHeight, m.height, tileHeight - 1);
    const long long loPixels = footprint(m.loWidth, m.width, kTileWidth - 1) * footprint(m.loHeight, m.height, tileHeight - 1);
    km.staged = (hiPixels <= hiCapacity && loPixels <= loCapacity) ? 1 : 0;
    // Tables that do not depend on the tile: with power-of-two sizes all the tap arithmetic is exact in
    // binary32, and when a tile's width and height map to whole latent pixels of both grids (and to whole
    // periods of the positional encoding) moving from tile to tile shifts every tap by an integer.
    auto powerOfTwo = [](long long v) { return v > 0 && (v & (v - 1)) == 0; };
    const float scaledColumns = m.positionScale * float(kTileWidth), scaledRows = m.positionScale * float(tileHeight);
    int exponent = 0;
    const bool scaleIsPowerOfTwo = m.positionScale > 0.f && frexpf(m.positionScale, &exponent) == 0.5f && exponent > -20 && exponent < 20;
    km.invariant = powerOfTwo(m.width) && powerOfTwo(m.height) && powerOfTwo(m.hiWidth) && powerOfTwo(m.hiHeight) &&
                   powerOfTwo(m.loWidth) && powerOfTwo(m.loHeight) && m.width >= kTileWidth && m.height >= tileHeight &&
                   (m.rowBegin % tileHeight) == 0 &&
                   ((long long)kTileWidth * m.hiWidth) % m.width == 0 && ((long long)kTileWidth * m.loWidth) % m.width == 0 &&
                   ((long long)tileHeight * m.hiHeight) % m.height == 0 && ((long long)tileHeight * m.loHeight) % m.height == 0 &&
                   scaledColumns == floorf(scaledColumns) && scaledRows == floorf(scaledRows) && scaleIsPowerOfTwo
        ? 1 : 0;
    km.hiStepX = km.hiStepY = km.loStepX = km.loStepY = 0;
    if (km.invariant)
    {
        km.hiStepX = int((long long)kTileWidth * m.hiWidth / m.width);
        km.loStepX = int((long long)kTileWidth * m.loWidth / m.width);
        km.hiStepY = int((long long)tileHeight * m.hiHeight / m.height);
        km.loStepY = int((long long)tileHeight * m.loHeight / m.height);
    }
    km.tilesX = (m.width + kTileWidth - 1) / kTileWidth;
    km.tilesXMagic = km.tilesX == 1 ? 0u : unsigned((0x100000000ull + km.tilesX - 1) / km.tilesX);
    km.firstTile = 0;
}

} // namespace

// Checks a client's conversion request against a texture set of `channels` channels and packs it
// for the kernels.
int MakeOutputConversion(const NtcbOutputConversion& request, int channels, OutputConversion& out)
{
    out = OutputConversion{};
    if (BytesPerComponent(request.channelFormat) == 0)
    {
        SetError("Unknown channel format %d.", request.channelFormat);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (request.components < 1 || request.components > NTCB_MAX_CHANNELS)
    {
        SetError("components (%d) must be between 1 and %d.", request.components, NTCB_MAX_CHANNELS);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (request.firstChannel < 0 || request.firstChannel >= channels)
    {
        SetError("firstChannel (%d) must be between 0 and %d.", request.firstChannel, channels - 1);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (request.numChannels < 1 || request.numChannels > channels - request.firstChannel)
    {
        SetError("For the provided firstChannel (%d), numChannels (%d) must be between 1 and %d.", request.firstChannel,
            request.numChannels, channels - request.firstChannel);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    out.format = request.channelFormat;
    out.dstChannels = request.components;
    out.dither = request.useDithering != 0;
    for (int c = 0; c < request.numChannels; ++c)
    {
        if (request.srcColorSpaces[c] > NTCB_COLOR_SPACE_HLG || request.dstColorSpaces[c] > NTCB_COLOR_SPACE_HLG)
        {
            SetError("Channel %d names an unknown color space (%d -> %d).", c, int(request.srcColorSpaces[c]),
                int(request.dstColorSpaces[c]));
            return NTCB_ERR_INVALID_ARGUMENT;
        }
        out.srcSpaces |= uint32_t(request.srcColorSpaces[c]) << (2 * c);
        out.dstSpaces |= uint32_t(request.dstColorSpaces[c]) << (2 * c);
    }
    return NTCB_OK;
}

namespace
{

// Number of CTAs that fill the current device, cached per device.
int ResidentCtas(bool fp8, bool converting, int* outCtas, bool reference = false, bool sample = false)
{
    static std::atomic<int> cache[64][6];
    const int variant = reference ? (fp8 ? 4 : sample ? 5 : 3) : converting ? 2 : fp8 ? 1 : 0;
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess)
        return CudaFailure("cudaGetDevice", err);
    if (device >= 0 && device < 64)
    {
        int cached = cache[device][variant].load(std::memory_order_relaxed);
        if (cached > 0)
        {
            *outCtas = cached;
            return NTCB_OK;
        }
    }
    int sms = 0, major = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (err == cudaSuccess)
        err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (err != cudaSuccess)
        return CudaFailure("cudaDeviceGetAttribute", err);
    if (major != 10)
    {
        SetError("The decode kernel needs a device of compute capability 10.x (tcgen05, tensor memory); device %d is %d.x.",
            device, major);
        return NTCB_ERR_CUDA;
    }
    // The kernel is compiled for kCtasPerSmInt8 / kCtasPerSmFp8 resident CTAs (__launch_bounds__), each of which holds
    // kTmemColumns of the SM's 512 tensor-memory columns for its whole lifetime.  (The runtime's
    // occupancy query reports one CTA per SM for kernels that allocate tensor memory, so it is not
    // used here.)
    static_assert(kCtasPerSmInt8 * kTmemColumns <= 512 && kCtasPerSmFp8 * kTmemColumns <= 512 &&
                      kCtasPerSmConverting * kTmemColumns <= 512 && kCtasPerSmRef * kRefTmemColumns <= 512 &&
                      kCtasPerSmRefSample * kRefTmemColumns <= 512 &&
                      kCtasPerSmRefFp8 * kTmemColumns <= 512,
        "resident CTAs must fit into tensor memory");
    const int perSm = reference ? (fp8 ? kCtasPerSmRefFp8 : sample ? kCtasPerSmRefSample : kCtasPerSmRef) : converting ? kCtasPerSmConverting : fp8 ? kCtasPerSmFp8 : kCtasPerSmInt8;
    *outCtas = sms * perSm;
    if (device >= 0 && device < 64)
        cache[device][variant].store(*outCtas, std::memory_order_relaxed);
    return NTCB_OK;
}

} // namespace
} // namespace ntcb

using namespace ntcb;

extern "C"
{

const char* ntcb_last_error(void)
{
    return g_lastError;
}

const char* ntcb_status_string(int status)
{
    switch (status)
    {
    case NTCB_OK: return "Ok";
    case NTCB_ERR_INVALID_ARGUMENT: return "InvalidArgument";
    case NTCB_ERR_CUDA: return "CudaError";
    case NTCB_ERR_FILE_UNRECOGNIZED: return "FileUnrecognized";
    case NTCB_ERR_FILE_INCOMPATIBLE: return "FileIncompatible";
    case NTCB_ERR_UNSUPPORTED: return "Unsupported";
    case NTCB_ERR_OUT_OF_MEMORY: return "OutOfMemory";
    case NTCB_ERR_DEVICE_TIMEOUT: return "DeviceTimeout";
    case NTCB_ERR_INVALID_STATE: return "InvalidState";
    case NTCB_ERR_OUT_OF_RANGE: return "OutOfRange";
    default: return "Unknown";
    }
}

uint64_t ntcb_launch_count(void)
{
    return g_launchCount.load(std::memory_order_relaxed);
}

int ntcb_decode_resident_ctas(int weightMode, int* outCtas)
{
    if (!outCtas || (weightMode != NTCB_WEIGHTS_INT8 && weightMode != NTCB_WEIGHTS_FP8))
    {
        SetError("ntcb_decode_resident_ctas: invalid arguments.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    return ResidentCtas(weightMode == NTCB_WEIGHTS_FP8, false, outCtas);
}

int ntcb_stage_network(const void* blob, size_t blobBytes, int weightMode, void* staged)
{
    if (!blob || !staged)
    {
        SetError("ntcb_stage_network: blob and staged must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const bool fp8 = weightMode == NTCB_WEIGHTS_FP8;
    if (weightMode != NTCB_WEIGHTS_INT8 && weightMode != NTCB_WEIGHTS_FP8)
    {
        SetError("ntcb_stage_network: unknown weight mode %d.", weightMode);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const size_t expected = fp8 ? NTCB_FP8_BLOB_BYTES : NTCB_INT8_BLOB_BYTES;
    if (blobBytes != expected)
    {
        SetError("ntcb_stage_network: the %s weight blob must be %zu bytes, got %zu.", fp8 ? "GenericFP8" : "GenericInt8",
            expected, blobBytes);
        return NTCB_ERR_INVALID_ARGUMENT;
    }

    const uint8_t* src = static_cast<const uint8_t*>(blob);
    uint8_t* dst = static_cast<uint8_t*>(staged);
    memset(dst, 0, kStagedNetworkBytes);

    // Weight matrices: row-major [out][in] bytes in the file (src/Quantizer.cu:144-146), laid out
    // one after another (src/WeightLayout.cpp:170-176) -> K-major core matrices, K zero-padded.
    size_t offset = 0;
    for (int layer = 0; layer < 4; ++layer)
    {
        const int nin = kLayerInputs[layer], nout = kLayerOutputs[layer];
        uint8_t* w = dst + kWeightOffsets[layer];
        for (int n = 0; n < nout; ++n)
            for (int k = 0; k < nin; ++k)
            {
                const uint8_t byte = src[offset + size_t(n) * nin + k];
                w[(k / 16) * (nout * 16) + n * 16 + (k % 16)] = byte;
            }
        offset += size_t(nin) * nout;
    }

    float* scale = reinterpret_cast<float*>(dst + kScaleOffset);
    for (int i = 0; i < 4 * 64; ++i)
        scale[i] = 1.f;
    int32_t fileBias[4][64] = {};
    if (!fp8)
    {
        // all fp32 scale vectors, then all int32 bias vectors (src/WeightLayout.cpp:228-238)
        for (int layer = 0; layer < 4; ++layer)
        {
            memcpy(scale + layer * 64, src + offset, 4u * kLayerOutputs[layer]);
            offset += 4u * kLayerOutputs[layer];
        }
        for (int layer = 0; layer < 4; ++layer)
        {
            memcpy(fileBias[layer], src + offset, 4u * kLayerOutputs[layer]);
            offset += 4u * kLayerOutputs[layer];
        }
    }
    else
    {
        // fp16 biases of layers 0-2, then the fp32 scale and int32 bias of the int8 output layer
        // (src/WeightLayout.cpp:240-255)
        for (int layer = 0; layer < 3; ++layer)
        {
            memcpy(dst + kBiasOffset + layer * 256, src + offset, 2u * kLayerOutputs[layer]);
            offset += 2u * kLayerOutputs[layer];
        }
        memcpy(scale + 3 * 64, src + offset, 4u * 16);
        offset += 4u * 16;
        memcpy(fileBias[3], src + offset, 4u * 16);
        offset += 4u * 16;
    }

    // Int8 layers: the bias the kernel needs, and its decomposition over the bias slots.
    bool fits = !fp8; // the FP8 network's only int8 layer (16 outputs) keeps the table
    int32_t bias[4][64] = {};
    for (int layer = fp8 ? 3 : 0; layer < 4; ++layer)
    {
        for (int n = 0; n < kLayerOutputs[layer]; ++n)
        {
            const long long adjusted = fileBias[layer][n];
            if (adjusted > 0x7FFFFFFFll || adjusted < -0x7FFFFFFFll)
            {
                SetError("ntcb_stage_network: the bias of output %d of layer %d is out of range.", n, layer);
                return NTCB_ERR_OUT_OF_RANGE;
            }
            bias[layer][n] = int32_t(adjusted);
            const int slots = kBiasSlots[layer];
            // (layer 2's 48 slots span two K steps: one of them is the first step's input-1 slot)
            if (std::llabs(adjusted) > (long long)kBiasSlotValue * 127 * (slots - (slots > 32 ? 2 : 1)) + 63)
                fits = false;
        }
    }
    uint32_t* flags = reinterpret_cast<uint32_t*>(dst + kFlagsOffset);
    for (int layer = fp8 ? 3 : 0; layer < 4; ++layer)
    {
        const int nout = kLayerOutputs[layer];
        if (!fits)
        {
            memcpy(dst + kBiasOffset + layer * 256, bias[layer], 4u * nout);
            continue;
        }
        uint8_t* w = dst + kWeightOffsets[layer];
        const int firstSlot = kLayerInputs[layer]; // layers 0 and 2: the 16 padding slots of their 48 inputs come first
        for (int n = 0; n < nout; ++n)
        {
            // bias = kBiasSlotValue * q + r with |r| <= 63; q spread over the first slots - 1 slots in
            // steps of at most 127, r in the last slot (whose input is 1)
            const int value = bias[layer][n];
            int q = (value >= 0 ? value + kBiasSlotValue / 2 : value - kBiasSlotValue / 2) / kBiasSlotValue;
            const int r = value - q * kBiasSlotValue;
            for (int slot = 0; slot < kBiasSlots[layer]; ++slot)
            {
                // the constant input is 1 in the last slot of a K step and kBiasSlotValue elsewhere; the
                // remainder goes to the last slot of all, the other slots of input 1 stay empty
                const int k = firstSlot + slot;
                int part;
                if (slot == kBiasSlots[layer] - 1)
                    part = r;
                else if ((k & 31) == 31)
                    part = 0;
                else
                {
                    part = q > 127 ? 127 : q < -127 ? -127 : q;
                    q -= part;
                }
                w[(k / 16) * (nout * 16) + n * 16 + (k % 16)] = uint8_t(int8_t(part));
            }
        }
    }
    flags[0] = fits ? 0u : kFlagBiasTable;
    if (offset != expected)
    {
        SetError("ntcb_stage_network: internal layout mismatch.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    ClearError();
    return NTCB_OK;
}

int ntcb_stage_network_reference(const void* blob, size_t blobBytes, int weightMode, void* staged)
{
    if (!blob || !staged)
    {
        SetError("ntcb_stage_network_reference: blob and staged must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const bool fp8 = weightMode == NTCB_WEIGHTS_FP8;
    if (weightMode != NTCB_WEIGHTS_INT8 && weightMode != NTCB_WEIGHTS_FP8)
    {
        SetError("ntcb_stage_network_reference: unknown weight mode %d.", weightMode);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const size_t expected = fp8 ? NTCB_FP8_BLOB_BYTES : NTCB_INT8_BLOB_BYTES;
    if (blobBytes != expected)
    {
        SetError("ntcb_stage_network_reference: the %s weight blob must be %zu bytes, got %zu.",
            fp8 ? "GenericFP8" : "GenericInt8", expected, blobBytes);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const uint8_t* src = static_cast<const uint8_t*>(blob);
    uint8_t* dst = static_cast<uint8_t*>(staged);
    memset(dst, 0, kRefNetworkBytes);

    // where the sections of the blob start (src/WeightLayout.cpp:170-176, 228-255)
    size_t weightStart[4], offset = 0;
    for (int layer = 0; layer < 4; ++layer)
    {
        weightStart[layer] = offset;
        offset += size_t(kLayerInputs[layer]) * kLayerOutputs[layer];
    }
    const uint8_t* scaleStart[4] = {};
    const uint8_t* biasStart[4] = {};
    if (!fp8)
    {
        for (int layer = 0; layer < 4; ++layer) { scaleStart[layer] = src + offset; offset += 4u * kLayerOutputs[layer]; }
        for (int layer = 0; layer < 4; ++layer) { biasStart[layer] = src + offset; offset += 4u * kLayerOutputs[layer]; }
    }
    else
    {
        for (int layer = 0; layer < 3; ++layer) { biasStart[layer] = src + offset; offset += 2u * kLayerOutputs[layer]; }
        scaleStart[3] = src + offset; offset += 4u * 16;
        biasStart[3] = src + offset; offset += 4u * 16;
    }
    if (offset != expected)
    {
        SetError("ntcb_stage_network_reference: internal layout mismatch.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }

    const float inputScale = 127.5f;             // tin::InputQuant::scale (src/tin/tin_mlp.h:42-45)
    const float activationStep = 3.1875f / 255.f; // tin::ActHGELUClamp::step (src/tin/tin_activation.h:109-121)
    const int activationBias = -113;             // tin::ActHGELUClamp::bias
    auto halfBits = [](float value) { return static_cast<__half_raw>(__float2half_rn(value)).x; };
    for (int layer = 0; layer < 4; ++layer)
    {
        const int nin = kLayerInputs[layer], nout = kLayerOutputs[layer];
        uint16_t* weights = reinterpret_cast<uint16_t*>(dst + kRefWeightOffsets[layer]);
        // FP8 networks: column 0 of the layer's N x 16 bias-step operand; Int8 networks: column `layer` of the
        // one 64 x 8 matrix all layers share
        uint16_t* biasStep = fp8 ? reinterpret_cast<uint16_t*>(dst + kRefBiasOffsets[layer])
                                 : reinterpret_cast<uint16_t*>(dst + kRefInt8BiasOffset) + layer;
        const bool layerFp8 = fp8 && layer < 3;
        for (int n = 0; n < nout; ++n)
        {
            uint16_t bias;
            if (layerFp8)
            {
                // UnquantizeColumnFP8 (src/Quantizer.cu:384-408) turns the e4m3 weights into the same numbers
                // in binary16, so the kernel multiplies the e4m3 bytes themselves.  Each 16-wide K step s gets
                // its own N x 32 byte matrix (K-major core matrices: byte (n, j) at (j / 16) * (N * 16) + n * 16
                // + j % 16) that holds the 16 weights of the step at their place inside the 32-wide chunk
                // s / 2 and zeros in the other half: 16 real products per 32-product instruction.
                uint8_t* bytes = dst + kRefWeightOffsets[layer];
                for (int k = 0; k < nin; ++k)
                {
                    const int step = k / 16, j = k % 32;
                    bytes[size_t(step) * nout * 32 + (j / 16) * (nout * 16) + n * 16 + (j % 16)] =
                        src[weightStart[layer] + size_t(n) * nin + k];
                }
                memcpy(&bias, biasStart[layer] + 2u * n, 2);
            }
            else
            {
                // UnquantizeColumnInt8 (src/Quantizer.cu:325-382), same fp32 operation order
                float layerScale;
                int32_t integerBias;
                memcpy(&layerScale, scaleStart[layer] + 4u * n, 4);
                memcpy(&integerBias, biasStart[layer] + 4u * n, 4);
                float layerBias = float(integerBias) * layerScale;
                layerScale *= (layer == 0) ? inputScale : (1.f / activationStep);
                int integerWeightSum = 0;
                for (int k = 0; k < nin; ++k)
                {
                    const int q = int8_t(src[weightStart[layer] + size_t(n) * nin + k]);
                    weights[(k / 8) * (nout * 8) + n * 8 + (k % 8)] = halfBits(float(q) * layerScale);
                    integerWeightSum += q;
                }
                if (layer != 0)
                    layerBias = fmaf(float(integerWeightSum * activationBias) * layerScale, activationStep, layerBias);
                bias = halfBits(layerBias);
            }
            biasStep[n * 8] = bias;
        }
    }
    ClearError();
    return NTCB_OK;
}

uint32_t ntcb_debug_set_network_wait_polls(uint32_t polls)
{
    return g_networkWaitPolls.exchange(polls, std::memory_order_relaxed);
}

int ntcb_decode(const NtcbDecodeParams* p, void* stream)
{
    if (!p || !p->latents || !p->network || !p->out || !p->status)
    {
        SetError("ntcb_decode: params, latents, network, out and status must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (p->numMips < 1 || p->numMips > NTCB_MAX_MIPS)
    {
        SetError("ntcb_decode: numMips (%d) must be 1..%d.", p->numMips, NTCB_MAX_MIPS);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (p->numFeatures < 4 || p->numFeatures > 16 || (p->numFeatures & 3))
    {
        SetError("ntcb_decode: numFeatures (%d) must be 4, 8, 12 or 16.", p->numFeatures);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (p->channels < 2 || p->channels > 16 || (p->channels & 1))
    {
        SetError("ntcb_decode: channels (%d) must be even and 2..16.", p->channels);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (p->weightMode != NTCB_WEIGHTS_INT8 && p->weightMode != NTCB_WEIGHTS_FP8)
    {
        SetError("ntcb_decode: unknown weight mode %d.", p->weightMode);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (p->outputLayout != NTCB_LAYOUT_PLANAR_PAIRS && p->outputLayout != NTCB_LAYOUT_INTERLEAVED)
    {
        SetError("ntcb_decode: unknown output layout %d.", p->outputLayout);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if ((reinterpret_cast<uintptr_t>(p->network) & 15) || (reinterpret_cast<uintptr_t>(p->out) & 3) ||
        (reinterpret_cast<uintptr_t>(p->latents) & 1))
    {
        SetError("ntcb_decode: network must be 16-byte aligned, out 4-byte aligned, latents 2-byte aligned.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }

    if (p->numerics != NTCB_NUMERICS_EXACT && p->numerics != NTCB_NUMERICS_REFERENCE)
    {
        SetError("ntcb_decode: unknown numerics %d.", p->numerics);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const bool reference = p->numerics == NTCB_NUMERICS_REFERENCE;
    KernelParams k{};
    if (p->conversion)
    {
        int rc = MakeOutputConversion(*p->conversion, p->channels, k.conversion);
        if (rc != NTCB_OK)
            return rc;
        k.convert = 1;
        k.firstChannel = p->conversion->firstChannel;
        k.numChannels = p->conversion->numChannels;
    }
    k.latents = p->latents;
    k.network = static_cast<const uint8_t*>(p->network);
    k.out = static_cast<__half*>(p->out);
    k.status = p->status;
    k.numLayers = p->numFeatures / 4;
    k.channels = p->channels;
    k.outputLayout = p->outputLayout;
    long long tiles = 0;
    int used = 0;
    for (int i = 0; i < p->numMips; ++i)
    {
        const NtcbMipDesc& m = p->mips[i];
        if (!ValidMip(m, k.convert == 0))
        {
            SetError("ntcb_decode: mip %d has invalid dimensions, row range or offsets.", i);
            return NTCB_ERR_INVALID_ARGUMENT;
        }
        if (k.convert && m.outOffset % uint64_t(k.conversion.dstChannels))
        {
            SetError("ntcb_decode: outOffset of mip %d must be a multiple of the %d components of a converted pixel.", i,
                k.conversion.dstChannels);
            return NTCB_ERR_INVALID_ARGUMENT;
        }
        if (k.convert)
        {
            // the converting epilogue stores a pixel with the widest vector its size allows
            const size_t componentBytes = size_t(BytesPerComponent(k.conversion.format));
            const size_t alignment = ConvertedPixelAlignment(size_t(k.conversion.dstChannels) * componentBytes);
            if ((reinterpret_cast<uintptr_t>(p->out) + size_t(m.outOffset) * componentBytes) % alignment)
            {
                SetError("ntcb_decode: converted pixels of %zu bytes need mip %d to start at a multiple of %zu bytes.",
                    size_t(k.conversion.dstChannels) * componentBytes, i, alignment);
                return NTCB_ERR_INVALID_ARGUMENT;
            }
        }
        else if (uint64_t(m.width) * uint64_t(m.height) * uint64_t(p->channels) > 0xFFFFFFFFull)
        {
            // the kernels index the elements of a mip with 32 bits
            SetError("ntcb_decode: mip %d has %llu x %d values; a mip may hold at most 2^32 - 1.", i,
                (unsigned long long)m.width * (unsigned long long)m.height, p->channels);
            return NTCB_ERR_OUT_OF_RANGE;
        }
        if (k.convert && uint64_t(m.width) * uint64_t(m.height) > 0xFFFFFFFFull)
        {
            SetError("ntcb_decode: mip %d has more than 2^32 - 1 pixels.", i);
            return NTCB_ERR_OUT_OF_RANGE;
        }
        if (m.rowBegin == m.rowEnd)
            continue; // nothing of this mip belongs to this launch
        KernelMip& km = k.mips[used++];
        const int tileHeight = reference ? kRefTileHeight : kTileHeight;
        if (reference)
            FillKernelMip(m, p->numFeatures / 4, km, kRefFootprintHiBytes,
                p->weightMode == NTCB_WEIGHTS_FP8 ? kRefFootprintLoBytes : kRefInt8FootprintLoBytes, kRefTileHeight);
        else
            FillKernelMip(m, p->numFeatures / 4, km);
        km.firstTile = int(tiles);
        km.storeBytes = 4;
        if (!k.convert && p->outputLayout == NTCB_LAYOUT_INTERLEAVED)
        {
            const uintptr_t address = reinterpret_cast<uintptr_t>(p->out) + size_t(m.outOffset) * 2;
            const size_t texelBytes = size_t(p->channels) * 2;
            km.storeBytes = !(address & 15) && !(texelBytes & 15) ? 16 : !(address & 7) && !(texelBytes & 7) ? 8 : 4;
        }
        const long long mipTiles = (long long)km.tilesX * ((m.rowEnd - m.rowBegin + tileHeight - 1) / tileHeight);
        if (mipTiles * km.tilesX >= 0x100000000ll)
        {
            SetError("ntcb_decode: mip %d is too large for one launch.", i);
            return NTCB_ERR_OUT_OF_RANGE;
        }
        tiles += mipTiles;
        if (tiles > 0x7FFFFFFF)
        {
            SetError("ntcb_decode: too many tiles for one launch.");
            return NTCB_ERR_OUT_OF_RANGE;
        }
    }
    ClearError();
    if (used == 0)
        return NTCB_OK;
    k.numMips = used;
    k.totalTiles = int(tiles);
    k.loadWaitPolls = g_networkWaitPolls.load(std::memory_order_relaxed);

    const bool fp8 = p->weightMode == NTCB_WEIGHTS_FP8;
    int resident = 0;
    int rc = ResidentCtas(fp8, k.convert != 0, &resident, reference);
    if (rc != NTCB_OK)
        return rc;
    const int ctas = k.totalTiles < resident ? k.totalTiles : resident;
    cudaError_t err = reference ? LaunchDecodeRef(k, fp8, ctas, static_cast<cudaStream_t>(stream)) : LaunchDecode(k, fp8, ctas, static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess)
        return CudaFailure("DecodeKernel launch", err);
    CountLaunch();
    return NTCB_OK;
}

int ntcb_sample(const NtcbSampleParams* p, void* stream)
{
    if (!p || !p->latents || !p->network || !p->status || ((!p->queries || !p->out) && p->numQueries))
    {
        SetError("ntcb_sample: params, latents, network, queries, out and status must not be NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (p->numMips < 1 || p->numMips > NTCB_MAX_MIPS || p->numFeatures < 4 || p->numFeatures > 16 || (p->numFeatures & 3) ||
        p->channels < 2 || p->channels > 16 || (p->channels & 1) ||
        (p->weightMode != NTCB_WEIGHTS_INT8 && p->weightMode != NTCB_WEIGHTS_FP8))
    {
        SetError("ntcb_sample: invalid mip count, feature count, channel count or weight mode.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (p->numerics != NTCB_NUMERICS_EXACT && p->numerics != NTCB_NUMERICS_REFERENCE)
    {
        SetError("ntcb_sample: unknown numerics %d.", p->numerics);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (p->latentLayout != NTCB_LATENTS_PLANAR && p->latentLayout != NTCB_LATENTS_INTERLEAVED)
    {
        SetError("ntcb_sample: unknown latent layout %d.", p->latentLayout);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (p->latentLayout == NTCB_LATENTS_INTERLEAVED && (reinterpret_cast<uintptr_t>(p->latents) & 7))
    {
        SetError("ntcb_sample: interleaved latents must be 8-byte aligned.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    const bool reference = p->numerics == NTCB_NUMERICS_REFERENCE;
    if ((reinterpret_cast<uintptr_t>(p->network) & 15) || (reinterpret_cast<uintptr_t>(p->out) & 3) ||
        (reinterpret_cast<uintptr_t>(p->queries) & 3))
    {
        SetError("ntcb_sample: network must be 16-byte aligned, out and queries 4-byte aligned.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    SampleParams k{};
    k.latents = p->latents;
    k.network = static_cast<const uint8_t*>(p->network);
    k.queries = p->queries;
    k.out = static_cast<__half*>(p->out);
    k.status = p->status;
    k.numQueries = p->numQueries;
    k.numMips = p->numMips;
    k.numLayers = p->numFeatures / 4;
    k.channels = p->channels;
    k.interleaved = p->latentLayout == NTCB_LATENTS_INTERLEAVED;
    for (int i = 0; i < p->numMips; ++i)
    {
        NtcbMipDesc m = p->mips[i];
        m.rowBegin = 0;
        m.rowEnd = m.height;
        m.outOffset = 0;
        if (!ValidMip(m, false))
        {
            SetError("ntcb_sample: mip %d has invalid dimensions or offsets.", i);
            return NTCB_ERR_INVALID_ARGUMENT;
        }
        FillKernelMip(m, k.numLayers, k.mips[i]);
        if (k.interleaved)
        {
            // the grid's place in the pixel-major copy: slots of 1, 2 or 4 elements per pixel
            const unsigned long long layers = (unsigned long long)k.numLayers, slot = k.numLayers == 3 ? 4 : layers;
            if (m.hiOffset % layers || m.loOffset % layers)
            {
                SetError("ntcb_sample: mip %d: the offset of a grid is not a multiple of the layer count.", i);
                return NTCB_ERR_INVALID_ARGUMENT;
            }
            k.mips[i].hiOffset = m.hiOffset / layers * slot;
            k.mips[i].loOffset = m.loOffset / layers * slot;
        }
    }
    k.loadWaitPolls = g_networkWaitPolls.load(std::memory_order_relaxed);
    ClearError();
    if (p->numQueries == 0)
        return NTCB_OK;
    const bool fp8 = p->weightMode == NTCB_WEIGHTS_FP8;
    int resident = 0;
    int rc = ResidentCtas(fp8, false, &resident, reference, true);
    if (rc != NTCB_OK)
        return rc;
    const unsigned long long perCta = reference ? kRefThreadsPerCta : kThreadsPerCta;
    const unsigned long long tiles = (p->numQueries + perCta - 1) / perCta;
    const int ctas = tiles < (unsigned long long)resident ? int(tiles) : resident;
    cudaError_t err = reference ? LaunchSampleRef(k, fp8, ctas, static_cast<cudaStream_t>(stream))
                                : LaunchSample(k, fp8, ctas, static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess)
        return CudaFailure("SampleKernel launch", err);
    CountLaunch();
    return NTCB_OK;
}

} // extern "C"
