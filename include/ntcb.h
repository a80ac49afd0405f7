/* ntcb.h - C ABI of the B200-native NTC decoder (libntcb200.so).
 *
 * This is the drop-in boundary for ONE path of LibNTC: CUDA decompression of a neural-compressed
 * texture set (latents -> 48-wide input -> 48-64-48-32-16 MLP -> fp16 texels).  Every entry point
 * takes plain pointers and sizes; each comment names the reference interface it replaces
 * (paths relative to the reference project root).
 *
 * Conventions: functions return 0 (NTCB_OK) or a negative NtcbStatus; ntcb_last_error() returns a
 * thread-local message for the last failing call on the calling thread (the reference's
 * ntc::GetLastErrorMessage convention, src/Errors.cpp:21-52).  Nothing throws.  Device work is
 * issued on the CUDA stream the caller passes (a cudaStream_t cast to void*; NULL = the legacy
 * default stream the reference always uses).  There is no CPU fallback: without a usable GPU the
 * compute entry points fail with NTCB_ERR_CUDA.
 */
#ifndef NTCB_H
#define NTCB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NTCB_MAX_CHANNELS 16     /* NTC_MAX_CHANNELS, include/libntc/shaders/InferenceConstants.h:23 */
#define NTCB_MAX_MIPS 16         /* NTC_MAX_MIPS, include/libntc/shaders/InferenceConstants.h:22 */
#define NTCB_MAX_NEURAL_MIPS 8   /* NTC_MAX_NEURAL_MIPS, :24 */
#define NTCB_INT8_BLOB_BYTES 9472 /* GenericInt8 weight blob, src/WeightLayout.cpp:142-268 */
#define NTCB_FP8_BLOB_BYTES 8608  /* GenericFP8 weight blob */
#define NTCB_STAGED_NETWORK_BYTES 14864 /* size of the device image ntcb_stage_network produces */
#define NTCB_STAGED_REFERENCE_NETWORK_BYTES 21504 /* ... and of the one ntcb_stage_network_reference produces */
#define NTCB_STATUS_WORDS 4

typedef enum NtcbStatus
{
    NTCB_OK = 0,
    NTCB_ERR_INVALID_ARGUMENT = -1, /* ntc::Status::InvalidArgument */
    NTCB_ERR_CUDA = -2,             /* ntc::Status::CudaError / CudaUnavailable */
    NTCB_ERR_FILE_UNRECOGNIZED = -3,/* ntc::Status::FileUnrecognized */
    NTCB_ERR_FILE_INCOMPATIBLE = -4,/* ntc::Status::FileIncompatible */
    NTCB_ERR_UNSUPPORTED = -5,      /* ntc::Status::Unsupported (e.g. GDeflate-compressed views) */
    NTCB_ERR_OUT_OF_MEMORY = -6,    /* ntc::Status::OutOfMemory */
    NTCB_ERR_DEVICE_TIMEOUT = -7,   /* a bounded wait inside a kernel gave up; see the status words */
    NTCB_ERR_INVALID_STATE = -8,    /* ntc::Status::InvalidState */
    NTCB_ERR_OUT_OF_RANGE = -9      /* ntc::Status::OutOfRange */
} NtcbStatus;

/* How the matrix products of the decoder network are accumulated.
   REFERENCE (the default everywhere): binary16 weights, activations and accumulators rounded once per
   16 products, as the reference's CUDA decoder does (src/Inference.cu:46-136,
   src/tin/tin_mma.h:126-163): the output reproduces that decoder's bit for bit.
   EXACT: int8 x int8 -> int32 and e4m3 x e4m3 -> fp32 without intermediate rounding, as the
   reference's integer inference path does (include/libntc/shaders/Inference.hlsli:133-182). */
typedef enum NtcbNumerics
{
    NTCB_NUMERICS_REFERENCE = 0,
    NTCB_NUMERICS_EXACT = 1
} NtcbNumerics;

/* Which weight set decodes: the `useInt8Weights` argument of ITextureSet::Decompress
   (include/libntc/ntc.h:933; src/TextureSet.cpp:1812,1826). */
typedef enum NtcbWeightMode
{
    NTCB_WEIGHTS_INT8 = 0, /* GenericInt8: four int8 layers, int32 accumulation */
    NTCB_WEIGHTS_FP8 = 1   /* GenericFP8: e4m3 layers 0-2 (fp32 accumulation), int8 output layer */
} NtcbWeightMode;

/* Layout of the decoded texels. */
typedef enum NtcbOutputLayout
{
    /* The reference's internal texture-data layout (src/RegressionKernels.h:36-45,
       src/ImageProcessing.h:20-33): per mip, half index = y*W*C + (c & ~1)*W + 2*x + (c & 1). */
    NTCB_LAYOUT_PLANAR_PAIRS = 0,
    /* Pixel-interleaved [y][x][c], what ITextureSet::ReadChannels(FLOAT16, pixelStride = 2*C)
       hands back (src/TextureSet.cpp:915-985). */
    NTCB_LAYOUT_INTERLEAVED = 1
} NtcbOutputLayout;

/* ntc::ChannelFormat (include/libntc/ntc.h:227-236) */
#define NTCB_CHANNEL_FORMAT_UNORM8 1
#define NTCB_CHANNEL_FORMAT_UNORM16 2
#define NTCB_CHANNEL_FORMAT_FLOAT16 3
#define NTCB_CHANNEL_FORMAT_FLOAT32 4
#define NTCB_CHANNEL_FORMAT_UINT32 5
/* ntc::ColorSpace (include/libntc/ntc.h:251-256) */
#define NTCB_COLOR_SPACE_LINEAR 0
#define NTCB_COLOR_SPACE_SRGB 1
#define NTCB_COLOR_SPACE_HLG 2

/* How decoded fp16 channels become the client's pixel components: the arithmetic of the
   reference's CopyImageKernel on its way out of a texture set (src/ImageProcessing.cu:86-164,
   220-266; src/CudaUtils.h:63-184).  Each pixel gets `components` values of `channelFormat`,
   tightly interleaved: component c < numChannels is channel firstChannel + c, taken out of
   srcColorSpaces[c], encoded to dstColorSpaces[c], dithered (UNORM formats, when useDithering) and
   rounded; the components past numChannels are 0, component 3 is 1. */
typedef struct NtcbOutputConversion
{
    int32_t channelFormat;  /* NTCB_CHANNEL_FORMAT_* */
    int32_t components;     /* 1..16 */
    int32_t firstChannel, numChannels;
    int32_t useDithering;
    int32_t reserved;
    uint8_t srcColorSpaces[NTCB_MAX_CHANNELS]; /* per requested channel: the colour space it is stored in */
    uint8_t dstColorSpaces[NTCB_MAX_CHANNELS]; /* per requested channel: the colour space to encode to */
} NtcbOutputConversion;

/* One colour mip to decode; mirrors the per-mip fields of InferenceKernelParams
   (src/RegressionCommon.h:55-80) as TextureSet::Decompress fills them (src/TextureSet.cpp:1806-1829). */
typedef struct NtcbMipDesc
{
    int32_t width, height;            /* referenceWidth / referenceHeight */
    int32_t hiWidth, hiHeight;        /* highResLatentWidth / Height */
    int32_t loWidth, loHeight;        /* lowResLatentWidth / Height */
    uint64_t hiOffset, loOffset;      /* element (uint16) offset of layer 0 of each grid in `latents` */
    uint64_t hiPlane, loPlane;        /* pixels per layer of each grid (distance between layers) */
    float positionScale, positionLod; /* src/TextureSet.cpp:457-462 */
    uint64_t outOffset;               /* element (fp16) offset of this mip in `out` */
    int32_t rowBegin, rowEnd;         /* rows [rowBegin, rowEnd) are decoded: the unit of tile-row sharding */
} NtcbMipDesc;

/* Everything one decode launch needs; replaces cuda::Inference(InferenceKernelParams) called once
   per mip (src/Inference.cu:159-165) together with its prologue kernels cuda::UnpackLatents
   (src/Quantizer.cu:574-586) and cuda::ConvertNetworkFromQuantizedToFp16 (src/Quantizer.cu:462-480),
   whose work happens inside the decode kernel / ntcb_stage_network. */
typedef struct NtcbDecodeParams
{
    const uint16_t* latents; /* device: BGRA4 latent pixels, for each neural mip, for each layer, rows
                                (the reference's encoded-pixel order, src/FeatureGridHost.cpp:140-155) */
    const void* network;     /* device: NTCB_STAGED_REFERENCE_NETWORK_BYTES produced by
                                ntcb_stage_network_reference (NTCB_NUMERICS_REFERENCE), or NTCB_STAGED_NETWORK_BYTES
                                produced by ntcb_stage_network (NTCB_NUMERICS_EXACT) */
    void* out;               /* device, 4-byte aligned: fp16 texels, or converted pixels when `conversion` is set.
                                A mip may hold at most 2^32 - 1 values (width x height x channels: the
                                kernels index a mip with 32 bits); a larger one is refused with
                                NTCB_ERR_OUT_OF_RANGE */
    uint32_t* status;        /* device: NTCB_STATUS_WORDS words, zeroed by the caller before the launch;
                                word 0 != 0 after the kernel means a bounded wait expired */
    int32_t numMips;
    int32_t numFeatures;     /* 4, 8, 12 or 16 */
    int32_t channels;        /* even, 2..16 */
    int32_t weightMode;      /* NtcbWeightMode, must match the staged network */
    int32_t outputLayout;    /* NtcbOutputLayout (ignored when `conversion` is set) */
    int32_t numerics;        /* NtcbNumerics */
    NtcbMipDesc mips[NTCB_MAX_MIPS];
    /* NULL: fp16 texels in `outputLayout`.  Otherwise the kernel's epilogue converts every texel as
       ITextureSet::ReadChannels would after Decompress (src/TextureSet.cpp:915-985) and writes
       pixel-interleaved rows without padding: the fp16 copy of the texels is never stored.  In this
       mode mips[i].outOffset counts components of the channel format (bytes / bytes-per-component)
       and must be a multiple of `components`; the dither pattern of a mip is seeded per pixel with
       x + y * width, as a full-mip ReadChannels does.  A pixel is stored with the widest vector its
       size (components x bytes per component) is a multiple of - 16, 8, 4, 2 or 1 bytes - so the
       first pixel of every mip (`out` plus its outOffset) must be aligned to that width; a request
       that is not is refused with NTCB_ERR_INVALID_ARGUMENT before anything is launched. */
    const NtcbOutputConversion* conversion;
} NtcbDecodeParams;

/* Thread-local message of the last failing call on this thread; never NULL.
   Replaces ntc::GetLastErrorMessage (include/libntc/ntc.h:1337). */
const char* ntcb_last_error(void);

/* Textual name of a status code.  Replaces ntc::StatusToString (include/libntc/ntc.h:1341). */
const char* ntcb_status_string(int status);

/* Host only, for NTCB_NUMERICS_EXACT.  Converts a row-major weight blob as stored in NTC files
   (GenericInt8, NTCB_INT8_BLOB_BYTES, or GenericFP8, NTCB_FP8_BLOB_BYTES) into the image the decode
   kernel copies to shared memory: int8 / e4m3 matrices in the tensor core's K-major core-matrix order with K
   padded to a multiple of 32, fp32 scales, int32 / fp16 biases.  `staged` receives
   NTCB_STAGED_NETWORK_BYTES; the caller uploads it.  Replaces the weight preparation of
   cuda::ConvertNetworkFromQuantizedToFp16 (src/Quantizer.cu:325-480). */
int ntcb_stage_network(const void* blob, size_t blobBytes, int weightMode, void* staged);

/* Host only.  The same for NTCB_NUMERICS_REFERENCE: rebuilds the binary16 weights and biases exactly
   as cuda::ConvertNetworkFromQuantizedToFp16 does (UnquantizeColumnInt8 / UnquantizeColumnFP8,
   src/Quantizer.cu:325-408, same fp32 operation order) and lays them out for the binary16 tensor-core
   path.  `staged` receives NTCB_STAGED_REFERENCE_NETWORK_BYTES. */
int ntcb_stage_network_reference(const void* blob, size_t blobBytes, int weightMode, void* staged);

/* Decodes the mips (and row ranges) listed in `params` with one kernel launch on `stream`.
   Asynchronous; the caller synchronises and may then read `status`.  Allocates nothing and waits for
   nothing, so a sequence of decodes can be captured in a CUDA graph and replayed - after one ordinary
   call of the same kind (weight mode, numerics, latent layer count, conversion or not) on the device:
   the first use of a kernel sets a function attribute. */
int ntcb_decode(const NtcbDecodeParams* params, void* stream);

/* Inference on sample: evaluates individual texels instead of whole mips.  Query q is
   (u, v, lod) = queries[3q .. 3q+2]; it selects mip = clamp(floor(lod), 0, numMips - 1) and the texel
   x = min(floor(u * width), width - 1), y = min(floor(v * height), height - 1) of that mip, which is
   decoded exactly as ntcb_decode would decode it; out[q * channels + c] receives the fp16 channels.
   The reference exposes this only to shaders, as NtcSampleTextureSet(texel, mipLevel)
   (include/libntc/shaders/Inference.hlsli:282-357) fed by IContext::MakeInferenceData
   (src/Context.cpp:864-922); the (u, v, lod) -> (texel, mip) rule above is this library's. */
typedef enum NtcbLatentLayout
{
    NTCB_LATENTS_PLANAR = 0,     /* the file's order: per grid, layer after layer (NtcbDecodeParams::latents) */
    NTCB_LATENTS_INTERLEAVED = 1 /* the pixel-major copy made by ntcb_interleave_latents */
} NtcbLatentLayout;

typedef struct NtcbSampleParams
{
    const uint16_t* latents; /* device, as in NtcbDecodeParams */
    const void* network;     /* device, as in NtcbDecodeParams */
    const float* queries;    /* device: numQueries x 3 floats */
    void* out;               /* device: numQueries x channels fp16 */
    uint32_t* status;        /* device: NTCB_STATUS_WORDS zeroed words */
    uint64_t numQueries;
    int32_t numMips;
    int32_t numFeatures;
    int32_t channels;
    int32_t weightMode;
    int32_t numerics;        /* NtcbNumerics; selects the network image as in NtcbDecodeParams */
    int32_t latentLayout;    /* NtcbLatentLayout: what `latents` points to (0: the file's order) */
    NtcbMipDesc mips[NTCB_MAX_MIPS]; /* outOffset, rowBegin and rowEnd are ignored; the grids are described as
                                        they lie in the file's order, whatever latentLayout says */
} NtcbSampleParams;

/* One kernel launch on `stream` for all queries.  Asynchronous; allocates nothing. */
int ntcb_sample(const NtcbSampleParams* params, void* stream);

/* Re-lays packed latents for inference on sample (NTCB_LATENTS_INTERLEAVED).  In the copy a latent pixel is one
   slot that holds its layers side by side: 1, 2 or 4 elements for 4, 8 and 12 / 16 features (the fourth element
   of a 12-feature slot is zero), and the grid that starts at element `offset` of `latents` starts at element
   offset / layers * slot of `interleaved`.  `interleaved` is a device buffer, 8-byte aligned, of as many elements
   as `latents` - of 4/3 as many with 12 features.  A bilinear tap of a random query is then ONE aligned load of
   8 (4) bytes instead of one 2-byte load per layer from planes that lie far apart, which is what bounds that
   kernel (the L1's rate of serving scattered words).  The answers are the same bits.  The
   grids are taken from `mips` as ntcb_sample reads them (colour mips that share a grid name it twice; it is
   converted once); every grid's offset must be a multiple of the layer count.  One launch on `stream`;
   asynchronous; allocates nothing.  No counterpart in the reference, whose sampling path is a shader reading the
   file's planes. */
int ntcb_interleave_latents(const uint16_t* latents, uint16_t* interleaved, const NtcbMipDesc* mips, int numMips,
    int numFeatures, void* stream);

/* ------------------------------------------------------------------------------------------
 * Texture-set level: the same path as the reference's host objects drive it.
 * ------------------------------------------------------------------------------------------ */

typedef struct NtcbContext NtcbContext;       /* stands in for ntc::IContext  (include/libntc/ntc.h:1123-1276) */
typedef struct NtcbTextureSet NtcbTextureSet; /* stands in for ntc::ITextureSet (include/libntc/ntc.h:855-945) */

/* ntc::TextureSetDesc + ntc::LatentShape (include/libntc/ntc.h:131-177) and the derived counts. */
typedef struct NtcbTextureSetDesc
{
    int32_t width, height, channels, mips;
    int32_t gridSizeScale, numFeatures;
    int32_t numNeuralMips, numLayers;
    uint64_t totalTexels;
} NtcbTextureSetDesc;

/* One texture of a set: a named range of channels and the formats its author intended for it.
   ITextureMetadata::GetName / GetChannels / GetChannelFormat / GetBlockCompressedFormat /
   GetRgbColorSpace / GetAlphaColorSpace (include/libntc/ntc.h:390-436). */
typedef struct NtcbTextureDesc
{
    char name[128];                /* truncated if longer */
    int32_t firstChannel, numChannels;
    int32_t channelFormat;         /* NTCB_CHANNEL_FORMAT_*; UNORM8 when the file says nothing */
    int32_t blockCompressedFormat; /* 0 = None, else NTCB_BLOCK_FORMAT_* (6 = BC6, 7 = BC7) */
    int32_t rgbColorSpace, alphaColorSpace; /* NTCB_COLOR_SPACE_* */
} NtcbTextureDesc;

/* Creation options; the reference's TextureSetFeatures (include/libntc/ntc.h:179-199) sizes staging
   and training buffers that this decoder does not have. */
typedef struct NtcbTextureSetFeatures
{
    int32_t outputLayout; /* NtcbOutputLayout of the internal decoded-texel buffer (default interleaved) */
    int32_t numerics;     /* NtcbNumerics used by Decompress (default: the reference's) */
} NtcbTextureSetFeatures;

/* ntc::DecompressionStats (include/libntc/ntc.h:810-816); the loss fields need a resident
   reference image, which a decoder-only texture set never has, so only the timing is kept. */
typedef struct NtcbDecompressionStats
{
    float gpuTimeMilliseconds; /* device time of the decode launch, as the reference times its mip loop */
} NtcbDecompressionStats;

#define NTCB_ADDRESS_SPACE_HOST 0   /* ntc::AddressSpace::Host */
#define NTCB_ADDRESS_SPACE_DEVICE 1 /* ntc::AddressSpace::Device */

/* ntc::ReadChannelsParameters (include/libntc/ntc.h:689-730).  The source page is always the
   decoded output. */
typedef struct NtcbReadChannelsParams
{
    int32_t mipLevel, firstChannel, numChannels;
    int32_t addressSpace;  /* NTCB_ADDRESS_SPACE_* */
    void* pOutData;
    int32_t width, height; /* the mip's size; any other positive size resizes bilinearly, as the reference does
                              (SetupBilinearFilter, src/ImageProcessing.cu:24-71) */
    int32_t channelFormat; /* NTCB_CHANNEL_FORMAT_* */
    int32_t useDithering;  /* nonzero: hash-based dither before rounding to UNORM8 / UNORM16 */
    size_t pixelStride, rowPitch; /* bytes; pixelStride / bytes-per-component components are written per
                                     pixel, those past numChannels as 0 (component 3: 1) */
    const int32_t* dstColorSpaces; /* numChannels NTCB_COLOR_SPACE_* values, or NULL for all Linear */
} NtcbReadChannelsParams;

/* Host only, no GPU needed.  Parses and validates an NTC container and reports what it holds.
   Replaces IContext::CreateTextureSetMetadataFromStream + ITextureSetMetadata::GetDesc /
   GetLatentShape (include/libntc/ntc.h:1161, 546-552; src/Context.cpp:236-283). */
int ntcb_probe_container(const void* data, size_t size, NtcbTextureSetDesc* outDesc);

/* Host only, no GPU needed.  Texture `index` of a container; *outCount (optional) receives the
   number of textures.  An index outside [0, count) returns NTCB_ERR_OUT_OF_RANGE after *outCount is
   written, so index -1 asks for the count alone.  Replaces ITextureSetMetadata::GetTextureCount /
   GetTexture (include/libntc/ntc.h:500-520) on a set opened with CreateTextureSetMetadataFromStream. */
int ntcb_probe_container_texture(const void* data, size_t size, int index, NtcbTextureDesc* outTexture, int* outCount);

/* Host only, no GPU needed.  Where the container keeps the BC7 mode bitmap of a texture's mip level:
   offset from the start of the container and stored size, both 0 when it keeps none; *outCompressed
   (optional) is 1 when the view is GDeflate-compressed.  Replaces ITextureMetadata::GetBC7ModeBufferFootprint
   (include/libntc/ntc.h:451-453, src/TextureMetadata.cpp:154-165). */
int ntcb_probe_container_bc7_mode_buffer(const void* data, size_t size, int textureIndex, int mipLevel, uint64_t* outOffset,
                                         uint64_t* outStoredSize, int* outCompressed);

/* Creates a decoder context on a CUDA device.  Replaces ntc::CreateContext
   (include/libntc/ntc.h:1330, src/PublicFunctions.cpp:62-162).  Fails with NTCB_ERR_CUDA when the
   device is not usable or is not compute capability 10.x. */
int ntcb_context_create(int cudaDevice, NtcbContext** outContext);

/* Replaces ntc::DestroyContext (include/libntc/ntc.h:1333).  Texture sets must be destroyed first. */
void ntcb_context_destroy(NtcbContext* context);

/* Loads a compressed texture set from an NTC container in host memory and allocates its device
   buffers.  Replaces IContext::CreateCompressedTextureSetFromMemory (include/libntc/ntc.h:1171,
   src/Context.cpp:295-366, src/TextureSet.cpp:154-294).  `features` may be NULL. */
int ntcb_texture_set_create_from_memory(NtcbContext* context, const void* data, size_t size,
    const NtcbTextureSetFeatures* features, NtcbTextureSet** outTextureSet);

/* Same from a file.  Replaces IContext::CreateCompressedTextureSetFromFile (include/libntc/ntc.h:1176). */
int ntcb_texture_set_create_from_file(NtcbContext* context, const char* fileName,
    const NtcbTextureSetFeatures* features, NtcbTextureSet** outTextureSet);

/* Replaces IContext::DestroyTextureSet (include/libntc/ntc.h:1153). */
void ntcb_texture_set_destroy(NtcbTextureSet* textureSet);

/* Replaces ITextureSetMetadata::GetDesc / GetLatentShape (include/libntc/ntc.h:546-552). */
int ntcb_texture_set_get_desc(const NtcbTextureSet* textureSet, NtcbTextureSetDesc* outDesc);

/* Uploads the compressed data (as the reference does on every call for a set loaded from a file,
   src/TextureSet.cpp:1691-1757) and decodes every mip into the internal texel buffer: one kernel
   launch, or - when mip 0 has 512 rows or more - four launches for row bands of mip 0 and one for
   the other mips, so that a host read can copy a band while the next is decoded.  With `stats` the call waits for the GPU and reports the device time; without it
   the work is only queued.  Replaces ITextureSet::Decompress (include/libntc/ntc.h:933,
   src/TextureSet.cpp:1664-1897). */
int ntcb_texture_set_decompress(NtcbTextureSet* textureSet, NtcbDecompressionStats* stats, int useInt8Weights);

/* Same, restricted to rows [rowRanges[2*m], rowRanges[2*m+1]) of each mip m: the unit of
   tile-row sharding across GPUs.  No counterpart in the reference, which always decodes whole mips
   on the CUDA path (its graphics path takes a rectangle, include/libntc/ntc.h:1029-1034). */
int ntcb_texture_set_decompress_rows(NtcbTextureSet* textureSet, const int32_t* rowRanges, NtcbDecompressionStats* stats,
    int useInt8Weights);

/* Decompress followed by ReadChannels of every mip, fused: one kernel launch decodes the texels and
   writes them in the client's format (no reference counterpart as one call; it stands in for
   ITextureSet::Decompress, include/libntc/ntc.h:933, plus one ITextureSet::ReadChannels per mip,
   :902, and gives the same bytes).  `destination` (NTCB_ADDRESS_SPACE_*) receives the mips one after
   the other - mip m starts at byte (texels of the mips before it) x components x bytes-per-component -
   each as rows of pixels without padding.  conversion->srcColorSpaces is ignored: the colour space
   each channel is stored in comes from the container.  The set's fp16 texels are not produced, so
   this call does not make ntcb_texture_set_read_channels usable.  Returns when the data is there. */
int ntcb_texture_set_decompress_converted(NtcbTextureSet* textureSet, NtcbDecompressionStats* stats, int useInt8Weights,
    const NtcbOutputConversion* conversion, int addressSpace, void* destination, size_t destinationBytes);

/* Converts decoded channels of one mip to the requested channel format and colour spaces, writes
   them pixel-interleaved with the given strides to host or device memory, and returns when the data
   is there.  Replaces ITextureSet::ReadChannels (include/libntc/ntc.h:902, src/TextureSet.cpp:915-985)
   and the CopyImageKernel behind it (src/ImageProcessing.cu:220-277).  Each channel is first taken
   out of the colour space the container stores it in (channels[].colorSpace), then encoded to its
   destination colour space. */
int ntcb_texture_set_read_channels(NtcbTextureSet* textureSet, const NtcbReadChannelsParams* params);

/* Device address and size in bytes of one decoded mip in the internal layout: the counterpart of
   TextureSet::GetTextureDataSlice (src/TextureSet.cpp:1958-1983) for callers that consume the
   texels on the GPU. */
int ntcb_texture_set_device_mip(NtcbTextureSet* textureSet, int mipLevel, void** outPointer, size_t* outBytes);

/* Loads another compressed texture set of the same dimensions, channel count, mip count and latent shape into
   an existing one, re-using every buffer it holds: ITextureSet::LoadFromMemory (include/libntc/ntc.h:869-881).
   NTCB_ERR_FILE_INCOMPATIBLE when the shapes differ (nothing changes then).  Waits for the set's stream; the
   decoded texels of the previous set stay in place until the next decompress, but calls that need decoded
   texels return NTCB_ERR_INVALID_STATE until then. */
int ntcb_texture_set_load_from_memory(NtcbTextureSet* textureSet, const void* data, size_t size);

/* The textures of a loaded set: see ntcb_probe_container_texture. */
int ntcb_texture_set_get_texture(NtcbTextureSet* textureSet, int index, NtcbTextureDesc* outTexture, int* outCount);

/* Inference on sample at the texture-set level: `deviceQueries` (numQueries x 3 floats: u, v, lod) and `deviceOut`
   (numQueries x channels binary16 values) lie in the memory of the set's device; query q selects a texel as
   ntcb_sample describes and receives the bits ntcb_texture_set_decompress would write there.  The compressed
   data is uploaded when the device copy is not current (first use, after ntcb_texture_set_load_from_memory), and
   its pixel-major copy (ntcb_interleave_latents) is made then too, so a set that is sampled again and again pays
   for neither; the call runs on the set's stream and waits for the answers (NTCB_ERR_DEVICE_TIMEOUT if a bounded
   wait inside the kernel expired).  The reference offers sampling to shaders only (NtcSampleTextureSet,
   include/libntc/shaders/Inference.hlsli:282-357, with the data of IContext::MakeInferenceData,
   src/Context.cpp:864-922). */
int ntcb_texture_set_sample(NtcbTextureSet* textureSet, const float* deviceQueries, uint64_t numQueries, void* deviceOut,
    int useInt8Weights);

/* Waits for everything queued on the texture set's stream. */
int ntcb_texture_set_synchronize(NtcbTextureSet* textureSet);

/* One decoded mip (fp16, device memory, `layout`, `channels` channels per texel) converted into
   pixel-interleaved client data in device memory with the given strides: the kernel behind
   ntcb_texture_set_read_channels, for callers that hold the decoded texels themselves.  Replaces
   cuda::CopyImage (src/ImageProcessing.cu:268-277) for the 1:1, texture-set-to-client direction.
   Queued on `stream`; returns without waiting. */
typedef struct NtcbConvertParams
{
    const void* deviceMip;   /* 4-byte aligned (channel pairs are read as 32-bit words) */
    int32_t layout;          /* NtcbOutputLayout of deviceMip */
    int32_t width, height, channels;
    int32_t reserved;
    void* deviceDestination;
    size_t pixelStride, rowPitch; /* bytes */
    NtcbOutputConversion conversion; /* components * bytes-per-component must not exceed pixelStride */
    int32_t dstWidth, dstHeight; /* size of the destination; 0, 0 = the mip's own size.  Another size resizes
                                    bilinearly as the reference's ReadChannels does; rowPitch then counts dstWidth pixels */
} NtcbConvertParams;
int ntcb_convert_channels(const NtcbConvertParams* params, void* stream);

/* ---- Encoder-side producers of what the decoder consumes -------------------------------------- */

/* Packs quantised fp16 latents into the 16-bit words the decode kernels read (four 4-bit codes per
   word, the first feature in the low bits; one width x height plane of words per layer, the layers
   one after another).  Replaces cuda::PackLatents (src/Quantizer.cu:497-541; called from
   TextureSet::FinalizeCompression, src/TextureSet.cpp:1589-1602) with the same input layout:
   `latents` holds, for layer z and texel t = y * width + x, features 0 and 1 at element
   z * latentStride * 2 + t * 2 and features 2 and 3 `latentStride` elements further on.  Each code
   is round(15 * clamp(value, 0, 1)).  Both pointers are device memory; queued on `stream`. */
int ntcb_pack_latents(const void* latents, int width, int height, int numLayers, size_t latentStride,
    void* packed, void* stream);

/* Quantises the decoder network from fp16 to a GenericInt8 or GenericFP8 blob, the form containers
   store and ntcb_stage_network* read.  Replaces cuda::QuantizeNetwork (src/Quantizer.cu:90-325;
   called from src/TextureSet.cpp:1610-1633).  Int8: per output column, codes round(w * 127.5 /
   max|w|), a float scale that folds the input or activation step (and, for the output layer, the
   channel's optimal-to-linear scale), and the bias as an integer multiple of that scale.  FP8:
   layers 0-2 rounded to e4m3 with their fp16 biases kept; the output layer as in Int8.
   All pointers but outputScale / outputBias are device memory. */
typedef struct NtcbQuantizeNetworkParams
{
    const void* weights;     /* fp16; per layer outputs x inputs values, the inputs of one output together
                                (the order of the blob's weight section): 3072 + 3072 + 1536 + 512 values */
    const void* biases;      /* fp16; 64 + 48 + 32 + 16 values */
    const float* outputScale; /* host, 16 values: optimal-to-linear scale per output channel; NULL = 1 */
    const float* outputBias;  /* host, 16 values: optimal-to-linear bias per output channel; NULL = 0 */
    int32_t weightMode;      /* NTCB_WEIGHTS_INT8 or NTCB_WEIGHTS_FP8 */
    int32_t reserved;
    void* blob;              /* NTCB_INT8_BLOB_BYTES or NTCB_FP8_BLOB_BYTES */
    void* roundedWeights;    /* optional, fp16, same order as `weights`: the weights as the decoder will apply
                                them (the reference overwrites its fp16 copy with these) */
} NtcbQuantizeNetworkParams;
int ntcb_quantize_network(const NtcbQuantizeNetworkParams* params, void* stream);

/* ---- Block compression of decoded texels ------------------------------------------------------ */

/* ntc::BlockCompressedFormat (include/libntc/ntc.h:238-249) */
#define NTCB_BLOCK_FORMAT_BC1 1
#define NTCB_BLOCK_FORMAT_BC2 2
#define NTCB_BLOCK_FORMAT_BC3 3
#define NTCB_BLOCK_FORMAT_BC4 4
#define NTCB_BLOCK_FORMAT_BC5 5
#define NTCB_BLOCK_FORMAT_BC7 7

/* Encodes channels of a decoded mip (fp16, device memory) as BC1 - BC5 or BC7 blocks in device memory.
   The CUDA counterpart of the compute pass that IContext::MakeBlockCompressionComputePass describes
   (include/libntc/ntc.h:1050-1100, src/Context.cpp:630-779) and that the reference runs as
   src/shaders/CompressBC1-5.hlsl, CompressBC7.hlsl through a graphics API; the encoders follow
   src/shaders/BlockCompressCommon.hlsli (BC1_EncodeSingleColor, BC1_CompressFast, BC1a_CompressFast,
   BC2_EncodeAlpha, BC4_CompressFast) and CompressBC7.hlsl.  srcLeft / srcTop and widthInBlocks /
   heightInBlocks mean what srcRect means there (texels outside the mip read as 0 in every
   component); the destination offset is folded into `deviceBlocks`.  BC6: NTCB_ERR_UNSUPPORTED.

   BC7 without a mode buffer searches every mode and partition (the reference's slow path, meant for
   offline use); with `deviceModeBuffer` it encodes each block in the mode and partition the buffer
   names (the reference's BlockCompressionModeBufferSource::Custom / TextureSet; 9 bits per block as
   ntcb_make_bc7_mode_buffer lays them out), and writes a block of four coloured squares where the
   buffer has no entry.  modeMapOffsetX / Y are added to a block's position before the look-up;
   modeBufferByteOffset must be a multiple of 4.

   The first call of a colour format (BC1 - BC3) on a device uploads two 512-byte tables (make it
   before any stream capture).  Queued on `stream`; returns without waiting. */
typedef struct NtcbBlockCompressParams
{
    const void* deviceMip;   /* decoded texels of one mip */
    int32_t layout;          /* NtcbOutputLayout of deviceMip */
    int32_t width, height, channels; /* of deviceMip */
    int32_t firstChannel;    /* BC4: the channel; BC5: it and the next; BC1-3, BC7: red, then green, blue, alpha */
    int32_t format;          /* NTCB_BLOCK_FORMAT_* */
    int32_t srcLeft, srcTop; /* texel position of the first block */
    int32_t widthInBlocks, heightInBlocks;
    int32_t numChannels;     /* BC1-3, BC7: channels that feed the block, 1..4 (green and blue then read 0, alpha 1);
                                0 = 3 for BC1, 4 for BC2 / BC3 / BC7.  BC4 / BC5: 0 */
    void* deviceBlocks;      /* 8 (BC1, BC4) or 16 (BC2, BC3, BC5, BC7) bytes per block */
    size_t rowPitch;         /* bytes between rows of blocks */
    float alphaThreshold;    /* BC1: texels with alpha <= this are transparent (the reference's default: 1/255) */
    int32_t reserved;
    /* BC7 only; all zero = full search */
    const void* deviceModeBuffer;   /* device memory, 4-byte aligned */
    uint32_t modeBufferByteOffset;
    uint32_t modeMapWidthInBlocks, modeMapHeightInBlocks; /* size of the block grid the buffer describes */
    int32_t modeMapOffsetX, modeMapOffsetY;
    int32_t reserved2;
} NtcbBlockCompressParams;
int ntcb_block_compress(const NtcbBlockCompressParams* params, void* stream);

/* Host side of the BC7 mode buffer: ntc::GetBC7ModeBufferSize and ntc::MakeBC7ModeBuffer
   (include/libntc/ntc.h:1381-1387, src/PublicFunctions.cpp:470-556).  From BC7 blocks (host memory, rows
   `rowPitch` bytes apart) to the 9-bit-per-block bitmap of their modes and partitions (3 bits mode, 6 bits
   partition; for modes 4 and 5 the rotation and index selector); the size is rounded up to 4 bytes.  The
   mode buffer is cleared before it is filled. */
size_t ntcb_bc7_mode_buffer_size(int widthInBlocks, int heightInBlocks);
int ntcb_make_bc7_mode_buffer(int widthInBlocks, int heightInBlocks, const void* blockData, size_t blockDataSize,
                              size_t rowPitch, void* modeBuffer, size_t modeBufferSize);

/* The same for one whole mip of a decompressed texture set (NTCB_ERR_INVALID_STATE before
   ntcb_texture_set_decompress): (width + 3) / 4 by (height + 3) / 4 blocks into device memory,
   `rowPitch` bytes between rows of blocks, queued on the texture set's stream
   (ntcb_texture_set_synchronize waits for it). */
int ntcb_texture_set_block_compress(NtcbTextureSet* textureSet, int mipLevel, int firstChannel, int numChannels, int format,
    float alphaThreshold, void* deviceBlocks, size_t rowPitch);

/* BC7 mode bitmaps of a texture of the set: ITextureMetadata::GetBC7ModeBuffer and
   ITextureMetadata::MakeAndStoreBC7ModeBuffer (include/libntc/ntc.h:436-449, src/TextureMetadata.cpp:96-152).
   The first returns the bitmap the file stores for that texture and mip level ("bcModeBuffers" of the
   texture's header) or one stored by the second call: a pointer into host memory owned by the texture set,
   NULL and 0 when there is none (NTCB_ERR_UNSUPPORTED when the file stores it GDeflate-compressed).  The
   second makes the bitmap from BC7 blocks whose size in blocks is exactly that of the mip level. */
int ntcb_texture_set_get_bc7_mode_buffer(NtcbTextureSet* textureSet, int textureIndex, int mipLevel, const void** outData,
                                         size_t* outSize);
int ntcb_texture_set_make_and_store_bc7_mode_buffer(NtcbTextureSet* textureSet, int textureIndex, int mipLevel, int widthInBlocks,
                                                    int heightInBlocks, const void* blockData, size_t blockDataSize,
                                                    size_t rowPitch);

/* One whole mip of one texture of a decompressed set to the block format the texture's header names
   (bcFormat: BC1 - BC5, BC7; NTCB_ERR_INVALID_ARGUMENT for None, NTCB_ERR_UNSUPPORTED for BC6), from the
   texture's channel range.  BC7 uses the texture's mode bitmap of that mip when it has one - the reference's
   BlockCompressionModeBufferSource::TextureSet (include/libntc/ntc.h:1042-1091, src/Context.cpp:675-706): the
   bitmap is uploaded on first use and kept - and searches every mode otherwise.  Queued on the set's stream. */
int ntcb_texture_set_block_compress_texture(NtcbTextureSet* textureSet, int textureIndex, int mipLevel, float alphaThreshold,
                                            void* deviceBlocks, size_t rowPitch);

/* ---- Several GPUs of one machine ------------------------------------------------------------ */

/* One texture set of a batch: its container, and the host image that receives the decoded chain. */
typedef struct NtcbBatchItem
{
    const void* container;   /* NTC container in host memory */
    size_t containerBytes;
    void* hostTexels;        /* host memory (pinned memory copies fastest): every mip one after the other as
                                fp16 [y][x][c] - what ReadChannels(FLOAT16) of each mip hands back; the devices
                                write disjoint rows of it: the final host gather */
    size_t hostTexelsBytes;  /* at least totalTexels x channels x 2 */
    int32_t useInt8Weights;
    int32_t status;          /* out: NTCB_OK, or the error that kept one of this item's units from being decoded */
} NtcbBatchItem;

/* One unit of work: rows [rowBegin[m], rowEnd[m]) of each mip m of one item. */
typedef struct NtcbBatchUnit
{
    int32_t item;
    int32_t device;          /* out: the device of the last attempt (-1: never tried) */
    int32_t attempts;        /* out */
    int32_t status;          /* out: result of the last attempt */
    int32_t rowBegin[NTCB_MAX_MIPS], rowEnd[NTCB_MAX_MIPS];
    uint64_t texels;
} NtcbBatchUnit;

typedef struct NtcbBatchOptions
{
    int32_t numerics;         /* NtcbNumerics */
    int32_t maxAttempts;      /* tries per unit, each on another device; 0 = 3 */
    int32_t unitsPerDevice;   /* the job is cut into about devices x this many units; 0 = 4 */
    int32_t workersPerDevice; /* host threads (each with its own context) per device, so that one's copy to the
                                 host overlaps the other's decode; 0 = 2 */
    /* Test hook: when set, it is called in place of the GPU work of a unit (no CUDA call is made at
       all) and its return value is the unit's result - a stand-in for a device that fails, or is slow. */
    int (*worker)(void* user, int device, const NtcbBatchUnit* unit);
    void* workerUser;
} NtcbBatchOptions;

/* Cuts a job into work units, largest first (host only).  With the target size = all texels /
   (numDevices x unitsPerDevice): an item of at most three quarters of it stays whole (there are enough
   items to balance the devices); one of at most ~1.5 times the target becomes two units - mip 0, and the
   other mips;
   a larger one becomes bands of tile rows (multiples of 8 rows, at least 64) of its tall mips, the
   short mips going whole to the lightest band.  `units` may be NULL to ask for the count. */
int ntcb_plan_batch(const NtcbTextureSetDesc* descs, int numItems, int numDevices, int unitsPerDevice, NtcbBatchUnit* units,
    int maxUnits, int* outNumUnits);

/* Decodes a batch of texture sets (or one large set) on several devices and gathers the texels in
   host memory.  No counterpart in the reference, which drives one device per context
   (include/libntc/ntc.h:1289-1290) and leaves this layer to the client: the units of ntcb_plan_batch
   are handed out, largest first, to one or more host threads per listed device, each with its own
   context; a thread decodes a unit's rows (ntcb_texture_set_decompress_rows on its copy of the set)
   and copies them to their place in the item's host image.  The devices share nothing: no peer
   access, no collective.  A device may be listed more than once.
   A unit that fails on a device (context creation, a CUDA error, NTCB_ERR_DEVICE_TIMEOUT) is tried
   again on another one, up to maxAttempts; a device that fails two units in a row takes no more
   work.  Returns NTCB_OK when every unit was decoded; otherwise an error, with the items' `status`
   and - when `outUnits` is given - the per-unit record telling what failed where.  Blocks until
   all work is done. */
int ntcb_decode_batch(NtcbBatchItem* items, int numItems, const int* devices, int numDevices, const NtcbBatchOptions* options,
    NtcbBatchUnit* outUnits, int maxUnits, int* outNumUnits);

/* The same with the worker threads, their contexts and the texture sets they have allocated kept between
   calls: for a client that decodes batch after batch.  Workers open their device when the first run
   reaches them; a device that cannot be opened takes no work in that run and is tried again in the next.
   One run at a time per decoder (a second caller waits).  ntcb_decode_batch is create + run + destroy. */
typedef struct NtcbBatchDecoder NtcbBatchDecoder;
int ntcb_batch_decoder_create(const int* devices, int numDevices, const NtcbBatchOptions* options, NtcbBatchDecoder** outDecoder);
int ntcb_batch_decoder_run(NtcbBatchDecoder* decoder, NtcbBatchItem* items, int numItems, NtcbBatchUnit* outUnits, int maxUnits,
    int* outNumUnits);
void ntcb_batch_decoder_destroy(NtcbBatchDecoder* decoder);

/* Size of the staging area built into the library for ntcb_read_channels_to_host_noalloc. */
#define NTCB_NOALLOC_STAGING_BYTES (4u << 20)

/* Reads decoded channels of one mip into HOST memory without allocating anything.
   (No counterpart in the reference: its ReadChannels stages through a buffer that the texture set
   allocates at creation, src/TextureSet.cpp:123-131.)

   Who this is for: ntcb_texture_set_read_channels grows a device staging buffer with cudaMalloc the
   first time a host read needs a layout conversion (a channel subset, padded strides, or the
   planar-pair internal layout).  Some callers must not reach cudaMalloc: code on a frame or
   streaming thread where an allocation's implicit device synchronisation is a stall, code that
   runs under a fixed memory budget handed out up front, or code inside a region where allocation
   is simply forbidden by the host application.  This variant runs the same gather kernel into a
   4 MiB array that is part of the library image (each GPU that loads the library carries it until
   the process exits), then copies to `hostDestination` and waits for `stream`.

   `deviceMip` is the device address of one decoded mip (ntcb_texture_set_device_mip, or the `out`
   buffer given to ntcb_decode plus the mip's offset) in `layout` with `channels` channels;
   firstChannel / numChannels / pixelStride / rowPitch mean what they mean in NtcbReadChannelsParams.
   height * rowPitch must not exceed NTCB_NOALLOC_STAGING_BYTES, otherwise NTCB_ERR_OUT_OF_RANGE is
   returned and nothing is done: read a large mip in row bands (offset `deviceMip` by whole rows;
   a row of either layout is width x channels values, so with an even channel count the address
   stays 4-byte aligned, which the gather kernel needs and the call checks) or channel groups.

   The first call on a device looks up the array's device address: make that call before any
   stream capture begins.  Every call waits for `stream` before it returns, so it must never be
   made on a stream that is being captured.  Every call uses the same array, which keeps the previous call's
   contents (gaps are cleared when a request has gaps): two calls whose GPU work overlaps - on
   different streams or from different threads - race on it, so serialise them. */
int ntcb_read_channels_to_host_noalloc(const void* deviceMip, int layout, int width, int height, int channels,
    int firstChannel, int numChannels, void* hostDestination, size_t pixelStride, size_t rowPitch, void* stream);

/* Number of CTAs the decode kernel keeps resident on the current device for a weight mode (the
   grid size of large launches): SM count x resident CTAs per SM, the latter bounded by registers,
   shared memory and tensor-memory columns.  For benchmarks and tests. */
int ntcb_decode_resident_ctas(int weightMode, int* outCtas);

/* Test hook for the kernels' timeout path (no counterpart in the reference).  Every wait inside the
   kernels is bounded; a CTA whose wait runs out records it in the status words (word 0 =
   1, word 1 = tile, word 2 = layer; 0xFFFFFFFF in both for the wait described here), lets the work it has in
   flight finish, releases its tensor memory and exits, and the host reports NTCB_ERR_DEVICE_TIMEOUT.
   This call sets, for every later launch of the process, how many polls a CTA spends on its FIRST
   wait - for the network image its bulk copy brings into shared memory, before any tile is touched
   and with no tensor-core work in flight - and returns the previous value.  0 makes that wait run
   out at once, which lets a test walk the whole error path without hanging or faulting anything;
   NTCB_DEFAULT_WAIT_POLLS restores normal operation.  No other wait is affected. */
#define NTCB_DEFAULT_WAIT_POLLS (1u << 20)
uint32_t ntcb_debug_set_network_wait_polls(uint32_t polls);

/* Number of kernel launches this library has issued from the calling process so far
   (bookkeeping for benchmarks). */
uint64_t ntcb_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
