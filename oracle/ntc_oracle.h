/* TEST INFRASTRUCTURE ONLY: nothing in the product library includes, links or calls this.
 *
 * CPU restatement of LibNTC's CUDA decompression (inference) path, used as the parity checker for
 * the sm_100a kernels and as the timed scalar CPU baseline.  LibNTC itself has no CPU decoder;
 * every function here restates reference CUDA/host code and cites the lines it follows
 * (paths are relative to the reference project root).
 *
 * Two numerics are implemented:
 *
 *  NTCO_NUMERICS_SPEC  The arithmetic contract of the sm_100a kernels.  Everything outside the
 *      matrix products follows the reference's CUDA kernel operation by operation in IEEE
 *      binary16 / binary32 (src/Inference.cu:46-136, src/FeatureGridDevice.h:33-98,
 *      src/RegressionKernels.h:59-85, src/tin/tin_mlp.h:22-37, src/tin/tin_activation.h:88-104).
 *      The matrix products accumulate exactly: int8 x int8 -> int32 plus the file's int32 bias and
 *      fp32 scale, as the reference's integer inference path does
 *      (include/libntc/shaders/Inference.hlsli:133-182), and e4m3 x e4m3 -> fp32 for the FP8 layers.
 *
 *  NTCO_NUMERICS_REF   An emulation of the reference CUDA kernel's own arithmetic: weights
 *      converted back to binary16 (src/Quantizer.cu:325-408), binary16 activations, binary16
 *      accumulators updated once per 16-wide k chunk (src/tin/tin_mma.h:126-163).  The chunk sum's
 *      internal precision is hardware defined, so this mode carries option switches and is pinned
 *      against outputs of the reference itself (tests/golden).
 */
#ifndef NTC_ORACLE_H
#define NTC_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NTCO_MAX_MIPS 16        /* include/libntc/shaders/InferenceConstants.h:22 */
#define NTCO_MAX_NEURAL_MIPS 8  /* include/libntc/shaders/InferenceConstants.h:24 */
#define NTCO_INT8_BLOB_BYTES 9472 /* src/WeightLayout.cpp:142-268: 8192 weights + 160 fp32 + 160 int32 */
#define NTCO_FP8_BLOB_BYTES 8608  /* 8192 weights + 144 fp16 bias + 16 fp32 scale + 16 int32 bias */

enum { NTCO_WEIGHTS_INT8 = 0, NTCO_WEIGHTS_FP8 = 1 };
enum { NTCO_NUMERICS_SPEC = 0, NTCO_NUMERICS_REF = 1 };

typedef struct NtcoTextureSet
{
    int width, height;   /* colour mip 0 */
    int channels;        /* output channels, rounded up to even (src/TextureSet.cpp:85-86) */
    int numMips;         /* colour mips */
    int gridSizeScale;   /* 1..6 */
    int numFeatures;     /* 4, 8, 12 or 16 */
    /* Encoded latent pixels (BGRA4, one uint16 per pixel per layer) in the reference's device
       order: for each neural mip, for each layer, rows of pixels (src/FeatureGridHost.cpp:140-155). */
    const uint16_t* latents;
    const uint8_t* int8Blob; /* GenericInt8 weight blob */
    const uint8_t* fp8Blob;  /* GenericFP8 weight blob */
} NtcoTextureSet;

typedef struct NtcoGeometry
{
    int numNeuralMips;
    int numLayers;
    int latentWidth[NTCO_MAX_NEURAL_MIPS];
    int latentHeight[NTCO_MAX_NEURAL_MIPS];
    uint64_t latentPixelOffset[NTCO_MAX_NEURAL_MIPS + 1]; /* in pixels of one layer, cumulative */
    int mipWidth[NTCO_MAX_MIPS];
    int mipHeight[NTCO_MAX_MIPS];
    int neuralLod[NTCO_MAX_MIPS];
    float positionScale[NTCO_MAX_MIPS];
    float positionLod[NTCO_MAX_MIPS];
    uint64_t mipTexelOffset[NTCO_MAX_MIPS + 1]; /* cumulative texel counts */
} NtcoGeometry;

typedef struct NtcoOptions
{
    int weights;   /* NTCO_WEIGHTS_* : Decompress(useInt8Weights) selects INT8, else FP8 */
    int numerics;  /* NTCO_NUMERICS_* */
    int threads;   /* host threads over rows; <= 0 means all */
    /* Switches of NTCO_NUMERICS_REF (ignored by SPEC).  The values that reproduce the reference's
       kernel on a B200 are refBlendFma = 2, refAccChunk = 16, refAccMode = 25 (see tests/golden). */
    int refBlendFma;   /* bilinear blend l00*w0 + l01*w1 + l10*w2 + l11*w3:
                          0: separate multiplies and adds;
                          1: fma chain seeded with round(l00*w0);
                          2: fma chain seeded with round(l01*w1), i.e. fma(l00, w0, round(l01*w1)), ... */
    int refQuantFma;   /* 1: input quantisation x*127.5-0.5 contracted into one fma */
    int refAccChunk;   /* products summed per rounding to binary16: 4, 8 or 16 */
    int refAccMode;    /* 0: exact chunk sum then one rounding; 1: fp32 sequential sum then rounding;
                          2: exact sum truncated to fp32 toward zero then rounding;
                          >= 16: addends aligned to the largest exponent and truncated below
                          2^(emax - refAccMode), summed exactly, then one rounding */
    int refActFma;     /* reserved */
} NtcoOptions;

/* Geometry of a texture set: neural mip sizes, colour-mip -> neural-LOD map, positional encoding
   constants, buffer offsets.  Returns 0, or -1 on invalid arguments. */
int ntco_geometry(const NtcoTextureSet* set, NtcoGeometry* out);

/* Decodes rows [y0, y1) of one colour mip into `out`, fp16 bit patterns interleaved per texel:
   out[((y - y0) * mipWidth + x) * channels + c].  Returns 0, or -1 on invalid arguments. */
int ntco_decode_mip(const NtcoTextureSet* set, const NtcoOptions* opt, int mip, int y0, int y1, uint16_t* out);

/* Inference-on-sample: for each query (u, v, lod) picks mip = clamp(floor(lod)), texel =
   min(floor(u * W_mip), W_mip - 1) (same for v) and evaluates that texel exactly as ntco_decode_mip
   does (the reference's NtcSampleTextureSet takes an integer texel and mip,
   include/libntc/shaders/Inference.hlsli:282-357).  out[q * channels + c]. */
int ntco_sample(const NtcoTextureSet* set, const NtcoOptions* opt, const float* queries /* [n][3] */,
    size_t numQueries, uint16_t* out);

/* ITextureSet::ReadChannels on a decoded mip without resizing (src/TextureSet.cpp:915-985 calling
   CopyImageKernel, src/ImageProcessing.cu:220-266): converts channels [firstChannel, firstChannel +
   numChannels) of `texels` (fp16 bit patterns, interleaved [y][x][channels]) to `channelFormat`
   (ntc::ChannelFormat values: 1 UNORM8, 2 UNORM16, 3 FLOAT16, 4 FLOAT32, 5 UINT32) and writes
   pixelStride / bytesPerComponent components per pixel; components beyond numChannels get 0, or 1
   for component 3.  Colour spaces are ntc::ColorSpace values (0 Linear, 1 sRGB, 2 HLG):
   srcColorSpaces per channel of the set, dstColorSpaces per requested channel, NULL = all Linear.
   The transfer functions are evaluated with the C library in binary32; the reference's kernel is
   built with --use_fast_math (src/CMakeLists.txt:33), so its sRGB / HLG results and its dither
   offsets can differ from these in the last bits.  Bytes of `out` outside the written components
   are left alone.  Returns 0, or -1 on invalid arguments. */
typedef struct NtcoReadChannels
{
    int width, height, channels;
    int firstChannel, numChannels;
    int channelFormat;
    size_t pixelStride, rowPitch;
    const int* srcColorSpaces;
    const int* dstColorSpaces;
    int useDithering;
} NtcoReadChannels;
int ntco_read_channels(const uint16_t* texels, const NtcoReadChannels* params, uint8_t* out);
/* The same with a destination of another size: the reference's bilinear resize (SetupBilinearFilter,
   src/ImageProcessing.cu:24-71); `params` keeps describing the source mip, rowPitch the destination. */
int ntco_read_channels_resized(const uint16_t* texels, const NtcoReadChannels* params, int dstWidth, int dstHeight, uint8_t* out);

/* PackLatentsKernel (src/Quantizer.cu:497-527): quantised fp16 latents (bit patterns) to 4-bit
   words; `packed` receives width * height * numLayers words.  Returns 0, or -1 on invalid arguments. */
int ntco_pack_latents(const uint16_t* latents, int width, int height, int numLayers, size_t latentStride, uint16_t* packed);

/* QuantizeNetwork (src/Quantizer.cu:90-325): fp16 weights (per layer outputs x inputs, the inputs
   of one output together) and 160 fp16 biases to a GenericInt8 (9472 bytes) or GenericFP8 (8608
   bytes) blob; `roundedWeights` (optional) receives the fp16 weights after quantisation.  Exact
   divisions stand in for the GPU's approximate ones: see the note in the source. */
int ntco_quantize_network(const uint16_t* weights, const uint16_t* biases, const float* outputScale, const float* outputBias,
    int useFP8, uint8_t* blob, uint16_t* roundedWeights);

/* BC4 (formatChannels 1) or BC5 (2) encoding of interleaved fp16 texels, following the reference's
   compute shaders (src/shaders/CompressBC4.hlsl, CompressBC5.hlsl, BlockCompressCommon.hlsli:510-796).
   PARITY UNPINNED: those shaders need a graphics API to run, which is unavailable here.  Texels
   outside the image read as 0.  `blocks` receives 8 * formatChannels bytes per block, row-major. */
int ntco_block_compress(const uint16_t* texels, int width, int height, int channels, int firstChannel, int formatChannels,
    int srcLeft, int srcTop, int widthInBlocks, int heightInBlocks, uint8_t* blocks);

/* BC1 (format 1), BC2 (2) or BC3 (3) encoding, following src/shaders/CompressBC1-3.hlsl and
   BlockCompressCommon.hlsli:82-508.  PARITY UNPINNED, as above.  `numChannels` (1..4) channels from
   `firstChannel` are red, green, blue, alpha (missing ones 0, alpha 1); texels outside the image
   read as 0 in all four.  8 (BC1) or 16 bytes per block. */
int ntco_block_compress_color(const uint16_t* texels, int width, int height, int channels, int firstChannel, int numChannels,
    int format, float alphaThreshold, int srcLeft, int srcTop, int widthInBlocks, int heightInBlocks, uint8_t* blocks);

/* The single-colour match table for 5- or 6-bit endpoints (256 entries: mx | mn << 8), generated:
   the pair minimising 1000 * |(2 e(mx) + e(mn)) / 3 - i| + 14 * |e(mx) - e(mn)|, mn in the outer
   loop, first minimum kept.  Reproduces c_ColorMatch5bit / c_ColorMatch6bit of
   BlockCompressCommon.hlsli:40-80 (checked by digest in tests/test_block_compress.py). */
int ntco_color_match_table(int bits, uint16_t* table);

/* Element helpers exposed for unit tests. */
uint16_t ntco_float_to_half(float value);
float ntco_half_to_float(uint16_t bits);
uint8_t ntco_half_to_e4m3(uint16_t bits);
float ntco_e4m3_to_float(uint8_t bits);
uint16_t ntco_hgelu_clamp_half(uint16_t x);

#ifdef __cplusplus
}
#endif
#endif
