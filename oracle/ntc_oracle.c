/* TEST INFRASTRUCTURE ONLY: nothing in the product library includes, links or calls this.
 *
 * CPU restatement of LibNTC's CUDA decompression path; see ntc_oracle.h for the two numerics.
 * Scalar code, one texel at a time, work items spread over host threads (pthreads).
 * Build: see oracle/Makefile (needs -mf16c, -ffp-contract=off).
 */
#include "ntc_oracle.h"

#include <float.h>
#include <immintrin.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <stdatomic.h>
#include <unistd.h>

/* Network geometry: include/libntc/shaders/InferenceConstants.h:26-40, src/MlpDesc.h:25-99. */
#define MLP_LAYERS 4
#define MLP_FEATURES 16
#define MLP_IN 48
static const int kLayerIn[MLP_LAYERS] = {48, 64, 48, 32};
static const int kLayerOut[MLP_LAYERS] = {64, 48, 32, 16};

typedef uint16_t h16;

/* ------------------------------------------------------------------------------------------ */
/* binary16 arithmetic, one IEEE operation per call                                             */
/* ------------------------------------------------------------------------------------------ */

static inline float h2f(h16 h) { return _cvtsh_ss(h); }
static inline h16 f2h(float f) { return _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC); }

static inline uint32_t f_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float f_from_bits(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* double -> binary16, round to nearest even in one step: first to binary32 with round-to-odd
   (24 bits >= 11 + 2 keeps the final rounding correct), then the hardware RNE conversion. */
static inline h16 d2h(double d)
{
    float f = (float)d;
    if (isfinite(f) && (double)f != d)
    {
        uint32_t bits = f_bits(f);
        if (fabs((double)f) > fabs(d))
            bits -= 1; /* step toward zero: now the truncated value */
        bits |= 1;     /* inexact: make it odd */
        f = f_from_bits(bits);
    }
    return f2h(f);
}

/* The product of two binary16 values is exact in binary32; the sum of two is exact or is rounded
   harmlessly (24 >= 2*11 + 2), so one binary32 operation plus one conversion is one binary16 op. */
static inline h16 hmul(h16 a, h16 b) { return f2h(h2f(a) * h2f(b)); }
static inline h16 hadd(h16 a, h16 b) { return f2h(h2f(a) + h2f(b)); }
static inline h16 hsub(h16 a, h16 b) { return f2h(h2f(a) - h2f(b)); }
static inline h16 hfma(h16 a, h16 b, h16 c) { return d2h((double)h2f(a) * (double)h2f(b) + (double)h2f(c)); }
static inline h16 hfma_sat(h16 a, h16 b, h16 c)
{
    double r = (double)h2f(a) * (double)h2f(b) + (double)h2f(c);
    if (!(r > 0.0)) return 0;          /* NaN and negatives -> +0, as fma.rn.sat.f16 */
    if (r > 1.0) return 0x3C00;
    return d2h(r);
}
static inline h16 hmin(h16 a, h16 b)
{
    float fa = h2f(a), fb = h2f(b);
    if (isnan(fa)) return b;
    if (isnan(fb)) return a;
    return fa < fb ? a : b;
}
static inline h16 hmax(h16 a, h16 b)
{
    float fa = h2f(a), fb = h2f(b);
    if (isnan(fa)) return b;
    if (isnan(fb)) return a;
    return fa > fb ? a : b;
}
static inline h16 hfloor(h16 a) { return f2h(floorf(h2f(a))); }
static inline h16 hrint(h16 a) { return f2h(nearbyintf(h2f(a))); } /* default mode: nearest even */
static inline int h_is_special(h16 a) { return (a & 0x7C00) == 0x7C00; } /* src/CudaUtils.h:30-35 */

uint16_t ntco_float_to_half(float value) { return f2h(value); }
float ntco_half_to_float(uint16_t bits) { return h2f(bits); }

/* ------------------------------------------------------------------------------------------ */
/* FP8 e4m3 (finite-only format: max 448, 0x7F/0xFF = NaN)                                      */
/* ------------------------------------------------------------------------------------------ */

float ntco_e4m3_to_float(uint8_t bits)
{
    int sign = bits >> 7, exponent = (bits >> 3) & 15, mantissa = bits & 7;
    float magnitude;
    if (exponent == 15 && mantissa == 7)
        magnitude = NAN;
    else if (exponent == 0)
        magnitude = ldexpf((float)mantissa, -9);
    else
        magnitude = ldexpf(1.0f + (float)mantissa / 8.0f, exponent - 7);
    return sign ? -magnitude : magnitude;
}

/* binary16 -> e4m3, round to nearest even, saturating to +-448; NaN -> 0x7F.
   This is what the reference's RoundHalfToFloatE4M3 does on sm_89 and newer, where it uses the
   hardware conversion (src/tin/tin_activation.h:44-48). */
uint8_t ntco_half_to_e4m3(uint16_t bits)
{
    float x = h2f(bits);
    if (isnan(x))
        return 0x7F;
    uint8_t sign = (bits & 0x8000) ? 0x80 : 0;
    float a = fabsf(x);
    if (a >= 448.0f)   /* includes infinity; values in (448, 464) round to 448 as well */
        return sign | 0x7E;
    if (a < 0x1p-6f)
    {
        /* subnormal range: multiples of 2^-9 */
        int q = (int)nearbyintf(a * 512.0f); /* exact scaling, nearest-even */
        return sign | (uint8_t)q;            /* q == 8 encodes the smallest normal, as it should */
    }
    int e;
    float m = frexpf(a, &e);                 /* a = m * 2^e, m in [0.5, 1) */
    int q = (int)nearbyintf(m * 16.0f);      /* 4 significant bits: q in [8, 16] */
    if (q == 16) { q = 8; e += 1; }
    int exponent = e - 1 + 7;                /* a = (q/8) * 2^(e-1) */
    if (exponent > 15 || (exponent == 15 && q - 8 == 7))
        return sign | 0x7E;
    return sign | (uint8_t)(exponent << 3) | (uint8_t)(q - 8);
}

/* ------------------------------------------------------------------------------------------ */
/* Geometry                                                                                     */
/* ------------------------------------------------------------------------------------------ */

static int imax(int a, int b) { return a > b ? a : b; }
static int imin(int a, int b) { return a < b ? a : b; }

/* src/FeatureGridMath.cpp:47-60 */
static int lod_to_neural_lod(int lod, int gridScale, int neuralLods)
{
    static const int sharedMipsForGridScale[6] = {2, 3, 3, 3, 4, 4};
    int sharedMips = sharedMipsForGridScale[gridScale - 1];
    int neuralLod = (lod - sharedMips + 2) & ~1;
    return imax(0, imin(neuralLod, neuralLods - 2));
}

/* src/FeatureGridMath.cpp:62-65 */
static int grid_dimension(int imageDimension, int neuralLod, int gridScale)
{
    return imax((imageDimension / gridScale) >> neuralLod, 1);
}

int ntco_geometry(const NtcoTextureSet* set, NtcoGeometry* out)
{
    if (!set || !out || set->width < 1 || set->height < 1 || set->numMips < 1 || set->numMips > NTCO_MAX_MIPS ||
        set->gridSizeScale < 1 || set->gridSizeScale > 6 || set->numFeatures < 4 || set->numFeatures > 16 ||
        (set->numFeatures & 3) || set->channels < 2 || set->channels > 16 || (set->channels & 1))
        return -1;
    memset(out, 0, sizeof *out);

    /* src/FeatureGridMath.cpp:72-77 and src/FeatureGridHost.cpp:33-37 */
    int minImageSize = imin(set->width, set->height);
    int minGridSize = (int)((float)minImageSize / (float)set->gridSizeScale);
    int theoretical = imax(2, (int)(1.f + floorf(log2f((float)minGridSize)))) & ~1;
    int lastNeuralMip = lod_to_neural_lod(set->numMips - 1, set->gridSizeScale, NTCO_MAX_NEURAL_MIPS);
    out->numNeuralMips = imin(theoretical, lastNeuralMip + 2);
    out->numLayers = (set->numFeatures + 3) / 4;

    uint64_t pixels = 0;
    for (int m = 0; m < out->numNeuralMips; ++m)
    {
        out->latentWidth[m] = grid_dimension(set->width, m, set->gridSizeScale);
        out->latentHeight[m] = grid_dimension(set->height, m, set->gridSizeScale);
        out->latentPixelOffset[m] = pixels;
        pixels += (uint64_t)out->latentWidth[m] * (uint64_t)out->latentHeight[m];
    }
    out->latentPixelOffset[out->numNeuralMips] = pixels;

    /* src/TextureSet.cpp:88-101 (mip offsets) and :450-463 (positional constants) */
    uint64_t texels = 0;
    for (int mip = 0; mip < set->numMips; ++mip)
    {
        int w = imax(1, set->width >> mip), h = imax(1, set->height >> mip);
        int lod = lod_to_neural_lod(mip, set->gridSizeScale, out->numNeuralMips);
        out->mipWidth[mip] = w;
        out->mipHeight[mip] = h;
        out->neuralLod[mip] = lod;
        float widthScale = (float)out->latentWidth[lod] / (float)w;
        float heightScale = (float)out->latentHeight[lod] / (float)h;
        out->positionScale[mip] = 0.5f * fmaxf(widthScale, heightScale);
        out->positionLod[mip] = fmaxf(-1.f, fminf(1.f, 0.25f * log2f(out->positionScale[mip])));
        out->mipTexelOffset[mip] = texels;
        texels += (uint64_t)w * (uint64_t)h;
    }
    out->mipTexelOffset[set->numMips] = texels;
    return 0;
}

/* ------------------------------------------------------------------------------------------ */
/* Prepared network                                                                             */
/* ------------------------------------------------------------------------------------------ */

typedef struct Network
{
    /* file contents, per layer */
    const int8_t* wq[MLP_LAYERS];   /* [out][in] bytes: int8, or e4m3 bit patterns */
    const float* scale[MLP_LAYERS]; /* fp32, NULL for FP8 hidden layers */
    const int32_t* biasI[MLP_LAYERS];
    const h16* biasH[MLP_LAYERS];   /* fp16 bias of FP8 hidden layers */
    int layerIsFp8[MLP_LAYERS];
    /* decoded FP8 weights (exact) */
    float wf[MLP_LAYERS][64 * 64];
    /* binary16 weights and biases as the reference's CUDA path builds them */
    h16 wh[MLP_LAYERS][64 * 64];
    h16 bh[MLP_LAYERS][64];
} Network;

/* Constants of the reference's quantisers: src/tin/tin_mlp.h:42-45, src/tin/tin_activation.h:109-121. */
static const float kInputScale = 127.5f;
static const float kActStep = 3.1875f / 255.f; /* 0.0125f */
static const int kActBias = -113;

static void prepare_network(const NtcoTextureSet* set, int weights, Network* net)
{
    memset(net, 0, sizeof *net);
    const uint8_t* blob = (weights == NTCO_WEIGHTS_INT8) ? set->int8Blob : set->fp8Blob;
    size_t offset = 0;
    for (int l = 0; l < MLP_LAYERS; ++l)
    {
        net->wq[l] = (const int8_t*)(blob + offset);
        offset += (size_t)kLayerIn[l] * kLayerOut[l];
        net->layerIsFp8[l] = (weights == NTCO_WEIGHTS_FP8) && (l < MLP_LAYERS - 1);
    }
    if (weights == NTCO_WEIGHTS_INT8)
    {
        /* src/WeightLayout.cpp:228-238: all scale vectors, then all bias vectors */
        for (int l = 0; l < MLP_LAYERS; ++l) { net->scale[l] = (const float*)(blob + offset); offset += 4u * kLayerOut[l]; }
        for (int l = 0; l < MLP_LAYERS; ++l) { net->biasI[l] = (const int32_t*)(blob + offset); offset += 4u * kLayerOut[l]; }
    }
    else
    {
        /* src/WeightLayout.cpp:240-255: fp16 biases of layers 0-2, then scale and bias of layer 3 */
        for (int l = 0; l < MLP_LAYERS - 1; ++l) { net->biasH[l] = (const h16*)(blob + offset); offset += 2u * kLayerOut[l]; }
        net->scale[MLP_LAYERS - 1] = (const float*)(blob + offset); offset += 4u * kLayerOut[MLP_LAYERS - 1];
        net->biasI[MLP_LAYERS - 1] = (const int32_t*)(blob + offset);
    }

    for (int l = 0; l < MLP_LAYERS; ++l)
    {
        int in = kLayerIn[l], outc = kLayerOut[l];
        for (int n = 0; n < outc; ++n)
        {
            if (net->layerIsFp8[l])
            {
                /* src/Quantizer.cu:384-408: exact e4m3 -> half, bias copied */
                for (int k = 0; k < in; ++k)
                {
                    float w = ntco_e4m3_to_float((uint8_t)net->wq[l][n * in + k]);
                    net->wf[l][n * in + k] = w;
                    net->wh[l][n * in + k] = f2h(w);
                }
                net->bh[l][n] = net->biasH[l][n];
            }
            else
            {
                /* src/Quantizer.cu:325-382 (UnquantizeColumnInt8), same fp32 operation order */
                float layerScale = net->scale[l][n];
                float layerBias = (float)net->biasI[l][n] * layerScale;
                layerScale *= (l == 0) ? kInputScale : (1.f / kActStep);
                int integerWeightSum = 0;
                for (int k = 0; k < in; ++k)
                {
                    int q = net->wq[l][n * in + k];
                    net->wh[l][n * in + k] = f2h((float)q * layerScale);
                    integerWeightSum += q;
                }
                if (l != 0)
                    layerBias = fmaf((float)(integerWeightSum * kActBias) * layerScale, kActStep, layerBias);
                net->bh[l][n] = f2h(layerBias);
            }
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* Input vector                                                                                 */
/* ------------------------------------------------------------------------------------------ */

typedef struct MipContext
{
    int width, height;
    float invWidth, invHeight;
    int hiW, hiH, loW, loH;
    const uint16_t* hi; /* layer 0 plane of the high-res grid */
    const uint16_t* lo;
    size_t hiPlane, loPlane; /* pixels per layer */
    float positionScale, positionLod;
    int numLayers, numFeatures, channels;
} MipContext;

/* src/Quantizer.cu:490-495: value = float(nibble) * (1.f / 15.f), stored as binary16 (:568-571) */
static h16 g_latentValue[16];
static void init_tables(void)
{
    const float quantizationStep = 1.f / 15.f;
    for (int n = 0; n < 16; ++n)
        g_latentValue[n] = f2h((float)n * quantizationStep);
}

/* src/FeatureGridDevice.h:33-98.  The sample position uses a precomputed reciprocal of the mip
   size (u = (x + 0.5) * (1 / W)); the reference divides under --use_fast_math, which is the same
   value for power-of-two sizes. */
static void sample_grid(const uint16_t* plane0, size_t planePixels, int w, int h, int numLayers, float u, float v,
    int blendFma, h16* out /* numLayers*4 values */)
{
    float x = fmaf(u, (float)w, -0.5f);
    float y = fmaf(v, (float)h, -0.5f);
    float xbf = floorf(x), ybf = floorf(y);
    int xb = (int)xbf, yb = (int)ybf;
    float dx = x - xbf, dy = y - ybf;
    float dxn = 1.f - dx, dyn = 1.f - dy;
    h16 w00 = f2h(dxn * dyn), w01 = f2h(dx * dyn), w10 = f2h(dxn * dy), w11 = f2h(dx * dy);
    if (xb < 0) xb += w;
    if (yb < 0) yb += h;
    int x0 = xb % w, y0 = yb % h, x1 = (xb + 1) % w, y1 = (yb + 1) % h;
    const h16 two = 0x4000, minusOne = 0xBC00;

    for (int layer = 0; layer < numLayers; ++layer)
    {
        const uint16_t* plane = plane0 + (size_t)layer * planePixels;
        uint16_t p00 = plane[(size_t)y0 * w + x0], p01 = plane[(size_t)y0 * w + x1];
        uint16_t p10 = plane[(size_t)y1 * w + x0], p11 = plane[(size_t)y1 * w + x1];
        for (int j = 0; j < 4; ++j)
        {
            h16 l00 = g_latentValue[(p00 >> (4 * j)) & 15], l01 = g_latentValue[(p01 >> (4 * j)) & 15];
            h16 l10 = g_latentValue[(p10 >> (4 * j)) & 15], l11 = g_latentValue[(p11 >> (4 * j)) & 15];
            h16 d;
            if (blendFma == 2)
                d = hfma(l11, w11, hfma(l10, w10, hfma(l00, w00, hmul(l01, w01))));
            else if (blendFma)
                d = hfma(l11, w11, hfma(l10, w10, hfma(l01, w01, hmul(l00, w00))));
            else
                d = hadd(hadd(hadd(hmul(l00, w00), hmul(l01, w01)), hmul(l10, w10)), hmul(l11, w11));
            out[layer * 4 + j] = hfma(d, two, minusOne); /* d*2 is exact: same value fused or not */
        }
    }
}

/* src/RegressionKernels.h:59-85 */
static float fracf_(float t) { return t - floorf(t); }
static void encode_position(float xf, float yf, float lod, h16* out /* 14 values */)
{
    int idx = 0;
    for (int wave = 0; wave < 3; ++wave)
    {
        out[idx++] = f2h(fracf_(xf) * 2 - 1);
        out[idx++] = f2h(fracf_(yf) * 2 - 1);
        out[idx++] = f2h(fracf_(xf + 0.25f) * 2 - 1);
        out[idx++] = f2h(fracf_(yf + 0.25f) * 2 - 1);
        xf *= 2.f;
        yf *= 2.f;
    }
    out[idx++] = f2h(lod);
    out[idx++] = f2h(lod);
}

/* src/Inference.cu:46-61: 16 high-res features, 16 low-res features, 14 positional values, 2 zeros */
static void build_input(const MipContext* mc, int x, int y, int blendFma, h16 in[MLP_IN])
{
    memset(in, 0, MLP_IN * sizeof(h16));
    float u = ((float)x + 0.5f) * mc->invWidth;
    float v = ((float)y + 0.5f) * mc->invHeight;
    sample_grid(mc->hi, mc->hiPlane, mc->hiW, mc->hiH, mc->numLayers, u, v, blendFma, in);
    sample_grid(mc->lo, mc->loPlane, mc->loW, mc->loH, mc->numLayers, u, v, blendFma, in + MLP_FEATURES);
    encode_position((float)x * mc->positionScale, (float)y * mc->positionScale, mc->positionLod, in + 2 * MLP_FEATURES);
}

/* ------------------------------------------------------------------------------------------ */
/* Activation and quantisers                                                                    */
/* ------------------------------------------------------------------------------------------ */

/* src/tin/tin_activation.h:88-92: min(x, 3) * sat(x/3 + 0.5), every operation in binary16 */
uint16_t ntco_hgelu_clamp_half(uint16_t x)
{
    const h16 third = f2h(1 / 3.f), half_ = 0x3800, three = 0x4200;
    return hmul(hmin(x, three), hfma_sat(third, x, half_));
}

/* src/tin/tin_mlp.h:25-31: the integer code before it is scaled back; fused = one fma */
static int input_code_int8(h16 x, int fused)
{
    const h16 scale = f2h(kInputScale), halfv = 0x3800;
    h16 y = fused ? hfma(x, scale, 0xB800 /* -0.5 */) : hsub(hmul(x, scale), halfv);
    y = hfloor(y);
    y = hmax(hmin(y, f2h(127.f)), f2h(-127.f));
    return (int)h2f(y);
}

/* src/tin/tin_activation.h:94-99: code k = rint(y * 80), the activation is k * 0.0125 */
static int activation_code_int8(h16 y)
{
    h16 k = hrint(hmul(y, f2h(1.f / kActStep)));
    int code = (int)h2f(k);
    return imax(-15, imin(240, code));
}

/* ------------------------------------------------------------------------------------------ */
/* SPEC numerics: exact accumulation                                                            */
/* ------------------------------------------------------------------------------------------ */

static void mlp_spec(const Network* net, int weights, const h16 in[MLP_IN], h16 out[16])
{
    /* Activations travel as int8 codes (Int8 layers) or e4m3 bit patterns (FP8 layers). */
    int code[64];
    uint8_t f8[64];
    int fp8 = (weights == NTCO_WEIGHTS_FP8);

    for (int i = 0; i < MLP_IN; ++i)
    {
        if (fp8) f8[i] = ntco_half_to_e4m3(in[i]);
        else code[i] = input_code_int8(in[i], 1);
    }

    for (int l = 0; l < MLP_LAYERS; ++l)
    {
        int nin = kLayerIn[l], nout = kLayerOut[l];
        h16 x[64];
        for (int n = 0; n < nout; ++n)
        {
            if (net->layerIsFp8[l])
            {
                /* exact products and sum, one rounding to fp32, then binary16, then the fp16 bias */
                double acc = 0.0;
                for (int k = 0; k < nin; ++k)
                    acc += (double)ntco_e4m3_to_float(f8[k]) * (double)net->wf[l][n * nin + k];
                x[n] = hadd(f2h((float)acc), net->biasH[l][n]);
            }
            else
            {
                /* include/libntc/shaders/Inference.hlsli:146-165: float(acc + bias) * scale */
                int32_t acc = net->biasI[l][n];
                for (int k = 0; k < nin; ++k)
                    acc += code[k] * (int)net->wq[l][n * nin + k];
                x[n] = f2h((float)acc * net->scale[l][n]);
            }
        }
        if (l == MLP_LAYERS - 1)
        {
            for (int n = 0; n < nout; ++n)
                out[n] = h_is_special(x[n]) ? 0 : x[n]; /* src/Inference.cu:125-126 */
            return;
        }
        /* layers 0,1 quantise in the run's mode, layer 2 always to int8 (src/Inference.cu:66) */
        int nextFp8 = fp8 && (l < MLP_LAYERS - 2);
        for (int n = 0; n < nout; ++n)
        {
            h16 y = ntco_hgelu_clamp_half(x[n]);
            if (nextFp8) f8[n] = ntco_half_to_e4m3(y);
            else code[n] = activation_code_int8(y) + kActBias;
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* REF numerics: binary16 weights, activations and accumulators                                 */
/* ------------------------------------------------------------------------------------------ */

/* Fixed-point model of a tensor-core dot product with a binary16 accumulator: every addend (the
   accumulator and the exact products) is aligned to the largest exponent among them and truncated
   toward zero below 2^(emax - bits); the truncated addends are summed exactly and the sum is
   rounded once to binary16 (nearest even). */
static h16 ref_accumulate_aligned(h16 acc, const h16* a, const h16* w, int count, int bits)
{
    double addend[17];
    int n = 0, emax = -1000;
    addend[n++] = (double)h2f(acc);
    for (int i = 0; i < count; ++i)
        addend[n++] = (double)h2f(a[i]) * (double)h2f(w[i]);
    for (int i = 0; i < n; ++i)
    {
        if (!isfinite(addend[i]))
            return f2h((float)addend[i]);
        if (addend[i] != 0.0)
        {
            int e;
            frexp(addend[i], &e); /* |x| in [2^(e-1), 2^e) */
            if (e - 1 > emax) emax = e - 1;
        }
    }
    if (emax == -1000)
        return 0;
    double quantum = ldexp(1.0, emax - bits);
    double sum = 0.0;
    for (int i = 0; i < n; ++i)
        sum += trunc(addend[i] / quantum) * quantum; /* exact: power-of-two scaling */
    return d2h(sum);
}

static h16 ref_accumulate(h16 acc, const h16* a, const h16* w, int count, int mode)
{
    if (mode >= 16)
        return ref_accumulate_aligned(acc, a, w, count, mode);
    if (mode == 1)
    {
        float s = h2f(acc);
        for (int i = 0; i < count; ++i)
            s += h2f(a[i]) * h2f(w[i]);
        return f2h(s);
    }
    double s = (double)h2f(acc);
    for (int i = 0; i < count; ++i)
        s += (double)h2f(a[i]) * (double)h2f(w[i]);
    if (mode == 2)
    {
        float f = (float)s;
        if (fabs((double)f) > fabs(s))
            f = f_from_bits(f_bits(f) - 1);
        return f2h(f);
    }
    return d2h(s);
}

static void mlp_ref(const Network* net, const NtcoOptions* opt, const h16 in[MLP_IN], h16 out[16])
{
    int fp8 = (opt->weights == NTCO_WEIGHTS_FP8);
    int chunk = (opt->refAccChunk == 4 || opt->refAccChunk == 8) ? opt->refAccChunk : 16;
    h16 act[64];

    /* src/tin/tin_mlp.h:22-37 */
    const h16 invInputScale = f2h(1 / kInputScale);
    for (int i = 0; i < MLP_IN; ++i)
    {
        if (fp8) act[i] = f2h(ntco_e4m3_to_float(ntco_half_to_e4m3(in[i])));
        else act[i] = hmul(f2h((float)input_code_int8(in[i], opt->refQuantFma)), invInputScale);
    }

    for (int l = 0; l < MLP_LAYERS; ++l)
    {
        int nin = kLayerIn[l], nout = kLayerOut[l];
        h16 x[64];
        for (int n = 0; n < nout; ++n)
        {
            /* src/tin/tin_mlp.h:71-89: accumulator starts at the bias; src/tin/tin_matrix.h:598-625 */
            h16 acc = net->bh[l][n];
            for (int k0 = 0; k0 < nin; k0 += chunk)
                acc = ref_accumulate(acc, act + k0, &net->wh[l][n * nin + k0], chunk, opt->refAccMode);
            x[n] = acc;
        }
        if (l == MLP_LAYERS - 1)
        {
            for (int n = 0; n < nout; ++n)
                out[n] = h_is_special(x[n]) ? 0 : x[n];
            return;
        }
        int nextFp8 = fp8 && (l < MLP_LAYERS - 2);
        const h16 step = f2h(kActStep);
        for (int n = 0; n < nout; ++n)
        {
            h16 y = ntco_hgelu_clamp_half(x[n]);
            if (nextFp8)
                act[n] = f2h(ntco_e4m3_to_float(ntco_half_to_e4m3(y)));
            else
                act[n] = hmul(hrint(hmul(y, f2h(1.f / kActStep))), step); /* tin_activation.h:94-99 */
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* Drivers                                                                                      */
/* ------------------------------------------------------------------------------------------ */

static int setup_mip(const NtcoTextureSet* set, const NtcoGeometry* geo, int mip, MipContext* mc)
{
    int lod = geo->neuralLod[mip];
    mc->width = geo->mipWidth[mip];
    mc->height = geo->mipHeight[mip];
    mc->invWidth = 1.0f / (float)mc->width;
    mc->invHeight = 1.0f / (float)mc->height;
    mc->hiW = geo->latentWidth[lod];
    mc->hiH = geo->latentHeight[lod];
    /* src/TextureSet.cpp:1816-1817 */
    mc->loW = imax(mc->hiW >> 1, 1);
    mc->loH = imax(mc->hiH >> 1, 1);
    mc->numLayers = geo->numLayers;
    mc->hiPlane = (size_t)mc->hiW * mc->hiH;
    mc->loPlane = (size_t)geo->latentWidth[lod + 1] * geo->latentHeight[lod + 1];
    if (mc->loW != geo->latentWidth[lod + 1] || mc->loH != geo->latentHeight[lod + 1])
        return -1;
    mc->hi = set->latents + geo->latentPixelOffset[lod] * (size_t)geo->numLayers;
    mc->lo = set->latents + geo->latentPixelOffset[lod + 1] * (size_t)geo->numLayers;
    mc->positionScale = geo->positionScale[mip];
    mc->positionLod = geo->positionLod[mip];
    mc->numFeatures = set->numFeatures;
    mc->channels = set->channels;
    return 0;
}

static void decode_texel(const MipContext* mc, const Network* net, const NtcoOptions* opt, int x, int y, h16* out)
{
    h16 in[MLP_IN], result[16];
    int spec = (opt->numerics == NTCO_NUMERICS_SPEC);
    build_input(mc, x, y, spec ? 2 : opt->refBlendFma, in);
    if (spec) mlp_spec(net, opt->weights, in, result);
    else mlp_ref(net, opt, in, result);
    memcpy(out, result, (size_t)mc->channels * sizeof(h16));
}

/* Minimal parallel-for: `count` items handed out in blocks through an atomic counter. */
typedef void (*ItemFn)(void* context, long long item);
typedef struct ParallelJob
{
    ItemFn fn;
    void* context;
    long long count, block;
    atomic_llong next;
} ParallelJob;

static void* parallel_worker(void* arg)
{
    ParallelJob* job = (ParallelJob*)arg;
    for (;;)
    {
        long long begin = atomic_fetch_add(&job->next, job->block);
        if (begin >= job->count)
            return NULL;
        long long end = begin + job->block < job->count ? begin + job->block : job->count;
        for (long long i = begin; i < end; ++i)
            job->fn(job->context, i);
    }
}

static void parallel_for(const NtcoOptions* opt, long long count, long long block, ItemFn fn, void* context)
{
    long online = sysconf(_SC_NPROCESSORS_ONLN);
    int threads = opt->threads > 0 ? opt->threads : (online > 0 ? (int)online : 1);
    if (threads > 256) threads = 256;
    ParallelJob job;
    job.fn = fn;
    job.context = context;
    job.count = count;
    job.block = block > 0 ? block : 1;
    atomic_init(&job.next, 0);
    pthread_t ids[256];
    int started = 0;
    for (int t = 1; t < threads; ++t)
        if (pthread_create(&ids[started], NULL, parallel_worker, &job) == 0)
            ++started;
    parallel_worker(&job);
    for (int t = 0; t < started; ++t)
        pthread_join(ids[t], NULL);
}

typedef struct RowJob
{
    const MipContext* mc;
    const Network* net;
    const NtcoOptions* opt;
    int y0;
    uint16_t* out;
} RowJob;

static void decode_row(void* context, long long item)
{
    const RowJob* job = (const RowJob*)context;
    int y = job->y0 + (int)item;
    for (int x = 0; x < job->mc->width; ++x)
        decode_texel(job->mc, job->net, job->opt, x, y, job->out + ((size_t)item * job->mc->width + x) * job->mc->channels);
}

int ntco_decode_mip(const NtcoTextureSet* set, const NtcoOptions* opt, int mip, int y0, int y1, uint16_t* out)
{
    NtcoGeometry geo;
    if (!opt || !out || ntco_geometry(set, &geo) != 0 || mip < 0 || mip >= set->numMips)
        return -1;
    MipContext mc;
    if (setup_mip(set, &geo, mip, &mc) != 0 || y0 < 0 || y1 > mc.height || y0 > y1)
        return -1;
    init_tables();
    Network* net = (Network*)malloc(sizeof(Network));
    if (!net)
        return -1;
    prepare_network(set, opt->weights, net);
    RowJob job = {&mc, net, opt, y0, out};
    parallel_for(opt, y1 - y0, 1, decode_row, &job);
    free(net);
    return 0;
}

typedef struct SampleJob
{
    const NtcoTextureSet* set;
    const MipContext* mips;
    const Network* net;
    const NtcoOptions* opt;
    const float* queries;
    uint16_t* out;
} SampleJob;

static void sample_one(void* context, long long q)
{
    const SampleJob* job = (const SampleJob*)context;
    float u = job->queries[3 * q], v = job->queries[3 * q + 1], lod = job->queries[3 * q + 2];
    int mip = imax(0, imin(job->set->numMips - 1, (int)floorf(lod)));
    const MipContext* mc = &job->mips[mip];
    int x = imax(0, imin(mc->width - 1, (int)floorf(u * (float)mc->width)));
    int y = imax(0, imin(mc->height - 1, (int)floorf(v * (float)mc->height)));
    decode_texel(mc, job->net, job->opt, x, y, job->out + (size_t)q * mc->channels);
}

int ntco_sample(const NtcoTextureSet* set, const NtcoOptions* opt, const float* queries, size_t numQueries, uint16_t* out)
{
    NtcoGeometry geo;
    if (!opt || !out || !queries || ntco_geometry(set, &geo) != 0)
        return -1;
    MipContext mips[NTCO_MAX_MIPS];
    for (int m = 0; m < set->numMips; ++m)
        if (setup_mip(set, &geo, m, &mips[m]) != 0)
            return -1;
    init_tables();
    Network* net = (Network*)malloc(sizeof(Network));
    if (!net)
        return -1;
    prepare_network(set, opt->weights, net);
    SampleJob job = {set, mips, net, opt, queries, out};
    parallel_for(opt, (long long)numQueries, 4096, sample_one, &job);
    free(net);
    return 0;
}

/* ---------------------------------------------------------------------------------------------
 * ReadChannels: output formats, colour spaces, dithering
 * ------------------------------------------------------------------------------------------- */

/* src/CudaUtils.h:92-108 */
static float srgb_encode(float linear)
{
    return (linear <= 0.0031308f) ? linear * 12.92f : 1.055f * powf(linear, 1.0f / 2.4f) - 0.055f;
}
static float srgb_decode(float encoded)
{
    return (encoded <= 0.04045f) ? encoded / 12.92f : powf((encoded + 0.055f) / 1.055f, 2.4f);
}

/* src/CudaUtils.h:63-89 */
static const float kHlgA = 0.17883277f, kHlgB = 0.28466892f, kHlgC = 0.55991073f;
static float hlg_encode(float e)
{
    float sign = (e < 0.f) ? -1.f : 1.f;
    e = fabsf(e);
    return (e < 1.f) ? 0.5f * sqrtf(e) * sign : (kHlgA * logf(e - kHlgB) + kHlgC) * sign;
}
static float hlg_decode(float h)
{
    float sign = (h < 0.f) ? -1.f : 1.f;
    h = fabsf(h);
    return (h < 0.5f) ? 4.f * h * h * sign : (expf((h - kHlgC) / kHlgA) + kHlgB) * sign;
}

static float colorspace_decode(int space, float v) /* src/ImageProcessing.cu:86-98 */
{
    return space == 1 ? srgb_decode(v) : space == 2 ? hlg_decode(v) : v;
}
static float colorspace_encode(int space, float v) /* src/ImageProcessing.cu:100-112 */
{
    return space == 1 ? srgb_encode(v) : space == 2 ? hlg_encode(v) : v;
}

/* src/CudaUtils.h:111-184: per-pixel generator, Jenkins hash of the pixel index as seed, one
   Murmur3 round per draw with the draw counter as key. */
static uint32_t jenkins_hash(uint32_t a)
{
    a = (a + 0x7ed55d16u) + (a << 12);
    a = (a ^ 0xc761c23cu) ^ (a >> 19);
    a = (a + 0x165667b1u) + (a << 5);
    a = (a + 0xd3a2646cu) ^ (a << 9);
    a = (a + 0xfd7046c5u) + (a << 3);
    a = (a ^ 0xb55a4f09u) ^ (a >> 16);
    return a;
}
static uint32_t rotl32(uint32_t x, int r) { return (x << r) | (x >> (32 - r)); }
static uint32_t murmur3_draw(uint32_t seed, uint32_t index)
{
    uint32_t k = index * 0xcc9e2d51u;
    k = rotl32(k, 15) * 0x1b873593u;
    uint32_t hash = seed ^ k;
    hash = rotl32(hash, 13) * 5u + 0xe6546b64u;
    hash ^= 4u;
    hash ^= hash >> 16;
    hash *= 0x85ebca6bu;
    hash ^= hash >> 13;
    hash *= 0xc2b2ae35u;
    hash ^= hash >> 16;
    return hash;
}
static float uint_to_unit_float(uint32_t v) /* NextFloat: [0, 1) from the low 23 bits */
{
    uint32_t bits = (v & 0x7fffffu) | 0x3f800000u;
    float f;
    memcpy(&f, &bits, 4);
    return f - 1.f;
}

static int bytes_per_component(int format) /* src/TextureSet.cpp GetBytesPerPixelComponent */
{
    switch (format)
    {
    case 1: return 1;
    case 2: case 3: return 2;
    case 4: case 5: return 4;
    default: return 0;
    }
}

/* src/ImageProcessing.cu:139-164 */
static void write_component(uint8_t* dst, int ch, int format, int space, float value, float dither)
{
    value = colorspace_encode(space, value);
    switch (format)
    {
    case 1:
    {
        value += dither / 255.f;
        float r = roundf(value * 255.f);
        r = r < 255.f ? r : 255.f; /* NaN -> 255 as min(255, NaN) gives */
        r = r > 0.f ? r : 0.f;
        dst[ch] = (uint8_t)r;
        break;
    }
    case 2:
    {
        value += dither / 65535.f;
        float r = roundf(value * 65535.f);
        r = r < 65535.f ? r : 65535.f;
        r = r > 0.f ? r : 0.f;
        uint16_t u = (uint16_t)r;
        memcpy(dst + 2 * ch, &u, 2);
        break;
    }
    case 3:
    {
        float c = value < 65504.f ? value : 65504.f;
        c = c > -65504.f ? c : -65504.f;
        uint16_t h = f2h(c);
        memcpy(dst + 2 * ch, &h, 2);
        break;
    }
    case 4:
        memcpy(dst + 4 * ch, &value, 4);
        break;
    case 5:
    {
        float c = value > 0.f ? value : 0.f;
        uint32_t u = c >= 4294967296.f ? 0xffffffffu : (uint32_t)c;
        memcpy(dst + 4 * ch, &u, 4);
        break;
    }
    }
}

/* SetupBilinearFilter, src/ImageProcessing.cu:24-71 (the reference's division here is the GPU's
   approximate one; an exact one stands in, so a tap position on an exact texel boundary or a
   weight's last bit can differ). */
static void bilinear_filter(int srcWidth, int srcHeight, int dstWidth, int dstHeight, int x, int y, int* sx, int* sy, float w[4])
{
    if (srcWidth == dstWidth && srcHeight == dstHeight)
    {
        *sx = x;
        *sy = y;
        w[0] = 1.f;
        w[1] = w[2] = w[3] = 0.f;
        return;
    }
    const float u = ((float)x + 0.5f) / (float)dstWidth, v = ((float)y + 0.5f) / (float)dstHeight;
    float px = fmaf(u, (float)srcWidth, -0.5f), py = fmaf(v, (float)srcHeight, -0.5f);
    px = fmaxf(0.f, fminf((float)srcWidth - 1.f, px));
    py = fmaxf(0.f, fminf((float)srcHeight - 1.f, py));
    *sx = (int)floorf(px);
    *sy = (int)floorf(py);
    const float fx = px - floorf(px), fy = py - floorf(py);
    w[0] = (1.f - fx) * (1.f - fy);
    w[1] = fx * (1.f - fy);
    w[2] = (1.f - fx) * fy;
    w[3] = fx * fy;
}

/* CopyImageKernel, src/ImageProcessing.cu:220-266: `p` describes the source mip and the request,
   (dstWidth, dstHeight) the size handed back (the mip's size: a 1:1 copy; any other: bilinear). */
int ntco_read_channels_resized(const uint16_t* texels, const NtcoReadChannels* p, int dstWidth, int dstHeight, uint8_t* out)
{
    if (!texels || !p || !out)
        return -1;
    const int componentBytes = bytes_per_component(p->channelFormat);
    if (!componentBytes || p->width <= 0 || p->height <= 0 || dstWidth <= 0 || dstHeight <= 0 || p->firstChannel < 0 ||
        p->numChannels < 1 || p->firstChannel + p->numChannels > p->channels || p->pixelStride < 1 || p->rowPitch < p->pixelStride)
        return -1;
    const int dstChannels = (int)(p->pixelStride / (size_t)componentBytes); /* src/TextureSet.cpp:957 */
    for (int y = 0; y < dstHeight; ++y)
    {
        for (int x = 0; x < dstWidth; ++x)
        {
            int sx, sy;
            float w[4];
            bilinear_filter(p->width, p->height, dstWidth, dstHeight, x, y, &sx, &sy, w);
            uint8_t* dst = out + (size_t)y * p->rowPitch + (size_t)x * p->pixelStride;
            const uint32_t seed = jenkins_hash((uint32_t)x + (uint32_t)y * (uint32_t)dstWidth);
            uint32_t draw = 1;
            for (int ch = 0; ch < dstChannels; ++ch)
            {
                float value;
                if (ch < p->numChannels)
                {
                    const int srcSpace = p->srcColorSpaces ? p->srcColorSpaces[p->firstChannel + ch] : 0;
                    float taps[4] = {0.f, 0.f, 0.f, 0.f};
                    for (int t = 0; t < 4; ++t)
                        if (w[t] > 0.f)
                        {
                            const size_t index = ((size_t)(sy + (t >> 1)) * p->width + (size_t)(sx + (t & 1))) * p->channels;
                            taps[t] = colorspace_decode(srcSpace, h2f(texels[index + p->firstChannel + ch]));
                        }
                    /* the reference build's contraction: the second product stays a multiplication */
                    value = fmaf(taps[3], w[3], fmaf(taps[2], w[2], fmaf(taps[0], w[0], taps[1] * w[1])));
                }
                else
                    value = ch == 3 ? 1.f : 0.f; /* src/ImageProcessing.cu:166-170 */
                float dither = 0.f;
                if (p->useDithering)
                    dither = uint_to_unit_float(murmur3_draw(seed, draw++)) - 0.5f;
                const int dstSpace = (ch < p->numChannels && p->dstColorSpaces) ? p->dstColorSpaces[ch] : 0;
                write_component(dst, ch, p->channelFormat, dstSpace, value, dither);
            }
        }
    }
    return 0;
}

int ntco_read_channels(const uint16_t* texels, const NtcoReadChannels* p, uint8_t* out)
{
    return p ? ntco_read_channels_resized(texels, p, p->width, p->height, out) : -1;
}

/* ------------------------------------------------------------------------------------------- */
/* Encoder-side producers (src/Quantizer.cu)                                                    */
/* ------------------------------------------------------------------------------------------- */

static float flush_denormal(float x)
{
    return fabsf(x) < 1.17549435e-38f ? copysignf(0.f, x) : x;
}

/* QuantizeValue(value, 4), src/Quantizer.cu:481-487.  std::min(1.f, NaN) is 1. */
static uint32_t latent_code(uint16_t bits)
{
    float value = h2f(bits);
    value = (value < 1.f) ? value : 1.f;
    value = (0.f < value) ? value : 0.f;
    const float step = 1.f / 15.f;
    return (uint32_t)roundf(value / step);
}

/* PackLatentsKernel, src/Quantizer.cu:497-527. */
int ntco_pack_latents(const uint16_t* latents, int width, int height, int numLayers, size_t latentStride, uint16_t* packed)
{
    if (!latents || !packed || width <= 0 || height <= 0 || numLayers <= 0)
        return -1;
    const size_t texels = (size_t)width * (size_t)height;
    for (int z = 0; z < numLayers; ++z)
        for (size_t t = 0; t < texels; ++t)
        {
            const uint16_t* src = latents + (size_t)z * latentStride * 2 + t * 2;
            packed[(size_t)z * texels + t] = (uint16_t)(latent_code(src[0]) | (latent_code(src[1]) << 4)
                | (latent_code(src[latentStride]) << 8) | (latent_code(src[latentStride + 1]) << 12));
        }
    return 0;
}

static const int kProducerInputs[4] = {48, 64, 48, 32};
static const int kProducerOutputs[4] = {64, 48, 32, 16};

/* QuantizeColumnInt8, src/Quantizer.cu:90-208.  The reference's divisions are the GPU's approximate
   ones (it is built with --use_fast_math); exact divisions stand in for them here, so a code or an
   integer bias whose unrounded value lies within a few units in the last place of a tie, and the
   last bits of the first layer's scales, can differ from what the GPU produces. */
static void quantize_column_int8(int layer, const uint16_t* weights, uint16_t bias, int8_t* codes, uint16_t* rounded,
    float* scaleOut, int32_t* biasOut, float outputScale, float outputBias)
{
    const int rows = kProducerInputs[layer];
    float low = FLT_MAX, high = FLT_MIN;
    for (int r = 0; r < rows; ++r)
    {
        const float w = h2f(weights[r]);
        low = (w < low) ? w : low;
        high = (high < w) ? w : high;
    }
    const float limit = fmaxf(fabsf(high), fabsf(low));
    const float inverseLimit = flush_denormal(1.f / limit);
    const float scale = 127.5f, inverseScale = 1.f / 127.5f;
    const float ratio = flush_denormal(scale / limit);
    int sum = 0;
    for (int r = 0; r < rows; ++r)
    {
        const float w = h2f(weights[r]);
        float q = (r & 1) ? roundf(flush_denormal(w * ratio)) : roundf(flush_denormal(flush_denormal(w * scale) * inverseLimit));
        q = (127.f < q) ? 127.f : q;   /* std::min / std::max keep a NaN first operand */
        q = (q < -127.f) ? -127.f : q;
        codes[r] = isnan(q) ? 0 : (int8_t)q;
        sum += codes[r];
        if (rounded)
            rounded[r] = f2h(flush_denormal(flush_denormal(q * limit) * inverseScale));
    }

    float layerScale = flush_denormal(limit * inverseScale);
    float layerBias = h2f(bias);
    if (layer == 0)
        layerScale = flush_denormal(layerScale / 127.5f);
    else
    {
        const float activationStep = 3.1875f / 255.f;
        const int activationBias = -113;
        layerScale = flush_denormal(layerScale * activationStep);
        layerBias = flush_denormal(fmaf(-(float)(sum * activationBias), layerScale, layerBias));
        if (layer == 3)
        {
            layerScale = flush_denormal(layerScale * outputScale);
            layerBias = flush_denormal(fmaf(layerBias, outputScale, outputBias));
        }
    }
    int32_t integerBias;
    if (layerScale == 0.f)
    {
        layerScale = 1.f / 65536.f;
        integerBias = (int32_t)roundf(layerBias * 65536.f);
        for (int r = 0; r < rows; ++r)
            codes[r] = 0;
    }
    else
        integerBias = (int32_t)roundf(layerBias / layerScale);
    *scaleOut = layerScale;
    *biasOut = integerBias;
}

/* QuantizeNetworkInt8Kernel / QuantizeNetworkFP8Kernel, src/Quantizer.cu:254-303; the blob's layout
   is the one of src/WeightLayout.cpp:142-268. */
int ntco_quantize_network(const uint16_t* weights, const uint16_t* biases, const float* outputScale, const float* outputBias,
    int useFP8, uint8_t* blob, uint16_t* roundedWeights)
{
    if (!weights || !biases || !blob)
        return -1;
    const size_t weightBytes = 48 * 64 + 64 * 48 + 48 * 32 + 32 * 16;
    size_t weightOffset = 0, columnOffset = 0;
    for (int layer = 0; layer < 4; ++layer)
    {
        const int rows = kProducerInputs[layer], cols = kProducerOutputs[layer];
        for (int col = 0; col < cols; ++col)
        {
            const uint16_t* w = weights + weightOffset + (size_t)col * rows;
            uint16_t* rounded = roundedWeights ? roundedWeights + weightOffset + (size_t)col * rows : NULL;
            uint8_t* codes = blob + weightOffset + (size_t)col * rows;
            const uint16_t bias = biases[columnOffset + col];
            const float os = outputScale ? outputScale[col & 15] : 1.f, ob = outputBias ? outputBias[col & 15] : 0.f;
            float scaleValue;
            int32_t biasValue;
            if (!useFP8)
            {
                quantize_column_int8(layer, w, bias, (int8_t*)codes, rounded, &scaleValue, &biasValue, os, ob);
                memcpy(blob + weightBytes + 4 * (columnOffset + col), &scaleValue, 4);
                memcpy(blob + weightBytes + 4 * 160 + 4 * (columnOffset + col), &biasValue, 4);
            }
            else if (layer < 3)
            {
                for (int r = 0; r < rows; ++r) /* QuantizeColumnFP8, src/Quantizer.cu:210-252 */
                {
                    codes[r] = ntco_half_to_e4m3(w[r]);
                    if (rounded)
                        rounded[r] = f2h(ntco_e4m3_to_float(codes[r]));
                }
                memcpy(blob + weightBytes + 2 * (columnOffset + col), &bias, 2);
            }
            else
            {
                quantize_column_int8(layer, w, bias, (int8_t*)codes, rounded, &scaleValue, &biasValue, os, ob);
                uint8_t* tail = blob + weightBytes + 2 * 144;
                memcpy(tail + 4 * col, &scaleValue, 4);
                memcpy(tail + 64 + 4 * col, &biasValue, 4);
            }
        }
        weightOffset += (size_t)rows * cols;
        columnOffset += (size_t)cols;
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------- */
/* BC4 / BC5 block compression (src/shaders/BlockCompressCommon.hlsli:510-796,                  */
/* CompressBC4.hlsl, CompressBC5.hlsl)                                                          */
/*                                                                                             */
/* PARITY UNPINNED: the reference runs these encoders as compute shaders through a graphics    */
/* API, which cannot run here; this is a restatement of the shader's arithmetic in C (binary32 */
/* operations in the shader's order, nothing fused; HLSL round = half to even; clamp and       */
/* saturate treat NaN as the shader's min / max do).                                            */
/* ------------------------------------------------------------------------------------------- */

typedef struct { uint32_t x, y; } bc_uint2;

static void bc4_palette(uint32_t a0, uint32_t a1, uint32_t alphas[8])
{
    alphas[0] = a0;
    alphas[1] = a1;
    if (a0 > a1)
    {
        alphas[2] = (6 * a0 + 1 * a1 + 3) / 7;
        alphas[3] = (5 * a0 + 2 * a1 + 3) / 7;
        alphas[4] = (4 * a0 + 3 * a1 + 3) / 7;
        alphas[5] = (3 * a0 + 4 * a1 + 3) / 7;
        alphas[6] = (2 * a0 + 5 * a1 + 3) / 7;
        alphas[7] = (1 * a0 + 6 * a1 + 3) / 7;
    }
    else
    {
        alphas[2] = (4 * a0 + 1 * a1 + 2) / 5;
        alphas[3] = (3 * a0 + 2 * a1 + 2) / 5;
        alphas[4] = (2 * a0 + 3 * a1 + 2) / 5;
        alphas[5] = (1 * a0 + 4 * a1 + 2) / 5;
        alphas[6] = 0;
        alphas[7] = 255;
    }
}

static uint32_t bc4_get_index(bc_uint2 block, int pixel)
{
    const uint64_t bits = (uint64_t)block.x | ((uint64_t)block.y << 32);
    return (uint32_t)(bits >> (16 + 3 * pixel)) & 7u;
}

static float bc4_compute_indices(const uint32_t values[16], bc_uint2* block) /* :605-632 */
{
    uint32_t alphas[8];
    bc4_palette(block->x & 0xff, (block->x >> 8) & 0xff, alphas);
    uint64_t bits = block->x & 0xffffu;
    float total = 0.f;
    for (int i = 0; i < 16; ++i)
    {
        int best = 0x7fffffff;
        uint32_t bestIndex = 8;
        for (uint32_t p = 0; p < 8; ++p)
        {
            int d = (int)values[i] - (int)alphas[p];
            d *= d;
            if (d < best)
            {
                best = d;
                bestIndex = p;
            }
        }
        total += (float)best;
        bits |= (uint64_t)(bestIndex & 7u) << (16 + 3 * i);
    }
    block->x = (uint32_t)bits;
    block->y = (uint32_t)(bits >> 32);
    return total;
}

static float bc_clamp_byte(float x) /* clamp(x, 0, 255): min(max(x, 0), 255), NaN -> 0 */
{
    x = fmaxf(x, 0.f);
    return fminf(x, 255.f);
}

static void bc4_optimize8(const uint32_t values[16], bc_uint2* block, int zeroAlpha1, int oneAlpha0) /* :634-670 */
{
    float alpha2 = 0, beta2 = 0, alphabeta = 0, alphax = 0, betax = 0;
    for (int i = 0; i < 16; ++i)
    {
        const uint32_t index = bc4_get_index(*block, i);
        const float alpha = index < 2 ? 1.0f - (float)index : (8.0f - (float)index) / 7.0f;
        const float beta = 1 - alpha;
        alpha2 += alpha * alpha;
        beta2 += beta * beta;
        alphabeta += alpha * beta;
        alphax += alpha * (float)values[i];
        betax += beta * (float)values[i];
    }
    const float factor = 1.0f / (alpha2 * beta2 - alphabeta * alphabeta);
    const float a = (alphax * beta2 - betax * alphabeta) * factor;
    const float b = (betax * alpha2 - alphax * alphabeta) * factor;
    uint32_t alpha0 = oneAlpha0 ? 255u : (uint32_t)rintf(bc_clamp_byte(a));
    uint32_t alpha1 = zeroAlpha1 ? 0u : (uint32_t)rintf(bc_clamp_byte(b));
    if (alpha0 < alpha1)
    {
        const uint32_t t = alpha0;
        alpha0 = alpha1;
        alpha1 = t;
    }
    block->x = (block->x & 0xffff0000u) | (alpha0 & 0xff) | ((alpha1 & 0xff) << 8);
}

static void bc4_optimize6(const uint32_t values[16], bc_uint2* block) /* :672-708 */
{
    float alpha2 = 0, beta2 = 0, alphabeta = 0, alphax = 0, betax = 0;
    for (int i = 0; i < 16; ++i)
    {
        const uint32_t index = bc4_get_index(*block, i);
        float alpha;
        if (index < 2)
            alpha = 1.0f - (float)index;
        else if (index < 6)
            alpha = (6.0f - (float)index) / 5.0f;
        else
            continue;
        const float beta = 1.0f - alpha;
        alpha2 += alpha * alpha;
        beta2 += beta * beta;
        alphabeta += alpha * beta;
        alphax += alpha * (float)values[i];
        betax += beta * (float)values[i];
    }
    const float factor = alpha2 * beta2 - alphabeta * alphabeta;
    if (factor == 0.0f)
        return;
    const float a = (alphax * beta2 - betax * alphabeta) / factor;
    const float b = (betax * alpha2 - alphax * alphabeta) / factor;
    const uint32_t alpha0 = (uint32_t)rintf(bc_clamp_byte(a)), alpha1 = (uint32_t)rintf(bc_clamp_byte(b));
    block->x = (block->x & 0xffff0000u) | (alpha0 & 0xff) | ((alpha1 & 0xff) << 8);
}

static int bc4_same_indices(bc_uint2 a, bc_uint2 b)
{
    return (a.x & 0xffff0000u) == (b.x & 0xffff0000u) && a.y == b.y;
}

static bc_uint2 bc4_compress_fast(const float pixels[16]) /* :710-796 */
{
    uint32_t values[16];
    uint32_t mina = 255, maxa = 0, mina_no01 = 255, maxa_no01 = 0;
    for (int i = 0; i < 16; ++i)
    {
        float s = pixels[i];
        s = isnan(s) ? 0.f : fminf(fmaxf(s, 0.f), 1.f);
        values[i] = (uint32_t)rintf(s * 255.0f);
        if (values[i] < mina) mina = values[i];
        if (values[i] > maxa) maxa = values[i];
        if (values[i] != 0 && values[i] < mina_no01) mina_no01 = values[i];
        if (values[i] != 255 && values[i] > maxa_no01) maxa_no01 = values[i];
    }
    const int zeroAlpha1 = mina == 0, oneAlpha0 = maxa == 255;

    bc_uint2 block = {0, 0};
    const uint32_t start0 = oneAlpha0 ? 255u : maxa - (maxa - mina) / 34u;
    const uint32_t start1 = zeroAlpha1 ? 0u : mina + (maxa - mina) / 34u;
    block.x = (start0 & 0xff) | ((start1 & 0xff) << 8);
    float besterror = bc4_compute_indices(values, &block);
    bc_uint2 bestblock = block;
    for (int i = 0; i < 8; ++i)
    {
        bc4_optimize8(values, &block, zeroAlpha1, oneAlpha0);
        const float error = bc4_compute_indices(values, &block);
        if (error >= besterror)
            break;
        if (bc4_same_indices(block, bestblock))
        {
            bestblock = block;
            break;
        }
        bestblock = block;
        besterror = error;
    }

    const uint32_t six0 = mina_no01 + (maxa_no01 - mina_no01) / 34u; /* unsigned wrap-around as in the shader */
    const uint32_t six1 = maxa_no01 - (maxa_no01 - mina_no01) / 34u;
    block.x = (block.x & 0xffff0000u) | (six0 & 0xff) | ((six1 & 0xff) << 8);
    float besterror2 = bc4_compute_indices(values, &block);
    bc_uint2 bestblock2 = block;
    for (int i = 0; i < 8; ++i)
    {
        bc4_optimize6(values, &block);
        const float error = bc4_compute_indices(values, &block);
        if (error >= besterror2)
            break;
        if (bc4_same_indices(block, bestblock2))
        {
            bestblock2 = block;
            break;
        }
        bestblock2 = block;
        besterror2 = error;
    }
    if (besterror2 < besterror)
        bestblock = bestblock2;
    return bestblock;
}

/* CompressBC4.hlsl / CompressBC5.hlsl main(): one block per 4x4 texels starting at (srcLeft, srcTop);
   texels outside the image read as 0.  `texels` is interleaved fp16 [height][width][channels];
   `formatChannels` 1 = BC4, 2 = BC5; `blocks` receives 8 * formatChannels bytes per block, row-major. */
int ntco_block_compress(const uint16_t* texels, int width, int height, int channels, int firstChannel, int formatChannels,
    int srcLeft, int srcTop, int widthInBlocks, int heightInBlocks, uint8_t* blocks)
{
    if (!texels || !blocks || (formatChannels != 1 && formatChannels != 2) || firstChannel < 0
        || firstChannel + formatChannels > channels || widthInBlocks <= 0 || heightInBlocks <= 0)
        return -1;
    for (int by = 0; by < heightInBlocks; ++by)
        for (int bx = 0; bx < widthInBlocks; ++bx)
            for (int c = 0; c < formatChannels; ++c)
            {
                float pixels[16];
                for (int i = 0; i < 16; ++i)
                {
                    const int x = srcLeft + bx * 4 + (i & 3), y = srcTop + by * 4 + (i >> 2);
                    pixels[i] = (x < width && y < height)
                        ? h2f(texels[((size_t)y * width + x) * channels + firstChannel + c]) : 0.f;
                }
                const bc_uint2 block = bc4_compress_fast(pixels);
                uint8_t* dst = blocks + (((size_t)by * widthInBlocks + bx) * formatChannels + c) * 8;
                memcpy(dst, &block.x, 4);
                memcpy(dst + 4, &block.y, 4);
            }
    return 0;
}

/* ------------------------------------------------------------------------------------------- */
/* BC1 / BC2 / BC3 (src/shaders/BlockCompressCommon.hlsli:82-508, CompressBC1-3.hlsl).          */
/* PARITY UNPINNED, as for BC4 / BC5 above.                                                     */
/* ------------------------------------------------------------------------------------------- */

typedef struct { float x, y, z; } bc_float3;
typedef struct { float x, y, z, w; } bc_float4;

static uint16_t g_match5[256], g_match6[256];
static int g_matchReady = 0;

/* Single-colour match tables; see the note at ntco_color_match_table in the header. */
static void bc_fill_match_table(int bits, uint16_t* table)
{
    const int size = 1 << bits;
    int expanded[64];
    for (int c = 0; c < size; ++c)
        expanded[c] = (c << (8 - bits)) | (c >> (2 * bits - 8));
    for (int i = 0; i < 256; ++i)
    {
        int best = 1 << 30;
        for (int mn = 0; mn < size; ++mn)
            for (int mx = 0; mx < size; ++mx)
            {
                const int cost = 1000 * abs((2 * expanded[mx] + expanded[mn]) / 3 - i) + 14 * abs(expanded[mx] - expanded[mn]);
                if (cost < best)
                {
                    best = cost;
                    table[i] = (uint16_t)(mx | (mn << 8));
                }
            }
    }
}

static void bc_ensure_tables(void)
{
    if (!g_matchReady)
    {
        bc_fill_match_table(5, g_match5);
        bc_fill_match_table(6, g_match6);
        g_matchReady = 1;
    }
}

int ntco_color_match_table(int bits, uint16_t* table)
{
    if ((bits != 5 && bits != 6) || !table)
        return -1;
    bc_fill_match_table(bits, table);
    return 0;
}

static float bc_saturate(float x) { return isnan(x) ? 0.f : fminf(fmaxf(x, 0.f), 1.f); }
static bc_float3 f3(float x, float y, float z) { bc_float3 v = {x, y, z}; return v; }
static bc_float3 f3_sub(bc_float3 a, bc_float3 b) { return f3(a.x - b.x, a.y - b.y, a.z - b.z); }
static bc_float3 f3_add(bc_float3 a, bc_float3 b) { return f3(a.x + b.x, a.y + b.y, a.z + b.z); }
static bc_float3 f3_mul(bc_float3 a, float s) { return f3(a.x * s, a.y * s, a.z * s); }
static bc_float3 f3_saturate(bc_float3 a) { return f3(bc_saturate(a.x), bc_saturate(a.y), bc_saturate(a.z)); }
static float f3_dot(bc_float3 a, bc_float3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
static bc_float3 f3_lerp(bc_float3 x, bc_float3 y, float s) { return f3_add(x, f3_mul(f3_sub(y, x), s)); }
static bc_float3 rgb_of(bc_float4 p) { return f3(p.x, p.y, p.z); }
static float f4_dot(bc_float4 a) { return a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w; }
static float color_distance(bc_float3 c0, bc_float3 c1) { const bc_float3 d = f3_sub(c0, c1); return f3_dot(d, d); }

static uint32_t bc1_select_best_index(const float d[4], float* error) /* :116-144 */
{
    if (fminf(d[0], d[1]) < fminf(d[2], d[3]))
    {
        if (d[0] < d[1]) { *error = d[0]; return 0; }
        *error = d[1];
        return 1;
    }
    if (d[2] < d[3]) { *error = d[2]; return 2; }
    *error = d[3];
    return 3;
}

static uint32_t bc1_compute_index4(bc_float4 color, bc_float3 maxColor, bc_float3 minColor, float* error) /* :146-159 */
{
    const bc_float3 color2 = f3_lerp(maxColor, minColor, 1.0f / 3.0f);
    const bc_float3 color3 = f3_lerp(maxColor, minColor, 2.0f / 3.0f);
    const float alphaDistance = (1.0f - color.w) * (1.0f - color.w);
    float d[4];
    d[0] = color_distance(maxColor, rgb_of(color)) + alphaDistance;
    d[1] = color_distance(minColor, rgb_of(color)) + alphaDistance;
    d[2] = color_distance(color2, rgb_of(color)) + alphaDistance;
    d[3] = color_distance(color3, rgb_of(color)) + alphaDistance;
    return bc1_select_best_index(d, error);
}

static uint32_t bc1_compute_index3(bc_float4 color, bc_float3 maxColor, bc_float3 minColor, float threshold, float* error) /* :161-179 */
{
    if (color.w <= threshold)
    {
        *error = 0;
        return 3;
    }
    const bc_float3 color2 = f3_lerp(maxColor, minColor, 0.5f);
    const float alphaDistance = (1.0f - color.w) * (1.0f - color.w);
    float d[4];
    d[0] = color_distance(maxColor, rgb_of(color)) + alphaDistance;
    d[1] = color_distance(minColor, rgb_of(color)) + alphaDistance;
    d[2] = color_distance(color2, rgb_of(color)) + alphaDistance;
    d[3] = f4_dot(color);
    return bc1_select_best_index(d, error);
}

static bc_float3 expand565(uint32_t w)
{
    return f3((float)((w >> 11) & 0x1f) * 1.0f / 31.0f, (float)((w >> 5) & 0x3f) * 1.0f / 63.0f, (float)(w & 0x1f) * 1.0f / 31.0f);
}

static bc_float3 round_and_expand565(bc_float3 v, uint32_t* w)
{
    const uint32_t x = (uint32_t)rintf(bc_saturate(v.x) * 31.0f);
    const uint32_t y = (uint32_t)rintf(bc_saturate(v.y) * 63.0f);
    const uint32_t z = (uint32_t)rintf(bc_saturate(v.z) * 31.0f);
    *w = (x << 11) | (y << 5) | z;
    return expand565(*w);
}

static int clamp_byte_index(float v)
{
    const int i = (int)rintf(v);
    return i < 0 ? 0 : i > 255 ? 255 : i; /* the shader indexes unclamped; both implementations here clamp */
}

static bc_uint2 bc1_encode_single_color(const bc_float4 pixels[16], float* blockError) /* :205-247 */
{
    bc_float3 average = f3(0, 0, 0);
    for (int i = 0; i < 16; ++i)
        average = f3_add(average, rgb_of(pixels[i]));
    average = f3(average.x / 16.0f, average.y / 16.0f, average.z / 16.0f);
    const uint32_t mr = g_match5[clamp_byte_index(average.x * 255.f)], mg = g_match6[clamp_byte_index(average.y * 255.f)],
                   mb = g_match5[clamp_byte_index(average.z * 255.f)];
    const uint32_t color0 = ((mr & 0x1f) << 11) | ((mg & 0x3f) << 5) | (mb & 0x1f);
    const uint32_t color1 = (((mr >> 8) & 0x1f) << 11) | (((mg >> 8) & 0x3f) << 5) | ((mb >> 8) & 0x1f);
    bc_uint2 result;
    if (color0 < color1)
    {
        result.x = (color0 << 16) | color1;
        result.y = 0xffffffffu;
    }
    else
    {
        result.x = (color1 << 16) | color0;
        result.y = 0xaaaaaaaau;
    }
    const bc_float3 encoded = f3_lerp(expand565(color0), expand565(color1), 1.0f / 3.0f);
    *blockError = 0;
    for (int i = 0; i < 16; ++i)
    {
        const bc_float4 diff = {pixels[i].x - encoded.x, pixels[i].y - encoded.y, pixels[i].z - encoded.z, pixels[i].w - 1.0f};
        *blockError += f4_dot(diff);
    }
    return result;
}

static void bc_swapf(float* a, float* b) { const float t = *a; *a = *b; *b = t; }

static void bc_orient(bc_float3* minColor, bc_float3* maxColor, float cov_rg, float cov_rb, float cov_gb)
{
    if (minColor->x != maxColor->x)
    {
        if (cov_rg < 0) bc_swapf(&minColor->y, &maxColor->y);
        if (cov_rb < 0) bc_swapf(&minColor->z, &maxColor->z);
    }
    else if (minColor->y != maxColor->y)
    {
        if (cov_gb < 0) bc_swapf(&minColor->z, &maxColor->z);
    }
}

static float keep_extreme(float current, float refitted)
{
    return (current == 0.0f || current == 1.0f) ? current : bc_saturate(refitted);
}

static bc_uint2 bc1_compress_fast(const bc_float4 pixels[16], float* blockError) /* :249-376 */
{
    bc_float3 sums = f3(0, 0, 0), minColor = f3(1, 1, 1), maxColor = f3(0, 0, 0);
    for (int i = 0; i < 16; ++i)
    {
        const bc_float3 c = rgb_of(pixels[i]);
        sums = f3_add(sums, c);
        minColor = f3(fminf(minColor.x, c.x), fminf(minColor.y, c.y), fminf(minColor.z, c.z));
        maxColor = f3(fmaxf(maxColor.x, c.x), fmaxf(maxColor.y, c.y), fmaxf(maxColor.z, c.z));
    }
    const bc_float3 center = f3(sums.x / 16.0f, sums.y / 16.0f, sums.z / 16.0f);
    float cov_rg = 0, cov_rb = 0, cov_gb = 0;
    for (int i = 0; i < 16; ++i)
    {
        const bc_float3 pix = f3_sub(rgb_of(pixels[i]), center);
        cov_rg += pix.x * pix.y;
        cov_rb += pix.x * pix.z;
        cov_gb += pix.y * pix.z;
    }
    bc_orient(&minColor, &maxColor, cov_rg, cov_rb, cov_gb);
    const bc_float3 extent = f3_sub(maxColor, minColor);
    const bc_float3 inset = f3(extent.x / 16.0f, extent.y / 16.0f, extent.z / 16.0f);
    maxColor = f3_saturate(f3_sub(maxColor, inset));
    minColor = f3_saturate(f3_add(minColor, inset));

    uint32_t color0 = 0, color1 = 0;
    for (int pass = 0; pass < 4; ++pass)
    {
        float alpha2 = 0, beta2 = 0, alphabeta = 0;
        bc_float3 alphax = f3(0, 0, 0), betax = f3(0, 0, 0);
        for (int i = 0; i < 16; ++i)
        {
            float pixelError;
            const uint32_t index = bc1_compute_index4(pixels[i], maxColor, minColor, &pixelError);
            float beta = (float)(index & 1);
            if (index & 2)
                beta = (1 + beta) / 3.0f;
            const float alpha = 1.0f - beta;
            alpha2 += alpha * alpha;
            beta2 += beta * beta;
            alphabeta += alpha * beta;
            alphax = f3_add(alphax, f3_mul(rgb_of(pixels[i]), alpha));
            betax = f3_add(betax, f3_mul(rgb_of(pixels[i]), beta));
        }
        const float denom = alpha2 * beta2 - alphabeta * alphabeta;
        if (fabsf(denom) > 0.0001f)
        {
            const float factor = 1.0f / denom;
            const bc_float3 a = f3_mul(f3_sub(f3_mul(alphax, beta2), f3_mul(betax, alphabeta)), factor);
            const bc_float3 b = f3_mul(f3_sub(f3_mul(betax, alpha2), f3_mul(alphax, alphabeta)), factor);
            minColor = f3(keep_extreme(minColor.x, b.x), keep_extreme(minColor.y, b.y), keep_extreme(minColor.z, b.z));
            maxColor = f3(keep_extreme(maxColor.x, a.x), keep_extreme(maxColor.y, a.y), keep_extreme(maxColor.z, a.z));
        }
        uint32_t newColor0, newColor1;
        maxColor = round_and_expand565(maxColor, &newColor0);
        minColor = round_and_expand565(minColor, &newColor1);
        if (newColor0 == color0 && newColor1 == color1)
            break;
        color0 = newColor0;
        color1 = newColor1;
    }
    if (color0 == color1)
    {
        if (color0 == 0)
        {
            color0 = 1;
            maxColor = expand565(color0);
        }
        else
        {
            color1 = color0 - 1;
            minColor = expand565(color1);
        }
    }
    else if (color0 < color1)
    {
        const bc_float3 t = maxColor;
        maxColor = minColor;
        minColor = t;
        const uint32_t c = color0;
        color0 = color1;
        color1 = c;
    }
    uint32_t indices = 0;
    *blockError = 0;
    for (int i = 0; i < 16; ++i)
    {
        float pixelError;
        const uint32_t index = bc1_compute_index4(pixels[i], maxColor, minColor, &pixelError);
        indices |= index << (2 * i);
        *blockError += pixelError;
    }
    bc_uint2 result = {(color1 << 16) | color0, indices};
    return result;
}

static bc_uint2 bc1a_compress_fast(const bc_float4 pixels[16], float threshold, float* blockError) /* :378-493 */
{
    bc_float3 sums = f3(0, 0, 0), minColor = f3(1, 1, 1), maxColor = f3(0, 0, 0);
    int opaqueCount = 0;
    for (int i = 0; i < 16; ++i)
        if (!(pixels[i].w <= threshold))
        {
            const bc_float3 c = rgb_of(pixels[i]);
            sums = f3_add(sums, c);
            minColor = f3(fminf(minColor.x, c.x), fminf(minColor.y, c.y), fminf(minColor.z, c.z));
            maxColor = f3(fmaxf(maxColor.x, c.x), fmaxf(maxColor.y, c.y), fmaxf(maxColor.z, c.z));
            opaqueCount += 1;
        }
    const float count = (float)opaqueCount;
    const bc_float3 center = opaqueCount > 0 ? f3(sums.x / count, sums.y / count, sums.z / count) : f3(0, 0, 0);
    float cov_rg = 0, cov_rb = 0, cov_gb = 0;
    for (int i = 0; i < 16; ++i)
        if (!(pixels[i].w <= threshold))
        {
            const bc_float3 pix = f3_sub(rgb_of(pixels[i]), center);
            cov_rg += pix.x * pix.y;
            cov_rb += pix.x * pix.z;
            cov_gb += pix.y * pix.z;
        }
    bc_orient(&minColor, &maxColor, cov_rg, cov_rb, cov_gb);
    const bc_float3 extent = f3_sub(maxColor, minColor);
    const bc_float3 inset = f3(extent.x / count, extent.y / count, extent.z / count);
    maxColor = f3_saturate(f3_sub(maxColor, inset));
    minColor = f3_saturate(f3_add(minColor, inset));

    float alpha2 = 0, beta2 = 0, alphabeta = 0;
    bc_float3 alphax = f3(0, 0, 0), betax = f3(0, 0, 0);
    for (int i = 0; i < 16; ++i)
    {
        float pixelError;
        const uint32_t index = bc1_compute_index3(pixels[i], maxColor, minColor, threshold, &pixelError);
        if (index != 3)
        {
            float beta = (float)(index & 1);
            if (index & 2)
                beta = 0.5f;
            const float alpha = 1.0f - beta;
            alpha2 += alpha * alpha;
            beta2 += beta * beta;
            alphabeta += alpha * beta;
            alphax = f3_add(alphax, f3_mul(rgb_of(pixels[i]), alpha));
            betax = f3_add(betax, f3_mul(rgb_of(pixels[i]), beta));
        }
    }
    const float denom = alpha2 * beta2 - alphabeta * alphabeta;
    if (fabsf(denom) > 0.0001f)
    {
        const float factor = 1.0f / denom;
        const bc_float3 a = f3_mul(f3_sub(f3_mul(alphax, beta2), f3_mul(betax, alphabeta)), factor);
        const bc_float3 b = f3_mul(f3_sub(f3_mul(betax, alpha2), f3_mul(alphax, alphabeta)), factor);
        minColor = f3(keep_extreme(minColor.x, a.x), keep_extreme(minColor.y, a.y), keep_extreme(minColor.z, a.z));
        maxColor = f3(keep_extreme(maxColor.x, b.x), keep_extreme(maxColor.y, b.y), keep_extreme(maxColor.z, b.z));
    }
    uint32_t color0, color1;
    maxColor = round_and_expand565(maxColor, &color0);
    minColor = round_and_expand565(minColor, &color1);
    if (color0 > color1)
    {
        const bc_float3 t = maxColor;
        maxColor = minColor;
        minColor = t;
        const uint32_t c = color0;
        color0 = color1;
        color1 = c;
    }
    uint32_t indices = 0;
    *blockError = 0;
    for (int i = 0; i < 16; ++i)
    {
        float pixelError;
        const uint32_t index = bc1_compute_index3(pixels[i], maxColor, minColor, threshold, &pixelError);
        indices |= index << (2 * i);
        if (index != 3 || !(pixels[i].w <= threshold))
            *blockError += pixelError;
    }
    bc_uint2 result = {(color1 << 16) | color0, indices};
    return result;
}

static bc_uint2 bc2_encode_alpha(const float alphas[16]) /* :495-508 */
{
    bc_uint2 block = {0, 0};
    for (int i = 0; i < 16; ++i)
    {
        const uint32_t value = (uint32_t)rintf(bc_saturate(alphas[i]) * 15.0f);
        if (i < 8)
            block.x |= value << (i * 4);
        else
            block.y |= value << ((i - 8) * 4);
    }
    return block;
}

/* CompressBC1.hlsl / CompressBC2.hlsl / CompressBC3.hlsl main().  `format` 1, 2 or 3; `numChannels`
   (1..4) consecutive channels from `firstChannel` are red, green, blue, alpha (missing: 0, alpha 1);
   texels outside the image read as 0 in all four.  8 (BC1) or 16 bytes per block, row-major. */
int ntco_block_compress_color(const uint16_t* texels, int width, int height, int channels, int firstChannel, int numChannels,
    int format, float alphaThreshold, int srcLeft, int srcTop, int widthInBlocks, int heightInBlocks, uint8_t* blocks)
{
    if (!texels || !blocks || format < 1 || format > 3 || numChannels < 1 || numChannels > 4 || firstChannel < 0
        || firstChannel + numChannels > channels || widthInBlocks <= 0 || heightInBlocks <= 0)
        return -1;
    bc_ensure_tables();
    const size_t blockBytes = format == 1 ? 8 : 16;
    for (int by = 0; by < heightInBlocks; ++by)
        for (int bx = 0; bx < widthInBlocks; ++bx)
        {
            bc_float4 colors[16];
            float alphas[16];
            for (int i = 0; i < 16; ++i)
            {
                const int x = srcLeft + bx * 4 + (i & 3), y = srcTop + by * 4 + (i >> 2);
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                if (x < width && y < height)
                {
                    c[3] = 1.f;
                    for (int k = 0; k < numChannels; ++k)
                        c[k] = h2f(texels[((size_t)y * width + x) * channels + firstChannel + k]);
                }
                colors[i].x = c[0];
                colors[i].y = c[1];
                colors[i].z = c[2];
                colors[i].w = format == 1 ? c[3] : 1.0f;
                alphas[i] = c[3];
            }
            float bestError, error;
            bc_uint2 best, candidate;
            if (format == 1)
            {
                bestError = 0; /* BC1a_TransparentBlock, :99-109 */
                for (int i = 0; i < 16; ++i)
                    if (!(colors[i].w <= alphaThreshold))
                        bestError += f4_dot(colors[i]);
                best.x = 0;
                best.y = 0xffffffffu;
                candidate = bc1_encode_single_color(colors, &error);
                if (error < bestError) { bestError = error; best = candidate; }
            }
            else
                best = bc1_encode_single_color(colors, &bestError);
            candidate = bc1_compress_fast(colors, &error);
            if (error < bestError) { bestError = error; best = candidate; }
            uint8_t* dst = blocks + ((size_t)by * widthInBlocks + bx) * blockBytes;
            if (format == 1)
            {
                candidate = bc1a_compress_fast(colors, alphaThreshold, &error);
                if (error < bestError) { bestError = error; best = candidate; }
                memcpy(dst, &best.x, 4);
                memcpy(dst + 4, &best.y, 4);
            }
            else
            {
                const bc_uint2 alpha = format == 2 ? bc2_encode_alpha(alphas) : bc4_compress_fast(alphas);
                memcpy(dst, &alpha.x, 4);
                memcpy(dst + 4, &alpha.y, 4);
                memcpy(dst + 8, &best.x, 4);
                memcpy(dst + 12, &best.y, 4);
            }
        }
    return 0;
}
