// TEST INFRASTRUCTURE ONLY.
//
// Runs one of the reference's block-compression compute shaders (src/shaders/CompressBC1.hlsl ...
// CompressBC5.hlsl, CompressBC7.hlsl, with BlockCompressCommon.hlsli) on the CPU: the shader source,
// made acceptable to a C++ compiler by oracle/transform_hlsl.py and given HLSL's types by
// oracle/hlsl_shim.h, is compiled into this translation unit (one per format:
// -DNTC_BC_SHADER="CompressBC1.hlsl" -DNTC_BC_FORMAT=1; BC7 twice, as the shader itself is built twice:
// -DUSE_MODE_BUFFER=0 for the full search and =1 for the path that reads each block's mode and
// partition from a mode buffer), and the entry point is called once per 4x4 block as a dispatch would
// call it per thread.  No
// graphics API is involved; the result is the reference's own encoder arithmetic in binary32 without
// contraction (-ffp-contract=off).
#include "hlsl_shim.h"

#if NTC_BC_FORMAT == 1 || NTC_BC_FORMAT == 4
#define NTC_BC_WORDS 2
#else
#define NTC_BC_WORDS 4
#endif

namespace
{
#include NTC_BC_SHADER
}

#define NTC_BC_CONCAT2(a, b) a##b
#define NTC_BC_CONCAT(a, b) NTC_BC_CONCAT2(a, b)

// texels: width x height RGBA binary32 (what the shader's Texture2D<float4> holds); blocks: widthInBlocks x
// heightInBlocks blocks of 8 or 16 bytes, rows of blocks without padding.
static void Bind(const float* texels, int width, int height, int srcLeft, int srcTop, int widthInBlocks, int heightInBlocks,
    float alphaThreshold, uint32_t* blocks)
{
    g_Const = NtcBlockCompressConstants();
    g_Const.srcLeft = srcLeft;
    g_Const.srcTop = srcTop;
    g_Const.widthInBlocks = widthInBlocks;
    g_Const.heightInBlocks = heightInBlocks;
    g_Const.alphaThreshold = alphaThreshold;
    t_Input.data = reinterpret_cast<const float4*>(texels);
    t_Input.width = width;
    t_Input.height = height;
    u_Output.data = reinterpret_cast<OUTPUT_FORMAT*>(blocks);
    u_Output.width = widthInBlocks;
    u_Output.height = heightInBlocks;
}

#if NTC_BC_FORMAT != 7
extern "C" int NTC_BC_CONCAT(ntcref_block_compress_bc, NTC_BC_FORMAT)(const float* texels, int width, int height, int srcLeft,
    int srcTop, int widthInBlocks, int heightInBlocks, float alphaThreshold, uint32_t* blocks)
{
    Bind(texels, width, height, srcLeft, srcTop, widthInBlocks, heightInBlocks, alphaThreshold, blocks);
    for (int by = 0; by < heightInBlocks; ++by)
        for (int bx = 0; bx < widthInBlocks; ++bx)
            shader_main(uint2(uint(bx), uint(by)));
    return 0;
}
#elif !USE_MODE_BUFFER
extern "C" int ntcref_block_compress_bc7(const float* texels, int width, int height, int srcLeft, int srcTop, int widthInBlocks,
    int heightInBlocks, float alphaThreshold, uint32_t* blocks)
{
    Bind(texels, width, height, srcLeft, srcTop, widthInBlocks, heightInBlocks, alphaThreshold, blocks);
    for (int by = 0; by < heightInBlocks; ++by)
        for (int bx = 0; bx < widthInBlocks; ++bx)
            shader_main(uint2(0u, 0u), uint2(uint(bx), uint(by)));
    return 0;
}
#else
// modeBuffer: the words of the buffer the shader binds as t_Modes (modeBufferWords of them).
extern "C" int ntcref_block_compress_bc7_modes(const float* texels, int width, int height, int srcLeft, int srcTop,
    int widthInBlocks, int heightInBlocks, const uint32_t* modeBuffer, uint32_t modeBufferByteOffset,
    uint32_t modeMapWidthInBlocks, uint32_t modeMapHeightInBlocks, int modeMapOffsetX, int modeMapOffsetY, uint32_t* blocks)
{
    Bind(texels, width, height, srcLeft, srcTop, widthInBlocks, heightInBlocks, 0.f, blocks);
    g_Const.modeBufferByteOffset = modeBufferByteOffset;
    g_Const.modeMapWidthInBlocks = modeMapWidthInBlocks;
    g_Const.modeMapHeightInBlocks = modeMapHeightInBlocks;
    g_Const.modeMapOffsetX = modeMapOffsetX;
    g_Const.modeMapOffsetY = modeMapOffsetY;
    t_Modes.data = modeBuffer;
    for (int by = 0; by < heightInBlocks; ++by)
        for (int bx = 0; bx < widthInBlocks; ++bx)
        {
            // this thread is alone in its group: nothing else has counted itself in
            s_ActiveThreadCount = 0;
            for (int m = 0; m < BC7_MODES; ++m)
                s_ModeCounts[m] = 0;
            shader_main(uint2(0u, 0u), uint2(uint(bx), uint(by)));
        }
    return 0;
}
#endif
