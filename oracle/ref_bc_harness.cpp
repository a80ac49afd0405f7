// TEST INFRASTRUCTURE ONLY.
//
// Runs one of the reference's block-compression compute shaders (src/shaders/CompressBC1.hlsl ...
// CompressBC5.hlsl with BlockCompressCommon.hlsli) on the CPU: the shader source, made acceptable to a
// C++ compiler by oracle/transform_hlsl.py and given HLSL's types by oracle/hlsl_shim.h, is compiled
// into this translation unit (one per format: -DNTC_BC_SHADER="CompressBC1.hlsl" -DNTC_BC_FORMAT=1),
// and the entry point is called once per 4x4 block as a dispatch would call it per thread.  No
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
extern "C" int NTC_BC_CONCAT(ntcref_block_compress_bc, NTC_BC_FORMAT)(const float* texels, int width, int height, int srcLeft,
    int srcTop, int widthInBlocks, int heightInBlocks, float alphaThreshold, uint32_t* blocks)
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
    for (int by = 0; by < heightInBlocks; ++by)
        for (int bx = 0; bx < widthInBlocks; ++bx)
            shader_main(uint2(uint(bx), uint(by)));
    return 0;
}
