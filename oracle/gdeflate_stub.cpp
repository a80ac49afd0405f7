// TEST INFRASTRUCTURE ONLY (never linked into the product library).
//
// Stand-in for the reference's src/GDeflate.cpp when building the reference library as the
// parity checker.  The reference's GDeflate codec needs NVIDIA's libdeflate fork, which is an
// un-vendored git submodule (external/libdeflate is empty), so that one file cannot be compiled.
// The synthetic NTC containers used for parity store every buffer view uncompressed, so none of
// these functions is reached on the decode path; they only have to link.
//
// Signatures follow the declarations in the reference's src/GDeflate.h:21-33 and
// include/libntc/ntc.h:1389.

#include "GDeflate.h"

namespace ntc
{

// Reporting failure makes BinaryChunkBuilder store the view raw (src/BinaryChunkBuilder.cpp:69-92).
bool CompressGDeflate(void const*, size_t, Vector<uint8_t>&, ThreadPool*, IAllocator*, uint32_t*, int)
{
    return false;
}

Status DecompressGDeflate(void const*, size_t, void*, size_t, IAllocator*, uint32_t)
{
    return Status::Unsupported;
}

Status DecompressGDeflateOnVulkanGPU(GraphicsResources const*, void*, void const*, size_t, uint64_t, uint64_t)
{
    return Status::Unsupported;
}

extern "C" size_t GetGDeflateHeaderSize(size_t)
{
    return 0;
}

} // namespace ntc
