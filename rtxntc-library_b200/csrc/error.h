// Error reporting shared by the translation units of the library: a thread-local message read
// through ntcb_last_error(), the reference's convention (src/Errors.cpp:21-52).
#pragma once

#include <cuda_runtime.h>

namespace ntcb
{

void SetError(const char* format, ...);
void ClearError();
// Records "Call to <call> failed, error code = <name>." and returns NTCB_ERR_CUDA.
int CudaFailure(const char* call, cudaError_t error);
// Bookkeeping behind ntcb_launch_count().
void CountLaunch();

} // namespace ntcb
