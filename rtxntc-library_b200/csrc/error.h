// Error reporting shared by the translation units of the library: a thread-local message read
// through ntcb_last_error(), the reference's convention (src/Errors.cpp:21-52).
#pragma once

#include <cuda_runtime.h>

#include <exception>
#include <new>

#include "ntcb.h"

namespace ntcb
{

void SetError(const char* format, ...);
void ClearError();
// Records "Call to <call> failed, error code = <name>." and returns NTCB_ERR_CUDA.
int CudaFailure(const char* call, cudaError_t error);
// Runs the body of a C entry point and turns a C++ exception (the host containers' std::bad_alloc, a
// std::system_error from a thread) into a status and a message: nothing propagates through the C interface.
template <typename Body>
int Guarded(const char* entryPoint, Body&& body) noexcept
{
    try
    {
        return body();
    }
    catch (const std::bad_alloc&)
    {
        SetError("%s: out of host memory.", entryPoint);
        return NTCB_ERR_OUT_OF_MEMORY;
    }
    catch (const std::exception& e)
    {
        SetError("%s: %s", entryPoint, e.what());
        return NTCB_ERR_INVALID_STATE;
    }
    catch (...)
    {
        SetError("%s: an exception of unknown type.", entryPoint);
        return NTCB_ERR_INVALID_STATE;
    }
}

// Bookkeeping behind ntcb_launch_count().
void CountLaunch();

} // namespace ntcb
