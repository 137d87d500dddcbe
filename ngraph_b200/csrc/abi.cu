// Library-wide pieces of the C ABI: status text, CUDA error capture, launch counter.
#include "common.cuh"
#include <cstdio>

namespace b200
{
    std::atomic<uint64_t> g_launches{0};
    static thread_local char g_err[256] = "no error";

    int cuda_status(cudaError_t err, const char* where)
    {
        if (err == cudaSuccess)
            return B200_OK;
        snprintf(g_err, sizeof(g_err), "%s: %s (%s)", where, cudaGetErrorString(err), cudaGetErrorName(err));
        return B200_ERR_CUDA;
    }
    void set_error_text(const char* text) { snprintf(g_err, sizeof(g_err), "%s", text); }
}

extern "C" const char* b200_status_string(int status)
{
    switch (status)
    {
    case B200_OK: return "ok";
    case B200_ERR_INVALID_ARGUMENT: return "invalid argument";
    case B200_ERR_UNSUPPORTED: return "unsupported on device";
    case B200_ERR_TOO_LARGE: return "size limit exceeded";
    case B200_ERR_DEVICE_STATUS: return "device kernel reported a bounded-wait timeout";
    case B200_ERR_CUDA: return "CUDA error (see b200_last_cuda_error)";
    default: return "unknown status";
    }
}
extern "C" const char* b200_last_cuda_error(void) { return b200::g_err; }
extern "C" uint64_t b200_launch_count(void) { return b200::g_launches.load(); }
extern "C" void b200_reset_launch_count(void) { b200::g_launches.store(0); }
