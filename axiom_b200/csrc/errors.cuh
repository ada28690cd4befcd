// errors.cuh — lets the kernel translation units leave a message where
// axb_last_error() will find it.
#pragma once
#include <cuda_runtime.h>

namespace axb {

// printf-style; returns `status` so call sites can `return set_error(...)`.
int set_error(int status, const char *fmt, ...);

// the stream and the device of the engine the calling thread drives (-1: none selected yet)
cudaStream_t engine_stream();
int engine_device();

// Function attributes (the dynamic shared-memory opt-in) belong to a device's context: a launcher keeps one of
// these per kernel instantiation and sets the attribute the first time it runs on each device.
struct PerDeviceOnce {
    bool done[64] = {};
    bool first()
    {
        int d = 0;
        if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return true;
        if (done[d]) return false;
        done[d] = true;
        return true;
    }
    int device() const
    {
        int d = 0;
        return (cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < 64) ? d : 0;
    }
};

}  // namespace axb
