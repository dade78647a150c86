// Launch accounting and optional per-kernel timing (CUDA events on the launching stream).
#pragma once
#include <cuda_runtime.h>

namespace sfm {

enum KernelClass { kClsLayout = 0, kClsRStep = 1, kClsLStep = 2, kClsLIter = 3, kClsDense = 4, kClsBackward = 5, kNumClasses = 6 };

// Counts one launch of `cls`; when profiling is enabled also brackets the launch with events.
struct LaunchScope {
    LaunchScope(int cls, cudaStream_t stream);
    ~LaunchScope();
    int cls_;
    cudaStream_t stream_;
    int slot_;
};

}  // namespace sfm
