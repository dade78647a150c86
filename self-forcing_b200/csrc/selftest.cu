// Self-test of the failure path every kernel of this library shares: a bounded wait that runs out.
//
// One CTA allocates TMEM the way the attention kernels do, then one thread waits, with a short poll limit, on an
// mbarrier that nothing ever arrives at.  The wait gives up, the thread records a status code in the workspace's
// status word and raises the CTA's abort flag, all threads meet, the TMEM allocation is released and the kernel
// returns normally: the context stays usable and the host reads the failure through sfm_workspace_status.  Nothing
// faults, traps or spins without a bound.  The reference has no counterpart (its kernels have no device-side waits).
#include "monarch_params.cuh"
#include "tc05.cuh"

namespace sfm {
namespace {

using namespace tc;

struct SelfTestShared {
    uint64_t never;            // nobody arrives here
    uint32_t tmem_base;
    volatile int abort_flag;
};

__global__ void __launch_bounds__(64, 1) selftest_bounded_wait_kernel(int* status, uint32_t polls, int code) {
    __shared__ SelfTestShared sh;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(&sh.never, 1);
        sh.abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) { tmem_alloc(&sh.tmem_base, 32); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0 && !mbar_wait_limit(&sh.never, 0, polls)) {
        sh.abort_flag = 1;
        atomicCAS(status, 0, code);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(sh.tmem_base, 32);
}

}  // namespace
}  // namespace sfm

// Runs the self-test on `stream`: clears the status word at the start of `workspace`, then lets a wait of `polls`
// polls (1 .. 65536) run out, which leaves `code` (1 .. 255) there.  Returns SFM_OK when the launch went through;
// sfm_workspace_status(workspace, stream) must then report SFM_ERR_DEVICE_STATUS.
extern "C" int sfm_selftest_bounded_wait(void* workspace, int polls, int code, void* stream) {
    if (!workspace) return SFM_ERR_NULL_POINTER;
    if (polls < 1 || polls > 65536 || code < 1 || code > 255) return SFM_ERR_BAD_SHAPE;
    if (reinterpret_cast<uintptr_t>(workspace) & 15) return SFM_ERR_ALIGNMENT;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(workspace, 0, sizeof(int), s);
    if (e != cudaSuccess) return (int)e;
    sfm::selftest_bounded_wait_kernel<<<1, 64, 0, s>>>((int*)workspace, (uint32_t)polls, code);
    return (int)cudaGetLastError();
}
