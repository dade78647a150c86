// Dense softmax attention without a mask over the whole key range: the dense-init chunk and the
// "regular" configuration.  Runs on the tensor-core flash kernel of monarch_lstep_tc.cu (dense
// instantiation): one unit = 128 consecutive queries of one (batch, head), keys and values stream
// from the cache view in 128-token tiles by TMA.
//
// Stands in for flash_attention / attention (wan/modules/attention.py:34-187).
#include "common.cuh"
#include "profile.cuh"
#include "tc05.cuh"

namespace sfm {
int launch_dense_tc(const CUtensorMap* maps, __nv_bfloat16* out, int B, int H, int n_q, int n_kv, float scale, int* status,
                    int num_sms, cudaStream_t s);
namespace {
// Set (once, by compare-and-swap from 0) by the kernel when one of its bounded waits gives up; 0 = ok.
// One word per device, shared by every stream, never cleared by a launch: it keeps the first failure since
// the last sfm_dense_status call, which reads and clears it.
__device__ int g_dense_status;
}  // namespace
}  // namespace sfm

using namespace sfm;

extern "C" int sfm_dense_fwd(const void* q, int64_t q_batch_stride, const void* k, const void* v,
                             int64_t kv_batch_stride, void* out, int B, int H, int D, int n_q, int n_kv,
                             float sm_scale, void* stream) {
    if (!q || !k || !v || !out) return SFM_ERR_NULL_POINTER;
    if (D != kHeadDim) return SFM_ERR_UNSUPPORTED;
    if (B <= 0 || H <= 0 || n_q <= 0 || n_kv <= 0) return SFM_ERR_BAD_SHAPE;
    if (!(sm_scale > 0.f)) return SFM_ERR_BAD_SHAPE;       // the row maximum is taken before scaling
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
    if (mis(q) || mis(k) || mis(v) || mis(out) || (q_batch_stride % 8) || (kv_batch_stride % 8)) return SFM_ERR_ALIGNMENT;

    int dev = 0, num_sms = 148;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    int* status = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_dense_status);
    if (e != cudaSuccess) return (int)e;

    const uint64_t row = (uint64_t)kHeadDim * 2, tok = (uint64_t)H * row;
    uint64_t dq[4] = {(uint64_t)kHeadDim, (uint64_t)H, (uint64_t)n_q, (uint64_t)B};
    uint64_t sq[3] = {row, tok, (uint64_t)q_batch_stride * 2};
    uint64_t dk[4] = {(uint64_t)kHeadDim, (uint64_t)H, (uint64_t)n_kv, (uint64_t)B};
    uint64_t sk[3] = {row, tok, (uint64_t)kv_batch_stride * 2};
    uint32_t box[4] = {64, 1, 128, 1};
    CUtensorMap maps[3];
    int rc;
    if ((rc = make_tmap_bf16(&maps[0], k, 4, dk, sk, box))) return rc;
    if ((rc = make_tmap_bf16(&maps[1], v, 4, dk, sk, box))) return rc;
    if ((rc = make_tmap_bf16(&maps[2], q, 4, dq, sq, box))) return rc;
    return launch_dense_tc(maps, (__nv_bfloat16*)out, B, H, n_q, n_kv, sm_scale, status, num_sms, (cudaStream_t)stream);
}

// Waits for `stream`, then reports (and clears) the status word of the dense-attention kernels on the
// current device: SFM_OK, or SFM_ERR_DEVICE_STATUS if a launch since the last call gave up on a bounded wait.
extern "C" int sfm_dense_status(void* stream) {
    int* status = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_dense_status);
    int st = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&st, status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e == cudaSuccess && st != 0) e = cudaMemsetAsync(status, 0, sizeof(int), (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    return st == 0 ? SFM_OK : SFM_ERR_DEVICE_STATUS;
}
