// Diagnostic: how fast can the CTAs of a thread-block cluster store into one another's shared memory?
//
// The Monarch forward hands the row step's results (two 256-byte rows per (query group, cached group,
// column, block row)) to the column step.  One candidate design keeps that hand-off on chip by splitting a
// (head, query group) over the CTAs of a cluster and writing each row into the shared memory of the CTA that
// owns its column.  This probe measures the ceiling of that traffic pattern on the device at hand: every CTA
// of every cluster streams 256-byte rows into its peers' shared memory with plain stores through
// cluster-mapped addresses (ordinary st instructions only), in the epilogue's access pattern (one row per lane, 32
// bytes per store) and fully coalesced (consecutive lanes, 16 bytes each).
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int kBufBytes = 96 * 1024;      // receive buffer per CTA: 256 rows of 256 bytes and slack
constexpr int kThreads = 256;

template <int PATTERN>
__global__ void __launch_bounds__(kThreads, 1) dsmem_store_kernel(int iters, int remote) {
    extern __shared__ __align__(128) unsigned char buf[];
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), csize = cluster.num_blocks();
    const int tid = threadIdx.x;
    cluster.sync();
    uint4 v = make_uint4(tid, rank, 3u, 4u);
    for (int it = 0; it < iters; ++it) {
        const unsigned dst = remote ? (rank + 1 + (it % (csize > 1 ? csize - 1 : 1))) % csize : rank;
        unsigned char* base = static_cast<unsigned char*>(cluster.map_shared_rank(static_cast<void*>(buf), dst));
        if (PATTERN == 0) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {                       // lane = row, 8 pieces of 32 bytes (2 x 16-byte stores)
                uint4* p = reinterpret_cast<uint4*>(base + (size_t)tid * 256 + c * 32);
                asm volatile("st.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                asm volatile("st.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p + 1), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
            }
        } else {
#pragma unroll
            for (int c = 0; c < 16; ++c) {                      // consecutive lanes, consecutive 16 bytes
                uint4* p = reinterpret_cast<uint4*>(base + (size_t)(c * kThreads + tid) * 16);
                asm volatile("st.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
            }
        }
        v.x += it;
    }
    cluster.sync();                                             // nobody leaves while peers still write here
}

template <int PATTERN>
int run(int csize, int ctas, int iters, int remote, float* ms) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kBufBytes;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = csize; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaEvent_t a, b;
    cudaError_t e = cudaEventCreate(&a);
    if (e == cudaSuccess) e = cudaEventCreate(&b);
    if (e != cudaSuccess) return (int)e;
    e = cudaLaunchKernelEx(&cfg, dsmem_store_kernel<PATTERN>, 10, remote);     // warm-up
    if (e == cudaSuccess) e = cudaEventRecord(a);
    if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, dsmem_store_kernel<PATTERN>, iters, remote);
    if (e == cudaSuccess) e = cudaEventRecord(b);
    if (e == cudaSuccess) e = cudaEventSynchronize(b);
    if (e == cudaSuccess) e = cudaEventElapsedTime(ms, a, b);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    return (int)e;
}

}  // namespace

// One measurement: `cluster` CTAs per cluster (1, 2, 4, 8, or 16 with the non-portable opt-in), as many
// clusters as fit the device at one CTA per SM, `iters` passes of 64 KB per CTA.  pattern 0 = one row per
// lane in 32-byte pieces, 1 = coalesced 16-byte stores; remote 0 = each CTA writes its own shared memory
// (baseline), 1 = its peers'.  Returns the elapsed milliseconds, the CTAs launched and the bytes stored.
extern "C" int sfm_probe_dsmem_store(int cluster, int pattern, int remote, int iters, float* ms, int* ctas,
                                     double* bytes) {
    if (!ms || !ctas || !bytes) return SFM_ERR_NULL_POINTER;
    if (cluster < 1 || cluster > 16 || (cluster & (cluster - 1)) || iters < 1 || pattern < 0 || pattern > 1)
        return SFM_ERR_BAD_SHAPE;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    auto prep = [&](auto kernel) -> int {
        cudaError_t er = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBufBytes);
        if (er == cudaSuccess && cluster > 8)
            er = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (er != cudaSuccess) return (int)er;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(cluster);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kBufBytes;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = cluster; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int n = 0;
        er = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
        if (er != cudaSuccess) return (int)er;
        int c = n * cluster;
        if (c > sms) c = (sms / cluster) * cluster;             // one CTA per SM
        *ctas = c;
        return c > 0 ? 0 : SFM_ERR_UNSUPPORTED;
    };
    int rc = pattern == 0 ? prep(dsmem_store_kernel<0>) : prep(dsmem_store_kernel<1>);
    if (rc) return rc;
    rc = pattern == 0 ? run<0>(cluster, *ctas, iters, remote, ms) : run<1>(cluster, *ctas, iters, remote, ms);
    *bytes = (double)*ctas * iters * 65536.0;
    return rc;
}
