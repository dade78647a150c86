// Monarch row step on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// One CTA owns (batch*head, block row k, a range of cached groups f, one tile of stacked query
// groups).  A tile stacks up to 128 query rows r = (query group a, column j); each group is padded to
// a multiple of 8 rows so that its 128-byte-swizzled shared-memory image starts on a swizzle atom.
// For every f the CTA computes, per query row, a complete softmax over the b2 keys of K[f,k,:]:
//   S  = Q_tile K[f,k]^T                 tcgen05.mma, both operands from shared memory (K-major)
//   P  = softmax rows of S (scaled)      one thread per row: tcgen05.ld, registers, tcgen05.st (bf16)
//   aL = P K[f,k],  Y = P V[f,k]         tcgen05.mma, A = P from TMEM, B = the same K / V tile (MN-major)
//   cL = sum_l P ln P                    from the softmax registers
// and streams aL, Y (bf16) to the chunk's bridge with TMA stores; cL goes out with plain stores.
//
// Warp roles (10 warps): 0 = TMA producer, 1 = MMA issuer (owns the TMEM allocation),
// 2..5 = softmax warpgroup, 6..9 = epilogue warpgroup.  S/P is double buffered in TMEM so the
// S GEMM of step i+1 overlaps the softmax of step i; the two output accumulators are single
// buffered.  Every wait is bounded; on a timeout the CTA records a status code and unwinds.
//
// Arithmetic follows monarch_attn_ref_op (wan/modules/monarch_attn.py:1813-1823, 1828); the sqrt(s)
// scaling of q and k is folded into the softmax scale, so aL here is the reference's aL / sqrt(s).
#include "monarch_params.cuh"
#include "profile.cuh"
#include "tc05.cuh"

namespace sfm {

using namespace tc;

namespace {

constexpr int kStages = 3;            // K/V tile ring
constexpr int kThreads = 320;
constexpr int kTileRows = 128;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColS1 = 64, kColOK = 128, kColOV = 256;

struct RTcParams {
    MonarchParams mp;
    int rows_per_group;    // b2 padded to a multiple of 8
    int groups_per_tile;   // 128 / rows_per_group
    int n_s;               // b2 padded to a multiple of 16: key rows per K/V tile and N of the S GEMM
    int* status;           // device status word (0 = ok)
};

struct __align__(8) Barriers {
    uint64_t q_full;
    uint64_t kv_full[kStages];
    uint64_t kv_empty[kStages];
    uint64_t s_full[2];
    uint64_t p_full[2];
    uint64_t o_full;
    uint64_t o_free;
    uint32_t tmem_base;
    volatile int abort_flag;
};

// shared memory carve-up (bytes from a 1024-aligned base)
constexpr int kQBytes = 2 * kTileRows * 128;               // two 64-column halves
constexpr int kKVTileBytes = 2 * 64 * 128;                 // one K or V tile (up to 64 rows), two halves
constexpr int kStageBytes = 2 * kKVTileBytes;              // K + V
constexpr int kStagingBytes = 2 * kQBytes;                 // aL and Y, bf16, TMA-store source
constexpr int kSmemBytes = 1024 + kQBytes + kStages * kStageBytes + kStagingBytes + 256;

__device__ __forceinline__ void named_bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
monarch_r_tc_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                    const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tal,
                    const __grid_constant__ CUtensorMap ty, RTcParams rp) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;
    unsigned char* kv_s = q_s + kQBytes;
    unsigned char* stg_s = kv_s + kStages * kStageBytes;
    Barriers* bars = reinterpret_cast<Barriers*>(stg_s + kStagingBytes);

    const MonarchParams& p = rp.mp;
    const Blocking& blk = p.blk;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b1 = blk.b1, b2 = blk.b2;
    const int k = blockIdx.x % b1, fs = blockIdx.x / b1;
    const int g_first = blockIdx.y * rp.groups_per_tile;                 // chunk-local first group of the tile
    const int ng = min(rp.groups_per_tile, p.na - g_first);
    const int bhl = blockIdx.z, bh = p.bh0 + bhl, b = bh / p.H, hd = bh - b * p.H;
    const int f_begin = fs * p.f_per, f_end = min(p.F, f_begin + p.f_per);
    const int n_it = f_end - f_begin;
    const int RG = rp.rows_per_group;
    const int n_s = rp.n_s;
    const int valid_rows = ng * RG;                                       // rows of the tile that carry groups

    if (tid == 0) {
        mbar_init(&bars->q_full, 1);
        for (int s = 0; s < kStages; ++s) { mbar_init(&bars->kv_full[s], 1); mbar_init(&bars->kv_empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&bars->s_full[s], 1); mbar_init(&bars->p_full[s], 128); }
        mbar_init(&bars->o_full, 1);
        mbar_init(&bars->o_free, 128);
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) { tmem_alloc(&bars->tmem_base, kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    if (n_it <= 0) {   // uniform for the CTA
        __syncthreads();
        if (warp == 1) tmem_dealloc(tmem, kTmemCols);
        return;
    }

    auto fail = [&](int code) {
        bars->abort_flag = 1;
        atomicCAS(rp.status, 0, code);
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tmap(&tq); prefetch_tmap(&tk); prefetch_tmap(&tv);
            mbar_arrive_expect_tx(&bars->q_full, (uint32_t)(ng * RG * 256));
            for (int g = 0; g < ng; ++g) {
                int tok = blk.row_token(p.a0 + g_first + g, k);
                tma_load_4d(q_s + g * RG * 128, &tq, &bars->q_full, 0, hd, tok, b);
                tma_load_4d(q_s + kTileRows * 128 + g * RG * 128, &tq, &bars->q_full, 64, hd, tok, b);
            }
            for (int i = 0; i < n_it && !bars->abort_flag; ++i) {
                const int s = i % kStages;
                if (i >= kStages && !mbar_wait(&bars->kv_empty[s], ((i / kStages) - 1) & 1)) { fail(11); break; }
                const int tok = ((f_begin + i) * b1 + k) * b2;
                unsigned char* ks = kv_s + s * kStageBytes;
                unsigned char* vs = ks + kKVTileBytes;
                mbar_arrive_expect_tx(&bars->kv_full[s], (uint32_t)(4 * n_s * 128));
                tma_load_4d(ks, &tk, &bars->kv_full[s], 0, hd, tok, b);
                tma_load_4d(ks + n_s * 128, &tk, &bars->kv_full[s], 64, hd, tok, b);
                tma_load_4d(vs, &tv, &bars->kv_full[s], 0, hd, tok, b);
                tma_load_4d(vs + n_s * 128, &tv, &bars->kv_full[s], 64, hd, tok, b);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc_s = idesc_bf16(kTileRows, n_s, 0, 0);
            const uint32_t idesc_o = idesc_bf16(kTileRows, kHeadDim, 0, 1);
            const uint32_t q_addr = smem_addr(q_s);
            const int ksteps_pv = n_s / 16;
            auto issue_s = [&](int i) -> bool {
                const int s = i % kStages;
                if (!mbar_wait(&bars->kv_full[s], (i / kStages) & 1)) { fail(21); return false; }
                tc_fence_after();
                const uint32_t k_addr = smem_addr(kv_s + s * kStageBytes);
                const uint32_t d = tmem + ((i & 1) ? kColS1 : kColS0);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    uint32_t qa = q_addr + (ks >> 2) * (kTileRows * 128) + (ks & 3) * 32;
                    uint32_t ka = k_addr + (ks >> 2) * (n_s * 128) + (ks & 3) * 32;
                    mma_ss(d, smem_desc_sw128(qa, 16, 1024), smem_desc_sw128(ka, 16, 1024), idesc_s, ks > 0);
                }
                mma_commit(&bars->s_full[i & 1]);
                return true;
            };
            bool ok = mbar_wait(&bars->q_full, 0);
            if (!ok) fail(20);
            ok = ok && issue_s(0);
            for (int i = 0; ok && i < n_it && !bars->abort_flag; ++i) {
                if (i + 1 < n_it && !issue_s(i + 1)) break;
                if (!mbar_wait(&bars->p_full[i & 1], (i >> 1) & 1)) { fail(22); break; }
                if (i > 0 && !mbar_wait(&bars->o_free, (i - 1) & 1)) { fail(23); break; }
                tc_fence_after();
                const int s = i % kStages;
                const uint32_t k_addr = smem_addr(kv_s + s * kStageBytes);
                const uint32_t v_addr = k_addr + kKVTileBytes;
                const uint32_t p_t = tmem + ((i & 1) ? kColS1 : kColS0);
                for (int kk = 0; kk < ksteps_pv; ++kk) {
                    mma_ts(tmem + kColOK, p_t + kk * 8, smem_desc_sw128(k_addr + kk * 2048, n_s * 128, 1024), idesc_o, kk > 0);
                    mma_ts(tmem + kColOV, p_t + kk * 8, smem_desc_sw128(v_addr + kk * 2048, n_s * 128, 1024), idesc_o, kk > 0);
                }
                mma_commit(&bars->o_full);
                mma_commit(&bars->kv_empty[s]);
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ softmax warpgroup
        const int quad = warp & 3;                      // TMEM lane quadrant this warp may access
        const int row = quad * 32 + lane;               // tile row == TMEM lane
        const bool warp_active = quad * 32 < valid_rows;
        const int g = row / RG, j = row - g * RG;
        const bool row_ok = g < ng && j < b2;
        const long long aj = ((long long)bhl * p.na + g_first + g) * b2 + j;
        const float scale_l2 = p.mult0 * kLog2e;
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        for (int i = 0; i < n_it && !bars->abort_flag; ++i) {
            if (!mbar_wait(&bars->s_full[i & 1], (i >> 1) & 1)) { fail(31); break; }
            tc_fence_after();
            if (warp_active) {
                const uint32_t s_t = tmem + lane_sel + ((i & 1) ? kColS1 : kColS0);
                uint32_t raw[64];
                if (n_s > 32) {
                    tmem_ld32(s_t, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
                    tmem_ld32(s_t + 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[32]));
                } else if (n_s > 16) {
                    tmem_ld32(s_t, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
                } else {
                    tmem_ld16(s_t, *reinterpret_cast<uint32_t(*)[16]>(&raw[0]));
                }
                tmem_wait_ld();
                float mx = -INFINITY;
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    float x = (c < b2) ? __uint_as_float(raw[c]) * scale_l2 : -INFINITY;
                    raw[c] = __float_as_uint(x);
                    mx = fmaxf(mx, x);
                }
                float z = 0.f, ent = 0.f;
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    float d = __uint_as_float(raw[c]) - mx;
                    float e = exp2f(d);
                    z += e;
                    ent += (c < b2) ? e * d : 0.f;
                    raw[c] = __float_as_uint(e);
                }
                const float inv_z = 1.0f / z;
                uint32_t pk[32];
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    pk[c] = pack_bf16(__uint_as_float(raw[2 * c]) * inv_z, __uint_as_float(raw[2 * c + 1]) * inv_z);
                if (n_s > 32) {
                    tmem_st32(s_t, pk);
                } else if (n_s > 16) {
                    tmem_st16(s_t, *reinterpret_cast<uint32_t(*)[16]>(&pk[0]));
                } else {
                    uint32_t p8[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) p8[c] = c < 8 ? pk[c] : 0u;
                    tmem_st16(s_t, p8);   // 8 packed columns are used; the other 8 belong to no operand
                }
                tmem_wait_st();
                if (row_ok) {
                    const int key = (f_begin + i) * b1 + k;
                    p.cL[aj * p.n_keys + key] = 0.6931471805599453f * ent * inv_z - __logf(z);
                }
            }
            tc_fence_before();
            mbar_arrive(&bars->p_full[i & 1]);
        }
    } else {
        // ------------------------------------------------------------------ epilogue warpgroup
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const bool warp_active = quad * 32 < valid_rows;
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const bool issuer = (warp == 6 && lane == 0);
        for (int i = 0; i < n_it && !bars->abort_flag; ++i) {
            if (!mbar_wait(&bars->o_full, i & 1)) { fail(41); break; }
            tc_fence_after();
            if (i > 0) {                                  // staging buffer free again?
                if (issuer) tma_store_wait_read<0>();
                named_bar_sync(1, 128);
            }
            if (warp_active) {
#pragma unroll 1
                for (int which = 0; which < 2; ++which) {
                    const uint32_t o_t = tmem + lane_sel + (which ? kColOV : kColOK);
                    unsigned char* dst = stg_s + which * kQBytes + row * 128;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t r[32];
                        tmem_ld32(o_t + c * 32, r);
                        tmem_wait_ld();
                        unsigned char* half = dst + (c >> 1) * (kTileRows * 128);
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {
                            uint4 v;
                            v.x = pack_bf16(__uint_as_float(r[ch * 8 + 0]), __uint_as_float(r[ch * 8 + 1]));
                            v.y = pack_bf16(__uint_as_float(r[ch * 8 + 2]), __uint_as_float(r[ch * 8 + 3]));
                            v.z = pack_bf16(__uint_as_float(r[ch * 8 + 4]), __uint_as_float(r[ch * 8 + 5]));
                            v.w = pack_bf16(__uint_as_float(r[ch * 8 + 6]), __uint_as_float(r[ch * 8 + 7]));
                            const int chunk = (c & 1) * 4 + ch;
                            *reinterpret_cast<uint4*>(half + ((chunk ^ (row & 7)) << 4)) = v;
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&bars->o_free);
            fence_async_smem();
            named_bar_sync(1, 128);
            if (issuer) {
                const int key = (f_begin + i) * b1 + k;
                for (int g = 0; g < ng; ++g) {
                    const int aj0 = (bhl * p.na + g_first + g) * b2;
                    const unsigned char* src = stg_s + g * RG * 128;
                    tma_store_3d(&tal, src, 0, key, aj0);
                    tma_store_3d(&tal, src + kTileRows * 128, 64, key, aj0);
                    tma_store_3d(&ty, src + kQBytes, 0, key, aj0);
                    tma_store_3d(&ty, src + kQBytes + kTileRows * 128, 64, key, aj0);
                }
                tma_store_commit();
            }
        }
        if (issuer) tma_store_wait_all<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

// Launches the tensor-core row step for one chunk.  `status` is a device int the kernel sets on an
// internal timeout.
int launch_r_step_tc(const MonarchParams& p, const CUtensorMap* maps /* q,k,v,aL,Y */, int rows_per_group, int n_s,
                     int* status, cudaStream_t s) {
    LaunchScope scope(kClsRStep, s);
    RTcParams rp;
    rp.mp = p;
    rp.rows_per_group = rows_per_group;
    rp.groups_per_tile = kTileRows / rows_per_group;
    rp.n_s = n_s;
    rp.status = status;
    int tiles = (p.na + rp.groups_per_tile - 1) / rp.groups_per_tile;
    dim3 grid(p.blk.b1 * p.fsplit, tiles, p.nbh);
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(monarch_r_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    monarch_r_tc_kernel<<<grid, kThreads, kSmemBytes, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4], rp);
    return (int)cudaGetLastError();
}

}  // namespace sfm
