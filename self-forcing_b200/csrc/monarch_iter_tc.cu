// Monarch iteration update on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Between two passes of the iterative variant the column side turns the row step's aL / cL into the next
// pass's query operand (monarch_attn_slow, wan/modules/monarch_attn.py:1726-1733):
//   L[i,(f,k)]  = exp(scale * q^[a,i,j] . aL[a,f,j,k] - cL[a,f,j,k] - lse[a,j,i])     (a normalised softmax over (f,k))
//   aR[a,f,k,j] = sum_i L[i,(f,k)] q^[a,i,j]            cR[a,f,k,j] = sum_i L[i,(f,k)]
// lse comes from the column step that ran just before (its softmax statistics).
//
// One unit = one (batch*head, query group a, column j); its keys (f,k) are walked in tiles of 128 with the KEYS on
// the M side of the tensor core, so that both products are plain GEMMs and every result row is one key:
//   S^T [128 keys x N_I]  = aL_tile [128 x 128] * Q_j^T                    tcgen05.mma, both operands in shared memory
//   P^T                   = exp(...) per element, bf16, written back over S^T in TMEM; cR = row sums (registers)
//   aR_tile [128 x 128]   = P^T * Q_j                                      tcgen05.mma, A from TMEM, B = Q_j MN-major
// N_I = block rows padded to 16.  Warp roles (12 warps): 0 = TMA producer, 1 = MMA issuer (owns TMEM), 2-3 idle,
// 4-7 and 8-11 = two warpgroups that take even / odd tiles: softmax-like pass, then drain of the accumulator and
// one 256-byte aR row per thread (32-byte stores).  Persistent CTAs take contiguous shares of the unit list; all
// roles walk the same (unit, tile) sequence and meet through mbarriers with bounded waits.
#include "monarch_params.cuh"
#include "profile.cuh"
#include "tc05.cuh"

namespace sfm {

using namespace tc;

namespace {

constexpr int kAStg = 3;                  // aL tile ring
constexpr int kThreadsIt = 384;
constexpr int kKTile = 128;               // keys per tile
constexpr uint32_t kTmemColsIt = 512;
__host__ __device__ constexpr uint32_t it_col_s(int w) { return (uint32_t)w * 128u; }
__host__ __device__ constexpr uint32_t it_col_o(int w) { return 256u + (uint32_t)w * 128u; }

struct ItParams {
    MonarchParams mp;
    int n_units;       // nbh * na * b2
    int R4;            // query rows per TMA box (ceil(b1 / 4))
    int q_rows_tma;    // query rows of a unit are consecutive rows of the token grid
    int* status;
};

struct __align__(16) ItBarriers {
    float lse2[2][128];                   // log2(e) * lse of the unit's queries, +inf past b1
    uint64_t q_full[2], q_empty[2];
    uint64_t a_full[kAStg], a_empty[kAStg];
    uint64_t s_full[2], p_full[2], sp_free[2];
    uint64_t o_full[2], o_free[2];
    uint32_t tmem_base;
    volatile int abort_flag;
};

constexpr int kItQBytes = 2 * 128 * 128;      // one query tile: two 64-column halves of 128 rows
constexpr int kItTileBytes = 2 * kKTile * 128;
constexpr int kItSmemBytes = 1024 + 2 * kItQBytes + kAStg * kItTileBytes + (int)sizeof(ItBarriers) + 64;

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void st_global_v8_it(void* ptr, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                 "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}

struct ItUnit { int bhl, al, j; };
__device__ __forceinline__ ItUnit it_decode(const MonarchParams& p, int u) {
    ItUnit r;
    r.j = u % p.blk.b2; u /= p.blk.b2;
    r.al = u % p.na;
    r.bhl = u / p.na;
    return r;
}

// tal = bridge aL map (box 64 x 128 keys x 1), tqr = query rows (5-D, box rows = R4).
template <int N_I>
__global__ void __launch_bounds__(kThreadsIt, 1)
monarch_iter_tc_kernel(const __grid_constant__ CUtensorMap tal, const __grid_constant__ CUtensorMap tqr, ItParams ip) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;                                   // two query tiles
    unsigned char* a_s = q_s + 2 * kItQBytes;
    ItBarriers* bars = reinterpret_cast<ItBarriers*>(a_s + kAStg * kItTileBytes);

    const MonarchParams& p = ip.mp;
    const Blocking& blk = p.blk;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b1 = blk.b1, b2 = blk.b2;
    const int n_keys = p.n_keys;
    const int n_tiles = (n_keys + kKTile - 1) / kKTile;
    const int R4 = ip.R4;
    const long long tok_pitch = (long long)p.H * kHeadDim;
    const int u_begin = (int)((long long)ip.n_units * blockIdx.x / gridDim.x);
    const int u_end = (int)((long long)ip.n_units * (blockIdx.x + 1) / gridDim.x);

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(&bars->q_full[s], 1); mbar_init(&bars->q_empty[s], 1); }
        for (int s = 0; s < kAStg; ++s) { mbar_init(&bars->a_full[s], 1); mbar_init(&bars->a_empty[s], 1); }
        for (int w = 0; w < 2; ++w) {
            mbar_init(&bars->s_full[w], 1); mbar_init(&bars->p_full[w], 128); mbar_init(&bars->sp_free[w], 1);
            mbar_init(&bars->o_full[w], 1); mbar_init(&bars->o_free[w], 128);
        }
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    // query rows that no load writes must hold finite numbers (their weights are zero)
    for (int i = tid; i < 2 * kItQBytes / 16; i += kThreadsIt) reinterpret_cast<uint4*>(q_s)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 1) { tmem_alloc(&bars->tmem_base, kTmemColsIt); tmem_relinquish(); }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    auto fail = [&](int code) {
        bars->abort_flag = 1;
        atomicCAS(ip.status, 0, code);
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) { prefetch_tmap(&tal); prefetch_tmap(&tqr); }
        int g = 0, uc = 0;
        bool ok = true;
        for (int u = u_begin; ok && u < u_end && !bars->abort_flag; ++u, ++uc) {
            const ItUnit un = it_decode(p, u);
            const int bh = p.bh0 + un.bhl, b = bh / p.H, hd = bh - b * p.H;
            const int qb = uc & 1;
            unsigned char* qd_s = q_s + qb * kItQBytes;
            if (uc >= 2) {
                int okw = 1;
                if (lane == 0) okw = mbar_wait(&bars->q_empty[qb], ((uc >> 1) - 1) & 1) ? 1 : 0;
                if (!__shfl_sync(0xffffffffu, okw, 0)) { fail(10); break; }
            }
            for (int i = lane; i < 128; i += 32)
                bars->lse2[qb][i] = i < b1 ? kLog2e * p.lse[(long long)u * b1 + i] : INFINITY;
            if (ip.q_rows_tma) {
                __syncwarp();
                if (lane == 0) {
                    const int nq = (b1 + R4 - 1) / R4;
                    mbar_arrive_expect_tx(&bars->q_full[qb], (uint32_t)(nq * R4 * 256));
                    const int tok0 = blk.row_token(p.a0 + un.al, 0);
                    const int frow0 = tok0 / blk.w, col = tok0 - frow0 * blk.w + un.j;
                    for (int qd = 0; qd < nq; ++qd) {
                        unsigned char* dst = qd_s + (qd * R4) * 128;
                        tma_load_5d(dst, &tqr, &bars->q_full[qb], 0, hd, col, frow0 + qd * R4, b);
                        tma_load_5d(dst + 128 * 128, &tqr, &bars->q_full[qb], 64, hd, col, frow0 + qd * R4, b);
                    }
                }
            } else {
                const __nv_bfloat16* qg = p.q + (long long)b * p.q_bs + (long long)hd * kHeadDim;
                for (int idx = lane; idx < b1 * 16; idx += 32) {
                    const int i = idx >> 4, ch = idx & 15;
                    const uint4 val = *reinterpret_cast<const uint4*>(
                        qg + (blk.row_token(p.a0 + un.al, i) + un.j) * tok_pitch + ch * 8);
                    *reinterpret_cast<uint4*>(qd_s + (ch >> 3) * (128 * 128) + i * 128 + (((ch & 7) ^ (i & 7)) << 4)) = val;
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->q_full[qb]);
            }
            if (lane == 0) {
                for (int t = 0; t < n_tiles; ++t, ++g) {
                    const int s = g % kAStg;
                    if (g >= kAStg && !mbar_wait(&bars->a_empty[s], ((g / kAStg) - 1) & 1)) { fail(11); ok = false; break; }
                    unsigned char* st = a_s + s * kItTileBytes;
                    mbar_arrive_expect_tx(&bars->a_full[s], (uint32_t)kItTileBytes);
                    tma_load_3d(st, &tal, &bars->a_full[s], 0, t * kKTile, u);
                    tma_load_3d(st + kKTile * 128, &tal, &bars->a_full[s], 64, t * kKTile, u);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            g = __shfl_sync(0xffffffffu, g, 0);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16(128, N_I, 0, 0);
            constexpr uint32_t idesc_o = idesc_bf16(128, kHeadDim, 0, 1);
            const uint64_t a_desc0 = smem_desc_sw128(smem_addr(a_s), 16, 1024);
            const uint64_t qk_desc0 = smem_desc_sw128(smem_addr(q_s), 16, 1024);             // K-major (S GEMM)
            const uint64_t qn_desc0 = smem_desc_sw128(smem_addr(q_s), 128 * 128, 1024);      // MN-major (aR GEMM)
            const int total = (u_end - u_begin) * n_tiles;
            bool ok = true;
            auto issue_s = [&](int g) -> bool {                  // S^T of tile g
                const int uc = g / n_tiles, t = g - uc * n_tiles, w = g & 1, s = g % kAStg, qb = uc & 1;
                if (t == 0 && !mbar_wait(&bars->q_full[qb], (uc >> 1) & 1)) { fail(20); return false; }
                if (!mbar_wait(&bars->a_full[s], (g / kAStg) & 1)) { fail(21); return false; }
                if (g >= 2 && !mbar_wait(&bars->sp_free[w], ((g >> 1) - 1) & 1)) { fail(22); return false; }
                tc_fence_after();
                const uint64_t ad = a_desc0 + (uint64_t)((s * kItTileBytes) >> 4);
                const uint64_t qd = qk_desc0 + (uint64_t)((qb * kItQBytes) >> 4);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = ((ks >> 2) * (128 * 128) + (ks & 3) * 32) >> 4;
                    mma_ss(tmem + it_col_s(w), ad + off, qd + off, idesc_s, ks > 0);
                }
                mma_commit(&bars->s_full[w]);
                mma_commit(&bars->a_empty[s]);
                return true;
            };
            if (total > 0) ok = issue_s(0);
            for (int g = 0; ok && g < total && !bars->abort_flag; ++g) {
                if (g + 1 < total && !issue_s(g + 1)) { ok = false; break; }
                const int uc = g / n_tiles, t = g - uc * n_tiles, w = g & 1, qb = uc & 1;
                if (!mbar_wait(&bars->p_full[w], (g >> 1) & 1)) { fail(23); break; }
                if (g >= 2 && !mbar_wait(&bars->o_free[w], ((g >> 1) - 1) & 1)) { fail(24); break; }
                tc_fence_after();
                const uint64_t qd = qn_desc0 + (uint64_t)((qb * kItQBytes) >> 4);
#pragma unroll
                for (int kk = 0; kk < N_I / 16; ++kk)
                    mma_ts(tmem + it_col_o(w), tmem + it_col_s(w) + kk * 8, qd + ((kk * 2048) >> 4), idesc_o, kk > 0);
                mma_commit(&bars->o_full[w]);
                mma_commit(&bars->sp_free[w]);
                if (t + 1 == n_tiles) mma_commit(&bars->q_empty[qb]);       // last read of this unit's query tile
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ the two working warpgroups
        const int w = (warp - 4) >> 2;
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                       // TMEM lane == key within the tile
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const uint32_t s_t = tmem + lane_sel + it_col_s(w);
        const uint32_t o_t = tmem + lane_sel + it_col_o(w);
        const float scale_l2 = p.scale * kLog2e;
        const int total = (u_end - u_begin) * n_tiles;
        bool ok = true;
        for (int g = w; ok && g < total && !bars->abort_flag; g += 2) {
            const int uc = g / n_tiles, t = g - uc * n_tiles, qb = uc & 1;
            const int u = u_begin + uc;
            const int key = t * kKTile + row;
            const bool valid = key < n_keys;
            // bias of this key in log2 units; a key past the end gets weight zero
            const float cl2 = valid ? kLog2e * p.cL[(long long)u * p.n_keys_c + key] : INFINITY;
            if (!mbar_wait(&bars->s_full[w], (g >> 1) & 1)) { fail(31); break; }
            tc_fence_after();
            const float* lse2 = bars->lse2[qb];
            float csum = 0.f;
#pragma unroll 1
            for (int c0 = 0; c0 < N_I; c0 += 16) {
                uint32_t r[16], pk[8];
                tmem_ld16(s_t + c0, r);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 16; c += 2) {
                    const float e0 = exp2f(fmaf(__uint_as_float(r[c]), scale_l2, -(cl2 + lse2[c0 + c])));
                    const float e1 = exp2f(fmaf(__uint_as_float(r[c + 1]), scale_l2, -(cl2 + lse2[c0 + c + 1])));
                    csum += e0 + e1;
                    pk[c >> 1] = pack_bf16(e0, e1);
                }
                tmem_st8(s_t + (c0 >> 1), pk);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&bars->p_full[w]);

            // ---- drain the accumulator: this thread's aR row
            if (!mbar_wait(&bars->o_full[w], (g >> 1) & 1)) { fail(41); break; }
            tc_fence_after();
            const ItUnit un = it_decode(p, u);
            const int f = key / b1, k = key - f * b1;
            const long long ridx = ((((long long)un.bhl * p.F + f) * b1 + k) * p.na + un.al) * b2 + un.j;
            __nv_bfloat16* dst = p.aR + ridx * kHeadDim;
#pragma unroll 1
            for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(o_t + c0, r);
                tmem_wait_ld();
                if (c0 + 32 == kHeadDim) {
                    tc_fence_before();
                    mbar_arrive(&bars->o_free[w]);
                }
                if (valid) {
#pragma unroll
                    for (int v8 = 0; v8 < 2; ++v8) {
                        uint32_t wv[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            wv[e] = pack_bf16(__uint_as_float(r[v8 * 16 + 2 * e]), __uint_as_float(r[v8 * 16 + 2 * e + 1]));
                        st_global_v8_it(dst + c0 + v8 * 16, wv);
                    }
                }
            }
            if (valid) p.cR[ridx] = csum;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemColsIt);
}

}  // namespace

// Launches the tensor-core iteration update for one chunk.  maps = {aL (box 64 x 128 keys x 1), query rows (5-D)}.
int launch_l_iter_tc(const MonarchParams& p, const CUtensorMap* map_al, const CUtensorMap* map_qrows, int* status,
                     int num_sms, cudaStream_t s) {
    if (p.blk.b1 > 128) return SFM_ERR_UNSUPPORTED;
    LaunchScope scope(kClsLIter, s);
    ItParams ip;
    ip.mp = p;
    ip.n_units = p.nbh * p.na * p.blk.b2;
    ip.R4 = (p.blk.b1 + 3) / 4;
    ip.q_rows_tma = (p.blk.f_tied == 1 || p.blk.h_reduce == 1) ? 1 : 0;
    ip.status = status;
    dim3 grid(ip.n_units < num_sms ? ip.n_units : num_sms);
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kItSmemBytes);
        if (e != cudaSuccess) return (int)e;
        kernel<<<grid, kThreadsIt, kItSmemBytes, s>>>(*map_al, *map_qrows, ip);
        return 0;
    };
    int rc;
    switch ((p.blk.b1 + 15) & ~15) {
        case 16: rc = go(monarch_iter_tc_kernel<16>); break;
        case 32: rc = go(monarch_iter_tc_kernel<32>); break;
        case 48: rc = go(monarch_iter_tc_kernel<48>); break;
        case 64: rc = go(monarch_iter_tc_kernel<64>); break;
        case 80: rc = go(monarch_iter_tc_kernel<80>); break;
        case 96: rc = go(monarch_iter_tc_kernel<96>); break;
        case 112: rc = go(monarch_iter_tc_kernel<112>); break;
        case 128: rc = go(monarch_iter_tc_kernel<128>); break;
        default: return SFM_ERR_UNSUPPORTED;
    }
    if (rc) return rc;
    return (int)cudaGetLastError();
}

}  // namespace sfm
