// Backward of the Monarch row step on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Forward row step, per (batch*head, block row k, cached group f) and stacked query row r = (query group a, column j):
//   z_l = scale * q[r] . K[f,k,l],  R = softmax_l z,  aL[r] = sum_l R_l K_l,  Y[r] = sum_l R_l V_l,  cL[r] = sum_l R_l ln R_l
// Given daL[r], dY[r] (bf16, in the bridge layout [slab][key][128], left there by the column step's backward) and dcL[r]:
//   dR_l = daL[r] . K_l + dY[r] . V_l + dcL[r] (ln R_l + 1)          dz_l = R_l (dR_l - sum_m R_m dR_m)
//   dQ[r] += scale * sum_l dz_l K_l
//   dK_l  += sum_r (R_l daL[r] + scale dz_l q[r])                      dV_l += sum_r R_l dY[r]
// Units are those of the forward row step: (batch*head, tile of stacked query groups, block row k), each walking
// all cached groups f; per step
//   S  = Q_tile K^T                 dR = daL_tile K^T + dY_tile V^T        three tcgen05.mma chains, operands in shared memory
//   R, dz                           one thread per query row (R recomputed exactly as in the forward)
//   dQ (+)= (scale dz) K            A = scale dz as bf16 in TMEM, B = the K tile MN-major; accumulates over f in TMEM
//   dK = R^T daL_tile + (scale dz)^T Q_tile,   dV = R^T dY_tile
//                                   A = bf16 copies of R / scale dz in shared memory read MN-major (M = key l, padded to
//                                   128 with a block of zeros), B = the row tiles read MN-major; only for the cached
//                                   groups whose dK / dV are wanted
// dK / dV of a (f, k) get one contribution per tile of query groups: each tile writes fp32 partials to its own
// buffer and a small kernel adds them in a fixed order and rounds to bf16 (no atomics).  dQ rows are owned by one
// unit each and added to what the column step's backward left in dq.
//
// Warp roles (12 warps): 0 = TMA producer, 1 = MMA issuer (owns TMEM), 2-3 idle, 4-7 = element-wise warpgroup,
// 8-11 = drain warpgroup (dK / dV per step, dQ per unit).  Every wait is bounded and reports through the status word.
//
// Stands in for the Triton kernel _al_cl_y_bwd (wan/modules/monarch_attn.py:403-596), without its atomic adds.
#include "monarch_params.cuh"
#include "profile.cuh"
#include "tc05.cuh"

namespace sfm {

using namespace tc;

namespace {

constexpr int kThreadsRB = 384;
constexpr int kRows = 128;
constexpr uint32_t kTmemColsRB = 512;
constexpr uint32_t kCS = 0, kCDR = 64, kCDQ = 128, kCDK = 256, kCDV = 384;

struct BwdRowParams {
    MonarchParams mp;              // q, kc, vc, blocking, slice; mp.aL / mp.Y hold daL / dY
    const float* dcL;              // [slab][n_keys_c]
    float* dq;                     // natural order fp32, already holds the column step's share
    float* part_k;                 // [tile][nbh][n_sel tokens][128] fp32 partial dK (n_sel = (g1 - g0) * b1 * b2)
    float* part_v;
    int g0, g1;                    // cached groups whose dK / dV are wanted
    int rows_per_group, groups_per_tile, tiles, n_units;
    int* status;
};

struct __align__(8) RBBarriers {
    uint64_t q_full, q_empty;
    uint64_t kv_full[2], kv_empty[2];
    uint64_t da_full, da_empty;
    uint64_t s_full, dr_full, p_full, sdr_free;
    uint64_t dkv_full, dkv_free, dq_full, dq_free;
    uint32_t tmem_base;
    volatile int abort_flag;
};

constexpr int kQB = 2 * kRows * 128;                 // a row tile: two 64-column halves of 128 rows (32 KB)
constexpr int kKVStage = 4 * 64 * 128;               // K lo, K hi, V lo, V hi (<= 64 rows each)
constexpr int kStageT = kRows * 128;                 // R or dz copy: 128 rows x 64 bf16 (16 KB)
constexpr int kRBSmem = 1024 + kQB + 2 * kKVStage + 2 * kQB + 3 * kStageT + (int)sizeof(RBBarriers) + 64;

struct RBUnit { int bhl, tile, k; };
__device__ __forceinline__ RBUnit rb_decode(const BwdRowParams& rp, int u) {
    RBUnit r;
    r.k = u % rp.mp.blk.b1; u /= rp.mp.blk.b1;
    r.tile = u % rp.tiles;
    r.bhl = u / rp.tiles;
    return r;
}

// tq, tk, tv: the forward's maps of q, K, V; tda, tdy: bridge maps of daL / dY with a (64, 1 key, rows_per_group) box.
template <int N_S>
__global__ void __launch_bounds__(kThreadsRB, 1)
monarch_bwd_row_tc_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                          const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tda,
                          const __grid_constant__ CUtensorMap tdy, BwdRowParams rp) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;
    unsigned char* kv_s = q_s + kQB;                       // 2 stages
    unsigned char* da_s = kv_s + 2 * kKVStage;             // daL tile
    unsigned char* dy_s = da_s + kQB;                      // dY tile
    unsigned char* r_s = dy_s + kQB;                       // R copy | dz copy | zeros
    unsigned char* z_s = r_s + kStageT;
    RBBarriers* bars = reinterpret_cast<RBBarriers*>(r_s + 3 * kStageT);

    const MonarchParams& p = rp.mp;
    const Blocking& blk = p.blk;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b1 = blk.b1, b2 = blk.b2;
    const int RG = rp.rows_per_group;
    const int F = p.F;
    constexpr int kHalf = N_S * 128;

    if (tid == 0) {
        mbar_init(&bars->q_full, 1); mbar_init(&bars->q_empty, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&bars->kv_full[s], 1); mbar_init(&bars->kv_empty[s], 1); }
        mbar_init(&bars->da_full, 1); mbar_init(&bars->da_empty, 1);
        mbar_init(&bars->s_full, 1); mbar_init(&bars->dr_full, 1); mbar_init(&bars->p_full, 128);
        mbar_init(&bars->sdr_free, 1);
        mbar_init(&bars->dkv_full, 1); mbar_init(&bars->dkv_free, 128);
        mbar_init(&bars->dq_full, 1); mbar_init(&bars->dq_free, 128);
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    // tile rows no load writes and the padding of the R / dz copies must read as zero
    for (int i = tid; i < (kQB + 2 * kKVStage + 2 * kQB + 3 * kStageT) / 16; i += kThreadsRB)
        reinterpret_cast<uint4*>(q_s)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 1) { tmem_alloc(&bars->tmem_base, kTmemColsRB); tmem_relinquish(); }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    auto fail = [&](int code) {
        bars->abort_flag = 1;
        atomicCAS(rp.status, 0, code);
    };
    const int u_first = blockIdx.x, u_stride = gridDim.x;
    auto wants_kv = [&](int f) { return f >= rp.g0 && f < rp.g1; };

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            prefetch_tmap(&tq); prefetch_tmap(&tk); prefetch_tmap(&tv); prefetch_tmap(&tda); prefetch_tmap(&tdy);
            int g = 0, uc = 0;
            bool ok = true;
            for (int u = u_first; ok && u < rp.n_units && !bars->abort_flag; u += u_stride, ++uc) {
                const RBUnit un = rb_decode(rp, u);
                const int bh = p.bh0 + un.bhl, b = bh / p.H, hd = bh - b * p.H;
                const int g_first = un.tile * rp.groups_per_tile;
                const int ng = min(rp.groups_per_tile, p.na - g_first);
                if (uc > 0 && !mbar_wait(&bars->q_empty, (uc - 1) & 1)) { fail(10); break; }
                mbar_arrive_expect_tx(&bars->q_full, (uint32_t)(ng * RG * 256));
                for (int gi = 0; gi < ng; ++gi) {
                    const int tok = blk.row_token(p.a0 + g_first + gi, un.k);
                    tma_load_4d(q_s + gi * RG * 128, &tq, &bars->q_full, 0, hd, tok, b);
                    tma_load_4d(q_s + kRows * 128 + gi * RG * 128, &tq, &bars->q_full, 64, hd, tok, b);
                }
                for (int f = 0; f < F; ++f, ++g) {
                    const int s = g & 1;
                    if (g >= 2 && !mbar_wait(&bars->kv_empty[s], ((g >> 1) - 1) & 1)) { fail(11); ok = false; break; }
                    const int tok = (f * b1 + un.k) * b2;
                    unsigned char* st = kv_s + s * kKVStage;
                    mbar_arrive_expect_tx(&bars->kv_full[s], (uint32_t)(4 * kHalf));
                    tma_load_4d(st, &tk, &bars->kv_full[s], 0, hd, tok, b);
                    tma_load_4d(st + kHalf, &tk, &bars->kv_full[s], 64, hd, tok, b);
                    tma_load_4d(st + 2 * kHalf, &tv, &bars->kv_full[s], 0, hd, tok, b);
                    tma_load_4d(st + 3 * kHalf, &tv, &bars->kv_full[s], 64, hd, tok, b);
                    if (g >= 1 && !mbar_wait(&bars->da_empty, (g - 1) & 1)) { fail(12); ok = false; break; }
                    const int key = f * b1 + un.k;
                    mbar_arrive_expect_tx(&bars->da_full, (uint32_t)(2 * ng * RG * 256));
                    for (int gi = 0; gi < ng; ++gi) {
                        const int slab = (un.bhl * p.na + g_first + gi) * b2;
                        tma_load_3d(da_s + gi * RG * 128, &tda, &bars->da_full, 0, key, slab);
                        tma_load_3d(da_s + kRows * 128 + gi * RG * 128, &tda, &bars->da_full, 64, key, slab);
                        tma_load_3d(dy_s + gi * RG * 128, &tdy, &bars->da_full, 0, key, slab);
                        tma_load_3d(dy_s + kRows * 128 + gi * RG * 128, &tdy, &bars->da_full, 64, key, slab);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16(kRows, N_S, 0, 0);            // S, dR
            constexpr uint32_t idesc_q = idesc_bf16(kRows, kHeadDim, 0, 1);        // dQ: A from TMEM, B MN-major
            constexpr uint32_t idesc_k = idesc_bf16(kRows, kHeadDim, 1, 1);        // dK, dV: both MN-major
            const uint64_t q_k = smem_desc_sw128(smem_addr(q_s), 16, 1024);
            const uint64_t q_mn = smem_desc_sw128(smem_addr(q_s), kRows * 128, 1024);
            const uint64_t da_k = smem_desc_sw128(smem_addr(da_s), 16, 1024);
            const uint64_t da_mn = smem_desc_sw128(smem_addr(da_s), kRows * 128, 1024);
            const uint64_t dy_k = smem_desc_sw128(smem_addr(dy_s), 16, 1024);
            const uint64_t dy_mn = smem_desc_sw128(smem_addr(dy_s), kRows * 128, 1024);
            const uint64_t kv_k0 = smem_desc_sw128(smem_addr(kv_s), 16, 1024);
            const uint64_t kv_mn0 = smem_desc_sw128(smem_addr(kv_s), kHalf, 1024);
            const uint64_t r_mn = smem_desc_sw128(smem_addr(r_s), 2 * kStageT, 1024);      // second M block = the zeros
            const uint64_t z_mn = smem_desc_sw128(smem_addr(z_s), kStageT, 1024);
            int g = 0, uc = 0, gd = 0;
            bool ok = true;
            for (int u = u_first; ok && u < rp.n_units && !bars->abort_flag; u += u_stride, ++uc) {
                if (!mbar_wait(&bars->q_full, uc & 1)) { fail(20); break; }
                for (int f = 0; f < F; ++f, ++g) {
                    const int s = g & 1;
                    const bool kvw = wants_kv(f);
                    if (!mbar_wait(&bars->kv_full[s], (g >> 1) & 1)) { fail(21); ok = false; break; }
                    if (g >= 1 && !mbar_wait(&bars->sdr_free, (g - 1) & 1)) { fail(22); ok = false; break; }
                    tc_fence_after();
                    const uint64_t kd = kv_k0 + (uint64_t)((s * kKVStage) >> 4);
                    const uint64_t vd = kd + (uint64_t)((2 * kHalf) >> 4);
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t qo = ((ks >> 2) * (kRows * 128) + (ks & 3) * 32) >> 4;
                        const uint32_t ko = ((ks >> 2) * kHalf + (ks & 3) * 32) >> 4;
                        mma_ss(tmem + kCS, q_k + qo, kd + ko, idesc_s, ks > 0);
                    }
                    mma_commit(&bars->s_full);
                    if (!mbar_wait(&bars->da_full, g & 1)) { fail(23); ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t qo = ((ks >> 2) * (kRows * 128) + (ks & 3) * 32) >> 4;
                        const uint32_t ko = ((ks >> 2) * kHalf + (ks & 3) * 32) >> 4;
                        mma_ss(tmem + kCDR, da_k + qo, kd + ko, idesc_s, ks > 0);
                    }
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t qo = ((ks >> 2) * (kRows * 128) + (ks & 3) * 32) >> 4;
                        const uint32_t ko = ((ks >> 2) * kHalf + (ks & 3) * 32) >> 4;
                        mma_ss(tmem + kCDR, dy_k + qo, vd + ko, idesc_s, 1u);
                    }
                    mma_commit(&bars->dr_full);
                    if (!kvw) mma_commit(&bars->da_empty);          // nothing else reads the row tiles this step
                    if (!mbar_wait(&bars->p_full, g & 1)) { fail(24); ok = false; break; }
                    if (f == 0 && uc >= 1 && !mbar_wait(&bars->dq_free, (uc - 1) & 1)) { fail(25); ok = false; break; }
                    tc_fence_after();
                    const uint64_t kmn = kv_mn0 + (uint64_t)((s * kKVStage) >> 4);
#pragma unroll
                    for (int kk = 0; kk < N_S / 16; ++kk)      // dQ (+)= (scale dz) K
                        mma_ts(tmem + kCDQ, tmem + kCDR + kk * 8, kmn + ((kk * 2048) >> 4), idesc_q, (f > 0 || kk > 0) ? 1u : 0u);
                    if (kvw) {
                        if (gd >= 1 && !mbar_wait(&bars->dkv_free, (gd - 1) & 1)) { fail(26); ok = false; break; }
                        tc_fence_after();
#pragma unroll
                        for (int kk = 0; kk < kRows / 16; ++kk)     // dK = R^T daL_tile
                            mma_ss(tmem + kCDK, r_mn + ((kk * 2048) >> 4), da_mn + ((kk * 2048) >> 4), idesc_k, kk > 0);
#pragma unroll
                        for (int kk = 0; kk < kRows / 16; ++kk)     // dK += (scale dz)^T Q_tile
                            mma_ss(tmem + kCDK, z_mn + ((kk * 2048) >> 4), q_mn + ((kk * 2048) >> 4), idesc_k, 1u);
#pragma unroll
                        for (int kk = 0; kk < kRows / 16; ++kk)     // dV = R^T dY_tile
                            mma_ss(tmem + kCDV, r_mn + ((kk * 2048) >> 4), dy_mn + ((kk * 2048) >> 4), idesc_k, kk > 0);
                        mma_commit(&bars->dkv_full);
                        mma_commit(&bars->da_empty);
                        ++gd;
                    }
                    mma_commit(&bars->sdr_free);
                    mma_commit(&bars->kv_empty[s]);
                    if (f + 1 == F) { mma_commit(&bars->dq_full); mma_commit(&bars->q_empty); }
                }
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------------------------------------------ element-wise warpgroup: one query row per thread
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int gl = row / RG, j = row - gl * RG;
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const float scale_l2 = p.mult0 * kLog2e;
        unsigned char* r_row = r_s + row * 128;
        unsigned char* z_row = z_s + row * 128;
        int g = 0;
        bool ok = true;
        for (int u = u_first; ok && u < rp.n_units && !bars->abort_flag; u += u_stride) {
            const RBUnit un = rb_decode(rp, u);
            const int g_first = un.tile * rp.groups_per_tile;
            const int ng = min(rp.groups_per_tile, p.na - g_first);
            const bool row_ok = gl < ng && j < b2;
            const long long slab = ((long long)un.bhl * p.na + g_first + gl) * b2 + j;
            for (int f = 0; f < F; ++f, ++g) {
                const float dcl = row_ok ? rp.dcL[slab * p.n_keys_c + f * b1 + un.k] : 0.f;
                if (!mbar_wait(&bars->s_full, g & 1)) { fail(31); ok = false; break; }
                tc_fence_after();
                uint32_t raw[N_S], dr[N_S];
                if constexpr (N_S == 64) {
                    tmem_ld32(tmem + lane_sel + kCS, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
                    tmem_ld32(tmem + lane_sel + kCS + 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[32]));
                } else if constexpr (N_S == 48) {
                    tmem_ld32(tmem + lane_sel + kCS, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
                    tmem_ld16(tmem + lane_sel + kCS + 32, *reinterpret_cast<uint32_t(*)[16]>(&raw[32]));
                } else if constexpr (N_S == 32) {
                    tmem_ld32(tmem + lane_sel + kCS, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
                } else {
                    tmem_ld16(tmem + lane_sel + kCS, *reinterpret_cast<uint32_t(*)[16]>(&raw[0]));
                }
                tmem_wait_ld();
                float mx = -INFINITY;
#pragma unroll
                for (int c = 0; c < N_S; ++c) {
                    if (c >= b2) raw[c] = 0xf149f2cau;                 // -1e30: weight zero
                    mx = fmaxf(mx, __uint_as_float(raw[c]));
                }
                const float m2 = mx * scale_l2;
                float z = 0.f;
#pragma unroll
                for (int c = 0; c < N_S; ++c) z += exp2f(fmaf(__uint_as_float(raw[c]), scale_l2, -m2));
                const float inv_z = 1.0f / z, l2z = __log2f(z);
                if (!mbar_wait(&bars->dr_full, g & 1)) { fail(32); ok = false; break; }
                tc_fence_after();
                if constexpr (N_S == 64) {
                    tmem_ld32(tmem + lane_sel + kCDR, *reinterpret_cast<uint32_t(*)[32]>(&dr[0]));
                    tmem_ld32(tmem + lane_sel + kCDR + 32, *reinterpret_cast<uint32_t(*)[32]>(&dr[32]));
                } else if constexpr (N_S == 48) {
                    tmem_ld32(tmem + lane_sel + kCDR, *reinterpret_cast<uint32_t(*)[32]>(&dr[0]));
                    tmem_ld16(tmem + lane_sel + kCDR + 32, *reinterpret_cast<uint32_t(*)[16]>(&dr[32]));
                } else if constexpr (N_S == 32) {
                    tmem_ld32(tmem + lane_sel + kCDR, *reinterpret_cast<uint32_t(*)[32]>(&dr[0]));
                } else {
                    tmem_ld16(tmem + lane_sel + kCDR, *reinterpret_cast<uint32_t(*)[16]>(&dr[0]));
                }
                tmem_wait_ld();
                // dR_l = (daL . K_l + dY . V_l) + dcL (ln R_l + 1); sum_l R_l dR_l
                float dot = 0.f;
#pragma unroll
                for (int c = 0; c < N_S; ++c) {
                    const float d2 = fmaf(__uint_as_float(raw[c]), scale_l2, -m2);     // log2 of the unnormalised weight
                    const float rr = exp2f(d2) * inv_z;
                    const float lnr = (d2 - l2z) * 0.6931471805599453f;
                    const float x = c < b2 ? fmaf(dcl, lnr + 1.0f, __uint_as_float(dr[c])) : 0.f;
                    dr[c] = __float_as_uint(x);
                    dot = fmaf(rr, x, dot);
                }
                uint32_t pr[N_S / 2], pz[N_S / 2];
#pragma unroll
                for (int c = 0; c < N_S; c += 2) {
                    float r0 = exp2f(fmaf(__uint_as_float(raw[c]), scale_l2, -m2)) * inv_z;
                    float r1 = exp2f(fmaf(__uint_as_float(raw[c + 1]), scale_l2, -m2)) * inv_z;
                    float z0 = r0 * (__uint_as_float(dr[c]) - dot) * p.scale;
                    float z1 = r1 * (__uint_as_float(dr[c + 1]) - dot) * p.scale;
                    if (!row_ok) { r0 = 0.f; r1 = 0.f; z0 = 0.f; z1 = 0.f; }   // rows of no unit must not reach dK / dV
                    pr[c >> 1] = pack_bf16(r0, r1);
                    pz[c >> 1] = pack_bf16(z0, z1);
                }
                // scale dz as the TMEM operand of the dQ GEMM (over the dR columns already read)
                if constexpr (N_S == 64) {
                    tmem_st32(tmem + lane_sel + kCDR, pz);
                } else if constexpr (N_S == 32) {
                    tmem_st16(tmem + lane_sel + kCDR, pz);
                } else if constexpr (N_S == 48) {
                    tmem_st16(tmem + lane_sel + kCDR, *reinterpret_cast<uint32_t(*)[16]>(&pz[0]));
                    uint32_t t2[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) t2[c] = c < 8 ? pz[16 + c] : 0u;
                    tmem_st16(tmem + lane_sel + kCDR + 16, t2);
                } else {
                    uint32_t t2[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) t2[c] = c < 8 ? pz[c] : 0u;
                    tmem_st16(tmem + lane_sel + kCDR, t2);
                }
                // bf16 copies of the R and scale dz rows for the dK / dV GEMMs (128-byte swizzled rows)
#pragma unroll
                for (int c = 0; c < N_S / 8; ++c) {
                    const int pc = (c ^ (row & 7)) << 4;
                    *reinterpret_cast<uint4*>(r_row + pc) = make_uint4(pr[4 * c], pr[4 * c + 1], pr[4 * c + 2], pr[4 * c + 3]);
                    *reinterpret_cast<uint4*>(z_row + pc) = make_uint4(pz[4 * c], pz[4 * c + 1], pz[4 * c + 2], pz[4 * c + 3]);
                }
                fence_async_smem();
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&bars->p_full);
            }
        }
    } else if (warp >= 8) {
        // ------------------------------------------------------------------ drain warpgroup
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                       // dK / dV: key l; dQ: query row
        const int gl = row / RG, j = row - gl * RG;
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const long long n_sel = (long long)(rp.g1 - rp.g0) * b1 * b2;
        int uc = 0, gd = 0;
        bool ok = true;
        for (int u = u_first; ok && u < rp.n_units && !bars->abort_flag; u += u_stride, ++uc) {
            const RBUnit un = rb_decode(rp, u);
            const int bh = p.bh0 + un.bhl, b = bh / p.H, hd = bh - b * p.H;
            const int g_first = un.tile * rp.groups_per_tile;
            const int ng = min(rp.groups_per_tile, p.na - g_first);
            for (int f = 0; f < F; ++f) {
                if (!wants_kv(f)) continue;
                if (!mbar_wait(&bars->dkv_full, gd & 1)) { fail(41); ok = false; break; }
                tc_fence_after();
                const long long prow = (((long long)un.tile * p.nbh + un.bhl) * n_sel + ((long long)(f - rp.g0) * b1 + un.k) * b2 + row) * kHeadDim;
#pragma unroll 1
                for (int half = 0; half < 2; ++half) {
                    float* dst = (half ? rp.part_v : rp.part_k) + prow;
                    const uint32_t col0 = half ? kCDV : kCDK;
#pragma unroll 1
                    for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
                        uint32_t r[32];
                        if (quad < 2) {                        // keys live on lanes 0..63
                            tmem_ld32(tmem + lane_sel + col0 + c0, r);
                            tmem_wait_ld();
                        }
                        if (half == 1 && c0 + 32 == kHeadDim) {
                            tc_fence_before();
                            mbar_arrive(&bars->dkv_free);
                        }
                        if (quad < 2 && row < b2) {
#pragma unroll
                            for (int v = 0; v < 8; ++v)
                                *reinterpret_cast<uint4*>(dst + c0 + 4 * v) = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                        }
                    }
                }
                ++gd;
            }
            if (!ok) break;
            // ---- the unit's dQ rows: added to the column step's share
            if (!mbar_wait(&bars->dq_full, uc & 1)) { fail(42); break; }
            tc_fence_after();
            const bool row_ok = gl < ng && j < b2;
            float* dqr = nullptr;
            if (row_ok) {
                const long long tok = blk.row_token(p.a0 + g_first + gl, un.k) + j;
                dqr = rp.dq + (((long long)b * p.n_q + tok) * p.H + hd) * kHeadDim;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem + lane_sel + kCDQ + c0, r);
                tmem_wait_ld();
                if (c0 + 32 == kHeadDim) {
                    tc_fence_before();
                    mbar_arrive(&bars->dq_free);
                }
                if (row_ok) {
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        float4 o = *reinterpret_cast<float4*>(dqr + c0 + 4 * v);
                        o.x += __uint_as_float(r[4 * v]); o.y += __uint_as_float(r[4 * v + 1]);
                        o.z += __uint_as_float(r[4 * v + 2]); o.w += __uint_as_float(r[4 * v + 3]);
                        *reinterpret_cast<float4*>(dqr + c0 + 4 * v) = o;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemColsRB);
}

// dk / dv [B, n_sel, H, 128] bf16 (Monarch order) = sum over the tiles' fp32 partials, in tile order.
__global__ void __launch_bounds__(256) bwd_merge_kv_kernel(const float* __restrict__ part_k, const float* __restrict__ part_v,
                                                           __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                                                           int tiles, int nbh, long long n_sel, int H, int bh0) {
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;          // one float4 of one (bh_local, token)
    const long long per_bh = n_sel * (kHeadDim / 4);
    if (idx >= per_bh * nbh) return;
    const int bhl = (int)(idx / per_bh);
    const long long rem = idx - (long long)bhl * per_bh;
    const long long tok = rem / (kHeadDim / 4);
    const int c4 = (int)(rem - tok * (kHeadDim / 4));
    const int bh = bh0 + bhl, b = bh / H, hd = bh - b * H;
    float4 k = make_float4(0.f, 0.f, 0.f, 0.f), v = k;
    for (int t = 0; t < tiles; ++t) {
        const long long o = ((long long)t * nbh + bhl) * n_sel * kHeadDim + tok * kHeadDim + c4 * 4;
        const float4 a = *reinterpret_cast<const float4*>(part_k + o);
        const float4 c = *reinterpret_cast<const float4*>(part_v + o);
        k.x += a.x; k.y += a.y; k.z += a.z; k.w += a.w;
        v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
    }
    const long long out = (((long long)b * n_sel + tok) * H + hd) * kHeadDim + c4 * 4;
    *reinterpret_cast<uint2*>(dk + out) = make_uint2(pack_bf16(k.x, k.y), pack_bf16(k.z, k.w));
    *reinterpret_cast<uint2*>(dv + out) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

}  // namespace

size_t bwd_row_tc_partial_bytes(const MonarchParams& mp, int g0, int g1) {
    const int rows_per_group = (mp.blk.b2 + 7) & ~7;
    const int gpt = kRows / rows_per_group;
    const int tiles = (mp.na + gpt - 1) / gpt;
    return (size_t)tiles * mp.nbh * (size_t)(g1 - g0) * mp.blk.b1 * mp.blk.b2 * kHeadDim * sizeof(float);
}

// Row-step backward for one slice.  maps = {q, K, V (the forward's), daL bridge, dY bridge (box 64 x 1 x rows_per_group)}.
int launch_bwd_row_tc(const MonarchParams& mp, const CUtensorMap* maps, const float* dcL, float* dq, float* part_k,
                      float* part_v, __nv_bfloat16* dk, __nv_bfloat16* dv, int g0, int g1, int* status, int num_sms,
                      cudaStream_t s) {
    if (mp.blk.b2 > 64) return SFM_ERR_UNSUPPORTED;
    BwdRowParams rp;
    rp.mp = mp;
    rp.dcL = dcL; rp.dq = dq; rp.part_k = part_k; rp.part_v = part_v;
    rp.g0 = g0; rp.g1 = g1;
    rp.rows_per_group = (mp.blk.b2 + 7) & ~7;
    rp.groups_per_tile = kRows / rp.rows_per_group;
    rp.tiles = (mp.na + rp.groups_per_tile - 1) / rp.groups_per_tile;
    rp.n_units = mp.nbh * rp.tiles * mp.blk.b1;
    rp.status = status;
    dim3 grid(rp.n_units < num_sms ? rp.n_units : num_sms);
    const int n_s = (mp.blk.b2 + 15) & ~15;
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRBSmem);
        if (e != cudaSuccess) return (int)e;
        kernel<<<grid, kThreadsRB, kRBSmem, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4], rp);
        return 0;
    };
    int rc;
    {
        LaunchScope scope(kClsBackward, s);
        switch (n_s) {
            case 16: rc = go(monarch_bwd_row_tc_kernel<16>); break;
            case 32: rc = go(monarch_bwd_row_tc_kernel<32>); break;
            case 48: rc = go(monarch_bwd_row_tc_kernel<48>); break;
            case 64: rc = go(monarch_bwd_row_tc_kernel<64>); break;
            default: return SFM_ERR_UNSUPPORTED;
        }
        if (rc) return rc;
        if (cudaGetLastError() != cudaSuccess) return SFM_ERR_UNSUPPORTED;
    }
    if (g1 > g0) {
        LaunchScope scope(kClsBackward, s);
        const long long n_sel = (long long)(g1 - g0) * mp.blk.b1 * mp.blk.b2;
        const long long n = n_sel * (kHeadDim / 4) * mp.nbh;
        bwd_merge_kv_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(part_k, part_v, dk, dv, rp.tiles, mp.nbh, n_sel, mp.H,
                                                                       mp.bh0);
        if (cudaGetLastError() != cudaSuccess) return SFM_ERR_UNSUPPORTED;
    }
    return SFM_OK;
}

}  // namespace sfm
