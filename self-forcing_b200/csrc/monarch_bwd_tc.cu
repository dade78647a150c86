// Backward of the Monarch column step on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Forward column step, per slab (batch*head, query group a, column j), query row i, key n = (f, k):
//   s[i,n] = scale * q[a,i,j] . aL[n] - cL[n],   P = softmax_n s,   out[a,i,j] = sum_n P[i,n] Y[n]
// with aL[n] = sum_l R_l K_l and Y[n] = sum_l R_l V_l the row step's results (bf16, in the bridge layout
// [slab][key][128]).  Given dOut, lse[i] = log sum_n exp s[i,n] (from a forward column step run just before)
// and delta[i] = dOut[i] . out[i], one sweep over the slab's keys in tiles of 128 gives every gradient:
//   dP[i,n] = dOut[i] . Y[n]                      dS = P (dP - delta)
//   dY[n]  = sum_i P[i,n] dOut[i]                 daL[n] = scale * sum_i dS[i,n] q[i]        dcL[n] = -sum_i dS[i,n]
//   dq[i]  = scale * sum_n dS[i,n] aL[n]          (the row step's share of dQ is added by its own backward)
// The KEYS sit on the M side of the tensor core (TMEM lane = key), the slab's b1 <= 32 queries on the N side, so
// that dY, daL and dcL come out one key per lane, ready for row-wise stores:
//   S^T  = aL_tile Q^T,  dP^T = Y_tile dOut^T               two tcgen05.mma, operands in shared memory
//   P^T, (scale dS)^T as bf16 over the S^T / dP^T columns     one thread per key; dcL from its registers
//   dY_tile = P^T dOut,  daL_tile = (scale dS)^T Q            A from TMEM, B = the query-side rows, MN-major
//   dq^T (+)= aL_tile^T (scale dS)^T                          A = the aL tile read MN-major, B = a bf16 copy of
//                                                             (scale dS)^T in shared memory; accumulates over the slab
// dY and daL are written over Y and aL in place (a tile is in shared memory before its rows are overwritten).
//
// Warp roles (12 warps): 0 = TMA producer, 1 = MMA issuer (owns TMEM), 2-3 idle, 4-7 and 8-11 = two warpgroups
// that take even / odd tiles (element-wise pass, then the drain of the dY / daL accumulators; the group that
// handled a slab's last tile also stores its dq).  Persistent CTAs over contiguous shares of the slab list.
// All waits are bounded and report through the status word.
//
// Stands in for the Triton kernel _z_bwd and its preprocess (wan/modules/monarch_attn.py:852-886, 1034-1222).
#include "monarch_params.cuh"
#include "profile.cuh"
#include "tc05.cuh"

namespace sfm {

using namespace tc;

namespace {

constexpr int kStgB = 2;                     // (aL, Y) tile-pair ring
constexpr int kThreadsB = 384;
constexpr int kKB = 128;                     // keys per tile
constexpr int kNI = 32;                      // query rows per slab, padded (block rows up to 32)
constexpr uint32_t kTmemColsB = 512;
// TMEM columns: per warpgroup S^T / P^T at w*64, dP^T / dS^T at w*64 + 32; accumulators after them
__host__ __device__ constexpr uint32_t bc_s(int w) { return (uint32_t)w * 64u; }
__host__ __device__ constexpr uint32_t bc_dp(int w) { return (uint32_t)w * 64u + 32u; }
constexpr uint32_t kColDaL = 128, kColDY = 256, kColDq = 384;

struct BwdColParams {
    const __nv_bfloat16* q;        // natural order [B, n_q, H, 128]
    long long q_bs;
    const float* delta;            // [B, n_q, H]: dOut . out per token and head
    const float* lse;              // [slab][b1]
    __nv_bfloat16* aL;             // bridge [slab][n_keys][128]: aL in, daL out
    __nv_bfloat16* Y;              // bridge: Y in, dY out
    const float* cL;               // [slab][n_keys_c]
    float* dcL;                    // [slab][n_keys_c]
    float* dq;                     // natural order [B, n_q, H, 128] fp32
    int H, n_q, A, n_keys, n_keys_c, bh0, nbh;
    int n_units;                   // nbh * A * b2
    int R4, q_rows_tma;
    float scale;
    Blocking blk;
    int* status;
};

constexpr int kQdHalf = kNI * 128;                 // one 64-column half of a query-side tile (32 rows)
constexpr int kQdTile = 2 * kQdHalf;               // 8 KB
constexpr int kQdBuf = 2 * kQdTile;                // q tile + dOut tile of one slab
constexpr int kBTile = 2 * kKB * 128;              // one aL or Y tile, 32 KB
constexpr int kBStage = 2 * kBTile;                // aL + Y
constexpr int kDsTile = kKB * 128;                 // (scale dS)^T copy: 128 keys x 64 bf16, 16 KB

struct __align__(16) BBarriers {
    float lse2[2][kNI];
    float delta[2][kNI];
    uint64_t q_full[2], q_empty[2];
    uint64_t a_full[kStgB], a_empty[kStgB];
    uint64_t s_full[2], p_full[2], sd_free[2];
    uint64_t acc_full[2], acc_free[2];      // per warpgroup: a parity wait may lag its barrier by one phase only
    uint64_t dq_full, dq_free;
    uint32_t tmem_base;
    volatile int abort_flag;
};

constexpr int kBSmemBytes = 1024 + 2 * kQdBuf + kStgB * kBStage + 2 * kDsTile + (int)sizeof(BBarriers) + 64;

__device__ __forceinline__ void tmem_st16b(uint32_t taddr, const uint32_t (&r)[16]) { tmem_st16(taddr, r); }
__device__ __forceinline__ void stg_v8(void* ptr, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                 "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}

struct BUnit { int bhl, a, j; };
__device__ __forceinline__ BUnit b_decode(const BwdColParams& p, int u) {
    BUnit r;
    r.j = u % p.blk.b2; u /= p.blk.b2;
    r.a = u % p.A;
    r.bhl = u / p.A;
    return r;
}

// tal / ty = bridge maps (box 64 x 128 keys x 1); tqr / tdo = query rows of q / dOut (5-D, box rows = R4).
__global__ void __launch_bounds__(kThreadsB, 1)
monarch_bwd_col_tc_kernel(const __grid_constant__ CUtensorMap tal, const __grid_constant__ CUtensorMap ty,
                          const __grid_constant__ CUtensorMap tqr, const __grid_constant__ CUtensorMap tdo,
                          BwdColParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* qd_s = base;                                   // [2 slabs][q tile | dOut tile]
    unsigned char* a_s = qd_s + 2 * kQdBuf;                        // [stage][aL tile | Y tile]
    unsigned char* ds_s = a_s + kStgB * kBStage;                   // [warpgroup] (scale dS)^T, 128 rows of 128 bytes
    BBarriers* bars = reinterpret_cast<BBarriers*>(ds_s + 2 * kDsTile);

    const Blocking& blk = p.blk;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b1 = blk.b1, b2 = blk.b2;
    const int n_keys = p.n_keys;
    const int n_tiles = (n_keys + kKB - 1) / kKB;
    const int R4 = p.R4;
    const long long tok_pitch = (long long)p.H * kHeadDim;
    const int u_begin = (int)((long long)p.n_units * blockIdx.x / gridDim.x);
    const int u_end = (int)((long long)p.n_units * (blockIdx.x + 1) / gridDim.x);
    const int total = (u_end - u_begin) * n_tiles;

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(&bars->q_full[s], 1); mbar_init(&bars->q_empty[s], 1); }
        for (int s = 0; s < kStgB; ++s) { mbar_init(&bars->a_full[s], 1); mbar_init(&bars->a_empty[s], 1); }
        for (int w = 0; w < 2; ++w) {
            mbar_init(&bars->s_full[w], 1); mbar_init(&bars->p_full[w], 128); mbar_init(&bars->sd_free[w], 1);
        }
        for (int w = 0; w < 2; ++w) { mbar_init(&bars->acc_full[w], 1); mbar_init(&bars->acc_free[w], 128); }
        mbar_init(&bars->dq_full, 1); mbar_init(&bars->dq_free, 128);
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    // query-side rows no load writes, and the padding columns of the (scale dS)^T copies, must read as zero
    for (int i = tid; i < (2 * kQdBuf + 0) / 16; i += kThreadsB) reinterpret_cast<uint4*>(qd_s)[i] = make_uint4(0, 0, 0, 0);
    for (int i = tid; i < 2 * kDsTile / 16; i += kThreadsB) reinterpret_cast<uint4*>(ds_s)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 1) { tmem_alloc(&bars->tmem_base, kTmemColsB); tmem_relinquish(); }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    auto fail = [&](int code) {
        bars->abort_flag = 1;
        atomicCAS(p.status, 0, code);
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) { prefetch_tmap(&tal); prefetch_tmap(&ty); prefetch_tmap(&tqr); prefetch_tmap(&tdo); }
        int g = 0, uc = 0;
        bool ok = true;
        for (int u = u_begin; ok && u < u_end && !bars->abort_flag; ++u, ++uc) {
            const BUnit un = b_decode(p, u);
            const int bh = p.bh0 + un.bhl, b = bh / p.H, hd = bh - b * p.H;
            const int qb = uc & 1;
            unsigned char* qt = qd_s + qb * kQdBuf;
            if (uc >= 2) {
                int okw = 1;
                if (lane == 0) okw = mbar_wait(&bars->q_empty[qb], ((uc >> 1) - 1) & 1) ? 1 : 0;
                if (!__shfl_sync(0xffffffffu, okw, 0)) { fail(10); break; }
            }
            if (lane < kNI) {
                const int i = lane;
                float l2 = INFINITY, dl = 0.f;
                if (i < b1) {
                    const long long tok = blk.row_token(un.a, i) + un.j;
                    l2 = kLog2e * p.lse[(long long)u * b1 + i];
                    dl = p.delta[((long long)b * p.n_q + tok) * p.H + hd];
                }
                bars->lse2[qb][i] = l2;
                bars->delta[qb][i] = dl;
            }
            if (p.q_rows_tma) {
                __syncwarp();
                if (lane == 0) {
                    const int nq = (b1 + R4 - 1) / R4;
                    mbar_arrive_expect_tx(&bars->q_full[qb], (uint32_t)(2 * nq * R4 * 256));
                    const int tok0 = blk.row_token(un.a, 0);
                    const int frow0 = tok0 / blk.w, col = tok0 - frow0 * blk.w + un.j;
                    for (int qd = 0; qd < nq; ++qd) {
                        unsigned char* dq_ = qt + (qd * R4) * 128;
                        tma_load_5d(dq_, &tqr, &bars->q_full[qb], 0, hd, col, frow0 + qd * R4, b);
                        tma_load_5d(dq_ + kQdHalf, &tqr, &bars->q_full[qb], 64, hd, col, frow0 + qd * R4, b);
                        tma_load_5d(dq_ + kQdTile, &tdo, &bars->q_full[qb], 0, hd, col, frow0 + qd * R4, b);
                        tma_load_5d(dq_ + kQdTile + kQdHalf, &tdo, &bars->q_full[qb], 64, hd, col, frow0 + qd * R4, b);
                    }
                }
            } else {
                fail(12);                      // the host only launches this kernel for blockings whose query rows come by TMA
                break;
            }
            if (lane == 0) {
                for (int t = 0; t < n_tiles; ++t, ++g) {
                    const int s = g % kStgB;
                    if (g >= kStgB && !mbar_wait(&bars->a_empty[s], ((g / kStgB) - 1) & 1)) { fail(11); ok = false; break; }
                    unsigned char* st = a_s + s * kBStage;
                    mbar_arrive_expect_tx(&bars->a_full[s], (uint32_t)kBStage);
                    tma_load_3d(st, &tal, &bars->a_full[s], 0, t * kKB, u);
                    tma_load_3d(st + kKB * 128, &tal, &bars->a_full[s], 64, t * kKB, u);
                    tma_load_3d(st + kBTile, &ty, &bars->a_full[s], 0, t * kKB, u);
                    tma_load_3d(st + kBTile + kKB * 128, &ty, &bars->a_full[s], 64, t * kKB, u);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            g = __shfl_sync(0xffffffffu, g, 0);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16(128, kNI, 0, 0);            // S^T, dP^T
            constexpr uint32_t idesc_o = idesc_bf16(128, kHeadDim, 0, 1);       // dY, daL: A from TMEM, B MN-major
            constexpr uint32_t idesc_q = idesc_bf16(128, 64, 1, 1);             // dq^T: both operands MN-major
            const uint64_t a_k0 = smem_desc_sw128(smem_addr(a_s), 16, 1024);               // aL / Y tile, K-major
            const uint64_t a_mn0 = smem_desc_sw128(smem_addr(a_s), kKB * 128, 1024);        // aL tile, MN-major (M = d)
            const uint64_t q_k0 = smem_desc_sw128(smem_addr(qd_s), 16, 1024);              // q / dOut rows, K-major
            const uint64_t q_mn0 = smem_desc_sw128(smem_addr(qd_s), kQdHalf, 1024);         // q / dOut rows, MN-major
            const uint64_t ds0 = smem_desc_sw128(smem_addr(ds_s), 16, 1024);                // (scale dS)^T copy, MN-major, N = 64
            bool ok = true;
            auto issue_s = [&](int g) -> bool {
                const int uc = g / n_tiles, t = g - uc * n_tiles, w = g & 1, s = g % kStgB, qb = uc & 1;
                if (t == 0 && !mbar_wait(&bars->q_full[qb], (uc >> 1) & 1)) { fail(20); return false; }
                if (!mbar_wait(&bars->a_full[s], (g / kStgB) & 1)) { fail(21); return false; }
                if (g >= 2 && !mbar_wait(&bars->sd_free[w], ((g >> 1) - 1) & 1)) { fail(22); return false; }
                tc_fence_after();
                const uint64_t al = a_k0 + (uint64_t)((s * kBStage) >> 4);
                const uint64_t yy = al + (uint64_t)(kBTile >> 4);
                const uint64_t qq = q_k0 + (uint64_t)((qb * kQdBuf) >> 4);
                const uint64_t dd = qq + (uint64_t)(kQdTile >> 4);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t ao = ((ks >> 2) * (kKB * 128) + (ks & 3) * 32) >> 4;
                    const uint32_t qo = ((ks >> 2) * kQdHalf + (ks & 3) * 32) >> 4;
                    mma_ss(tmem + bc_s(w), al + ao, qq + qo, idesc_s, ks > 0);
                }
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t ao = ((ks >> 2) * (kKB * 128) + (ks & 3) * 32) >> 4;
                    const uint32_t qo = ((ks >> 2) * kQdHalf + (ks & 3) * 32) >> 4;
                    mma_ss(tmem + bc_dp(w), yy + ao, dd + qo, idesc_s, ks > 0);
                }
                mma_commit(&bars->s_full[w]);
                return true;
            };
            if (total > 0) ok = issue_s(0);
            for (int g = 0; ok && g < total && !bars->abort_flag; ++g) {
                if (g + 1 < total && !issue_s(g + 1)) { ok = false; break; }
                const int uc = g / n_tiles, t = g - uc * n_tiles, w = g & 1, s = g % kStgB, qb = uc & 1;
                if (!mbar_wait(&bars->p_full[w], (g >> 1) & 1)) { fail(23); break; }
                // the accumulators are shared: the other warpgroup must have drained the previous tile
                if (g >= 1 && !mbar_wait(&bars->acc_free[(g - 1) & 1], ((g - 1) >> 1) & 1)) { fail(24); break; }
                if (t == 0 && uc >= 1 && !mbar_wait(&bars->dq_free, (uc - 1) & 1)) { fail(25); break; }
                tc_fence_after();
                const uint64_t qn = q_mn0 + (uint64_t)((qb * kQdBuf) >> 4);
                const uint64_t dn = qn + (uint64_t)(kQdTile >> 4);
#pragma unroll
                for (int kk = 0; kk < kNI / 16; ++kk)          // dY_tile = P^T dOut
                    mma_ts(tmem + kColDY, tmem + bc_s(w) + kk * 8, dn + ((kk * 2048) >> 4), idesc_o, kk > 0);
#pragma unroll
                for (int kk = 0; kk < kNI / 16; ++kk)          // daL_tile = (scale dS)^T Q
                    mma_ts(tmem + kColDaL, tmem + bc_dp(w) + kk * 8, qn + ((kk * 2048) >> 4), idesc_o, kk > 0);
                const uint64_t am = a_mn0 + (uint64_t)((s * kBStage) >> 4);
                const uint64_t dsd = ds0 + (uint64_t)((w * kDsTile) >> 4);
#pragma unroll
                for (int kk = 0; kk < kKB / 16; ++kk)          // dq^T (+)= aL_tile^T (scale dS)^T
                    mma_ss(tmem + kColDq, am + ((kk * 2048) >> 4), dsd + ((kk * 2048) >> 4), idesc_q, (t > 0 || kk > 0) ? 1u : 0u);
                mma_commit(&bars->acc_full[w]);
                mma_commit(&bars->sd_free[w]);
                mma_commit(&bars->a_empty[s]);
                if (t + 1 == n_tiles) { mma_commit(&bars->dq_full); mma_commit(&bars->q_empty[qb]); }
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ the two working warpgroups
        const int w = (warp - 4) >> 2;
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                       // TMEM lane: key within the tile (d for the dq drain)
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const float scale_l2 = p.scale * kLog2e;
        unsigned char* ds_row = ds_s + w * kDsTile + row * 128;
        for (int g = w; g < total && !bars->abort_flag; g += 2) {
            const int uc = g / n_tiles, t = g - uc * n_tiles, qb = uc & 1;
            const int u = u_begin + uc;
            const int key = t * kKB + row;
            const bool valid = key < n_keys;
            const float cl2 = valid ? kLog2e * p.cL[(long long)u * p.n_keys_c + key] : INFINITY;
            if (!mbar_wait(&bars->s_full[w], (g >> 1) & 1)) { fail(31); break; }
            tc_fence_after();
            uint32_t rs[kNI], rd[kNI];
            tmem_ld32(tmem + lane_sel + bc_s(w), rs);
            tmem_ld32(tmem + lane_sel + bc_dp(w), rd);
            tmem_wait_ld();
            const float* lse2 = bars->lse2[qb];
            const float* dlt = bars->delta[qb];
            float dsum = 0.f;
            uint32_t pp[kNI / 2], pd[kNI / 2];
#pragma unroll
            for (int c = 0; c < kNI; c += 2) {
                const float p0 = exp2f(fmaf(__uint_as_float(rs[c]), scale_l2, -(cl2 + lse2[c])));
                const float p1 = exp2f(fmaf(__uint_as_float(rs[c + 1]), scale_l2, -(cl2 + lse2[c + 1])));
                const float d0 = p0 * (__uint_as_float(rd[c]) - dlt[c]);
                const float d1 = p1 * (__uint_as_float(rd[c + 1]) - dlt[c + 1]);
                dsum += d0 + d1;
                pp[c >> 1] = pack_bf16(p0, p1);
                pd[c >> 1] = pack_bf16(d0 * p.scale, d1 * p.scale);
            }
            tmem_st16b(tmem + lane_sel + bc_s(w), pp);
            tmem_st16b(tmem + lane_sel + bc_dp(w), pd);
            // bf16 copy of this key's (scale dS) row for the dq GEMM: 64 bytes of data, 128-byte swizzled row
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4*>(ds_row + ((c ^ (row & 7)) << 4)) = make_uint4(pd[4 * c], pd[4 * c + 1], pd[4 * c + 2], pd[4 * c + 3]);
            fence_async_smem();
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&bars->p_full[w]);
            if (valid) p.dcL[(long long)u * p.n_keys_c + key] = -dsum;

            // ---- drain dY and daL of this tile: one 256-byte row each, written over Y and aL
            if (!mbar_wait(&bars->acc_full[w], (g >> 1) & 1)) { fail(41); break; }
            tc_fence_after();
            const long long ro = ((long long)u * n_keys + key) * kHeadDim;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                __nv_bfloat16* dst = (half ? p.Y : p.aL) + ro;
                const uint32_t col0 = half ? kColDY : kColDaL;
#pragma unroll 1
                for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem + lane_sel + col0 + c0, r);
                    tmem_wait_ld();
                    if (half == 1 && c0 + 32 == kHeadDim) {
                        tc_fence_before();
                        mbar_arrive(&bars->acc_free[w]);
                    }
                    if (valid) {
#pragma unroll
                        for (int v8 = 0; v8 < 2; ++v8) {
                            uint32_t wv[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                wv[e] = pack_bf16(__uint_as_float(r[v8 * 16 + 2 * e]), __uint_as_float(r[v8 * 16 + 2 * e + 1]));
                            stg_v8(dst + c0 + v8 * 16, wv);
                        }
                    }
                }
            }
            // ---- last tile of the slab: its dq (TMEM lane = d, column = query row)
            if (t + 1 == n_tiles) {
                if (!mbar_wait(&bars->dq_full, uc & 1)) { fail(42); break; }
                tc_fence_after();
                uint32_t r[kNI];
                tmem_ld32(tmem + lane_sel + kColDq, r);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(&bars->dq_free);
                const BUnit un = b_decode(p, u);
                const int bh = p.bh0 + un.bhl, b = bh / p.H, hd = bh - b * p.H;
#pragma unroll 1
                for (int i = 0; i < b1; ++i) {
                    const long long tok = blk.row_token(un.a, i) + un.j;
                    p.dq[(((long long)b * p.n_q + tok) * p.H + hd) * kHeadDim + row] = __uint_as_float(r[i]);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemColsB);
}

// delta[b, token, head] = sum_d dOut * out.  One warp per (token, head) row.
__global__ void __launch_bounds__(256) bwd_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                                        float* __restrict__ delta, long long rows) {
    const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint2 a = *reinterpret_cast<const uint2*>(dout + r * kHeadDim + lane * 4);
    const uint2 b = *reinterpret_cast<const uint2*>(out + r * kHeadDim + lane * 4);
    const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
    const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
    const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
    const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
    float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) delta[r] = s;
}

}  // namespace

int launch_bwd_delta(const void* dout, const void* out, float* delta, long long rows, cudaStream_t s) {
    LaunchScope scope(kClsBackward, s);
    bwd_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, delta, rows);
    return (int)cudaGetLastError();
}

// Column-step backward for one slice of (batch, head) pairs.  maps = {aL bridge, Y bridge, q rows, dOut rows}.
int launch_bwd_col_tc(const MonarchParams& mp, const CUtensorMap* maps, const float* delta, float* dcL, float* dq,
                      int* status, int num_sms, cudaStream_t s) {
    if (mp.blk.b1 > kNI) return SFM_ERR_UNSUPPORTED;
    LaunchScope scope(kClsBackward, s);
    BwdColParams p;
    p.q = mp.q; p.q_bs = mp.q_bs; p.delta = delta; p.lse = mp.lse;
    p.aL = mp.aL; p.Y = mp.Y; p.cL = mp.cL; p.dcL = dcL; p.dq = dq;
    p.H = mp.H; p.n_q = mp.n_q; p.A = mp.na; p.n_keys = mp.n_keys; p.n_keys_c = mp.n_keys_c;
    p.bh0 = mp.bh0; p.nbh = mp.nbh;
    p.n_units = mp.nbh * mp.na * mp.blk.b2;
    p.R4 = (mp.blk.b1 + 3) / 4;
    p.q_rows_tma = (mp.blk.f_tied == 1 || mp.blk.h_reduce == 1) ? 1 : 0;
    if (!p.q_rows_tma) return SFM_ERR_UNSUPPORTED;
    p.scale = mp.scale;
    p.blk = mp.blk;
    p.status = status;
    dim3 grid(p.n_units < num_sms ? p.n_units : num_sms);
    cudaError_t e = cudaFuncSetAttribute(monarch_bwd_col_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBSmemBytes);
    if (e != cudaSuccess) return (int)e;
    monarch_bwd_col_tc_kernel<<<grid, kThreadsB, kBSmemBytes, s>>>(maps[0], maps[1], maps[2], maps[3], p);
    return (int)cudaGetLastError();
}

}  // namespace sfm
