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
// The KEYS sit on the M side of the tensor core (TMEM lane = key), the slab's queries on the N side in chunks of
// 32 rows (NC = 1, 2 or 3 chunks: block rows up to 96), so that dY, daL and dcL come out one key per lane, ready
// for row-wise stores.  Per (key tile, chunk of query rows):
//   S^T  = aL_tile Q^T,  dP^T = Y_tile dOut^T               two tcgen05.mma, operands in shared memory
//   P^T, (scale dS)^T as bf16 over the S^T / dP^T columns     one thread per key; dcL from its registers
//   dY_tile = P^T dOut,  daL_tile = (scale dS)^T Q            A from TMEM, B = the query-side rows, MN-major
//   dq^T (+)= aL_tile^T (scale dS)^T                          A = the aL tile read MN-major, B = a bf16 copy of
//                                                             (scale dS)^T in shared memory; accumulates over the slab
// dY and daL accumulate over the chunks of a tile in TMEM, dq^T has 32 columns per chunk and accumulates over the
// tiles.  dY and daL are written over Y and aL in place (a tile is in shared memory before its rows are overwritten).
//
// Warp roles (12 warps): 0 = TMA producer, 1 = MMA issuer (owns TMEM), 2-3 idle, 4-7 and 8-11 = two warpgroups
// that take even / odd (tile, chunk) steps (element-wise pass; the group that had a tile's last chunk then drains
// the dY / daL accumulators and adds up dcL, and after a slab's last tile stores its dq).  Persistent CTAs over contiguous shares of the slab list.
// All waits are bounded and report through the status word.
//
// Stands in for the Triton kernel _z_bwd and its preprocess (wan/modules/monarch_attn.py:852-886, 1034-1222).
#include <algorithm>

#include "monarch_params.cuh"
#include "profile.cuh"
#include "tc05.cuh"

namespace sfm {

using namespace tc;

namespace {

constexpr int kStgB = 2;                     // (aL, Y) tile-pair ring
constexpr int kThreadsB = 384;
constexpr int kKB = 128;                     // keys per tile
constexpr int kNI = 32;                      // query rows per chunk
constexpr int kMaxNC = 3;                    // chunks per slab: block rows up to 96
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
    int q_rows_tma;
    int q_box_rows;                // rows per box of the q / dOut row maps (32, or all the grid rows there are)
    float scale;
    Blocking blk;
    int* status;
};

constexpr int kQdHalf = kNI * 128;                 // one 64-column half of a query-side tile (32 rows)
constexpr int kQdTile = 2 * kQdHalf;               // 8 KB
constexpr int kQdBuf = 2 * kQdTile;                // q rows + dOut rows of one chunk
constexpr int kBTile = 2 * kKB * 128;              // one aL or Y tile, 32 KB
constexpr int kBStage = 2 * kBTile;                // aL + Y
constexpr int kDsTile = kKB * 128;                 // (scale dS)^T copy: 128 keys x 64 bf16, 16 KB

struct __align__(16) BBarriers {
    float lse2[2][kMaxNC * kNI];
    float delta[2][kMaxNC * kNI];
    float dsum[2][kMaxNC][kKB];             // [tile parity][chunk][key]: -dcL shares of the chunks
    uint64_t q_full[2], q_empty[2];
    uint64_t a_full[kStgB], a_empty[kStgB];
    uint64_t s_full[2], p_full[2], sd_free[2];
    uint64_t acc_full[2], acc_free[2];      // per warpgroup: a parity wait may lag its barrier by one phase only
    uint64_t dq_full, dq_free;
    uint32_t tmem_base;
    volatile int abort_flag;
};

// query-side buffers: two slabs of one chunk (the next slab's rows load while this one is worked on), or one slab of NC
__host__ __device__ constexpr int qd_bytes(int nc) { return (nc == 1 ? 2 : nc) * kQdBuf; }
__host__ __device__ constexpr int b_smem_bytes(int nc) {
    return 1024 + qd_bytes(nc) + kStgB * kBStage + 2 * kDsTile + (int)sizeof(BBarriers) + 64;
}

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

// tal / ty = bridge maps (box 64 x 128 keys x 1); tqr / tdo = query rows of q / dOut (5-D, box of 32 rows).
template <int NC>
__global__ void __launch_bounds__(kThreadsB, 1)
monarch_bwd_col_tc_kernel(const __grid_constant__ CUtensorMap tal, const __grid_constant__ CUtensorMap ty,
                          const __grid_constant__ CUtensorMap tqr, const __grid_constant__ CUtensorMap tdo,
                          BwdColParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* qd_s = base;                                   // [slab buffer][chunk][q rows | dOut rows]
    unsigned char* a_s = qd_s + qd_bytes(NC);                      // [stage][aL tile | Y tile]
    unsigned char* ds_s = a_s + kStgB * kBStage;                   // [warpgroup] (scale dS)^T, 128 rows of 128 bytes
    BBarriers* bars = reinterpret_cast<BBarriers*>(ds_s + 2 * kDsTile);

    const Blocking& blk = p.blk;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b1 = blk.b1;
    const int n_keys = p.n_keys;
    const int n_tiles = (n_keys + kKB - 1) / kKB;
    const int u_begin = (int)((long long)p.n_units * blockIdx.x / gridDim.x);
    const int u_end = (int)((long long)p.n_units * (blockIdx.x + 1) / gridDim.x);
    const int total = (u_end - u_begin) * n_tiles * NC;            // (slab, tile, chunk) steps of this CTA
    constexpr int kQBufs = NC == 1 ? 2 : 1;

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
    for (int i = tid; i < qd_bytes(NC) / 16; i += kThreadsB) reinterpret_cast<uint4*>(qd_s)[i] = make_uint4(0, 0, 0, 0);
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
        int g = 0, uc = 0;                                       // tiles loaded, slabs started
        bool ok = true;
        for (int u = u_begin; ok && u < u_end && !bars->abort_flag; ++u, ++uc) {
            const BUnit un = b_decode(p, u);
            const int bh = p.bh0 + un.bhl, b = bh / p.H, hd = bh - b * p.H;
            const int qb = kQBufs == 2 ? (uc & 1) : 0;
            unsigned char* qt = qd_s + qb * kQdBuf;
            auto load_tiles = [&](int t_begin, int t_end) {      // lane 0 only
                for (int t = t_begin; t < t_end; ++t, ++g) {
                    const int s = g % kStgB;
                    if (g >= kStgB && !mbar_wait(&bars->a_empty[s], ((g / kStgB) - 1) & 1)) { fail(11); ok = false; break; }
                    unsigned char* st = a_s + s * kBStage;
                    mbar_arrive_expect_tx(&bars->a_full[s], (uint32_t)kBStage);
                    tma_load_3d(st, &tal, &bars->a_full[s], 0, t * kKB, u);
                    tma_load_3d(st + kKB * 128, &tal, &bars->a_full[s], 64, t * kKB, u);
                    tma_load_3d(st + kBTile, &ty, &bars->a_full[s], 0, t * kKB, u);
                    tma_load_3d(st + kBTile + kKB * 128, &ty, &bars->a_full[s], 64, t * kKB, u);
                }
            };
            // the slab's first tile does not wait for the query-side buffer
            if (lane == 0) load_tiles(0, 1);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (uc >= kQBufs) {
                int okw = 1;
                if (lane == 0) okw = mbar_wait(&bars->q_empty[qb], ((uc / kQBufs) - 1) & 1) ? 1 : 0;
                if (!__shfl_sync(0xffffffffu, okw, 0)) { fail(10); break; }
            }
            for (int i = lane; i < NC * kNI; i += 32) {
                float l2 = INFINITY, dl = 0.f;
                if (i < b1) {
                    const long long tok = blk.row_token(un.a, i) + un.j;
                    l2 = kLog2e * p.lse[(long long)u * b1 + i];
                    dl = p.delta[((long long)b * p.n_q + tok) * p.H + hd];
                }
                bars->lse2[qb][i] = l2;
                bars->delta[qb][i] = dl;
            }
            __syncwarp();
            if (lane == 0) {
                // 32 consecutive rows of the token grid per chunk; rows past the slab's b1 hold other tokens (or the
                // fill value) and are masked by an infinite log-sum-exp
                mbar_arrive_expect_tx(&bars->q_full[qb], (uint32_t)(NC * 4 * p.q_box_rows * 128));
                const int tok0 = blk.row_token(un.a, 0);
                const int frow0 = tok0 / blk.w, col = tok0 - frow0 * blk.w + un.j;
                for (int c = 0; c < NC; ++c) {
                    unsigned char* dq_ = qt + c * kQdBuf;
                    tma_load_5d(dq_, &tqr, &bars->q_full[qb], 0, hd, col, frow0 + c * kNI, b);
                    tma_load_5d(dq_ + kQdHalf, &tqr, &bars->q_full[qb], 64, hd, col, frow0 + c * kNI, b);
                    tma_load_5d(dq_ + kQdTile, &tdo, &bars->q_full[qb], 0, hd, col, frow0 + c * kNI, b);
                    tma_load_5d(dq_ + kQdTile + kQdHalf, &tdo, &bars->q_full[qb], 64, hd, col, frow0 + c * kNI, b);
                }
                load_tiles(1, n_tiles);
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
            // step g = ((slab, tile), chunk); its warpgroup is g & 1
            auto issue_s = [&](int g) -> bool {
                const int gt = g / NC, c = g - gt * NC;
                const int uc = gt / n_tiles, t = gt - uc * n_tiles, w = g & 1, s = gt % kStgB;
                const int qb = kQBufs == 2 ? (uc & 1) : 0;
                if (t == 0 && c == 0 && !mbar_wait(&bars->q_full[qb], (uc / kQBufs) & 1)) { fail(20); return false; }
                if (c == 0 && !mbar_wait(&bars->a_full[s], (gt / kStgB) & 1)) { fail(21); return false; }
                if (g >= 2 && !mbar_wait(&bars->sd_free[w], ((g >> 1) - 1) & 1)) { fail(22); return false; }
                tc_fence_after();
                const uint64_t al = a_k0 + (uint64_t)((s * kBStage) >> 4);
                const uint64_t yy = al + (uint64_t)(kBTile >> 4);
                const uint64_t qq = q_k0 + (uint64_t)(((qb + c) * kQdBuf) >> 4);
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
            int drains[2] = {0, 0};               // accumulator hand-overs to each warpgroup so far
            int last_drainer = 0;
            if (total > 0) ok = issue_s(0);
            for (int g = 0; ok && g < total && !bars->abort_flag; ++g) {
                // The S GEMMs of the next step are issued ahead of this step's, except across a slab boundary when the
                // query-side rows are single buffered: the next slab's rows can only load once this slab's last
                // GEMMs have released the buffer, so waiting for them here would never end.
                const bool ahead = g + 1 < total && !(kQBufs == 1 && (g + 1) % (n_tiles * NC) == 0);
                if (ahead && !issue_s(g + 1)) { ok = false; break; }
                const int gt = g / NC, c = g - gt * NC;
                const int uc = gt / n_tiles, t = gt - uc * n_tiles, w = g & 1, s = gt % kStgB;
                const int qb = kQBufs == 2 ? (uc & 1) : 0;
                if (!mbar_wait(&bars->p_full[w], (g >> 1) & 1)) { fail(23); break; }
                // the accumulators are shared by all tiles: the previous tile's must have been drained
                if (c == 0 && gt >= 1 && !mbar_wait(&bars->acc_free[last_drainer], (drains[last_drainer] - 1) & 1)) { fail(24); break; }
                if (t == 0 && c == 0 && uc >= 1 && !mbar_wait(&bars->dq_free, (uc - 1) & 1)) { fail(25); break; }
                tc_fence_after();
                const uint64_t qn = q_mn0 + (uint64_t)(((qb + c) * kQdBuf) >> 4);
                const uint64_t dn = qn + (uint64_t)(kQdTile >> 4);
#pragma unroll
                for (int kk = 0; kk < kNI / 16; ++kk)          // dY_tile (+)= P^T dOut
                    mma_ts(tmem + kColDY, tmem + bc_s(w) + kk * 8, dn + ((kk * 2048) >> 4), idesc_o, (c > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < kNI / 16; ++kk)          // daL_tile (+)= (scale dS)^T Q
                    mma_ts(tmem + kColDaL, tmem + bc_dp(w) + kk * 8, qn + ((kk * 2048) >> 4), idesc_o, (c > 0 || kk > 0) ? 1u : 0u);
                const uint64_t am = a_mn0 + (uint64_t)((s * kBStage) >> 4);
                const uint64_t dsd = ds0 + (uint64_t)((w * kDsTile) >> 4);
                // dq^T of chunk c (+)= aL_tile^T (scale dS)^T: 64 output columns of which the upper 32 receive zeros
                // (and, on a slab's first tile, are set to zero before the next chunk sets its own)
#pragma unroll
                for (int kk = 0; kk < kKB / 16; ++kk)
                    mma_ss(tmem + kColDq + c * kNI, am + ((kk * 2048) >> 4), dsd + ((kk * 2048) >> 4), idesc_q, (t > 0 || kk > 0) ? 1u : 0u);
                if (c == NC - 1) {
                    mma_commit(&bars->acc_full[w]);
                    ++drains[w];
                    last_drainer = w;
                    mma_commit(&bars->a_empty[s]);
                }
                mma_commit(&bars->sd_free[w]);
                if (t + 1 == n_tiles && c == NC - 1) { mma_commit(&bars->dq_full); mma_commit(&bars->q_empty[qb]); }
                if (g + 1 < total && !ahead && !issue_s(g + 1)) { ok = false; break; }
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
        int my_drains = 0;
        for (int g = w; g < total && !bars->abort_flag; g += 2) {
            const int gt = g / NC, c = g - gt * NC;
            const int uc = gt / n_tiles, t = gt - uc * n_tiles;
            const int qb = kQBufs == 2 ? (uc & 1) : 0;
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
            const float* lse2 = bars->lse2[qb] + c * kNI;
            const float* dlt = bars->delta[qb] + c * kNI;
            float dsum = 0.f;
            uint32_t pp[kNI / 2], pd[kNI / 2];
#pragma unroll
            for (int cc = 0; cc < kNI; cc += 2) {
                const float p0 = exp2f(fmaf(__uint_as_float(rs[cc]), scale_l2, -(cl2 + lse2[cc])));
                const float p1 = exp2f(fmaf(__uint_as_float(rs[cc + 1]), scale_l2, -(cl2 + lse2[cc + 1])));
                const float d0 = p0 * (__uint_as_float(rd[cc]) - dlt[cc]);
                const float d1 = p1 * (__uint_as_float(rd[cc + 1]) - dlt[cc + 1]);
                dsum += d0 + d1;
                pp[cc >> 1] = pack_bf16(p0, p1);
                pd[cc >> 1] = pack_bf16(d0 * p.scale, d1 * p.scale);
            }
            tmem_st16b(tmem + lane_sel + bc_s(w), pp);
            tmem_st16b(tmem + lane_sel + bc_dp(w), pd);
            // bf16 copy of this key's (scale dS) row for the dq GEMM: 64 bytes of data, 128-byte swizzled row
#pragma unroll
            for (int cc = 0; cc < 4; ++cc)
                *reinterpret_cast<uint4*>(ds_row + ((cc ^ (row & 7)) << 4)) = make_uint4(pd[4 * cc], pd[4 * cc + 1], pd[4 * cc + 2], pd[4 * cc + 3]);
            bars->dsum[gt & 1][c][row] = dsum;
            fence_async_smem();
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&bars->p_full[w]);
            if (c != NC - 1) continue;

            // ---- the tile's last chunk: drain dY and daL, one 256-byte row each, written over Y and aL
            if (!mbar_wait(&bars->acc_full[w], my_drains & 1)) { fail(41); break; }
            ++my_drains;
            tc_fence_after();
            if (valid) {
                float acc = 0.f;                     // the chunks' shares in a fixed order
#pragma unroll
                for (int cc = 0; cc < NC; ++cc) acc += bars->dsum[gt & 1][cc][row];
                p.dcL[(long long)u * p.n_keys_c + key] = -acc;
            }
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
                uint32_t r[NC][kNI];
#pragma unroll
                for (int cc = 0; cc < NC; ++cc) tmem_ld32(tmem + lane_sel + kColDq + cc * kNI, r[cc]);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(&bars->dq_free);
                const BUnit un = b_decode(p, u);
                const int bh = p.bh0 + un.bhl, b = bh / p.H, hd = bh - b * p.H;
#pragma unroll
                for (int cc = 0; cc < NC; ++cc) {
#pragma unroll
                    for (int ii = 0; ii < kNI; ++ii) {
                        const int i = cc * kNI + ii;
                        if (i < b1) {
                            const long long tok = blk.row_token(un.a, i) + un.j;
                            p.dq[(((long long)b * p.n_q + tok) * p.H + hd) * kHeadDim + row] = __uint_as_float(r[cc][ii]);
                        }
                    }
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

// Column-step backward for one slice of (batch, head) pairs.  maps = {aL bridge, Y bridge, q rows, dOut rows}; the
// two row maps are 5-D (d, head, column, row of the token grid, batch) with boxes of 32 rows.
int launch_bwd_col_tc(const MonarchParams& mp, const CUtensorMap* maps, const float* delta, float* dcL, float* dq,
                      int* status, int num_sms, cudaStream_t s) {
    if (mp.blk.b1 > kMaxNC * kNI) return SFM_ERR_UNSUPPORTED;
    LaunchScope scope(kClsBackward, s);
    BwdColParams p;
    p.q = mp.q; p.q_bs = mp.q_bs; p.delta = delta; p.lse = mp.lse;
    p.aL = mp.aL; p.Y = mp.Y; p.cL = mp.cL; p.dcL = dcL; p.dq = dq;
    p.H = mp.H; p.n_q = mp.n_q; p.A = mp.na; p.n_keys = mp.n_keys; p.n_keys_c = mp.n_keys_c;
    p.bh0 = mp.bh0; p.nbh = mp.nbh;
    p.n_units = mp.nbh * mp.na * mp.blk.b2;
    p.q_box_rows = std::min(32, mp.n_q / mp.blk.w);
    p.q_rows_tma = (mp.blk.f_tied == 1 || mp.blk.h_reduce == 1) ? 1 : 0;
    if (!p.q_rows_tma) return SFM_ERR_UNSUPPORTED;
    p.scale = mp.scale;
    p.blk = mp.blk;
    p.status = status;
    dim3 grid(p.n_units < num_sms ? p.n_units : num_sms);
    const int nc = (mp.blk.b1 + kNI - 1) / kNI;
    auto go = [&](auto kernel, int smem) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        kernel<<<grid, kThreadsB, smem, s>>>(maps[0], maps[1], maps[2], maps[3], p);
        return 0;
    };
    int rc = nc == 1 ? go(monarch_bwd_col_tc_kernel<1>, b_smem_bytes(1))
                     : (nc == 2 ? go(monarch_bwd_col_tc_kernel<2>, b_smem_bytes(2)) : go(monarch_bwd_col_tc_kernel<3>, b_smem_bytes(3)));
    if (rc) return rc;
    return (int)cudaGetLastError();
}

}  // namespace sfm
