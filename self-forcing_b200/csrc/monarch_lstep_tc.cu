// Monarch column step, and dense attention, on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Column step.  One unit = (batch*head, query group a, column j): the b1 queries Q[a,:,j] attend the
// n_keys = F*b1 summary keys aL[a,f,j,k] (bias -cL, values Y) produced by the row step.  The MMA tile
// is 128 rows tall but a unit has only b1 queries (30 at 480p framewise), so a CTA works on a GROUP
// of U = floor(32 / ceil(b1/4)) consecutive units at once: query i of unit slot u sits on tile row
// (i / R4)*32 + u*R4 + i % R4 with R4 = ceil(b1/4), i.e. every TMEM lane quadrant carries R4 rows of
// every unit.  Keys stream through shared memory in tiles of 128 per unit:
//   S  = Q_tile aL_tile(u)^T        tcgen05.mma with a lane mask that only updates unit u's rows
//   P  = exp2(scale*S - cL - m)     one thread per tile row, running max / sum in registers
//   O += P Y_tile(u)                tcgen05.mma, A = P (bf16) from TMEM, same lane mask
// Even and odd key tiles go to two softmax warpgroups with their own S/P buffer and accumulator
// (split-KV); the epilogue warpgroup merges the two partial softmaxes, normalises and writes each
// row to natural token order with 32-byte stores (the inverse layout map is the store address).
//
// Dense attention (kDense = true): a unit is 128 consecutive queries of one (batch, head), U = 1, key /
// value tiles come straight from the KV cache, there is no bias and no lane mask.
//
// Warp roles (16 warps): 0 = key-side producer (queries, aL tiles, bias slices), 3 = value-tile
// producer, 1 = PV-GEMM issuer (owns the TMEM allocation), 2 = S-GEMM issuer, 4..7 / 8..11 = softmax
// warpgroups, 12..15 = epilogue warpgroup.  All roles run the same loops and meet only through
// mbarriers with bounded waits; a timeout records a status code and the CTA unwinds.
//
// Arithmetic follows monarch_attn_ref_op (wan/modules/monarch_attn.py:1821-1829) and, for the dense
// instantiation, softmax(q k^T * scale) v (wan/modules/attention.py:177-187).
#include "monarch_params.cuh"
#include "profile.cuh"
#include "tc05.cuh"

namespace sfm {

using namespace tc;

namespace {

constexpr int kAStages = 2;    // key (aL) tile ring, released as soon as the S GEMM has read a tile
constexpr int kYStages = 3;    // value (Y) tile ring, released after the PV GEMM
constexpr int kThreads = 512;
constexpr int kKT = 128;                   // keys per tile
constexpr int kMaxU = 8;                   // units per group (the bias ring is sized for it)
constexpr uint32_t kTmemCols = 512;
// TMEM columns: S / P buffers of the two softmax warpgroups at 0 and 128, their accumulators at 256 and 384
__host__ __device__ constexpr uint32_t col_s(int w) { return (uint32_t)w * 128u; }
__host__ __device__ constexpr uint32_t col_o(int w) { return 256u + (uint32_t)w * 128u; }
constexpr float kRescaleThreshold = 8.0f;  // log2 units: accumulators are rescaled only past this growth

struct LTcParams {
    MonarchParams mp;
    int n_units;     // column step: nbh * na * b2;  dense: B*H * ceil(n_q / 128)
    int U;           // units per group
    int R4;          // tile rows per unit per lane quadrant
    int q_rows_tma;  // the query rows of a unit are consecutive rows of the token grid: load them with TMA
    int n_kv;        // dense: keys per (batch, head)
    int q_tiles;     // dense: ceil(n_q / 128)
    int write_lse;   // column step: also store the log-sum-exp of every query row (iterative variant)
    int lse_only;    // column step: nothing but that (no value tiles, no PV GEMMs, no output rows)
    int* status;
};


struct __align__(16) Barriers {
    alignas(16) float cl[4][kMaxU][kKT];   // bias slices, per unit slot: two ring slots for each softmax warpgroup
    float stats[2][2][128];                // [warpgroup][m | l][tile row]
    uint64_t q_full, q_empty;
    uint64_t a_full[kAStages], a_empty[kAStages];
    uint64_t y_full[kYStages], y_empty[kYStages];
    uint64_t cl_full[4], cl_empty[4];
    uint64_t s_full[4], p_full[4], sp_free[4];   // [warpgroup * 2 + half]: dense attention works on 64-key halves of a tile
    uint64_t pv_done[2];                   // all PV GEMMs issued so far into accumulator w have completed
    uint64_t o_full, o_free;
    uint32_t tmem_base;
    volatile int abort_flag;
};

constexpr int kQBytes = 2 * 128 * 128;     // query tile, two 64-column halves
constexpr int kTileBytes = 2 * kKT * 128;  // one key or value tile
constexpr int kSmemBytes = 1024 + kQBytes + (kAStages + kYStages) * kTileBytes + (int)sizeof(Barriers) + 64;

__device__ __forceinline__ void st_global_v8(void* ptr, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                 "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}
// tcgen05.mma with an output-lane mask: bit i of `dis` set = rows i, 32+i, 64+i, 96+i of D are NOT written.
__device__ __forceinline__ void mma_ss_masked(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accum, uint32_t dis) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accum), "r"(dis) : "memory");
}
__device__ __forceinline__ void mma_ts_masked(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accum, uint32_t dis) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accum), "r"(dis) : "memory");
}

struct LUnit { int bhl, al, j; };
__device__ __forceinline__ LUnit decode_unit(const MonarchParams& p, int u) {
    LUnit r;
    r.j = u % p.blk.b2; u /= p.blk.b2;
    r.al = u % p.na;
    r.bhl = u / p.na;
    return r;
}

// Column step: tal / ty = bridge aL / Y maps (box 64 x 128 keys x 1), tqr = query rows (5-D).
// Dense:       tal / ty = K / V cache maps (4-D, box 64 x 1 x 128 tokens x 1), tqr = q map (same geometry).
template <bool kDense, bool kCausal>
__global__ void __launch_bounds__(kThreads, 1)
monarch_l_tc_kernel(const __grid_constant__ CUtensorMap tal, const __grid_constant__ CUtensorMap ty,
                    const __grid_constant__ CUtensorMap tqr, LTcParams lp) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;
    unsigned char* a_s = q_s + kQBytes;
    unsigned char* y_s = a_s + kAStages * kTileBytes;
    Barriers* bars = reinterpret_cast<Barriers*>(y_s + kYStages * kTileBytes);

    const MonarchParams& p = lp.mp;
    const Blocking& blk = p.blk;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b1 = blk.b1, b2 = blk.b2;
    // Dense attention splits every 128-key tile into two 64-key halves with an S / P buffer each (64 columns), so that
    // the S GEMM of one half runs while the other half's softmax does; the column step, bound by its bridge reads,
    // keeps whole tiles.
    constexpr int kH = kDense ? 2 : 1;
    constexpr int kNS = kKT / kH;
    const int n_keys = kDense ? lp.n_kv : p.n_keys;
    const int n_tiles_all = (n_keys + kKT - 1) / kKT;
    // Key tiles a group of units has to walk.  Block-causal (no-cache path): the keys past the last cached
    // group any of the group's units may see carry an infinite bias, so the walk stops before them.
    auto group_tiles = [&](int u0, int nu) -> int {
        if (!kCausal) return n_tiles_all;
        int fmax = 0;
        for (int us = 0; us < nu; ++us) {
            const int a_abs = p.a0 + decode_unit(p, u0 + us).al;
            fmax = max(fmax, min(p.F, (a_abs / p.causal_groups + 1) * p.causal_groups));
        }
        return (fmax * b1 + kKT - 1) / kKT;
    };
    const long long tok_pitch = (long long)p.H * kHeadDim;
    const int U = lp.U, R4 = lp.R4;
    // this CTA's contiguous share of the unit list, walked in groups of at most U units
    // (dense: units are dealt round-robin instead, so that the CTAs running at the same time share keys in L2)
    const int u_begin = kDense ? (int)blockIdx.x : (int)((long long)lp.n_units * blockIdx.x / gridDim.x);
    const int u_end = kDense ? lp.n_units : (int)((long long)lp.n_units * (blockIdx.x + 1) / gridDim.x);
    const int u_step = kDense ? (int)gridDim.x : U;

    if (tid == 0) {
        mbar_init(&bars->q_full, 1);
        mbar_init(&bars->q_empty, 1);
        for (int s = 0; s < kAStages; ++s) { mbar_init(&bars->a_full[s], 1); mbar_init(&bars->a_empty[s], 1); }
        for (int s = 0; s < kYStages; ++s) { mbar_init(&bars->y_full[s], 1); mbar_init(&bars->y_empty[s], 1); }
        for (int w = 0; w < 2; ++w) {
            mbar_init(&bars->cl_full[w], 1); mbar_init(&bars->cl_full[w + 2], 1);
            mbar_init(&bars->cl_empty[w], 128); mbar_init(&bars->cl_empty[w + 2], 128);
            for (int hh = 0; hh < 2; ++hh) {
                mbar_init(&bars->s_full[2 * w + hh], 1); mbar_init(&bars->p_full[2 * w + hh], 128);
                mbar_init(&bars->sp_free[2 * w + hh], 1);
            }
            mbar_init(&bars->pv_done[w], 1);
        }
        mbar_init(&bars->o_full, 1);
        mbar_init(&bars->o_free, 128);
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    // rows of the query tile that no unit writes must still hold finite numbers
    for (int i = tid; i < kQBytes / 16; i += kThreads) reinterpret_cast<uint4*>(q_s)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 1) { tmem_alloc(&bars->tmem_base, kTmemCols); tmem_relinquish(); }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    // tile rows that belong to no unit are never written by a GEMM: give their logits a defined value
    if (warp >= 4 && warp < 12) {
        uint32_t z[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) z[c] = 0u;
        const uint32_t s_t = tmem + ((uint32_t)((warp & 3) * 32) << 16) + col_s((warp - 4) >> 2);
#pragma unroll 1
        for (int c0 = 0; c0 < kKT; c0 += 32) tmem_st32(s_t + c0, z);
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    auto fail = [&](int code) {
        bars->abort_flag = 1;
        atomicCAS(lp.status, 0, code);
    };
    // lane mask of unit slot u: only its R4 lanes of each quadrant are written
    auto dis_mask = [&](int u) -> uint32_t {
        if (kDense) return 0u;
        const uint32_t en = (R4 >= 32 ? 0xffffffffu : ((1u << R4) - 1u)) << (u * R4);
        return ~en;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ key-side producer
        if (lane == 0) { prefetch_tmap(&tal); prefetch_tmap(&tqr); }
        int ga = 0, gc = 0;                  // running counters: aL tiles, groups
        int cnt[2] = {0, 0};                 // tiles given to each softmax warpgroup so far
        bool ok = true;
        for (int u0 = u_begin; ok && u0 < u_end && !bars->abort_flag; u0 += u_step, ++gc) {
            const int nu = kDense ? 1 : min(U, u_end - u0);
            const int n_tiles = group_tiles(u0, nu);
            if (gc > 0) {
                int okw = 1;
                if (lane == 0) okw = mbar_wait(&bars->q_empty, (gc - 1) & 1) ? 1 : 0;
                if (!__shfl_sync(0xffffffffu, okw, 0)) { fail(10); break; }
            }
            // ---- queries of the group
            if (kDense) {
                if (lane == 0) {
                    const int qt = u0 % lp.q_tiles, bh = u0 / lp.q_tiles, b = bh / p.H, hd = bh - b * p.H;
                    mbar_arrive_expect_tx(&bars->q_full, (uint32_t)kQBytes);
                    tma_load_4d(q_s, &tqr, &bars->q_full, 0, hd, qt * 128, b);
                    tma_load_4d(q_s + 128 * 128, &tqr, &bars->q_full, 64, hd, qt * 128, b);
                }
            } else if (lp.q_rows_tma) {
                if (lane == 0) {
                    const int nq = (b1 + R4 - 1) / R4;                       // quadrants that hold rows
                    mbar_arrive_expect_tx(&bars->q_full, (uint32_t)(nu * nq * R4 * 256));
                    for (int us = 0; us < nu; ++us) {
                        const LUnit un = decode_unit(p, u0 + us);
                        const int bh = p.bh0 + un.bhl, b = bh / p.H, hd = bh - b * p.H;
                        const int tok0 = blk.row_token(p.a0 + un.al, 0);
                        const int frow0 = tok0 / blk.w, col = tok0 - frow0 * blk.w + un.j;
                        for (int qd = 0; qd < nq; ++qd) {
                            unsigned char* dst = q_s + (qd * 32 + us * R4) * 128;
                            tma_load_5d(dst, &tqr, &bars->q_full, 0, hd, col, frow0 + qd * R4, b);
                            tma_load_5d(dst + 128 * 128, &tqr, &bars->q_full, 64, hd, col, frow0 + qd * R4, b);
                        }
                    }
                }
            } else {
                for (int us = 0; us < nu; ++us) {
                    const LUnit un = decode_unit(p, u0 + us);
                    const int bh = p.bh0 + un.bhl, b = bh / p.H, hd = bh - b * p.H;
                    const __nv_bfloat16* qb = p.q + (long long)b * p.q_bs + (long long)hd * kHeadDim;
                    for (int idx = lane; idx < b1 * 16; idx += 32) {
                        const int i = idx >> 4, ch = idx & 15;
                        const uint4 val = *reinterpret_cast<const uint4*>(
                            qb + (blk.row_token(p.a0 + un.al, i) + un.j) * tok_pitch + ch * 8);
                        const int r = (i / R4) * 32 + us * R4 + (i % R4);
                        *reinterpret_cast<uint4*>(q_s + (ch >> 3) * (128 * 128) + r * 128 + (((ch & 7) ^ (r & 7)) << 4)) = val;
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->q_full);
            }
            // ---- per key tile: the bias slices of all units, then each unit's aL tile
            for (int t = 0; ok && t < n_tiles; ++t) {
                const int w = t & 1;
                const int idx = cnt[w]++;
                const int gt = cnt[0] + cnt[1] - 1;
                if (!kDense) {
                    // ring slot: two per softmax warpgroup, released by its threads after their last read
                    const int cslot = w + 2 * (idx & 1);
                    int okw = 1;
                    if (lane == 0 && idx >= 2) okw = mbar_wait(&bars->cl_empty[cslot], ((idx >> 1) - 1) & 1) ? 1 : 0;
                    if (!__shfl_sync(0xffffffffu, okw, 0)) { fail(13); ok = false; break; }
                    const int have = min(kKT, p.n_keys_c - t * kKT);            // floats that exist (multiple of 4)
                    if (have < kKT) {                                            // the rest masks its keys
                        for (int us = 0; us < nu; ++us)
                            for (int e = have + lane; e < kKT; e += 32) bars->cl[cslot][us][e] = INFINITY;
                        __syncwarp();
                    }
                    if (lane == 0) {
                        mbar_arrive_expect_tx(&bars->cl_full[cslot], (uint32_t)(nu * have * 4));
                        for (int us = 0; us < nu; ++us) {
                            const LUnit un = decode_unit(p, u0 + us);
                            const long long aj = ((long long)un.bhl * p.na + un.al) * b2 + un.j;
                            bulk_load(bars->cl[cslot][us], p.cL + aj * p.n_keys_c + t * kKT, (uint32_t)(have * 4), &bars->cl_full[cslot]);
                        }
                    }
                }
                for (int us = 0; us < nu; ++us, ++ga) {
                    const int sa = ga % kAStages;
                    int okw = 1;
                    if (lane == 0 && ga >= kAStages) okw = mbar_wait(&bars->a_empty[sa], ((ga / kAStages) - 1) & 1) ? 1 : 0;
                    if (!__shfl_sync(0xffffffffu, okw, 0)) { fail(11); ok = false; break; }
                    if (lane == 0) {
                        unsigned char* at = a_s + sa * kTileBytes;
                        mbar_arrive_expect_tx(&bars->a_full[sa], (uint32_t)kTileBytes);
                        if (kDense) {
                            const int bh = u0 / lp.q_tiles, b = bh / p.H, hd = bh - b * p.H;
                            tma_load_4d(at, &tal, &bars->a_full[sa], 0, hd, t * kKT, b);
                            tma_load_4d(at + kKT * 128, &tal, &bars->a_full[sa], 64, hd, t * kKT, b);
                        } else {
                            const LUnit un = decode_unit(p, u0 + us);
                            const int aj = (un.bhl * p.na + un.al) * b2 + un.j;
                            tma_load_3d(at, &tal, &bars->a_full[sa], 0, t * kKT, aj);
                            tma_load_3d(at + kKT * 128, &tal, &bars->a_full[sa], 64, t * kKT, aj);
                        }
                    }
                }
            }
        }
    } else if (warp == 3) {
        // ------------------------------------------------------------------ value-tile producer
        if (lane == 0 && !lp.lse_only) {
            prefetch_tmap(&ty);
            int gy = 0;
            bool ok = true;
            for (int u0 = u_begin; ok && u0 < u_end && !bars->abort_flag; u0 += u_step) {
                const int nu = kDense ? 1 : min(U, u_end - u0);
            const int n_tiles = group_tiles(u0, nu);
                for (int t = 0; ok && t < n_tiles; ++t)
                    for (int us = 0; us < nu; ++us, ++gy) {
                        const int sy = gy % kYStages;
                        if (gy >= kYStages && !mbar_wait(&bars->y_empty[sy], ((gy / kYStages) - 1) & 1)) { fail(12); ok = false; break; }
                        unsigned char* yt = y_s + sy * kTileBytes;
                        mbar_arrive_expect_tx(&bars->y_full[sy], (uint32_t)kTileBytes);
                        if (kDense) {
                            const int bh = u0 / lp.q_tiles, b = bh / p.H, hd = bh - b * p.H;
                            tma_load_4d(yt, &ty, &bars->y_full[sy], 0, hd, t * kKT, b);
                            tma_load_4d(yt + kKT * 128, &ty, &bars->y_full[sy], 64, hd, t * kKT, b);
                        } else {
                            const LUnit un = decode_unit(p, u0 + us);
                            const int aj = (un.bhl * p.na + un.al) * b2 + un.j;
                            tma_load_3d(yt, &ty, &bars->y_full[sy], 0, t * kKT, aj);
                            tma_load_3d(yt + kKT * 128, &ty, &bars->y_full[sy], 64, t * kKT, aj);
                        }
                    }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ S-GEMM issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16(128, kNS, 0, 0);
            const uint64_t q_desc = smem_desc_sw128(smem_addr(q_s), 16, 1024);
            const uint64_t a_desc0 = smem_desc_sw128(smem_addr(a_s), 16, 1024);
            int ga = 0, gc = 0, cnt[2] = {0, 0};
            bool ok = true;
            for (int u0 = u_begin; ok && u0 < u_end && !bars->abort_flag; u0 += u_step, ++gc) {
                const int nu = kDense ? 1 : min(U, u_end - u0);
            const int n_tiles = group_tiles(u0, nu);
                if (!mbar_wait(&bars->q_full, gc & 1)) { fail(20); break; }
                for (int t = 0; ok && t < n_tiles; ++t) {
                    const int w = t & 1;
                    const int idx = cnt[w]++;
                    const int gt = cnt[0] + cnt[1] - 1;
                    if (!kDense && idx >= 1 && !mbar_wait(&bars->sp_free[2 * w], (idx - 1) & 1)) { fail(25); ok = false; break; }
                    for (int us = 0; us < nu; ++us, ++ga) {
                        const int sa = ga % kAStages;
                        if (!mbar_wait(&bars->a_full[sa], (ga / kAStages) & 1)) { fail(21); ok = false; break; }
                        tc_fence_after();
                        const uint64_t ad = a_desc0 + (uint64_t)((sa * kTileBytes) >> 4);
                        const uint32_t dis = dis_mask(us);
                        if (kDense) {
                            for (int hh = 0; hh < 2; ++hh) {                   // keys [64 hh, 64 hh + 64) of the tile
                                if (idx >= 1 && !mbar_wait(&bars->sp_free[2 * w + hh], (idx - 1) & 1)) { fail(25); ok = false; break; }
                                tc_fence_after();
#pragma unroll
                                for (int ks = 0; ks < 8; ++ks) {
                                    const uint32_t off = ((ks >> 2) * (128 * 128) + (ks & 3) * 32) >> 4;
                                    mma_ss(tmem + col_s(w) + hh * kNS, q_desc + off, ad + off + (uint32_t)((hh * kNS * 128) >> 4), idesc_s, ks > 0);
                                }
                                mma_commit(&bars->s_full[2 * w + hh]);
                            }
                            if (!ok) break;
                        } else {
#pragma unroll
                            for (int ks = 0; ks < 8; ++ks) {
                                const uint32_t off = ((ks >> 2) * (128 * 128) + (ks & 3) * 32) >> 4;   // same geometry for both tiles
                                mma_ss_masked(tmem + col_s(w), q_desc + off, ad + off, idesc_s, ks > 0, dis);
                            }
                        }
                        mma_commit(&bars->a_empty[sa]);
                    }
                    if (!ok) break;
                    if (!kDense) mma_commit(&bars->s_full[2 * w]);
                    if (t + 1 == n_tiles) mma_commit(&bars->q_empty);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ PV-GEMM issuer
        if (lane == 0) {
            constexpr uint32_t idesc_o = idesc_bf16(128, kHeadDim, 0, 1);
            const uint64_t y_desc0 = smem_desc_sw128(smem_addr(y_s), kKT * 128, 1024);
            int gy = 0, gc = 0, cnt[2] = {0, 0};
            bool ok = true;
            for (int u0 = u_begin; ok && u0 < u_end && !bars->abort_flag; u0 += u_step, ++gc) {
                const int nu = kDense ? 1 : min(U, u_end - u0);
            const int n_tiles = group_tiles(u0, nu);
                for (int t = 0; ok && t < n_tiles; ++t) {
                    const int w = t & 1;
                    const int idx = cnt[w]++;
                    const int gt = cnt[0] + cnt[1] - 1;
                    if (!mbar_wait(&bars->p_full[2 * w], idx & 1)) { fail(22); ok = false; break; }
                    // first GEMM of the group into this accumulator overwrites it: the previous group's
                    // result must have been read
                    if (t < 2 && gc > 0 && !mbar_wait(&bars->o_free, (gc - 1) & 1)) { fail(23); ok = false; break; }
                    for (int us = 0; us < nu && !lp.lse_only; ++us, ++gy) {
                        const int sy = gy % kYStages;
                        if (!mbar_wait(&bars->y_full[sy], (gy / kYStages) & 1)) { fail(26); ok = false; break; }
                        tc_fence_after();
                        const uint64_t yd = y_desc0 + (uint64_t)((sy * kTileBytes) >> 4);
                        const uint32_t dis = dis_mask(us);
                        if (kDense) {
                            for (int hh = 0; hh < 2; ++hh) {                   // the tile's two 64-key halves
                                if (hh == 1 && !mbar_wait(&bars->p_full[2 * w + 1], idx & 1)) { fail(22); ok = false; break; }
                                tc_fence_after();
#pragma unroll
                                for (int kk = 0; kk < kNS / 16; ++kk)
                                    mma_ts(tmem + col_o(w), tmem + col_s(w) + hh * kNS + kk * 8,
                                           yd + (((hh * (kNS / 16) + kk) * 2048) >> 4), idesc_o, (t >= 2) || hh > 0 || (kk > 0));
                                mma_commit(&bars->pv_done[w]);
                                mma_commit(&bars->sp_free[2 * w + hh]);
                            }
                            if (!ok) break;
                        } else {
#pragma unroll
                            for (int kk = 0; kk < kKT / 16; ++kk)
                                mma_ts_masked(tmem + col_o(w), tmem + col_s(w) + kk * 8, yd + ((kk * 2048) >> 4), idesc_o,
                                              (t >= 2) || (kk > 0), dis);
                        }
                        mma_commit(&bars->y_empty[sy]);
                    }
                    if (!ok) break;
                    if (!kDense) {
                        mma_commit(&bars->pv_done[w]);
                        mma_commit(&bars->sp_free[2 * w]);
                    }
                    if (t + 1 == n_tiles) mma_commit(&bars->o_full);
                }
            }
        }
    } else if (warp >= 4 && warp < 12) {
        // ------------------------------------------------------------------ softmax warpgroups
        const int w = (warp - 4) >> 2;
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int us = kDense ? 0 : min(lane / R4, kMaxU - 1);       // unit slot whose bias this tile row uses
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const uint32_t s_t0 = tmem + lane_sel + col_s(w);
        const uint32_t o_t = tmem + lane_sel + col_o(w);
        const float scale_l2 = p.scale * kLog2e;
        int gc = 0, idx = 0;                  // idx: tiles this warpgroup has handled so far
        bool ok = true;
        for (int u0 = u_begin; ok && u0 < u_end && !bars->abort_flag; u0 += u_step, ++gc) {
            const int n_tiles = group_tiles(u0, kDense ? 1 : min(U, u_end - u0));
            float m_run = -INFINITY, l_run = 0.f;
            int my_tiles = 0;
            for (int t = w; ok && t < n_tiles; t += 2) {
              for (int hh = 0; hh < kH; ++hh) {                              // dense attention: the tile's two 64-key halves
                const uint32_t s_t = s_t0 + hh * kNS;
                const int valid = max(0, min(kNS, n_keys - t * kKT - hh * kNS));   // keys of this (half) tile that exist
                if (!mbar_wait(&bars->s_full[2 * w + hh], idx & 1)) { fail(31); ok = false; break; }
                const int cslot = w + 2 * (idx & 1);
                const float* cs = bars->cl[cslot][us];
                if (!kDense && !mbar_wait(&bars->cl_full[cslot], (idx >> 1) & 1)) { fail(33); ok = false; break; }
                tc_fence_after();
                // pass 1: row maximum of the biased logits (log2 units)
                const bool tail = kDense && valid < kNS;
                const uint64_t scale2 = f2_pack(scale_l2, scale_l2), nl2 = f2_pack(-kLog2e, -kLog2e);
                float lsum = 0.f;
                bool spec_done = false;
                if constexpr (kDense) {
                    // After a warpgroup's first half tile the row maximum rarely moves past the rescale threshold, so
                    // the half is first taken in ONE pass against the running reference; the packed P is only stored
                    // if every row of the warp stayed below 2^threshold in total (then no weight exceeded it and the
                    // two-pass path below would have produced the same bits), else the two passes run on the
                    // untouched S.
                    if (my_tiles > 0 && !tail) {
                        const float nm = -m_run;
                        const uint64_t nm2 = f2_pack(nm, nm);
                        uint64_t ls2 = f2_pack(0.f, 0.f);
                        uint32_t pk0[16], pk1[16];
                        {
                            uint32_t r[64];
                            tmem_ld64(s_t, r);
                            tmem_wait_ld();
#pragma unroll
                            for (int c = 0; c < 64; c += 2) {
                                float d0, d1;
                                f2_unpack(f2_fma(f2_pack(__uint_as_float(r[c]), __uint_as_float(r[c + 1])), scale2, nm2), d0, d1);
                                const float e0 = exp2f(d0), e1 = exp2f(d1);
                                ls2 = f2_add(ls2, f2_pack(e0, e1));
                                if (c < 32) pk0[c >> 1] = pack_bf16_alu(e0, e1);
                                else pk1[(c - 32) >> 1] = pack_bf16_alu(e0, e1);
                            }
                        }
                        float la, lb;
                        f2_unpack(ls2, la, lb);
                        const float ls = la + lb;
                        if (!__any_sync(0xffffffffu, !(ls < 256.0f))) {      // 2^kRescaleThreshold; also catches inf / nan
                            tmem_st16(s_t, pk0);
                            tmem_st16(s_t + 16, pk1);
                            tmem_wait_st();
                            lsum = ls;
                            spec_done = true;
                        }
                    }
                }
                if (!spec_done) {
                float mx = -INFINITY;
#pragma unroll 1
                for (int c0 = 0; c0 < kNS; c0 += 64) {
                    uint32_t r[64];
                    tmem_ld64(s_t + c0, r);
                    tmem_wait_ld();
                    if (kDense && !tail) {
                        // no bias: the maximum of the raw dot products (the scale is positive), two per instruction
#pragma unroll
                        for (int c = 0; c < 64; c += 2) mx = max3(mx, __uint_as_float(r[c]), __uint_as_float(r[c + 1]));
                    } else if (kDense) {
#pragma unroll
                        for (int c = 0; c < 64; ++c)                         // keys past the end of the cache view
                            mx = fmaxf(mx, c0 + c < valid ? __uint_as_float(r[c]) : -INFINITY);
                    } else {
#pragma unroll
                        for (int c = 0; c < 64; c += 2) {                    // packed fp32 pairs: S * scale - log2(e) * cL
                            const uint64_t bias2 = f2_mul(nl2, *reinterpret_cast<const uint64_t*>(&cs[c0 + c]));
                            float x0, x1;
                            f2_unpack(f2_fma(f2_pack(__uint_as_float(r[c]), __uint_as_float(r[c + 1])), scale2, bias2), x0, x1);
                            mx = max3(mx, x0, x1);
                        }
                    }
                }
                if (kDense) mx *= scale_l2;
                // lazy rescale: keep the old reference while the maximum grew by less than the threshold
                bool rescale = false;
                float corr = 1.0f;
                if (my_tiles == 0) {
                    m_run = mx;
                } else if (mx > m_run + kRescaleThreshold) {
                    corr = exp2f(m_run - mx);
                    m_run = mx;
                    l_run *= corr;
                    rescale = true;
                }
                if (__any_sync(0xffffffffu, rescale)) {
                    // the accumulator may only be touched once the previous GEMMs into it have finished
                    if (!mbar_wait(&bars->pv_done[w], (kH * idx + hh - 1) & 1)) { fail(32); ok = false; break; }
                    tc_fence_after();
#pragma unroll 1
                    for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
                        uint32_t r[32];
                        tmem_ld32(o_t + c0, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * corr);
                        tmem_st32(o_t + c0, r);
                    }
                    tmem_wait_st();
                }
                const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
                // pass 2: P = exp2(logit - m), packed bf16 written back over the S columns already consumed
                const uint64_t negm2 = f2_pack(neg_m, neg_m);
                uint64_t lsum2 = f2_pack(0.f, 0.f);
#pragma unroll 1
                for (int c0 = 0; c0 < kNS; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(s_t + c0, r);
                    tmem_wait_ld();
                    uint32_t pk[16];
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        uint64_t shift2 = negm2;
                        if (!kDense) shift2 = f2_fma(nl2, *reinterpret_cast<const uint64_t*>(&cs[c0 + c]), negm2);
                        float d0, d1;
                        f2_unpack(f2_fma(f2_pack(__uint_as_float(r[c]), __uint_as_float(r[c + 1])), scale2, shift2), d0, d1);
                        float e0 = exp2f(d0), e1 = exp2f(d1);
                        if (tail) {
                            if (c0 + c >= valid) e0 = 0.f;
                            if (c0 + c + 1 >= valid) e1 = 0.f;
                        }
                        lsum2 = f2_add(lsum2, f2_pack(e0, e1));
                        pk[c >> 1] = pack_bf16_alu(e0, e1);
                    }
                    if (!lp.lse_only) tmem_st16(s_t + (c0 >> 1), pk);
                }
                tmem_wait_st();
                float lsum_hi;
                f2_unpack(lsum2, lsum, lsum_hi);
                lsum += lsum_hi;
                }
                if (!kDense) mbar_arrive(&bars->cl_empty[cslot]);
                l_run += lsum;
                ++my_tiles;
                if (hh == kH - 1) ++idx;
                if (t + 2 >= n_tiles && hh == kH - 1) {   // this warpgroup's last tile of the group: publish (m, l)
                    // the previous group's statistics must have been consumed
                    if (gc > 0 && !mbar_wait(&bars->o_free, (gc - 1) & 1)) { fail(34); ok = false; break; }
                    bars->stats[w][0][row] = m_run;
                    bars->stats[w][1][row] = l_run;
                }
                tc_fence_before();
                mbar_arrive(&bars->p_full[2 * w + hh]);
              }
            }
        }
    } else if (warp >= 12) {
        // ------------------------------------------------------------------ epilogue warpgroup
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int us = kDense ? 0 : lane / R4;                       // unit slot of this tile row
        const int i_row = kDense ? row : quad * R4 + lane % R4;      // query index of this tile row
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        int gc = 0;
        for (int u0 = u_begin; u0 < u_end && !bars->abort_flag; u0 += u_step, ++gc) {
            const int nu = kDense ? 1 : min(U, u_end - u0);
            const int n_tiles = group_tiles(u0, nu);
            if (!mbar_wait(&bars->o_full, gc & 1)) { fail(41); break; }
            tc_fence_after();
            // even tiles went to warpgroup 0, odd tiles to warpgroup 1
            const bool has1 = n_tiles > 1;
            const float m0 = bars->stats[0][0][row], l0 = bars->stats[0][1][row];
            const float m1 = has1 ? bars->stats[1][0][row] : -INFINITY, l1 = has1 ? bars->stats[1][1][row] : 0.f;
            const float ms = fmaxf(m0, m1);
            const float w0 = exp2f(m0 - ms);
            const float w1 = has1 ? exp2f(m1 - ms) : 0.f;
            const float inv = 1.0f / (w0 * l0 + w1 * l1);
            bool row_ok;
            __nv_bfloat16* out_row = nullptr;
            if (kDense) {
                const int qt = u0 % lp.q_tiles, bh = u0 / lp.q_tiles, b = bh / p.H, hd = bh - b * p.H;
                const long long tok = (long long)qt * 128 + row;
                row_ok = tok < p.n_q;
                if (row_ok) out_row = p.out + (((long long)b * p.n_q + tok) * p.H + hd) * kHeadDim;
            } else {
                row_ok = us < nu && i_row < b1;
                if (row_ok) {
                    const LUnit un = decode_unit(p, u0 + us);
                    const int bh = p.bh0 + un.bhl, b = bh / p.H, hd = bh - b * p.H;
                    const long long tok = blk.row_token(p.a0 + un.al, i_row) + un.j;
                    out_row = p.out_row(b, tok, hd);
                    // iterative variant: the softmax's log-sum-exp (natural log) feeds the iteration update
                    if (lp.write_lse) p.lse[(long long)(u0 + us) * b1 + i_row] = (ms + log2f(w0 * l0 + w1 * l1)) * 0.6931471805599453f;
                }
            }
#pragma unroll 1
            for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
                uint32_t ra[32], rb[32];
                if (!lp.lse_only) {
                    tmem_ld32(tmem + lane_sel + col_o(0) + c0, ra);
                    tmem_ld32(tmem + lane_sel + col_o(1) + c0, rb);
                    tmem_wait_ld();
                }
                if (c0 + 32 == kHeadDim) {
                    tc_fence_before();
                    mbar_arrive(&bars->o_free);               // accumulators and statistics are in registers
                }
                if (row_ok && !lp.lse_only) {
#pragma unroll
                    for (int v8 = 0; v8 < 2; ++v8) {
                        uint32_t wv[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const int c = v8 * 16 + 2 * e;
                            float x0 = __uint_as_float(ra[c]) * w0, x1 = __uint_as_float(ra[c + 1]) * w0;
                            if (has1) { x0 = fmaf(__uint_as_float(rb[c]), w1, x0); x1 = fmaf(__uint_as_float(rb[c + 1]), w1, x1); }
                            wv[e] = pack_bf16(x0 * inv, x1 * inv);
                        }
                        st_global_v8(out_row + c0 + v8 * 16, wv);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace


// Launches the tensor-core column step for one chunk as a persistent grid.  maps = {aL, Y} with a
// (64, 128 keys, 1) box and the 5-D query-row map (box rows = ceil(b1/4)).
int launch_l_step_tc(const MonarchParams& p, const CUtensorMap* maps /* aL, Y, q rows */, int* status, int num_sms,
                     cudaStream_t s, int write_lse) {
    LaunchScope scope(kClsLStep, s);
    LTcParams lp;
    lp.mp = p;
    lp.n_units = p.nbh * p.na * p.blk.b2;
    lp.R4 = (p.blk.b1 + 3) / 4;
    lp.U = 32 / lp.R4;
    if (lp.U < 1) lp.U = 1;
    if (lp.U > kMaxU) lp.U = kMaxU;
    lp.status = status;
    // Query rows that are consecutive rows of the token grid come by TMA (the 128-byte swizzle is a function
    // of the shared-memory address, so a box may land on any 128-byte row of the tile); other blockings
    // are gathered by the producer warp with plain loads.
    lp.q_rows_tma = (p.blk.f_tied == 1 || p.blk.h_reduce == 1) ? 1 : 0;
    lp.n_kv = 0;
    lp.q_tiles = 0;
    lp.write_lse = write_lse != 0;
    lp.lse_only = write_lse == 2;
    const int n_groups = (lp.n_units + lp.U - 1) / lp.U;
    dim3 grid(n_groups < num_sms ? n_groups : num_sms);
    auto kernel = p.causal_groups > 0 ? monarch_l_tc_kernel<false, true> : monarch_l_tc_kernel<false, false>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    kernel<<<grid, kThreads, kSmemBytes, s>>>(maps[0], maps[1], maps[2], lp);
    return (int)cudaGetLastError();
}

// Dense attention on the same kernel.  maps = {K, V, q}: 4-D (d, head, token, batch), box 64 x 1 x 128 x 1.
int launch_dense_tc(const CUtensorMap* maps, __nv_bfloat16* out, int B, int H, int n_q, int n_kv, float scale, int* status,
                    int num_sms, cudaStream_t s) {
    LaunchScope scope(kClsDense, s);
    LTcParams lp;
    lp.mp = MonarchParams();
    lp.mp.out = out;
    lp.mp.H = H;
    lp.mp.n_q = n_q;
    lp.mp.scale = scale;
    lp.mp.blk.b1 = 128;            // every tile row is a query
    lp.mp.blk.b2 = 1;
    lp.q_tiles = (n_q + 127) / 128;
    lp.n_units = B * H * lp.q_tiles;
    lp.U = 1;
    lp.R4 = 32;
    lp.n_kv = n_kv;
    lp.q_rows_tma = 1;
    lp.write_lse = 0;
    lp.lse_only = 0;
    lp.status = status;
    dim3 grid(lp.n_units < num_sms ? lp.n_units : num_sms);
    cudaError_t e = cudaFuncSetAttribute(monarch_l_tc_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    monarch_l_tc_kernel<true, false><<<grid, kThreads, kSmemBytes, s>>>(maps[0], maps[1], maps[2], lp);
    return (int)cudaGetLastError();
}

}  // namespace sfm
