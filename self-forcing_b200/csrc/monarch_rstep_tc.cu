// Monarch row step on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Work is cut into units (batch*head, tile of stacked query groups, block row k, range of cached
// groups f).  A tile stacks up to 128 query rows r = (query group a, column j); each group is padded
// to a multiple of 8 rows so that its 128-byte-swizzled shared-memory image starts on a swizzle atom.
// CTAs are persistent: each walks the unit list with a fixed stride and, for every (unit, f),
// computes per query row a complete softmax over the b2 keys of K[f,k,:]:
//   S  = Q_tile K[f,k]^T                 tcgen05.mma, both operands from shared memory (K-major)
//   P  = softmax rows of S (scaled)      one thread per row: tcgen05.ld, registers, tcgen05.st (bf16)
//   [aL | Y] = P [K[f,k] | V[f,k]]       one N=256 tcgen05.mma per 16 keys, A = P from TMEM,
//                                        B = the K and V tiles side by side (MN-major)
//   cL = sum_l P ln P                    from the softmax registers
// and streams aL, Y (bf16) and cL to the chunk's bridge.
//
// Warp roles (19 warps): 0 = TMA producer, 1 = issuer of the [aL | Y] GEMMs (owns the TMEM
// allocation), 2 = issuer of the S GEMMs,
// 3..6 and 7..10 = two softmax warpgroups that take even / odd steps (each owns one of the two
// S/P buffers in TMEM; a warp reaches TMEM lane quadrant warp % 4, and four consecutive warps cover
// all four), 11..14 and 15..18 = two epilogue warpgroups (aL half / Y half of the
// accumulator).  The S GEMM of step i+1 overlaps the softmax of step i; the output accumulator is
// single buffered and handed back to the MMA warp as soon as both halves sit in registers.  Each
// epilogue thread owns one bridge row and writes it straight from registers with 32-byte stores.  All roles run the same unit loop and meet
// only through mbarriers whose phases follow running step counters, so the pipeline keeps flowing
// across unit boundaries.  Every wait is bounded; on a timeout the CTA records a status code and
// unwinds.
//
// Arithmetic follows monarch_attn_ref_op (wan/modules/monarch_attn.py:1813-1823, 1828); the sqrt(s)
// scaling of q and k is folded into the softmax scale, so aL here is the reference's aL / sqrt(s).
#include "monarch_params.cuh"
#include "profile.cuh"
#include "tc05.cuh"

namespace sfm {

using namespace tc;

namespace {

constexpr int kStages = 8;            // K/V tile ring, at most (128 KB: 2 x 64 KB, 4 x 32 KB or 8 x 16 KB stages by block width)
constexpr int kThreads = 608;          // 19 warps: one more would lower the register ceiling from 104 to 96
constexpr int kTileRows = 128;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColS1 = 64, kColO = 128;   // O = [aL | Y], 256 columns

struct RTcParams {
    MonarchParams mp;
    int rows_per_group;    // b2 padded to a multiple of 8
    int groups_per_tile;   // 128 / rows_per_group
    int tiles;             // tiles per (batch*head) of the chunk
    int n_units;           // nbh * tiles * b1 * fsplit
    int* status;           // device status word (0 = ok)
};


struct RUnit {
    int bhl, tile, k, f_begin, n_it;
};

template <bool kCausal>
__device__ __forceinline__ RUnit decode_unit(const RTcParams& rp, int u) {
    const MonarchParams& p = rp.mp;
    RUnit r;
    int fs = u % p.fsplit; u /= p.fsplit;
    r.k = u % p.blk.b1; u /= p.blk.b1;
    r.tile = u % rp.tiles;
    r.bhl = u / rp.tiles;
    r.f_begin = fs * p.f_per;
    int f_end = min(p.F, r.f_begin + p.f_per);
    if (kCausal) {
        // block-causal (no-cache path): the tile's last query group sees the most; later groups f are skipped
        const int a_hi = p.a0 + min((r.tile + 1) * rp.groups_per_tile, p.na) - 1;
        f_end = min(f_end, (a_hi / p.causal_groups + 1) * p.causal_groups);
    }
    r.n_it = max(0, f_end - r.f_begin);               // 0: nothing to do, every role skips the unit
    return r;
}

struct __align__(8) Barriers {
    uint64_t q_full[2], q_empty[2];   // single pass: buffer 0, once per unit; iterative variant: one per step, alternating
    uint64_t kv_full[kStages];
    uint64_t kv_empty[kStages];
    uint64_t s_full[2];
    uint64_t p_full[2];
    uint64_t sp_free[2];       // PV GEMM has consumed the P operand held in S/P buffer 0 / 1
    uint64_t o_full;
    uint64_t o_free;
    uint32_t tmem_base;
    volatile int abort_flag;
};

// shared memory carve-up (bytes from a 1024-aligned base)
constexpr int kQBytes = 2 * kTileRows * 128;               // two 64-column halves
constexpr int kStageBytes = 4 * 64 * 128;                  // K half 0, K half 1, V half 0, V half 1 (<= 64 rows each)
constexpr int kSmemBytes = 1024 + 2 * kQBytes + 4 * kStageBytes + 256;   // two query tiles, 128 KB of K / V stages

// 32-byte store of 16 bf16 to global memory (pointer 32-byte aligned).
__device__ __forceinline__ void st_global_v8(void* ptr, const uint32_t (&w)[8]) {
    asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                 "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}

// kIter: a pass of the iterative variant after the first one.  The query operand is no longer the chunk's q
// (one tile per unit) but the state aR[a,f,k,j,:] of the previous pass, which differs for every cached group f:
// one tile per STEP, loaded through `tq` = a 3-D map of aR ([bh*F*b1][na*b2][128]) into two alternating
// buffers, and every row's logits are divided by its cR (monarch_attn.py:1716-1719).
template <int N_S, bool kCausal, bool kIter>
__global__ void __launch_bounds__(kThreads, 1)
monarch_r_tc_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                    const __grid_constant__ CUtensorMap tv, RTcParams rp) {
    static_assert(!kIter || (N_S <= 64 && !kCausal), "the iterative variant exists for block columns up to 64, no mask");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;
    unsigned char* kv_s = q_s + 2 * kQBytes;                 // two query tiles: the next unit's loads while this one is worked on
    Barriers* bars = reinterpret_cast<Barriers*>(kv_s + 4 * kStageBytes);

    const MonarchParams& p = rp.mp;
    const Blocking& blk = p.blk;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b1 = blk.b1, b2 = blk.b2;
    const int RG = rp.rows_per_group;
    constexpr int kHalf = N_S * 128;                    // bytes of one 64-column half of a K or V tile
    // Block columns above 64 (wide grids): 128-row K / V stages (two of them fit), S/P buffers and the
    // accumulator move up in TMEM, and the softmax walks its row in 32-column chunks (see below).
    constexpr bool kWide = N_S > 64;
    // a stage holds K lo, K hi, V lo, V hi of N_S rows each: 16 KB up to 32 block columns, 32 KB up to 64, 64 KB beyond
    constexpr int kStg = kWide ? 2 : (N_S <= 32 ? 8 : 4);
    constexpr int kStgBytes = kWide ? 2 * kStageBytes : (N_S <= 32 ? kStageBytes / 2 : kStageBytes);
    constexpr uint32_t cS1 = kWide ? 128u : kColS1, cO = kWide ? 256u : kColO;
    // Single pass: the next unit's query tile loads into the other buffer while this unit is worked on (short units
    // at small cache lengths otherwise wait for it); measured slower for narrow blocks (up to 32 columns), which keep one.
    constexpr bool kQDouble = kIter || N_S > 32;
    constexpr int kQBufs = kQDouble ? 2 : 1;

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(&bars->q_full[s], 1); mbar_init(&bars->q_empty[s], 1); }
        for (int s = 0; s < kStg; ++s) { mbar_init(&bars->kv_full[s], 1); mbar_init(&bars->kv_empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&bars->s_full[s], 1); mbar_init(&bars->p_full[s], 128); }
        for (int s = 0; s < 2; ++s) mbar_init(&bars->sp_free[s], 1);
        mbar_init(&bars->o_full, 1);
        mbar_init(&bars->o_free, 256);
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) { tmem_alloc(&bars->tmem_base, kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    auto fail = [&](int code) {
        bars->abort_flag = 1;
        atomicCAS(rp.status, 0, code);
    };
    const int u_first = blockIdx.x, u_stride = gridDim.x;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tmap(&tq); prefetch_tmap(&tk); prefetch_tmap(&tv);
            int g = 0, uc = 0;
            for (int u = u_first; u < rp.n_units && !bars->abort_flag; u += u_stride) {
                const RUnit un = decode_unit<kCausal>(rp, u);
                if (kCausal && un.n_it == 0) continue;
                const int bh = p.bh0 + un.bhl, b = bh / p.H, hd = bh - b * p.H;
                const int g_first = un.tile * rp.groups_per_tile;
                const int ng = min(rp.groups_per_tile, p.na - g_first);
                if constexpr (!kIter) {
                    const int qb = kQDouble ? (uc & 1) : 0;
                    unsigned char* qd = q_s + qb * kQBytes;
                    if (uc >= kQBufs && !mbar_wait(&bars->q_empty[qb], ((uc / kQBufs) - 1) & 1)) { fail(10); break; }
                    mbar_arrive_expect_tx(&bars->q_full[qb], (uint32_t)(ng * RG * 256));
                    for (int gi = 0; gi < ng; ++gi) {
                        int tok = blk.row_token(p.a0 + g_first + gi, un.k);
                        tma_load_4d(qd + gi * RG * 128, &tq, &bars->q_full[qb], 0, hd, tok, b);
                        tma_load_4d(qd + kTileRows * 128 + gi * RG * 128, &tq, &bars->q_full[qb], 64, hd, tok, b);
                    }
                }
                for (int i = 0; i < un.n_it; ++i, ++g) {
                    const int s = g % kStg;
                    if constexpr (kIter) {
                        // this step's query tile: the state rows (a, j) of (f, k), group by group
                        const int qb = g & 1;
                        if (g >= 2 && !mbar_wait(&bars->q_empty[qb], ((g >> 1) - 1) & 1)) { fail(10); break; }
                        unsigned char* qd = q_s + qb * kQBytes;
                        const int fk = (un.bhl * p.F + un.f_begin + i) * b1 + un.k;
                        mbar_arrive_expect_tx(&bars->q_full[qb], (uint32_t)(ng * RG * 256));
                        for (int gi = 0; gi < ng; ++gi) {
                            tma_load_3d(qd + gi * RG * 128, &tq, &bars->q_full[qb], 0, (g_first + gi) * b2, fk);
                            tma_load_3d(qd + kTileRows * 128 + gi * RG * 128, &tq, &bars->q_full[qb], 64, (g_first + gi) * b2, fk);
                        }
                    }
                    if (g >= kStg && !mbar_wait(&bars->kv_empty[s], ((g / kStg) - 1) & 1)) { fail(11); break; }
                    const int tok = ((un.f_begin + i) * b1 + un.k) * b2;
                    unsigned char* st = kv_s + s * kStgBytes;
                    mbar_arrive_expect_tx(&bars->kv_full[s], (uint32_t)(4 * kHalf));
                    tma_load_4d(st, &tk, &bars->kv_full[s], 0, hd, tok, b);
                    tma_load_4d(st + kHalf, &tk, &bars->kv_full[s], 64, hd, tok, b);
                    tma_load_4d(st + 2 * kHalf, &tv, &bars->kv_full[s], 0, hd, tok, b);
                    tma_load_4d(st + 3 * kHalf, &tv, &bars->kv_full[s], 64, hd, tok, b);
                }
                ++uc;
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ S-GEMM issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16(kTileRows, N_S, 0, 0);
            // Descriptors differ from step to step only in the start-address field (16-byte units
            // in the low word), so they are built once and advanced with integer adds.
            const uint64_t q_desc = smem_desc_sw128(smem_addr(q_s), 16, 1024);
            const uint64_t k_desc0 = smem_desc_sw128(smem_addr(kv_s), 16, 1024);
            int g = 0, uc = 0;
            bool ok = true;
            for (int u = u_first; ok && u < rp.n_units && !bars->abort_flag; u += u_stride) {
                const RUnit un = decode_unit<kCausal>(rp, u);
                if (kCausal && un.n_it == 0) continue;
                if constexpr (!kIter) {
                    if (!mbar_wait(&bars->q_full[kQDouble ? (uc & 1) : 0], (uc / kQBufs) & 1)) { fail(20); break; }
                }
                for (int i = 0; i < un.n_it; ++i, ++g) {
                    const int s = g % kStg;
                    if constexpr (kIter) {
                        if (!mbar_wait(&bars->q_full[g & 1], (g >> 1) & 1)) { fail(20); ok = false; break; }
                    }
                    if (!mbar_wait(&bars->kv_full[s], (g / kStg) & 1)) { fail(21); ok = false; break; }
                    if (g >= 2 && !mbar_wait(&bars->sp_free[g & 1], ((g >> 1) - 1) & 1)) { fail(25); ok = false; break; }
                    tc_fence_after();
                    const uint64_t kd = k_desc0 + (uint64_t)((s * kStgBytes) >> 4);
                    const uint32_t d = tmem + ((g & 1) ? cS1 : kColS0);
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t q_off = ((ks >> 2) * (kTileRows * 128) + (ks & 3) * 32) >> 4;
                        const uint32_t k_off = ((ks >> 2) * kHalf + (ks & 3) * 32) >> 4;
                        mma_ss(d, q_desc + (uint32_t)((((kIter ? g : (kQDouble ? uc : 0)) & 1) * kQBytes) >> 4) + q_off, kd + k_off, idesc_s, ks > 0);
                    }
                    mma_commit(&bars->s_full[g & 1]);
                    if constexpr (kIter) {
                        mma_commit(&bars->q_empty[g & 1]);                 // this step's query tile has been read
                    } else {
                        if (i + 1 == un.n_it) mma_commit(&bars->q_empty[kQDouble ? (uc & 1) : 0]);   // last read of this unit's Q tile
                    }
                }
                ++uc;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ PV-GEMM issuer
        if (lane == 0) {
            // [aL | Y] in one N = 256 GEMM; the passes of the iterative variant that only need aL and cL stop at N = 128
            const uint32_t idesc_o = p.write_Y ? idesc_bf16(kTileRows, 2 * kHeadDim, 0, 1) : idesc_bf16(kTileRows, kHeadDim, 0, 1);
            constexpr int ksteps_pv = N_S / 16;
            const uint64_t kv_desc_mn0 = smem_desc_sw128(smem_addr(kv_s), kHalf, 1024);   // 4 column blocks: K lo, K hi, V lo, V hi
            int g = 0;
            bool ok = true;
            for (int u = u_first; ok && u < rp.n_units && !bars->abort_flag; u += u_stride) {
                const RUnit un = decode_unit<kCausal>(rp, u);
                for (int i = 0; i < un.n_it; ++i, ++g) {
                    if (!mbar_wait(&bars->p_full[g & 1], (g >> 1) & 1)) { fail(22); ok = false; break; }
                    if (g > 0 && !mbar_wait(&bars->o_free, (g - 1) & 1)) { fail(23); ok = false; break; }
                    tc_fence_after();
                    const int s = g % kStg;
                    const uint64_t bd = kv_desc_mn0 + (uint64_t)((s * kStgBytes) >> 4);
                    const uint32_t p_t = tmem + ((g & 1) ? cS1 : kColS0);
#pragma unroll
                    for (int kk = 0; kk < ksteps_pv; ++kk)
                        mma_ts(tmem + cO, p_t + kk * 8, bd + ((kk * 2048) >> 4), idesc_o, kk > 0);
                    mma_commit(&bars->o_full);
                    mma_commit(&bars->kv_empty[s]);
                    mma_commit(&bars->sp_free[g & 1]);
                }
            }
        }
    } else if (warp >= 3 && warp < 11) {
        // ------------------------------------------------------------------ softmax warpgroups
        const int wg = (warp - 3) >> 2;                 // 0: even steps / buffer 0, 1: odd steps / buffer 1
        const int quad = warp & 3;                      // TMEM lane quadrant this warp may access
        const int row = quad * 32 + lane;               // tile row == TMEM lane
        const int gl = row / RG, j = row - gl * RG;
        const float scale_l2 = p.mult0 * kLog2e;
        const uint32_t s_t = tmem + ((uint32_t)(quad * 32) << 16) + (wg ? cS1 : kColS0);
        int g = 0;
        bool ok = true;
        for (int u = u_first; ok && u < rp.n_units && !bars->abort_flag; u += u_stride) {
            const RUnit un = decode_unit<kCausal>(rp, u);
            const int g_first = un.tile * rp.groups_per_tile;
            const int ng = min(rp.groups_per_tile, p.na - g_first);
            const bool warp_active = quad * 32 < ng * RG;
            const bool row_ok = gl < ng && j < b2;
            const long long aj = ((long long)un.bhl * p.na + g_first + gl) * b2 + j;
            // block-causal: groups f this row's query group may not see get an infinite bias
            const int f_allowed = kCausal ? ((p.a0 + g_first + gl) / p.causal_groups + 1) * p.causal_groups : p.F;
            for (int i = 0; i < un.n_it; ++i, ++g) {
                if ((g & 1) != wg) continue;
                float scale_row = scale_l2;
                if constexpr (kIter) {
                    // logits are divided by the row's cR of the previous pass (clamped as in the reference)
                    if (row_ok) {
                        const long long ci = (((long long)un.bhl * p.F + un.f_begin + i) * b1 + un.k) * (long long)(p.na * b2) +
                                             (long long)(g_first + gl) * b2 + j;
                        scale_row = p.scale * kLog2e * fminf(1.0f / (p.cR[ci] + 1e-6f), 1e4f);
                    }
                }
                if (!mbar_wait(&bars->s_full[wg], (g >> 1) & 1)) { fail(31); ok = false; break; }
                tc_fence_after();
                if (warp_active) {
                    if constexpr (!kWide) {
                    uint32_t raw[N_S];
                    if constexpr (N_S == 64) {
                        tmem_ld32(s_t, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
                        tmem_ld32(s_t + 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[32]));
                    } else if constexpr (N_S == 32) {
                        tmem_ld32(s_t, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
                    } else if constexpr (N_S == 48) {
                        tmem_ld32(s_t, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
                        tmem_ld16(s_t + 32, *reinterpret_cast<uint32_t(*)[16]>(&raw[32]));
                    } else {
                        tmem_ld16(s_t, *reinterpret_cast<uint32_t(*)[16]>(&raw[0]));
                    }
                    tmem_wait_ld();
                    // only the last 16 columns can lie beyond b2
#pragma unroll
                    for (int c = N_S - 16; c < N_S; ++c)
                        if (c >= b2) raw[c] = 0xf149f2cau;   // -1e30: exp2 gives 0 and 0 * (finite) stays 0 below
                    float mx = -INFINITY;
#pragma unroll
                    for (int c = 0; c < N_S; c += 2) mx = max3(mx, __uint_as_float(raw[c]), __uint_as_float(raw[c + 1]));
                    const float neg_m = -mx * scale_row;
                    // two columns at a time on the packed fp32 pipe
                    const uint64_t scale2 = f2_pack(scale_row, scale_row), negm2 = f2_pack(neg_m, neg_m);
                    uint64_t z2 = f2_pack(0.f, 0.f), ent2 = z2;
                    uint64_t e2[N_S / 2];
#pragma unroll
                    for (int c = 0; c < N_S / 2; ++c) {
                        const uint64_t d2 = f2_fma(f2_pack(__uint_as_float(raw[2 * c]), __uint_as_float(raw[2 * c + 1])), scale2, negm2);
                        float d0, d1;                         // log2 units, <= 0 (about -1e29 if masked)
                        f2_unpack(d2, d0, d1);
                        e2[c] = f2_pack(exp2f(d0), exp2f(d1));
                        z2 = f2_add(z2, e2[c]);
                        ent2 = f2_fma(e2[c], d2, ent2);       // masked: 0 * (-1e29) = 0
                    }
                    float z, zh, ent, enth;
                    f2_unpack(z2, z, zh);
                    f2_unpack(ent2, ent, enth);
                    z += zh;
                    ent += enth;
                    const float inv_z = 1.0f / z;
                    const uint64_t invz2 = f2_pack(inv_z, inv_z);
                    uint32_t pk[N_S / 2];
#pragma unroll
                    for (int c = 0; c < N_S / 2; ++c) {
                        float p0, p1;
                        f2_unpack(f2_mul(e2[c], invz2), p0, p1);
                        pk[c] = pack_bf16_alu(p0, p1);
                    }
                    if constexpr (N_S == 64) {
                        tmem_st32(s_t, pk);
                    } else if constexpr (N_S == 32) {
                        tmem_st16(s_t, pk);
                    } else if constexpr (N_S == 48) {
                        tmem_st16(s_t, *reinterpret_cast<uint32_t(*)[16]>(&pk[0]));
                        uint32_t p2[16];
#pragma unroll
                        for (int c = 0; c < 16; ++c) p2[c] = c < 8 ? pk[16 + c] : 0u;
                        tmem_st16(s_t + 16, p2);
                    } else {
                        uint32_t p2[16];
#pragma unroll
                        for (int c = 0; c < 16; ++c) p2[c] = c < 8 ? pk[c] : 0u;
                        tmem_st16(s_t, p2);   // 8 packed columns are the operand; the other 8 lie inside the S buffer
                    }
                    tmem_wait_st();
                    if (row_ok) {
                        const int key = (un.f_begin + i) * b1 + un.k;
                        p.cL[aj * p.n_keys_c + key] =
                            (!kCausal || un.f_begin + i < f_allowed) ? 0.6931471805599453f * ent * inv_z - __logf(z) : INFINITY;
                    }
                    } else {
                    // Wide rows: three passes over the row in 32-column chunks read back from TMEM (maximum;
                    // sum and entropy; normalised P written over the S columns already consumed).
                    auto load_chunk = [&](int c0, uint32_t (&r)[32]) {
                        if (c0 + 32 <= N_S) {
                            tmem_ld32(s_t + c0, r);
                        } else {
                            tmem_ld16(s_t + c0, *reinterpret_cast<uint32_t(*)[16]>(&r[0]));
                        }
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c)
                            if (c0 + c >= b2) r[c] = 0xf149f2cau;          // -1e30, as above
                    };
                    float mx = -INFINITY;
#pragma unroll 1
                    for (int c0 = 0; c0 < N_S; c0 += 32) {
                        uint32_t r[32];
                        load_chunk(c0, r);
#pragma unroll
                        for (int c = 0; c < 32; c += 2) mx = max3(mx, __uint_as_float(r[c]), __uint_as_float(r[c + 1]));
                    }
                    const float neg_m = -mx * scale_l2;
                    const uint64_t scale2 = f2_pack(scale_l2, scale_l2), negm2 = f2_pack(neg_m, neg_m);
                    uint64_t z2 = f2_pack(0.f, 0.f), ent2 = z2;
#pragma unroll 1
                    for (int c0 = 0; c0 < N_S; c0 += 32) {
                        uint32_t r[32];
                        load_chunk(c0, r);
#pragma unroll
                        for (int c = 0; c < 32; c += 2) {
                            const uint64_t d2 = f2_fma(f2_pack(__uint_as_float(r[c]), __uint_as_float(r[c + 1])), scale2, negm2);
                            float d0, d1;
                            f2_unpack(d2, d0, d1);
                            const uint64_t e2 = f2_pack(exp2f(d0), exp2f(d1));
                            z2 = f2_add(z2, e2);
                            ent2 = f2_fma(e2, d2, ent2);
                        }
                    }
                    float z, zh, ent, enth;
                    f2_unpack(z2, z, zh);
                    f2_unpack(ent2, ent, enth);
                    z += zh;
                    ent += enth;
                    const float inv_z = 1.0f / z;
                    const uint64_t invz2 = f2_pack(inv_z, inv_z);
#pragma unroll 1
                    for (int c0 = 0; c0 < N_S; c0 += 32) {
                        uint32_t r[32], pk[16];
                        load_chunk(c0, r);
#pragma unroll
                        for (int c = 0; c < 32; c += 2) {
                            float d0, d1, p0, p1;
                            f2_unpack(f2_fma(f2_pack(__uint_as_float(r[c]), __uint_as_float(r[c + 1])), scale2, negm2), d0, d1);
                            f2_unpack(f2_mul(f2_pack(exp2f(d0), exp2f(d1)), invz2), p0, p1);
                            pk[c >> 1] = pack_bf16_alu(p0, p1);
                        }
                        tmem_st16(s_t + (c0 >> 1), pk);
                    }
                    tmem_wait_st();
                    if (row_ok) {
                        const int key = (un.f_begin + i) * b1 + un.k;
                        p.cL[aj * p.n_keys_c + key] =
                            (!kCausal || un.f_begin + i < f_allowed) ? 0.6931471805599453f * ent * inv_z - __logf(z) : INFINITY;
                    }
                    }
                }
                tc_fence_before();
                mbar_arrive(&bars->p_full[wg]);
            }
        }
    } else if (warp >= 11) {
        // ------------------------------------------------------------------ epilogue warpgroups
        const int which = (warp - 11) >> 2;              // 0: aL (columns 0..127 of O), 1: Y (columns 128..255)
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const uint32_t o_t = tmem + ((uint32_t)(quad * 32) << 16) + cO + which * kHeadDim;
        int g = 0;
        bool ok = true;
        for (int u = u_first; ok && u < rp.n_units && !bars->abort_flag; u += u_stride) {
            const RUnit un = decode_unit<kCausal>(rp, u);
            const int g_first = un.tile * rp.groups_per_tile;
            const int ng = min(rp.groups_per_tile, p.na - g_first);
            const bool warp_active = quad * 32 < ng * RG;
            for (int i = 0; ok && i < un.n_it; ++i, ++g) {
                if (!mbar_wait(&bars->o_full, g & 1)) { fail(41); ok = false; break; }
                tc_fence_after();
                // This thread's bridge row: 256 bytes at (aj, key), written as 32-byte vectors.
                const int gl = row / RG, j = row - gl * RG;
                const bool row_ok = warp_active && gl < ng && j < b2 && (which == 0 || p.write_Y);
                const long long aj = ((long long)un.bhl * p.na + g_first + gl) * b2 + j;
                const int key = (un.f_begin + i) * b1 + un.k;
                __nv_bfloat16* const out_row = (which ? p.Y : p.aL) + (aj * p.n_keys + key) * kHeadDim;
#pragma unroll
                for (int h = 0; h < 2; ++h) {                 // 64 columns at a time
                    uint32_t ra[32], rb[32];
                    if (warp_active && (which == 0 || p.write_Y)) {
                        tmem_ld32(o_t + h * 64, ra);
                        tmem_ld32(o_t + h * 64 + 32, rb);
                        tmem_wait_ld();
                    }
                    if (h == 1) {
                        tc_fence_before();
                        mbar_arrive(&bars->o_free);            // accumulator may be overwritten from here on
                    }
                    if (row_ok) {
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const uint32_t (&r)[32] = c ? rb : ra;
#pragma unroll
                            for (int v8 = 0; v8 < 2; ++v8) {
                                uint32_t w[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e)
                                    w[e] = pack_bf16_alu(__uint_as_float(r[v8 * 16 + 2 * e]), __uint_as_float(r[v8 * 16 + 2 * e + 1]));
                                st_global_v8(out_row + h * 64 + c * 32 + v8 * 16, w);
                            }
                        }
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


// Launches the tensor-core row step for one chunk as a persistent grid.  `status` is a device int the
// kernel sets on an internal timeout.
int launch_r_step_tc(const MonarchParams& p, const CUtensorMap* maps /* q (or the aR state), k, v */, int rows_per_group,
                     int n_s, int* status, int num_sms, cudaStream_t s) {
    LaunchScope scope(kClsRStep, s);
    RTcParams rp;
    rp.mp = p;
    rp.rows_per_group = rows_per_group;
    rp.groups_per_tile = kTileRows / rows_per_group;
    rp.tiles = (p.na + rp.groups_per_tile - 1) / rp.groups_per_tile;
    rp.n_units = p.nbh * rp.tiles * p.blk.b1 * p.fsplit;
    rp.status = status;
    dim3 grid(rp.n_units < num_sms ? rp.n_units : num_sms);
    // wide blocks: two 64 KB K / V stages instead of five 32 KB ones
    const bool iter = p.use_aR != 0;
    if (iter && (n_s > 64 || p.causal_groups > 0)) return SFM_ERR_UNSUPPORTED;
    const int smem_bytes = kSmemBytes;
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return (int)e;
        kernel<<<grid, kThreads, smem_bytes, s>>>(maps[0], maps[1], maps[2], rp);
        return 0;
    };
    int rc;
    const bool causal = p.causal_groups > 0;
    if (iter) {
        switch (n_s) {
            case 16: rc = go(monarch_r_tc_kernel<16, false, true>); break;
            case 32: rc = go(monarch_r_tc_kernel<32, false, true>); break;
            case 48: rc = go(monarch_r_tc_kernel<48, false, true>); break;
            case 64: rc = go(monarch_r_tc_kernel<64, false, true>); break;
            default: return SFM_ERR_UNSUPPORTED;
        }
    } else switch (n_s) {
        case 16: rc = causal ? go(monarch_r_tc_kernel<16, true, false>) : go(monarch_r_tc_kernel<16, false, false>); break;
        case 32: rc = causal ? go(monarch_r_tc_kernel<32, true, false>) : go(monarch_r_tc_kernel<32, false, false>); break;
        case 48: rc = causal ? go(monarch_r_tc_kernel<48, true, false>) : go(monarch_r_tc_kernel<48, false, false>); break;
        case 64: rc = causal ? go(monarch_r_tc_kernel<64, true, false>) : go(monarch_r_tc_kernel<64, false, false>); break;
        case 80: rc = causal ? go(monarch_r_tc_kernel<80, true, false>) : go(monarch_r_tc_kernel<80, false, false>); break;
        case 96: rc = causal ? go(monarch_r_tc_kernel<96, true, false>) : go(monarch_r_tc_kernel<96, false, false>); break;
        case 112: rc = causal ? go(monarch_r_tc_kernel<112, true, false>) : go(monarch_r_tc_kernel<112, false, false>); break;
        case 128: rc = causal ? go(monarch_r_tc_kernel<128, true, false>) : go(monarch_r_tc_kernel<128, false, false>); break;
        default: return SFM_ERR_UNSUPPORTED;
    }
    if (rc) return rc;
    return (int)cudaGetLastError();
}

}  // namespace sfm
