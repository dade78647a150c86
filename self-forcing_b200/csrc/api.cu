// extern "C" entry points for the Monarch forward and their host-side planning.
#include <algorithm>
#include <cstdlib>

#include "monarch_params.cuh"
#include "tc05.cuh"

using namespace sfm;

namespace sfm {
int launch_r_step_tc(const MonarchParams& p, const CUtensorMap* maps, int rows_per_group, int n_s, int* status,
                     int num_sms, cudaStream_t s);
int launch_l_step_tc(const MonarchParams& p, const CUtensorMap* maps, int* status, int num_sms, cudaStream_t s,
                     int write_lse = 0);
int launch_l_iter_tc(const MonarchParams& p, const CUtensorMap* map_al, const CUtensorMap* map_qrows, int* status,
                     int num_sms, cudaStream_t s);
}

namespace {

constexpr size_t kDefaultBridgeBudget = 1ull << 30;    // bytes of row-step results kept per chunk

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// How one call is cut into chunks and how the workspace is laid out.
struct Plan {
    Blocking blk;
    int A, F, n_keys;
    int nbh_chunk, na_chunk, na_cta;
    size_t off_status, off_aL, off_Y, off_cL, off_lse, off_aR, off_cR, total;
};

int make_plan(Plan* pl, int B, int H, int D, int n_q, int n_kv, int f_tied, int h_reduce, int w_reduce, int h,
              int w, int num_iters, size_t budget) {
    if (D != kHeadDim) return SFM_ERR_UNSUPPORTED;
    if (B <= 0 || H <= 0 || n_q <= 0 || n_kv <= 0 || num_iters < 1) return SFM_ERR_BAD_SHAPE;
    int rc = make_blocking(&pl->blk, f_tied, h_reduce, w_reduce, h, w);
    if (rc) return rc;
    const Blocking& blk = pl->blk;
    if (blk.b2 > kB2MaxTc) return SFM_ERR_UNSUPPORTED;
    if (n_q % blk.tied_tokens) return SFM_ERR_BAD_SHAPE;
    const int group_tokens = blk.b1 * blk.b2;
    if (n_kv % group_tokens) return SFM_ERR_BAD_SHAPE;
    if (num_iters > 1 && blk.b1 > kIterMaxB1) return SFM_ERR_UNSUPPORTED;
    pl->A = n_q / group_tokens;
    pl->F = n_kv / group_tokens;
    pl->n_keys = pl->F * blk.b1;
    if (budget == 0) {
        budget = kDefaultBridgeBudget;
        if (const char* e = getenv("SFM_BRIDGE_MB")) {
            long mb = atol(e);
            if (mb > 0) budget = (size_t)mb << 20;
        }
    }
    const size_t per_a = (size_t)blk.b2 * pl->n_keys * (2 * kHeadDim * 2 + 4) * (num_iters > 1 ? 2 : 1);
    const int BH = B * H;
    pl->na_cta = std::max(1, std::min(pl->A, kRMaxRows / blk.b2));
    if (per_a * pl->A <= budget) {
        pl->na_chunk = pl->A;
        pl->nbh_chunk = (int)std::min<size_t>((size_t)BH, std::max<size_t>(1, budget / (per_a * pl->A)));
    } else {
        pl->nbh_chunk = 1;
        int na = (int)std::max<size_t>(1, std::min<size_t>((size_t)pl->A, budget / per_a));
        if (na >= pl->na_cta) na -= na % pl->na_cta;
        pl->na_chunk = na;
    }
    const size_t aj = (size_t)pl->nbh_chunk * pl->na_chunk * blk.b2;
    size_t off = 0;
    pl->off_status = off; off = align256(off + sizeof(int));
    pl->off_aL = off; off = align256(off + aj * pl->n_keys * kHeadDim * 2);
    pl->off_Y = off;  off = align256(off + aj * pl->n_keys * kHeadDim * 2);
    pl->off_cL = off; off = align256(off + aj * (size_t)((pl->n_keys + 3) & ~3) * 4);
    pl->off_lse = pl->off_aR = pl->off_cR = off;
    if (num_iters > 1) {
        pl->off_lse = off; off = align256(off + aj * blk.b1 * 4);
        pl->off_aR = off;  off = align256(off + aj * pl->n_keys * kHeadDim * 2);
        pl->off_cR = off;  off = align256(off + aj * pl->n_keys * 4);
    }
    pl->total = off;
    return SFM_OK;
}

// Output sharded by token over the GPUs of one box (head-sharded attention); null = plain `out`.
struct OutShards {
    void* const* shards;
    int world, rank;
};

int run_monarch(const void* q, int64_t q_bs, const void* kc, const void* vc, int64_t c_bs, void* out, void* ws,
                size_t ws_bytes, int B, int H, int D, int n_q, int n_kv, int f_tied, int h_reduce, int w_reduce,
                int h, int w, float sm_scale, int num_iters, int causal_groups, size_t budget, cudaStream_t stream,
                const OutShards* os = nullptr) {
    if (!q || !kc || !vc || !ws) return SFM_ERR_NULL_POINTER;
    if (!os && !out) return SFM_ERR_NULL_POINTER;
    if (os) {
        if (!os->shards || os->world < 1 || os->world > kMaxPeers || os->rank < 0 || os->rank >= os->world)
            return SFM_ERR_BAD_SHAPE;
        if (n_q % os->world) return SFM_ERR_BAD_SHAPE;
        for (int i = 0; i < os->world; ++i) {
            if (!os->shards[i]) return SFM_ERR_NULL_POINTER;
            if (reinterpret_cast<uintptr_t>(os->shards[i]) & 31) return SFM_ERR_ALIGNMENT;
        }
        out = os->shards[os->rank];
    }
    Plan pl;
    int rc = make_plan(&pl, B, H, D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, num_iters, budget);
    if (rc) return rc;
    if (ws_bytes < pl.total) return SFM_ERR_WORKSPACE;
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
    if (mis(q) || mis(kc) || mis(vc) || mis(out) || (reinterpret_cast<uintptr_t>(ws) & 255) || (q_bs % 8) || (c_bs % 8))
        return SFM_ERR_ALIGNMENT;
    if (causal_groups < 0 || (causal_groups > 0 && num_iters != 1)) return SFM_ERR_UNSUPPORTED;

    MonarchParams p;
    p.q = (const __nv_bfloat16*)q; p.q_bs = q_bs;
    p.kc = (const __nv_bfloat16*)kc; p.vc = (const __nv_bfloat16*)vc; p.c_bs = c_bs;
    p.out = (__nv_bfloat16*)out;
    for (int i = 0; i < kMaxPeers; ++i) p.out_peers[i] = nullptr;
    if (os) {
        for (int i = 0; i < os->world; ++i) p.out_peers[i] = (__nv_bfloat16*)os->shards[i];
        p.out_tokens = n_q / os->world; p.out_heads = H * os->world; p.out_head0 = os->rank * H;
    } else {
        p.out_peers[0] = (__nv_bfloat16*)out;
        p.out_tokens = n_q; p.out_heads = H; p.out_head0 = 0;
    }
    unsigned char* base = (unsigned char*)ws;
    p.aL = (__nv_bfloat16*)(base + pl.off_aL);
    p.Y = (__nv_bfloat16*)(base + pl.off_Y);
    p.cL = (float*)(base + pl.off_cL);
    p.lse = (float*)(base + pl.off_lse);
    p.aR = (__nv_bfloat16*)(base + pl.off_aR);
    p.cR = (float*)(base + pl.off_cR);
    p.H = H; p.n_q = n_q; p.A = pl.A; p.F = pl.F; p.n_keys = pl.n_keys;
    p.n_keys_c = (pl.n_keys + 3) & ~3;
    p.na_cta = pl.na_cta;
    p.causal_groups = causal_groups;
    p.scale = sm_scale;
    p.blk = pl.blk;

    // Tensor-core path: single pass (block-causal included, for block rows up to 128) and the iterative variant
    // for block rows up to 128 and block columns up to 64; everything else runs on the mma.sync kernels.
    const bool iter_tc = num_iters > 1 && pl.blk.b1 <= 128 && pl.blk.b2 <= kB2Max;
    const bool use_tc = (num_iters == 1 && (causal_groups == 0 || pl.blk.b1 <= 128)) || iter_tc;
    // block columns above 64 exist on the tensor-core kernels only (single pass, block rows up to 128)
    if (pl.blk.b2 > kB2Max && !(use_tc && pl.blk.b1 <= 128)) return SFM_ERR_UNSUPPORTED;
    // only the tensor-core column step knows how to scatter its rows
    if (os && os->world > 1 && !(use_tc && pl.blk.b1 <= 128)) return SFM_ERR_UNSUPPORTED;
    int num_sms = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    int* status = reinterpret_cast<int*>(base + pl.off_status);
    CUtensorMap maps[7];
    const int rows_per_group = (pl.blk.b2 + 7) & ~7;
    const int n_s = (pl.blk.b2 + 15) & ~15;
    {
        // Every path starts from a clear status word: the workspace may be recycled memory, and the kernels
        // without bounded waits (iterative variant, block rows above 128) never write it.
        cudaError_t e = cudaMemsetAsync(status, 0, sizeof(int), stream);
        if (e != cudaSuccess) return (int)e;
    }
    if (use_tc) {
        cudaError_t e;
        // cL rows are padded to 16 bytes; the pad floats travel with the column step's bulk copies and
        // must act as "key masked": fill the buffer with a huge positive bias (0x7f7f7f7f = 3.4e38).
        e = cudaMemsetAsync(p.cL, 0x7f, (size_t)pl.nbh_chunk * pl.na_chunk * pl.blk.b2 * p.n_keys_c * sizeof(float), stream);
        if (e != cudaSuccess) return (int)e;
        const uint64_t row = (uint64_t)kHeadDim * 2, tok = (uint64_t)H * row;
        uint64_t dq[4] = {(uint64_t)kHeadDim, (uint64_t)H, (uint64_t)n_q, (uint64_t)B};
        uint64_t sq[3] = {row, tok, (uint64_t)q_bs * 2};
        uint32_t bq[4] = {64, 1, (uint32_t)rows_per_group, 1};
        uint64_t dk[4] = {(uint64_t)kHeadDim, (uint64_t)H, (uint64_t)n_kv, (uint64_t)B};
        uint64_t sk[3] = {row, tok, (uint64_t)c_bs * 2};
        uint32_t bk[4] = {64, 1, (uint32_t)n_s, 1};
        const uint64_t n_aj = (uint64_t)pl.nbh_chunk * pl.na_chunk * pl.blk.b2;
        uint64_t db[3] = {(uint64_t)kHeadDim, (uint64_t)pl.n_keys, n_aj};
        uint64_t sb[2] = {row, (uint64_t)pl.n_keys * row};
        uint32_t bb[3] = {64, 128, 1};   // column step: 128 keys of one (query group, column) per load
        if ((rc = make_tmap_bf16(&maps[0], q, 4, dq, sq, bq))) return rc;
        if ((rc = make_tmap_bf16(&maps[1], kc, 4, dk, sk, bk))) return rc;
        if ((rc = make_tmap_bf16(&maps[2], vc, 4, dk, sk, bk))) return rc;
        if ((rc = make_tmap_bf16(&maps[3], p.aL, 3, db, sb, bb))) return rc;
        if ((rc = make_tmap_bf16(&maps[4], p.Y, 3, db, sb, bb))) return rc;
        // queries of one (query group, column): rows of the token grid at a fixed column
        const int rows_per_quadrant = (pl.blk.b1 + 3) / 4;
        uint64_t dqr[5] = {(uint64_t)kHeadDim, (uint64_t)H, (uint64_t)w, (uint64_t)(n_q / w), (uint64_t)B};
        uint64_t sqr[4] = {row, tok, (uint64_t)w * tok, (uint64_t)q_bs * 2};
        uint32_t bqr[5] = {64, 1, 1, (uint32_t)rows_per_quadrant, 1};
        if ((rc = make_tmap_bf16(&maps[5], q, 5, dqr, sqr, bqr))) return rc;
    }

    const int BH = B * H;
    for (int bh0 = 0; bh0 < BH; bh0 += pl.nbh_chunk) {
        p.bh0 = bh0; p.nbh = std::min(pl.nbh_chunk, BH - bh0);
        for (int a0 = 0; a0 < pl.A; a0 += pl.na_chunk) {
            p.a0 = a0; p.na = std::min(pl.na_chunk, pl.A - a0);
            if (use_tc && causal_groups > 0) {
                // Block-causal: the row step skips the (query group, f) pairs no query may see, so the
                // column step finds bridge rows nobody wrote.  Give them defined contents: zero keys /
                // values and the "masked" bias.
                const size_t rows = (size_t)p.nbh * p.na * pl.blk.b2;
                cudaError_t e = cudaMemsetAsync(p.aL, 0, rows * pl.n_keys * kHeadDim * 2, stream);
                if (e == cudaSuccess) e = cudaMemsetAsync(p.Y, 0, rows * pl.n_keys * kHeadDim * 2, stream);
                if (e == cudaSuccess) e = cudaMemsetAsync(p.cL, 0x7f, rows * p.n_keys_c * sizeof(float), stream);
                if (e != cudaSuccess) return (int)e;
            }
            // enough row-step CTAs to fill the GPU about twice over
            int asubs = use_tc ? (p.na + (128 / rows_per_group) - 1) / (128 / rows_per_group)
                               : (p.na + p.na_cta - 1) / p.na_cta;
            int base_ctas = pl.blk.b1 * asubs * p.nbh;
            int fsplit;
            if (use_tc) {
                // Persistent CTAs take whole units round-robin, so the launch lasts (units per CTA, rounded
                // up) x (steps per unit).  Pick the split of the F loop that makes that smallest, with at
                // least three steps per unit (every unit reloads its query tile) and an extra step's worth
                // charged per unit for that reload.
                fsplit = 1;
                long long best = -1;
                for (int fs = 1; fs <= std::max(1, pl.F / 3); ++fs) {
                    const int per = (pl.F + fs - 1) / fs;
                    const int splits = (pl.F + per - 1) / per;
                    const long long units = (long long)base_ctas * splits;
                    const long long cost = ((units + num_sms - 1) / num_sms) * (per + 1);
                    if (best < 0 || cost < best) { best = cost; fsplit = fs; }
                }
            } else {
                fsplit = std::max(1, std::min(pl.F, (2 * num_sms + base_ctas - 1) / base_ctas));
            }
            p.f_per = (pl.F + fsplit - 1) / fsplit;
            p.fsplit = (pl.F + p.f_per - 1) / p.f_per;
            if (iter_tc) {
                // iteration state aR of this chunk as [nbh * F * b1][na * b2][128]: one (f, k) block of stacked
                // (query group, column) rows per index of the slowest dimension
                const uint64_t row = (uint64_t)kHeadDim * 2;
                uint64_t dar[3] = {(uint64_t)kHeadDim, (uint64_t)p.na * pl.blk.b2, (uint64_t)p.nbh * pl.F * pl.blk.b1};
                uint64_t sar[2] = {row, (uint64_t)p.na * pl.blk.b2 * row};
                uint32_t bar[3] = {64, (uint32_t)rows_per_group, 1};
                if ((rc = make_tmap_bf16(&maps[6], p.aR, 3, dar, sar, bar))) return rc;
            }

            for (int it = 0; it < num_iters; ++it) {
                const bool last = it == num_iters - 1;
                p.use_aR = it > 0;
                p.write_Y = last;
                p.mult0 = num_iters > 1 ? sm_scale * (1.0f / (1.0f + 1e-6f)) : sm_scale;
                if (use_tc) {
                    // later passes of the iterative variant read their query operand from the state aR
                    CUtensorMap rmaps[3] = {p.use_aR ? maps[6] : maps[0], maps[1], maps[2]};
                    if ((rc = launch_r_step_tc(p, rmaps, rows_per_group, n_s, status, num_sms, stream))) return rc;
                } else {
                    if ((rc = launch_r_step(p, stream))) return rc;
                }
                if (last) {
                    if (use_tc && pl.blk.b1 <= 128) {
                        if ((rc = launch_l_step_tc(p, maps + 3, status, num_sms, stream))) return rc;
                    } else if ((rc = launch_l_step(p, 0, stream))) return rc;
                } else if (iter_tc) {
                    // the column step's softmax statistics (its output row is overwritten by the last pass), then
                    // the update of the state
                    if ((rc = launch_l_step_tc(p, maps + 3, status, num_sms, stream, 2))) return rc;
                    if ((rc = launch_l_iter_tc(p, &maps[3], &maps[5], status, num_sms, stream))) return rc;
                } else {
                    if ((rc = launch_l_step(p, 1, stream))) return rc;
                    if ((rc = launch_l_iter(p, stream))) return rc;
                }
            }
        }
    }
    return SFM_OK;
}

}  // namespace

namespace sfm {
// Single-pass forward on the tensor-core kernels for the (batch, head) pairs [bh0, bh0 + nbh) with all query
// groups at once, into caller-given bridge buffers (aL, Y: bf16 [slab][n_keys][128], cL: fp32 [slab][n_keys_c],
// slab = (bh_local * A + a) * b2 + j) and, optionally, the column step's log-sum-exp per query row
// (lse: fp32 [slab][b1]).  The backward uses it to recompute what the forward did not keep.  Returns the launch
// parameters and the six tensor maps (q, K, V, aL bridge, Y bridge, query rows) for the kernels that follow.
int forward_tc_slice(const void* q, int64_t q_bs, const void* kc, const void* vc, int64_t c_bs, void* out,
                     __nv_bfloat16* aL, __nv_bfloat16* Y, float* cL, float* lse, int* status, int B, int H, int n_q,
                     int n_kv, const Blocking& blk, float scale, int bh0, int nbh, MonarchParams* p_out,
                     CUtensorMap* maps, cudaStream_t stream) {
    if (blk.b1 > 128 || blk.b2 > kB2MaxTc) return SFM_ERR_UNSUPPORTED;
    const int group = blk.b1 * blk.b2;
    MonarchParams p;
    p.q = (const __nv_bfloat16*)q; p.q_bs = q_bs;
    p.kc = (const __nv_bfloat16*)kc; p.vc = (const __nv_bfloat16*)vc; p.c_bs = c_bs;
    p.out = (__nv_bfloat16*)out;
    for (int i = 0; i < kMaxPeers; ++i) p.out_peers[i] = nullptr;
    p.out_peers[0] = (__nv_bfloat16*)out;
    p.out_tokens = n_q; p.out_heads = H; p.out_head0 = 0;
    p.aL = aL; p.Y = Y; p.cL = cL; p.lse = lse; p.aR = nullptr; p.cR = nullptr;
    p.H = H; p.n_q = n_q; p.A = n_q / group; p.F = n_kv / group; p.n_keys = p.F * blk.b1;
    p.n_keys_c = (p.n_keys + 3) & ~3;
    p.na_cta = std::max(1, std::min(p.A, kRMaxRows / blk.b2));
    p.causal_groups = 0;
    p.scale = scale; p.mult0 = scale;
    p.blk = blk;
    p.bh0 = bh0; p.nbh = nbh; p.a0 = 0; p.na = p.A;
    p.use_aR = 0; p.write_Y = 1;
    int num_sms = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const int rows_per_group = (blk.b2 + 7) & ~7;
    const int n_s = (blk.b2 + 15) & ~15;
    const size_t slabs = (size_t)nbh * p.A * blk.b2;
    // the caller owns the status word (set once per call, shared by its slices)
    cudaError_t e = cudaMemsetAsync(cL, 0x7f, slabs * p.n_keys_c * sizeof(float), stream);
    if (e != cudaSuccess) return (int)e;
    int rc;
    const uint64_t row = (uint64_t)kHeadDim * 2, tok = (uint64_t)H * row;
    uint64_t dq[4] = {(uint64_t)kHeadDim, (uint64_t)H, (uint64_t)n_q, (uint64_t)B};
    uint64_t sq[3] = {row, tok, (uint64_t)q_bs * 2};
    uint32_t bq[4] = {64, 1, (uint32_t)rows_per_group, 1};
    uint64_t dk[4] = {(uint64_t)kHeadDim, (uint64_t)H, (uint64_t)n_kv, (uint64_t)B};
    uint64_t sk[3] = {row, tok, (uint64_t)c_bs * 2};
    uint32_t bk[4] = {64, 1, (uint32_t)n_s, 1};
    uint64_t db[3] = {(uint64_t)kHeadDim, (uint64_t)p.n_keys, (uint64_t)slabs};
    uint64_t sb[2] = {row, (uint64_t)p.n_keys * row};
    uint32_t bb[3] = {64, 128, 1};
    const int rows_per_quadrant = (blk.b1 + 3) / 4;
    uint64_t dqr[5] = {(uint64_t)kHeadDim, (uint64_t)H, (uint64_t)blk.w, (uint64_t)(n_q / blk.w), (uint64_t)B};
    uint64_t sqr[4] = {row, tok, (uint64_t)blk.w * tok, (uint64_t)q_bs * 2};
    uint32_t bqr[5] = {64, 1, 1, (uint32_t)rows_per_quadrant, 1};
    if ((rc = make_tmap_bf16(&maps[0], q, 4, dq, sq, bq))) return rc;
    if ((rc = make_tmap_bf16(&maps[1], kc, 4, dk, sk, bk))) return rc;
    if ((rc = make_tmap_bf16(&maps[2], vc, 4, dk, sk, bk))) return rc;
    if ((rc = make_tmap_bf16(&maps[3], aL, 3, db, sb, bb))) return rc;
    if ((rc = make_tmap_bf16(&maps[4], Y, 3, db, sb, bb))) return rc;
    if ((rc = make_tmap_bf16(&maps[5], q, 5, dqr, sqr, bqr))) return rc;
    // split of the F loop over persistent CTAs, as in the forward proper
    const int asubs = (p.na + (128 / rows_per_group) - 1) / (128 / rows_per_group);
    const int base_ctas = blk.b1 * asubs * nbh;
    int fsplit = 1;
    long long best = -1;
    for (int fs = 1; fs <= std::max(1, p.F / 3); ++fs) {
        const int per = (p.F + fs - 1) / fs;
        const int splits = (p.F + per - 1) / per;
        const long long units = (long long)base_ctas * splits;
        const long long cost = ((units + num_sms - 1) / num_sms) * (per + 1);
        if (best < 0 || cost < best) { best = cost; fsplit = fs; }
    }
    p.f_per = (p.F + fsplit - 1) / fsplit;
    p.fsplit = (p.F + p.f_per - 1) / p.f_per;
    if ((rc = launch_r_step_tc(p, maps, rows_per_group, n_s, status, num_sms, stream))) return rc;
    if ((rc = launch_l_step_tc(p, maps + 3, status, num_sms, stream, lse ? 1 : 0))) return rc;
    *p_out = p;
    return SFM_OK;
}
}  // namespace sfm

extern "C" int sfm_version(void) { return 100; }

// Reads (and thereby waits for) the status word the kernels of the last call on `workspace` left.
extern "C" int sfm_workspace_status(const void* workspace, void* stream) {
    if (!workspace) return SFM_ERR_NULL_POINTER;
    int st = 0;
    cudaError_t e = cudaMemcpyAsync(&st, workspace, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    return st == 0 ? SFM_OK : SFM_ERR_DEVICE_STATUS;
}

extern "C" const char* sfm_error_string(int code) {
    switch (code) {
        case SFM_OK: return "success";
        case SFM_ERR_NULL_POINTER: return "null pointer argument";
        case SFM_ERR_BAD_SHAPE: return "sizes inconsistent with the blocking";
        case SFM_ERR_UNSUPPORTED: return "unsupported size (head_dim must be 128; block columns <= 128, and <= 64 for the iterative variant or block rows above 128)";
        case SFM_ERR_ALIGNMENT: return "pointer or stride not 16-byte aligned";
        case SFM_ERR_WORKSPACE: return "workspace too small";
        case SFM_ERR_NO_DEVICE: return "no sm_100 device";
        case SFM_ERR_DEVICE_STATUS: return "kernel recorded an internal error status";
        case SFM_ERR_STATIC_SCRATCH:
            return "problem too large for the library's built-in scratch array: one (batch*head, query group) slice of "
                   "row-step results must fit 32 MiB; use sfm_monarch_fwd with a caller-provided workspace";
        default: break;
    }
    if (code > 0) return cudaGetErrorString((cudaError_t)code);
    return "unknown error";
}

extern "C" size_t sfm_monarch_workspace_bytes(int B, int H, int D, int n_q, int n_kv, int f_tied, int h_reduce,
                                              int w_reduce, int h, int w, int num_iters, size_t bridge_budget_bytes) {
    Plan pl;
    if (make_plan(&pl, B, H, D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, num_iters, bridge_budget_bytes)) return 0;
    return pl.total;
}

extern "C" int sfm_monarch_fwd_scatter(const void* q, int64_t q_batch_stride, const void* k_cache, const void* v_cache,
                                       int64_t cache_batch_stride, void* const* out_shards, int world, int rank,
                                       void* workspace, size_t workspace_bytes, int B, int H, int D, int n_q, int n_kv,
                                       int f_tied, int h_reduce, int w_reduce, int h, int w, float sm_scale,
                                       size_t bridge_budget_bytes, void* stream) {
    OutShards os = {out_shards, world, rank};
    return run_monarch(q, q_batch_stride, k_cache, v_cache, cache_batch_stride, nullptr, workspace, workspace_bytes, B, H,
                       D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, sm_scale, 1, 0, bridge_budget_bytes,
                       (cudaStream_t)stream, &os);
}

extern "C" int sfm_monarch_fwd(const void* q, int64_t q_batch_stride, const void* k_cache, const void* v_cache,
                               int64_t cache_batch_stride, void* out, void* workspace, size_t workspace_bytes, int B,
                               int H, int D, int n_q, int n_kv, int f_tied, int h_reduce, int w_reduce, int h, int w,
                               float sm_scale, int num_iters, size_t bridge_budget_bytes, void* stream) {
    return run_monarch(q, q_batch_stride, k_cache, v_cache, cache_batch_stride, out, workspace, workspace_bytes, B, H,
                       D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, sm_scale, num_iters, 0, bridge_budget_bytes,
                       (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// Forward pass on library-owned scratch, for callers that must not allocate.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr size_t kStaticScratchBytes = 32ull << 20;
// Lives in every CUDA context that loads this library, for the life of the process.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {};   // device address of the array, per device ordinal
}  // namespace

extern "C" size_t sfm_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int sfm_monarch_fwd_static(const void* q, int64_t q_batch_stride, const void* k_cache, const void* v_cache,
                                      int64_t cache_batch_stride, void* out, int B, int H, int D, int n_q, int n_kv,
                                      int f_tied, int h_reduce, int w_reduce, int h, int w, float sm_scale,
                                      int num_iters, void* stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return SFM_ERR_UNSUPPORTED;
    if (!g_static_scratch_ptr[dev]) {
        // The array's name is only a host-side handle; kernels need its address on the current device.
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        g_static_scratch_ptr[dev] = ptr;
    }
    // Cut the work so that one chunk of row-step results fits the array; refuse what cannot fit.
    const size_t budget = kStaticScratchBytes - (64u << 10);
    Plan pl;
    int rc = make_plan(&pl, B, H, D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, num_iters, budget);
    if (rc) return rc;
    if (pl.total > kStaticScratchBytes) return SFM_ERR_STATIC_SCRATCH;
    return run_monarch(q, q_batch_stride, k_cache, v_cache, cache_batch_stride, out, g_static_scratch_ptr[dev],
                       kStaticScratchBytes, B, H, D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, sm_scale, num_iters, 0,
                       budget, (cudaStream_t)stream);
}

// Status word of the last sfm_monarch_fwd_static call on the current device (first word of the built-in
// array): waits for `stream` and reports SFM_OK or SFM_ERR_DEVICE_STATUS, like sfm_workspace_status.
extern "C" int sfm_static_scratch_status(void* stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return SFM_ERR_UNSUPPORTED;
    if (!g_static_scratch_ptr[dev]) return SFM_OK;                 // never used on this device
    return sfm_workspace_status(g_static_scratch_ptr[dev], stream);
}

extern "C" int sfm_monarch_nocache_fwd(const void* q, const void* k, const void* v, void* k_mon, void* v_mon,
                                       void* out, void* workspace, size_t workspace_bytes, int B, int H, int D, int N,
                                       int f_tied, int h_reduce, int w_reduce, int h, int w, float sm_scale,
                                       int causal_groups, int num_iters, size_t bridge_budget_bytes, void* stream) {
    if (!k_mon || !v_mon) return SFM_ERR_NULL_POINTER;
    int rc = sfm_rope_cache_write(nullptr, k, v, nullptr, k_mon, v_mon, (int64_t)N * H * D, nullptr, B, N, H, D, 0,
                                  f_tied, h_reduce, w_reduce, h, w, 0, 1, stream);
    if (rc) return rc;
    return run_monarch(q, (int64_t)N * H * D, k_mon, v_mon, (int64_t)N * H * D, out, workspace, workspace_bytes, B, H,
                       D, N, N, f_tied, h_reduce, w_reduce, h, w, sm_scale, num_iters, causal_groups,
                       bridge_budget_bytes, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// launch accounting / per-kernel timing
// ---------------------------------------------------------------------------------------------
#include <atomic>
#include <mutex>
#include <vector>

#include "profile.cuh"

namespace {
std::atomic<long long> g_launches[kNumClasses];
std::atomic<int> g_profile_on{0};
struct EventPair { int cls; cudaEvent_t start, stop; };
std::mutex g_prof_mutex;
std::vector<EventPair> g_pairs;       // recorded since the last read
std::vector<EventPair> g_free_pairs;  // recycled events
}  // namespace

namespace sfm {
LaunchScope::LaunchScope(int cls, cudaStream_t stream) : cls_(cls), stream_(stream), slot_(-1) {
    g_launches[cls].fetch_add(1, std::memory_order_relaxed);
    if (!g_profile_on.load(std::memory_order_relaxed)) return;
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    EventPair ep;
    if (!g_free_pairs.empty()) {
        ep = g_free_pairs.back();
        g_free_pairs.pop_back();
    } else {
        if (cudaEventCreate(&ep.start) != cudaSuccess || cudaEventCreate(&ep.stop) != cudaSuccess) return;
    }
    ep.cls = cls;
    cudaEventRecord(ep.start, stream);
    g_pairs.push_back(ep);
    slot_ = (int)g_pairs.size() - 1;
}
LaunchScope::~LaunchScope() {
    if (slot_ < 0) return;
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    if (slot_ < (int)g_pairs.size()) cudaEventRecord(g_pairs[slot_].stop, stream_);
}
}  // namespace sfm

extern "C" long long sfm_launch_count(void) {
    long long n = 0;
    for (int c = 0; c < kNumClasses; ++c) n += g_launches[c].load();
    return n;
}

extern "C" int sfm_profile_enable(int on) {
    g_profile_on.store(on ? 1 : 0);
    return SFM_OK;
}

extern "C" int sfm_profile_read(float* ms, long long* launches, int n_classes) {
    if (!ms || !launches) return SFM_ERR_NULL_POINTER;
    if (n_classes != kNumClasses) return SFM_ERR_BAD_SHAPE;
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    for (int c = 0; c < kNumClasses; ++c) { ms[c] = 0.f; launches[c] = 0; }
    for (auto& ep : g_pairs) {
        cudaError_t e = cudaEventSynchronize(ep.stop);
        if (e != cudaSuccess) return (int)e;
        float t = 0.f;
        e = cudaEventElapsedTime(&t, ep.start, ep.stop);
        if (e != cudaSuccess) return (int)e;
        ms[ep.cls] += t;
        launches[ep.cls] += 1;
        g_free_pairs.push_back(ep);
    }
    g_pairs.clear();
    return SFM_OK;
}
