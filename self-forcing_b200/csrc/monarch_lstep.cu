// Monarch column step: for one (batch, head, query group a, column j) the b1 queries Q[a,:,j]
// attend the n_keys = F*b1 summary keys aL[a,f,j,k] with additive bias -cL[a,f,j,k]; the values
// are Y[a,f,j,k].  This is a flash-style pass with an online softmax over all (f, k):
//   out[a,i,j,:] = sum_(f,k) softmax_(f,k)( s * Q[a,i,j].aL[a,f,j,k] - cL[a,f,j,k] ) Y[a,f,j,k,:]
// written straight to natural token order (the inverse layout map is the store address).
// A second kernel produces, for the iterative path, the next row-step operand
//   aR[a,f,k,j,:] = sum_i L[a,f,j,k,i] Q[a,i,j,:],   cR[a,f,k,j] = sum_i L[a,f,j,k,i]
// from the normalised L (log-sum-exp taken from a first, lse-only pass of the kernel above).
//
// Follows monarch_attn_ref_op (wan/modules/monarch_attn.py:1821-1829) and monarch_attn_slow
// (wan/modules/monarch_attn.py:1727-1733, 1744-1749).
#include "monarch_params.cuh"
#include "profile.cuh"

namespace sfm {

namespace {

constexpr int kMergePitch = kHeadDim + 4;  // floats per merged row: 128 outputs, running max, sum

__device__ __forceinline__ int keys_visible(const MonarchParams& p, int a_abs) {
    if (p.causal_groups <= 0) return p.n_keys;
    int fmax = min(p.F, (a_abs / p.causal_groups + 1) * p.causal_groups);
    return fmax * p.blk.b1;
}

// grid: x = (a_local, j) pairs of the chunk, y = 32-row slices of the b1 queries, z = (b,h) of chunk
template <bool kLseOnly>
__global__ void __launch_bounds__(kLWarps * 32, 1) monarch_l_kernel(MonarchParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [32][kLds]
    __nv_bfloat16* As = Qs + kLQRows * kLds;                                   // [2][128][kLds]
    __nv_bfloat16* Ys = As + 2 * kLTileKeys * kLds;                            // [2][128][kLds]
    float* cs = reinterpret_cast<float*>(Ys + 2 * kLTileKeys * kLds);          // [2][128]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const Blocking& blk = p.blk;
    const int b1 = blk.b1, b2 = blk.b2;
    const int al = blockIdx.x / b2, j = blockIdx.x - al * b2;
    const int i0 = blockIdx.y * kLQRows;
    const int bhl = blockIdx.z, bh = p.bh0 + bhl, b = bh / p.H, hd = bh - b * p.H;
    const int a_abs = p.a0 + al;
    const long long aj = ((long long)bhl * p.na + al) * b2 + j;
    const int nkeys = keys_visible(p, a_abs);
    const int ntiles = (nkeys + kLTileKeys - 1) / kLTileKeys;
    const long long tok_pitch = (long long)p.H * kHeadDim;

    const __nv_bfloat16* a_src = p.aL + aj * p.n_keys * kHeadDim;
    const __nv_bfloat16* y_src = kLseOnly ? nullptr : p.Y + aj * p.n_keys * kHeadDim;
    const float* c_src = p.cL + aj * p.n_keys_c;

    {   // queries Q[a, i0.., j]: rows of 256 bytes gathered from natural order
        const __nv_bfloat16* qb = p.q + (long long)b * p.q_bs + (long long)hd * kHeadDim;
        for (int idx = tid; idx < kLQRows * 16; idx += kLWarps * 32) {
            int r = idx >> 4, vec = idx & 15;
            int i = i0 + r;
            bool ok = i < b1;
            long long off = ok ? (blk.row_token(a_abs, i) + j) * tok_pitch + vec * 8 : 0;
            cp_async16(Qs + r * kLds + vec * 8, qb + off, ok ? 16 : 0);
        }
    }
    auto load_tile = [&](int stage, int tile) {
        int key0 = tile * kLTileKeys;
        __nv_bfloat16* Ad = As + stage * kLTileKeys * kLds;
        __nv_bfloat16* Yd = Ys + stage * kLTileKeys * kLds;
        for (int idx = tid; idx < kLTileKeys * 16; idx += kLWarps * 32) {
            int r = idx >> 4, vec = idx & 15;
            bool ok = key0 + r < nkeys;
            long long off = ok ? (long long)(key0 + r) * kHeadDim + vec * 8 : 0;
            cp_async16(Ad + r * kLds + vec * 8, a_src + off, ok ? 16 : 0);
            if (!kLseOnly) cp_async16(Yd + r * kLds + vec * 8, y_src + off, ok ? 16 : 0);
        }
        if (tid < kLTileKeys) {
            int key = key0 + tid;
            cs[stage * kLTileKeys + tid] = key < nkeys ? c_src[key] : INFINITY;   // bias -inf when masked
        }
    };
    load_tile(0, 0);
    cp_async_commit();

    float o[2][kHeadDim / 8][4];
    float m_run[2][2], l_run[2][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
        m_run[mt][0] = m_run[mt][1] = -INFINITY;
        l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
        for (int i = 0; i < kHeadDim / 8; ++i) { o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f; }
    }
    const float scale_l2 = p.scale * kLog2e;

    for (int tile = 0; tile < ntiles; ++tile) {
        const int st = tile & 1;
        if (tile + 1 < ntiles) load_tile(st ^ 1, tile + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const int wkey0 = tile * kLTileKeys + warp * 32;   // this warp's 32 keys
        if (wkey0 < nkeys) {
            const __nv_bfloat16* At = As + st * kLTileKeys * kLds;
            const __nv_bfloat16* Yt = Ys + st * kLTileKeys * kLds;
            const float* ct = cs + st * kLTileKeys + warp * 32;
            float s[2][4][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) { s[mt][nt][0] = s[mt][nt][1] = s[mt][nt][2] = s[mt][nt][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < kHeadDim / 16; ++ks) {
                uint32_t a0[4], a1[4];
                load_a_frag(a0, Qs, 0, ks * 16, lane);
                load_a_frag(a1, Qs, 16, ks * 16, lane);
#pragma unroll
                for (int np = 0; np < 2; ++np) {
                    uint32_t bb[4];
                    load_b_frag_nk(bb, At, warp * 32 + np * 16, ks * 16, lane);
                    mma_bf16(s[0][2 * np], a0, bb[0], bb[1]);
                    mma_bf16(s[0][2 * np + 1], a0, bb[2], bb[3]);
                    mma_bf16(s[1][2 * np], a1, bb[0], bb[1]);
                    mma_bf16(s[1][2 * np + 1], a1, bb[2], bb[3]);
                }
            }
            // logits (log2 units) = s*scale*log2e - cL*log2e ; masked keys carry cL = +inf
            float bias[4][2];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                bias[nt][0] = ct[nt * 8 + 2 * t] * kLog2e;
                bias[nt][1] = ct[nt * 8 + 2 * t + 1] * kLog2e;
            }
            uint32_t pa[2][2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float x = s[mt][nt][e] * scale_l2 - bias[nt][e & 1];
                        s[mt][nt][e] = x;
                        mx[e >> 1] = fmaxf(mx[e >> 1], x);
                    }
                float corr[2], msafe[2];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    float mnew = fmaxf(m_run[mt][hh], quad_max(mx[hh]));
                    msafe[hh] = (mnew == -INFINITY) ? 0.f : mnew;
                    corr[hh] = exp2f(m_run[mt][hh] - msafe[hh]);
                    m_run[mt][hh] = mnew;
                }
                float rs[2] = {0.f, 0.f};
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float ex = exp2f(s[mt][nt][e] - msafe[e >> 1]);
                        s[mt][nt][e] = ex;
                        rs[e >> 1] += ex;
                    }
                l_run[mt][0] = l_run[mt][0] * corr[0] + rs[0];
                l_run[mt][1] = l_run[mt][1] * corr[1] + rs[1];
                if (!kLseOnly) {
#pragma unroll
                    for (int nt = 0; nt < kHeadDim / 8; ++nt) {
                        o[mt][nt][0] *= corr[0]; o[mt][nt][1] *= corr[0];
                        o[mt][nt][2] *= corr[1]; o[mt][nt][3] *= corr[1];
                    }
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) {
                        pa[mt][kk][0] = pack_bf16(s[mt][2 * kk][0], s[mt][2 * kk][1]);
                        pa[mt][kk][1] = pack_bf16(s[mt][2 * kk][2], s[mt][2 * kk][3]);
                        pa[mt][kk][2] = pack_bf16(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
                        pa[mt][kk][3] = pack_bf16(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
                    }
                }
            }
            if (!kLseOnly) {
#pragma unroll
                for (int kk = 0; kk < 2; ++kk)
#pragma unroll
                    for (int np = 0; np < kHeadDim / 16; ++np) {
                        uint32_t bb[4];
                        load_b_frag_kn(bb, Yt, np * 16, warp * 32 + kk * 16, lane);
                        mma_bf16(o[0][2 * np], pa[0][kk], bb[0], bb[1]);
                        mma_bf16(o[0][2 * np + 1], pa[0][kk], bb[2], bb[3]);
                        mma_bf16(o[1][2 * np], pa[1][kk], bb[0], bb[1]);
                        mma_bf16(o[1][2 * np + 1], pa[1][kk], bb[2], bb[3]);
                    }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- merge the four warps' partial softmax states through shared memory ---------------
    float* Mg = reinterpret_cast<float*>(As);   // [4 warps][32 rows][kMergePitch]; fits inside As+Ys
    float* mine = Mg + warp * kLQRows * kMergePitch;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
        float l0 = quad_sum(l_run[mt][0]), l1 = quad_sum(l_run[mt][1]);
        int r_lo = mt * 16 + g, r_hi = r_lo + 8;
        if (!kLseOnly) {
#pragma unroll
            for (int nt = 0; nt < kHeadDim / 8; ++nt) {
                *reinterpret_cast<float2*>(mine + r_lo * kMergePitch + nt * 8 + 2 * t) = make_float2(o[mt][nt][0], o[mt][nt][1]);
                *reinterpret_cast<float2*>(mine + r_hi * kMergePitch + nt * 8 + 2 * t) = make_float2(o[mt][nt][2], o[mt][nt][3]);
            }
        }
        if (t == 0) {
            mine[r_lo * kMergePitch + kHeadDim] = m_run[mt][0];
            mine[r_lo * kMergePitch + kHeadDim + 1] = l0;
            mine[r_hi * kMergePitch + kHeadDim] = m_run[mt][1];
            mine[r_hi * kMergePitch + kHeadDim + 1] = l1;
        }
    }
    __syncthreads();
    {
        const int r = tid >> 2, quarter = tid & 3;       // 32 rows x 4 column quarters
        const int i = i0 + r;
        float mw[kLWarps], lw[kLWarps], mstar = -INFINITY;
#pragma unroll
        for (int w = 0; w < kLWarps; ++w) {
            mw[w] = Mg[(w * kLQRows + r) * kMergePitch + kHeadDim];
            lw[w] = Mg[(w * kLQRows + r) * kMergePitch + kHeadDim + 1];
            mstar = fmaxf(mstar, mw[w]);
        }
        float wt[kLWarps], lsum = 0.f;
#pragma unroll
        for (int w = 0; w < kLWarps; ++w) {
            wt[w] = (mw[w] == -INFINITY) ? 0.f : exp2f(mw[w] - mstar);
            lsum += wt[w] * lw[w];
        }
        if (i < b1) {
            if (kLseOnly) {
                if (quarter == 0)   // natural-log units
                    p.lse[aj * b1 + i] = (mstar + log2f(lsum)) * 0.6931471805599453f;
            } else {
                float inv = 1.0f / lsum;
                long long tok = blk.row_token(a_abs, i) + j;
                __nv_bfloat16* dst = p.out + (((long long)b * p.n_q + tok) * p.H + hd) * kHeadDim + quarter * 32;
#pragma unroll
                for (int v4 = 0; v4 < 4; ++v4) {
                    float acc[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
                    for (int w = 0; w < kLWarps; ++w) {
                        const float* src = Mg + (w * kLQRows + r) * kMergePitch + quarter * 32 + v4 * 8;
                        float4 x0 = *reinterpret_cast<const float4*>(src);
                        float4 x1 = *reinterpret_cast<const float4*>(src + 4);
                        acc[0] += wt[w] * x0.x; acc[1] += wt[w] * x0.y; acc[2] += wt[w] * x0.z; acc[3] += wt[w] * x0.w;
                        acc[4] += wt[w] * x1.x; acc[5] += wt[w] * x1.y; acc[6] += wt[w] * x1.z; acc[7] += wt[w] * x1.w;
                    }
                    uint4 pk;
                    pk.x = pack_bf16(acc[0] * inv, acc[1] * inv);
                    pk.y = pack_bf16(acc[2] * inv, acc[3] * inv);
                    pk.z = pack_bf16(acc[4] * inv, acc[5] * inv);
                    pk.w = pack_bf16(acc[6] * inv, acc[7] * inv);
                    *reinterpret_cast<uint4*>(dst + v4 * 8) = pk;
                }
            }
        }
    }
}

// Iteration update.  grid: x = (a_local, j), y = 64-key tiles, z = (b,h) of chunk.  4 warps, each
// owns 16 keys (one m-tile) of the tile; loops over the b1 queries in slices of 32.
//   S^T[key, i] = aL[key,:] . Q[i,:]     P = exp(s*S^T - cL[key] - lse[i])     (normalised L)
//   cR[key] = sum_i P,   aR[key,:] = sum_i P Q[i,:]
__global__ void __launch_bounds__(128, 2) monarch_l_iter_kernel(MonarchParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [kIterMaxB1][kLds]
    __nv_bfloat16* As = Qs + kIterMaxB1 * kLds;                                // [64][kLds]
    float* lse_s = reinterpret_cast<float*>(As + 64 * kLds);                   // [kIterMaxB1]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const Blocking& blk = p.blk;
    const int b1 = blk.b1, b2 = blk.b2;
    const int al = blockIdx.x / b2, j = blockIdx.x - al * b2;
    const int key0 = blockIdx.y * 64;
    const int bhl = blockIdx.z, bh = p.bh0 + bhl, b = bh / p.H, hd = bh - b * p.H;
    const int a_abs = p.a0 + al;
    const long long aj = ((long long)bhl * p.na + al) * b2 + j;
    const int nkeys = p.n_keys;
    if (key0 >= nkeys) return;
    const int b1p = (b1 + 31) & ~31;
    const long long tok_pitch = (long long)p.H * kHeadDim;

    const __nv_bfloat16* qb = p.q + (long long)b * p.q_bs + (long long)hd * kHeadDim;
    for (int idx = tid; idx < b1p * 16; idx += 128) {
        int r = idx >> 4, vec = idx & 15;
        bool ok = r < b1;
        long long off = ok ? (blk.row_token(a_abs, r) + j) * tok_pitch + vec * 8 : 0;
        cp_async16(Qs + r * kLds + vec * 8, qb + off, ok ? 16 : 0);
    }
    const __nv_bfloat16* a_src = p.aL + aj * nkeys * kHeadDim;
    for (int idx = tid; idx < 64 * 16; idx += 128) {
        int r = idx >> 4, vec = idx & 15;
        bool ok = key0 + r < nkeys;
        long long off = ok ? (long long)(key0 + r) * kHeadDim + vec * 8 : 0;
        cp_async16(As + r * kLds + vec * 8, a_src + off, ok ? 16 : 0);
    }
    cp_async_commit();
    for (int i = tid; i < b1p; i += 128) lse_s[i] = i < b1 ? p.lse[aj * b1 + i] : INFINITY;
    cp_async_wait<0>();
    __syncthreads();

    const int kr[2] = {key0 + warp * 16 + g, key0 + warp * 16 + g + 8};
    float cl[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) cl[hh] = kr[hh] < nkeys ? p.cL[aj * p.n_keys_c + kr[hh]] : INFINITY;

    float o[kHeadDim / 8][4];
#pragma unroll
    for (int i = 0; i < kHeadDim / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float csum[2] = {0.f, 0.f};

    for (int ic = 0; ic < b1p; ic += 32) {
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < kHeadDim / 16; ++ks) {
            uint32_t a[4];
            load_a_frag(a, As, warp * 16, ks * 16, lane);
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t bb[4];
                load_b_frag_nk(bb, Qs, ic + np * 16, ks * 16, lane);
                mma_bf16(s[2 * np], a, bb[0], bb[1]);
                mma_bf16(s[2 * np + 1], a, bb[2], bb[3]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int i = ic + nt * 8 + 2 * t + (e & 1);
                float x = s[nt][e] * p.scale - cl[e >> 1] - lse_s[i];   // -inf for padded i / masked key
                float ex = __expf(x);
                s[nt][e] = ex;
                csum[e >> 1] += ex;
            }
        uint32_t pa[2][4];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            pa[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
#pragma unroll
            for (int np = 0; np < kHeadDim / 16; ++np) {
                uint32_t bb[4];
                load_b_frag_kn(bb, Qs, np * 16, ic + kk * 16, lane);
                mma_bf16(o[2 * np], pa[kk], bb[0], bb[1]);
                mma_bf16(o[2 * np + 1], pa[kk], bb[2], bb[3]);
            }
    }
    csum[0] = quad_sum(csum[0]);
    csum[1] = quad_sum(csum[1]);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        int key = kr[hh];
        if (key >= nkeys) continue;
        int f = key / b1, k = key - f * b1;
        long long row = ((((long long)bhl * p.F + f) * b1 + k) * p.na + al) * b2 + j;
        if (t == 0) p.cR[row] = csum[hh];
        __nv_bfloat16* dst = p.aR + row * kHeadDim;
#pragma unroll
        for (int nt = 0; nt < kHeadDim / 8; ++nt)
            *reinterpret_cast<uint32_t*>(dst + nt * 8 + 2 * t) = pack_bf16(o[nt][2 * hh], o[nt][2 * hh + 1]);
    }
}

}  // namespace

size_t l_smem_bytes() {
    return (size_t)(kLQRows + 4 * kLTileKeys) * kLds * sizeof(__nv_bfloat16) + 2 * kLTileKeys * sizeof(float);
}
size_t iter_smem_bytes() {
    return (size_t)(kIterMaxB1 + 64) * kLds * sizeof(__nv_bfloat16) + kIterMaxB1 * sizeof(float);
}

int launch_l_step(const MonarchParams& p, int lse_only, cudaStream_t s) {
    LaunchScope scope(kClsLStep, s);
    dim3 grid(p.na * p.blk.b2, (p.blk.b1 + kLQRows - 1) / kLQRows, p.nbh);
    size_t smem = l_smem_bytes();
    static_assert(kLWarps * kLQRows * kMergePitch * sizeof(float) <=
                      4 * (size_t)kLTileKeys * kLds * sizeof(__nv_bfloat16), "merge buffer must fit the tile buffers");
    cudaError_t e;
    if (lse_only) {
        e = cudaFuncSetAttribute(monarch_l_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        monarch_l_kernel<true><<<grid, kLWarps * 32, smem, s>>>(p);
    } else {
        e = cudaFuncSetAttribute(monarch_l_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        monarch_l_kernel<false><<<grid, kLWarps * 32, smem, s>>>(p);
    }
    return (int)cudaGetLastError();
}

int launch_l_iter(const MonarchParams& p, cudaStream_t s) {
    if (p.blk.b1 > kIterMaxB1) return SFM_ERR_UNSUPPORTED;
    LaunchScope scope(kClsLIter, s);
    dim3 grid(p.na * p.blk.b2, (p.n_keys + 63) / 64, p.nbh);
    size_t smem = iter_smem_bytes();
    cudaError_t e = cudaFuncSetAttribute(monarch_l_iter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    monarch_l_iter_kernel<<<grid, 128, smem, s>>>(p);
    return (int)cudaGetLastError();
}

}  // namespace sfm
