// Monarch row step: for one (batch, head, block row k) and a range of cached groups f, every
// stacked query row (query group a, column j) runs a softmax over the b2 keys of row block
// K[f,k,:] and produces
//   aL[a,f,j,k,:] = sum_l R K[f,k,l,:]     Y[a,f,j,k,:] = sum_l R V[f,k,l,:]     cL = sum_l R ln R
// with R = softmax_l(mult * q_row . K[f,k,l]).  The K/V row block is read once for all stacked
// query groups.  Results go to the chunk's bridge buffers (see monarch_params.cuh).
//
// Follows the arithmetic of monarch_attn_ref_op / monarch_attn_slow
// (wan/modules/monarch_attn.py:1813-1823, 1735-1742); the scale sqrt(s) the reference applies
// to both q and k is folded into `mult`, so aL here is the reference's aL / sqrt(s).
#include "monarch_params.cuh"
#include "profile.cuh"

namespace sfm {

namespace {

struct RSmem {
    __nv_bfloat16* q[2];
    __nv_bfloat16* k[2];
    __nv_bfloat16* v[2];
    __nv_bfloat16* stage;  // per warp [16][kLds]
};

__device__ __forceinline__ RSmem carve(unsigned char* raw, bool per_f_query) {
    RSmem s;
    __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(raw);
    s.q[0] = p; p += kRMaxRows * kLds;
    if (per_f_query) { s.q[1] = p; p += kRMaxRows * kLds; } else { s.q[1] = s.q[0]; }
    for (int i = 0; i < 2; ++i) { s.k[i] = p; p += kB2Max * kLds; }
    for (int i = 0; i < 2; ++i) { s.v[i] = p; p += kB2Max * kLds; }
    s.stage = p;
    return s;
}

template <bool kPerFQuery>
__global__ void __launch_bounds__(kRWarps * 32, 1) monarch_r_kernel(MonarchParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    RSmem sm = carve(smem_raw, kPerFQuery);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const Blocking& blk = p.blk;
    const int b1 = blk.b1, b2 = blk.b2;
    const int k = blockIdx.x % b1, fs = blockIdx.x / b1;
    const int a_first = blockIdx.y * p.na_cta;                 // chunk-local first query group
    const int na_here = min(p.na_cta, p.na - a_first);
    const int bhl = blockIdx.z, bh = p.bh0 + bhl, b = bh / p.H, hd = bh - b * p.H;
    const int rows = na_here * b2;
    const int rows_pad = (rows + 15) & ~15;
    const int mtiles = rows_pad >> 4;
    const int b2p = (b2 + 15) & ~15;
    const int npairs = b2p >> 4;                               // pairs of 8-wide key tiles == 16-deep k steps

    int f_begin = fs * p.f_per, f_end = min(p.F, f_begin + p.f_per);
    if (p.causal_groups > 0) {                                 // last query group of the CTA sees the most
        int a_last = p.a0 + a_first + na_here - 1;
        f_end = min(f_end, (a_last / p.causal_groups + 1) * p.causal_groups);
    }
    if (f_begin >= f_end) return;

    const __nv_bfloat16* kbase = p.kc + (long long)b * p.c_bs + (long long)hd * kHeadDim;
    const __nv_bfloat16* vbase = p.vc + (long long)b * p.c_bs + (long long)hd * kHeadDim;
    const long long tok_pitch = (long long)p.H * kHeadDim;

    auto load_q_natural = [&](__nv_bfloat16* dst) {
        const __nv_bfloat16* qb = p.q + (long long)b * p.q_bs + (long long)hd * kHeadDim;
        for (int idx = tid; idx < rows_pad * 16; idx += kRWarps * 32) {
            int r = idx >> 4, vec = idx & 15;
            const __nv_bfloat16* src = qb;
            int bytes = 0;
            if (r < rows) {
                int al = r / b2, j = r - al * b2;
                int tok = blk.row_token(p.a0 + a_first + al, k) + j;
                src = qb + tok * tok_pitch + vec * 8;
                bytes = 16;
            }
            cp_async16(dst + r * kLds + vec * 8, src, bytes);
        }
    };
    auto load_q_state = [&](__nv_bfloat16* dst, int f) {       // aR rows (a, j) of (f, k), contiguous
        const __nv_bfloat16* src0 =
            p.aR + ((((long long)bhl * p.F + f) * b1 + k) * p.na + a_first) * (long long)b2 * kHeadDim;
        for (int idx = tid; idx < rows_pad * 16; idx += kRWarps * 32) {
            int r = idx >> 4, vec = idx & 15;
            bool ok = r < rows;
            cp_async16(dst + r * kLds + vec * 8, ok ? src0 + (long long)r * kHeadDim + vec * 8 : src0, ok ? 16 : 0);
        }
    };
    auto load_kv = [&](int stage, int f) {
        long long tok0 = ((long long)f * b1 + k) * b2;
        for (int idx = tid; idx < b2p * 16; idx += kRWarps * 32) {
            int l = idx >> 4, vec = idx & 15;
            bool ok = l < b2;
            long long off = ok ? (tok0 + l) * tok_pitch + vec * 8 : 0;
            cp_async16(sm.k[stage] + l * kLds + vec * 8, kbase + off, ok ? 16 : 0);
            cp_async16(sm.v[stage] + l * kLds + vec * 8, vbase + off, ok ? 16 : 0);
        }
    };

    if (!kPerFQuery) load_q_natural(sm.q[0]); else load_q_state(sm.q[0], f_begin);
    load_kv(0, f_begin);
    cp_async_commit();

    __nv_bfloat16* stg = sm.stage + warp * 16 * kLds;
    const float scale_l2 = (kPerFQuery ? p.scale : p.mult0) * kLog2e;

    for (int f = f_begin; f < f_end; ++f) {
        const int st = (f - f_begin) & 1;
        if (f + 1 < f_end) {
            if (kPerFQuery) load_q_state(sm.q[st ^ 1], f + 1);
            load_kv(st ^ 1, f + 1);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const __nv_bfloat16* Qs = sm.q[kPerFQuery ? st : 0];
        const __nv_bfloat16* Ks = sm.k[st];
        const __nv_bfloat16* Vs = sm.v[st];
        const int key = f * b1 + k;

        for (int mt = warp; mt < mtiles; mt += kRWarps) {
            const int r0 = mt * 16;
            // causal (no-cache path): skip the tile when none of its query groups may see f
            if (p.causal_groups > 0) {
                int a_hi = p.a0 + a_first + min(r0 + 15, rows - 1) / b2;
                if (f >= (a_hi / p.causal_groups + 1) * p.causal_groups) continue;
            }
            // ---- S = Q K^T (16 x b2p) ------------------------------------------------
            float s[kB2Max / 8][4];
#pragma unroll
            for (int i = 0; i < kB2Max / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < kHeadDim / 16; ++ks) {
                uint32_t a[4];
                load_a_frag(a, Qs, r0, ks * 16, lane);
#pragma unroll
                for (int np = 0; np < kB2Max / 16; ++np) {
                    if (np < npairs) {
                        uint32_t bb[4];
                        load_b_frag_nk(bb, Ks, np * 16, ks * 16, lane);
                        mma_bf16(s[2 * np], a, bb[0], bb[1]);
                        mma_bf16(s[2 * np + 1], a, bb[2], bb[3]);
                    }
                }
            }
            // ---- row softmax in registers (rows r0+g and r0+g+8) ---------------------
            float mult[2] = {scale_l2, scale_l2};
            if (kPerFQuery) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    int r = r0 + g + hh * 8;
                    if (r < rows) {
                        float c = p.cR[((((long long)bhl * p.F + f) * b1 + k) * p.na + a_first) * (long long)b2 + r];
                        mult[hh] = scale_l2 * fminf(1.0f / (c + 1e-6f), 1e4f);
                    }
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < kB2Max / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    int col = nt * 8 + 2 * t + (e & 1);
                    float x = (col < b2 && nt < 2 * npairs) ? s[nt][e] * mult[e >> 1] : -INFINITY;
                    s[nt][e] = x;                                   // log2 units from here on
                    mx[e >> 1] = fmaxf(mx[e >> 1], x);
                }
            }
            mx[0] = quad_max(mx[0]); mx[1] = quad_max(mx[1]);
            float z[2] = {0.f, 0.f}, ent[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < kB2Max / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float d = s[nt][e] - mx[e >> 1];                // <= 0, -inf when masked
                    float ex = exp2f(d);
                    z[e >> 1] += ex;
                    ent[e >> 1] += (ex > 0.f) ? ex * d : 0.f;
                    s[nt][e] = ex;
                }
            }
            z[0] = quad_sum(z[0]); z[1] = quad_sum(z[1]);
            ent[0] = quad_sum(ent[0]); ent[1] = quad_sum(ent[1]);
            float inv_z[2] = {1.0f / z[0], 1.0f / z[1]};
            // sum_l R ln R = ln2 * (sum e*d)/Z - ln Z      (d in log2 units)
            float cl[2] = {0.6931471805599453f * ent[0] * inv_z[0] - __logf(z[0]),
                           0.6931471805599453f * ent[1] * inv_z[1] - __logf(z[1])};

            uint32_t pa[kB2Max / 16][4];
#pragma unroll
            for (int kk = 0; kk < kB2Max / 16; ++kk) {
                pa[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pa[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pa[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            }

            // bridge rows of this m-tile
            long long aj_row[2];
            bool row_ok[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                int r = r0 + g + hh * 8;
                row_ok[hh] = r < rows;
                if (p.causal_groups > 0 && row_ok[hh]) {
                    int a_abs = p.a0 + a_first + r / b2;
                    row_ok[hh] = f < (a_abs / p.causal_groups + 1) * p.causal_groups;
                }
                aj_row[hh] = ((long long)bhl * p.na + a_first) * b2 + r;
            }
            if (t == 0) {
                if (row_ok[0]) p.cL[aj_row[0] * p.n_keys_c + key] = cl[0];
                if (row_ok[1]) p.cL[aj_row[1] * p.n_keys_c + key] = cl[1];
            }

            // ---- aL = P K, then Y = P V; normalise, stage through shared, 16-byte stores --
#pragma unroll 1
            for (int which = 0; which < 2; ++which) {
                if (which == 1 && !p.write_Y) break;
                const __nv_bfloat16* T = which ? Vs : Ks;
                float o[kHeadDim / 8][4];
#pragma unroll
                for (int i = 0; i < kHeadDim / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
#pragma unroll
                for (int kk = 0; kk < kB2Max / 16; ++kk) {
                    if (kk < npairs) {
#pragma unroll
                        for (int np = 0; np < kHeadDim / 16; ++np) {
                            uint32_t bb[4];
                            load_b_frag_kn(bb, T, np * 16, kk * 16, lane);
                            mma_bf16(o[2 * np], pa[kk], bb[0], bb[1]);
                            mma_bf16(o[2 * np + 1], pa[kk], bb[2], bb[3]);
                        }
                    }
                }
                __syncwarp();
#pragma unroll
                for (int nt = 0; nt < kHeadDim / 8; ++nt) {
                    *reinterpret_cast<uint32_t*>(stg + g * kLds + nt * 8 + 2 * t) =
                        pack_bf16(o[nt][0] * inv_z[0], o[nt][1] * inv_z[0]);
                    *reinterpret_cast<uint32_t*>(stg + (g + 8) * kLds + nt * 8 + 2 * t) =
                        pack_bf16(o[nt][2] * inv_z[1], o[nt][3] * inv_z[1]);
                }
                __syncwarp();
                __nv_bfloat16* dst_base = which ? p.Y : p.aL;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    int idx = it * 32 + lane, rr = idx >> 4, vec = idx & 15;
                    int r = r0 + rr;
                    bool ok = r < rows;
                    if (ok && p.causal_groups > 0) {
                        int a_abs = p.a0 + a_first + r / b2;
                        ok = f < (a_abs / p.causal_groups + 1) * p.causal_groups;
                    }
                    if (ok) {
                        long long aj = ((long long)bhl * p.na + a_first) * b2 + r;
                        uint4 val = *reinterpret_cast<const uint4*>(stg + rr * kLds + vec * 8);
                        *reinterpret_cast<uint4*>(dst_base + (aj * p.n_keys + key) * kHeadDim + vec * 8) = val;
                    }
                }
            }
        }
        __syncthreads();  // everyone is done with stage `st` before it is refilled
    }
    cp_async_wait<0>();
}

}  // namespace

size_t r_smem_bytes(bool per_f_query) {
    size_t elems = (size_t)(per_f_query ? 2 : 1) * kRMaxRows * kLds + 4 * (size_t)kB2Max * kLds +
                   (size_t)kRWarps * 16 * kLds;
    return elems * sizeof(__nv_bfloat16);
}

int launch_r_step(const MonarchParams& p, cudaStream_t s) {
    LaunchScope scope(kClsRStep, s);
    int asubs = (p.na + p.na_cta - 1) / p.na_cta;
    dim3 grid(p.blk.b1 * p.fsplit, asubs, p.nbh);
    if (p.use_aR) {
        size_t smem = r_smem_bytes(true);
        cudaError_t e = cudaFuncSetAttribute(monarch_r_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        monarch_r_kernel<true><<<grid, kRWarps * 32, smem, s>>>(p);
    } else {
        size_t smem = r_smem_bytes(false);
        cudaError_t e = cudaFuncSetAttribute(monarch_r_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        monarch_r_kernel<false><<<grid, kRWarps * 32, smem, s>>>(p);
    }
    return (int)cudaGetLastError();
}

}  // namespace sfm
