// Dense softmax attention without a mask over the whole key range (flash-style, online softmax).
// Used for the dense-init chunk and the "regular" configuration.  One CTA = 64 queries of one
// (batch, head); 4 warps x 16 query rows; keys stream through shared memory in 64-row tiles.
//
// Stands in for flash_attention / attention (wan/modules/attention.py:34-187).
#include "common.cuh"
#include "profile.cuh"

namespace sfm {

namespace {

constexpr int kDWarps = 4;
constexpr int kDQTile = 64;
constexpr int kDKTile = 64;

struct DenseParams {
    const __nv_bfloat16* q; long long q_bs;
    const __nv_bfloat16* k; const __nv_bfloat16* v; long long kv_bs;
    __nv_bfloat16* out;
    int H, n_q, n_kv;
    float scale;
};

__global__ void __launch_bounds__(kDWarps * 32, 2) dense_fwd_kernel(DenseParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [64][kLds]
    __nv_bfloat16* Ks = Qs + kDQTile * kLds;                           // [2][64][kLds]
    __nv_bfloat16* Vs = Ks + 2 * kDKTile * kLds;                       // [2][64][kLds]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int q0 = blockIdx.x * kDQTile;
    const int bh = blockIdx.y, b = bh / p.H, hd = bh - b * p.H;
    const long long tok_pitch = (long long)p.H * kHeadDim;
    const __nv_bfloat16* qb = p.q + (long long)b * p.q_bs + (long long)hd * kHeadDim;
    const __nv_bfloat16* kb = p.k + (long long)b * p.kv_bs + (long long)hd * kHeadDim;
    const __nv_bfloat16* vb = p.v + (long long)b * p.kv_bs + (long long)hd * kHeadDim;

    for (int idx = tid; idx < kDQTile * 16; idx += kDWarps * 32) {
        int r = idx >> 4, vec = idx & 15;
        bool ok = q0 + r < p.n_q;
        long long off = ok ? (long long)(q0 + r) * tok_pitch + vec * 8 : 0;
        cp_async16(Qs + r * kLds + vec * 8, qb + off, ok ? 16 : 0);
    }
    auto load_kv = [&](int stage, int tile) {
        int k0 = tile * kDKTile;
        for (int idx = tid; idx < kDKTile * 16; idx += kDWarps * 32) {
            int r = idx >> 4, vec = idx & 15;
            bool ok = k0 + r < p.n_kv;
            long long off = ok ? (long long)(k0 + r) * tok_pitch + vec * 8 : 0;
            cp_async16(Ks + (stage * kDKTile + r) * kLds + vec * 8, kb + off, ok ? 16 : 0);
            cp_async16(Vs + (stage * kDKTile + r) * kLds + vec * 8, vb + off, ok ? 16 : 0);
        }
    };
    load_kv(0, 0);
    cp_async_commit();

    const int ntiles = (p.n_kv + kDKTile - 1) / kDKTile;
    float o[kHeadDim / 8][4];
#pragma unroll
    for (int i = 0; i < kHeadDim / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float scale_l2 = p.scale * kLog2e;
    uint32_t qa[kHeadDim / 16][4];

    for (int tile = 0; tile < ntiles; ++tile) {
        const int st = tile & 1;
        if (tile + 1 < ntiles) load_kv(st ^ 1, tile + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (tile == 0) {
#pragma unroll
            for (int ks = 0; ks < kHeadDim / 16; ++ks) load_a_frag(qa[ks], Qs, warp * 16, ks * 16, lane);
        }
        const __nv_bfloat16* Kt = Ks + st * kDKTile * kLds;
        const __nv_bfloat16* Vt = Vs + st * kDKTile * kLds;
        float s[kDKTile / 8][4];
#pragma unroll
        for (int i = 0; i < kDKTile / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < kHeadDim / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < kDKTile / 16; ++np) {
                uint32_t bb[4];
                load_b_frag_nk(bb, Kt, np * 16, ks * 16, lane);
                mma_bf16(s[2 * np], qa[ks], bb[0], bb[1]);
                mma_bf16(s[2 * np + 1], qa[ks], bb[2], bb[3]);
            }
        }
        const int kbase = tile * kDKTile;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < kDKTile / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int col = kbase + nt * 8 + 2 * t + (e & 1);
                float x = col < p.n_kv ? s[nt][e] * scale_l2 : -INFINITY;
                s[nt][e] = x;
                mx[e >> 1] = fmaxf(mx[e >> 1], x);
            }
        float corr[2], msafe[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float mnew = fmaxf(m_run[hh], quad_max(mx[hh]));
            msafe[hh] = (mnew == -INFINITY) ? 0.f : mnew;
            corr[hh] = exp2f(m_run[hh] - msafe[hh]);
            m_run[hh] = mnew;
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < kDKTile / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float ex = exp2f(s[nt][e] - msafe[e >> 1]);
                s[nt][e] = ex;
                rs[e >> 1] += ex;
            }
        l_run[0] = l_run[0] * corr[0] + rs[0];
        l_run[1] = l_run[1] * corr[1] + rs[1];
#pragma unroll
        for (int nt = 0; nt < kHeadDim / 8; ++nt) {
            o[nt][0] *= corr[0]; o[nt][1] *= corr[0];
            o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < kDKTile / 16; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < kHeadDim / 16; ++np) {
                uint32_t bb[4];
                load_b_frag_kn(bb, Vt, np * 16, kk * 16, lane);
                mma_bf16(o[2 * np], pa, bb[0], bb[1]);
                mma_bf16(o[2 * np + 1], pa, bb[2], bb[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    float inv[2] = {1.0f / quad_sum(l_run[0]), 1.0f / quad_sum(l_run[1])};
    // stage the 16 x 128 result through this warp's slice of Qs (its own rows) for 16-byte stores
    __nv_bfloat16* stg = Qs + warp * 16 * kLds;
    __syncwarp();
#pragma unroll
    for (int nt = 0; nt < kHeadDim / 8; ++nt) {
        *reinterpret_cast<uint32_t*>(stg + g * kLds + nt * 8 + 2 * t) = pack_bf16(o[nt][0] * inv[0], o[nt][1] * inv[0]);
        *reinterpret_cast<uint32_t*>(stg + (g + 8) * kLds + nt * 8 + 2 * t) = pack_bf16(o[nt][2] * inv[1], o[nt][3] * inv[1]);
    }
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        int idx = it * 32 + lane, rr = idx >> 4, vec = idx & 15;
        int qi = q0 + warp * 16 + rr;
        if (qi < p.n_q) {
            uint4 val = *reinterpret_cast<const uint4*>(stg + rr * kLds + vec * 8);
            *reinterpret_cast<uint4*>(p.out + (((long long)b * p.n_q + qi) * p.H + hd) * kHeadDim + vec * 8) = val;
        }
    }
}

}  // namespace
}  // namespace sfm

using namespace sfm;

extern "C" int sfm_dense_fwd(const void* q, int64_t q_batch_stride, const void* k, const void* v,
                             int64_t kv_batch_stride, void* out, int B, int H, int D, int n_q, int n_kv,
                             float sm_scale, void* stream) {
    if (!q || !k || !v || !out) return SFM_ERR_NULL_POINTER;
    if (D != kHeadDim) return SFM_ERR_UNSUPPORTED;
    if (B <= 0 || H <= 0 || n_q <= 0 || n_kv <= 0) return SFM_ERR_BAD_SHAPE;
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
    if (mis(q) || mis(k) || mis(v) || mis(out) || (q_batch_stride % 8) || (kv_batch_stride % 8)) return SFM_ERR_ALIGNMENT;
    DenseParams p;
    p.q = (const __nv_bfloat16*)q; p.q_bs = q_batch_stride;
    p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v; p.kv_bs = kv_batch_stride;
    p.out = (__nv_bfloat16*)out; p.H = H; p.n_q = n_q; p.n_kv = n_kv; p.scale = sm_scale;
    size_t smem = (size_t)(kDQTile + 4 * kDKTile) * kLds * sizeof(__nv_bfloat16);
    cudaError_t e = cudaFuncSetAttribute(dense_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((n_q + kDQTile - 1) / kDQTile, B * H);
    LaunchScope scope(kClsDense, (cudaStream_t)stream);
    dense_fwd_kernel<<<grid, kDWarps * 32, smem, (cudaStream_t)stream>>>(p);
    return (int)cudaGetLastError();
}
