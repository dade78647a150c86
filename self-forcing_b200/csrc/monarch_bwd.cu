// Backward of single-pass (T = 1) Monarch attention against a KV cache: dQ, dK, dV from dOut.
//
// Forward, per (batch, head), with q^ = sqrt(scale) Q and k^ = sqrt(scale) K:
//   row step     unit (a, f, k, j):  z_l = q^[a,k,j] . k^[f,k,l],  R = softmax_l z,
//                aL = sum_l R_l k^[f,k,l],  Y = sum_l R_l V[f,k,l],  cL = sum_l R_l ln R_l
//   column step  slab (a, j), query row i, key n = (f, k):  s = q^[a,i,j] . aL_n - cL_n,
//                P = softmax_n s,  out[a,i,j] = sum_n P_n Y_n
// Backward, three launches per slice of (batch, head) pairs, all arithmetic in fp32:
//   1. bwd_row_forward_kernel   recomputes aL, Y, cL into the scratch area (fp32)
//   2. bwd_col_kernel           per slab, two sweeps over its keys: the softmax statistics and
//                               delta_i = sum_n P dP (accumulated with the running maximum), then
//                               ds = P (dP - delta), dq^_i = sum_n ds aL_n (stored to dQ),
//                               daL_n = sum_i ds q^_i and dY_n = sum_i P dOut_i (written over aL and Y in
//                               place, tile by tile), dcL_n = -sum_i ds
//   3. bwd_row_kernel           per block row k, looping over the cached groups f: per unit
//                               dR_l = daL.k^_l + dY.V_l + dcL (ln R_l + 1), dz = R (dR - sum R dR),
//                               dQ[a,k,j] += scale sum_l dz_l K_l (the two CTAs of a block row, one per half of
//                               the cached groups, own those rows in dq and in a second buffer merged afterwards:
//                               no atomics),
//                               dK[f,k,l] = sqrt(scale) sum_(a,j) (R_l daL + dz_l q^), dV[f,k,l] = sum_(a,j) R_l dY
// The kernels of this file are plain fp32 FMA code staged through shared memory: deterministic, any block size
// up to 128 x 128, block-causal mask included.  Without a mask and for block rows up to 96 and block columns up
// to 64 the entry point runs the same three stages on the tensor cores instead (tcgen05): the forward's own row-
// and column-step kernels for the recompute, then the column- and row-step backward kernels of
// monarch_bwd_tc.cu / monarch_bwd_row_tc.cu, with aL, Y and their gradients in bf16 as in the reference.
//
// Stands in for _attention_with_cache.backward and its Triton kernels
// (wan/modules/monarch_attn.py:403-596, 1034-1222, 1325-1470), including grad_only_new_kv
// (dK / dV only for a range of cached groups).  Unlike that code it accumulates dQ without atomics and keeps
// the intermediate gradients in fp32.
#include <algorithm>
#include <cstdlib>

#include "monarch_params.cuh"
#include "profile.cuh"
#include "tc05.cuh"

namespace sfm {
int forward_tc_slice(const void* q, int64_t q_bs, const void* kc, const void* vc, int64_t c_bs, void* out,
                     __nv_bfloat16* aL, __nv_bfloat16* Y, float* cL, float* lse, int* status, int B, int H, int n_q,
                     int n_kv, const Blocking& blk, float scale, int bh0, int nbh, MonarchParams* p_out,
                     CUtensorMap* maps, cudaStream_t stream);
int launch_bwd_delta(const void* dout, const void* out, float* delta, long long rows, cudaStream_t s);
int launch_bwd_col_tc(const MonarchParams& mp, const CUtensorMap* maps, const float* delta, float* dcL, float* dq,
                      int* status, int num_sms, cudaStream_t s);
size_t bwd_row_tc_partial_bytes(const MonarchParams& mp, int g0, int g1);
int launch_bwd_row_tc(const MonarchParams& mp, const CUtensorMap* maps, const float* dcL, float* dq, float* part_k,
                      float* part_v, __nv_bfloat16* dk, __nv_bfloat16* dv, int g0, int g1, int* status, int num_sms,
                      cudaStream_t s);
namespace {

using bf16 = __nv_bfloat16;
constexpr int kD = kHeadDim;
constexpr int kKs = kD + 4;        // bf16 row stride of a K / V tile in shared memory (66 words: conflict-free 8-byte loads by row)
constexpr int kFs = kD + 4;        // fp32 row stride of the column kernel's tiles: 16-byte rows, conflict-free float4 by row
constexpr int kQs = kD;             // fp32 row stride of its q^ / dOut rows (read as broadcasts or by consecutive lanes)
constexpr int kTileN = 32;         // keys per tile of the column kernel
constexpr int kRowBatch = 32;      // unit rows per batch of the row kernel

// 32-bit words of one K or V tile in shared memory, rounded to 16 bytes
__host__ __device__ inline int kv_tile_words(int b2) { return (b2 * (kKs / 2) + 3) & ~3; }

struct BwdParams {
    const bf16 *q, *k, *v, *dout;
    float* dq;
    float* dq2;                    // scratch like dq: the share of the second half of the cached groups (row kernel)
    bf16 *dk, *dv;
    float *aL, *Y, *cL, *dcL;      // scratch; aL / Y hold daL / dY after the column kernel
    const bf16 *aLb, *Yb;          // tensor-core path: daL / dY as bf16 (gradients of the UNSCALED aL), else null
    int dcl_pitch;                 // row pitch of dcL in floats
    int64_t q_bs, kv_bs;           // batch strides of q and of the cache, in elements
    int H, A, F, b1, b2, n_keys, n_q;
    int bh0;                       // first (batch, head) pair of this slice
    int g0, g1;                    // cached groups whose dK / dV are wanted
    int causal_groups;             // block-causal: query group a sees cached groups < (a / cg + 1) * cg; 0 = all

    __device__ __forceinline__ int groups_seen(int a) const {
        return causal_groups > 0 ? min(F, (a / causal_groups + 1) * causal_groups) : F;
    }
    float scale, rs;               // softmax scale and its square root
    Blocking blk;
};

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float2 bf2(uint32_t w) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
}
__device__ __forceinline__ float f2_hsum(uint64_t v) {
    float lo, hi;
    f2_unpack(v, lo, hi);
    return lo + hi;
}

// K or V rows [b2][128] bf16 of cached group f, block row k -> shared memory (row stride kKs).
__device__ __forceinline__ void load_kv_tile(uint32_t* dst, const bf16* src_row0, int64_t tok_stride, int b2, int tid,
                                             int nthr) {
    for (int idx = tid; idx < b2 * 16; idx += nthr) {
        const int l = idx >> 4, c = idx & 15;
        const uint4 u = *reinterpret_cast<const uint4*>(src_row0 + (int64_t)l * tok_stride + c * 8);
        uint2* d = reinterpret_cast<uint2*>(dst + l * (kKs / 2) + c * 4);
        d[0] = make_uint2(u.x, u.y); d[1] = make_uint2(u.z, u.w);
    }
}

// 4 consecutive bf16 -> 4 floats
__device__ __forceinline__ float4 ld4(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = bf2(u.x), b = bf2(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
}

// ---------------------------------------------------------------------------------------------------------
// 1. forward recompute of the row step.  grid (n_keys, slice of batch*head), 256 threads; a warp per pair of unit rows.
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bwd_row_forward_kernel(const BwdParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int b2 = p.b2, n = blockIdx.x, f = n / p.b1, k = n - f * p.b1;
    const int bhl = blockIdx.y, bh = p.bh0 + bhl, b = bh / p.H, hd = bh - b * p.H;
    uint32_t* Ks = reinterpret_cast<uint32_t*>(smem);
    uint32_t* Vs = Ks + kv_tile_words(b2);
    float* qrow = reinterpret_cast<float*>(Vs + kv_tile_words(b2));      // [8 warps][2 rows][128]
    float* rrow = qrow + 8 * 2 * kD;                                   // [8 warps][2 rows][128]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t tok = (int64_t)p.H * kD;
    const int64_t kv_off = (int64_t)b * p.kv_bs + ((int64_t)n * b2) * tok + hd * kD;
    load_kv_tile(Ks, p.k + kv_off, tok, b2, threadIdx.x, 256);
    load_kv_tile(Vs, p.v + kv_off, tok, b2, threadIdx.x, 256);
    __syncthreads();
    float* qs = qrow + warp * 2 * kD;                                  // two unit rows per warp at a time
    float* rs_ = rrow + warp * 2 * kD;
    const int n_rows = p.A * b2;
    for (int row0 = warp; row0 < n_rows; row0 += 16) {
        // rows row0 and row0 + 8 share every K / V element read from shared memory; a missing second row repeats the first
        const bool two = row0 + 8 < n_rows;
        int64_t out_at[2], cl_at[2];
        __syncwarp();
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int row = row0 + ((e == 1 && two) ? 8 : 0);
            const int a = row / b2, j = row - a * b2;
            const bf16* qp = p.q + (int64_t)b * p.q_bs + (int64_t)(p.blk.row_token(a, k) + j) * tok + hd * kD;
            const float4 q4 = ld4(qp + lane * 4);
            *reinterpret_cast<float4*>(qs + e * kD + lane * 4) = make_float4(q4.x * p.rs, q4.y * p.rs, q4.z * p.rs, q4.w * p.rs);
            const int64_t slab = ((int64_t)bhl * p.A + a) * b2 + j;
            cl_at[e] = slab * p.n_keys + n;
            out_at[e] = cl_at[e] * kD;
        }
        __syncwarp();
        float z[2][4];
        // key columns lane + 32 u, two at a time: the broadcast reads of the two q^ rows serve both
#pragma unroll
        for (int u = 0; u < 4; u += 2) {
            const int l0 = lane + 32 * u, l1 = l0 + 32;
            z[0][u] = z[1][u] = z[0][u + 1] = z[1][u + 1] = -INFINITY;
            if (32 * u < b2) {                                          // warp-uniform
                const uint32_t* kr0 = Ks + min(l0, b2 - 1) * (kKs / 2);   // lanes past the end recompute the last column
                const uint32_t* kr1 = Ks + min(l1, b2 - 1) * (kKs / 2);
                uint64_t acc[2][2] = {{0, 0}, {0, 0}};                  // [row][column], packed (even d, odd d) partial sums
#pragma unroll 4
                for (int w = 0; w < kD / 4; ++w) {
                    const uint2 kw0 = *reinterpret_cast<const uint2*>(kr0 + 2 * w);
                    const uint2 kw1 = *reinterpret_cast<const uint2*>(kr1 + 2 * w);
                    const float2 a0 = bf2(kw0.x), a1 = bf2(kw0.y), b0 = bf2(kw1.x), b1 = bf2(kw1.y);
                    const uint64_t ka0 = f2_pack(a0.x, a0.y), ka1 = f2_pack(a1.x, a1.y);
                    const uint64_t kb0 = f2_pack(b0.x, b0.y), kb1 = f2_pack(b1.x, b1.y);
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const ulonglong2 qv = *reinterpret_cast<const ulonglong2*>(qs + e * kD + 4 * w);
                        acc[e][0] = f2_fma(qv.x, ka0, acc[e][0]); acc[e][0] = f2_fma(qv.y, ka1, acc[e][0]);
                        acc[e][1] = f2_fma(qv.x, kb0, acc[e][1]); acc[e][1] = f2_fma(qv.y, kb1, acc[e][1]);
                    }
                }
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    if (l0 < b2) z[e][u] = f2_hsum(acc[e][0]) * p.rs;
                    if (l1 < b2) z[e][u + 1] = f2_hsum(acc[e][1]) * p.rs;
                }
            }
        }
        float cl[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float mx = wmax(fmaxf(fmaxf(z[e][0], z[e][1]), fmaxf(z[e][2], z[e][3])));
            float ex[4], sum = 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) { ex[u] = (lane + 32 * u < b2) ? __expf(z[e][u] - mx) : 0.f; sum += ex[u]; }
            sum = wsum(sum);
            const float lse = mx + __logf(sum), inv = 1.f / sum;
            float c = 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int l = lane + 32 * u;
                if (l < b2) {
                    const float r = ex[u] * inv;
                    rs_[e * kD + l] = r;
                    c += r * (z[e][u] - lse);
                }
            }
            cl[e] = wsum(c);
        }
        __syncwarp();
        uint64_t a01[2] = {0, 0}, a23[2] = {0, 0}, y01[2] = {0, 0}, y23[2] = {0, 0};
#pragma unroll 2
        for (int l = 0; l < b2; ++l) {
            const float2 k0 = bf2(Ks[l * (kKs / 2) + lane]), k1 = bf2(Ks[l * (kKs / 2) + 32 + lane]);
            const float2 v0 = bf2(Vs[l * (kKs / 2) + lane]), v1 = bf2(Vs[l * (kKs / 2) + 32 + lane]);
            const uint64_t k01 = f2_pack(k0.x, k0.y), k23 = f2_pack(k1.x, k1.y);
            const uint64_t v01 = f2_pack(v0.x, v0.y), v23 = f2_pack(v1.x, v1.y);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float r = rs_[e * kD + l];
                const uint64_t r2 = f2_pack(r, r);
                a01[e] = f2_fma(r2, k01, a01[e]); a23[e] = f2_fma(r2, k23, a23[e]);
                y01[e] = f2_fma(r2, v01, y01[e]); y23[e] = f2_fma(r2, v23, y23[e]);
            }
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            if (e == 0 || two) {
                float a0, a1, a2, a3, y0, y1, y2, y3;
                f2_unpack(a01[e], a0, a1); f2_unpack(a23[e], a2, a3);
                f2_unpack(y01[e], y0, y1); f2_unpack(y23[e], y2, y3);
                const int64_t o = out_at[e];
                *reinterpret_cast<float2*>(p.aL + o + 2 * lane) = make_float2(a0 * p.rs, a1 * p.rs);
                *reinterpret_cast<float2*>(p.aL + o + 64 + 2 * lane) = make_float2(a2 * p.rs, a3 * p.rs);
                *reinterpret_cast<float2*>(p.Y + o + 2 * lane) = make_float2(y0, y1);
                *reinterpret_cast<float2*>(p.Y + o + 64 + 2 * lane) = make_float2(y2, y3);
                if (lane == 0) p.cL[cl_at[e]] = cl[e];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// 2. column step backward.  grid (A * b2, slice of batch*head), 256 threads.  T = query rows per warp
//    (row i = warp + 8 t), so block rows up to 8 T.
// ---------------------------------------------------------------------------------------------------------
template <int T>
__global__ void __launch_bounds__(256) bwd_col_kernel(const BwdParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int kRows = 8 * T;
    float* qs = reinterpret_cast<float*>(smem);        // [kRows][kQs]   q^ rows (zero beyond b1)
    float* dos = qs + kRows * kQs;                     // [kRows][kQs]   dOut rows
    float* aLs = dos + kRows * kQs;                    // [kTileN][kFs]
    float* Ys = aLs + kTileN * kFs;                    // [kTileN][kFs]
    float* sP = Ys + kTileN * kFs;                     // [kRows][kTileN]
    float* sDS = sP + kRows * kTileN;            // [kRows][kTileN]
    float* cls = sDS + kRows * kTileN;           // [kTileN]
    const int b1 = p.b1, b2 = p.b2, a = blockIdx.x / b2, j = blockIdx.x - a * b2;
    const int bhl = blockIdx.y, bh = p.bh0 + bhl, b = bh / p.H, hd = bh - b * p.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int64_t tok = (int64_t)p.H * kD;
    const int64_t slab = ((int64_t)bhl * p.A + a) * b2 + j;
    float* g_aL = p.aL + slab * p.n_keys * kD;
    float* g_Y = p.Y + slab * p.n_keys * kD;
    const float* g_cL = p.cL + slab * p.n_keys;
    float* g_dcL = p.dcL + slab * p.n_keys;
    const int n_seen = p.groups_seen(a) * b1;          // keys beyond are masked: the row kernel treats their gradients as zero

    for (int idx = tid; idx < kRows * 32; idx += 256) {
        const int i = idx >> 5, c = idx & 31;
        float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f), d4 = q4;
        if (i < b1) {
            const int64_t t = p.blk.row_token(a, i) + j;
            q4 = ld4(p.q + (int64_t)b * p.q_bs + t * tok + hd * kD + c * 4);
            d4 = ld4(p.dout + ((int64_t)b * p.n_q + t) * tok + hd * kD + c * 4);
        }
        *reinterpret_cast<float4*>(qs + i * kQs + c * 4) = make_float4(q4.x * p.rs, q4.y * p.rs, q4.z * p.rs, q4.w * p.rs);
        *reinterpret_cast<float4*>(dos + i * kQs + c * 4) = d4;
    }

    float m[T], ls[T], delta[T];
    uint64_t dq[T][2];                                 // packed: head-dim elements (lane, lane + 32), (lane + 64, lane + 96)
#pragma unroll
    for (int t = 0; t < T; ++t) {
        m[t] = -INFINITY; ls[t] = 0.f; delta[t] = 0.f;
        dq[t][0] = 0; dq[t][1] = 0;
    }

    for (int pass = 0; pass < 2; ++pass) {
        for (int t0 = 0; t0 < n_seen; t0 += kTileN) {
            __syncthreads();                           // previous tile's readers are done (also covers qs / dos)
            for (int idx = tid; idx < kTileN * 32; idx += 256) {
                const int n = idx >> 5, c = idx & 31;
                float4 a4 = make_float4(0.f, 0.f, 0.f, 0.f), y4 = a4;
                if (t0 + n < n_seen) {
                    a4 = *reinterpret_cast<const float4*>(g_aL + (int64_t)(t0 + n) * kD + c * 4);
                    y4 = *reinterpret_cast<const float4*>(g_Y + (int64_t)(t0 + n) * kD + c * 4);
                }
                *reinterpret_cast<float4*>(aLs + n * kFs + c * 4) = a4;
                *reinterpret_cast<float4*>(Ys + n * kFs + c * 4) = y4;
            }
            if (tid < kTileN) cls[tid] = (t0 + tid < n_seen) ? g_cL[t0 + tid] : 0.f;
            __syncthreads();

            // logits (and dP = dOut_i . Y_n) for key `lane`, rows warp + 8 t
            const bool valid = t0 + lane < n_seen;
            float s[T], dp[T];
            {
                uint64_t s2[T], dp2[T];                               // packed (even d, odd d) partial sums
#pragma unroll
                for (int t = 0; t < T; ++t) { s2[t] = 0; dp2[t] = 0; }
                const float* ar = aLs + lane * kFs;
                const float* yr = Ys + lane * kFs;
#pragma unroll 2
                for (int d = 0; d < kD; d += 4) {
                    const ulonglong2 av = *reinterpret_cast<const ulonglong2*>(ar + d);
                    const ulonglong2 yv = *reinterpret_cast<const ulonglong2*>(yr + d);
#pragma unroll
                    for (int t = 0; t < T; ++t) {
                        const ulonglong2 qv = *reinterpret_cast<const ulonglong2*>(qs + (warp + 8 * t) * kQs + d);
                        const ulonglong2 ov = *reinterpret_cast<const ulonglong2*>(dos + (warp + 8 * t) * kQs + d);
                        s2[t] = f2_fma(qv.x, av.x, s2[t]); s2[t] = f2_fma(qv.y, av.y, s2[t]);
                        dp2[t] = f2_fma(ov.x, yv.x, dp2[t]); dp2[t] = f2_fma(ov.y, yv.y, dp2[t]);
                    }
                }
#pragma unroll
                for (int t = 0; t < T; ++t) { s[t] = f2_hsum(s2[t]); dp[t] = f2_hsum(dp2[t]); }
            }
            const float cl = cls[lane];
#pragma unroll
            for (int t = 0; t < T; ++t) s[t] = valid ? s[t] - cl : -INFINITY;

            if (pass == 0) {
                // running maximum, sum of exponentials and sum of exponentials x dP (rescaled together)
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    const float mn = fmaxf(m[t], wmax(s[t]));
                    const float e = valid ? __expf(s[t] - mn) : 0.f;
                    const float c = __expf(m[t] - mn);
                    ls[t] = ls[t] * c + wsum(e);
                    delta[t] = delta[t] * c + wsum(e * dp[t]);
                    m[t] = mn;
                }
                continue;
            }
            // pass 1
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const float pr = valid ? __expf(s[t] - m[t]) : 0.f;          // m holds the log-sum-exp now
                sP[(warp + 8 * t) * kTileN + lane] = pr;
                sDS[(warp + 8 * t) * kTileN + lane] = pr * (dp[t] - delta[t]);
            }
            __syncthreads();
            // dq^_i += sum_n ds[i][n] aL_n
            for (int n = 0; n < kTileN; ++n) {
                const float* ar = aLs + n * kFs + lane;
                const uint64_t a01 = f2_pack(ar[0], ar[32]), a23 = f2_pack(ar[64], ar[96]);
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    const float ds = sDS[(warp + 8 * t) * kTileN + n];
                    const uint64_t ds2 = f2_pack(ds, ds);
                    dq[t][0] = f2_fma(ds2, a01, dq[t][0]);
                    dq[t][1] = f2_fma(ds2, a23, dq[t][1]);
                }
            }
            // daL_n = sum_i ds q^_i, dY_n = sum_i P dOut_i for keys warp + 8 v; written over aL / Y
            {
                uint64_t ga[4][2], gy[4][2];                       // packed like dq
#pragma unroll
                for (int v = 0; v < 4; ++v) { ga[v][0] = ga[v][1] = 0; gy[v][0] = gy[v][1] = 0; }
#pragma unroll 2
                for (int i = 0; i < b1; ++i) {
                    const float* qr = qs + i * kQs + lane;
                    const float* dr = dos + i * kQs + lane;
                    const uint64_t q01 = f2_pack(qr[0], qr[32]), q23 = f2_pack(qr[64], qr[96]);
                    const uint64_t d01 = f2_pack(dr[0], dr[32]), d23 = f2_pack(dr[64], dr[96]);
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const float ds = sDS[i * kTileN + warp + 8 * v];
                        const float pr = sP[i * kTileN + warp + 8 * v];
                        const uint64_t ds2 = f2_pack(ds, ds), pr2 = f2_pack(pr, pr);
                        ga[v][0] = f2_fma(ds2, q01, ga[v][0]); ga[v][1] = f2_fma(ds2, q23, ga[v][1]);
                        gy[v][0] = f2_fma(pr2, d01, gy[v][0]); gy[v][1] = f2_fma(pr2, d23, gy[v][1]);
                    }
                }
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const int n = t0 + warp + 8 * v;
                    if (n < n_seen) {
                        float a[4], y[4];
                        f2_unpack(ga[v][0], a[0], a[1]); f2_unpack(ga[v][1], a[2], a[3]);
                        f2_unpack(gy[v][0], y[0], y[1]); f2_unpack(gy[v][1], y[2], y[3]);
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            g_aL[(int64_t)n * kD + lane + 32 * u] = a[u];
                            g_Y[(int64_t)n * kD + lane + 32 * u] = y[u];
                        }
                    }
                }
            }
            if (tid < kTileN && t0 + tid < n_seen) {
                float acc = 0.f;
                for (int i = 0; i < b1; ++i) acc += sDS[i * kTileN + tid];
                g_dcL[t0 + tid] = -acc;
            }
        }
        if (pass == 0) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                delta[t] = delta[t] / ls[t];
                m[t] = m[t] + __logf(ls[t]);
            }
        }
    }
    // dQ = sqrt(scale) dq^ (the row kernel adds its share afterwards)
#pragma unroll
    for (int t = 0; t < T; ++t) {
        const int i = warp + 8 * t;
        if (i < b1) {
            float* o = p.dq + (((int64_t)b * p.n_q + p.blk.row_token(a, i) + j) * p.H + hd) * kD;
            float g[4];
            f2_unpack(dq[t][0], g[0], g[1]);
            f2_unpack(dq[t][1], g[2], g[3]);
#pragma unroll
            for (int u = 0; u < 4; ++u) o[lane + 32 * u] = g[u] * p.rs;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// 3. row step backward.  grid (b1, slice of batch*head), 512 threads.  Per cached group f: phase 1, a warp per
//    unit row (a, j), leaves R, dz, q^, daL, dY of a batch of rows in shared memory and adds the unit's
//    share to dQ; phase 2, thread (d = tid % 128, l = tid / 128 + 4 t), accumulates dK[l][d], dV[l][d] over
//    the batch.  LT = key columns per thread (block columns up to 4 LT).
// ---------------------------------------------------------------------------------------------------------
template <int LT>
__global__ void __launch_bounds__(512) bwd_row_kernel(const BwdParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int b2 = p.b2, k = blockIdx.x;
    const int bhl = blockIdx.y, bh = p.bh0 + bhl, b = bh / p.H, hd = bh - b * p.H;
    uint32_t* Ks = reinterpret_cast<uint32_t*>(smem);
    uint32_t* Vs = Ks + kv_tile_words(b2);
    float* qS = reinterpret_cast<float*>(Vs + kv_tile_words(b2));      // [kRowBatch][128]
    float* daS = qS + kRowBatch * kD;
    float* dyS = daS + kRowBatch * kD;
    float* Rs = dyS + kRowBatch * kD;                                // [kRowBatch][4][LT]: column l at [l % 4][l / 4]
    float* dzs = Rs + kRowBatch * 4 * LT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int d_own = tid & 127, lq = tid >> 7;
    const int64_t tok = (int64_t)p.H * kD;
    const int n_rows = p.A * b2;

    // blockIdx.z halves the cached groups; the second half adds up its dQ share in dq2 (merged afterwards)
    const int f_half = (p.F + (int)gridDim.z - 1) / (int)gridDim.z;
    const int f_begin = blockIdx.z * f_half, f_end = min(p.F, f_begin + f_half);
    float* const dq_out = blockIdx.z == 0 ? p.dq : p.dq2;
    for (int f = f_begin; f < f_end; ++f) {
        const int n = f * p.b1 + k;
        const int64_t kv_off = (int64_t)b * p.kv_bs + ((int64_t)n * b2) * tok + hd * kD;
        __syncthreads();                                             // the previous group's readers are done
        load_kv_tile(Ks, p.k + kv_off, tok, b2, tid, 512);
        load_kv_tile(Vs, p.v + kv_off, tok, b2, tid, 512);
        uint64_t accK[LT / 2], accV[LT / 2];                         // packed pairs: columns lq + 4 (2 i), lq + 4 (2 i + 1)
#pragma unroll
        for (int t = 0; t < LT / 2; ++t) { accK[t] = 0; accV[t] = 0; }
        __syncthreads();

        for (int r0 = 0; r0 < n_rows; r0 += kRowBatch) {
            // ---- phase 1: each warp takes rows r0 + warp and r0 + warp + 16 together, so that every K / V element it
            //      reads from shared memory serves both; a missing second row repeats the first into a slot nobody reads
            if (r0 + warp < n_rows) {
                const bool two = r0 + warp + 16 < n_rows;
                int64_t t_nat[2];
                float dcl[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int row = r0 + warp + ((e == 1 && two) ? 16 : 0);
                    const int slot = warp + 16 * e;
                    const int a = row / b2, j = row - a * b2;
                    t_nat[e] = p.blk.row_token(a, k) + j;
                    const int64_t slab = ((int64_t)bhl * p.A + a) * b2 + j;
                    const int64_t o = (slab * p.n_keys + n) * kD;
                    const float4 q4 = ld4(p.q + (int64_t)b * p.q_bs + t_nat[e] * tok + hd * kD + lane * 4);
                    // a pair (a, f) the query group may not see has zero gradients (its scratch rows still hold forward values)
                    const bool seen = f < p.groups_seen(a);
                    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
                    float4 a4 = zero4, y4 = zero4;
                    if (seen) {
                        if (p.aLb) {            // bf16 gradients of the unscaled aL: daL of the scaled one = that / sqrt(scale)
                            const float4 t4 = ld4(p.aLb + o + lane * 4);
                            const float ir = 1.0f / p.rs;
                            a4 = make_float4(t4.x * ir, t4.y * ir, t4.z * ir, t4.w * ir);
                            y4 = ld4(p.Yb + o + lane * 4);
                        } else {
                            a4 = *reinterpret_cast<const float4*>(p.aL + o + lane * 4);
                            y4 = *reinterpret_cast<const float4*>(p.Y + o + lane * 4);
                        }
                    }
                    dcl[e] = seen ? p.dcL[slab * p.dcl_pitch + n] : 0.f;
                    *reinterpret_cast<float4*>(qS + slot * kD + lane * 4) =
                        make_float4(q4.x * p.rs, q4.y * p.rs, q4.z * p.rs, q4.w * p.rs);
                    *reinterpret_cast<float4*>(daS + slot * kD + lane * 4) = a4;
                    *reinterpret_cast<float4*>(dyS + slot * kD + lane * 4) = y4;
                }
                __syncwarp();
                float z[2][4], ga[2][4];
                // key columns lane + 32 u, two at a time (u, u + 1): the broadcast reads of the q^ / daL / dY rows serve both
#pragma unroll
                for (int u = 0; u < 4; u += 2) {
                    const int l0 = lane + 32 * u, l1 = l0 + 32;
                    z[0][u] = z[1][u] = z[0][u + 1] = z[1][u + 1] = -INFINITY;
                    ga[0][u] = ga[1][u] = ga[0][u + 1] = ga[1][u + 1] = 0.f;
                    if (32 * u < b2) {                                  // warp-uniform: some lane has a column in this pair
                        const int c0 = min(l0, b2 - 1), c1 = min(l1, b2 - 1);          // lanes past the end recompute the last column
                        const uint32_t* kr0 = Ks + c0 * (kKs / 2);
                        const uint32_t* vr0 = Vs + c0 * (kKs / 2);
                        const uint32_t* kr1 = Ks + c1 * (kKs / 2);
                        const uint32_t* vr1 = Vs + c1 * (kKs / 2);
                        uint64_t az[2][2] = {{0, 0}, {0, 0}}, aa[2][2] = {{0, 0}, {0, 0}}, ay[2][2] = {{0, 0}, {0, 0}};   // [row][column]
#pragma unroll 2
                        for (int w = 0; w < kD / 4; ++w) {
                            uint64_t kk[2][2], vv[2][2];                                 // [column][d pair]
                            {
                                const uint2 kw = *reinterpret_cast<const uint2*>(kr0 + 2 * w);
                                const uint2 vw = *reinterpret_cast<const uint2*>(vr0 + 2 * w);
                                const float2 k0 = bf2(kw.x), k1 = bf2(kw.y), v0 = bf2(vw.x), v1 = bf2(vw.y);
                                kk[0][0] = f2_pack(k0.x, k0.y); kk[0][1] = f2_pack(k1.x, k1.y);
                                vv[0][0] = f2_pack(v0.x, v0.y); vv[0][1] = f2_pack(v1.x, v1.y);
                            }
                            {
                                const uint2 kw = *reinterpret_cast<const uint2*>(kr1 + 2 * w);
                                const uint2 vw = *reinterpret_cast<const uint2*>(vr1 + 2 * w);
                                const float2 k0 = bf2(kw.x), k1 = bf2(kw.y), v0 = bf2(vw.x), v1 = bf2(vw.y);
                                kk[1][0] = f2_pack(k0.x, k0.y); kk[1][1] = f2_pack(k1.x, k1.y);
                                vv[1][0] = f2_pack(v0.x, v0.y); vv[1][1] = f2_pack(v1.x, v1.y);
                            }
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int slot = warp + 16 * e;
                                const ulonglong2 qv = *reinterpret_cast<const ulonglong2*>(qS + slot * kD + 4 * w);
                                const ulonglong2 av = *reinterpret_cast<const ulonglong2*>(daS + slot * kD + 4 * w);
                                const ulonglong2 yv = *reinterpret_cast<const ulonglong2*>(dyS + slot * kD + 4 * w);
#pragma unroll
                                for (int c = 0; c < 2; ++c) {
                                    az[e][c] = f2_fma(qv.x, kk[c][0], az[e][c]); az[e][c] = f2_fma(qv.y, kk[c][1], az[e][c]);
                                    aa[e][c] = f2_fma(av.x, kk[c][0], aa[e][c]); aa[e][c] = f2_fma(av.y, kk[c][1], aa[e][c]);
                                    ay[e][c] = f2_fma(yv.x, vv[c][0], ay[e][c]); ay[e][c] = f2_fma(yv.y, vv[c][1], ay[e][c]);
                                }
                            }
                        }
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            if (l0 < b2) {
                                z[e][u] = f2_hsum(az[e][0]) * p.rs;
                                ga[e][u] = f2_hsum(aa[e][0]) * p.rs + f2_hsum(ay[e][0]);
                            }
                            if (l1 < b2) {
                                z[e][u + 1] = f2_hsum(az[e][1]) * p.rs;
                                ga[e][u + 1] = f2_hsum(aa[e][1]) * p.rs + f2_hsum(ay[e][1]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int slot = warp + 16 * e;
                    float mx = fmaxf(fmaxf(z[e][0], z[e][1]), fmaxf(z[e][2], z[e][3]));
                    mx = wmax(mx);
                    float ex[4], sum = 0.f;
#pragma unroll
                    for (int u = 0; u < 4; ++u) { ex[u] = (lane + 32 * u < b2) ? __expf(z[e][u] - mx) : 0.f; sum += ex[u]; }
                    sum = wsum(sum);
                    const float lse = mx + __logf(sum), inv = 1.f / sum;
                    float r[4], dr[4], rdr = 0.f;
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        r[u] = ex[u] * inv;
                        dr[u] = (lane + 32 * u < b2) ? ga[e][u] + dcl[e] * (z[e][u] - lse + 1.f) : 0.f;
                        rdr += r[u] * dr[u];
                    }
                    rdr = wsum(rdr);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int l = lane + 32 * u;
                        if (l < b2) {
                            const int at = slot * 4 * LT + (l & 3) * LT + (l >> 2);
                            Rs[at] = r[u];
                            dzs[at] = r[u] * (dr[u] - rdr);
                        }
                    }
                }
                __syncwarp();
                uint64_t dq01[2] = {0, 0}, dq23[2] = {0, 0};
#pragma unroll 2
                for (int l = 0; l < b2; ++l) {
                    const float2 k0 = bf2(Ks[l * (kKs / 2) + lane]), k1 = bf2(Ks[l * (kKs / 2) + 32 + lane]);
                    const uint64_t k01 = f2_pack(k0.x, k0.y), k23 = f2_pack(k1.x, k1.y);
                    const int at = (l & 3) * LT + (l >> 2);
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float dz = dzs[(warp + 16 * e) * 4 * LT + at];
                        const uint64_t dz2 = f2_pack(dz, dz);
                        dq01[e] = f2_fma(dz2, k01, dq01[e]);
                        dq23[e] = f2_fma(dz2, k23, dq23[e]);
                    }
                }
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    if (e == 0 || two) {
                        float d0, d1, d2, d3;
                        f2_unpack(dq01[e], d0, d1);
                        f2_unpack(dq23[e], d2, d3);
                        float* g = dq_out + (((int64_t)b * p.n_q + t_nat[e]) * p.H + hd) * kD;
                        float2 g0 = make_float2(0.f, 0.f), g1 = g0;
                        if (blockIdx.z == 0 || f > f_begin) {            // dq2 starts from nothing
                            g0 = *reinterpret_cast<float2*>(g + 2 * lane);
                            g1 = *reinterpret_cast<float2*>(g + 64 + 2 * lane);
                        }
                        g0.x += p.scale * d0; g0.y += p.scale * d1;
                        g1.x += p.scale * d2; g1.y += p.scale * d3;
                        *reinterpret_cast<float2*>(g + 2 * lane) = g0;
                        *reinterpret_cast<float2*>(g + 64 + 2 * lane) = g1;
                    }
                }
            }
            __syncthreads();
            // ---- phase 2
            const int nb = min(kRowBatch, n_rows - r0);
            for (int rr = 0; rr < nb; ++rr) {
                const float qd = qS[rr * kD + d_own], ad = daS[rr * kD + d_own], yd = dyS[rr * kD + d_own];
                const uint64_t qd2 = f2_pack(qd, qd), ad2 = f2_pack(ad, ad), yd2 = f2_pack(yd, yd);
                // columns beyond b2 hold whatever shared memory held: they only reach accumulators that are never stored
#pragma unroll
                for (int t = 0; t < LT; t += 4) {
                    const ulonglong2 rv = *reinterpret_cast<const ulonglong2*>(Rs + rr * 4 * LT + lq * LT + t);
                    const ulonglong2 dz = *reinterpret_cast<const ulonglong2*>(dzs + rr * 4 * LT + lq * LT + t);
                    accK[t / 2] = f2_fma(rv.x, ad2, f2_fma(dz.x, qd2, accK[t / 2]));
                    accK[t / 2 + 1] = f2_fma(rv.y, ad2, f2_fma(dz.y, qd2, accK[t / 2 + 1]));
                    accV[t / 2] = f2_fma(rv.x, yd2, accV[t / 2]);
                    accV[t / 2 + 1] = f2_fma(rv.y, yd2, accV[t / 2 + 1]);
                }
            }
            __syncthreads();
        }
        if (f >= p.g0 && f < p.g1) {
            const int64_t base = (int64_t)b * (p.g1 - p.g0) * p.b1 * b2 + ((int64_t)(f - p.g0) * p.b1 + k) * b2;
#pragma unroll
            for (int t = 0; t < LT; t += 2) {
                float gk[2], gv[2];
                f2_unpack(accK[t / 2], gk[0], gk[1]);
                f2_unpack(accV[t / 2], gv[0], gv[1]);
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int l = lq + 4 * (t + e);
                    if (l < b2) {
                        const int64_t o = ((base + l) * p.H + hd) * kD + d_own;
                        p.dk[o] = __float2bfloat16(gk[e] * p.rs);
                        p.dv[o] = __float2bfloat16(gv[e]);
                    }
                }
            }
        }
    }
}

}  // namespace

namespace {
// dq += dq2 for the heads of one slice.  grid (n_q, slice of batch*head), 32 threads: one token row of one head.
__global__ void bwd_merge_dq_kernel(const BwdParams p) {
    const int bh = p.bh0 + blockIdx.y, b = bh / p.H, hd = bh - b * p.H;
    const int64_t o = (((int64_t)b * p.n_q + blockIdx.x) * p.H + hd) * kD + threadIdx.x * 4;
    float4 a = *reinterpret_cast<float4*>(p.dq + o);
    const float4 c = *reinterpret_cast<const float4*>(p.dq2 + o);
    a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
    *reinterpret_cast<float4*>(p.dq + o) = a;
}

constexpr size_t kDefaultBwdBudget = (size_t)2 << 30;     // scratch per slice of (batch, head) pairs

inline size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

struct BwdPlan {
    Blocking blk;
    int A, F, n_keys, nbh;
    size_t off_aL, off_Y, off_cL, off_dcL, off_dq2, total;
};

int make_bwd_plan(BwdPlan* pl, int B, int H, int D, int n_q, int n_kv, int f_tied, int h_reduce, int w_reduce, int h,
                  int w, size_t budget) {
    if (D != kHeadDim) return SFM_ERR_UNSUPPORTED;
    if (B <= 0 || H <= 0 || n_q <= 0 || n_kv <= 0) return SFM_ERR_BAD_SHAPE;
    if (int rc = make_blocking(&pl->blk, f_tied, h_reduce, w_reduce, h, w)) return rc;
    const Blocking& blk = pl->blk;
    if (blk.b1 > 128 || blk.b2 > 128) return SFM_ERR_UNSUPPORTED;
    if (n_q % blk.tied_tokens) return SFM_ERR_BAD_SHAPE;
    const int group = blk.b1 * blk.b2;
    if (n_kv % group) return SFM_ERR_BAD_SHAPE;
    pl->A = n_q / group;
    pl->F = n_kv / group;
    pl->n_keys = pl->F * blk.b1;
    if (budget == 0) budget = kDefaultBwdBudget;
    const size_t per_bh = (size_t)pl->A * blk.b2 * pl->n_keys * (2 * kHeadDim + 2) * sizeof(float);
    pl->nbh = (int)std::max<size_t>(1, std::min<size_t>((size_t)B * H, budget / per_bh));
    const size_t units = (size_t)pl->nbh * pl->A * blk.b2 * pl->n_keys;
    size_t o = 256;                                   // the status word of the call sits at the start, in both layouts
    pl->off_aL = o; o = up256(o + units * kHeadDim * sizeof(float));
    pl->off_Y = o; o = up256(o + units * kHeadDim * sizeof(float));
    pl->off_cL = o; o = up256(o + units * sizeof(float));
    pl->off_dcL = o; o = up256(o + units * sizeof(float));
    pl->off_dq2 = o; o = up256(o + (size_t)B * n_q * H * kHeadDim * sizeof(float));
    // the tensor-core path lays the same region out differently (bf16 bridge, log-sum-exp, a scratch output,
    // delta, a status word) and never needs more than this
    o += up256((size_t)B * n_q * H * (kHeadDim * 2 + 4)) + up256((size_t)pl->nbh * pl->A * blk.b2 * (blk.b1 + 8) * sizeof(float)) + 4096;
    // its row kernel also keeps one fp32 copy of dK and dV per tile of stacked query groups (worst case: all cached
    // groups wanted); the bf16 bridge leaves half of the fp32 one's space free for them
    {
        const int gpt = 128 / ((blk.b2 + 7) & ~7);
        const size_t tiles = gpt > 0 ? (size_t)(pl->A + gpt - 1) / gpt : 0;
        const size_t parts = 2 * (tiles * pl->nbh * (size_t)n_kv * kHeadDim * sizeof(float) + 256);
        const size_t slack = units * kHeadDim * sizeof(float);
        if (blk.b2 <= 64 && parts > slack) o += up256(parts - slack);
    }
    pl->total = o;
    return SFM_OK;
}

template <typename K>
int opt_in_smem(K kernel, size_t bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) == cudaSuccess ? 0 : 1;
}
}  // namespace
}  // namespace sfm

using namespace sfm;

extern "C" size_t sfm_monarch_bwd_workspace_bytes(int B, int H, int D, int n_q, int n_kv, int f_tied, int h_reduce,
                                                  int w_reduce, int h, int w, size_t budget_bytes) {
    BwdPlan pl;
    if (make_bwd_plan(&pl, B, H, D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, budget_bytes)) return 0;
    return pl.total;
}

extern "C" int sfm_monarch_bwd(const void* q, int64_t q_batch_stride, const void* k_cache, const void* v_cache,
                               int64_t kv_batch_stride, const void* dout, void* dq, void* dk, void* dv, void* workspace,
                               size_t workspace_bytes, int B, int H, int D, int n_q, int n_kv, int f_tied, int h_reduce,
                               int w_reduce, int h, int w, float sm_scale, int kv_group_begin, int kv_group_end,
                               int causal_groups, size_t budget_bytes, void* stream) {
    if (!q || !k_cache || !v_cache || !dout || !dq || !workspace) return SFM_ERR_NULL_POINTER;
    BwdPlan pl;
    if (int rc = make_bwd_plan(&pl, B, H, D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, budget_bytes)) return rc;
    if (!(sm_scale > 0.f)) return SFM_ERR_BAD_SHAPE;
    if (kv_group_begin < 0 || kv_group_end > pl.F || kv_group_begin > kv_group_end) return SFM_ERR_BAD_SHAPE;
    if (causal_groups < 0 || (causal_groups > 0 && (pl.A != pl.F || pl.A % causal_groups))) return SFM_ERR_BAD_SHAPE;
    if (kv_group_end > kv_group_begin && (!dk || !dv)) return SFM_ERR_NULL_POINTER;
    if (workspace_bytes < pl.total) return SFM_ERR_WORKSPACE;
    for (const void* ptr : {q, k_cache, v_cache, dout, (const void*)dq, (const void*)dk, (const void*)dv,
                            (const void*)workspace})
        if (reinterpret_cast<uintptr_t>(ptr) & 15) return SFM_ERR_ALIGNMENT;
    if ((q_batch_stride & 7) || (kv_batch_stride & 7)) return SFM_ERR_ALIGNMENT;

    const Blocking& blk = pl.blk;
    BwdParams p{};
    p.q = (const bf16*)q; p.k = (const bf16*)k_cache; p.v = (const bf16*)v_cache; p.dout = (const bf16*)dout;
    p.dq = (float*)dq; p.dk = (bf16*)dk; p.dv = (bf16*)dv;
    unsigned char* ws = (unsigned char*)workspace;
    p.aL = (float*)(ws + pl.off_aL); p.Y = (float*)(ws + pl.off_Y);
    p.cL = (float*)(ws + pl.off_cL); p.dcL = (float*)(ws + pl.off_dcL);
    p.dq2 = (float*)(ws + pl.off_dq2);
    p.q_bs = q_batch_stride; p.kv_bs = kv_batch_stride;
    p.H = H; p.A = pl.A; p.F = pl.F; p.b1 = blk.b1; p.b2 = blk.b2; p.n_keys = pl.n_keys; p.n_q = n_q;
    p.g0 = kv_group_begin; p.g1 = kv_group_end;
    p.causal_groups = causal_groups;
    p.scale = sm_scale; p.rs = sqrtf(sm_scale);
    p.blk = blk;
    p.aLb = p.Yb = nullptr;
    p.dcl_pitch = pl.n_keys;
    // Tensor-core path: recompute of the forward's row step (and of the column step, for its softmax statistics
    // and output) on the forward's own tcgen05 kernels, column- and row-step backward on tcgen05; block rows up to 96,
    // block columns up to 64, query rows reachable by TMA, no block-causal mask.  SFM_BWD_FP32=1 keeps everything on the fp32 kernels.
    const char* force_fp32 = getenv("SFM_BWD_FP32");
    const bool use_tc = causal_groups == 0 && blk.b1 <= 96 && blk.b2 <= 64 && (blk.f_tied == 1 || blk.h_reduce == 1) &&
                        !(force_fp32 && force_fp32[0] == '1');

    const int T = blk.b1 <= 16 ? 2 : (blk.b1 <= 32 ? 4 : (blk.b1 <= 64 ? 8 : 16));
    const int LT = blk.b2 <= 64 ? 16 : 32;
    const size_t smem_fwd = (size_t)2 * kv_tile_words(blk.b2) * 4 + 2 * 8 * 2 * kD * sizeof(float);
    const size_t smem_col = ((size_t)2 * 8 * T * kQs + 2 * kTileN * kFs + 2 * 8 * T * kTileN + kTileN) * sizeof(float);
    const size_t smem_row = (size_t)2 * kv_tile_words(blk.b2) * 4 +
                            ((size_t)3 * kRowBatch * kD + 2 * kRowBatch * 4 * LT) * sizeof(float);
    int bad = opt_in_smem(bwd_row_forward_kernel, smem_fwd);
    bad |= T == 2 ? opt_in_smem(bwd_col_kernel<2>, smem_col)
                  : (T == 4 ? opt_in_smem(bwd_col_kernel<4>, smem_col)
                            : (T == 8 ? opt_in_smem(bwd_col_kernel<8>, smem_col) : opt_in_smem(bwd_col_kernel<16>, smem_col)));
    bad |= LT == 16 ? opt_in_smem(bwd_row_kernel<16>, smem_row) : opt_in_smem(bwd_row_kernel<32>, smem_row);
    if (bad) return SFM_ERR_UNSUPPORTED;

    cudaStream_t s = (cudaStream_t)stream;
    const int BH = B * H;
    int num_sms = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    // one status word per call: a kernel that gives up on a bounded wait sets it, nothing clears it before the end
    if (cudaMemsetAsync(ws, 0, sizeof(int), s) != cudaSuccess) return SFM_ERR_UNSUPPORTED;
    for (int bh0 = 0; bh0 < BH; bh0 += pl.nbh) {
        const int nbh = std::min(pl.nbh, BH - bh0);
        p.bh0 = bh0;
        if (use_tc) {
            // workspace of this slice: status | aL, Y (bf16 bridge) | cL, dcL | lse | out (scratch) | delta | dq2
            const size_t slabs = (size_t)nbh * pl.A * blk.b2;
            const int n_keys_c = (pl.n_keys + 3) & ~3;
            const size_t rows = (size_t)B * n_q * H;
            size_t o = 0;
            int* status = (int*)(ws + o); o = up256(o + sizeof(int));
            bf16* aLb = (bf16*)(ws + o); o = up256(o + slabs * pl.n_keys * kHeadDim * sizeof(bf16));
            bf16* Yb = (bf16*)(ws + o); o = up256(o + slabs * pl.n_keys * kHeadDim * sizeof(bf16));
            float* cL = (float*)(ws + o); o = up256(o + slabs * n_keys_c * sizeof(float));
            float* dcL = (float*)(ws + o); o = up256(o + slabs * n_keys_c * sizeof(float));
            float* lse = (float*)(ws + o); o = up256(o + slabs * blk.b1 * sizeof(float));
            bf16* out_s = (bf16*)(ws + o); o = up256(o + rows * kHeadDim * sizeof(bf16));
            float* delta = (float*)(ws + o); o = up256(o + rows * sizeof(float));
            p.dq2 = (float*)(ws + o); o = up256(o + rows * kHeadDim * sizeof(float));
            if (o > workspace_bytes) return SFM_ERR_WORKSPACE;
            MonarchParams mp;
            CUtensorMap maps[8];
            int rc = forward_tc_slice(q, q_batch_stride, k_cache, v_cache, kv_batch_stride, out_s, aLb, Yb, cL, lse, status,
                                      B, H, n_q, n_kv, blk, sm_scale, bh0, nbh, &mp, maps, s);
            if (rc) return rc;
            // delta = dOut . out for every (token, head); the scratch output holds this slice's heads only, the
            // other heads' products are never read
            if ((rc = launch_bwd_delta(dout, out_s, delta, (long long)rows, s))) return rc;
            // query rows of q and dOut for the column kernel: (d, head, column, row of the token grid, batch), boxes of
            // 32 consecutive grid rows (fewer when the whole call has fewer)
            {
                const uint64_t row = (uint64_t)kHeadDim * 2, tok = (uint64_t)H * row;
                const uint32_t box_rows = (uint32_t)std::min(32, n_q / blk.w);
                uint64_t dqr[5] = {(uint64_t)kHeadDim, (uint64_t)H, (uint64_t)blk.w, (uint64_t)(n_q / blk.w), (uint64_t)B};
                uint64_t sq_[4] = {row, tok, (uint64_t)blk.w * tok, (uint64_t)q_batch_stride * 2};
                uint64_t sdo[4] = {row, tok, (uint64_t)blk.w * tok, (uint64_t)n_q * tok};
                uint32_t bqr[5] = {64, 1, 1, box_rows, 1};
                if ((rc = make_tmap_bf16(&maps[5], q, 5, dqr, sq_, bqr))) return rc;
                if ((rc = make_tmap_bf16(&maps[6], dout, 5, dqr, sdo, bqr))) return rc;
            }
            CUtensorMap cmaps[4] = {maps[3], maps[4], maps[5], maps[6]};
            if ((rc = launch_bwd_col_tc(mp, cmaps, delta, dcL, p.dq, status, num_sms, s))) return rc;
            p.aLb = aLb; p.Yb = Yb; p.dcL = dcL; p.dcl_pitch = n_keys_c;
            // Row-step backward on tcgen05 when its per-tile dK / dV partials fit what is left of the workspace;
            // SFM_BWD_ROW_FP32=1 keeps the fp32 row kernel.
            const char* row_fp32 = getenv("SFM_BWD_ROW_FP32");
            const size_t part = up256(bwd_row_tc_partial_bytes(mp, p.g0, p.g1));
            if (!(row_fp32 && row_fp32[0] == '1') && o + 2 * part <= workspace_bytes) {
                float* part_k = (float*)(ws + o);
                float* part_v = (float*)(ws + o + part);
                const int rows_per_group = (blk.b2 + 7) & ~7;
                uint64_t db[3] = {(uint64_t)kHeadDim, (uint64_t)pl.n_keys, (uint64_t)slabs};
                uint64_t sb[2] = {(uint64_t)kHeadDim * 2, (uint64_t)pl.n_keys * kHeadDim * 2};
                uint32_t bb[3] = {64, 1, (uint32_t)rows_per_group};
                CUtensorMap rmaps[5] = {maps[0], maps[1], maps[2]};
                if ((rc = make_tmap_bf16(&rmaps[3], aLb, 3, db, sb, bb))) return rc;
                if ((rc = make_tmap_bf16(&rmaps[4], Yb, 3, db, sb, bb))) return rc;
                if ((rc = launch_bwd_row_tc(mp, rmaps, dcL, p.dq, part_k, part_v, p.dk, p.dv, p.g0, p.g1, status, num_sms, s)))
                    return rc;
                continue;
            }
        } else {
        {
            LaunchScope scope(kClsBackward, s);
            bwd_row_forward_kernel<<<dim3(pl.n_keys, nbh), 256, smem_fwd, s>>>(p);
        }
        {
            LaunchScope scope(kClsBackward, s);
            const dim3 grid(pl.A * blk.b2, nbh);
            if (T == 2) bwd_col_kernel<2><<<grid, 256, smem_col, s>>>(p);
            else if (T == 4) bwd_col_kernel<4><<<grid, 256, smem_col, s>>>(p);
            else if (T == 8) bwd_col_kernel<8><<<grid, 256, smem_col, s>>>(p);
            else bwd_col_kernel<16><<<grid, 256, smem_col, s>>>(p);
        }
        }
        {
            LaunchScope scope(kClsBackward, s);
            const int halves = pl.F >= 2 ? 2 : 1;       // 2 x b1 x heads CTAs fill the SMs' rounds more evenly
            const dim3 grid(blk.b1, nbh, halves);
            if (LT == 16) bwd_row_kernel<16><<<grid, 512, smem_row, s>>>(p);
            else bwd_row_kernel<32><<<grid, 512, smem_row, s>>>(p);
            if (halves == 2) bwd_merge_dq_kernel<<<dim3(n_q, nbh), 32, 0, s>>>(p);
        }
    }
    return cudaGetLastError() == cudaSuccess ? SFM_OK : SFM_ERR_UNSUPPORTED;
}
