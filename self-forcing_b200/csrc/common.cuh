// Shared device helpers and the blocking descriptor.  sm_100a only.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sfmonarch.h"

namespace sfm {

constexpr int kHeadDim = 128;            // the only head size the kernels are built for
constexpr int kLds = kHeadDim + 8;       // padded shared-memory row (bf16 elements): conflict-free ldmatrix
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kMaxPeers = 8;             // GPUs of one box that may share a head-sharded call

// Monarch blocking of an h x w token grid (see sfmonarch.h).
struct Blocking {
    int f_tied, h_reduce, w_reduce, h, w;
    int hh, ww;        // rows / columns per band
    int b1, b2;        // block rows (f_tied*hh) and block columns (ww)
    int gpt;           // groups per tied frame set = h_reduce*w_reduce
    int tied_tokens;   // f_tied*h*w

    // Natural-order token index of column 0 of row `r` of group `g` (groups counted over
    // the whole tensor).  Columns j are contiguous from there.
    __host__ __device__ __forceinline__ int row_token(int g, int r) const {
        int a = g / gpt, ce = g - a * gpt;
        int c = ce / w_reduce, e = ce - c * w_reduce;
        int f = r / hh, i = r - f * hh;
        return ((((a * f_tied + f) * h_reduce + c) * hh + i) * w_reduce + e) * ww;
    }
    // Monarch position of natural token n.
    __host__ __device__ __forceinline__ int nat2mon(int n) const {
        int j = n % ww; int t = n / ww;
        int e = t % w_reduce; t /= w_reduce;
        int i = t % hh; t /= hh;
        int c = t % h_reduce; t /= h_reduce;
        int f = t % f_tied; int a = t / f_tied;
        return ((((a * h_reduce + c) * w_reduce + e) * f_tied + f) * hh + i) * ww + j;
    }
};

inline int make_blocking(Blocking* b, int f_tied, int h_reduce, int w_reduce, int h, int w) {
    if (f_tied <= 0 || h_reduce <= 0 || w_reduce <= 0 || h <= 0 || w <= 0) return SFM_ERR_BAD_SHAPE;
    if (h % h_reduce || w % w_reduce) return SFM_ERR_BAD_SHAPE;
    b->f_tied = f_tied; b->h_reduce = h_reduce; b->w_reduce = w_reduce; b->h = h; b->w = w;
    b->hh = h / h_reduce; b->ww = w / w_reduce;
    b->b1 = f_tied * b->hh; b->b2 = b->ww;
    b->gpt = h_reduce * w_reduce;
    b->tied_tokens = f_tied * h * w;
    return SFM_OK;
}

// ---------------------------------------------------------------------------------------
// small PTX wrappers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous global->shared copy; src_bytes == 0 writes zeros.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes = 16) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem)));
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Same packing without the conversion instruction (which issues on the 16-lane transcendental
// pipe, shared with exp2): add half an ulp of bf16 to the fp32 bit patterns and keep the upper
// halves.  Rounds to nearest with ties away from zero in magnitude; Inf stays Inf.
__device__ __forceinline__ uint32_t pack_bf16_alu(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}

// Packed fp32 pairs (sm_100 has two-wide fp32 fma / mul / add on 64-bit register pairs).
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// A-operand fragment (16 rows x 16 k) from a row-major [row][k] shared tile with row pitch kLds.
__device__ __forceinline__ void load_a_frag(uint32_t (&a)[4], const __nv_bfloat16* tile, int row0, int k0, int lane) {
    int mat = lane >> 3, r = lane & 7;
    ldmatrix_x4(a, tile + (row0 + (mat & 1) * 8 + r) * kLds + k0 + (mat >> 1) * 8);
}
// B-operand fragments for two adjacent 8-wide n tiles (n0, n0+8) and one 16-deep k step, from a
// tile stored [n][k] (the contraction index contiguous): b[0],b[1] -> tile n0; b[2],b[3] -> n0+8.
__device__ __forceinline__ void load_b_frag_nk(uint32_t (&b)[4], const __nv_bfloat16* tile, int n0, int k0, int lane) {
    int mat = lane >> 3, r = lane & 7;
    ldmatrix_x4(b, tile + (n0 + (mat >> 1) * 8 + r) * kLds + k0 + (mat & 1) * 8);
}
// Same, from a tile stored [k][n] (the contraction index is the row): uses the transposing load.
__device__ __forceinline__ void load_b_frag_kn(uint32_t (&b)[4], const __nv_bfloat16* tile, int n0, int k0, int lane) {
    int mat = lane >> 3, r = lane & 7;
    ldmatrix_x4_trans(b, tile + (k0 + (mat & 1) * 8 + r) * kLds + n0 + (mat >> 1) * 8);
}

}  // namespace sfm
