// Layout maps, rotary table and the fused RoPE + layout + in-place KV-cache write kernel.
#include <math.h>

#include "common.cuh"
#include "profile.cuh"

namespace sfm {

// One CTA moves one token: all heads x 16 vectors of 16 bytes (8 bf16 = 4 rotary pairs) of q, k and
// v.  The token's position arithmetic (grid coordinates, Monarch slot) is done once per CTA and its
// 64 (cos, sin) pairs are staged in shared memory for all heads.  Reads and writes are 16-byte
// vectors; consecutive threads cover consecutive 256-byte rows.  The kernel is HBM bound: it reads
// 3 tensors and writes 3 (2 when q is absent).
//
// Sources may be sharded by token over up to kMaxPeers GPUs of one box (head-sharded attention): token n
// then lives in buffer n / src_tokens, a [B, src_tokens, src_heads, 128] tensor of which this GPU takes
// heads [head0, head0 + H).  Buffers of other GPUs are read with plain loads over NVLink.  Unsharded
// input is the case of one buffer with src_tokens = n_new, src_heads = H, head0 = 0.
//
// Sliding-window eviction (causal_model.py:912-926) can ride along: before the new tokens land, the cached
// tokens after the sink move left by `roll_shift` positions, cache[p] = cache[p + roll_shift] for
// roll_dst <= p < start_idx, and the new tokens follow them at start_idx.  The move overlaps itself, but it
// splits into independent chains p, p + shift, p + 2 shift, ... one per residue of p; the chain that ends at
// position start_idx + m is walked, front to back, by the CTA that afterwards writes the new token of slot
// m < shift there (every element is read before the same thread overwrites it), so the whole eviction needs
// no temporary and no ordering between CTAs.
struct PeerSrc {
    const uint4* q[kMaxPeers];
    const uint4* k[kMaxPeers];
    const uint4* v[kMaxPeers];
};

__global__ void __launch_bounds__(256)
rope_cache_write_kernel(const __grid_constant__ PeerSrc src, int src_tokens, int src_heads, int head0,
                        uint4* __restrict__ q_out, uint4* k_cache, uint4* v_cache,
                        long long cache_batch_stride_vec, const float2* __restrict__ rope,
                        int B, int n_new, int H, int start_idx, Blocking blk, int start_frame,
                        int monarch_order, int p0, int p1,
                        const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk, float eps,
                        int roll_dst, int roll_shift, int rope_tok0) {
    constexpr int kVecPerRow = kHeadDim / 8;  // 16
    __shared__ float2 cs_s[kHeadDim / 2];
    __shared__ float red_s[2][8];
    __shared__ float rs_s[2];                  // 1/rms of the token's q and k rows (full width)
    const int frame_tokens = blk.h * blk.w;
    for (long long bn = blockIdx.x; bn < (long long)B * n_new; bn += gridDim.x) {
        const int n = (int)(bn % n_new);
        const int b = (int)(bn / n_new);
        if (rope) {
            __syncthreads();                                    // previous token's table no longer in use
            for (int m = threadIdx.x; m < kHeadDim / 2; m += blockDim.x) {   // m: rotary pair index within the head
                const int np = n + rope_tok0;                   // position in the chunk's token grid (token slices)
                const int fr = np / frame_tokens, rem = np - fr * frame_tokens;
                const int rw = rem / blk.w, cl = rem - rw * blk.w;
                const int pos = m < p0 ? start_frame + fr : (m < p0 + p1 ? rw : cl);
                cs_s[m] = rope[pos * (kHeadDim / 2) + m];
            }
            __syncthreads();
        }
        const int dst_tok = start_idx + (monarch_order ? blk.nat2mon(n) : n);
        const int peer = n / src_tokens;
        const uint4* __restrict__ q = src.q[peer];
        const uint4* __restrict__ k = src.k[peer];
        const uint4* __restrict__ v = src.v[peer];
        const long long src_vec0 = (((long long)b * src_tokens + (n - peer * src_tokens)) * src_heads + head0) * kVecPerRow;
        const long long out_vec0 = bn * H * kVecPerRow;
        if (wk) {
            // RMS normalisation over the token's full width (all heads), q and k separately
            float sq = 0.f, sk = 0.f;
            for (int t = threadIdx.x; t < H * kVecPerRow; t += blockDim.x) {
                const uint4 kv = k[src_vec0 + t];
                const uint32_t* kw = reinterpret_cast<const uint32_t*>(&kv);
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&kw[p]);
                    const float a = __low2float(x), c = __high2float(x);
                    sk = fmaf(a, a, fmaf(c, c, sk));
                }
                if (q) {
                    const uint4 qv = q[src_vec0 + t];
                    const uint32_t* qw = reinterpret_cast<const uint32_t*>(&qv);
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&qw[p]);
                        const float a = __low2float(x), c = __high2float(x);
                        sq = fmaf(a, a, fmaf(c, c, sq));
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
            }
            __syncthreads();                                    // previous token's factors no longer in use
            if ((threadIdx.x & 31) == 0) { red_s[0][threadIdx.x >> 5] = sq; red_s[1][threadIdx.x >> 5] = sk; }
            __syncthreads();
            if (threadIdx.x < 2) {
                float tot = 0.f;
                for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red_s[threadIdx.x][i];
                rs_s[threadIdx.x] = rsqrtf(tot / (float)(H * kHeadDim) + eps);
            }
            __syncthreads();
        }
        const long long dst_row = (long long)b * cache_batch_stride_vec + (long long)dst_tok * H * kVecPerRow;
        if (roll_shift > 0 && dst_tok - start_idx < roll_shift) {
            // this token's slot ends a chain of the eviction shift: walk it (same thread-to-vector mapping as
            // the write below, so the last source element is read by the thread that then overwrites it)
            const long long tok_vecs = (long long)H * kVecPerRow;
            const long long base = (long long)b * cache_batch_stride_vec;
            const int first = roll_dst + (dst_tok - roll_dst) % roll_shift;
            for (int pos = first; pos < dst_tok; pos += roll_shift) {
                for (int t = threadIdx.x; t < H * kVecPerRow; t += blockDim.x) {
                    const long long d = base + pos * tok_vecs + t, sidx = d + roll_shift * tok_vecs;
                    const uint4 kk = k_cache[sidx];
                    const uint4 vv = v_cache[sidx];
                    k_cache[d] = kk;
                    v_cache[d] = vv;
                }
            }
        }
        for (int t = threadIdx.x; t < H * kVecPerRow; t += blockDim.x) {
            const int vec = t & (kVecPerRow - 1);
            const long long idx = src_vec0 + t;
            uint4 kv = k[idx];
            uint4 vv = v[idx];
            uint4 qv = make_uint4(0, 0, 0, 0);
            if (q) qv = q[idx];
            if (wk) {
                // y = bf16(bf16(x * rsqrt(mean x^2 + eps)) * weight): the two roundings of the reference
                const uint4 wkv = reinterpret_cast<const uint4*>(wk)[t];
                const uint32_t* wkw = reinterpret_cast<const uint32_t*>(&wkv);
                uint32_t* kw = reinterpret_cast<uint32_t*>(&kv);
                const float rk = rs_s[1];
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&kw[p]);
                    const __nv_bfloat162 wv = *reinterpret_cast<const __nv_bfloat162*>(&wkw[p]);
                    const __nv_bfloat162 y = __floats2bfloat162_rn(__low2float(x) * rk, __high2float(x) * rk);
                    kw[p] = pack_bf16(__low2float(y) * __low2float(wv), __high2float(y) * __high2float(wv));
                }
                if (q) {
                    const uint4 wqv = reinterpret_cast<const uint4*>(wq)[t];
                    const uint32_t* wqw = reinterpret_cast<const uint32_t*>(&wqv);
                    uint32_t* qw = reinterpret_cast<uint32_t*>(&qv);
                    const float rq = rs_s[0];
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&qw[p]);
                        const __nv_bfloat162 wv = *reinterpret_cast<const __nv_bfloat162*>(&wqw[p]);
                        const __nv_bfloat162 y = __floats2bfloat162_rn(__low2float(x) * rq, __high2float(x) * rq);
                        qw[p] = pack_bf16(__low2float(y) * __low2float(wv), __high2float(y) * __high2float(wv));
                    }
                }
            }
            if (rope) {
                uint32_t* kw = reinterpret_cast<uint32_t*>(&kv);
                uint32_t* qw = reinterpret_cast<uint32_t*>(&qv);
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const float2 cs = cs_s[vec * 4 + p];
                    {
                        __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&kw[p]);
                        float re = __low2float(x), im = __high2float(x);
                        kw[p] = pack_bf16(re * cs.x - im * cs.y, re * cs.y + im * cs.x);
                    }
                    if (q) {
                        __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&qw[p]);
                        float re = __low2float(x), im = __high2float(x);
                        qw[p] = pack_bf16(re * cs.x - im * cs.y, re * cs.y + im * cs.x);
                    }
                }
            }
            if (q) q_out[out_vec0 + t] = qv;
            k_cache[dst_row + t] = kv;
            v_cache[dst_row + t] = vv;
        }
    }
}

}  // namespace sfm

using namespace sfm;

extern "C" int sfm_build_maps(int32_t* nat2mon, int32_t* mon2nat, int n_tokens, int f_tied, int h_reduce,
                              int w_reduce, int h, int w) {
    Blocking blk;
    int rc = make_blocking(&blk, f_tied, h_reduce, w_reduce, h, w);
    if (rc) return rc;
    if (n_tokens <= 0 || n_tokens % blk.tied_tokens) return SFM_ERR_BAD_SHAPE;
    for (int n = 0; n < n_tokens; ++n) {
        int m = blk.nat2mon(n);
        if (nat2mon) nat2mon[n] = m;
        if (mon2nat) mon2nat[m] = n;
    }
    return SFM_OK;
}

extern "C" int sfm_rope_table(float* out, int head_dim, int max_len, double theta) {
    if (!out) return SFM_ERR_NULL_POINTER;
    if (head_dim <= 0 || head_dim % 2 || max_len <= 0) return SFM_ERR_BAD_SHAPE;
    int c = head_dim / 2;
    int split[3] = {c - 2 * (c / 3), c / 3, c / 3};
    for (int pos = 0; pos < max_len; ++pos) {
        int m = 0;
        for (int ax = 0; ax < 3; ++ax) {
            for (int mm = 0; mm < split[ax]; ++mm, ++m) {
                double inv = 1.0 / pow(theta, (double)(2 * mm) / (double)(2 * split[ax]));
                double ang = (double)pos * inv;
                out[((size_t)pos * c + m) * 2 + 0] = (float)cos(ang);
                out[((size_t)pos * c + m) * 2 + 1] = (float)sin(ang);
            }
        }
    }
    return SFM_OK;
}

namespace {
int rope_cache_write_impl(const PeerSrc& src, bool have_q, int src_tokens, int src_heads, int head0, void* q_out,
                          void* k_cache, void* v_cache, int64_t cache_batch_stride, const float* rope, int B, int n_new,
                          int H, int D, int start_idx, int f_tied, int h_reduce, int w_reduce, int h, int w,
                          int start_frame, int monarch_order, void* stream, const void* wq = nullptr,
                          const void* wk = nullptr, float eps = 0.f, int roll_dst = 0, int roll_shift = 0,
                          int rope_tok0 = -1) {
    if (!k_cache || !v_cache) return SFM_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(wk)) & 15) return SFM_ERR_ALIGNMENT;
    if (have_q && !q_out) return SFM_ERR_NULL_POINTER;
    if (D != kHeadDim) return SFM_ERR_UNSUPPORTED;
    Blocking blk;
    int rc = make_blocking(&blk, f_tied, h_reduce, w_reduce, h, w);
    if (rc) return rc;
    if (B <= 0 || H <= 0 || n_new <= 0 || start_idx < 0) return SFM_ERR_BAD_SHAPE;
    if (monarch_order && n_new % blk.tied_tokens) return SFM_ERR_BAD_SHAPE;
    if (rope) {
        // whole frames, unless the caller rotates a token slice of a chunk (rope_tok0 >= 0: its first token's
        // index in the chunk's grid)
        if (rope_tok0 < 0 && n_new % (h * w)) return SFM_ERR_BAD_SHAPE;
        const int last_frame = start_frame + ((rope_tok0 < 0 ? 0 : rope_tok0) + n_new - 1) / (h * w);
        if (start_frame < 0 || last_frame >= 1024 || h > 1024 || w > 1024) return SFM_ERR_BAD_SHAPE;
    }
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
    if (mis(q_out) || mis(k_cache) || mis(v_cache) || (cache_batch_stride % 8)) return SFM_ERR_ALIGNMENT;
    if (cache_batch_stride < (int64_t)(start_idx + n_new) * H * D && B > 1) return SFM_ERR_BAD_SHAPE;
    // eviction shift: the moved tokens end where the new ones start, and every chain ends in a new token's slot
    if (roll_shift < 0 || (roll_shift > 0 && (roll_dst > start_idx || roll_shift > n_new))) return SFM_ERR_BAD_SHAPE;
    int c = D / 2;
    int p0 = c - 2 * (c / 3), p1 = c / 3;
    int threads = H * (D / 8);
    threads = threads > 256 ? 256 : ((threads + 31) & ~31);
    long long want = (long long)B * n_new;                       // one token per CTA pass
    int blocks = (int)(want < 148LL * 32 ? want : 148LL * 32);  // grid-stride over tokens
    LaunchScope scope(kClsLayout, (cudaStream_t)stream);
    rope_cache_write_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(
        src, src_tokens, src_heads, head0, (uint4*)q_out, (uint4*)k_cache, (uint4*)v_cache, cache_batch_stride / 8,
        (const float2*)rope, B, n_new, H, start_idx, blk, start_frame, monarch_order, p0, p1,
        (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, eps, roll_dst, roll_shift, rope_tok0 < 0 ? 0 : rope_tok0);
    return (int)cudaGetLastError();
}
}  // namespace

extern "C" int sfm_rope_cache_write(const void* q, const void* k, const void* v, void* q_out, void* k_cache,
                                    void* v_cache, int64_t cache_batch_stride, const float* rope, int B,
                                    int n_new, int H, int D, int start_idx, int f_tied, int h_reduce,
                                    int w_reduce, int h, int w, int start_frame, int monarch_order,
                                    void* stream) {
    if (!k || !v) return SFM_ERR_NULL_POINTER;
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
    if (mis(q) || mis(k) || mis(v)) return SFM_ERR_ALIGNMENT;
    PeerSrc src = {};
    src.q[0] = (const uint4*)q; src.k[0] = (const uint4*)k; src.v[0] = (const uint4*)v;
    return rope_cache_write_impl(src, q != nullptr, n_new > 0 ? n_new : 1, H, 0, q_out, k_cache, v_cache,
                                 cache_batch_stride, rope, B, n_new, H, D, start_idx, f_tied, h_reduce, w_reduce, h, w,
                                 start_frame, monarch_order, stream);
}

extern "C" int sfm_norm_rope_cache_write(const void* q, const void* k, const void* v, const void* norm_q_weight,
                                         const void* norm_k_weight, float eps, void* q_out, void* k_cache,
                                         void* v_cache, int64_t cache_batch_stride, const float* rope, int B,
                                         int n_new, int H, int D, int start_idx, int f_tied, int h_reduce,
                                         int w_reduce, int h, int w, int start_frame, int monarch_order,
                                         void* stream) {
    if (!q || !k || !v || !norm_q_weight || !norm_k_weight) return SFM_ERR_NULL_POINTER;
    if (!(eps >= 0.f)) return SFM_ERR_BAD_SHAPE;
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
    if (mis(q) || mis(k) || mis(v)) return SFM_ERR_ALIGNMENT;
    PeerSrc src = {};
    src.q[0] = (const uint4*)q; src.k[0] = (const uint4*)k; src.v[0] = (const uint4*)v;
    return rope_cache_write_impl(src, true, n_new > 0 ? n_new : 1, H, 0, q_out, k_cache, v_cache, cache_batch_stride,
                                 rope, B, n_new, H, D, start_idx, f_tied, h_reduce, w_reduce, h, w, start_frame,
                                 monarch_order, stream, norm_q_weight, norm_k_weight, eps);
}

extern "C" int sfm_rope_cache_write_roll(const void* q, const void* k, const void* v, const void* norm_q_weight,
                                         const void* norm_k_weight, float eps, void* q_out, void* k_cache,
                                         void* v_cache, int64_t cache_batch_stride, const float* rope, int B,
                                         int n_new, int H, int D, int start_idx, int roll_dst, int roll_shift,
                                         int f_tied, int h_reduce, int w_reduce, int h, int w, int start_frame,
                                         int monarch_order, void* stream) {
    if (!q || !k || !v) return SFM_ERR_NULL_POINTER;
    if ((norm_q_weight == nullptr) != (norm_k_weight == nullptr)) return SFM_ERR_NULL_POINTER;
    if (!(eps >= 0.f)) return SFM_ERR_BAD_SHAPE;
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
    if (mis(q) || mis(k) || mis(v)) return SFM_ERR_ALIGNMENT;
    PeerSrc src = {};
    src.q[0] = (const uint4*)q; src.k[0] = (const uint4*)k; src.v[0] = (const uint4*)v;
    return rope_cache_write_impl(src, true, n_new > 0 ? n_new : 1, H, 0, q_out, k_cache, v_cache, cache_batch_stride,
                                 rope, B, n_new, H, D, start_idx, f_tied, h_reduce, w_reduce, h, w, start_frame,
                                 monarch_order, stream, norm_q_weight, norm_k_weight, eps, roll_dst, roll_shift);
}

extern "C" int sfm_norm_rope_token_slice(const void* q, const void* k, const void* v, const void* norm_q_weight,
                                        const void* norm_k_weight, float eps, void* q_out, void* k_out, void* v_out,
                                        const float* rope, int B, int n_tokens, int H, int D, int token0, int h, int w,
                                        int start_frame, void* stream) {
    if (!q || !k || !v || !q_out || !k_out || !v_out || !rope) return SFM_ERR_NULL_POINTER;
    if ((norm_q_weight == nullptr) != (norm_k_weight == nullptr)) return SFM_ERR_NULL_POINTER;
    if (!(eps >= 0.f) || token0 < 0) return SFM_ERR_BAD_SHAPE;
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
    if (mis(q) || mis(k) || mis(v)) return SFM_ERR_ALIGNMENT;
    PeerSrc src = {};
    src.q[0] = (const uint4*)q; src.k[0] = (const uint4*)k; src.v[0] = (const uint4*)v;
    // natural order, slot 0 of a "cache" that is just the output tensors
    return rope_cache_write_impl(src, true, n_tokens > 0 ? n_tokens : 1, H, 0, q_out, k_out, v_out,
                                 (int64_t)n_tokens * H * D, rope, B, n_tokens, H, D, 0, 1, 1, 1, h, w, start_frame, 0,
                                 stream, norm_q_weight, norm_k_weight, eps, 0, 0, token0);
}

extern "C" int sfm_rope_cache_write_gather(const void* const* q_shards, const void* const* k_shards,
                                           const void* const* v_shards, int world, int rank, void* q_out, void* k_cache,
                                           void* v_cache, int64_t cache_batch_stride, const float* rope, int B,
                                           int n_new, int H, int D, int start_idx, int f_tied, int h_reduce,
                                           int w_reduce, int h, int w, int start_frame, int monarch_order,
                                           void* stream) {
    if (!q_shards || !k_shards || !v_shards) return SFM_ERR_NULL_POINTER;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return SFM_ERR_BAD_SHAPE;
    if (n_new <= 0 || n_new % world) return SFM_ERR_BAD_SHAPE;
    PeerSrc src = {};
    for (int p = 0; p < world; ++p) {
        if (!q_shards[p] || !k_shards[p] || !v_shards[p]) return SFM_ERR_NULL_POINTER;
        if ((reinterpret_cast<uintptr_t>(q_shards[p]) | reinterpret_cast<uintptr_t>(k_shards[p]) |
             reinterpret_cast<uintptr_t>(v_shards[p])) & 15)
            return SFM_ERR_ALIGNMENT;
        src.q[p] = (const uint4*)q_shards[p]; src.k[p] = (const uint4*)k_shards[p]; src.v[p] = (const uint4*)v_shards[p];
    }
    return rope_cache_write_impl(src, true, n_new / world, H * world, rank * H, q_out, k_cache, v_cache,
                                 cache_batch_stride, rope, B, n_new, H, D, start_idx, f_tied, h_reduce, w_reduce, h, w,
                                 start_frame, monarch_order, stream);
}

namespace sfm {
// Stand-alone rotation of one tensor (same arithmetic as the fused kernel above).
__global__ void __launch_bounds__(256)
rope_apply_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, const float2* __restrict__ rope, int B,
                  int L, int H, int seq, int hgrid, int wgrid, int start_frame, int p0, int p1) {
    constexpr int kVecPerRow = kHeadDim / 8;
    const long long total = (long long)B * L * H * kVecPerRow;
    const int frame_tokens = hgrid * wgrid;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        int vec = (int)(idx % kVecPerRow);
        long long row = idx / kVecPerRow;
        int n = (int)((row / H) % L);
        uint4 xv = x[idx];
        if (n < seq) {
            int fr = n / frame_tokens, rem = n - fr * frame_tokens;
            int rw = rem / wgrid, cl = rem - rw * wgrid;
            uint32_t* xw = reinterpret_cast<uint32_t*>(&xv);
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                int m = vec * 4 + p;
                int pos = m < p0 ? start_frame + fr : (m < p0 + p1 ? rw : cl);
                float2 cs = rope[pos * (kHeadDim / 2) + m];
                __nv_bfloat162 v2 = *reinterpret_cast<__nv_bfloat162*>(&xw[p]);
                float re = __low2float(v2), im = __high2float(v2);
                xw[p] = pack_bf16(re * cs.x - im * cs.y, re * cs.y + im * cs.x);
            }
        }
        out[idx] = xv;
    }
}
}  // namespace sfm

extern "C" int sfm_rope_apply(const void* x, void* out, const float* rope, int B, int L, int H, int D, int frames,
                              int h, int w, int start_frame, void* stream) {
    if (!x || !out || !rope) return SFM_ERR_NULL_POINTER;
    if (D != kHeadDim) return SFM_ERR_UNSUPPORTED;
    if (B <= 0 || L <= 0 || H <= 0 || frames <= 0 || h <= 0 || w <= 0) return SFM_ERR_BAD_SHAPE;
    if ((long long)frames * h * w > L) return SFM_ERR_BAD_SHAPE;
    if (start_frame < 0 || start_frame + frames > 1024 || h > 1024 || w > 1024) return SFM_ERR_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return SFM_ERR_ALIGNMENT;
    int c = D / 2, p0 = c - 2 * (c / 3), p1 = c / 3;
    long long total = (long long)B * L * H * (D / 8);
    long long want = (total + 255) / 256;
    int blocks = (int)(want < 148LL * 16 ? want : 148LL * 16);
    LaunchScope scope(kClsLayout, (cudaStream_t)stream);
    rope_apply_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)x, (uint4*)out, (const float2*)rope, B,
                                                                 L, H, frames * h * w, h, w, start_frame, p0, p1);
    return (int)cudaGetLastError();
}
