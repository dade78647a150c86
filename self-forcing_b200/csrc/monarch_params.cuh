// Launch parameters shared by the Monarch row-step / column-step kernels and their host driver.
#pragma once
#include "common.cuh"

namespace sfm {

// One "chunk" = nbh consecutive flattened (batch, head) indices x na consecutive query groups.
// The row step writes its results for the chunk into the bridge; the column step consumes them.
//
// Bridge layout (chunk-local), with aj = (bh_local*na + a_local)*b2 + j and key = f*b1 + k:
//   aL, Y : bf16 [aj][n_keys][128]      cL : fp32 [aj][n_keys_c] (pitch rounded up to 16 bytes)
// Iteration state (chunk-local too, only when num_iters > 1):
//   aR : bf16 [bh_local][F][b1][na][b2][128]   cR : fp32 [bh_local][F][b1][na][b2]
struct MonarchParams {
    const __nv_bfloat16* q;        // natural order [B, n_q, H, 128]
    long long q_bs;                // batch stride of q (elements)
    const __nv_bfloat16* kc;       // caches, Monarch order [B, n_kv, H, 128]
    const __nv_bfloat16* vc;
    long long c_bs;                // batch stride of the caches (elements)
    __nv_bfloat16* out;            // natural order [B, n_q, H, 128], contiguous
    __nv_bfloat16* aL;
    __nv_bfloat16* Y;
    float* cL;
    __nv_bfloat16* aR;             // iteration state (may be null)
    float* cR;
    float* lse;                    // fp32 [aj][b1] (chunk-local), iteration path only
    int use_aR;                    // row step: take the query operand from aR/cR instead of q
    int write_Y;                   // row step: also produce Y
    int H, n_q, A, F, n_keys;      // A query groups, F cached groups, n_keys = F*b1
    int n_keys_c;                  // row pitch of cL in floats: n_keys rounded up to a multiple of 4
    int bh0, nbh, a0, na, na_cta;  // chunk and per-CTA stacking of query groups
    int fsplit, f_per;             // row step: split of the F loop over CTAs
    int causal_groups;             // 0: none; else groups per causal block (no-cache path)
    float scale;                   // softmax scale (applied once, to the dot products)
    float mult0;                   // row-step multiplier when the operand is q itself (scale, or
                                   // scale/(1+1e-6) on the first pass of the iterative path)
    Blocking blk;
    // Where the column step puts its result.  Unsharded: one [B, n_q, H, 128] tensor (out_peers[0] = out,
    // out_tokens = n_q, out_heads = H, out_head0 = 0).  Head-sharded call: the output is sharded by token
    // over the GPUs of the box, shard t / out_tokens being a [B, out_tokens, out_heads, 128] tensor on that
    // GPU, of which this GPU writes heads [out_head0, out_head0 + H) with plain stores over NVLink.
    __nv_bfloat16* out_peers[kMaxPeers];
    int out_tokens, out_heads, out_head0;

    __device__ __forceinline__ __nv_bfloat16* out_row(int b, long long tok, int hd) const {
        const int peer = (int)(tok / out_tokens);
        const long long t = tok - (long long)peer * out_tokens;
        return out_peers[peer] + (((long long)b * out_tokens + t) * out_heads + out_head0 + hd) * kHeadDim;
    }
};

constexpr int kRWarps = 8;         // row-step CTA: 8 warps, one 16-row m-tile at a time each
constexpr int kRMaxRows = 160;     // stacked (query group, column) rows per row-step CTA
constexpr int kB2Max = 64;         // block columns the mma.sync kernels support (padded to a multiple of 16)
constexpr int kB2MaxTc = 128;      // block columns the tensor-core kernels support
constexpr int kLWarps = 4;         // column-step CTA: 4 warps splitting each 128-key tile
constexpr int kLTileKeys = 128;
constexpr int kLQRows = 32;        // query rows (i) per column-step CTA
constexpr int kIterMaxB1 = 160;    // block rows supported by the iteration kernel

size_t r_smem_bytes(bool per_f_query);
size_t l_smem_bytes();
size_t iter_smem_bytes();
int launch_r_step(const MonarchParams& p, cudaStream_t s);
int launch_l_step(const MonarchParams& p, int lse_only, cudaStream_t s);
int launch_l_iter(const MonarchParams& p, cudaStream_t s);

}  // namespace sfm
