// Attention over a latent cache on the tensor cores (bfloat16 cache rows; see latent_attn.cu for the operation).
//
// All H heads of a token read the same cached rows, and neighbouring tokens of a prompt nearly the same, so a
// block's 64 rows of the score matrix are (token, head) pairs: 64 / H consecutive tokens of one sequence with all
// their heads (or 64 heads of one token).  The wide queries [Dk = R + dr] sit in shared memory as bfloat16; keys
// come in tiles of 32 cached rows (cp.async, padded rows); S = Q K^T and O += P V run on mma.sync m16n8k16 with
// float32 accumulation, the softmax online in float32 as in attn_prefill.cu.  The values are the first R columns of
// the very tile that served as keys, read transposed.  A warp cannot hold 16 x R accumulators for a latent of
// several hundred numbers, so the R columns are cut into chunks of CW (64, 128 or 256), each accumulated by its own
// group of four warps that makes the scores again: for R = 512, Dk = 576 that is 1.5 times the products of one
// pass.  Two such groups share a block, and with it the queries and the key tiles in shared memory (two tiles, the
// next one on its way while the current one is multiplied).
//
// Prompts and portions: a work list made on the host (sequence, first packed row, tokens, first position), the
// blocks with the most keys first.  Steps of one token per sequence: a block per token, the token's keys cut into
// `splits` slices (blockIdx.z) whose partial results lq_latent_merge of this file combines.
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr int BM = 64;          // rows of a block: (token, head) pairs
constexpr int BN = 32;          // keys of a tile
constexpr int PAD = 8;
constexpr int NT = 128;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    int bytes = valid ? 16 : 0;     // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct LatentArgs {
    const float* q;                  // [T, H, Dk]
    const __nv_bfloat16* pages;      // [pages, page_size, Dk]
    const int* page_table;
    int pt_stride;
    const int* slots;
    const int* qb_seq;               // work list of a step with prompts (null: a block per token)
    const int* qb_row;
    const int* qb_rows;
    const int* qb_pos;
    const int* tok_pos;              // steps of single tokens
    const int* tok_seq;
    float* out;                      // [T, H, R] (bfloat16 with out_bf16)
    float* part_o;                   // [T, H, splits, R]
    float* part_ml;                  // [T, H, splits, 2]: maximum (natural logarithm units) and sum
    int H, R, Dk, page_size, window, splits, head_blocks, chunks;
    int out_bf16;                    // the final rows go out as bfloat16 (the partial results of slices stay float32)
    float scale_log2;
};

// CW: value columns that a group of four warps accumulates; NCH: groups (chunks of columns) of a block.
template <int CW, int NCH>
__global__ void __launch_bounds__(NT * NCH, 1) latent_attention_tc_kernel(LatentArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int H = a.H, R = a.R, Dk = a.Dk;
    const int DKP = (Dk + 15) & ~15;                                  // k16 steps cover the padded width (zeros beyond Dk)
    const int LD = max(DKP, a.chunks * CW) + PAD;                     // the value columns of the last chunk stay inside a row
    __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [BM][DKP + PAD]
    const int LQ = DKP + PAD;                                         // the key tiles follow the queries: [2][BN][LD]
    constexpr int THREADS = NT * NCH;
    const int tid = threadIdx.x, warp = (tid >> 5) & 3, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int blk = blockIdx.x, hb = blockIdx.y % a.head_blocks, split = blockIdx.z;
    const int chunk = (blockIdx.y / a.head_blocks) * NCH + (tid >> 7);
    const bool chunk_live = chunk < a.chunks;
    const int Hb = min(H - hb * BM, BM), h0 = hb * BM;                // heads of this block
    const int TB = BM / Hb;                                           // tokens whose heads fit into the block's rows
    const int c0 = chunk * CW;
    pdl_launch_dependents();
    pdl_wait();
    int seq, row0, n_tok, pos0;
    if (a.qb_seq) { seq = a.qb_seq[blk]; row0 = a.qb_row[blk]; n_tok = min(a.qb_rows[blk], TB); pos0 = a.qb_pos[blk]; }
    else { seq = a.tok_seq[blk]; row0 = blk; n_tok = 1; pos0 = a.tok_pos[blk]; }
    const int* pt = a.page_table + (size_t)a.slots[seq] * a.pt_stride;
    const int window = a.window;
    const int key_last = pos0 + n_tok - 1;
    const int key_first = (window > 0 && pos0 >= window) ? pos0 - window + 1 : 0;
    const int t_lo = key_first / BN, t_n = key_last / BN + 1 - t_lo;
    const int tile_lo = t_lo + (int)((long long)split * t_n / a.splits), tile_hi = t_lo + (int)((long long)(split + 1) * t_n / a.splits);

    // ---- the block's queries: row r is head h0 + r % Hb of token r / Hb
    for (int i = tid; i < BM * (DKP / 2); i += THREADS) {
        const int r = i / (DKP / 2), c = (i % (DKP / 2)) * 2;
        const int tl = r / Hb, hl = r % Hb;
        float v0 = 0.f, v1 = 0.f;
        if (tl < n_tok) {
            const float* src = a.q + ((size_t)(row0 + tl) * H + h0 + hl) * Dk;
            if (c < Dk) v0 = src[c];
            if (c + 1 < Dk) v1 = src[c + 1];
        }
        *reinterpret_cast<uint32_t*>(sq + r * LQ + c) = pack_bf16(v0, v1);
    }
    auto load_keys = [&](int tile, int stage) {
        const int kb = tile * BN;
        __nv_bfloat16* sk = sq + BM * LQ + stage * BN * LD;
        // A tile of 32 keys lies inside one page (pages are multiples of 32 keys long): one look at the page table.
        const __nv_bfloat16* rows = a.pages + ((size_t)pt[kb / a.page_size] * a.page_size + kb % a.page_size) * Dk;
        for (int i = tid; i < BN * (DKP / 8); i += THREADS) {
            const int r = i / (DKP / 8), c = (i % (DKP / 8)) * 8;
            const bool ok = kb + r <= key_last && c < Dk;
            cp_async16((uint32_t)__cvta_generic_to_shared(sk + r * LD + c), ok ? rows + (size_t)r * Dk + c : a.pages, ok);
        }
    };

    float o[CW / 8][4];
#pragma unroll
    for (int j = 0; j < CW / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
    // This thread's two rows, and what the warp's 16 rows span.
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const bool row0ok = r0 / Hb < n_tok, row1ok = r1 / Hb < n_tok;
    const int prow0 = pos0 + r0 / Hb, prow1 = pos0 + r1 / Hb;
    const int w_tl_lo = (warp * 16) / Hb, w_tl_hi = min((warp * 16 + 15) / Hb, n_tok - 1);
    const bool warp_live = w_tl_lo < n_tok && chunk_live;
    const int warp_pos_hi = pos0 + w_tl_hi;
    const int warp_key_lo = window > 0 ? max(0, pos0 + w_tl_lo - window + 1) : 0;
    const int kd = DKP / 16;

    if (tile_lo < tile_hi) load_keys(tile_lo, 0);
    cp_async_commit();
    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int stage = (tile - tile_lo) & 1;
        __syncthreads();                                  // the other stage has been read (and the queries are written)
        if (tile + 1 < tile_hi) load_keys(tile + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* sk = sq + BM * LQ + stage * BN * LD;
        const int kb = tile * BN;
        if (!warp_live || kb > warp_pos_hi || kb + BN <= warp_key_lo) continue;
        float s[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll 4
        for (int kk = 0; kk < kd; ++kk) {
            uint32_t a0, a1, a2, a3;
            {
                const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = kk * 16 + (lane >> 4) * 8;
                ldsm_x4((uint32_t)__cvta_generic_to_shared(sq + r * LQ + c), a0, a1, a2, a3);
            }
#pragma unroll
            for (int jp = 0; jp < 2; ++jp) {
                const int r = jp * 16 + (lane & 7) + (lane >> 4) * 8, c = kk * 16 + ((lane >> 3) & 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4((uint32_t)__cvta_generic_to_shared(sk + r * LD + c), b0, b1, b2, b3);
                mma_bf16(s[2 * jp], a0, a1, a2, a3, b0, b1);
                mma_bf16(s[2 * jp + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        float tm0 = -CUDART_INF_F, tm1 = -CUDART_INF_F;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int key = kb + j * 8 + 2 * t + i;
                const bool ok0 = row0ok && key <= prow0 && (window <= 0 || key > prow0 - window);
                const bool ok1 = row1ok && key <= prow1 && (window <= 0 || key > prow1 - window);
                s[j][i] = ok0 ? s[j][i] * a.scale_log2 : -CUDART_INF_F;
                s[j][2 + i] = ok1 ? s[j][2 + i] * a.scale_log2 : -CUDART_INF_F;
                tm0 = fmaxf(tm0, s[j][i]);
                tm1 = fmaxf(tm1, s[j][2 + i]);
            }
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1));
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
        const float nm0 = fmaxf(m0, tm0), nm1 = fmaxf(m1, tm1);
        const float u0 = nm0 == -CUDART_INF_F ? 0.f : nm0, u1 = nm1 == -CUDART_INF_F ? 0.f : nm1;
        const float f0 = exp2f(m0 - u0), f1 = exp2f(m1 - u1);     // m = -inf gives 0
        m0 = nm0;
        m1 = nm1;
        float ps0 = 0.f, ps1 = 0.f;
        uint32_t pa[2][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // The sums run over the probabilities as the product sees them (rounded to bfloat16).
            const float p00 = round_bf16(exp2f(s[j][0] - u0)), p01 = round_bf16(exp2f(s[j][1] - u0));
            const float p10 = round_bf16(exp2f(s[j][2] - u1)), p11 = round_bf16(exp2f(s[j][3] - u1));
            ps0 += p00 + p01;
            ps1 += p10 + p11;
            pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p00, p01);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p10, p11);
        }
        l0 = l0 * f0 + ps0;
        l1 = l1 * f1 + ps1;
#pragma unroll
        for (int j = 0; j < CW / 8; ++j) { o[j][0] *= f0; o[j][1] *= f0; o[j][2] *= f1; o[j][3] *= f1; }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {                  // 16 keys per step
#pragma unroll
            for (int dp = 0; dp < CW / 16; ++dp) {
                const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = c0 + dp * 16 + (lane >> 4) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t((uint32_t)__cvta_generic_to_shared(sk + r * LD + c), b0, b1, b2, b3);
                mma_bf16(o[2 * dp], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                mma_bf16(o[2 * dp + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
            }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const bool whole = a.splits == 1;
    const float i0 = whole ? 1.0f / l0 : 1.f, i1 = whole ? 1.0f / l1 : 1.f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = half ? r1 : r0;
        if (!(half ? row1ok : row0ok) || !chunk_live) continue;
        const size_t pair = (size_t)(row0 + r / Hb) * H + h0 + r % Hb;
        const float inv = half ? i1 : i0;
        if (whole && a.out_bf16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.out) + pair * R;
#pragma unroll
            for (int j = 0; j < CW / 8; ++j) {
                const int d = c0 + j * 8 + 2 * t;
                if (d < R) dst[d] = __float2bfloat16_rn(o[j][2 * half] * inv);
                if (d + 1 < R) dst[d + 1] = __float2bfloat16_rn(o[j][2 * half + 1] * inv);
            }
        } else {
            float* dst = whole ? a.out + pair * R : a.part_o + (pair * a.splits + split) * R;
#pragma unroll
            for (int j = 0; j < CW / 8; ++j) {
                const int d = c0 + j * 8 + 2 * t;
                if (d < R) dst[d] = o[j][2 * half] * inv;
                if (d + 1 < R) dst[d + 1] = o[j][2 * half + 1] * inv;
            }
        }
        if (!whole && chunk == 0 && t == 0) {
            float* ml = a.part_ml + (pair * a.splits + split) * 2;
            ml[0] = (half ? m1 : m0) * 0.6931471805599453f;      // -inf for a slice without keys
            ml[1] = half ? l1 : l0;
        }
    }
}

// One block per (row, head): the slices' weights once, then a thread per value column, the slices added in their order.
template <typename TO>
__global__ void __launch_bounds__(128) latent_merge_tc_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                              TO* __restrict__ out, int n_pairs, int R, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float wgt[64];
    __shared__ float inv_s;
    const int pair = blockIdx.x, tid = threadIdx.x;
    const float* ml = part_ml + (size_t)pair * splits * 2;
    if (tid < 32) {
        float m = -CUDART_INF_F;
        for (int s = tid; s < splits; s += 32) m = fmaxf(m, ml[2 * s]);
        m = warp_max(m);
        float l = 0.f;
        for (int s = tid; s < splits; s += 32) {
            const float w = ml[2 * s] == -CUDART_INF_F ? 0.f : expf(ml[2 * s] - m);
            wgt[s] = w;
            l += w * ml[2 * s + 1];
        }
        l = warp_sum(l);
        if (tid == 0) inv_s = 1.f / l;
    }
    __syncthreads();
    const float inv = inv_s;
    for (int d = tid; d < R; d += 128) {
        float o = 0.f;
        for (int s = 0; s < splits; ++s)
            if (wgt[s] != 0.f) o = fmaf(part_o[((size_t)pair * splits + s) * R + d], wgt[s], o);
        out[(size_t)pair * R + d] = from_f32<TO>(o * inv);
    }
}

template <int CW, int NCH>
int launch(LatentArgs a, int n_blocks, int T, cudaStream_t stream) {
    a.chunks = (a.R + CW - 1) / CW;
    const int DKP = (a.Dk + 15) & ~15;
    const int LD = (DKP > a.chunks * CW ? DKP : a.chunks * CW) + PAD;
    const size_t smem = ((size_t)BM * (DKP + PAD) + (size_t)2 * BN * LD) * 2;
    if (smem > 220 * 1024) return LQ_BAD_SIZE;
    if (cudaFuncSetAttribute(latent_attention_tc_kernel<CW, NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return lq_launch_status();
    dim3 grid(n_blocks, a.head_blocks * ((a.chunks + NCH - 1) / NCH), a.splits);
    int rc = launch_pdl(latent_attention_tc_kernel<CW, NCH>, grid, dim3(NT * NCH), smem, stream, a);
    if (rc != LQ_OK || a.splits == 1) return rc;
    const int n = T * a.H;
    if (a.out_bf16)
        return launch_pdl(latent_merge_tc_kernel<__nv_bfloat16>, dim3(n), dim3(128), 0, stream, (const float*)a.part_o,
                          (const float*)a.part_ml, reinterpret_cast<__nv_bfloat16*>(a.out), n, a.R, a.splits);
    return launch_pdl(latent_merge_tc_kernel<float>, dim3(n), dim3(128), 0, stream, (const float*)a.part_o,
                      (const float*)a.part_ml, a.out, n, a.R, a.splits);
}

}  // namespace

// Tokens of a block's work-list entry for H heads: as many as fit into the block's 64 rows.
LQ_EXPORT int lq_latent_attention_tc_tokens(int H) { return H >= BM ? 1 : BM / H; }

// qb_* (n_blocks entries: sequence, first packed row, tokens <= lq_latent_attention_tc_tokens(H), first position) for a
// step with prompts; null with n_blocks = T for a step of one token per sequence (tok_pos, tok_seq give each token's
// place).  Dk a multiple of 8, page_size a multiple of 32, bfloat16 cache rows.
LQ_EXPORT int lq_latent_attention_tc(const float* q, const void* pages, const int* page_table, int pt_stride, const int* slots,
                                     const int* qb_seq, const int* qb_row, const int* qb_rows, const int* qb_pos,
                                     const int* tok_pos, const int* tok_seq, void* out, int out_dtype, float* part_o, float* part_ml,
                                     int n_blocks, int T, int H, int R, int Dk, int page_size, float scale, int window,
                                     int splits, cudaStream_t stream) {
    if (n_blocks <= 0) return LQ_OK;
    if (Dk % 8 || R < 1 || R > Dk || page_size % BN || splits < 1 || (splits > 1 && (!part_o || !part_ml)) || splits > 64) return LQ_BAD_SIZE;
    if (!qb_seq && (!tok_pos || !tok_seq)) return LQ_BAD_SIZE;
    if (out_dtype != LQ_F32 && out_dtype != LQ_BF16) return LQ_BAD_DTYPE;
    LatentArgs a{q, (const __nv_bfloat16*)pages, page_table, pt_stride, slots, qb_seq, qb_row, qb_rows, qb_pos, tok_pos, tok_seq,
                 (float*)out, part_o, part_ml, H, R, Dk, page_size, window, splits, (H + BM - 1) / BM, 1, out_dtype == LQ_BF16,
                 scale * 1.4426950408889634f};
    if (R <= 64) return launch<64, 1>(a, n_blocks, T, stream);
    if (R <= 128) return launch<128, 1>(a, n_blocks, T, stream);
    if (R <= 256) return launch<256, 1>(a, n_blocks, T, stream);
    return launch<256, 2>(a, n_blocks, T, stream);
}
