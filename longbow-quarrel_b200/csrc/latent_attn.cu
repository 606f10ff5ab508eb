// Attention over a latent cache: every token keeps ONE row [R + dr] for all heads -- a normed latent c (R) from
// which each head's keys and values are linear maps, and one rotated key part (dr) that all heads share.
//
// The per-head maps are moved to the query's side, so nothing is expanded per key:
//     score_h(t, j) = (W_uk,h^T q_h) . c_j + q_rot,h . k_rot,j         (a query of R + dr numbers per head)
//     o_h(t)        = W_uv,h (sum_j p_j c_j)                           (a weighted mean of latents per head)
// which makes the attention itself multi-query attention with one "kv head" whose values are the first R
// numbers of its keys.  Kernels here:
//   lq_latent_kv_store   RMS norm of the latent, rotation of the shared key part, the row's cache write
//   lq_rope_tail         rotation of the rotated part of every query head into the wide query
//   lq_head_matmul       out[t, h, :] = in[t, h, :] . W[h] for per-head matrices W [H, K, N] (queries onto the
//                        latent; latent means onto values)
//   lq_latent_attention  the attention (prompts, portions and single tokens; the keys of a row may be cut into
//                        slices whose partial results a second kernel merges)
// Scores, softmax, norms and angles are float32; intermediates (wide queries, latent means) are float32 rows.
#include "common.cuh"
#include <math_constants.h>

// ------------------------------------------------------------------ cache write
// rows [T, stride] (TI): the latent at column c_off (R wide), the shared key part at r_off (dr wide).
// page row = [ c / rms(c) * gain | rotate(k_rot) ]; the first `rot` dimensions of the key part are rotated
// (pairs i, i + rot/2), the rest pass.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) latent_kv_store_kernel(const TI* __restrict__ rows, int stride, int c_off, int r_off,
                                                              const float* __restrict__ gain, float eps,
                                                              const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                              int rot, const int* __restrict__ tok_pos,
                                                              const int* __restrict__ tok_seq, const int* __restrict__ slots,
                                                              const int* __restrict__ page_table, int pt_stride,
                                                              TO* __restrict__ pages, int R, int dr, int page_size) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[8];
    const int t = blockIdx.x, tid = threadIdx.x;
    const TI* x = rows + (size_t)t * stride;
    const int pos = tok_pos[t], slot = slots[tok_seq[t]];
    const int page = page_table[(size_t)slot * pt_stride + pos / page_size];
    TO* out = pages + ((size_t)page * page_size + pos % page_size) * (R + dr);
    float s = 0.f;
    for (int i = tid; i < R; i += 256) {
        const float v = to_f32(x[c_off + i]);
        s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    if ((tid & 31) == 0) red[tid >> 5] = s;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += red[w];
    const float inv = 1.f / sqrtf(total / (float)R + eps);
    for (int i = tid; i < R; i += 256) out[i] = from_f32<TO>(to_f32(x[c_off + i]) * inv * gain[i]);
    const int half = rot >> 1;
    for (int i = tid; i < dr; i += 256) {
        float v = to_f32(x[r_off + i]);
        if (i < rot) {
            const int f = i < half ? i : i - half, ip = i < half ? i + half : i - half;
            const float cs = cos_t[(size_t)pos * half + f], sn = sin_t[(size_t)pos * half + f];
            const float other = to_f32(x[r_off + ip]);
            v = i < half ? v * cs - other * sn : v * cs + other * sn;
        }
        out[R + i] = from_f32<TO>(v);
    }
}

LQ_EXPORT int lq_latent_kv_store(const void* rows, int in_dtype, int stride, int c_off, int r_off, const float* gain, float eps,
                                 const float* cos_t, const float* sin_t, int rot, const int* tok_pos, const int* tok_seq,
                                 const int* slots, const int* page_table, int pt_stride, void* pages, int out_dtype, int T,
                                 int R, int dr, int page_size, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (rot % 2 || rot > dr || (rot && (!cos_t || !sin_t)) || R < 1) return LQ_BAD_SIZE;
    typedef __nv_bfloat16 bf;
#define LQ_GO(TI, TO) return launch_pdl(latent_kv_store_kernel<TI, TO>, dim3(T), dim3(256), 0, stream, (const TI*)rows, stride, \
        c_off, r_off, gain, eps, cos_t, sin_t, rot, tok_pos, tok_seq, slots, page_table, pt_stride, (TO*)pages, R, dr, page_size)
    if (in_dtype == LQ_F32 && out_dtype == LQ_F32) LQ_GO(float, float);
    if (in_dtype == LQ_F32 && out_dtype == LQ_BF16) LQ_GO(float, bf);
    if (in_dtype == LQ_BF16 && out_dtype == LQ_BF16) LQ_GO(bf, bf);
#undef LQ_GO
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ rotation of a part of every head
// in [T, in_stride]: head h's part starts at column h * in_head + in_off and is n wide; its first `rot` dimensions
// are rotated by the row's position, the rest pass; it goes to out [T, out_stride] at h * out_head + out_off.
template <typename TI>
__global__ void rope_tail_kernel(const TI* __restrict__ in, int in_stride, int in_head, int in_off, float* __restrict__ out,
                                 int out_stride, int out_head, int out_off, const float* __restrict__ cos_t,
                                 const float* __restrict__ sin_t, int rot, const int* __restrict__ tok_pos, int T, int H, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (size_t)T * H * n) return;
    const int i = e % n, h = (e / n) % H, t = e / ((size_t)n * H);
    const TI* x = in + (size_t)t * in_stride + h * in_head + in_off;
    float v = to_f32(x[i]);
    if (i < rot) {
        const int half = rot >> 1, f = i < half ? i : i - half, ip = i < half ? i + half : i - half;
        const size_t at = (size_t)tok_pos[t] * half + f;
        const float cs = cos_t[at], sn = sin_t[at], other = to_f32(x[ip]);
        v = i < half ? v * cs - other * sn : v * cs + other * sn;
    }
    out[(size_t)t * out_stride + h * out_head + out_off + i] = v;
}

LQ_EXPORT int lq_rope_tail(const void* in, int in_dtype, int in_stride, int in_head, int in_off, float* out, int out_stride,
                           int out_head, int out_off, const float* cos_t, const float* sin_t, int rot, const int* tok_pos, int T,
                           int H, int n, cudaStream_t stream) {
    const size_t total = (size_t)T * H * n;
    if (total == 0) return LQ_OK;
    if (rot % 2 || rot > n || (rot && (!cos_t || !sin_t))) return LQ_BAD_SIZE;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (in_dtype == LQ_F32)
        return launch_pdl(rope_tail_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)in, in_stride, in_head, in_off,
                          out, out_stride, out_head, out_off, cos_t, sin_t, rot, tok_pos, T, H, n);
    if (in_dtype == LQ_BF16)
        return launch_pdl(rope_tail_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)in, in_stride,
                          in_head, in_off, out, out_stride, out_head, out_off, cos_t, sin_t, rot, tok_pos, T, H, n);
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ one small matrix per head
// out[t, h * out_head + out_off + n] = sum_k in[t, h * in_head + in_off + k] * W[h, k, n]   (W [H, K, N], float32 sums
// over k in rising order).  A block takes one head and HM_ROWS rows: W[h] is read once for all of them; a thread
// owns output columns n = tid, tid + 256, ...
constexpr int HM_ROWS = 8;
template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(256) head_matmul_kernel(const TI* __restrict__ in, int in_stride, int in_head, int in_off,
                                                          const TW* __restrict__ w, TO* __restrict__ out, int out_stride,
                                                          int out_head, int out_off, int T, int K, int N) {
    pdl_launch_dependents();
    extern __shared__ float xs[];                 // [HM_ROWS][K]
    const int h = blockIdx.y, t0 = blockIdx.x * HM_ROWS, tid = threadIdx.x;
    const int rows = min(HM_ROWS, T - t0);
    pdl_wait();
    for (int e = tid; e < HM_ROWS * K; e += 256) {
        const int r = e / K, k = e % K;
        xs[e] = r < rows ? to_f32(in[(size_t)(t0 + r) * in_stride + h * in_head + in_off + k]) : 0.f;
    }
    __syncthreads();
    const TW* wh = w + (size_t)h * K * N;
    for (int n = tid; n < N; n += 256) {
        float acc[HM_ROWS] = {};
        for (int k = 0; k < K; ++k) {
            const float wv = to_f32(wh[(size_t)k * N + n]);
#pragma unroll
            for (int r = 0; r < HM_ROWS; ++r) acc[r] = fmaf(xs[r * K + k], wv, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < HM_ROWS; ++r)
            if (r < rows) out[(size_t)(t0 + r) * out_stride + h * out_head + out_off + n] = from_f32<TO>(acc[r]);
    }
}

LQ_EXPORT int lq_head_matmul(const void* in, int in_dtype, int in_stride, int in_head, int in_off, const void* w, int w_dtype,
                             void* out, int out_dtype, int out_stride, int out_head, int out_off, int T, int H, int K, int N,
                             cudaStream_t stream) {
    if (T <= 0 || H <= 0) return LQ_OK;
    const size_t smem = (size_t)HM_ROWS * K * sizeof(float);
    if (smem > 200 * 1024) return LQ_BAD_SIZE;
    dim3 grid((T + HM_ROWS - 1) / HM_ROWS, H);
    typedef __nv_bfloat16 bf;
#define LQ_GO(TI, TW, TO) do { \
        if (smem > 48 * 1024) cudaFuncSetAttribute(head_matmul_kernel<TI, TW, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return launch_pdl(head_matmul_kernel<TI, TW, TO>, grid, dim3(256), smem, stream, (const TI*)in, in_stride, in_head, in_off, \
                          (const TW*)w, (TO*)out, out_stride, out_head, out_off, T, K, N); } while (0)
    if (in_dtype == LQ_F32 && w_dtype == LQ_F32 && out_dtype == LQ_F32) LQ_GO(float, float, float);
    if (in_dtype == LQ_F32 && w_dtype == LQ_BF16 && out_dtype == LQ_F32) LQ_GO(float, bf, float);
    if (in_dtype == LQ_F32 && w_dtype == LQ_BF16 && out_dtype == LQ_BF16) LQ_GO(float, bf, bf);
    if (in_dtype == LQ_BF16 && w_dtype == LQ_BF16 && out_dtype == LQ_F32) LQ_GO(bf, bf, float);
    if (in_dtype == LQ_BF16 && w_dtype == LQ_BF16 && out_dtype == LQ_BF16) LQ_GO(bf, bf, bf);
#undef LQ_GO
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ the attention
// q [T, H, Dk] float32 (Dk = R + dr); pages [page][page_size][Dk] (TC); out [T, H, R] float32.
// Row t (position p of the sequence in slot s) sees the keys at positions first..p, first = max(0, p - window + 1)
// (window 0: all).  grid = (T, ceil(H / LA_WARPS), splits): a block takes one row, up to LA_WARPS heads (a warp
// each) and one slice of the row's keys; tiles of 32 keys are staged in shared memory as float32 once for all
// the block's heads; lane j takes key j's score, then the lanes share out the R value columns.
// With splits > 1 a block leaves (max, sum, unnormalised mean) in scratch and lq_latent_merge finishes the row.
constexpr int LA_WARPS = 8;
constexpr int LA_KEYS = 32;

template <typename TC, int NACC>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attention_kernel(
        const float* __restrict__ q, const TC* __restrict__ pages, const int* __restrict__ page_table, int pt_stride,
        const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ slots,
        float* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
        int H, int R, int Dk, int page_size, float scale, int window, int splits) {
    pdl_launch_dependents();
    extern __shared__ float sm[];
    const int ld = Dk | 1;                                  // odd: lane j's row starts in its own bank
    float* qs = sm;                                         // [LA_WARPS][Dk]
    float* tile = sm + LA_WARPS * Dk;                       // [LA_KEYS][ld]
    const int t = blockIdx.x, h0 = blockIdx.y * LA_WARPS, split = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = h0 + warp;
    const bool live = h < H;
    pdl_wait();
    const int pos = tok_pos[t], slot = slots[tok_seq[t]];
    const int first = (window > 0 && pos >= window) ? pos - window + 1 : 0;
    // The slice of this block: whole tiles, counted from `first`.
    const int n_keys = pos + 1 - first, n_tiles = (n_keys + LA_KEYS - 1) / LA_KEYS;
    const int tile_lo = (int)((long long)split * n_tiles / splits), tile_hi = (int)((long long)(split + 1) * n_tiles / splits);
    for (int e = tid; e < LA_WARPS * Dk; e += LA_WARPS * 32) {
        const int w = e / Dk, d = e % Dk;
        qs[e] = (h0 + w < H) ? q[((size_t)t * H + h0 + w) * Dk + d] : 0.f;
    }
    float m = -CUDART_INF_F, l = 0.f, acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    const int* pt = page_table + (size_t)slot * pt_stride;
    for (int tl = tile_lo; tl < tile_hi; ++tl) {
        const int k0 = first + tl * LA_KEYS;
        __syncthreads();                                    // the tile of the last pass has been read
        for (int e = tid; e < LA_KEYS * Dk; e += LA_WARPS * 32) {
            const int j = e / Dk, d = e % Dk, kp = k0 + j;
            float v = 0.f;
            if (kp <= pos) v = to_f32(pages[((size_t)pt[kp / page_size] * page_size + kp % page_size) * Dk + d]);
            tile[j * ld + d] = v;
        }
        __syncthreads();
        if (!live) continue;
        const float* qh = qs + warp * Dk;
        const float* kr = tile + lane * ld;
        float s0 = 0.f, s1 = 0.f;
        int d = 0;
        for (; d + 1 < Dk; d += 2) {
            s0 = fmaf(qh[d], kr[d], s0);
            s1 = fmaf(qh[d + 1], kr[d + 1], s1);
        }
        if (d < Dk) s0 = fmaf(qh[d], kr[d], s0);
        const bool seen = k0 + lane <= pos;
        const float s = seen ? (s0 + s1) * scale : -CUDART_INF_F;
        const float m_new = fmaxf(m, warp_max(s));          // key k0 is always seen: finite
        const float alpha = expf(m - m_new), p = seen ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
        const int n_j = min(LA_KEYS, pos + 1 - k0);
        for (int j = 0; j < n_j; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const float* vr = tile + j * ld + lane;
#pragma unroll
            for (int i = 0; i < NACC; ++i)
                if (lane + 32 * i < R) acc[i] = fmaf(pj, vr[32 * i], acc[i]);
        }
    }
    if (!live) return;
    if (splits == 1) {
        const float inv = 1.f / l;
        float* o = out + ((size_t)t * H + h) * R;
#pragma unroll
        for (int i = 0; i < NACC; ++i)
            if (lane + 32 * i < R) o[lane + 32 * i] = acc[i] * inv;
        return;
    }
    const size_t at = ((size_t)t * H + h) * splits + split;
    float* o = part_o + at * R;
#pragma unroll
    for (int i = 0; i < NACC; ++i)
        if (lane + 32 * i < R) o[lane + 32 * i] = acc[i];
    if (lane == 0) {
        part_ml[2 * at] = m;                               // -inf for an empty slice
        part_ml[2 * at + 1] = l;
    }
}

// One warp per (row, head): the slices' results combined in the order of the slices.
__global__ void __launch_bounds__(128) latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                           float* __restrict__ out, int n_pairs, int R, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_pairs) return;
    const float* ml = part_ml + (size_t)pair * splits * 2;
    float m = -CUDART_INF_F;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, ml[2 * s]);
    float l = 0.f;
    for (int s = 0; s < splits; ++s) l += ml[2 * s] == -CUDART_INF_F ? 0.f : ml[2 * s + 1] * expf(ml[2 * s] - m);
    const float inv = 1.f / l;
    for (int d = lane; d < R; d += 32) {
        float o = 0.f;
        for (int s = 0; s < splits; ++s)
            if (ml[2 * s] != -CUDART_INF_F) o = fmaf(part_o[((size_t)pair * splits + s) * R + d], expf(ml[2 * s] - m), o);
        out[(size_t)pair * R + d] = o * inv;
    }
}

template <typename TC, int NACC>
static int latent_attention_launch(const float* q, const void* pages, const int* page_table, int pt_stride, const int* tok_pos,
                                   const int* tok_seq, const int* slots, float* out, float* part_o, float* part_ml, int T, int H,
                                   int R, int Dk, int page_size, float scale, int window, int splits, cudaStream_t stream) {
    const size_t smem = ((size_t)LA_WARPS * Dk + (size_t)LA_KEYS * (Dk + 1)) * sizeof(float);
    if (smem > 220 * 1024) return LQ_BAD_SIZE;
    auto kernel = latent_attention_kernel<TC, NACC>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(T, (H + LA_WARPS - 1) / LA_WARPS, splits);
    int rc = launch_pdl(kernel, grid, dim3(LA_WARPS * 32), smem, stream, q, (const TC*)pages, page_table, pt_stride, tok_pos,
                        tok_seq, slots, out, part_o, part_ml, H, R, Dk, page_size, scale, window, splits);
    if (rc != LQ_OK || splits == 1) return rc;
    const int n = T * H;
    return launch_pdl(latent_merge_kernel, dim3((n + 3) / 4), dim3(128), 0, stream, (const float*)part_o, (const float*)part_ml,
                      out, n, R, splits);
}

LQ_EXPORT int lq_latent_attention(const float* q, const void* pages, int cache_dtype, const int* page_table, int pt_stride,
                                  const int* tok_pos, const int* tok_seq, const int* slots, float* out, float* part_o,
                                  float* part_ml, int T, int H, int R, int Dk, int page_size, float scale, int window,
                                  int splits, cudaStream_t stream) {
    if (T <= 0) return LQ_OK;
    if (R < 1 || R > Dk || R > 1024 || splits < 1 || (splits > 1 && (!part_o || !part_ml))) return LQ_BAD_SIZE;
    typedef __nv_bfloat16 bf;
#define LQ_GO(TC, NACC) return latent_attention_launch<TC, NACC>(q, pages, page_table, pt_stride, tok_pos, tok_seq, slots, out, \
        part_o, part_ml, T, H, R, Dk, page_size, scale, window, splits, stream)
#define LQ_BY_R(TC) do { if (R <= 64) LQ_GO(TC, 2); if (R <= 128) LQ_GO(TC, 4); if (R <= 256) LQ_GO(TC, 8); if (R <= 512) LQ_GO(TC, 16); LQ_GO(TC, 32); } while (0)
    if (cache_dtype == LQ_F32) LQ_BY_R(float);
    if (cache_dtype == LQ_BF16) LQ_BY_R(bf);
#undef LQ_BY_R
#undef LQ_GO
    return LQ_BAD_DTYPE;
}
