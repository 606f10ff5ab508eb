// Mixers that carry a matrix of fixed size per head from token to token instead of keys and values:
//
//   S_t = a_t S_(t-1) + b_t k_t v_t^T          o_t = S_t^T q_t
//
// with a_t, b_t scalars per head and token.  Two instances:
//   retention   a_t = the head's fixed decay, b_t = 1
//   mlstm       a_t = exp(f_t + m_(t-1) - m_t), b_t = exp(i_t - m_t), m_t = max(f_t + m_(t-1), i_t), m_0 = 0,
//               i_t = cap tanh(x_i / cap), f_t = logsigmoid(cap tanh(x_f / cap)); the normaliser n_t (the same
//               recurrence with v = 1) rides along as one more value column, so n_t . q_t is that column's output
//
// State, products and gates are float32 whatever the activations' storage is; q and k are rotated (optionally)
// and scaled in float32 as they are staged, so nothing that enters the recurrence is rounded on the way.
// One kernel serves prompts and single tokens: a sequence's tokens are walked in order from the state that the
// step before left in the sequence's slot, so every way of cutting a prompt gives the same bits.
#include "common.cuh"
#include <math_constants.h>

constexpr int SC_R = 8;          // threads that share one value column (each holds every 8th key row of it)
constexpr int SC_COLS = 16;      // value columns of a block
constexpr int SC_THREADS = SC_R * SC_COLS;
constexpr int SC_CHUNK = 16;     // tokens staged in shared memory at a time

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

struct ScanArgs {
    const void* qkv;             // [rows, stride]: q at q_off, k at k_off (H heads of dk each), v at v_off (H heads of dv)
    int stride, q_off, k_off, v_off;
    const float* cos_t;          // [positions, rot/2] or null
    const float* sin_t;
    int rot;                     // rotated dimensions of a head (pairs i, i + rot/2)
    const int* tok_pos;          // position of every row
    const float* gate_pre;       // mlstm: [rows, 2H] pre-activations of the input gates (H) and forget gates (H), no bias
    const float* gate_bias;      // mlstm: [2H]
    float gate_cap;
    const float* decay;          // retention: [H]
    float q_scale, k_scale;
    float* state;                // [slots][H][dk (+1)][dvx]; mlstm's extra row holds m (in every column)
    long long slot_stride;
    const int* cu_rows;          // [B + 1]
    const int* slots;            // [B]
    float* out;                  // [rows, H, dvx] raw S^T q (mlstm: column dv holds n . q)
    float* exp_neg_m;            // mlstm: [rows, H] exp(-m_t)
    int H, dk, dv;
};

template <typename T, int KR, bool MLSTM>
__global__ void __launch_bounds__(SC_THREADS) linear_scan_kernel(ScanArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    const int dk = a.dk, dv = a.dv, dvx = dv + (MLSTM ? 1 : 0), H = a.H;
    float* qs = sm;                              // [CHUNK][dk]
    float* ks = qs + SC_CHUNK * dk;              // [CHUNK][dk]
    float* vs = ks + SC_CHUNK * dk;              // [CHUNK][COLS], already times b_t
    float* as = vs + SC_CHUNK * SC_COLS;         // [CHUNK] a_t
    float* gi = as + SC_CHUNK;                   // [CHUNK] i_t, then b_t
    float* gf = gi + SC_CHUNK;                   // [CHUNK] f_t
    float* ms = gf + SC_CHUNK;                   // [CHUNK + 1] m before each token of the chunk, and after the last
    const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * SC_COLS;
    const int tid = threadIdx.x, c = tid / SC_R, rr = tid % SC_R, col = col0 + c;
    const bool live = col < dvx;
    const int row0 = a.cu_rows[b], row1 = a.cu_rows[b + 1];
    float* st = a.state + (long long)a.slots[b] * a.slot_stride + (size_t)h * (dk + (MLSTM ? 1 : 0)) * dvx;
    float S[KR];
#pragma unroll
    for (int i = 0; i < KR; ++i) {
        const int r = i * SC_R + rr;
        S[i] = (live && r < dk) ? st[(size_t)r * dvx + col] : 0.f;
    }
    float m = 0.f;
    if (MLSTM) m = st[(size_t)dk * dvx + (live ? col : col0)];
    const float decay = MLSTM ? 0.f : a.decay[h];
    const T* base = (const T*)a.qkv;
    const int half = a.rot >> 1;

    for (int t0 = row0; t0 < row1; t0 += SC_CHUNK) {
        const int n = min(SC_CHUNK, row1 - t0);
        // ---- stage q and k (rotated, scaled) and this block's value columns
        for (int e = tid; e < n * dk; e += SC_THREADS) {
            const int t = e / dk, j = e % dk;
            const T* row = base + (size_t)(t0 + t) * a.stride;
            const T* qh = row + a.q_off + h * dk;
            const T* kh = row + a.k_off + h * dk;
            float qv = to_f32(qh[j]), kv = to_f32(kh[j]);
            if (j < a.rot) {
                const int f = j < half ? j : j - half, jp = j < half ? j + half : j - half;
                const size_t at = (size_t)a.tok_pos[t0 + t] * half + f;
                const float cs = a.cos_t[at], sn = j < half ? -a.sin_t[at] : a.sin_t[at];
                qv = qv * cs + to_f32(qh[jp]) * sn;
                kv = kv * cs + to_f32(kh[jp]) * sn;
            }
            qs[t * dk + j] = qv * a.q_scale;
            ks[t * dk + j] = kv * a.k_scale;
        }
        if (MLSTM) {
            if (tid < n) {
                const float* g = a.gate_pre + (size_t)(t0 + tid) * 2 * H;
                const float cap = a.gate_cap;
                gi[tid] = cap * tanhf((g[h] + a.gate_bias[h]) / cap);
                gf[tid] = log_sigmoid(cap * tanhf((g[H + h] + a.gate_bias[H + h]) / cap));
            }
            __syncthreads();
            if (tid == 0) {
                float mm = m;
                for (int t = 0; t < n; ++t) {
                    ms[t] = mm;
                    mm = fmaxf(gf[t] + mm, gi[t]);
                }
                ms[n] = mm;
            }
            __syncthreads();
            m = ms[n];
            if (tid < n) {
                const float m_new = ms[tid + 1];
                as[tid] = expf(gf[tid] + ms[tid] - m_new);
                gi[tid] = expf(gi[tid] - m_new);
                if (blockIdx.z == 0) a.exp_neg_m[(size_t)(t0 + tid) * H + h] = expf(-m_new);
            }
            __syncthreads();
        }
        for (int e = tid; e < n * SC_COLS; e += SC_THREADS) {
            const int t = e / SC_COLS, cc = e % SC_COLS, vc = col0 + cc;
            float v = 0.f;
            if (vc < dv) v = to_f32(base[(size_t)(t0 + t) * a.stride + a.v_off + h * dv + vc]);
            else if (MLSTM && vc == dv) v = 1.f;
            vs[e] = MLSTM ? v * gi[t] : v;
        }
        __syncthreads();
        // ---- the recurrence, token by token
        for (int t = 0; t < n; ++t) {
            const float at = MLSTM ? as[t] : decay;
            const float bv = vs[t * SC_COLS + c];
            const float* kt = ks + t * dk;
            const float* qt = qs + t * dk;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < KR; ++i) {
                const int r = i * SC_R + rr;
                if (r < dk) {
                    S[i] = fmaf(at, S[i], bv * kt[r]);
                    acc = fmaf(S[i], qt[r], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (rr == 0 && live) a.out[((size_t)(t0 + t) * H + h) * dvx + col] = acc;
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < KR; ++i) {
            const int r = i * SC_R + rr;
            if (r < dk) st[(size_t)r * dvx + col] = S[i];
        }
        if (MLSTM && rr == 0) st[(size_t)dk * dvx + col] = m;
    }
}

template <typename T, bool MLSTM>
static int scan_launch(const ScanArgs& a, int B, cudaStream_t stream) {
    const int dvx = a.dv + (MLSTM ? 1 : 0);
    dim3 grid(B, a.H, (dvx + SC_COLS - 1) / SC_COLS);
    size_t smem = (size_t)(2 * SC_CHUNK * a.dk + SC_CHUNK * SC_COLS + 4 * SC_CHUNK + 1) * sizeof(float);
    if (a.dk <= 8 * SC_R) return launch_pdl(linear_scan_kernel<T, 8, MLSTM>, grid, dim3(SC_THREADS), smem, stream, a);
    if (a.dk <= 16 * SC_R) return launch_pdl(linear_scan_kernel<T, 16, MLSTM>, grid, dim3(SC_THREADS), smem, stream, a);
    if (a.dk <= 32 * SC_R) return launch_pdl(linear_scan_kernel<T, 32, MLSTM>, grid, dim3(SC_THREADS), smem, stream, a);
    return LQ_BAD_SIZE;
}

LQ_EXPORT int lq_linear_scan(const void* qkv, int dtype, int stride, int q_off, int k_off, int v_off, const float* cos_t,
                             const float* sin_t, int rot, const int* tok_pos, const float* gate_pre,
                             const float* gate_bias, float gate_cap, const float* decay, float q_scale, float k_scale,
                             float* state, long long slot_stride, const int* cu_rows, const int* slots, float* out,
                             float* exp_neg_m, int B, int H, int dk, int dv, int mlstm, cudaStream_t stream) {
    if (B <= 0) return LQ_OK;
    if (rot % 2 || rot > dk || (rot && (!cos_t || !sin_t))) return LQ_BAD_SIZE;
    if (mlstm ? (!gate_pre || !gate_bias || !exp_neg_m) : !decay) return LQ_BAD_SIZE;
    ScanArgs a{qkv, stride, q_off, k_off, v_off, cos_t, sin_t, rot, tok_pos, gate_pre, gate_bias, gate_cap, decay,
               q_scale, k_scale, state, slot_stride, cu_rows, slots, out, exp_neg_m, H, dk, dv};
    if (dtype == LQ_F32) return mlstm ? scan_launch<float, true>(a, B, stream) : scan_launch<float, false>(a, B, stream);
    if (dtype == LQ_BF16)
        return mlstm ? scan_launch<__nv_bfloat16, true>(a, B, stream) : scan_launch<__nv_bfloat16, false>(a, B, stream);
    return LQ_BAD_DTYPE;
}

// ------------------------------------------------------------------ per-head unit norm, weight and gate
// raw [rows, H, dvx] float32 -> out [rows, H * dv]: each head's dv values (divided by the head's denominator
// first, where there is one) over their root mean square, times weight [H * dv] (optional), times
// act(gate[row, h * dv + d]) (0: no gate, 1: sigmoid, 2: silu).  One warp per (row, head); the sum of squares
// runs in an order that depends on dv alone.
// Denominator (mlstm): max(|raw[row, h, dv]|, exp_neg_m[row, h]) + 1e-6.
template <typename T>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(const float* __restrict__ raw, int dvx,
                                                             const float* __restrict__ exp_neg_m,
                                                             const float* __restrict__ weight, const T* __restrict__ gate,
                                                             int gate_stride, int act, T* __restrict__ out, int n_pairs,
                                                             int H, int dv, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_pairs) return;
    const int row = pair / H, h = pair % H;
    const float* r = raw + (size_t)pair * dvx;
    float inv = 1.f;
    if (exp_neg_m) inv = 1.f / (fmaxf(fabsf(r[dv]), exp_neg_m[pair]) + 1e-6f);
    float s = 0.f;
    for (int d = lane; d < dv; d += 32) {
        const float v = r[d] * inv;
        s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    const float scale = inv / sqrtf(s / (float)dv + eps);
    for (int d = lane; d < dv; d += 32) {
        float v = r[d] * scale;
        if (weight) v *= weight[h * dv + d];
        if (act) {
            const float g = to_f32(gate[(size_t)row * gate_stride + h * dv + d]);
            const float sg = 1.f / (1.f + expf(-g));
            v *= act == 1 ? sg : g * sg;
        }
        out[(size_t)row * H * dv + h * dv + d] = from_f32<T>(v);
    }
}

LQ_EXPORT int lq_head_norm_gate(const float* raw, int dvx, const float* exp_neg_m, const float* weight, const void* gate,
                                int gate_stride, int act, void* out, int dtype, int rows, int H, int dv, float eps,
                                cudaStream_t stream) {
    const int n = rows * H;
    if (n <= 0) return LQ_OK;
    if (act < 0 || act > 2 || (act && !gate)) return LQ_BAD_SIZE;
    dim3 grid((n + 3) / 4);
    if (dtype == LQ_F32)
        return launch_pdl(head_norm_gate_kernel<float>, grid, dim3(128), 0, stream, raw, dvx, exp_neg_m, weight,
                          (const float*)gate, gate_stride, act, (float*)out, n, H, dv, eps);
    if (dtype == LQ_BF16)
        return launch_pdl(head_norm_gate_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, raw, dvx, exp_neg_m, weight,
                          (const __nv_bfloat16*)gate, gate_stride, act, (__nv_bfloat16*)out, n, H, dv, eps);
    return LQ_BAD_DTYPE;
}
