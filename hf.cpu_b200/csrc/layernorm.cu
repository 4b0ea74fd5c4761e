// Layer norm of rows of the float32 stream, and the token shift behind a norm.
//
//     norm(x)_i = (x_i - mean) / sqrt(var + eps) * w_i        var = mean((x - mean)^2)            (center = 1)
//     norm(x)_i = x_i / sqrt(mean(x^2) + eps) * w_i                                                (center = 0)
//
// Mean and variance are taken in two passes over the row (the deviations are squared, not the values), in float32, with
// one fixed summation order per row, so a row's result depends on nothing but the row.
//
// Token shift: what the sublayer behind the norm reads is h_t + (h_(t-1) - h_t) * mu, with h = norm(x), mu a vector per
// layer, and h_(t-1) the previous token's h before its own shift: the previous row of the step, or, for a request's
// first token of the step, what the request's state slot holds (zeros for a new request).  The block of a request's
// first token of the step reads the slot and then leaves the h of the request's last token of the step there; no other
// block touches that slot, so a step is one launch whatever its mix of portions and single tokens, and replays as a graph.
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;

namespace hfb {
int *error_word();

constexpr int LN_THREADS = 256;

// Sum over the block, the same value in every thread; `red` holds one float per warp.
__device__ __forceinline__ float ln_block_sum(float v, float *red)
{
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                                   // the last sum's readers are done with red
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); i++) t += red[i];
    return t;
}

// row[i] = norm(x)[i] for the thread's own i (i = threadIdx.x, + blockDim.x, ...): nobody reads another thread's entries.
__device__ __forceinline__ void ln_row(const float *x, const float *w, float eps, int center, int E, float *row, float *red)
{
    float s = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) { const float v = x[i]; row[i] = v; s += v; }
    const float mean = center ? ln_block_sum(s, red) / (float)E : 0.f;
    float ss = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) { const float d = row[i] - mean; ss = fmaf(d, d, ss); }
    const float r = 1.0f / sqrtf(ln_block_sum(ss, red) / (float)E + eps);
    for (int i = threadIdx.x; i < E; i += blockDim.x) row[i] = (row[i] - mean) * r * w[i];
}

// out[r] = norm(x[rows ? rows[r] : r]); one block per output row.
template <typename TO>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_kernel(const float *x, const float *w, float eps, int center, const int32_t *rows, int n_src, TO *out, int E, int *err)
{
    pdl_entry();
    pdl_sync_small();
    extern __shared__ float ln_smem[];
    float *row = ln_smem, *red = ln_smem + E;
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    if (src < 0 || src >= n_src) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); return; }
    ln_row(x + (size_t)src * E, w, eps, center, E, row, red);
    for (int i = threadIdx.x; i < E; i += blockDim.x) out[(size_t)r * E + i] = from_f32<TO>(row[i]);
}

// out[t] = h_t + (h_(t-1) - h_t) * mu with h = norm(x); one block per token.  state [slots][slot_stride] float32.
template <typename TO>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_shift_kernel(const float *x, const float *w, const float *mu, float eps, int center, float *state, size_t slot_stride,
                       const int32_t *token_seq, const int32_t *cu_tokens, const int32_t *seq_slots, int n_slots, TO *out, int T,
                       int E, int *err)
{
    pdl_entry();
    pdl_sync_small();
    extern __shared__ float ln_smem[];
    float *mine = ln_smem, *other = ln_smem + E, *red = ln_smem + 2 * E;
    const int t = blockIdx.x;
    const int seq = token_seq[t];
    const int t0 = cu_tokens[seq], t_last = cu_tokens[seq + 1] - 1;
    ln_row(x + (size_t)t * E, w, eps, center, E, mine, red);
    if (t > t0) {
        // the previous token's row is in this step: its norm is made again here rather than passed between blocks
        ln_row(x + (size_t)(t - 1) * E, w, eps, center, E, other, red);
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            const float h = mine[i];
            out[(size_t)t * E + i] = from_f32<TO>(fmaf(other[i] - h, mu[i], h));
        }
        return;
    }
    const int slot = seq_slots[seq];
    if (slot < 0 || slot >= n_slots) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); return; }
    float *st = state + (size_t)slot * slot_stride;
    const float *leave = mine;
    if (t_last > t) {
        ln_row(x + (size_t)t_last * E, w, eps, center, E, other, red);
        leave = other;
    }
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        const float h = mine[i], before = st[i];
        st[i] = leave[i];
        out[(size_t)t * E + i] = from_f32<TO>(fmaf(before - h, mu[i], h));
    }
}

// out = a * sigmoid(g) (gate 1) or a * silu(g) (gate 0), g the sum of `splits` float32 planes [T, g_stride] read from
// column g_col0 on, plus a bias where there is one.
template <typename TA>
__global__ void gate_mul_kernel(const TA *a, const float *g, int splits, int g_stride, int g_col0, const float *bias, int gate,
                                TA *out, int T, int C)
{
    pdl_entry();
    pdl_sync_small();
    const size_t total = (size_t)T * C, plane = (size_t)T * g_stride;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const float *gp = g + (i / C) * g_stride + g_col0 + c;
        float z = 0.f;
        for (int s = 0; s < splits; s++) z += gp[(size_t)s * plane];
        if (bias) z += bias[c];
        const float sg = 1.0f / (1.0f + expf(-z));
        out[i] = from_f32<TA>(to_f32(a[i]) * (gate ? sg : z * sg));
    }
}


// The tail of a product that ends a sublayer, for streams normed by the norms above: residual[m] += sum of the product's
// `splits` partial sums (+ bias), then xn[m] = norm(residual[m]) for the next product, one pass over the row with its
// values in registers (one block per row, up to PER values a thread).  splits = 0: the product has already been
// added to the stream, only the norm is left.  With `mu`, the token shift of a step in which every request brings ONE
// token: row m is request m, the previous token's h comes from the request's slot and the row's h is left there.
constexpr int LNT_PER = 16;

template <typename TO, int PER>
__global__ void __launch_bounds__(1024)
reduce_residual_layernorm_kernel(const float *partial, int splits, int M, int N, const void *bias, int bias_dt, float *residual,
                                 const float *w, float eps, int center, const float *mu, float *state, size_t slot_stride,
                                 const int32_t *seq_slots, int n_slots, TO *xn, int *err)
{
    pdl_entry();
    __shared__ float red[32];
    const int m = blockIdx.x;
    float vals[PER];
    pdl_sync_small();
    const size_t MN = (size_t)M * N;
    float *res = residual + (size_t)m * N;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PER; j++) vals[j] = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 4) {              // four splits' reads in flight for every value: their latency is what this costs
        float q[4][PER];
#pragma unroll
        for (int k = 0; k < 4; k++)
#pragma unroll
            for (int j = 0; j < PER; j++) {
                const int i = threadIdx.x + j * blockDim.x;
                q[k][j] = (s0 + k < splits && i < N) ? partial[(size_t)(s0 + k) * MN + (size_t)m * N + i] : 0.f;
            }
#pragma unroll
        for (int k = 0; k < 4; k++)
#pragma unroll
            for (int j = 0; j < PER; j++) vals[j] += q[k][j];
    }
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        float v = vals[j];
        if (i < N) {
            if (bias) v += load_any(bias, bias_dt, i);
            v += res[i];
            if (splits > 0 || bias) res[i] = v;
        }
        vals[j] = v;
        sum += v;
    }
    if (!xn) return;
    const float mean = center ? ln_block_sum(sum, red) / (float)N : 0.f;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        const float d = i < N ? vals[j] - mean : 0.f;
        ss = fmaf(d, d, ss);
    }
    const float r = 1.0f / sqrtf(ln_block_sum(ss, red) / (float)N + eps);
    float *st = nullptr;
    if (mu) {
        const int slot = seq_slots[m];
        if (slot < 0 || slot >= n_slots) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); return; }
        st = state + (size_t)slot * slot_stride;
    }
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i >= N) continue;
        float h = (vals[j] - mean) * r * w[i];
        if (mu) {
            const float before = st[i];
            st[i] = h;
            h = fmaf(before - h, mu[i], h);
        }
        xn[(size_t)m * N + i] = from_f32<TO>(h);
    }
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_layernorm(const float *x, const float *w, float eps, int center, const int32_t *rows, int n_src, void *out,
                             int out_dt, int N, int E, hfb_stream s)
{
    if (N <= 0) return HFB_OK;
    if (!x || !w || !out || !valid_dt(out_dt) || E <= 0 || n_src <= 0) return fail(HFB_EINVAL, "layernorm: bad arguments (E=%d)", E);
    const size_t smem = ((size_t)E + 32) * sizeof(float);
    if (smem > 48 * 1024) return fail(HFB_ENOTSUP, "layernorm: rows of %d values exceed %d", E, 48 * 256 - 32);
    if (out_dt == HFB_F32)
        g_launch_err = launch_pdl(layernorm_kernel<float>, dim3(N), dim3(LN_THREADS), smem, (cudaStream_t)s, x, w, eps, center, rows, n_src,
                                  (float *)out, E, error_word());
    else
        g_launch_err = launch_pdl(layernorm_kernel<__nv_bfloat16>, dim3(N), dim3(LN_THREADS), smem, (cudaStream_t)s, x, w, eps, center, rows,
                                  n_src, (__nv_bfloat16 *)out, E, error_word());
    return check_pdl_launch(g_launch_err, "layernorm");
}

extern "C" int hfb_layernorm_shift(const float *x, const float *w, const float *mu, float eps, int center, float *state,
                                   int64_t slot_stride, const int32_t *token_seq, const int32_t *cu_tokens, const int32_t *seq_slots,
                                   int n_slots, void *out, int out_dt, int T, int E, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!x || !w || !mu || !state || !token_seq || !cu_tokens || !seq_slots || !out || !valid_dt(out_dt) || E <= 0 || slot_stride < E)
        return fail(HFB_EINVAL, "layernorm_shift: bad arguments (E=%d)", E);
    const size_t smem = (2 * (size_t)E + 32) * sizeof(float);
    if (smem > 48 * 1024) return fail(HFB_ENOTSUP, "layernorm_shift: rows of %d values exceed %d", E, 24 * 256 - 16);
    if (out_dt == HFB_F32)
        g_launch_err = launch_pdl(layernorm_shift_kernel<float>, dim3(T), dim3(LN_THREADS), smem, (cudaStream_t)s, x, w, mu, eps, center, state,
                                  (size_t)slot_stride, token_seq, cu_tokens, seq_slots, n_slots, (float *)out, T, E, error_word());
    else
        g_launch_err = launch_pdl(layernorm_shift_kernel<__nv_bfloat16>, dim3(T), dim3(LN_THREADS), smem, (cudaStream_t)s, x, w, mu, eps, center,
                                  state, (size_t)slot_stride, token_seq, cu_tokens, seq_slots, n_slots, (__nv_bfloat16 *)out, T, E,
                                  error_word());
    return check_pdl_launch(g_launch_err, "layernorm_shift");
}

extern "C" int hfb_gate_mul(const void *a, int dt, const float *g, int splits, int g_stride, int g_col0, const float *bias, int gate,
                            void *out, int T, int C, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!a || !g || !out || !valid_dt(dt) || splits < 1 || C <= 0 || g_col0 < 0 || g_col0 + C > g_stride || (gate != 0 && gate != 1))
        return fail(HFB_EINVAL, "gate_mul: bad arguments (C=%d)", C);
    const size_t total = (size_t)T * C;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dt == HFB_F32)
        g_launch_err = launch_pdl(gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, (const float *)a, g, splits, g_stride,
                                  g_col0, bias, gate, (float *)out, T, C);
    else
        g_launch_err = launch_pdl(gate_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, (const __nv_bfloat16 *)a, g,
                                  splits, g_stride, g_col0, bias, gate, (__nv_bfloat16 *)out, T, C);
    return check_pdl_launch(g_launch_err, "gate_mul");
}

extern "C" int hfb_reduce_residual_layernorm(const float *partial, int splits, int M, int N, const void *bias, int bias_dt,
                                             float *residual, const float *w, float eps, int center, const float *mu, float *state,
                                             int64_t slot_stride, const int32_t *seq_slots, int n_slots, void *xn, int xn_dt,
                                             hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    if (splits < 0 || (splits > 0 && !partial) || N <= 0 || !residual || (bias && !valid_dt(bias_dt)) || (xn && (!w || !valid_dt(xn_dt))) ||
        (mu && (!xn || !state || !seq_slots || slot_stride < N)))
        return fail(HFB_EINVAL, "reduce_residual_layernorm: bad arguments (N=%d splits=%d)", N, splits);
    if (N > LNT_PER * 1024) return fail(HFB_ENOTSUP, "reduce_residual_layernorm: rows of %d values exceed %d", N, LNT_PER * 1024);
    int threads = ((N + 3) / 4 + 31) / 32 * 32;           // four values a thread where the row allows
    if (threads > 1024) threads = 1024;
#define HFB_LNT(TY, PER) \
    g_launch_err = launch_pdl(reduce_residual_layernorm_kernel<TY, PER>, dim3(M), dim3(threads), 0, (cudaStream_t)s, partial, splits, M, N, bias, \
                              bias_dt, residual, w, eps, center, mu, state, (size_t)slot_stride, seq_slots, n_slots, (TY *)xn, error_word())
    const bool few = N <= 4 * threads;                     // rows of up to 4,096 values: four a thread, all in registers
    if (xn_dt == HFB_F32 || !xn) { if (few) HFB_LNT(float, 4); else HFB_LNT(float, LNT_PER); }
    else { if (few) HFB_LNT(__nv_bfloat16, 4); else HFB_LNT(__nv_bfloat16, LNT_PER); }
#undef HFB_LNT
    return check_pdl_launch(g_launch_err, "reduce_residual_layernorm");
}
