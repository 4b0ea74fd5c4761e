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
constexpr int LNT_PER = 16;         // values a thread holds of a row of more than 8,192 (the register kernels)

// Sum over the block, the same value in every thread; `red` holds one float per warp.  The warps' sums meet in one more
// warp-wide sum that every warp makes for itself: one fixed order, whatever the block's size.
__device__ __forceinline__ float ln_block_sum(float v, float *red)
{
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                                   // the last sum's readers are done with red
    if (lane == 0) red[warp] = v;
    __syncthreads();
    return warp_sum(lane < (int)(blockDim.x >> 5) ? red[lane] : 0.f);
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

// Two sums over the block at once.
__device__ __forceinline__ void ln_block_sum2(float &a, float &b, float *red)
{
    a = warp_sum(a);
    b = warp_sum(b);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) { red[warp] = a; red[32 + warp] = b; }
    __syncthreads();
    a = warp_sum(lane < nw ? red[lane] : 0.f);
    b = warp_sum(lane < nw ? red[32 + lane] : 0.f);
}

// out[t] = h_t + (h_(t-1) - h_t) * mu with h = norm(x); one block per token, a row's values in registers (PER a thread).
// A block norms two rows side by side, its own and one other: the previous token's where that is in this step (its norm
// is made again here rather than passed between blocks), or, in the block of a request's first token of the step, the
// request's last token's, which goes to the slot.  state [slots][slot_stride] float32.
template <typename TO, int PER>
__global__ void __launch_bounds__(PER <= 8 ? 512 : 1024)
layernorm_shift_kernel(const float *x, const float *w, const float *mu, float eps, int center, float *state, size_t slot_stride,
                       const int32_t *token_seq, const int32_t *cu_tokens, const int32_t *seq_slots, int n_slots, TO *out, int T,
                       int E, int *err)
{
    pdl_entry();
    __shared__ float red[64];
    const int t = blockIdx.x;
    // the weights and the shift do not come from the kernel in front: fetch them while it finishes (rows of up to 4,096
    // values; wider rows read them at the end, for want of registers)
    constexpr bool EARLY = PER <= 8;
    float wv[EARLY ? PER : 1], muv[EARLY ? PER : 1];
    if (EARLY) {
#pragma unroll
        for (int j = 0; j < (EARLY ? PER : 1); j++) {
            const int i = threadIdx.x + j * blockDim.x;
            wv[j] = i < E ? w[i] : 0.f;
            muv[j] = i < E ? mu[i] : 0.f;
        }
    }
    pdl_sync_small();
    const int seq = token_seq[t];
    const int t0 = cu_tokens[seq], t_last = cu_tokens[seq + 1] - 1;
    const bool first = t == t0;
    const int t_other = first ? t_last : t - 1;
    const bool two = t_other != t;
    const float *xa = x + (size_t)t * E, *xb = x + (size_t)t_other * E;
    float va[PER], vb[PER];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        va[j] = i < E ? xa[i] : 0.f;
        vb[j] = (two && i < E) ? xb[i] : 0.f;
    }
    float *st = nullptr;
    float bef[EARLY ? PER : 1];
    if (first) {
        const int slot = seq_slots[seq];
        if (slot < 0 || slot >= n_slots) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); return; }
        st = state + (size_t)slot * slot_stride;
        if (EARLY) {
#pragma unroll
            for (int j = 0; j < (EARLY ? PER : 1); j++) {
                const int i = threadIdx.x + j * blockDim.x;
                bef[j] = i < E ? st[i] : 0.f;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < PER; j++) {
        sa += va[j];
        sb += vb[j];
    }
    float mean_a = 0.f, mean_b = 0.f;
    if (center) {
        ln_block_sum2(sa, sb, red);
        mean_a = sa / (float)E;
        mean_b = sb / (float)E;
    }
    float qa = 0.f, qb = 0.f;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        const float da = i < E ? va[j] - mean_a : 0.f, db = i < E ? vb[j] - mean_b : 0.f;
        qa = fmaf(da, da, qa);
        qb = fmaf(db, db, qb);
    }
    ln_block_sum2(qa, qb, red);
    const float ra = 1.0f / sqrtf(qa / (float)E + eps), rb = 1.0f / sqrtf(qb / (float)E + eps);
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i >= E) continue;
        const float wi = EARLY ? wv[EARLY ? j : 0] : w[i], mi = EARLY ? muv[EARLY ? j : 0] : mu[i];
        const float h = (va[j] - mean_a) * ra * wi;
        const float other = two ? (vb[j] - mean_b) * rb * wi : h;
        float before;
        if (first) {
            before = EARLY ? bef[EARLY ? j : 0] : st[i];
            st[i] = other;                           // the request's last row of the step (this one, if it is the only one)
        } else {
            before = other;
        }
        out[(size_t)t * E + i] = from_f32<TO>(fmaf(before - h, mi, h));
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
    constexpr int FLY = PER <= 8 ? 32 / PER : 1;          // splits whose reads are in flight together: their latency is what this costs
    for (int s0 = 0; s0 < splits; s0 += FLY) {
        float q[FLY][PER];
#pragma unroll
        for (int k = 0; k < FLY; k++)
#pragma unroll
            for (int j = 0; j < PER; j++) {
                const int i = threadIdx.x + j * blockDim.x;
                q[k][j] = (s0 + k < splits && i < N) ? partial[(size_t)(s0 + k) * MN + (size_t)m * N + i] : 0.f;
            }
#pragma unroll
        for (int k = 0; k < FLY; k++)
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


// The same tail with 16-byte accesses, for rows whose length is a multiple of four: PV float4 a thread.  Everything the
// row needs is requested before anything is used (the request's slot first, then the partial sums, the stream's row,
// the weights, the shift and the slot's row), so the pass costs about one round trip to memory and two block sums.
__device__ __forceinline__ float4 f4_add(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

template <typename TO> __device__ __forceinline__ void store4(TO *p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float *p, float4 v) { *(float4 *)p = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16 *p, float4 v)
{
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *(uint32_t *)&lo;
    u.y = *(uint32_t *)&hi;
    *(uint2 *)p = u;
}

template <typename TO, int PV>
__global__ void __launch_bounds__(1024)
reduce_residual_layernorm_vec_kernel(const float *partial, int splits, int M, int N, const void *bias, int bias_dt, float *residual,
                                     const float *w, float eps, int center, const float *mu, float *state, size_t slot_stride,
                                     const int32_t *seq_slots, int n_slots, TO *xn, int *err)
{
    pdl_entry();
    __shared__ float red[32];
    const int m = blockIdx.x, N4 = N >> 2;
    pdl_sync_small();
    int slot = 0;
    if (mu) slot = seq_slots[m];
    const size_t MN4 = ((size_t)M * N) >> 2;
    const float4 *part = (const float4 *)partial + (size_t)m * N4;
    float4 *res = (float4 *)(residual + (size_t)m * N);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 vals[PV], wv[PV], muv[PV], bef[PV];
    constexpr int FLY = PV == 1 ? 8 : 4 / PV;            // splits whose reads are in flight together (registers decide)
    float4 acc[PV];
#pragma unroll
    for (int j = 0; j < PV; j++) acc[j] = zero;
    for (int s0 = 0; s0 < splits; s0 += FLY) {
        float4 q[FLY][PV];
#pragma unroll
        for (int k = 0; k < FLY; k++)
#pragma unroll
            for (int j = 0; j < PV; j++) {
                const int i = threadIdx.x + j * blockDim.x;
                q[k][j] = (s0 + k < splits && i < N4) ? part[(size_t)(s0 + k) * MN4 + i] : zero;
            }
        if (s0 == 0) {
            // the row's other operands go out behind the first partial sums
#pragma unroll
            for (int j = 0; j < PV; j++) {
                const int i = threadIdx.x + j * blockDim.x;
                vals[j] = i < N4 ? res[i] : zero;
                wv[j] = (xn && i < N4) ? ((const float4 *)w)[i] : zero;
                muv[j] = (mu && i < N4) ? ((const float4 *)mu)[i] : zero;
            }
        }
#pragma unroll
        for (int k = 0; k < FLY; k++)
#pragma unroll
            for (int j = 0; j < PV; j++) acc[j] = f4_add(acc[j], q[k][j]);
    }
    if (splits == 0) {
#pragma unroll
        for (int j = 0; j < PV; j++) {
            const int i = threadIdx.x + j * blockDim.x;
            vals[j] = i < N4 ? res[i] : zero;
            wv[j] = (xn && i < N4) ? ((const float4 *)w)[i] : zero;
            muv[j] = (mu && i < N4) ? ((const float4 *)mu)[i] : zero;
        }
    }
    float4 *st = nullptr;
    if (mu) {
        if (slot < 0 || slot >= n_slots) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); return; }
        st = (float4 *)(state + (size_t)slot * slot_stride);
#pragma unroll
        for (int j = 0; j < PV; j++) {
            const int i = threadIdx.x + j * blockDim.x;
            bef[j] = i < N4 ? st[i] : zero;
        }
    }
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PV; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < N4) {
            float4 v = acc[j];
            if (bias) v = f4_add(v, make_float4(load_any(bias, bias_dt, 4 * i), load_any(bias, bias_dt, 4 * i + 1),
                                                load_any(bias, bias_dt, 4 * i + 2), load_any(bias, bias_dt, 4 * i + 3)));
            v = f4_add(v, vals[j]);
            if (splits > 0 || bias) res[i] = v;
            vals[j] = v;
            sum += (v.x + v.y) + (v.z + v.w);
        }
    }
    if (!xn) return;
    const float mean = center ? ln_block_sum(sum, red) / (float)N : 0.f;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PV; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < N4) {
            const float4 v = vals[j];
            const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
            ss += (a * a + b * b) + (c * c + d * d);
        }
    }
    const float r = 1.0f / sqrtf(ln_block_sum(ss, red) / (float)N + eps);
#pragma unroll
    for (int j = 0; j < PV; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i >= N4) continue;
        const float4 v = vals[j];
        float4 h = make_float4((v.x - mean) * r * wv[j].x, (v.y - mean) * r * wv[j].y, (v.z - mean) * r * wv[j].z, (v.w - mean) * r * wv[j].w);
        if (mu) {
            st[i] = h;
            h = make_float4(fmaf(bef[j].x - h.x, muv[j].x, h.x), fmaf(bef[j].y - h.y, muv[j].y, h.y),
                            fmaf(bef[j].z - h.z, muv[j].z, h.z), fmaf(bef[j].w - h.w, muv[j].w, h.w));
        }
        store4<TO>(xn + (size_t)m * N + 4 * (size_t)i, h);
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
    if (E > LNT_PER * 1024) return fail(HFB_ENOTSUP, "layernorm_shift: rows of %d values exceed %d", E, LNT_PER * 1024);
    int threads = ((E + 7) / 8 + 31) / 32 * 32;           // eight values a thread for rows of up to 4,096, sixteen beyond
    const bool few = threads <= 512;
    if (!few) threads = ((E + 15) / 16 + 31) / 32 * 32;
#define HFB_LNS(TY, PER) \
    g_launch_err = launch_pdl(layernorm_shift_kernel<TY, PER>, dim3(T), dim3(threads), 0, (cudaStream_t)s, x, w, mu, eps, center, state, \
                              (size_t)slot_stride, token_seq, cu_tokens, seq_slots, n_slots, (TY *)out, T, E, error_word())
    if (out_dt == HFB_F32) { if (few) HFB_LNS(float, 8); else HFB_LNS(float, LNT_PER); }
    else { if (few) HFB_LNS(__nv_bfloat16, 8); else HFB_LNS(__nv_bfloat16, LNT_PER); }
#undef HFB_LNS
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
    auto aligned = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    // steps of few rows (their cost is latency) take the form with 16-byte accesses and everything requested up front;
    // passes over thousands of rows run faster with eight values a thread and half as many threads
    if (M <= 1024 && (N & 3) == 0 && N <= 16 * 1024 && aligned(partial) && aligned(residual) && aligned(w) && aligned(mu) && aligned(state) &&
        aligned(xn) && (slot_stride & 3) == 0) {
        // 16-byte accesses: one float4 a thread up to 4,096 values (a warp at least), then two, then four
        const int N4 = N >> 2, pv = N4 <= 1024 ? 1 : (N4 <= 2048 ? 2 : 4);
        int threads = ((N4 + pv - 1) / pv + 31) / 32 * 32;
#define HFB_LNV(TY, PV) \
    g_launch_err = launch_pdl(reduce_residual_layernorm_vec_kernel<TY, PV>, dim3(M), dim3(threads), 0, (cudaStream_t)s, partial, splits, M, N, \
                              bias, bias_dt, residual, w, eps, center, mu, state, (size_t)slot_stride, seq_slots, n_slots, (TY *)xn, error_word())
        if (xn_dt == HFB_F32 || !xn) { if (pv == 1) HFB_LNV(float, 1); else if (pv == 2) HFB_LNV(float, 2); else HFB_LNV(float, 4); }
        else { if (pv == 1) HFB_LNV(__nv_bfloat16, 1); else if (pv == 2) HFB_LNV(__nv_bfloat16, 2); else HFB_LNV(__nv_bfloat16, 4); }
#undef HFB_LNV
        return check_pdl_launch(g_launch_err, "reduce_residual_layernorm");
    }
    int threads = ((N + 7) / 8 + 31) / 32 * 32;           // eight values a thread where the row allows
    if (threads > 1024) threads = 1024;
#define HFB_LNT(TY, PER) \
    g_launch_err = launch_pdl(reduce_residual_layernorm_kernel<TY, PER>, dim3(M), dim3(threads), 0, (cudaStream_t)s, partial, splits, M, N, bias, \
                              bias_dt, residual, w, eps, center, mu, state, (size_t)slot_stride, seq_slots, n_slots, (TY *)xn, error_word())
    const bool few = N <= 8 * threads;                     // rows of up to 8,192 values: eight a thread, all in registers
    if (xn_dt == HFB_F32 || !xn) { if (few) HFB_LNT(float, 8); else HFB_LNT(float, LNT_PER); }
    else { if (few) HFB_LNT(__nv_bfloat16, 8); else HFB_LNT(__nv_bfloat16, LNT_PER); }
#undef HFB_LNT
    return check_pdl_launch(g_launch_err, "reduce_residual_layernorm");
}
