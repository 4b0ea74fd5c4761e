// Hyper-connections: the residual stream kept in S copies x[t, s, :] (float32, [T, S, E]).  A sublayer reads one
// mixture of them, u = sum_s in[s] x_s, and its output y, scaled per feature, is written back into every copy while
// the copies are mixed among themselves:  x'_t = sum_s mix[s, t] x_s + out[t] * (scale .* y), all t from the old copies.
//
// Three kernels: the copies made from the embedding; the mixture (of all or of chosen rows) with the Dynamic Tanh norm
// tanh(alpha u) w + b behind it (weights in == NULL: the plain sum, which is what the model's head reads); and the
// update, which sums the sublayer's output from its pieces in a fixed order (the split-K partial sums of up to two
// products, each with a factor, and the weighted sum of a routed feed-forward's chosen experts, where a choice beyond
// the real experts stands for the sublayer's input itself), writes the new copies, and hands out the next sublayer's
// normed mixture of them from the same pass.  All arithmetic in float32.
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {

constexpr int HC_MAX = 8;          // copies of the stream

struct HcNorm { const void *alpha, *w, *b; int dt; };

__device__ __forceinline__ float hc_norm_one(const HcNorm &p, float alpha, float x, int c)
{
    return tanhf(alpha * x) * load_any(p.w, p.dt, c) + load_any(p.b, p.dt, c);
}

__global__ void hc_spread_kernel(const float *emb, float *x, int S, int T, int E)
{
    pdl_entry();
    pdl_sync_small();
    const size_t total = (size_t)T * E;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / E;
        const int c = (int)(i % E);
        const float v = emb[i];
        for (int s = 0; s < S; s++) x[(t * S + s) * E + c] = v;
    }
}

// out[m, c] = norm(sum_s in_w[s] * x[row(m), s, c]); without a norm the sum itself (float32 or the run's type)
__global__ void hc_in_norm_kernel(const float *x, int S, const float *in_w, const int32_t *rows, int has_norm, HcNorm p,
                                  void *out, int out_dt, int M, int E)
{
    pdl_entry();
    pdl_sync_small();
    const float alpha = has_norm ? load_any(p.alpha, p.dt, 0) : 0.f;
    float w[HC_MAX];
#pragma unroll
    for (int s = 0; s < HC_MAX; s++) w[s] = s < S ? (in_w ? in_w[s] : 1.0f) : 0.f;
    const size_t total = (size_t)M * E;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / E), c = (int)(i % E);
        const float *src = x + ((size_t)(rows ? rows[m] : m) * S) * E + c;
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < HC_MAX; s++)
            if (s < S) u = fmaf(w[s], src[(size_t)s * E], u);
        store_any(out, out_dt, i, has_norm ? hc_norm_one(p, alpha, u, c) : u);
    }
}

struct HcSource { const float *y; int splits; float factor; };

struct HcMix {
    const float *y;             // [T * top, E] outputs of the chosen experts
    const float *w;             // [T, top]
    const int32_t *ids;         // [T, top] or NULL; ids >= n_real: the choice's output is the sublayer's input
    const void *h;              // [T, E] the sublayer's input
    int h_dt, top, n_real;
};

__global__ void hc_update_kernel(float *x, int S, HcSource a, HcSource b, HcMix mix, const void *scale, int scale_dt,
                                 const float *mix_w, const float *out_w, const float *next_in, int has_norm, HcNorm next,
                                 void *out, int out_dt, int T, int E)
{
    pdl_entry();
    pdl_sync_small();
    __shared__ float s_mix[HC_MAX * HC_MAX], s_out[HC_MAX], s_in[HC_MAX];
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = mix_w[i];
    if (threadIdx.x < S) {
        s_out[threadIdx.x] = out_w[threadIdx.x];
        s_in[threadIdx.x] = next_in ? next_in[threadIdx.x] : 1.0f;
    }
    __syncthreads();
    const float alpha = has_norm ? load_any(next.alpha, next.dt, 0) : 0.f;
    const size_t total = (size_t)T * E;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / E;
        const int c = (int)(i % E);
        float y = 0.f;
        if (a.y) {
            float v = 0.f;
            for (int s = 0; s < a.splits; s++) v += a.y[(size_t)s * total + i];
            y = a.factor * v;
        }
        if (b.y) {
            float v = 0.f;
            for (int s = 0; s < b.splits; s++) v += b.y[(size_t)s * total + i];
            y = fmaf(b.factor, v, y);
        }
        if (mix.w) {
            float acc = 0.f;
            for (int j = 0; j < mix.top; j++) {
                const size_t pj = t * mix.top + j;
                const float v = (mix.ids && mix.ids[pj] >= mix.n_real) ? load_any(mix.h, mix.h_dt, i) : mix.y[pj * E + c];
                acc = fmaf(mix.w[pj], v, acc);
            }
            y += acc;
        }
        if (scale) y *= load_any(scale, scale_dt, c);
        float *xs = x + t * S * E + c;
        float old[HC_MAX];
#pragma unroll
        for (int s = 0; s < HC_MAX; s++) old[s] = s < S ? xs[(size_t)s * E] : 0.f;
        float u = 0.f;
#pragma unroll
        for (int d = 0; d < HC_MAX; d++) {
            if (d < S) {
                float v = 0.f;
#pragma unroll
                for (int s = 0; s < HC_MAX; s++)
                    if (s < S) v = fmaf(s_mix[s * S + d], old[s], v);
                v = fmaf(s_out[d], y, v);
                xs[(size_t)d * E] = v;
                u = fmaf(s_in[d], v, u);
            }
        }
        if (out) store_any(out, out_dt, i, has_norm ? hc_norm_one(next, alpha, u, c) : u);
    }
}

static unsigned hc_blocks(size_t total)
{
    size_t b = (total + 255) / 256;
    return (unsigned)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_hc_spread(const float *emb, float *x, int S, int T, int E, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!emb || !x || S < 1 || S > HC_MAX || E <= 0) return fail(HFB_EINVAL, "hc_spread: bad arguments (streams=%d)", S);
    g_launch_err = launch_pdl(hc_spread_kernel, dim3(hc_blocks((size_t)T * E)), dim3(256), 0, (cudaStream_t)s, emb, x, S, T, E);
    return check_pdl_launch(g_launch_err, "hc_spread");
}

extern "C" int hfb_hc_in_norm(const float *x, int S, const float *in_w, const int32_t *rows, const void *alpha, const void *w,
                              const void *b, int p_dt, void *out, int out_dt, int M, int E, hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    const int has_norm = alpha != nullptr;
    if (!x || !out || S < 1 || S > HC_MAX || E <= 0 || !valid_dt(out_dt) || (has_norm && (!w || !b || !valid_dt(p_dt))))
        return fail(HFB_EINVAL, "hc_in_norm: bad arguments (streams=%d)", S);
    HcNorm p{alpha, w, b, p_dt};
    g_launch_err = launch_pdl(hc_in_norm_kernel, dim3(hc_blocks((size_t)M * E)), dim3(256), 0, (cudaStream_t)s, x, S, in_w, rows, has_norm, p, out, out_dt, M, E);
    return check_pdl_launch(g_launch_err, "hc_in_norm");
}

extern "C" int hfb_hc_update(float *x, int S, const float *ya, int splits_a, float factor_a, const float *yb, int splits_b,
                             float factor_b, const float *mix_y, const float *mix_w, const int32_t *mix_ids, int top, int n_real,
                             const void *mix_h, int mix_h_dt, const void *scale, int scale_dt, const float *hc_mix,
                             const float *hc_out, const float *next_in, const void *alpha, const void *w, const void *b,
                             int p_dt, void *out, int out_dt, int T, int E, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    const int has_norm = alpha != nullptr;
    if (!x || S < 1 || S > HC_MAX || E <= 0 || !hc_mix || !hc_out || (ya && splits_a < 1) || (yb && splits_b < 1) ||
        (!ya && !yb && !mix_w) || (mix_w && (!mix_y || top < 1)) || (mix_ids && (!mix_h || !valid_dt(mix_h_dt))) ||
        (scale && !valid_dt(scale_dt)) || (out && !valid_dt(out_dt)) || (has_norm && (!out || !w || !b || !valid_dt(p_dt))))
        return fail(HFB_EINVAL, "hc_update: bad arguments (streams=%d)", S);
    HcSource a{ya, splits_a, factor_a}, bb{yb, splits_b, factor_b};
    HcMix mix{mix_y, mix_w, mix_ids, mix_h, mix_h_dt, top, n_real};
    HcNorm p{alpha, w, b, p_dt};
    g_launch_err = launch_pdl(hc_update_kernel, dim3(hc_blocks((size_t)T * E)), dim3(256), 0, (cudaStream_t)s, x, S, a, bb, mix, scale, scale_dt,
                              hc_mix, hc_out, next_in, has_norm, p, out, out_dt, T, E);
    return check_pdl_launch(g_launch_err, "hc_update");
}
