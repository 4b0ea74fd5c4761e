// Mixers that carry a matrix of fixed size per request and head instead of keys and values per token: the gated
// linear recurrence
//     S <- diag(a_t) S + k_t u_t^T,   o_t = S^T q_t,   u_t = v_t                         (gated linear attention)
//                                                     u_t = beta_t (v_t - (diag(a_t) S)^T k_t)   (gated delta rule)
// with S [d, dv] per head (the decay a_t acts on the rows, which belong to key channels), and what stands around it:
// the decays from their logits, the short causal convolution over time with its carried inputs, unit-length queries
// and keys, and the heads' root-mean-square norm with its gate.  The state, the decays and every sum are float32; the
// state of a request lives in its slot between steps, so a step continues exactly where the last one stopped and a
// token's result does not depend on how the request was cut into steps nor on what else a step holds.
//
// Layout of a head's state in a slot: [dv][d], a column of S (one value channel) contiguous.  Columns are independent
// of each other in both forms of the recurrence, so the work is spread over (request, head, column) and only the walk
// along a request's tokens is sequential.
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();

constexpr int CONV_MAX_TAPS = 16;
constexpr int REC_WARPS = 4;
constexpr int REC_MAX_D = 512;

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
// the same from the special-function unit's exponential and reciprocal: relative error of a few 1e-7
__device__ __forceinline__ float sigmoid_fast(float z) { return __fdividef(1.0f, 1.0f + __expf(-z)); }

// a[t, h, i] = exp(-rate[h] * softplus(sign * (z[t, h, i] + bias[h, i]))), z the sum of `splits` planes [T, z_stride] read
// from column z_col0 on.  sign = +1 with rate = exp(A_log): exp(-exp(A_log) softplus(z + dt_bias)); sign = -1 with rate
// = 1 / tau: sigmoid(z + bias)^(1 / tau).
__global__ void decay_kernel(const float *z, int splits, int z_stride, int z_col0, const void *bias, int bias_dt,
                             const float *rate, float sign, float *out, int T, int H, int d)
{
    pdl_entry();
    pdl_sync_small();
    const size_t row = (size_t)H * d, total = (size_t)T * row, plane = (size_t)T * z_stride;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % row);
        const float *zp = z + (i / row) * z_stride + z_col0 + c;
        float v = 0.f;
        for (int s = 0; s < splits; s++) v += zp[(size_t)s * plane];
        if (bias) v += load_any(bias, bias_dt, c);
        out[i] = expf(-rate[c / d] * softplus_f(sign * v));
    }
}

// Short causal convolution over time, per channel, then silu; the heads of the first `n_unit` units are then brought
// to unit length, x / sqrt(sum(x^2) + unit_eps), and those of the first `n_scaled` also multiplied by `scale`.  A row of
// x is a list of units (heads): `n_a` units of `d_a` channels followed by `n_b` units of `d_b`.  One warp per (token,
// unit).  Inputs before a request's first token of this step come from its slot, carried [taps - 1][C] oldest first
// (zeros for a new request).  w [C, taps], the last column is the current token's.
__global__ void __launch_bounds__(REC_WARPS * 32)
short_conv_kernel(const float *x, int splits, const void *w, int w_dt, int taps, const float *carried, size_t slot_stride,
                  const int32_t *token_seq, const int32_t *cu_tokens, const int32_t *seq_slots, int n_slots, float *out,
                  int T, int n_a, int d_a, int n_b, int d_b, int n_unit, int n_scaled, float scale, float unit_eps, int *err)
{
    pdl_entry();
    pdl_sync_small();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x, u = blockIdx.y * REC_WARPS + warp;
    if (u >= n_a + n_b) return;
    const int C = n_a * d_a + n_b * d_b;
    const int col0 = u < n_a ? u * d_a : n_a * d_a + (u - n_a) * d_b;
    const int n = u < n_a ? d_a : d_b;
    const int seq = token_seq[t];
    const int t0 = cu_tokens[seq];
    const int slot = seq_slots[seq];
    if (slot < 0 || slot >= n_slots) { if (lane == 0) atomicOr(err, HFB_ERR_SLOT); return; }
    const float *old = carried + (size_t)slot * slot_stride;
    const size_t plane = (size_t)T * C;
    const int K = taps - 1;
    float ss = 0.f;
    for (int c = lane; c < n; c += 32) {
        const int ch = col0 + c;
        float acc = 0.f;
        for (int i = 0; i < taps; i++) {
            const int tt = t - K + i;                        // the input i - K tokens back
            float v = 0.f;
            if (tt >= t0) {
                for (int s = 0; s < splits; s++) v += x[(size_t)s * plane + (size_t)tt * C + ch];
            } else {
                v = old[(size_t)(tt - t0 + K) * C + ch];
            }
            acc = fmaf(load_any(w, w_dt, (size_t)ch * taps + i), v, acc);
        }
        const float y = acc * sigmoid_f(acc);
        out[(size_t)t * C + ch] = y;
        ss = fmaf(y, y, ss);
    }
    if (u < n_unit) {
        ss = warp_sum(ss);
        float r = 1.0f / sqrtf(ss + unit_eps);
        if (u < n_scaled) r *= scale;
        __syncwarp();
        for (int c = lane; c < n; c += 32) out[(size_t)t * C + col0 + c] *= r;
    }
}

// The convolution's carried inputs after a step: the last taps - 1 inputs of each request, from this step's rows and,
// where the step brought fewer, from what was carried before.  One thread per (request, channel) reads all it needs
// before it writes.
__global__ void conv_carry_kernel(const float *x, int splits, int taps, float *carried, size_t slot_stride,
                                  const int32_t *cu_tokens, const int32_t *seq_slots, int n_slots, int S, int T, int C)
{
    pdl_entry();
    pdl_sync_small();
    const int K = taps - 1;
    const size_t plane = (size_t)T * C;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)S * C; i += (size_t)gridDim.x * blockDim.x) {
        const int seq = (int)(i / C), ch = (int)(i % C);
        const int slot = seq_slots[seq];
        if (slot < 0 || slot >= n_slots) continue;
        const int t0 = cu_tokens[seq], n = cu_tokens[seq + 1] - t0;
        float *st = carried + (size_t)slot * slot_stride;
        float keep[CONV_MAX_TAPS];
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; j++) {
            if (j < K) {
                const int rel = n - K + j;                   // relative to the step's first token of the request
                float v = 0.f;
                if (rel >= 0) { for (int s = 0; s < splits; s++) v += x[(size_t)s * plane + (size_t)(t0 + rel) * C + ch]; }
                else v = st[(size_t)(rel + K) * C + ch];
                keep[j] = v;
            }
        }
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; j++)
            if (j < K) st[(size_t)j * C + ch] = keep[j];
    }
}

// The recurrence.  Block = (request, head, slice of value channels); L lanes share a column of S, each holding R of its
// d entries in registers (entry i of the column sits in lane i / R).  q and k rows are [Hq heads of d] (head h reads head
// h / (H / Hq)), a (the decays) [H heads of d], v and o [H heads of dv]; every row pointer comes with its own stride so
// that the operands may be slices of wider product outputs.  beta_logit [T, beta_stride]: u = sigmoid(beta_logit) (v -
// S^T k); NULL: u = v.
//
// The walk along the tokens is a chain of dependent steps, so what a step waits for decides the kernel's speed: the
// operands of `ct` tokens at a time (the head's q, k and a rows, the block's slice of v, beta) come into shared memory by
// cp.async, two chunks deep, and a step reads them from there instead of from global memory.  A row of d values lies in
// shared memory as L groups of R with 4 floats between the groups, so that the lanes of a column read their 16-byte
// pieces from different banks.  Only the state's update is a chain from token to token; a lane's piece of o = S^T q
// goes to shared memory as it is, and the pieces of a chunk's tokens are summed (in lane order) and stored when the
// chunk is done.
__device__ __forceinline__ void cp_async4(float *dst, const float *src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int R, int L>
__global__ void __launch_bounds__(256)
linear_scan_kernel(const float *q, int q_stride, const float *k, int k_stride, const float *v, int v_stride,
                   const float *a, int a_stride, const float *beta_logit, int beta_stride, float q_scale, float *state,
                   size_t slot_stride, const int32_t *cu_tokens, const int32_t *seq_slots, int n_slots, float *o,
                   int o_stride, int H, int Hq, int d, int dv, int ct, int *err)
{
    pdl_wait();                                      // (a long kernel: its successor is released when the walk is done)
    extern __shared__ float4 scan_smem4[];
    float *smem = (float *)scan_smem4;
    constexpr int COLS = 256 / L, RS = L * (R + 4);              // columns of a block; floats of a padded row
    const int stage_floats = (ct * (3 * RS + COLS + 1) + 3) & ~3;
    float *ob = smem + 2 * stage_floats;                         // [ct][256]: every lane's piece of o
    const int seq = blockIdx.x, h = blockIdx.y;
    const int lcol = threadIdx.x / L, col = blockIdx.z * COLS + lcol, part = threadIdx.x % L;
    const int slot = seq_slots[seq];
    if (slot < 0 || slot >= n_slots) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); return; }
    const int t0 = cu_tokens[seq], t1 = cu_tokens[seq + 1];
    const bool live = col < dv;                                  // (lanes beyond the last column follow along on column 0)
    const int cj = live ? col : 0;
    const int hq = h / (H / Hq);
    const int i0 = part * R;
    float *sp = state + (size_t)slot * slot_stride + ((size_t)h * dv + cj) * d + i0;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; r++) S[r] = (i0 + r < d) ? sp[r] : 0.f;
    bool in[R];
#pragma unroll
    for (int r = 0; r < R; r++) in[r] = i0 + r < d;

    auto issue = [&](int c) {
        float *st = smem + (c & 1) * stage_floats;
        const int tb = t0 + c * ct, n = min(ct, t1 - tb);
        for (int idx = threadIdx.x; idx < n * d; idx += 256) {
            const int tt = idx / d, i = idx - tt * d;
            float *dst = st + tt * RS + (i / R) * (R + 4) + i % R;
            cp_async4(dst, q + (size_t)(tb + tt) * q_stride + hq * d + i);
            cp_async4(dst + ct * RS, k + (size_t)(tb + tt) * k_stride + hq * d + i);
            cp_async4(dst + 2 * ct * RS, a + (size_t)(tb + tt) * a_stride + h * d + i);
        }
        float *sv = st + 3 * ct * RS;
        for (int idx = threadIdx.x; idx < n * COLS; idx += 256) {
            const int tt = idx / COLS, c_ = idx % COLS, gc = blockIdx.z * COLS + c_;
            cp_async4(sv + idx, v + (size_t)(tb + tt) * v_stride + h * dv + (gc < dv ? gc : 0));
        }
        if (beta_logit)
            for (int idx = threadIdx.x; idx < n; idx += 256) cp_async4(sv + ct * COLS + idx, beta_logit + (size_t)(tb + idx) * beta_stride + h);
        cp_async_commit();
    };

    const int n_chunks = (t1 - t0 + ct - 1) / ct;
    if (n_chunks > 0) issue(0);
    for (int c = 0; c < n_chunks; c++) {
        if (c + 1 < n_chunks) { issue(c + 1); cp_async_wait<1>(); } else cp_async_wait<0>();
        __syncthreads();
        const float *st = smem + (c & 1) * stage_floats;
        const int tb = t0 + c * ct, n = min(ct, t1 - tb);
#pragma unroll 2
        for (int tt = 0; tt < n; tt++) {
            float qa[R], ka[R], aa[R];
            const float4 *rq = (const float4 *)(st + tt * RS + part * (R + 4));
            const float4 *rk = (const float4 *)(st + (ct + tt) * RS + part * (R + 4));
            const float4 *ra = (const float4 *)(st + (2 * ct + tt) * RS + part * (R + 4));
#pragma unroll
            for (int r4 = 0; r4 < R / 4; r4++) {
                const float4 x = rq[r4], y = rk[r4], z = ra[r4];
                qa[4 * r4] = x.x; qa[4 * r4 + 1] = x.y; qa[4 * r4 + 2] = x.z; qa[4 * r4 + 3] = x.w;
                ka[4 * r4] = y.x; ka[4 * r4 + 1] = y.y; ka[4 * r4 + 2] = y.z; ka[4 * r4 + 3] = y.w;
                aa[4 * r4] = z.x; aa[4 * r4 + 1] = z.y; aa[4 * r4 + 2] = z.z; aa[4 * r4 + 3] = z.w;
            }
#pragma unroll
            for (int r = 0; r < R; r++) {                         // beyond d the shared memory holds nothing
                qa[r] = in[r] ? qa[r] : 0.f; ka[r] = in[r] ? ka[r] : 0.f; aa[r] = in[r] ? aa[r] : 0.f;
            }
            const float vt = st[3 * ct * RS + tt * COLS + lcol];
            float u = vt;
            if (beta_logit) {
                const float gate = sigmoid_f(st[3 * ct * RS + ct * COLS + tt]);
                float dot4[4] = {0.f, 0.f, 0.f, 0.f};                // four chains, summed in a fixed order
#pragma unroll
                for (int r = 0; r < R; r++) { S[r] *= aa[r]; dot4[r & 3] = fmaf(S[r], ka[r], dot4[r & 3]); }
                float dot = (dot4[0] + dot4[1]) + (dot4[2] + dot4[3]);
#pragma unroll
                for (int m = L / 2; m > 0; m >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, m);
                u = gate * (vt - dot);
#pragma unroll
                for (int r = 0; r < R; r++) S[r] = fmaf(ka[r], u, S[r]);
            } else {
#pragma unroll
                for (int r = 0; r < R; r++) S[r] = fmaf(aa[r], S[r], ka[r] * u);
            }
            float acc4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < R; r++) acc4[r & 3] = fmaf(S[r], qa[r], acc4[r & 3]);
            ob[tt * 256 + threadIdx.x] = (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]);
        }
        __syncthreads();                                         // the stage is free for the chunk after the next
        for (int idx = threadIdx.x; idx < n * COLS; idx += 256) {
            const int tt = idx / COLS, c_ = idx % COLS, gc = blockIdx.z * COLS + c_;
            float acc = 0.f;
#pragma unroll
            for (int l = 0; l < L; l++) acc += ob[tt * 256 + c_ * L + l];
            if (gc < dv) o[(size_t)(tb + tt) * o_stride + h * dv + gc] = acc * q_scale;
        }
    }
    pdl_trigger();
    if (live) {
#pragma unroll
        for (int r = 0; r < R; r++)
            if (i0 + r < d) sp[r] = S[r];
    }
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * w * gate(g[t, h, :]); gate 0: silu, 1: sigmoid.  g is the sum of
// `g_splits` planes [T, g_stride] (float32) read from column g_col0 on.  One warp per (token, head).
template <typename TO>
__global__ void __launch_bounds__(REC_WARPS * 32)
gate_norm_kernel(const float *o, const void *w, int w_dt, float eps, const float *g, int g_splits, int g_stride, int g_col0,
                 int gate, TO *out, int T, int H, int dv)
{
    pdl_entry();
    pdl_sync_small();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x, h = blockIdx.y * REC_WARPS + warp;
    if (h >= H) return;
    const float *x = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(x[c], x[c], ss);
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)dv + eps);
    const size_t plane = (size_t)T * g_stride;
    for (int c = lane; c < dv; c += 32) {
        float z = 0.f;
        const float *gp = g + (size_t)t * g_stride + g_col0 + h * dv + c;
        for (int s = 0; s < g_splits; s++) z += gp[(size_t)s * plane];
        const float gv = gate == 0 ? z * sigmoid_f(z) : sigmoid_f(z);
        out[((size_t)t * H + h) * dv + c] = from_f32<TO>(x[c] * r * load_any(w, w_dt, c) * gv);
    }
}

static unsigned rec_blocks(size_t total)
{
    size_t b = (total + 255) / 256;
    return (unsigned)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}


// minGRU: a gated recurrence per channel whose gates read the current token only.  With a = row[.., c] (update gate's
// sum), b = row[.., W + c] (candidate's sum), g = row[.., 2 W + c] (output gate's sum), each the sum of `splits` float32
// planes [T, 3 W], and biases on the first two:
//     z = sigmoid(a + bz);  u = b + bx;  cand = u >= 0 ? u + 1/2 : sigmoid(u);  S <- (1 - z) S + z cand;
//     out = S * silu(g)
// S [W] float32 per request lives in its state slot.  A block takes MG_CH channels of one request.  Its fill warps
// compute, for a chunk of MG_CT tokens, everything that does not depend on S (1 - z, z * cand, silu(g): three
// exponentials a token and channel) into shared memory, in parallel over tokens, from operands they requested one chunk
// earlier (MG_PER tokens a thread, all of a chunk's reads in flight together: their latency is what a chunk would
// cost); meanwhile the first warp walks the chunk before, one channel a lane, a multiply-add a token.  The walk is the
// same sequence of operations whatever the step's cutting, so a position's result does not depend on it.
constexpr int MG_CH = 32, MG_FILL = 8, MG_PER = 8, MG_CT = MG_FILL * MG_PER;

template <typename TO>
__global__ void __launch_bounds__((MG_FILL + 1) * 32)
mingru_scan_kernel(const float *row, int splits, const void *bz, const void *bx, int b_dt, float *state, size_t slot_stride,
                   const int32_t *cu_tokens, const int32_t *seq_slots, int n_slots, TO *out, int T, int W, int *err)
{
    pdl_entry();
    pdl_sync_small();
    __shared__ float s_a[2][MG_CT][MG_CH], s_b[2][MG_CT][MG_CH], s_g[2][MG_CT][MG_CH];
    const int seq = blockIdx.y, c0 = blockIdx.x * MG_CH;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = c0 + lane;
    const bool live = c < W;
    const int slot = seq_slots[seq];
    if (slot < 0 || slot >= n_slots) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); return; }
    const int t0 = cu_tokens[seq], n = cu_tokens[seq + 1] - t0;
    const size_t C3 = 3 * (size_t)W, plane = (size_t)T * C3;
    const int chunks = (n + MG_CT - 1) / MG_CT;
    const int fw = warp - 1;                           // which of the fill warps (the first warp walks)
    const float vbz = (live && bz) ? load_any(bz, b_dt, c) : 0.f, vbx = (live && bx) ? load_any(bx, b_dt, c) : 0.f;
    // two chunks' operands on their way: tokens fw, fw + MG_FILL, ... of the chunk after next are requested before the
    // next chunk's are used, so a read has a whole round (a walk and a fill) to arrive
    float ra[2][MG_PER], rb[2][MG_PER], rg[2][MG_PER];

    auto request = [&](int k, float *qa, float *qb, float *qg) {
        // the first split's values are taken as they are: a register that is only loaded does not hold its thread up
        // until it is used, so the reads of a product that is not split stay in flight behind this call
#pragma unroll
        for (int u = 0; u < MG_PER; u++) {
            const int i = k * MG_CT + fw + u * MG_FILL;
            const bool ok = i < n && live;
            const float *p = row + (size_t)(t0 + (ok ? i : 0)) * C3 + (live ? c : 0);
            qa[u] = ok ? p[0] : 0.f; qb[u] = ok ? p[W] : 0.f; qg[u] = ok ? p[2 * (size_t)W] : 0.f;
        }
        for (int s = 1; s < splits; s++) {
#pragma unroll
            for (int u = 0; u < MG_PER; u++) {
                const int i = k * MG_CT + fw + u * MG_FILL;
                if (i < n && live) {
                    const float *p = row + (size_t)s * plane + (size_t)(t0 + i) * C3 + c;
                    qa[u] += p[0]; qb[u] += p[W]; qg[u] += p[2 * (size_t)W];
                }
            }
        }
    };
    auto finish = [&](int k, const float *qa, const float *qb, const float *qg) {
        const int buf = k & 1;
#pragma unroll
        for (int u = 0; u < MG_PER; u++) {
            const int j = fw + u * MG_FILL;
            const float z = sigmoid_fast(qa[u] + vbz), v = qb[u] + vbx, g = qg[u];
            const float cand = v >= 0.f ? v + 0.5f : sigmoid_fast(v);
            s_a[buf][j][lane] = 1.0f - z;
            s_b[buf][j][lane] = z * cand;
            s_g[buf][j][lane] = g * sigmoid_fast(g);
        }
    };

    float S = 0.f;
    if (warp == 0) {
        if (live) S = state[(size_t)slot * slot_stride + c];
    } else {
        request(0, ra[0], rb[0], rg[0]);
        if (chunks > 1) request(1, ra[1], rb[1], rg[1]);
        finish(0, ra[0], rb[0], rg[0]);
        if (chunks > 2) request(2, ra[0], rb[0], rg[0]);
    }
    __syncthreads();
    // (the loop is unrolled by two so that the register sets are named at compile time)
    for (int k = 0; k < chunks; k += 2) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int kk = k + h;
            if (kk < chunks) {
                if (warp == 0) {
                    const int buf = kk & 1, m = min(MG_CT, n - kk * MG_CT);
                    if (live) {
                        TO *o = out + (size_t)(t0 + kk * MG_CT) * W + c;
#pragma unroll 4
                        for (int j = 0; j < m; j++) {
                            S = fmaf(s_a[buf][j][lane], S, s_b[buf][j][lane]);
                            o[(size_t)j * W] = from_f32<TO>(S * s_g[buf][j][lane]);
                        }
                    }
                } else if (kk + 1 < chunks) {
                    // chunk kk + 1 sits in set (kk + 1) & 1 = 1 - h; once used, that set takes chunk kk + 3
                    finish(kk + 1, ra[1 - h], rb[1 - h], rg[1 - h]);
                    if (kk + 3 < chunks) request(kk + 3, ra[1 - h], rb[1 - h], rg[1 - h]);
                }
            }
            __syncthreads();
        }
    }
    if (warp == 0 && live) state[(size_t)slot * slot_stride + c] = S;
}


// The same for a step in which every request brings one token (row s is request s): one thread per (request, channel),
// nothing to walk along.  The operations on S are those of the kernel above, in the same order.
template <typename TO>
__global__ void mingru_step_kernel(const float *row, int splits, const void *bz, const void *bx, int b_dt, float *state,
                                   size_t slot_stride, const int32_t *seq_slots, int n_slots, TO *out, int T, int W, int *err)
{
    pdl_entry();
    pdl_sync_small();
    const size_t C3 = 3 * (size_t)W, plane = (size_t)T * C3;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)T * W; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / W), c = (int)(i % W);
        const int slot = seq_slots[t];
        if (slot < 0 || slot >= n_slots) { atomicOr(err, HFB_ERR_SLOT); continue; }
        const float *p = row + (size_t)t * C3 + c;
        float a = p[0], b = p[W], g = p[2 * (size_t)W];
        for (int s = 1; s < splits; s++) {
            a += p[(size_t)s * plane]; b += p[(size_t)s * plane + W]; g += p[(size_t)s * plane + 2 * (size_t)W];
        }
        float *st = state + (size_t)slot * slot_stride + c;
        const float z = sigmoid_fast(a + (bz ? load_any(bz, b_dt, c) : 0.f)), v = b + (bx ? load_any(bx, b_dt, c) : 0.f);
        const float cand = v >= 0.f ? v + 0.5f : sigmoid_fast(v);
        const float S = fmaf(1.0f - z, *st, z * cand);
        *st = S;
        out[i] = from_f32<TO>(S * (g * sigmoid_fast(g)));
    }
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_decay(const float *z, int splits, int z_stride, int z_col0, const void *bias, int bias_dt, const float *rate,
                         float sign, float *out, int T, int H, int d, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!z || !rate || !out || splits < 1 || H <= 0 || d <= 0 || (bias && !valid_dt(bias_dt)) || z_col0 < 0 || z_col0 + H * d > z_stride)
        return fail(HFB_EINVAL, "decay: bad arguments (H=%d d=%d)", H, d);
    g_launch_err = launch_pdl(decay_kernel, dim3(rec_blocks((size_t)T * H * d)), dim3(256), 0, (cudaStream_t)s, z, splits, z_stride, z_col0,
                              bias, bias_dt, rate, sign, out, T, H, d);
    return check_pdl_launch(g_launch_err, "decay");
}

extern "C" int hfb_short_conv(const float *x, int splits, const void *w, int w_dt, int taps, float *carried, int64_t slot_stride,
                              const int32_t *token_seq, const int32_t *cu_tokens, const int32_t *seq_slots, int n_slots, int S,
                              float *out, int T, int n_a, int d_a, int n_b, int d_b, int n_unit, int n_scaled, float scale,
                              float unit_eps, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!x || !w || !carried || !out || !valid_dt(w_dt) || splits < 1 || taps < 1 || n_a < 0 || n_b < 0 || n_a + n_b < 1 ||
        d_a <= 0 || d_b <= 0 || S < 1)
        return fail(HFB_EINVAL, "short_conv: bad arguments (taps=%d)", taps);
    if (taps > CONV_MAX_TAPS) return fail(HFB_ENOTSUP, "short_conv: %d taps exceed %d", taps, CONV_MAX_TAPS);
    const int unit_blocks = (n_a + n_b + REC_WARPS - 1) / REC_WARPS;
    if (unit_blocks > 65535) return fail(HFB_ENOTSUP, "short_conv: %d heads exceed the grid limit", n_a + n_b);
    g_launch_err = launch_pdl(short_conv_kernel, dim3(T, unit_blocks), dim3(REC_WARPS * 32), 0, (cudaStream_t)s, x, splits, w, w_dt, taps,
                              (const float *)carried, (size_t)slot_stride, token_seq, cu_tokens, seq_slots, n_slots, out, T, n_a, d_a,
                              n_b, d_b, n_unit, n_scaled, scale, unit_eps, error_word());
    int rc = check_pdl_launch(g_launch_err, "short_conv");
    if (rc != HFB_OK || taps == 1) return rc;
    const int C = n_a * d_a + n_b * d_b;
    g_launch_err = launch_pdl(conv_carry_kernel, dim3(rec_blocks((size_t)S * C)), dim3(256), 0, (cudaStream_t)s, x, splits, taps, carried,
                              (size_t)slot_stride, cu_tokens, seq_slots, n_slots, S, T, C);
    return check_pdl_launch(g_launch_err, "conv_carry");
}

extern "C" int hfb_linear_scan(const float *q, int q_stride, const float *k, int k_stride, const float *v, int v_stride,
                               const float *a, int a_stride, const float *beta_logit, int beta_stride, float q_scale,
                               float *state, int64_t slot_stride, const int32_t *cu_tokens, const int32_t *seq_slots,
                               int n_slots, int S, float *o, int o_stride, int H, int Hq, int d, int dv, hfb_stream s)
{
    if (S <= 0) return HFB_OK;
    if (!q || !k || !v || !a || !state || !o || H <= 0 || Hq <= 0 || H % Hq || d <= 0 || dv <= 0)
        return fail(HFB_EINVAL, "linear_scan: bad arguments (H=%d Hq=%d d=%d dv=%d)", H, Hq, d, dv);
    if (d > REC_MAX_D) return fail(HFB_ENOTSUP, "linear_scan: key heads above %d are not supported", REC_MAX_D);
    if (H > 65535) return fail(HFB_ENOTSUP, "linear_scan: %d heads exceed the grid limit", H);
    // tokens per chunk: two stages of ct * (3 padded rows + the columns' values + beta) floats and the lanes' pieces of o
    // (ct * 256 floats) within 46 KB, 16 at most
#define HFB_SCAN(R, L) do { \
        const int per_token = (3 * L * (R + 4) + 256 / L + 1) * 4; \
        int ct = (46 * 1024 - 32) / (2 * per_token + 1024); \
        ct = ct < 1 ? 1 : (ct > 16 ? 16 : ct); \
        const size_t smem = 2 * (size_t)(((ct * (per_token / 4)) + 3) & ~3) * 4 + (size_t)ct * 1024; \
        g_launch_err = launch_pdl(linear_scan_kernel<R, L>, dim3(S, H, (dv + 256 / L - 1) / (256 / L)), dim3(256), smem, (cudaStream_t)s, q, q_stride, \
            k, k_stride, v, v_stride, a, a_stride, beta_logit, beta_stride, q_scale, state, (size_t)slot_stride, cu_tokens, seq_slots, n_slots, \
            o, o_stride, H, Hq, d, dv, ct, error_word()); \
    } while (0)
    if (d <= 32) HFB_SCAN(4, 8);
    else if (d <= 64) HFB_SCAN(8, 8);
    else if (d <= 128) HFB_SCAN(16, 8);
    else if (d <= 256) HFB_SCAN(16, 16);
    else HFB_SCAN(16, 32);
#undef HFB_SCAN
    return check_pdl_launch(g_launch_err, "linear_scan");
}

extern "C" int hfb_gate_norm(const float *o, const void *w, int w_dt, float eps, const float *g, int g_splits, int g_stride,
                             int g_col0, int gate, void *out, int out_dt, int T, int H, int dv, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!o || !w || !g || !out || !valid_dt(w_dt) || !valid_dt(out_dt) || g_splits < 1 || H <= 0 || dv <= 0 || (gate != 0 && gate != 1))
        return fail(HFB_EINVAL, "gate_norm: bad arguments (H=%d dv=%d)", H, dv);
    const int hb = (H + REC_WARPS - 1) / REC_WARPS;
    if (hb > 65535) return fail(HFB_ENOTSUP, "gate_norm: %d heads exceed the grid limit", H);
    if (out_dt == HFB_F32)
        g_launch_err = launch_pdl(gate_norm_kernel<float>, dim3(T, hb), dim3(REC_WARPS * 32), 0, (cudaStream_t)s, o, w, w_dt, eps, g, g_splits,
                                  g_stride, g_col0, gate, (float *)out, T, H, dv);
    else
        g_launch_err = launch_pdl(gate_norm_kernel<__nv_bfloat16>, dim3(T, hb), dim3(REC_WARPS * 32), 0, (cudaStream_t)s, o, w, w_dt, eps, g,
                                  g_splits, g_stride, g_col0, gate, (__nv_bfloat16 *)out, T, H, dv);
    return check_pdl_launch(g_launch_err, "gate_norm");
}

extern "C" int hfb_mingru_scan(const float *row, int splits, const void *bz, const void *bx, int b_dt, float *state, int64_t slot_stride,
                               const int32_t *cu_tokens, const int32_t *seq_slots, int n_slots, int S, void *out, int out_dt, int T,
                               int W, hfb_stream s)
{
    if (S <= 0 || T <= 0) return HFB_OK;
    if (!row || !state || !cu_tokens || !seq_slots || !out || !valid_dt(out_dt) || splits < 1 || W <= 0 || slot_stride < W ||
        ((bz || bx) && !valid_dt(b_dt)))
        return fail(HFB_EINVAL, "mingru_scan: bad arguments (W=%d)", W);
    if (S > 65535) return fail(HFB_ENOTSUP, "mingru_scan: %d requests exceed the grid limit", S);
    if (T == S) {
        // every request brings one token
        const int blocks = rec_blocks((size_t)T * W);
        if (out_dt == HFB_F32)
            g_launch_err = launch_pdl(mingru_step_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, row, splits, bz, bx, b_dt, state,
                                      (size_t)slot_stride, seq_slots, n_slots, (float *)out, T, W, error_word());
        else
            g_launch_err = launch_pdl(mingru_step_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, row, splits, bz, bx, b_dt,
                                      state, (size_t)slot_stride, seq_slots, n_slots, (__nv_bfloat16 *)out, T, W, error_word());
        return check_pdl_launch(g_launch_err, "mingru_step");
    }
    const dim3 grid((W + MG_CH - 1) / MG_CH, S);
    const dim3 block((MG_FILL + 1) * 32);
    if (out_dt == HFB_F32)
        g_launch_err = launch_pdl(mingru_scan_kernel<float>, grid, block, 0, (cudaStream_t)s, row, splits, bz, bx, b_dt, state,
                                  (size_t)slot_stride, cu_tokens, seq_slots, n_slots, (float *)out, T, W, error_word());
    else
        g_launch_err = launch_pdl(mingru_scan_kernel<__nv_bfloat16>, grid, block, 0, (cudaStream_t)s, row, splits, bz, bx, b_dt,
                                  state, (size_t)slot_stride, cu_tokens, seq_slots, n_slots, (__nv_bfloat16 *)out, T, W, error_word());
    return check_pdl_launch(g_launch_err, "mingru_scan");
}
