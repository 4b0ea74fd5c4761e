// The tail of a q|k|v product for attention whose queries and keys are brought to unit root mean square per head
// after the rotation, whose value heads may have another size than the key heads, and whose layer may have no
// keys and values of its own (it reads another layer's cache): sum of split-K partials + bias -> rotation of the
// first n_rot dimensions (pairs i, i + n_rot/2) -> x / sqrt(mean(x^2) + eps) over the head -> queries to q_out,
// times a weight shared by the heads where the layer has one -> queries to q_out, keys and values to the token's cache
// slot.  A layer whose values are mixed with those of an earlier layer (v <- (1 - lambda) v + lambda v_first, v_first the
// same token's values in the first such layer) does that here, before the store, so that the cache holds the mixed
// values; the first such layer leaves its own values behind for the others.  Everything between the float32 sums and the
// stores is float32.  pairing 1 rotates the pairs (2i, 2i + 1) instead.  dv = 0: the row has no value heads (the layer's
// values are its keys) and nothing is written to v_cache.
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();

__device__ __forceinline__ void store4(float *dst, float4 v) { *(float4 *)dst = v; }
__device__ __forceinline__ void store4(__nv_bfloat16 *dst, float4 v)
{
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *(uint32_t *)&a;
    u.y = *(uint32_t *)&b;
    *(uint2 *)dst = u;
}

constexpr int RN_WARPS = 4;
constexpr int RN_MAX_D = 256;

// One warp per (token, head) of the row [H query heads of d | G key heads of d | G value heads of dv].
template <typename TO>
__global__ void __launch_bounds__(RN_WARPS * 32)
rope_norm_kv_kernel(const float *src, int splits, const void *bias, int bias_dt, const float *cos_sin, int n_rot,
                    int n_positions, const int32_t *positions, const int32_t *slots, TO *q_out, TO *k_cache, TO *v_cache,
                    long long cache_slots, int T, int H, int G, int d, int dv, int norm, float eps, const float *q_w,
                    const float *k_w, float *v_first, int v_mode, float v_lambda, int pairing, int *err)
{
    pdl_entry();
    pdl_sync_small();
    __shared__ __align__(16) float buf[RN_WARPS][RN_MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // a token per blockIdx.x, four of its units per blockIdx.y (no division to find them)
    const int units = H + (dv > 0 ? 2 : 1) * G;
    const int t = blockIdx.x, u = blockIdx.y * RN_WARPS + warp;
    if (u >= units) return;
    const int C = H * d + G * d + G * dv;
    int col0, n;
    TO *dst;
    bool is_value = false;
    if (u < H) { col0 = u * d; n = d; dst = q_out + ((size_t)t * H + u) * d; }
    else {
        if (!slots) return;
        const long long slot = slots[t];
        if (slot < 0) return;
        if (slot >= cache_slots) { if (lane == 0) atomicOr(err, HFB_ERR_SLOT); return; }
        if (u < H + G) { col0 = H * d + (u - H) * d; n = d; dst = k_cache + ((size_t)slot * G + (u - H)) * d; }
        else { col0 = H * d + G * d + (u - H - G) * dv; n = dv; dst = v_cache + ((size_t)slot * G + (u - H - G)) * dv; is_value = true; }
    }
    float *x = buf[warp];
    const size_t plane = (size_t)T * C;
    // (16-byte reads where the heads' sizes allow: a warp then fetches a head of 128 values with one instruction a lane)
    const bool vec = ((d | dv) & 3) == 0 && ((uintptr_t)src & 15) == 0;
    if (vec) {
        for (int c = lane * 4; c < n; c += 128) {
            const float *p = src + (size_t)t * C + col0 + c;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < splits; s++) {
                const float4 g = *(const float4 *)(p + (size_t)s * plane);
                acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
            }
            if (bias) {
                acc.x += load_any(bias, bias_dt, col0 + c); acc.y += load_any(bias, bias_dt, col0 + c + 1);
                acc.z += load_any(bias, bias_dt, col0 + c + 2); acc.w += load_any(bias, bias_dt, col0 + c + 3);
            }
            *(float4 *)(x + c) = acc;
        }
    } else {
        for (int c = lane; c < n; c += 32) {
            float v = bias ? load_any(bias, bias_dt, col0 + c) : 0.f;
            const float *p = src + (size_t)t * C + col0 + c;
            float acc = 0.f;
            for (int s = 0; s < splits; s++) acc += p[(size_t)s * plane];
            x[c] = acc + v;
        }
    }
    __syncwarp();
    if (is_value) {
        float *first = v_first ? v_first + (size_t)t * G * dv + (size_t)(u - H - G) * dv : nullptr;
        for (int c = lane; c < n; c += 32) {
            float v = x[c];
            if (v_mode == 1) first[c] = v;
            else if (v_mode == 2) v = (1.0f - v_lambda) * v + v_lambda * first[c];
            dst[c] = from_f32<TO>(v);
        }
        return;
    }
    const float *w = u < H ? q_w : k_w;
    const int half = n_rot / 2;
    if (half > 0) {
        int pos = positions[t];
        if (pos < 0 || pos >= n_positions) { if (lane == 0) atomicOr(err, HFB_ERR_POSITION); pos = 0; }
        const float *cs = cos_sin + (size_t)pos * half * 2;
        for (int i = lane; i < half; i += 32) {
            float lo, hi;
            const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
            rope_pair(x[ia], x[ib], cs[2 * i], cs[2 * i + 1], lo, hi);
            x[ia] = lo;
            x[ib] = hi;
        }
        __syncwarp();
    }
    float r = 1.0f;
    if (norm) {
        float ss = 0.f;
        for (int c = lane; c < n; c += 32) ss = fmaf(x[c], x[c], ss);
        ss = warp_sum(ss);
        r = 1.0f / sqrtf(ss / (float)n + eps);
    }
    if (vec && ((uintptr_t)dst & (4 * sizeof(TO) - 1)) == 0) {
        for (int c = lane * 4; c < n; c += 128) {
            float4 v = *(const float4 *)(x + c);
            v.x *= r; v.y *= r; v.z *= r; v.w *= r;
            if (norm && w) { v.x *= w[c]; v.y *= w[c + 1]; v.z *= w[c + 2]; v.w *= w[c + 3]; }
            store4(dst + c, v);
        }
        return;
    }
    if (norm && w) { for (int c = lane; c < n; c += 32) dst[c] = from_f32<TO>(x[c] * r * w[c]); }
    else { for (int c = lane; c < n; c += 32) dst[c] = from_f32<TO>(x[c] * r); }
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_rope_norm_kv_write(const float *src, int splits, const void *bias, int bias_dt, const float *cos_sin,
                                      int n_rot, int n_positions, const int32_t *positions, const int32_t *slots,
                                      void *q_out, void *k_cache, void *v_cache, int out_dt, int64_t cache_slots, int T,
                                      int H, int G, int d, int dv, int norm, float eps, const float *q_w, const float *k_w,
                                      float *v_first, int v_mode, float v_lambda, int pairing, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(out_dt) || (bias && !valid_dt(bias_dt)) || splits < 1 || H <= 0 || G < 0 || d <= 0 || dv < 0 ||
        n_rot < 0 || n_rot > d || (n_rot & 1))
        return fail(HFB_EINVAL, "rope_norm_kv_write: bad arguments (H=%d G=%d d=%d dv=%d n_rot=%d)", H, G, d, dv, n_rot);
    if (d > RN_MAX_D || dv > RN_MAX_D) return fail(HFB_ENOTSUP, "rope_norm_kv_write: head sizes above %d are not supported", RN_MAX_D);
    if (n_rot > 0 && (!cos_sin || !positions)) return fail(HFB_EINVAL, "rope_norm_kv_write: rotation needs a table and positions");
    if (v_mode < 0 || v_mode > 2 || (v_mode && (!v_first || G <= 0))) return fail(HFB_EINVAL, "rope_norm_kv_write: value mixing needs the first layer's values");
    if (G > 0 && slots && (!k_cache || (dv > 0 && !v_cache))) return fail(HFB_EINVAL, "rope_norm_kv_write: keys and values need a cache");
    const int unit_blocks = (H + (dv > 0 ? 2 : 1) * G + RN_WARPS - 1) / RN_WARPS;
    if (unit_blocks > 65535) return fail(HFB_ENOTSUP, "rope_norm_kv_write: %d heads exceed the grid limit", H + 2 * G);
    const dim3 blocks(T, unit_blocks);
    if (out_dt == HFB_F32)
        g_launch_err = launch_pdl(rope_norm_kv_kernel<float>, blocks, dim3(RN_WARPS * 32), 0, (cudaStream_t)s, src, splits, bias, bias_dt, cos_sin, n_rot,
            n_positions, positions, slots, (float *)q_out, (float *)k_cache, (float *)v_cache, (long long)cache_slots, T, H, G, d, dv, norm, eps, q_w, k_w, v_first, v_mode, v_lambda, pairing, error_word());
    else
        g_launch_err = launch_pdl(rope_norm_kv_kernel<__nv_bfloat16>, blocks, dim3(RN_WARPS * 32), 0, (cudaStream_t)s, src, splits, bias, bias_dt, cos_sin, n_rot,
            n_positions, positions, slots, (__nv_bfloat16 *)q_out, (__nv_bfloat16 *)k_cache, (__nv_bfloat16 *)v_cache, (long long)cache_slots, T, H, G, d, dv, norm, eps,
            q_w, k_w, v_first, v_mode, v_lambda, pairing, error_word());
    return check_pdl_launch(g_launch_err, "rope_norm_kv_write");
}
