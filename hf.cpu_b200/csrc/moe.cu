// Mixture of experts without a trip to the host: router (float32 logits, top-k, softmax over the chosen logits),
// grouping of the (token, choice) pairs by expert, a grouped product over the groups' tiles, and the weighted sum.
// Every size the host needs for a launch is an upper bound (tiles <= pairs / tile + experts); the device-side tile
// count decides which blocks work, so a step of single tokens can be replayed as a graph.
//
// An output row is computed from its own input row and its expert's weights only, with one fixed summation order
// over k, and a token's choices are summed in the order the router made them: what a token gets does not depend on
// which other tokens are in the step nor on the order of the lists.
#include "common.cuh"
#include <stdlib.h>
#include <string.h>

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {

constexpr int ROUTE_WARPS = 4;

__device__ __forceinline__ float moe_act(float v, int act)
{
    if (act == HFB_ACT_RELU2) { v = fmaxf(v, 0.f); v *= v; }
    else if (act == HFB_ACT_RELU) v = fmaxf(v, 0.f);
    else if (act == HFB_ACT_SILU) v = v / (1.0f + expf(-v));
    else if (act == HFB_ACT_GELU_TANH) v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v;
}

// The choice of experts from the router's logits z [splits, T, E] (float32: partial sums of the router's product,
// summed in split order, plus its bias; finished logits have one split and no bias): one warp per token; the `top`
// largest, the lower index among equals; weights = softmax over the chosen logits only.  smem per warp: E logits, `top`
// chosen.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_topk_kernel(const float *zs, int splits, const void *bias, int bias_dt, int T, int E, int top, int32_t *ids, float *weights)
{
    pdl_entry();
    pdl_sync_small();
    extern __shared__ float route_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= T) return;
    float *z = route_smem + (size_t)warp * (E + top), *zc = z + E;
    for (int e = lane; e < E; e += 32) {
        float v = 0.f;
        for (int s = 0; s < splits; s++) v += zs[((size_t)s * T + t) * E + e];
        z[e] = bias ? v + load_any(bias, bias_dt, e) : v;
    }
    __syncwarp();
    for (int j = 0; j < top; j++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < bi)) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;                 // (nothing comparable left: logits that are not numbers)
        if (lane == 0) { zc[j] = best; ids[(size_t)t * top + j] = bi; z[bi] = -INFINITY; }
        __syncwarp();
    }
    if (lane == 0) {
        const float m = zc[0];                        // the first chosen is the largest
        float sum = 0.f;
        for (int j = 0; j < top; j++) { zc[j] = expf(zc[j] - m); sum += zc[j]; }
        const float inv = 1.0f / sum;
        for (int j = 0; j < top; j++) weights[(size_t)t * top + j] = zc[j] * inv;
    }
}

// A router that scores with a softmax over all of its outputs and chooses among groups: z [splits, T, E] as above;
// s = softmax(z) over all E; the choice score of an output is s + correction; the E outputs form `n_groups` equal groups
// of neighbours, a group's score is its largest choice score, and only the outputs of the `keep` best groups can be
// chosen (the lower group among equals); of those the `top` largest choice scores choose (the lower index among equals).
// weights = s of the chosen (without the correction) * scale, not renormalised.  An index at or above the number of real
// experts names an identity expert; whoever reads `ids` decides what that means.  One warp per token; smem per warp:
// 2 E + n_groups floats.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_softmax_kernel(const float *zs, int splits, const void *correction, int corr_dt, int T, int E, int top, int n_groups,
                         int keep, float scale, int32_t *ids, float *weights)
{
    pdl_entry();
    pdl_sync_small();
    extern __shared__ float route_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= T) return;
    float *sc = route_smem + (size_t)warp * (2 * E + n_groups), *ch = sc + E, *gs = ch + E;
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) {
        float v = 0.f;
        for (int s = 0; s < splits; s++) v += zs[((size_t)s * T + t) * E + e];
        sc[e] = v;
        m = fmaxf(m, v);
    }
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float p = expf(sc[e] - m); sc[e] = p; sum += p; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) {
        const float p = sc[e] * inv;
        sc[e] = p;
        ch[e] = correction ? p + load_any(correction, corr_dt, e) : p;
    }
    __syncwarp();
    if (n_groups > 1 && keep < n_groups) {
        const int per = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float b = -INFINITY;
            for (int i = 0; i < per; i++) b = fmaxf(b, ch[g * per + i]);
            gs[g] = b;
        }
        __syncwarp();
        // a group is kept when fewer than `keep` groups come before it in the order (score descending, index ascending)
        for (int g = lane; g < n_groups; g += 32) {
            const float mine = gs[g];
            int before = 0;
            for (int o = 0; o < n_groups; o++) before += (gs[o] > mine || (gs[o] == mine && o < g)) ? 1 : 0;
            if (before >= keep)
                for (int i = 0; i < per; i++) ch[g * per + i] = -INFINITY;
        }
        __syncwarp();
    }
    for (int j = 0; j < top; j++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = ch[e];
            if (v > best || (v == best && e < bi && v > -INFINITY)) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;                 // (nothing left to choose from)
        if (lane == 0) {
            ids[(size_t)t * top + j] = bi;
            weights[(size_t)t * top + j] = sc[bi] * scale;
            ch[bi] = -INFINITY;
        }
        __syncwarp();
    }
}

// One block.  smem: counts[E], offsets[E], cursor[E].
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int32_t *ids, int pairs, int E, int tile, int32_t *order, int32_t *tile_expert, int32_t *tile_p0,
                int32_t *tile_n, int32_t *n_tiles)
{
    pdl_entry();
    pdl_sync_small();
    extern __shared__ int sort_smem[];
    int *counts = sort_smem, *offsets = counts + E, *cursor = offsets + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, n = 0;
        for (int e = 0; e < E; e++) {
            offsets[e] = at;
            for (int p0 = 0; p0 < counts[e]; p0 += tile) {
                tile_expert[n] = e;
                tile_p0[n] = at + p0;
                tile_n[n] = min(tile, counts[e] - p0);
                n++;
            }
            at += counts[e];
        }
        *n_tiles = n;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) order[offsets[e] + atomicAdd(&cursor[e], 1)] = p;
    }
}

constexpr int GT = 64, GK = 16;       // tile of 64 places x 64 features, 16 of k at a time

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TA *__restrict__ a, const TW *__restrict__ w, void *out, int out_dt, int act, int N, int K,
                const int32_t *order, int src_div, int scatter, const int32_t *tile_expert, const int32_t *tile_p0,
                const int32_t *tile_n, const int32_t *n_tiles)
{
    const int glu = act >> 8;          // HFB_ACT_GLU set: see the epilogue
    act &= 255;
    pdl_sync();
    const int ti = blockIdx.y;
    if (ti >= *n_tiles) return;
    __shared__ float sa[GK][GT + 1];
    __shared__ float sw[GK][GT + 1];
    __shared__ int s_src[GT], s_dst[GT];
    // (a tile of the lists holds up to 128 places: this kernel takes them as two halves of 64, blockIdx.z)
    const int e = tile_expert[ti], p0 = tile_p0[ti] + GT * blockIdx.z, rows = tile_n[ti] - GT * (int)blockIdx.z;
    if (rows <= 0) return;
    const int n0 = blockIdx.x * GT;
    if (threadIdx.x < GT) {
        const int r = threadIdx.x;
        int src = -1, dst = -1;
        if (r < rows) {
            const int p = p0 + r, pair = order[p];
            src = src_div > 0 ? pair / src_div : p;
            dst = scatter ? pair : p;
        }
        s_src[r] = src;
        s_dst[r] = dst;
    }
    __syncthreads();
    const TW *we = w + (size_t)e * N * K;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += GK) {
        for (int x = threadIdx.x; x < GT * GK; x += 256) {
            const int r = x / GK, c = x % GK;
            const int gk = k0 + c, src = s_src[r];
            sa[c][r] = (src >= 0 && gk < K) ? to_f32(a[(size_t)src * K + gk]) : 0.f;
        }
        for (int x = threadIdx.x; x < GT * GK; x += 256) {
            const int r = x / GK, c = x % GK;
            const int gn = n0 + r, gk = k0 + c;
            sw[c][r] = (gn < N && gk < K) ? to_f32(we[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; kk++) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) wv[j] = sw[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int dst = s_dst[ty * 4 + i];
        if (dst < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            if (glu) {              // rows of w alternate gate, up: features (2f, 2f + 1) give out[f] = act(gate) * up
                if (!(j & 1)) store_any(out, out_dt, (size_t)dst * (N / 2) + gn / 2, moe_act(acc[i][j], act) * acc[i][j + 1]);
                continue;
            }
            store_any(out, out_dt, (size_t)dst * N + gn, moe_act(acc[i][j], act));
        }
    }
}

// The same grouped product for bfloat16 operands on the tensor cores (mma.sync m16n8k16, float32 accumulators): a tile
// of 128 places x 128 features, eight warps of 32 places x 64 features each; operands come into padded shared memory
// by cp.async, 32 of k at a time in three stages, so that two pieces are on their way while one is multiplied;
// fragments come out of shared memory with ldmatrix.x4.  A warp whose places lie beyond the tile's count multiplies
// nothing.  K is a multiple of 8 and the operands are 16-byte aligned (every 16-byte piece of a row lies wholly inside
// or outside K).
constexpr int MT = 128, MK = 32, MPAD = 8;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *p)
{
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

constexpr int MSTAGES = 3;

__device__ __forceinline__ void cp_async_16(void *smem, const void *gmem, bool valid)
{
    // 16 bytes global -> shared without passing registers; src-size 0 fills the 16 bytes with zeros instead
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int MN = 128;                                       // features per tile of the tensor-core form
constexpr size_t MMA_SMEM = (size_t)MSTAGES * (MT + MN) * (MK + MPAD) * sizeof(__nv_bfloat16) + 2 * MT * sizeof(int);

__global__ void __launch_bounds__(256)
moe_gemm_mma_kernel(const __nv_bfloat16 *__restrict__ a, const __nv_bfloat16 *__restrict__ w, void *out, int out_dt, int act,
                    int N, int K, const int32_t *order, int src_div, int scatter, const int32_t *tile_expert,
                    const int32_t *tile_p0, const int32_t *tile_n, const int32_t *n_tiles)
{
    const int glu = act >> 8;          // HFB_ACT_GLU set: see the epilogue
    act &= 255;
    pdl_sync();
    const int ti = blockIdx.y;
    if (ti >= *n_tiles) return;
    extern __shared__ __align__(16) uint8_t mma_smem[];
    typedef __nv_bfloat16 (*Stage)[MK + MPAD];
    __nv_bfloat16 *sa_base = (__nv_bfloat16 *)mma_smem, *sw_base = sa_base + (size_t)MSTAGES * MT * (MK + MPAD);
    int *s_src = (int *)(sw_base + (size_t)MSTAGES * MN * (MK + MPAD)), *s_dst = s_src + MT;
    auto sa = [&](int st) { return (Stage)(sa_base + (size_t)st * MT * (MK + MPAD)); };
    auto sw = [&](int st) { return (Stage)(sw_base + (size_t)st * MN * (MK + MPAD)); };
    const int e = tile_expert[ti], p0 = tile_p0[ti], rows = tile_n[ti];
    const int n0 = blockIdx.x * MN, n_end = min(N, n0 + MN);
    if (threadIdx.x < MT) {
        const int r = threadIdx.x;
        int src = -1, dst = -1;
        if (r < rows) {
            const int p = p0 + r, pair = order[p];
            src = src_div > 0 ? pair / src_div : p;
            dst = scatter ? pair : p;
        }
        s_src[r] = src;
        s_dst[r] = dst;
    }
    __syncthreads();
    const __nv_bfloat16 *we = w + (size_t)e * N * K;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int wm = warp & 3, wn = warp >> 2;                // this warp: places 32 wm .. + 32, features 64 wn .. + 64
    const bool live0 = 32 * wm < rows, live1 = 32 * wm + 16 < rows;
    // the 16-byte pieces this thread moves per 32 of k: two of the places' rows, two of the weights' rows
    const int vr = threadIdx.x >> 2, vk = (threadIdx.x & 3) * 8;
    const __nv_bfloat16 *pa[2], *pw[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int src = s_src[vr + 64 * i], gn = n0 + vr + 64 * i;
        pa[i] = src >= 0 ? a + (size_t)src * K + vk : nullptr;
        pw[i] = gn < n_end ? we + (size_t)gn * K + vk : nullptr;
    }
    // a piece of k on its way into stage `st` (rows that do not exist and k beyond K arrive as zeros)
    auto fetch = [&](int k0, int st) {
        const bool in = k0 + vk < K;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            cp_async_16(&sa(st)[vr + 64 * i][vk], pa[i] && in ? pa[i] + k0 : a, pa[i] && in);
            cp_async_16(&sw(st)[vr + 64 * i][vk], pw[i] && in ? pw[i] + k0 : w, pw[i] && in);
        }
    };
    float acc[2][8][4];
#pragma unroll
    for (int m = 0; m < 2; m++)
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[m][i][j] = 0.f;
    // ldmatrix row addresses: A 16x16 = (rows 0-7 | 8-15) x (k 0-7 | 8-15); B pairs of 8-feature tiles x (k 0-7 | 8-15)
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
    const int chunks = (K + MK - 1) / MK;
#pragma unroll
    for (int c = 0; c < MSTAGES - 1; c++) {
        if (c < chunks) fetch(c * MK, c);
        cp_async_commit();
    }
    for (int c = 0; c < chunks; c++) {
        const int st = c % MSTAGES;
        cp_async_wait<MSTAGES - 2>();            // piece c has landed (the newer groups may still be in flight)
        __syncthreads();                         // ... for every thread, and piece c - 1 has been multiplied by all
        if (c + MSTAGES - 1 < chunks) fetch((c + MSTAGES - 1) * MK, (c + MSTAGES - 1) % MSTAGES);
        cp_async_commit();
        if (live0) {
#pragma unroll
            for (int ks = 0; ks < MK; ks += 16) {
                uint32_t af[2][4];
                ldmatrix_x4(af[0], &sa(st)[32 * wm + a_row][ks + a_col]);
                if (live1) ldmatrix_x4(af[1], &sa(st)[32 * wm + 16 + a_row][ks + a_col]);
#pragma unroll
                for (int np = 0; np < 4; np++) {
                    uint32_t bf[4];
                    ldmatrix_x4(bf, &sw(st)[64 * wn + np * 16 + b_row][ks + b_col]);
                    mma_bf16(acc[0][2 * np], af[0], bf[0], bf[1]);
                    mma_bf16(acc[0][2 * np + 1], af[0], bf[2], bf[3]);
                    if (live1) {
                        mma_bf16(acc[1][2 * np], af[1], bf[0], bf[1]);
                        mma_bf16(acc[1][2 * np + 1], af[1], bf[2], bf[3]);
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int m = 0; m < 2; m++) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int dst = s_dst[32 * wm + 16 * m + g + 8 * half];
            if (dst < 0) continue;
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int gn = n0 + 64 * wn + nt * 8 + 2 * t + j;
                    if (gn >= n_end) continue;
                    if (glu) {
                        if (j == 0) store_any(out, out_dt, (size_t)dst * (N / 2) + gn / 2, moe_act(acc[m][nt][2 * half], act) * acc[m][nt][2 * half + 1]);
                        continue;
                    }
                    store_any(out, out_dt, (size_t)dst * N + gn, moe_act(acc[m][nt][2 * half + j], act));
                }
            }
        }
    }
}

// The form for steps of a few tokens, whose tiles hold at most 16 places (the grouping is asked for tiles of 16): a
// block only streams its slice of an expert's weights, so slices are narrow (64 features: many blocks, spread evenly
// over the SMs), pieces are long (64 of k) and many are in flight (eight stages, two blocks an SM).  Four warps, each
// 16 places x 16 features.
constexpr int ST_ROWS = 16, ST_N = 64, ST_K = 64, ST_STAGES = 8;
constexpr size_t SMALL_SMEM = (size_t)ST_STAGES * (ST_ROWS + ST_N) * (ST_K + MPAD) * sizeof(__nv_bfloat16);

__global__ void __launch_bounds__(128)
moe_gemm_small_kernel(const __nv_bfloat16 *__restrict__ a, const __nv_bfloat16 *__restrict__ w, void *out, int out_dt, int act,
                      int N, int K, const int32_t *order, int src_div, int scatter, const int32_t *tile_expert,
                      const int32_t *tile_p0, const int32_t *tile_n, const int32_t *n_tiles)
{
    const int glu = act >> 8;          // HFB_ACT_GLU set: see the epilogue
    act &= 255;
    pdl_sync();
    const int ti = blockIdx.y;
    if (ti >= *n_tiles) return;
    extern __shared__ __align__(16) uint8_t small_smem[];
    typedef __nv_bfloat16 (*Stage)[ST_K + MPAD];
    __nv_bfloat16 *sa_base = (__nv_bfloat16 *)small_smem, *sw_base = sa_base + (size_t)ST_STAGES * ST_ROWS * (ST_K + MPAD);
    auto sa = [&](int st) { return (Stage)(sa_base + (size_t)st * ST_ROWS * (ST_K + MPAD)); };
    auto sw = [&](int st) { return (Stage)(sw_base + (size_t)st * ST_N * (ST_K + MPAD)); };
    __shared__ int s_src[ST_ROWS], s_dst[ST_ROWS];
    const int e = tile_expert[ti], p0 = tile_p0[ti], rows = min(tile_n[ti], ST_ROWS);
    const int n0 = blockIdx.x * ST_N;
    if (threadIdx.x < ST_ROWS) {
        const int r = threadIdx.x;
        int src = -1, dst = -1;
        if (r < rows) {
            const int p = p0 + r, pair = order[p];
            src = src_div > 0 ? pair / src_div : p;
            dst = scatter ? pair : p;
        }
        s_src[r] = src;
        s_dst[r] = dst;
    }
    __syncthreads();
    const __nv_bfloat16 *we = w + (size_t)e * N * K;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // the 16-byte pieces this thread moves per 64 of k: one of a place's row, four of the weights' rows
    const int vk = (threadIdx.x & 7) * 8, ar = threadIdx.x >> 3, wr = threadIdx.x >> 3;
    const int asrc = s_src[ar];
    const __nv_bfloat16 *pa = asrc >= 0 ? a + (size_t)asrc * K + vk : nullptr, *pw[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int gn = n0 + wr + 16 * i;
        pw[i] = gn < N ? we + (size_t)gn * K + vk : nullptr;
    }
    auto fetch = [&](int k0, int st) {
        const bool in = k0 + vk < K;
        cp_async_16(&sa(st)[ar][vk], pa && in ? pa + k0 : a, pa && in);
#pragma unroll
        for (int i = 0; i < 4; i++) cp_async_16(&sw(st)[wr + 16 * i][vk], pw[i] && in ? pw[i] + k0 : w, pw[i] && in);
    };
    float acc[2][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
    const int chunks = (K + ST_K - 1) / ST_K;
#pragma unroll
    for (int c = 0; c < ST_STAGES - 1; c++) {
        if (c < chunks) fetch(c * ST_K, c);
        cp_async_commit();
    }
    for (int c = 0; c < chunks; c++) {
        const int st = c % ST_STAGES;
        cp_async_wait<ST_STAGES - 2>();
        __syncthreads();
        if (c + ST_STAGES - 1 < chunks) fetch((c + ST_STAGES - 1) * ST_K, (c + ST_STAGES - 1) % ST_STAGES);
        cp_async_commit();
#pragma unroll
        for (int ks = 0; ks < ST_K; ks += 16) {
            uint32_t af[4], bf[4];
            ldmatrix_x4(af, &sa(st)[a_row][ks + a_col]);
            ldmatrix_x4(bf, &sw(st)[16 * warp + b_row][ks + b_col]);
            mma_bf16(acc[0], af, bf[0], bf[1]);
            mma_bf16(acc[1], af, bf[2], bf[3]);
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int dst = s_dst[g + 8 * half];
        if (dst < 0) continue;
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int gn = n0 + 16 * warp + nt * 8 + 2 * t + j;
                if (gn >= N) continue;
                if (glu) {
                    if (j == 0) store_any(out, out_dt, (size_t)dst * (N / 2) + gn / 2, moe_act(acc[nt][2 * half], act) * acc[nt][2 * half + 1]);
                    continue;
                }
                store_any(out, out_dt, (size_t)dst * N + gn, moe_act(acc[nt][2 * half + j], act));
            }
        }
    }
}

template <typename TY>
__global__ void moe_combine_kernel(const TY *y, const float *weights, float *out, int T, int top, int N)
{
    pdl_entry();
    pdl_sync_small();
    const size_t total = (size_t)T * N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / N;
        const int c = (int)(i % N);
        float acc = 0.f;
        for (int j = 0; j < top; j++) acc = fmaf(weights[t * top + j], to_f32(y[(t * top + j) * N + c]), acc);
        out[i] = acc;
    }
}

}  // namespace hfb

using namespace hfb;

// HFB_GEMM=plain in the environment keeps the grouped products on the float32 multiply-add kernel, as it does the others.
static bool plain_products()
{
    static const int v = [] { const char *e = getenv("HFB_GEMM"); return e && strcmp(e, "plain") == 0 ? 1 : 0; }();
    return v != 0;
}

extern "C" int hfb_moe_topk(const float *z, int splits, const void *bias, int bias_dt, int T, int E, int top, int32_t *ids,
                            float *weights, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (E <= 0 || top <= 0 || top > E || splits < 1 || (bias && !valid_dt(bias_dt))) return fail(HFB_EINVAL, "moe_topk: bad arguments (experts=%d top=%d)", E, top);
    const size_t smem = (size_t)ROUTE_WARPS * (E + top) * sizeof(float);
    if (smem > 48 * 1024) return fail(HFB_ENOTSUP, "moe_topk: %d experts are more than the kernel takes", E);
    g_launch_err = launch_pdl(moe_topk_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, (cudaStream_t)s, z, splits, bias, bias_dt, T, E, top, ids, weights);
    return check_pdl_launch(g_launch_err, "moe_topk");
}

extern "C" int hfb_moe_route_softmax(const float *z, int splits, const void *correction, int corr_dt, int T, int E, int top,
                                     int n_groups, int keep, float scale, int32_t *ids, float *weights, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (E <= 0 || top <= 0 || top > E || splits < 1 || (correction && !valid_dt(corr_dt)) || n_groups < 1 || E % n_groups ||
        keep < 1 || keep > n_groups || keep * (E / n_groups) < top)
        return fail(HFB_EINVAL, "moe_route_softmax: bad arguments (outputs=%d top=%d groups=%d keep=%d)", E, top, n_groups, keep);
    const size_t smem = (size_t)ROUTE_WARPS * (2 * E + n_groups) * sizeof(float);
    if (smem > 48 * 1024) return fail(HFB_ENOTSUP, "moe_route_softmax: %d router outputs are more than the kernel takes", E);
    g_launch_err = launch_pdl(moe_route_softmax_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, (cudaStream_t)s,
                              z, splits, correction, corr_dt, T, E, top, n_groups, keep, scale, ids, weights);
    return check_pdl_launch(g_launch_err, "moe_route_softmax");
}

extern "C" int hfb_moe_max_tiles(int pairs, int E, int tile)
{
    if (pairs <= 0 || E <= 0 || tile <= 0) return 0;
    return pairs / tile + (E < pairs ? E : pairs);
}

extern "C" int hfb_moe_sort(const int32_t *ids, int pairs, int E, int tile, int32_t *order, int32_t *tile_expert,
                            int32_t *tile_p0, int32_t *tile_n, int32_t *n_tiles, hfb_stream s)
{
    if (pairs <= 0) return HFB_OK;
    if (E <= 0 || tile <= 0) return fail(HFB_EINVAL, "moe_sort: bad arguments");
    const size_t smem = (size_t)3 * E * sizeof(int);
    if (smem > 48 * 1024) return fail(HFB_ENOTSUP, "moe_sort: %d experts are more than the grouping kernel takes", E);
    g_launch_err = launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)s, ids, pairs, E, tile, order, tile_expert, tile_p0, tile_n, n_tiles);
    return check_pdl_launch(g_launch_err, "moe_sort");
}

extern "C" int hfb_moe_gemm(const void *a, int a_dt, const void *w, int w_dt, void *out, int out_dt, int act, int N, int K,
                            const int32_t *order, int src_div, int scatter, const int32_t *tile_expert, const int32_t *tile_p0,
                            const int32_t *tile_n, const int32_t *n_tiles, int max_tiles, int tile, hfb_stream s)
{
    if (max_tiles <= 0) return HFB_OK;
    if (!valid_dt(a_dt) || !valid_dt(w_dt) || !valid_dt(out_dt) || N <= 0 || K <= 0 || tile < 1 || tile > MT || act < 0 || (act & 255) > HFB_ACT_NONE ||
        (act >> 8) > 1 || ((act >> 8) && (N & 1)))
        return fail(HFB_EINVAL, "moe_gemm: bad arguments (N=%d K=%d tile=%d)", N, K, tile);
    if (max_tiles > 65535) return fail(HFB_ENOTSUP, "moe_gemm: %d tiles exceed the grid", max_tiles);
    const dim3 grid((N + GT - 1) / GT, max_tiles);
    cudaStream_t st = (cudaStream_t)s;
    if (a_dt == HFB_BF16 && w_dt == HFB_BF16 && (K & 7) == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0 &&
        !plain_products()) {
        static bool opted[64] = {};              // more than 48 KB of shared memory: asked for once per device
        const int dev = current_device();
        if (!opted[dev]) {
            if (cudaFuncSetAttribute(moe_gemm_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMALL_SMEM) != cudaSuccess ||
                cudaFuncSetAttribute(moe_gemm_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM) != cudaSuccess)
                return fail(HFB_ECUDA, "moe_gemm: the kernel's shared memory could not be set");
            opted[dev] = true;
        }
        if (tile <= ST_ROWS) {                  // tiles of at most 16 places: the form for steps of a few tokens
            g_launch_err = launch_pdl(moe_gemm_small_kernel, dim3((N + ST_N - 1) / ST_N, max_tiles), dim3(128), SMALL_SMEM, st, (const __nv_bfloat16 *)a,
                                      (const __nv_bfloat16 *)w, out, out_dt, act, N, K, order, src_div, scatter, tile_expert, tile_p0, tile_n, n_tiles);
            return check_pdl_launch(g_launch_err, "moe_gemm_small");
        }
        g_launch_err = launch_pdl(moe_gemm_mma_kernel, dim3((N + MN - 1) / MN, max_tiles), dim3(256), MMA_SMEM, st, (const __nv_bfloat16 *)a, (const __nv_bfloat16 *)w, out, out_dt, act, N, K,
                                  order, src_div, scatter, tile_expert, tile_p0, tile_n, n_tiles);
        return check_pdl_launch(g_launch_err, "moe_gemm_mma");
    }
#define LAUNCH(TA, TW) g_launch_err = launch_pdl(moe_gemm_kernel<TA, TW>, dim3(grid.x, grid.y, (tile + GT - 1) / GT), dim3(256), 0, st, (const TA *)a, (const TW *)w, out, out_dt, act, N, K, order, src_div, scatter, tile_expert, tile_p0, tile_n, n_tiles)
    if (a_dt == HFB_F32 && w_dt == HFB_F32) LAUNCH(float, float);
    else if (a_dt == HFB_F32) LAUNCH(float, __nv_bfloat16);
    else if (w_dt == HFB_F32) LAUNCH(__nv_bfloat16, float);
    else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
    return check_pdl_launch(g_launch_err, "moe_gemm");
}

extern "C" int hfb_moe_combine(const void *y, int y_dt, const float *weights, float *out, int T, int top, int N, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(y_dt) || top <= 0 || N <= 0) return fail(HFB_EINVAL, "moe_combine: bad arguments");
    size_t b = ((size_t)T * N + 255) / 256;
    const unsigned blocks = (unsigned)(b > 148 * 16 ? 148 * 16 : b);
    if (y_dt == HFB_F32) g_launch_err = launch_pdl(moe_combine_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, (const float *)y, weights, out, T, top, N);
    else g_launch_err = launch_pdl(moe_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, (const __nv_bfloat16 *)y, weights, out, T, top, N);
    return check_pdl_launch(g_launch_err, "moe_combine");
}
