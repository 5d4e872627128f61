// A feed-forward of routed experts: the router's choice per token, and the chosen experts' gated units on the
// CUDA cores with 32-bit sums, token by token (steps of few tokens, the 32-bit mode, and sizes the tiled kernel of
// moe_grouped.cu does not take).
//
// Choice (one warp per token, all 32-bit): s_e = sigmoid(z_e), or softmax(z)_e over all experts.  The experts form
// n_groups equal groups of neighbours; a group's mark is the sum of its two largest choice scores (of its one, if it has
// one expert); only experts of the `keep` groups with the largest marks can be chosen; of those the `top` with the
// largest choice scores are, and their weights are s / (sum of the chosen s + 1e-20) * scale.  The choice score is s, or
// s plus a correction per expert that the weights do not see.  Equal values: the lower index wins.
//
// Identity experts: the experts numbered n_real and above have no matrices; what they give is the token's own row.
#include <math.h>

#include "common.cuh"

constexpr int MOE_MAX_EXPERTS = 1024;
constexpr int MOE_MAX_TOP = 32;

static int moe_smem(const void* kernel, size_t bytes, const char* what) {
    if (bytes <= 48 * 1024) return 0;
    if (bytes > 200 * 1024) return gb_fail("%s: rows of %zu bytes do not fit shared memory", what, bytes);
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)) != cudaSuccess)
        return gb_fail("%s: cannot get %zu bytes of shared memory", what, bytes);
    return 0;
}

// The choice for one token by one warp; z: the token's logits (shared or global memory).
__device__ void moe_route_warp(const float* z, int E, int n_groups, int keep, int top, float scale, int* __restrict__ ids,
                               float* __restrict__ weights, float* s, float* c, float* mark, unsigned char* open_, int* chosen,
                               int lane, int softmax, const float* __restrict__ corr) {
    const int size = E / n_groups;
    float zmax = -INFINITY, zsum = 0.f;
    if (softmax) {
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
        zmax = gb_warp_max(zmax);
        for (int e = lane; e < E; e += 32) zsum += expf(z[e] - zmax);
        zsum = gb_warp_sum(zsum);
    }
    for (int e = lane; e < E; e += 32) {
        s[e] = softmax ? expf(z[e] - zmax) / zsum : 1.f / (1.f + expf(-z[e]));
        c[e] = corr ? s[e] + corr[e] : s[e];
        open_[e] = 0;
    }
    __syncwarp();
    for (int g = lane; g < n_groups; g += 32) {
        float a = -INFINITY, b = -INFINITY;                 // the two largest
        for (int i = 0; i < size; ++i) {
            const float v = c[g * size + i];
            if (v > a) { b = a; a = v; }
            else if (v > b) b = v;
        }
        mark[g] = a + (b > -INFINITY ? b : 0.f);
    }
    __syncwarp();
    for (int r = 0; r < keep; ++r) {                        // the group with the largest mark, `keep` times
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int g = lane; g < n_groups; g += 32)
            if (mark[g] > best) { best = mark[g]; arg = g; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg != 0x7fffffff) {
            for (int i = lane; i < size; i += 32) open_[arg * size + i] = 1;
            if (lane == 0) mark[arg] = -INFINITY;
        }
        __syncwarp();
    }
    float sum = 0.f;
    for (int r = 0; r < top; ++r) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (open_[e] && c[e] > best) { best = c[e]; arg = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (lane == 0) {
            chosen[r] = arg == 0x7fffffff ? 0 : arg;
            if (arg != 0x7fffffff) open_[arg] = 0;
        }
        __syncwarp();
        sum += arg == 0x7fffffff ? 0.f : s[arg];
    }
    for (int r = lane; r < top; r += 32) {
        ids[r] = chosen[r];
        weights[r] = s[chosen[r]] / (sum + 1e-20f) * scale;
    }
}

__global__ void __launch_bounds__(32) moe_route_kernel(const float* __restrict__ z, int E, int n_groups, int keep, int top,
                                                       float scale, int* __restrict__ ids, float* __restrict__ weights,
                                                       int softmax, const float* __restrict__ corr) {
    __shared__ float s[MOE_MAX_EXPERTS];
    __shared__ float c[MOE_MAX_EXPERTS];
    __shared__ float mark[MOE_MAX_EXPERTS];
    __shared__ unsigned char open_[MOE_MAX_EXPERTS];        // 1: the expert may still be chosen
    __shared__ int chosen[MOE_MAX_TOP];
    const int t = blockIdx.x;
    moe_route_warp(z + size_t(t) * E, E, n_groups, keep, top, scale, ids + size_t(t) * top, weights + size_t(t) * top, s, c, mark,
                   open_, chosen, threadIdx.x, softmax, corr);
}

// z float32 [T, E] router logits -> ids int32 [T, top], weights float32 [T, top], largest score first.
// softmax: the scores are softmax(z) instead of sigmoids; corr [E] float32 or null: added to the scores for the choice only.
GB_API int gb_moe_route(const float* z, int T, int E, int n_groups, int keep, int top, float scale, int* ids, float* weights,
                        int softmax, const float* corr, cudaStream_t stream) {
    GB_REQUIRE(E > 0 && E <= MOE_MAX_EXPERTS, "gb_moe_route: %d experts (1..%d)", E, MOE_MAX_EXPERTS);
    GB_REQUIRE(n_groups > 0 && E % n_groups == 0 && keep > 0 && keep <= n_groups, "gb_moe_route: %d experts in %d groups, %d kept", E, n_groups, keep);
    GB_REQUIRE(top > 0 && top <= MOE_MAX_TOP && top <= keep * (E / n_groups), "gb_moe_route: %d experts cannot be chosen from %d groups of %d (at most %d)", top, keep, E / n_groups, MOE_MAX_TOP);
    if (T == 0) return 0;
    moe_route_kernel<<<T, 32, 0, stream>>>(z, E, n_groups, keep, top, scale, ids, weights, softmax, corr);
    GB_LAUNCH_OK("gb_moe_route");
    return 0;
}

// The router's product and the choice in one kernel: one block per token; the token's row lies in shared memory as
// 32-bit floats, the warps take the experts' rows in turn (32-bit sums), the first warp then chooses.
template <typename TW>
__device__ __forceinline__ float moe_row_dot(const TW* __restrict__ w, const float* __restrict__ hs, int K, int lane);

template <typename TW>
__global__ void __launch_bounds__(256) moe_router_kernel(const void* __restrict__ x, int x_dtype, long long ldx, int K,
                                                         const TW* __restrict__ w, int E, int n_groups, int keep, int top,
                                                         float scale, int* __restrict__ ids, float* __restrict__ weights,
                                                         int softmax, const float* __restrict__ corr) {
    extern __shared__ float moe_xs[];
    __shared__ float z[MOE_MAX_EXPERTS];
    __shared__ float s[MOE_MAX_EXPERTS];
    __shared__ float c[MOE_MAX_EXPERTS];
    __shared__ float mark[MOE_MAX_EXPERTS];
    __shared__ unsigned char open_[MOE_MAX_EXPERTS];
    __shared__ int chosen[MOE_MAX_TOP];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < K; i += blockDim.x) moe_xs[i] = gb_load(x, x_dtype, size_t(t) * ldx + i);
    __syncthreads();
    for (int e = warp; e < E; e += (blockDim.x >> 5)) {
        const float v = gb_warp_sum(moe_row_dot<TW>(w + size_t(e) * K, moe_xs, K, lane));
        if (lane == 0) z[e] = v;
    }
    __syncthreads();
    if (warp == 0)
        moe_route_warp(z, E, n_groups, keep, top, scale, ids + size_t(t) * top, weights + size_t(t) * top, s, c, mark, open_, chosen,
                       lane, softmax, corr);
}

// ---------------------------------------------------------------- experts, token by token
// y[t, r, f] = unit(Wg[e] h_t, Wu[e] h_t)_f with e = ids[t, r]; unit = gb_act_glu_clamped.  One block per (token,
// choice) and slice of 32 features; the token's row lies in shared memory as 32-bit floats, a warp takes a feature at a
// time and its lanes share the two matrix rows in pieces of eight (bfloat16) or four (float32) entries.
// a lane's share of the product of a matrix row with the row in shared memory; the caller sums over the lanes
template <typename TW>
__device__ __forceinline__ float moe_row_dot(const TW* __restrict__ w, const float* __restrict__ hs, int K, int lane);

template <>
__device__ __forceinline__ float moe_row_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ hs, int K, int lane) {
    float acc = 0.f;
    if (K % 8 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
        for (int i = lane * 8; i < K; i += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(w + i);
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 v = __bfloat1622float2(p2[e]);
                acc = fmaf(v.x, hs[i + 2 * e], acc);
                acc = fmaf(v.y, hs[i + 2 * e + 1], acc);
            }
        }
    } else {
        for (int i = lane; i < K; i += 32) acc = fmaf(__bfloat162float(w[i]), hs[i], acc);
    }
    return acc;
}
template <>
__device__ __forceinline__ float moe_row_dot<float>(const float* __restrict__ w, const float* __restrict__ hs, int K, int lane) {
    float acc = 0.f;
    if (K % 4 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
        for (int i = lane * 4; i < K; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(w + i);
            acc = fmaf(v.x, hs[i], acc);
            acc = fmaf(v.y, hs[i + 1], acc);
            acc = fmaf(v.z, hs[i + 2], acc);
            acc = fmaf(v.w, hs[i + 3], acc);
        }
    } else {
        for (int i = lane; i < K; i += 32) acc = fmaf(w[i], hs[i], acc);
    }
    return acc;
}

constexpr int MOE_SLICE = 16;

template <typename TW>
__global__ void __launch_bounds__(128) moe_gate_up_kernel(const void* __restrict__ h, int h_dtype, long long ldh, int K, int F,
                                                          int top, const int* __restrict__ ids, const TW* __restrict__ wg,
                                                          const TW* __restrict__ wu, float limit, void* __restrict__ y,
                                                          int y_dtype, int n_real) {
    extern __shared__ float moe_hs[];
    const int pair = blockIdx.x, t = pair / top;
    const int e = ids[pair];
    if (e >= n_real) return;                       // an identity expert has no unit
    for (int i = threadIdx.x; i < K; i += blockDim.x) moe_hs[i] = gb_load(h, h_dtype, size_t(t) * ldh + i);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f_end = min(F, (blockIdx.y + 1) * MOE_SLICE);
    for (int f = blockIdx.y * MOE_SLICE + warp; f < f_end; f += 4) {
        const size_t row = (size_t(e) * F + f) * K;
        float g = moe_row_dot<TW>(wg + row, moe_hs, K, lane);
        float u = moe_row_dot<TW>(wu + row, moe_hs, K, lane);
        g = gb_warp_sum(g);
        u = gb_warp_sum(u);
        if (lane == 0) gb_store(y, y_dtype, size_t(pair) * F + f, gb_act_glu_clamped(g, u, limit));
    }
}

// z[pair, n] = sum_f Wd[ids[pair]][n, f] y[pair, f]: one block per (token, choice) pair and slice of results, the pair's unit
// outputs in shared memory as 32-bit floats (the shape of moe_gate_up_kernel, which keeps memory busy where one block per
// token did not: 0.18 ms against 0.06 ms for the same bytes).  moe_pair_sum_kernel then adds a token's rows with the
// router's weights in the order of the choices: out[t, n] (+)= sum_r weights[t, r] z[t * top + r, n].
template <typename TW>
__global__ void __launch_bounds__(128) moe_down_kernel(const void* __restrict__ y, int y_dtype, int F, int N,
                                                       const int* __restrict__ ids, const TW* __restrict__ wd,
                                                       float* __restrict__ z, int n_real, const void* __restrict__ h,
                                                       int h_dtype, long long ldh, int top) {
    extern __shared__ float moe_ys[];
    const int pair = blockIdx.x;
    const int e = ids[pair];
    if (e >= n_real) {                             // an identity expert: the pair's row is the token's own row
        const int n_end = min(N, (blockIdx.y + 1) * MOE_SLICE);
        for (int n = blockIdx.y * MOE_SLICE + threadIdx.x; n < n_end; n += blockDim.x)
            z[size_t(pair) * N + n] = gb_load(h, h_dtype, size_t(pair / top) * ldh + n);
        return;
    }
    for (int i = threadIdx.x; i < F; i += blockDim.x) moe_ys[i] = gb_load(y, y_dtype, size_t(pair) * F + i);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_end = min(N, (blockIdx.y + 1) * MOE_SLICE);
    for (int n = blockIdx.y * MOE_SLICE + warp; n < n_end; n += 4) {
        const float acc = gb_warp_sum(moe_row_dot<TW>(wd + (size_t(e) * N + n) * F, moe_ys, F, lane));
        if (lane == 0) z[size_t(pair) * N + n] = acc;
    }
}

__global__ void moe_pair_sum_kernel(const float* __restrict__ z, const float* __restrict__ weights, int top, int N,
                                    float* __restrict__ out, int accumulate, long long total) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / N;
    const int n = int(i - t * N);
    float acc = 0.f;
    for (int r = 0; r < top; ++r) acc = fmaf(weights[t * top + r], z[(t * top + r) * N + n], acc);
    out[i] = accumulate ? out[i] + acc : acc;
}

// x [T, K] rows ldx apart (the rows the router reads, 32-bit where the caller has them); w [E, K] contiguous.
GB_API int gb_moe_router(const void* x, int x_dtype, long long ldx, int T, int K, const void* w, int w_dtype, int E, int n_groups,
                         int keep, int top, float scale, int* ids, float* weights, int softmax, const float* corr,
                         cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(x_dtype) && gb_is_dtype(w_dtype), "gb_moe_router: bad dtype");
    GB_REQUIRE(E > 0 && E <= MOE_MAX_EXPERTS && K > 0, "gb_moe_router: %d experts (1..%d)", E, MOE_MAX_EXPERTS);
    GB_REQUIRE(n_groups > 0 && E % n_groups == 0 && keep > 0 && keep <= n_groups, "gb_moe_router: %d experts in %d groups, %d kept", E, n_groups, keep);
    GB_REQUIRE(top > 0 && top <= MOE_MAX_TOP && top <= keep * (E / n_groups), "gb_moe_router: %d experts cannot be chosen from %d groups of %d (at most %d)", top, keep, E / n_groups, MOE_MAX_TOP);
    if (T == 0) return 0;
    const size_t smem = size_t(K) * 4;
    if (w_dtype == GB_F32) {
        if (moe_smem((const void*)moe_router_kernel<float>, smem + 20 * 1024, "gb_moe_router")) return 1;
        moe_router_kernel<float><<<T, 256, smem, stream>>>(x, x_dtype, ldx, K, (const float*)w, E, n_groups, keep, top, scale, ids, weights, softmax, corr);
    } else {
        if (moe_smem((const void*)moe_router_kernel<__nv_bfloat16>, smem + 20 * 1024, "gb_moe_router")) return 1;
        moe_router_kernel<__nv_bfloat16><<<T, 256, smem, stream>>>(x, x_dtype, ldx, K, (const __nv_bfloat16*)w, E, n_groups, keep, top, scale, ids, weights, softmax, corr);
    }
    GB_LAUNCH_OK("gb_moe_router");
    return 0;
}

// h [T, K] rows ldh apart; ids [T, top]; wg, wu [E, F, K] contiguous (dtype w_dtype); y [T, top, F] contiguous.
GB_API int gb_moe_gate_up(const void* h, int h_dtype, long long ldh, int T, int K, int F, int top, const int* ids,
                          const void* wg, const void* wu, int w_dtype, float limit, void* y, int y_dtype, int n_real,
                          cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(h_dtype) && gb_is_dtype(w_dtype) && gb_is_dtype(y_dtype), "gb_moe_gate_up: bad dtype");
    GB_REQUIRE(K > 0 && F > 0 && top > 0 && limit > 0.f, "gb_moe_gate_up: bad sizes K=%d F=%d top=%d limit=%g", K, F, top, limit);
    if (T == 0) return 0;
    const size_t smem = size_t(K) * 4;
    dim3 grid(T * top, (F + MOE_SLICE - 1) / MOE_SLICE);
    GB_REQUIRE(grid.y <= 65535, "gb_moe_gate_up: an expert of %d hidden entries is too wide", F);
    if (w_dtype == GB_F32) {
        if (moe_smem((const void*)moe_gate_up_kernel<float>, smem, "gb_moe_gate_up")) return 1;
        moe_gate_up_kernel<float><<<grid, 128, smem, stream>>>(h, h_dtype, ldh, K, F, top, ids, (const float*)wg, (const float*)wu, limit, y, y_dtype, n_real);
    } else {
        if (moe_smem((const void*)moe_gate_up_kernel<__nv_bfloat16>, smem, "gb_moe_gate_up")) return 1;
        moe_gate_up_kernel<__nv_bfloat16><<<grid, 128, smem, stream>>>(h, h_dtype, ldh, K, F, top, ids, (const __nv_bfloat16*)wg,
                                                                        (const __nv_bfloat16*)wu, limit, y, y_dtype, n_real);
    }
    GB_LAUNCH_OK("gb_moe_gate_up");
    return 0;
}

// y [T, top, F]; wd [E, N, F] contiguous; z float32 [T * top, N] scratch; out float32 [T, N] contiguous (added to when
// accumulate).  Experts numbered n_real and above are identity experts: their pairs' rows are the tokens' own rows h
// [T, N] (rows ldh apart).  Two launches.
GB_API int gb_moe_down(const void* y, int y_dtype, int T, int F, int N, int top, const int* ids, const float* weights,
                       const void* wd, int w_dtype, float* z, float* out, int accumulate, int n_real, const void* h, int h_dtype,
                       long long ldh, cudaStream_t stream) {
    GB_REQUIRE(n_real > 0 && (!h || gb_is_dtype(h_dtype)), "gb_moe_down: bad identity arguments");
    GB_REQUIRE(gb_is_dtype(y_dtype) && gb_is_dtype(w_dtype), "gb_moe_down: bad dtype");
    GB_REQUIRE(F > 0 && N > 0 && top > 0 && z, "gb_moe_down: bad sizes F=%d N=%d top=%d", F, N, top);
    if (T == 0) return 0;
    const size_t smem = size_t(F) * 4;
    dim3 grid(T * top, (N + MOE_SLICE - 1) / MOE_SLICE);
    GB_REQUIRE(grid.y <= 65535, "gb_moe_down: rows of %d entries are too wide", N);
    if (w_dtype == GB_F32) {
        if (moe_smem((const void*)moe_down_kernel<float>, smem, "gb_moe_down")) return 1;
        moe_down_kernel<float><<<grid, 128, smem, stream>>>(y, y_dtype, F, N, ids, (const float*)wd, z, h ? n_real : 0x7fffffff, h, h_dtype, ldh, top);
    } else {
        if (moe_smem((const void*)moe_down_kernel<__nv_bfloat16>, smem, "gb_moe_down")) return 1;
        moe_down_kernel<__nv_bfloat16><<<grid, 128, smem, stream>>>(y, y_dtype, F, N, ids, (const __nv_bfloat16*)wd, z, h ? n_real : 0x7fffffff, h, h_dtype, ldh, top);
    }
    GB_LAUNCH_OK("gb_moe_down");
    const long long total = (long long)T * N;
    moe_pair_sum_kernel<<<unsigned((total + 255) / 256), 256, 0, stream>>>(z, weights, top, N, out, accumulate, total);
    GB_LAUNCH_OK("gb_moe_down (sum)");
    return 0;
}

// ---------------------------------------------------------------- activations of whole buffers
__global__ void unary_act_kernel(void* __restrict__ x, int dtype, long long n, int act) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i < n) gb_store(x, dtype, size_t(i), gb_act_unary(gb_load(x, dtype, size_t(i)), act));
}

// The same for a block of `cols` columns of rows that lie ld entries apart.
__global__ void unary_act_rows_kernel(void* __restrict__ x, int dtype, long long n, int cols, long long ld, int act) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t at = size_t(i / cols) * ld + size_t(i % cols);
    gb_store(x, dtype, at, gb_act_unary(gb_load(x, dtype, at), act));
}

GB_API int gb_unary_act_rows(void* x, int dtype, int rows, int cols, long long ld, int act, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && act >= 1 && act <= 4, "gb_unary_act_rows: bad dtype or activation %d", act);
    GB_REQUIRE(rows >= 0 && cols >= 0 && ld >= cols, "gb_unary_act_rows: bad sizes rows=%d cols=%d ld=%lld", rows, cols, ld);
    const long long n = (long long)rows * cols;
    if (n == 0) return 0;
    unary_act_rows_kernel<<<unsigned((n + 255) / 256), 256, 0, stream>>>(x, dtype, n, cols, ld, act);
    GB_LAUNCH_OK("gb_unary_act_rows");
    return 0;
}

// x <- act(x) entry by entry, in place (contiguous).  act: GbGateAct or GbUnaryAct.
GB_API int gb_unary_act(void* x, int dtype, long long n, int act, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && act >= 1 && act <= 4, "gb_unary_act: bad dtype or activation %d", act);
    if (n == 0) return 0;
    unary_act_kernel<<<unsigned((n + 255) / 256), 256, 0, stream>>>(x, dtype, n, act);
    GB_LAUNCH_OK("gb_unary_act");
    return 0;
}

__global__ void glu_clamped_kernel(const void* __restrict__ gu, long long ld, void* __restrict__ out, int T, int F, int dtype,
                                   float limit) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= (long long)T * F) return;
    const long long t = i / F;
    const int f = int(i - t * F);
    gb_store(out, dtype, size_t(i), gb_act_glu_clamped(gb_load(gu, dtype, size_t(t) * ld + f), gb_load(gu, dtype, size_t(t) * ld + F + f), limit));
}

// gate_up [T, 2F] (gate in the first F columns, rows ld apart) -> out [T, F] contiguous = gb_act_glu_clamped(gate, up).
GB_API int gb_glu_clamped(const void* gate_up, long long ld, void* out, int T, int F, int dtype, float limit, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && F > 0 && limit > 0.f, "gb_glu_clamped: bad arguments");
    if (T == 0) return 0;
    const long long n = (long long)T * F;
    glu_clamped_kernel<<<unsigned((n + 255) / 256), 256, 0, stream>>>(gate_up, ld, out, T, F, dtype, limit);
    GB_LAUNCH_OK("gb_glu_clamped");
    return 0;
}
