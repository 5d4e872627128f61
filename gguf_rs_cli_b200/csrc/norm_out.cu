// The norm of a sublayer's result on its way into the residual stream, for layers that norm what a sublayer
// gives and not what it reads:
//   x[t,:] += y[t,:] / sqrt(mean(y[t,:]^2) + eps) * w        (32-bit; x is the residual stream)
//   xb[t,:] = bfloat16(x[t,:])                               (optional: the rows that the next sublayer's products read)
// y null: only the copy is made.  One block per token; the row of y is read twice (the second time from cache).
#include "common.cuh"

__global__ void __launch_bounds__(256) norm_residual_add_kernel(float* __restrict__ x, const void* __restrict__ y, int y_dtype,
                                                                long long ldy, int E, const void* __restrict__ w, int w_dtype,
                                                                float eps, __nv_bfloat16* __restrict__ xb) {
    __shared__ float red[8];
    const int t = blockIdx.x;
    float* xr = x + size_t(t) * E;
    float f = 0.f;
    if (y) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            const float v = gb_load(y, y_dtype, size_t(t) * ldy + i);
            ss = fmaf(v, v, ss);
        }
        ss = gb_warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int k = 0; k < (blockDim.x >> 5); ++k) tot += red[k];
        f = 1.f / sqrtf(tot / float(E) + eps);
    }
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float v = xr[i];
        if (y) {
            v += gb_load(y, y_dtype, size_t(t) * ldy + i) * f * gb_load(w, w_dtype, i);
            xr[i] = v;
        }
        if (xb) xb[size_t(t) * E + i] = __float2bfloat16_rn(v);
    }
}

// x float32 [T, E] contiguous; y [T, E] with rows ldy apart (or null); w [E]; xb bfloat16 [T, E] contiguous (or null).
GB_API int gb_norm_residual_add(float* x, const void* y, int y_dtype, long long ldy, int T, int E, const void* w, int w_dtype,
                                float eps, void* xb, cudaStream_t stream) {
    GB_REQUIRE(!y || (gb_is_dtype(y_dtype) && gb_is_dtype(w_dtype) && w && eps > 0.f), "gb_norm_residual_add: bad arguments");
    GB_REQUIRE(T >= 0 && E > 0 && (y || xb), "gb_norm_residual_add: bad sizes T=%d E=%d", T, E);
    if (T == 0) return 0;
    norm_residual_add_kernel<<<T, 256, 0, stream>>>(x, y, y_dtype, ldy, E, w, w_dtype, eps, (__nv_bfloat16*)xb);
    GB_LAUNCH_OK("gb_norm_residual_add");
    return 0;
}

// The same for layers that norm a sublayer's input AND its result, with what stands around it in one pass over the row:
//   u = y                                                        (one result), or
//   u = mix * (y / rms(y) * wy + y2 / rms(y2) * wy2)             (two results that are normed and blended first)
//   x += u / rms(u) * w            (w null: u itself is the result and goes to u_out; x is not touched)
//   h = x / rms(x) * w_next        (optional: the rows the next sublayer reads, in h's dtype)
//   xb = bfloat16(x)               (optional)
// rms(v) = sqrt(mean(v^2) + eps); every sum is 32-bit.  y null: only the last two steps.  One block per token, the row
// in shared memory.
struct SandwichParams {
    float* x;
    const void *y, *y2;
    long long ldy, ldy2;
    const void *wy, *wy2, *w, *w_next;
    void* h;
    __nv_bfloat16* xb;
    float* u_out;
    float mix, eps;
    int y_dtype, y2_dtype, w_dtype, h_dtype, E;
};

__device__ __forceinline__ float nr_block_sum(float v, float* red) {
    v = gb_warp_sum(v);
    __syncthreads();                       // red may still be read from the sum before
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < (blockDim.x >> 5); ++k) tot += red[k];
    return tot;
}

__global__ void __launch_bounds__(256) norm_sandwich_kernel(const SandwichParams p) {
    extern __shared__ float nr_row[];
    __shared__ float red[8];
    const int t = blockIdx.x, E = p.E;
    float* xr = p.x ? p.x + size_t(t) * E : nullptr;
    if (p.y) {
        if (p.y2) {
            float s1 = 0.f, s2 = 0.f;
            for (int i = threadIdx.x; i < E; i += blockDim.x) {
                const float a = gb_load(p.y, p.y_dtype, size_t(t) * p.ldy + i), b = gb_load(p.y2, p.y2_dtype, size_t(t) * p.ldy2 + i);
                s1 = fmaf(a, a, s1);
                s2 = fmaf(b, b, s2);
            }
            const float f1 = 1.f / sqrtf(nr_block_sum(s1, red) / float(E) + p.eps);
            const float f2 = 1.f / sqrtf(nr_block_sum(s2, red) / float(E) + p.eps);
            for (int i = threadIdx.x; i < E; i += blockDim.x) {
                const float a = gb_load(p.y, p.y_dtype, size_t(t) * p.ldy + i) * f1 * gb_load(p.wy, p.w_dtype, i);
                const float b = gb_load(p.y2, p.y2_dtype, size_t(t) * p.ldy2 + i) * f2 * gb_load(p.wy2, p.w_dtype, i);
                nr_row[i] = p.mix * (a + b);
            }
        } else {
            for (int i = threadIdx.x; i < E; i += blockDim.x) nr_row[i] = gb_load(p.y, p.y_dtype, size_t(t) * p.ldy + i);
        }
        if (!p.w) {
            for (int i = threadIdx.x; i < E; i += blockDim.x) p.u_out[size_t(t) * E + i] = nr_row[i];
            return;
        }
        float ss = 0.f;
        for (int i = threadIdx.x; i < E; i += blockDim.x) ss = fmaf(nr_row[i], nr_row[i], ss);
        const float f = 1.f / sqrtf(nr_block_sum(ss, red) / float(E) + p.eps);
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            const float v = xr[i] + nr_row[i] * f * gb_load(p.w, p.w_dtype, i);
            xr[i] = v;
            nr_row[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) nr_row[i] = xr[i];
    }
    if (p.xb)
        for (int i = threadIdx.x; i < E; i += blockDim.x) p.xb[size_t(t) * E + i] = __float2bfloat16_rn(nr_row[i]);
    if (p.h) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < E; i += blockDim.x) ss = fmaf(nr_row[i], nr_row[i], ss);
        const float f = 1.f / sqrtf(nr_block_sum(ss, red) / float(E) + p.eps);
        for (int i = threadIdx.x; i < E; i += blockDim.x)
            gb_store(p.h, p.h_dtype, size_t(t) * E + i, nr_row[i] * f * gb_load(p.w_next, p.w_dtype, i));
    }
}

// x float32 [T, E] contiguous (null with w null); y, y2 [T, E] rows ldy, ldy2 apart (y2 null: one result; y null: none);
// wy, wy2, w, w_next [E] of w_dtype; h [T, E] contiguous of h_dtype, with w_next; xb bfloat16 [T, E]; u_out float32 [T, E].
GB_API int gb_norm_sandwich(float* x, const void* y, int y_dtype, long long ldy, const void* y2, int y2_dtype, long long ldy2,
                            const void* wy, const void* wy2, float mix, const void* w, const void* w_next, int w_dtype, float eps,
                            void* h, int h_dtype, void* xb, float* u_out, int T, int E, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(w_dtype) && eps > 0.f && E > 0 && T >= 0, "gb_norm_sandwich: bad arguments");
    GB_REQUIRE(!y || gb_is_dtype(y_dtype), "gb_norm_sandwich: bad dtype of the result");
    GB_REQUIRE(!y2 || (y && gb_is_dtype(y2_dtype) && wy && wy2), "gb_norm_sandwich: two results need weights of their own");
    GB_REQUIRE(w ? x != nullptr : (y && u_out && !h && !xb) || (!y && x), "gb_norm_sandwich: nowhere to put the result");
    GB_REQUIRE((h == nullptr) == (w_next == nullptr) && (!h || gb_is_dtype(h_dtype)), "gb_norm_sandwich: the next norm needs a weight and a place");
    GB_REQUIRE(size_t(E) * 4 <= 200 * 1024, "gb_norm_sandwich: rows of %d entries do not fit shared memory", E);
    if (T == 0) return 0;
    const size_t smem = size_t(E) * sizeof(float);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(norm_sandwich_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
        return gb_fail("gb_norm_sandwich: cannot get %zu bytes of shared memory", smem);
    SandwichParams p;
    p.x = x; p.y = y; p.y2 = y2; p.ldy = ldy; p.ldy2 = ldy2; p.wy = wy; p.wy2 = wy2; p.w = w; p.w_next = w_next; p.h = h;
    p.xb = (__nv_bfloat16*)xb; p.u_out = u_out; p.mix = mix; p.eps = eps; p.y_dtype = y_dtype; p.y2_dtype = y2_dtype;
    p.w_dtype = w_dtype; p.h_dtype = h_dtype; p.E = E;
    norm_sandwich_kernel<<<T, 256, smem, stream>>>(p);
    GB_LAUNCH_OK("gb_norm_sandwich");
    return 0;
}
