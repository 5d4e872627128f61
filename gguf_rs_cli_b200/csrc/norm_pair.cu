// RMS norm of the residual stream with several pending terms and up to two weights at once:
//   v = x[s,:] + sum_d delta_d[s,:]          (32-bit; written back to x when write_x)
//   out1[r,:] = v / sqrt(mean(v^2) + eps) * (offset + w1),   out2[r,:] = the same with w2 (when given)
// for each output row r (source row s = rows ? rows[r] : r).  offset 1 serves weights that are stored around zero.
// A layer whose mixer and feed-forward read two norms of the same x gets both from one pass over the row, and the
// terms that the layer before left (its mixer's, its feed-forward's, and what a repeated pass adds) are summed here.
#include "common.cuh"

constexpr int NP_MAX_TERMS = 3;

struct NormPairParams {
    float* x;
    const void* delta[NP_MAX_TERMS];
    int delta_dtype[NP_MAX_TERMS];
    int n_delta;
    const int* rows;
    int E;
    const void *w1, *w2;
    int w_dtype;
    float offset, eps;
    void *out1, *out2;
    int out_dtype, write_x;
};

__device__ __forceinline__ float4 np_load4(const void* p, int dtype, size_t i) {
    if (dtype == GB_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void np_store4(void* p, int dtype, size_t i, float4 v) {
    if (dtype == GB_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = v;
    } else {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<const unsigned*>(&a);
        raw.y = *reinterpret_cast<const unsigned*>(&b);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = raw;
    }
}

// The row's sum v is kept in shared memory between the two passes (E floats).  VEC: four entries at a time.
template <bool VEC>
__global__ void __launch_bounds__(256) norm_pair_kernel(const NormPairParams p) {
    extern __shared__ __align__(16) float np_row[];
    __shared__ float red[8];
    const int r = blockIdx.x, s = p.rows ? p.rows[r] : r, E = p.E;
    const size_t base = size_t(s) * E;
    float ss = 0.f;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(p.x + base + i);
            for (int d = 0; d < p.n_delta; ++d) {
                const float4 t = np_load4(p.delta[d], p.delta_dtype[d], base + i);
                v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
            }
            if (p.write_x && p.n_delta) *reinterpret_cast<float4*>(p.x + base + i) = v;
            *reinterpret_cast<float4*>(np_row + i) = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            float v = p.x[base + i];
            for (int d = 0; d < p.n_delta; ++d) v += gb_load(p.delta[d], p.delta_dtype[d], base + i);
            if (p.write_x && p.n_delta) p.x[base + i] = v;
            np_row[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = gb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
    const float rms = sqrtf(tot / float(E) + p.eps);
    const size_t orow = size_t(r) * E;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(np_row + i);
            const float4 n = make_float4(v.x / rms, v.y / rms, v.z / rms, v.w / rms);
            const float4 a = np_load4(p.w1, p.w_dtype, i);
            np_store4(p.out1, p.out_dtype, orow + i,
                      make_float4(n.x * (p.offset + a.x), n.y * (p.offset + a.y), n.z * (p.offset + a.z), n.w * (p.offset + a.w)));
            if (p.out2) {
                const float4 b = np_load4(p.w2, p.w_dtype, i);
                np_store4(p.out2, p.out_dtype, orow + i,
                          make_float4(n.x * (p.offset + b.x), n.y * (p.offset + b.y), n.z * (p.offset + b.z), n.w * (p.offset + b.w)));
            }
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            const float n = np_row[i] / rms;
            gb_store(p.out1, p.out_dtype, orow + i, n * (p.offset + gb_load(p.w1, p.w_dtype, i)));
            if (p.out2) gb_store(p.out2, p.out_dtype, orow + i, n * (p.offset + gb_load(p.w2, p.w_dtype, i)));
        }
    }
}

// x float32 [T, E]; d0, d1, d2: the first n_delta of them are terms [T, E] of dtypes dt0, dt1, dt2 to be added; rows: the
// rows to produce (null: all n_rows = T); w1, w2 [E] of one dtype (w2 and out2 null: one result only).
GB_API int gb_add_rmsnorm_pair(float* x, const void* d0, int dt0, const void* d1, int dt1, const void* d2, int dt2, int n_delta,
                               const int* rows, int n_rows, int E, const void* w1, const void* w2, int w_dtype, float offset,
                               float eps, void* out1, void* out2, int out_dtype, int write_x, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(w_dtype) && gb_is_dtype(out_dtype), "gb_add_rmsnorm_pair: bad dtype");
    GB_REQUIRE(n_delta >= 0 && n_delta <= NP_MAX_TERMS, "gb_add_rmsnorm_pair: %d terms (at most %d)", n_delta, NP_MAX_TERMS);
    GB_REQUIRE(E > 0 && n_rows >= 0 && eps > 0.f, "gb_add_rmsnorm_pair: bad sizes E=%d rows=%d eps=%g", E, n_rows, eps);
    if (n_rows == 0) return 0;
    GB_REQUIRE(w1 && out1, "gb_add_rmsnorm_pair: weight or result missing");
    GB_REQUIRE((w2 == nullptr) == (out2 == nullptr), "gb_add_rmsnorm_pair: the second weight and the second result go together");
    GB_REQUIRE(size_t(E) * 4 <= 200 * 1024, "gb_add_rmsnorm_pair: rows of %d entries are too long", E);
    NormPairParams p;
    const void* ds[NP_MAX_TERMS] = {d0, d1, d2};
    const int dts[NP_MAX_TERMS] = {dt0, dt1, dt2};
    auto aligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    bool vec = E % 4 == 0 && aligned(x) && aligned(w1) && aligned(out1) && (!w2 || (aligned(w2) && aligned(out2)));
    for (int d = 0; d < NP_MAX_TERMS; ++d) {
        p.delta[d] = d < n_delta ? ds[d] : nullptr;
        p.delta_dtype[d] = dts[d];
        if (d < n_delta) {
            GB_REQUIRE(ds[d] && gb_is_dtype(dts[d]), "gb_add_rmsnorm_pair: bad term %d", d);
            vec = vec && aligned(ds[d]);
        }
    }
    p.x = x; p.n_delta = n_delta; p.rows = rows; p.E = E; p.w1 = w1; p.w2 = w2; p.w_dtype = w_dtype; p.offset = offset; p.eps = eps;
    p.out1 = out1; p.out2 = out2; p.out_dtype = out_dtype; p.write_x = write_x;
    const size_t smem = size_t(E) * 4;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(norm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(norm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return gb_fail("gb_add_rmsnorm_pair: cannot get %zu bytes of shared memory", smem);
    }
    const int threads = E >= 1024 ? 256 : 128;
    if (vec) norm_pair_kernel<true><<<n_rows, threads, smem, stream>>>(p);
    else norm_pair_kernel<false><<<n_rows, threads, smem, stream>>>(p);
    GB_LAUNCH_OK("gb_add_rmsnorm_pair");
    return 0;
}
