// Dynamic tanh in the place of a norm, fused with the residual add that precedes it, and a
// plain scaling of 32-bit rows.
//
// For each output row r (source row s = rows ? rows[r] : r):
//   v = x[s,:] + sum_d delta[d][s,:]            (32-bit sum; written back to x when write_x)
//   out[r,i] = tanh(alpha * v[i]) * w[i] + b[i]
// No statistic of the row is taken, so nothing crosses threads: blockIdx.x is the row, blockIdx.y a slice
// of it.  All arithmetic is 32-bit with the accurate tanhf.
#include "common.cuh"

__global__ void add_dyt_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype, int n_delta,
                               size_t delta_stride, const int* __restrict__ rows, int E, const void* __restrict__ w,
                               const void* __restrict__ b, int w_dtype, float alpha, void* __restrict__ out,
                               int out_dtype, int write_x) {
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* xr = x + size_t(s) * E;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < E; i += gridDim.y * blockDim.x) {
        float v = xr[i];
        for (int d = 0; d < n_delta; ++d) v += gb_load(delta, delta_dtype, d * delta_stride + size_t(s) * E + i);
        if (write_x && n_delta) xr[i] = v;
        gb_store(out, out_dtype, size_t(r) * E + i, tanhf(alpha * v) * gb_load(w, w_dtype, i) + gb_load(b, w_dtype, i));
    }
}

GB_API int gb_add_dyt(float* x, const void* delta, int delta_dtype, int n_delta, long long delta_stride, const int* rows,
                      int n_rows, int E, const void* w, const void* b, int w_dtype, float alpha, void* out, int out_dtype,
                      int write_x, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(w_dtype) && gb_is_dtype(out_dtype), "gb_add_dyt: bad dtype");
    GB_REQUIRE(n_delta == 0 || (delta && gb_is_dtype(delta_dtype)), "gb_add_dyt: bad delta");
    GB_REQUIRE(E > 0 && n_rows >= 0 && w && b, "gb_add_dyt: bad sizes E=%d rows=%d", E, n_rows);
    if (n_rows == 0) return 0;
    const int threads = 128;
    int slices = (E + threads - 1) / threads;
    slices = slices > 16 ? 16 : slices;
    add_dyt_kernel<<<dim3(n_rows, slices), threads, 0, stream>>>(x, delta, delta_dtype, n_delta, size_t(delta_stride), rows, E, w, b,
                                                   w_dtype, alpha, out, out_dtype, write_x);
    GB_LAUNCH_OK("gb_add_dyt");
    return 0;
}

// x[i] *= scale for n 32-bit values (logits that a model multiplies by a constant).
__global__ void scale_kernel(float* __restrict__ x, size_t n, float scale) {
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) x[i] *= scale;
}

GB_API int gb_scale(float* x, long long n, float scale, cudaStream_t stream) {
    GB_REQUIRE(n >= 0, "gb_scale: bad size %lld", n);
    if (n == 0) return 0;
    const long long blocks = (n + 255) / 256;
    scale_kernel<<<int(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, stream>>>(x, size_t(n), scale);
    GB_LAUNCH_OK("gb_scale");
    return 0;
}

// x[i] <- cap tanh(x[i] / cap) for n 32-bit values (logits that a model bounds softly).
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) x[i] = cap * tanhf(x[i] / cap);
}

GB_API int gb_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && cap > 0.f, "gb_softcap: bad size %lld or cap %g", n, cap);
    if (n == 0) return 0;
    const long long blocks = (n + 255) / 256;
    softcap_kernel<<<int(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, stream>>>(x, size_t(n), cap);
    GB_LAUNCH_OK("gb_softcap");
    return 0;
}
