// The recurrence of a selective state-space mixer with one decay per head and token (the state-space-duality form):
//   dt = softplus(dt_raw + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x
// per head, with B and C [N] shared by the heads of a group and S [N, P].  This is the walk of linear_walk.h with the
// decay the same for all key channels: its preparation writes q = C, k = dt B, the decay, v = x and D as the number
// whose product with v is added to what the state gives.  Step sizes, decays, their exponentials and softplus, and the
// state are 32-bit.
#include <math.h>

#include "common.cuh"
#include "linear_walk.h"

struct SsdPrepParams {
    const void *x, *bm, *cm;        // x [T, H*P], B and C [T, G*N]: column slices of one buffer with rows ld apart
    const void* dt;                 // [T, H] before the bias, rows ld_dt apart
    const void *dt_bias, *a_log, *skip;   // [H] each
    LinearWalkRows rows;
    long long ld, ld_dt;
    int dtype, dt_dtype, w_dtype, H, G, N, P;
};

// One warp per (token, head).
__global__ void __launch_bounds__(128) ssd_prep_kernel(const SsdPrepParams p) {
    const int t = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= p.H) return;
    const int N = p.N, DA = p.rows.DA, VA = p.rows.VA;
    const int g = h / (p.H / p.G);
    const float z = gb_load(p.dt, p.dt_dtype, size_t(t) * p.ld_dt + h) + gb_load(p.dt_bias, p.w_dtype, h);
    const float dt = z > 20.f ? z : log1pf(expf(z));
    const float decay = expf(-expf(gb_load(p.a_log, p.w_dtype, h)) * dt);
    float* o = p.rows.qkg + (size_t(t) * p.H + h) * 3 * DA;
    const size_t col = size_t(t) * p.ld + size_t(g) * N;
    for (int d = lane; d < DA; d += 32) {
        const bool in = d < N;
        o[d] = in ? gb_load(p.cm, p.dtype, col + d) : 0.f;
        o[DA + d] = in ? dt * gb_load(p.bm, p.dtype, col + d) : 0.f;
        o[2 * DA + d] = in ? decay : 0.f;
    }
    float* vo = p.rows.vf + (size_t(t) * p.H + h) * VA;
    for (int d = lane; d < VA; d += 32) vo[d] = d < p.P ? gb_load(p.x, p.dtype, size_t(t) * p.ld + size_t(h) * p.P + d) : 0.f;
    if (lane < 4) p.rows.bonus[(size_t(t) * p.H + h) * 4 + lane] = lane == 0 ? gb_load(p.skip, p.w_dtype, h) : 0.f;
}

// x [T, H*P], bm, cm [T, G*N]: column slices of one buffer (after the convolution and its activation), rows ld apart;
// dt [T, H] the step sizes' projection; dt_bias, a_log, skip [H]; state [slots, H, N, P] float32, read and renewed;
// out float32 [T, H*P].  scratch: gb_linear_walk_scratch_floats(T, H, N, P).
GB_API int gb_ssd(const void* x, const void* bm, const void* cm, int dtype, long long ld, const void* dt, int dt_dtype,
                  long long ld_dt, const void* dt_bias, const void* a_log, const void* skip, int w_dtype, float* state, float* out,
                  long long ldo, const int* cu, const int* slots, const int* qlens, int T, int B, int H, int G, int N, int P,
                  float* scratch, int max_qlen, float* seg_scratch, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(dt_dtype) && gb_is_dtype(w_dtype), "gb_ssd: bad dtype");
    GB_REQUIRE(H > 0 && G > 0 && H % G == 0 && N > 0 && N <= 2048 && P > 0 && (H + 3) / 4 <= 65535,
               "gb_ssd: bad sizes heads=%d groups=%d state=%d vdim=%d (state up to 2048)", H, G, N, P);
    GB_REQUIRE(scratch && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0, "gb_ssd: scratch missing or misaligned");
    if (B == 0 || T == 0) return 0;
    SsdPrepParams pp;
    pp.rows = gb_linear_walk_rows(scratch, T, H, N, P, true);
    pp.x = x; pp.bm = bm; pp.cm = cm; pp.dt = dt; pp.dt_bias = dt_bias; pp.a_log = a_log; pp.skip = skip;
    pp.ld = ld; pp.ld_dt = ld_dt; pp.dtype = dtype; pp.dt_dtype = dt_dtype; pp.w_dtype = w_dtype;
    pp.H = H; pp.G = G; pp.N = N; pp.P = P;
    ssd_prep_kernel<<<dim3(T, (H + 3) / 4), 128, 0, stream>>>(pp);
    GB_LAUNCH_OK("gb_ssd (prepare)");
    return gb_linear_walk_launch(pp.rows, false, state, out, ldo, cu, slots, qlens, B, H, N, P, max_qlen, seg_scratch, stream, "gb_ssd");
}
