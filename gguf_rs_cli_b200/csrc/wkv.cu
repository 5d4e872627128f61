// The pieces of a mixer in the manner of RWKV's time mixing with a decay per head and key channel that depends on the token:
//   1. the token shift: every projection reads its own blend of the token's row and the row of the token before it,
//      h + (h_before - h) mu_s; the last row of a sequence is carried from step to step;
//   2. the preparation of the walk over tokens (linear_walk.h): r, k, v as 32-bit rows, the decays
//      w = exp(-exp(a + w0)) from the low-rank pair's result a, and the current token's bonus sum_i u_i k_i r_i, whose
//      product with v is what (S + diag(u) k v^T)^T r adds to S^T r;
//   3. the walk itself, reading the state before the token's own update: o = S^T r + bonus v, S <- diag(w) S + k v^T.
// Decays, their exponentials, the bonus and the state are 32-bit.
#include <math.h>

#include "common.cuh"
#include "linear_walk.h"

// blockIdx.x is the token, blockIdx.y a slice of blockDim.x entries of its row.  out holds n_mix blends [T, E] one after the other (mix_stride elements apart); mu [n_mix, E].
// The block of a sequence's first token of the step reads the carried row and then replaces it with the step's last.
__global__ void __launch_bounds__(256) token_shift_mix_kernel(const void* __restrict__ h, int dtype, long long ldh, int E,
                                                              const void* __restrict__ mu, int mu_dtype, int n_mix,
                                                              float* __restrict__ carried, const int* __restrict__ seq_of,
                                                              const int* __restrict__ cu, const int* __restrict__ slots,
                                                              const int* __restrict__ qlens, void* __restrict__ out,
                                                              long long mix_stride) {
    const int t = blockIdx.x, b = seq_of[t];
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i >= E) return;
    if (b < 0) {
        for (int s = 0; s < n_mix; ++s) gb_store(out, dtype, size_t(s) * mix_stride + size_t(t) * E + i, 0.f);
        return;
    }
    const int first = cu[b], slot = slots[b];
    const bool head = t == first;
    float* keep = carried + size_t(slot) * E;
    const size_t last = size_t(first + qlens[b] - 1) * ldh;
    {
        const float cur = gb_load(h, dtype, size_t(t) * ldh + i);
        float before;
        if (head) {
            before = keep[i];
            keep[i] = gb_load(h, dtype, last + i);
        } else {
            before = gb_load(h, dtype, size_t(t - 1) * ldh + i);
        }
        const float d = before - cur;
        for (int s = 0; s < n_mix; ++s)
            gb_store(out, dtype, size_t(s) * mix_stride + size_t(t) * E + i, fmaf(d, gb_load(mu, mu_dtype, size_t(s) * E + i), cur));
    }
}

// The same for bfloat16 rows whose length and distance are multiples of 8: a thread takes 8 neighbouring entries with
// 16-byte loads and stores (one entry a thread moves 0.25 of the copy bandwidth, this 0.6).
__device__ __forceinline__ void ts_unpack8(const uint4& raw, float* f) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(p[j]);
        f[2 * j] = a.x;
        f[2 * j + 1] = a.y;
    }
}

__global__ void __launch_bounds__(128) token_shift_mix_vec_kernel(const __nv_bfloat16* __restrict__ h, long long ldh, int E,
                                                                  const __nv_bfloat16* __restrict__ mu, int n_mix,
                                                                  float* __restrict__ carried, const int* __restrict__ seq_of,
                                                                  const int* __restrict__ cu, const int* __restrict__ slots,
                                                                  const int* __restrict__ qlens, __nv_bfloat16* __restrict__ out,
                                                                  long long mix_stride) {
    const int t = blockIdx.x, b = seq_of[t];
    const int i = 8 * (blockIdx.y * blockDim.x + threadIdx.x);
    if (i >= E) return;
    if (b < 0) {
        for (int s = 0; s < n_mix; ++s)
            *reinterpret_cast<uint4*>(out + size_t(s) * mix_stride + size_t(t) * E + i) = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const int first = cu[b];
    float cur[8], before[8];
    ts_unpack8(*reinterpret_cast<const uint4*>(h + size_t(t) * ldh + i), cur);
    if (t == first) {
        float* keep = carried + size_t(slots[b]) * E + i;
        float last[8];
        ts_unpack8(*reinterpret_cast<const uint4*>(h + size_t(first + qlens[b] - 1) * ldh + i), last);
        const float4 k0 = *reinterpret_cast<const float4*>(keep), k1 = *reinterpret_cast<const float4*>(keep + 4);
        before[0] = k0.x; before[1] = k0.y; before[2] = k0.z; before[3] = k0.w;
        before[4] = k1.x; before[5] = k1.y; before[6] = k1.z; before[7] = k1.w;
        *reinterpret_cast<float4*>(keep) = make_float4(last[0], last[1], last[2], last[3]);
        *reinterpret_cast<float4*>(keep + 4) = make_float4(last[4], last[5], last[6], last[7]);
    } else {
        ts_unpack8(*reinterpret_cast<const uint4*>(h + size_t(t - 1) * ldh + i), before);
    }
    for (int s = 0; s < n_mix; ++s) {
        float m[8];
        ts_unpack8(*reinterpret_cast<const uint4*>(mu + size_t(s) * E + i), m);
        uint4 packed;
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            o[j] = __floats2bfloat162_rn(fmaf(before[2 * j] - cur[2 * j], m[2 * j], cur[2 * j]),
                                         fmaf(before[2 * j + 1] - cur[2 * j + 1], m[2 * j + 1], cur[2 * j + 1]));
        *reinterpret_cast<uint4*>(out + size_t(s) * mix_stride + size_t(t) * E + i) = packed;
    }
}

// h [T, E] rows ldh apart; mu [n_mix, E]; carried float32 [slots, E] (zero for a sequence that starts), read and renewed;
// out [n_mix, T, E] of h's dtype, the blends mix_stride elements apart (0: T * E; more where a caller pads them).
GB_API int gb_token_shift_mix(const void* h, int dtype, long long ldh, int T, int E, const void* mu, int mu_dtype, int n_mix,
                              float* carried, const int* seq_of, const int* cu, const int* slots, const int* qlens, void* out,
                              long long mix_stride, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(mu_dtype), "gb_token_shift_mix: bad dtype");
    if (mix_stride == 0) mix_stride = (long long)T * E;
    GB_REQUIRE(mix_stride >= (long long)T * E, "gb_token_shift_mix: blends %lld elements apart overlap", mix_stride);
    GB_REQUIRE(E > 0 && n_mix > 0 && ldh >= E && carried, "gb_token_shift_mix: bad sizes E=%d blends=%d", E, n_mix);
    if (T == 0) return 0;
    GB_REQUIRE((E + 255) / 256 <= 65535, "gb_token_shift_mix: rows of %d entries are too long", E);
    const auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (dtype == GB_BF16 && mu_dtype == GB_BF16 && E % 8 == 0 && ldh % 8 == 0 && aligned16(h) && aligned16(mu) && aligned16(out) &&
        aligned16(carried) && mix_stride % 8 == 0) {
        token_shift_mix_vec_kernel<<<dim3(T, (E / 8 + 127) / 128), 128, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(h), ldh, E, static_cast<const __nv_bfloat16*>(mu), n_mix, carried, seq_of, cu, slots,
            qlens, static_cast<__nv_bfloat16*>(out), mix_stride);
        GB_LAUNCH_OK("gb_token_shift_mix");
        return 0;
    }
    token_shift_mix_kernel<<<dim3(T, (E + 255) / 256), 256, 0, stream>>>(h, dtype, ldh, E, mu, mu_dtype, n_mix, carried, seq_of, cu, slots, qlens, out,
                                                  mix_stride);
    GB_LAUNCH_OK("gb_token_shift_mix");
    return 0;
}

struct WkvPrepParams {
    const void *r, *k, *v;          // [T, H*D] each, rows ld_r, ld_k, ld_v apart
    const void* a;                  // [T, H*D]: the decay's low-rank result before w0, rows ld_a apart
    const void *w0, *u;             // [H*D]
    LinearWalkRows rows;
    long long ld_r, ld_k, ld_v, ld_a;
    int dtype, a_dtype, w_dtype, H, D;
};

// One warp per (token, head).
__global__ void __launch_bounds__(128) wkv_prep_kernel(const WkvPrepParams p) {
    const int t = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= p.H) return;
    const int D = p.D, DA = p.rows.DA, VA = p.rows.VA;
    float* o = p.rows.qkg + (size_t(t) * p.H + h) * 3 * DA;
    float* vo = p.rows.vf + (size_t(t) * p.H + h) * VA;
    const size_t col = size_t(h) * D;
    float bonus = 0.f;
    for (int d = lane; d < DA; d += 32) {
        float rv = 0.f, kv = 0.f, gv = 0.f;
        if (d < D) {
            rv = gb_load(p.r, p.dtype, size_t(t) * p.ld_r + col + d);
            kv = gb_load(p.k, p.dtype, size_t(t) * p.ld_k + col + d);
            const float z = gb_load(p.a, p.a_dtype, size_t(t) * p.ld_a + col + d) + gb_load(p.w0, p.w_dtype, col + d);
            gv = expf(-expf(z));
            bonus = fmaf(gb_load(p.u, p.w_dtype, col + d) * kv, rv, bonus);
        }
        o[d] = rv;
        o[DA + d] = kv;
        o[2 * DA + d] = gv;
    }
    for (int d = lane; d < VA; d += 32) vo[d] = d < D ? gb_load(p.v, p.dtype, size_t(t) * p.ld_v + col + d) : 0.f;
    bonus = gb_warp_sum(bonus);
    if (lane < 4) p.rows.bonus[(size_t(t) * p.H + h) * 4 + lane] = lane == 0 ? bonus : 0.f;
}

// r, k, v [T, H*D] (one dtype, unit stride along a row); a [T, H*D] the decay's projection before w0 [H*D]; u [H*D] the
// bonus; state [slots, H, D, D] float32, read and renewed; out float32 [T, H*D].  scratch: gb_linear_walk_scratch_floats.
GB_API int gb_wkv(const void* r, long long ld_r, const void* k, long long ld_k, const void* v, long long ld_v, int dtype,
                  const void* a, int a_dtype, long long ld_a, const void* w0, const void* u, int w_dtype, float* state, float* out,
                  long long ldo, const int* cu, const int* slots, const int* qlens, int T, int B, int H, int D, float* scratch,
                  int max_qlen, float* seg_scratch, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(a_dtype) && gb_is_dtype(w_dtype), "gb_wkv: bad dtype");
    GB_REQUIRE(H > 0 && D > 0 && D <= 2048 && (H + 3) / 4 <= 65535, "gb_wkv: bad sizes heads=%d dim=%d (dim up to 2048)", H, D);
    GB_REQUIRE(scratch && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0, "gb_wkv: scratch missing or misaligned");
    if (B == 0 || T == 0) return 0;
    WkvPrepParams pp;
    pp.rows = gb_linear_walk_rows(scratch, T, H, D, D, true);
    pp.r = r; pp.k = k; pp.v = v; pp.a = a; pp.w0 = w0; pp.u = u;
    pp.ld_r = ld_r; pp.ld_k = ld_k; pp.ld_v = ld_v; pp.ld_a = ld_a;
    pp.dtype = dtype; pp.a_dtype = a_dtype; pp.w_dtype = w_dtype; pp.H = H; pp.D = D;
    wkv_prep_kernel<<<dim3(T, (H + 3) / 4), 128, 0, stream>>>(pp);
    GB_LAUNCH_OK("gb_wkv (prepare)");
    return gb_linear_walk_launch(pp.rows, true, state, out, ldo, cu, slots, qlens, B, H, D, D, max_qlen, seg_scratch, stream, "gb_wkv");
}
