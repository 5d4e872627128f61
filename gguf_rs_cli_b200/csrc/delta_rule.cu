// The pieces of a gated delta-rule mixer with one decay per head and key channel:
//   1. a short causal convolution over time per channel, followed by SiLU, whose last inputs
//      are carried from step to step per sequence;
//   2. the recurrence itself, state in 32-bit;
//   3. the per-head RMS norm of what the recurrence reads out, times a weight and a sigmoid gate.
// Everything that enters the recurrence is computed in 32-bit from the projections' outputs:
// unit vectors, decays (exponentials, softplus), the write strength, the state.
#include <math.h>

#include "common.cuh"

// ------------------------------------------------- short convolution + SiLU
// out[t, c] = silu(sum_j taps[c, j] * in[t - (K-1-j), c]); rows before the step's first token come from
// the sequence's carried inputs state[slot, 0..K-2, c] (oldest first; zero for a sequence that starts).
// blockIdx.x is the token, blockIdx.y a slice of blockDim.x channels.  Padding tokens (seq_of < 0) give zeros.
__global__ void short_conv_silu_kernel(const void* __restrict__ xin, int dtype, long long ldx, int C, int K,
                                       const void* __restrict__ taps, int taps_dtype, const float* __restrict__ state,
                                       const int* __restrict__ seq_of, const int* __restrict__ cu,
                                       const int* __restrict__ slots, void* __restrict__ out, long long ldo,
                                       const void* __restrict__ bias, int act) {
    const int t = blockIdx.x;
    const int b = seq_of[t];
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    if (b < 0) {
        gb_store(out, dtype, size_t(t) * ldo + c, 0.f);
        return;
    }
    const int first = cu[b], i = t - first, slot = slots[b];
    const float* st = state + size_t(slot) * (K - 1) * C;
    {
        float acc = 0.f;
        for (int j = 0; j < K; ++j) {
            const int src = i - (K - 1 - j);
            const float xv = src >= 0 ? gb_load(xin, dtype, size_t(first + src) * ldx + c)
                                      : st[size_t(K - 1 + src) * C + c];
            acc = fmaf(xv, gb_load(taps, taps_dtype, size_t(c) * K + j), acc);
        }
        if (bias) acc += gb_load(bias, taps_dtype, c);
        gb_store(out, dtype, size_t(t) * ldo + c, act ? acc / (1.f + expf(-acc)) : acc);
    }
}

// The same for bfloat16 rows that start on 16 bytes: a thread takes 8 neighbouring channels with 16-byte loads
// and stores; taps_t [K, C] holds the taps tap by tap.  The products are added in the same order as above.
__device__ __forceinline__ void conv_unpack8(uint4 raw, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 v = __bfloat1622float2(h[e]);
        f[2 * e] = v.x;
        f[2 * e + 1] = v.y;
    }
}

__global__ void __launch_bounds__(128) short_conv_silu_vec_kernel(
        const __nv_bfloat16* __restrict__ xin, long long ldx, int C, int K, const __nv_bfloat16* __restrict__ taps_t,
        const float* __restrict__ state, const int* __restrict__ seq_of, const int* __restrict__ cu,
        const int* __restrict__ slots, __nv_bfloat16* __restrict__ out, long long ldo, const __nv_bfloat16* __restrict__ bias,
        int act) {
    const int t = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int b = seq_of[t];
    uint4* dst = reinterpret_cast<uint4*>(out + size_t(t) * ldo + c);
    if (b < 0) {
        *dst = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const int first = cu[b], i = t - first, slot = slots[b];
    const float* st = state + size_t(slot) * (K - 1) * C;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int j = 0; j < K; ++j) {
        const int src = i - (K - 1 - j);
        float xv[8], tw[8];
        if (src >= 0) {
            conv_unpack8(*reinterpret_cast<const uint4*>(xin + size_t(first + src) * ldx + c), xv);
        } else {
            const float4* sp = reinterpret_cast<const float4*>(st + size_t(K - 1 + src) * C + c);
            const float4 lo = sp[0], hi = sp[1];
            xv[0] = lo.x; xv[1] = lo.y; xv[2] = lo.z; xv[3] = lo.w; xv[4] = hi.x; xv[5] = hi.y; xv[6] = hi.z; xv[7] = hi.w;
        }
        conv_unpack8(*reinterpret_cast<const uint4*>(taps_t + size_t(j) * C + c), tw);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(xv[e], tw[e], acc[e]);
    }
    if (bias) {
        float bv[8];
        conv_unpack8(*reinterpret_cast<const uint4*>(bias + c), bv);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += bv[e];
    }
    if (act) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = acc[e] / (1.f + expf(-acc[e]));
    }
    uint4 packed;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    *dst = packed;
}

// After the convolution: the sequence's carried inputs become the last K-1 inputs including this step's.
// blockIdx.x is the sequence, blockIdx.y a slice of channels; a thread owns a channel, reads all it needs and
// then writes.
constexpr int CONV_MAX_TAPS = 16;

__global__ void short_conv_carry_kernel(const void* __restrict__ xin, int dtype, long long ldx, int C, int K,
                                        float* __restrict__ state, const int* __restrict__ cu,
                                        const int* __restrict__ slots, const int* __restrict__ qlens) {
    const int b = blockIdx.x;
    const int slot = slots[b], n = qlens[b];
    if (slot < 0 || n <= 0) return;
    const int first = cu[b];
    float* st = state + size_t(slot) * (K - 1) * C;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c < C) {
        float keep[CONV_MAX_TAPS - 1];
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
            if (j < K - 1) {
                const int src = n - (K - 1) + j;
                keep[j] = src >= 0 ? gb_load(xin, dtype, size_t(first + src) * ldx + c) : st[size_t(j + n) * C + c];
            }
        }
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
            if (j < K - 1) st[size_t(j) * C + c] = keep[j];
    }
}

// xin: [T, C] with pitch ldx (the projections' outputs); taps [C, K], last column on the current token;
// state f32 [slots, K-1, C]; out [T, C] with pitch ldo, same dtype as xin.  The carried inputs are renewed.
// taps_t (optional): the taps again as bfloat16 [K, C], for the kernel of 16-byte accesses.
// bias [C] (optional, of the taps' dtype) is added to the sum; act 1: SiLU follows, 0: nothing does.
GB_API int gb_short_conv(const void* xin, int dtype, long long ldx, int T, int B, int C, int K, const void* taps,
                         int taps_dtype, const void* taps_t, const void* bias, int act, float* state, const int* seq_of,
                         const int* cu, const int* slots, const int* qlens, void* out, long long ldo, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(taps_dtype), "gb_short_conv: bad dtype");
    GB_REQUIRE(C > 0 && K >= 1 && K <= CONV_MAX_TAPS && ldx >= C && ldo >= C, "gb_short_conv: bad sizes C=%d taps=%d (1..%d)",
               C, K, CONV_MAX_TAPS);
    GB_REQUIRE(K == 1 || state, "gb_short_conv: a convolution of %d taps needs the carried inputs", K);
    GB_REQUIRE(act == 0 || act == 1, "gb_short_conv: unknown activation %d", act);
    if (T == 0) return 0;
    const int threads = 128, slices = (C + threads - 1) / threads;
    GB_REQUIRE(slices <= 65535, "gb_short_conv: too many channels (%d)", C);
    auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    if (taps_t && dtype == GB_BF16 && C % 8 == 0 && ldx % 8 == 0 && ldo % 8 == 0 && aligned16(xin) && aligned16(out) &&
        aligned16(taps_t) && (K == 1 || (reinterpret_cast<uintptr_t>(state) & 31) == 0) &&
        (!bias || (taps_dtype == GB_BF16 && aligned16(bias)))) {
        short_conv_silu_vec_kernel<<<dim3(T, (C / 8 + threads - 1) / threads), threads, 0, stream>>>(
            (const __nv_bfloat16*)xin, ldx, C, K, (const __nv_bfloat16*)taps_t, state, seq_of, cu, slots, (__nv_bfloat16*)out, ldo,
            (const __nv_bfloat16*)bias, act);
    } else {
        short_conv_silu_kernel<<<dim3(T, slices), threads, 0, stream>>>(xin, dtype, ldx, C, K, taps, taps_dtype, state, seq_of, cu,
                                                                       slots, out, ldo, bias, act);
    }
    GB_LAUNCH_OK("gb_short_conv");
    if (K > 1 && B > 0) {
        short_conv_carry_kernel<<<dim3(B, slices), threads, 0, stream>>>(xin, dtype, ldx, C, K, state, cu, slots, qlens);
        GB_LAUNCH_OK("gb_short_conv (carry)");
    }
    return 0;
}

// The convolution followed by SiLU, without a bias.
GB_API int gb_short_conv_silu(const void* xin, int dtype, long long ldx, int T, int B, int C, int K, const void* taps,
                              int taps_dtype, const void* taps_t, float* state, const int* seq_of, const int* cu,
                              const int* slots, const int* qlens, void* out, long long ldo, cudaStream_t stream) {
    return gb_short_conv(xin, dtype, ldx, T, B, C, K, taps, taps_dtype, taps_t, nullptr, 1, state, seq_of, cu, slots, qlens, out,
                         ldo, stream);
}

// ------------------------------------------------------------ the recurrence
// Per sequence and head, with S [D, Dv] (key channel i, value column j), for every token in order:
//   qn = q / sqrt(sum q^2 + 1e-6) * q_scale,  kn = k / sqrt(sum k^2 + 1e-6)
//   decay_i = exp(-exp(A_log_h) * softplus(a_i + dt_bias_i)),  beta = sigmoid(b)
//   S_ij <- decay_i S_ij;  u_j = beta (v_j - sum_i S_ij kn_i);  S_ij <- S_ij + kn_i u_j;  o_j = sum_i S_ij qn_i
// Two kernels.  The first computes, for all tokens at once, what does not depend on the state: qn and kn per
// q/k head, decays and beta per head, and the values as 32-bit floats, in rows padded to a multiple of four
// entries.  The second walks the tokens.  Columns of S do not interact, so a block takes a slice of columns
// of one (sequence, head): a column is shared by R lanes of a warp (R a power of two), lane r holding the NR
// rows r*NR .. r*NR + NR - 1 in registers; the sums over i end with shuffles over those lanes.  The prepared
// rows of a few tokens at a time are copied into shared memory with cp.async, the next chunk while this one
// is worked on; a lane's share of a row lies NR + 4 floats after its neighbour's, so that 16-byte reads of
// different lanes fall into different banks.  The state is read once at the start and written once at the end.
struct DeltaPrepParams {
    const void *q, *k, *v;          // after convolution and SiLU: q, k [T, G*D], v [T, H*Dv], rows `ld` apart
    const void* beta;               // [T, H] before the sigmoid, rows ld_beta apart
    const void* a;                  // [T, H*D] before bias and softplus, rows ld_a apart
    const void *dt_bias, *A_log;    // [H*D], [H]
    float* qk;                      // [T, G, 2, DA]: qn, kn
    float* gb;                      // [T, H, DA + 4]: decays, then beta
    float* vf;                      // [T, H, VA]
    long long ld, ld_beta, ld_a;
    int dtype, w_dtype, H, G, D, Dv, DA, VA;
    float q_scale;
};

// One warp per item: items 0..H-1 are the heads (decays, beta, values), items H..H+G-1 the q/k heads.
__global__ void __launch_bounds__(128) delta_prep_kernel(const DeltaPrepParams p) {
    const int t = blockIdx.x, item = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= p.H + p.G) return;
    const int D = p.D, DA = p.DA;
    if (item < p.H) {
        const int h = item;
        const float rate = expf(gb_load(p.A_log, p.w_dtype, h));
        float* g = p.gb + (size_t(t) * p.H + h) * (DA + 4);
        for (int d = lane; d < DA; d += 32) {
            float gv = 0.f;
            if (d < D) {
                const float z = gb_load(p.a, p.dtype, size_t(t) * p.ld_a + size_t(h) * D + d) +
                                gb_load(p.dt_bias, p.w_dtype, size_t(h) * D + d);
                gv = expf(-rate * (z > 20.f ? z : log1pf(expf(z))));
            }
            g[d] = gv;
        }
        if (lane < 4) g[DA + lane] = lane == 0 ? 1.f / (1.f + expf(-gb_load(p.beta, p.dtype, size_t(t) * p.ld_beta + h))) : 0.f;
        float* vo = p.vf + (size_t(t) * p.H + h) * p.VA;
        for (int d = lane; d < p.VA; d += 32) vo[d] = d < p.Dv ? gb_load(p.v, p.dtype, size_t(t) * p.ld + size_t(h) * p.Dv + d) : 0.f;
    } else {
        const int g = item - p.H;
        const size_t row = size_t(t) * p.ld + size_t(g) * D;
        float sq = 0.f, sk = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float qv = gb_load(p.q, p.dtype, row + d), kv = gb_load(p.k, p.dtype, row + d);
            sq = fmaf(qv, qv, sq);
            sk = fmaf(kv, kv, sk);
        }
        const float qn = p.q_scale / sqrtf(gb_warp_sum(sq) + 1e-6f), kn = 1.f / sqrtf(gb_warp_sum(sk) + 1e-6f);
        float* o = p.qk + (size_t(t) * p.G + g) * 2 * DA;
        for (int d = lane; d < DA; d += 32) {
            o[d] = d < D ? gb_load(p.q, p.dtype, row + d) * qn : 0.f;
            o[DA + d] = d < D ? gb_load(p.k, p.dtype, row + d) * kn : 0.f;
        }
    }
}

struct DeltaRuleParams {
    const float *qk, *gb, *vf;      // what delta_prep_kernel wrote
    float* state;                   // [slots, H, D, Dv]
    float* out;                     // [T, H*Dv], rows ldo apart
    const int *cu, *slots, *qlens;
    long long ldo;
    int H, G, D, Dv, DA, VA, R, TC;
};

__device__ __forceinline__ void dr_cp16(float* dst, const float* src) {
    unsigned d = unsigned(__cvta_generic_to_shared(dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

template <int NR>
__global__ void __launch_bounds__(128) delta_rule_kernel(const DeltaRuleParams p) {
    extern __shared__ __align__(16) float sm[];
    const int b = blockIdx.x, h = blockIdx.y;
    const int slot = p.slots[b], n = p.qlens[b];
    if (slot < 0 || n <= 0) return;
    const int R = p.R, CW = 32 / R, CB = 4 * CW, D = p.D, Dv = p.Dv, DA = p.DA, TC = p.TC;
    const int RS = R * (NR + 4);                        // floats of one padded row of q, k or decays
    const int TOK = 3 * RS + 4 + CB;                    // floats per token: q, k, decays, beta (+3), values of the slice
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane / CW, jj = lane - r * CW;
    const int col0 = blockIdx.z * CB;
    const int j = col0 + warp * CW + jj;
    const bool col_ok = j < Dv;
    const int g = h / (p.H / p.G);
    float* sp = p.state + (size_t(slot) * p.H + h) * size_t(D) * Dv;
    float S[NR];
#pragma unroll
    for (int m = 0; m < NR; ++m) {
        const int i = r * NR + m;
        S[m] = (i < D && col_ok) ? sp[size_t(i) * Dv + j] : 0.f;
    }
    for (int i = threadIdx.x; i < 2 * TC * TOK; i += 128) sm[i] = 0.f;      // what no copy reaches stays zero
    __syncthreads();
    const int t0 = p.cu[b];
    const int q4 = DA / 4, v4 = max(0, min(CB, p.VA - col0)) / 4;         // 16-byte pieces per row
    auto load_chunk = [&](int c0, int buf) {
        const int nt = min(TC, n - c0);
        float* base = sm + buf * TC * TOK;
        const int per = 3 * q4 + 1 + v4;
        for (int idx = threadIdx.x; idx < nt * per; idx += 128) {
            const int tt = idx / per, e = idx - tt * per;
            const size_t t = size_t(t0 + c0 + tt);
            float* row = base + tt * TOK;
            if (e < 2 * q4) {
                const int which = e / q4, k4 = e - which * q4, i = 4 * k4;
                dr_cp16(row + which * RS + (i / NR) * (NR + 4) + (i % NR), p.qk + ((t * p.G + g) * 2 + which) * DA + i);
            } else if (e < 3 * q4) {
                const int i = 4 * (e - 2 * q4);
                dr_cp16(row + 2 * RS + (i / NR) * (NR + 4) + (i % NR), p.gb + (t * p.H + h) * (DA + 4) + i);
            } else if (e == 3 * q4) {
                dr_cp16(row + 3 * RS, p.gb + (t * p.H + h) * (DA + 4) + DA);
            } else {
                const int i = 4 * (e - 3 * q4 - 1);
                dr_cp16(row + 3 * RS + 4 + i, p.vf + (t * p.H + h) * p.VA + col0 + i);
            }
        }
    };
    load_chunk(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    int buf = 0;
    for (int c0 = 0; c0 < n; c0 += TC, buf ^= 1) {
        const int nt = min(TC, n - c0);
        if (c0 + TC < n) load_chunk(c0 + TC, buf ^ 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const float* base = sm + buf * TC * TOK;
        for (int tt = 0; tt < nt; ++tt) {
            const float* row = base + tt * TOK;
            const float4* qq = reinterpret_cast<const float4*>(row + r * (NR + 4));
            const float4* kk = reinterpret_cast<const float4*>(row + RS + r * (NR + 4));
            const float4* gg = reinterpret_cast<const float4*>(row + 2 * RS + r * (NR + 4));
            float4 kr[NR / 4];
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
            for (int m = 0; m < NR / 4; ++m) {
                const float4 gv = gg[m];
                kr[m] = kk[m];
                S[4 * m] *= gv.x;     d0 = fmaf(S[4 * m], kr[m].x, d0);
                S[4 * m + 1] *= gv.y; d1 = fmaf(S[4 * m + 1], kr[m].y, d1);
                S[4 * m + 2] *= gv.z; d2 = fmaf(S[4 * m + 2], kr[m].z, d2);
                S[4 * m + 3] *= gv.w; d3 = fmaf(S[4 * m + 3], kr[m].w, d3);
            }
            float dot = (d0 + d1) + (d2 + d3);
            for (int off = CW; off < 32; off <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
            const float u = row[3 * RS] * (row[3 * RS + 4 + warp * CW + jj] - dot);
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int m = 0; m < NR / 4; ++m) {
                const float4 qv = qq[m];
                S[4 * m] = fmaf(kr[m].x, u, S[4 * m]);         o0 = fmaf(S[4 * m], qv.x, o0);
                S[4 * m + 1] = fmaf(kr[m].y, u, S[4 * m + 1]); o1 = fmaf(S[4 * m + 1], qv.y, o1);
                S[4 * m + 2] = fmaf(kr[m].z, u, S[4 * m + 2]); o2 = fmaf(S[4 * m + 2], qv.z, o2);
                S[4 * m + 3] = fmaf(kr[m].w, u, S[4 * m + 3]); o3 = fmaf(S[4 * m + 3], qv.w, o3);
            }
            float o = (o0 + o1) + (o2 + o3);
            for (int off = CW; off < 32; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
            if (r == 0 && col_ok) p.out[size_t(t0 + c0 + tt) * p.ldo + size_t(h) * Dv + j] = o;
        }
        __syncthreads();                                   // this buffer is loaded again two chunks on
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int m = 0; m < NR; ++m) {
        const int i = r * NR + m;
        if (i < D && col_ok) sp[size_t(i) * Dv + j] = S[m];
    }
}

// Rows per lane and lanes per column for key size D: 8 rows a lane up to D = 32, 16 up to 64, 32 up to 1024, 64
// beyond.  The walk is bound by latency (a prompt of 2,048 tokens, 16 heads of 128 x 128: 1.26 ms with 32 rows a
// lane, 64 blocks and one warp per scheduler issuing 28% of the time; 1.32 ms with 8 rows a lane and 256 blocks,
// whose blocks each repeat the copies and the shuffles: three times the instructions for the same time).
static void delta_rule_shape(int D, int* nr, int* r) {
    int NR = D > 1024 ? 64 : D > 64 ? 32 : D > 32 ? 16 : 8, R = 1;
    while (R * NR < D) R <<= 1;
    *nr = NR;
    *r = R;
}

// Floats of scratch for the prepared rows of T tokens: qk, gb and vf one after the other.
GB_API long long gb_delta_rule_scratch_floats(int T, int H, int G, int D, int Dv) {
    const long long DA = (D + 3) / 4 * 4, VA = (Dv + 3) / 4 * 4;
    return (long long)T * (G * 2 * DA + H * (DA + 4) + H * VA);
}

GB_API int gb_delta_rule(const void* q, const void* k, const void* v, int dtype, long long ld, const void* beta,
                         long long ld_beta, const void* a, long long ld_a, const void* dt_bias, const void* A_log,
                         int w_dtype, float* state, float* out, long long ldo, const int* cu, const int* slots,
                         const int* qlens, int T, int B, int H, int G, int D, int Dv, float q_scale, float* scratch,
                         cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(w_dtype), "gb_delta_rule: bad dtype");
    GB_REQUIRE(H > 0 && G > 0 && H % G == 0 && D > 0 && Dv > 0, "gb_delta_rule: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d", H, G, D, Dv);
    GB_REQUIRE(D <= 2048, "gb_delta_rule: key size %d exceeds 2048", D);
    GB_REQUIRE(H + G <= 4 * 65535, "gb_delta_rule: too many heads (%d)", H);
    GB_REQUIRE(scratch && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0, "gb_delta_rule: scratch missing or misaligned");
    if (B == 0 || T == 0) return 0;
    const int DA = (D + 3) / 4 * 4, VA = (Dv + 3) / 4 * 4;
    DeltaPrepParams pp;
    pp.q = q; pp.k = k; pp.v = v; pp.beta = beta; pp.a = a; pp.dt_bias = dt_bias; pp.A_log = A_log;
    pp.qk = scratch;
    pp.gb = pp.qk + size_t(T) * G * 2 * DA;
    pp.vf = pp.gb + size_t(T) * H * (DA + 4);
    pp.ld = ld; pp.ld_beta = ld_beta; pp.ld_a = ld_a; pp.dtype = dtype; pp.w_dtype = w_dtype;
    pp.H = H; pp.G = G; pp.D = D; pp.Dv = Dv; pp.DA = DA; pp.VA = VA; pp.q_scale = q_scale;
    delta_prep_kernel<<<dim3(T, (H + G + 3) / 4), 128, 0, stream>>>(pp);
    GB_LAUNCH_OK("gb_delta_rule (prepare)");
    DeltaRuleParams p;
    p.qk = pp.qk; p.gb = pp.gb; p.vf = pp.vf; p.state = state; p.out = out; p.cu = cu; p.slots = slots; p.qlens = qlens;
    p.ldo = ldo; p.H = H; p.G = G; p.D = D; p.Dv = Dv; p.DA = DA; p.VA = VA;
    int NR, R;
    delta_rule_shape(D, &NR, &R);
    const int CB = 4 * (32 / R);
    const int per_token = 4 * (3 * R * (NR + 4) + 4 + CB);
    int TC = (20 * 1024) / per_token;                    // two buffers of at most 20 KB each
    TC = TC < 1 ? 1 : (TC > 16 ? 16 : TC);
    p.R = R; p.TC = TC;
    const size_t smem = size_t(2) * TC * per_token;
    GB_REQUIRE(smem <= 64 * 1024, "gb_delta_rule: key size %d needs %zu bytes of shared memory", D, smem);
    if (smem > 48 * 1024) {                              // only the widest shape (64 rows a lane, 32 lanes a column)
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(delta_rule_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess)
                return gb_fail("gb_delta_rule: cannot get %zu bytes of shared memory", smem);
            configured = true;
        }
    }
    dim3 grid(B, H, (Dv + CB - 1) / CB);
    GB_REQUIRE(grid.z <= 65535 && H <= 65535, "gb_delta_rule: too many heads or value columns");
    if (NR == 8) delta_rule_kernel<8><<<grid, 128, smem, stream>>>(p);
    else if (NR == 16) delta_rule_kernel<16><<<grid, 128, smem, stream>>>(p);
    else if (NR == 32) delta_rule_kernel<32><<<grid, 128, smem, stream>>>(p);
    else delta_rule_kernel<64><<<grid, 128, smem, stream>>>(p);
    GB_LAUNCH_OK("gb_delta_rule");
    return 0;
}

// --------------------------------------------- per-head RMS norm, weight, gate
// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * w[:] * f(gate[t, h, :]); one warp per
// (token, head); w [Dv] is shared by the heads, or every head has its own (w_per_head: w [H, Dv]).
// f: 0 the sigmoid, 1 SiLU (z sigmoid(z)).  gate_first: the gate comes before the norm,
// out = y / sqrt(mean(y^2) + eps) * w with y = o f(gate).
__global__ void gated_head_norm_kernel(const float* __restrict__ o, long long ldo, const void* __restrict__ gate,
                                       int gate_dtype, long long ldg, const void* __restrict__ w, int w_dtype, float eps,
                                       void* __restrict__ out, int out_dtype, long long ld_out, long long items, int H, int Dv,
                                       int gate_act, int w_per_head, int gate_first) {
    const long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int lane = threadIdx.x & 31;
    const long long t = item / H;
    const int h = int(item - t * H);
    const float* orow = o + t * ldo + size_t(h) * Dv;
    const size_t wrow = w_per_head ? size_t(h) * Dv : 0;
    float ss = 0.f;
    if (gate_first) {
        for (int d = lane; d < Dv; d += 32) {
            const float gt = gb_load(gate, gate_dtype, size_t(t) * ldg + size_t(h) * Dv + d);
            const float y = orow[d] * ((gate_act ? gt : 1.f) / (1.f + expf(-gt)));
            ss = fmaf(y, y, ss);
        }
        const float rms = sqrtf(gb_warp_sum(ss) / float(Dv) + eps);
        for (int d = lane; d < Dv; d += 32) {
            const float gt = gb_load(gate, gate_dtype, size_t(t) * ldg + size_t(h) * Dv + d);
            const float y = orow[d] * ((gate_act ? gt : 1.f) / (1.f + expf(-gt)));
            gb_store(out, out_dtype, size_t(t) * ld_out + size_t(h) * Dv + d, y / rms * gb_load(w, w_dtype, wrow + d));
        }
        return;
    }
    for (int d = lane; d < Dv; d += 32) ss = fmaf(orow[d], orow[d], ss);
    const float rms = sqrtf(gb_warp_sum(ss) / float(Dv) + eps);
    for (int d = lane; d < Dv; d += 32) {
        const float gt = gb_load(gate, gate_dtype, size_t(t) * ldg + size_t(h) * Dv + d);
        gb_store(out, out_dtype, size_t(t) * ld_out + size_t(h) * Dv + d,
                 orow[d] / rms * gb_load(w, w_dtype, wrow + d) * ((gate_act ? gt : 1.f) / (1.f + expf(-gt))));
    }
}

// The same for long heads (a norm over a whole row in one or a few parts): one block per (token, head).
__global__ void __launch_bounds__(1024) gated_head_norm_block_kernel(const float* __restrict__ o, long long ldo, const void* __restrict__ gate,
                                                                    int gate_dtype, long long ldg, const void* __restrict__ w, int w_dtype,
                                                                    float eps, void* __restrict__ out, int out_dtype, long long ld_out, int H,
                                                                    int Dv, int gate_act, int w_per_head, int gate_first) {
    __shared__ float red[32];
    const long long t = blockIdx.x / H;
    const int h = int(blockIdx.x - t * H);
    const float* orow = o + t * ldo + size_t(h) * Dv;
    const size_t grow = size_t(t) * ldg + size_t(h) * Dv, wrow = w_per_head ? size_t(h) * Dv : 0;
    float ss = 0.f;
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        float y = orow[d];
        if (gate_first) {
            const float gt = gb_load(gate, gate_dtype, grow + d);
            y *= (gate_act ? gt : 1.f) / (1.f + expf(-gt));
        }
        ss = fmaf(y, y, ss);
    }
    ss = gb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
    const float rms = sqrtf(tot / float(Dv) + eps);
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        const float gt = gb_load(gate, gate_dtype, grow + d);
        const float f = (gate_act ? gt : 1.f) / (1.f + expf(-gt));
        const float wv = gb_load(w, w_dtype, wrow + d);
        gb_store(out, out_dtype, size_t(t) * ld_out + size_t(h) * Dv + d, gate_first ? orow[d] * f / rms * wv : orow[d] / rms * wv * f);
    }
}

GB_API int gb_gated_head_norm(const float* o, long long ldo, const void* gate, int gate_dtype, long long ldg, const void* w,
                              int w_dtype, float eps, void* out, int out_dtype, long long ld_out, int T, int H, int Dv,
                              int gate_act, int w_per_head, int gate_first, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(gate_dtype) && gb_is_dtype(w_dtype) && gb_is_dtype(out_dtype), "gb_gated_head_norm: bad dtype");
    GB_REQUIRE(H > 0 && Dv > 0 && eps > 0.f, "gb_gated_head_norm: bad sizes heads=%d vdim=%d eps=%g", H, Dv, eps);
    GB_REQUIRE(gate_act == 0 || gate_act == 1, "gb_gated_head_norm: unknown gate function %d", gate_act);
    if (T == 0) return 0;
    const long long items = (long long)T * H;
    if (Dv >= 1024 && items <= 0x7fffffffLL) {
        gated_head_norm_block_kernel<<<unsigned(items), Dv >= 4096 ? 1024 : Dv >= 2048 ? 512 : 256, 0, stream>>>(o, ldo, gate, gate_dtype, ldg, w, w_dtype, eps, out, out_dtype,
                                                                          ld_out, H, Dv, gate_act, w_per_head, gate_first);
        GB_LAUNCH_OK("gb_gated_head_norm");
        return 0;
    }
    gated_head_norm_kernel<<<unsigned((items + 3) / 4), 128, 0, stream>>>(o, ldo, gate, gate_dtype, ldg, w, w_dtype, eps, out,
                                                                          out_dtype, ld_out, items, H, Dv, gate_act, w_per_head, gate_first);
    GB_LAUNCH_OK("gb_gated_head_norm");
    return 0;
}
