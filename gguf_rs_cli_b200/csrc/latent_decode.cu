// Latent attention for steps in which every sequence brings one token: all heads of a token share one key/value
// head, the cached rows [c (C entries), rotated part (R entries)], and each head's query has already been
// brought into that space (q' = W_uk^T q, then the rotated part).  score_h(j) = q_h . row_j * scale over the
// C + R entries; the mix of values is the mix of the rows' first C entries.
//
// Two kernels follow, both with one block per (token, split of the token's keys) that serves ALL heads from one
// pass over its keys; the second, on the tensor cores, is taken where its sizes fit.  The first: 32 rows at a
// time are copied into shared memory once (16-byte pieces, rows padded by 16 bytes so that lanes reading
// different rows fall into different banks) and every warp takes its heads (warp, warp + 8, ...) over them:
// lane = key for the scores, lane = pair of entries for the values.  The general kernel, with a block per
// (token, head), reads every row once per head.  Scores, softmax and mix are 32-bit.  A split leaves its
// maximum, its sum and its unnormalised mix in scratch memory; a second kernel merges the splits in split
// order, so the result does not depend on timing.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int LD_WARPS = 8;
constexpr int LD_THREADS = LD_WARPS * 32;
constexpr int LD_MAX_HEADS = 16;                    // heads per token: at most 2 per warp (with 32 heads the general
                                                    // kernel's block per head was measured faster: 0.774 against 0.799 ms a step)
constexpr int LD_HW = LD_MAX_HEADS / LD_WARPS;
constexpr int LD_MAX_C = 512;                       // entries of the value: at most 8 pairs per lane
constexpr int LD_PAIRS = LD_MAX_C / 64;

// Entries between two rows of the tile in shared memory: 16 bytes of padding, 32 where 16 would put all rows
// on the same banks.
__host__ __device__ inline int ld_row_stride(int hdk) { return (hdk + 8) % 64 ? hdk + 8 : hdk + 16; }

struct LdParams {
    const __nv_bfloat16* q;       // [T, H*(C+R)] rows ldq apart
    const __nv_bfloat16* cache;   // [pages, 1, 64, C+R]
    const int *seq_of, *pos, *table;
    float* scratch;               // [T, H, splits, C + 2]: unnormalised mix, maximum, sum
    long long ldq;
    int H, C, R, splits, table_width, ring_pages;
    float scale;
    int window;                   // > 0: a token sees the last `window` positions only
};

__global__ void __launch_bounds__(LD_THREADS) latent_decode_kernel(const LdParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int t = blockIdx.x, split = blockIdx.y;
    const int b = p.seq_of[t];
    if (b < 0) return;                                       // padding: the merge writes zeros
    const int H = p.H, C = p.C, HDK = p.C + p.R, KS = ld_row_stride(HDK);   // KS: entries of a padded row in shared memory
    float* qs = reinterpret_cast<float*>(smem_raw);                                   // [H][HDK]
    __nv_bfloat16* kt = reinterpret_cast<__nv_bfloat16*>(qs + size_t(H) * HDK);       // [32][KS]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = p.pos[t];
    const int lo = gb_first_visible(pos, p.window, 0);
    const int kbf = lo >> 5, nkb = (pos >> 5) - kbf + 1;      // blocks of 32 keys from the first one seen up to the token's own
    const int per = (nkb + p.splits - 1) / p.splits;
    const int kb0 = kbf + split * per, kb1 = min(kbf + nkb, kb0 + per);
    const int* trow = p.table + size_t(b) * p.table_width;

    for (int i = threadIdx.x; i < H * HDK; i += LD_THREADS)
        qs[i] = __bfloat162float(p.q[size_t(t) * p.ldq + i]);

    float m[LD_HW], l[LD_HW], acc[LD_HW][2 * LD_PAIRS];
#pragma unroll
    for (int hi = 0; hi < LD_HW; ++hi) {
        m[hi] = -INFINITY;
        l[hi] = 0.f;
#pragma unroll
        for (int c = 0; c < 2 * LD_PAIRS; ++c) acc[hi][c] = 0.f;
    }
    const int pieces = HDK / 8;
    for (int kb = kb0; kb < kb1; ++kb) {
        __syncthreads();                                     // the tile before has been used (and qs is written)
        for (int i = threadIdx.x; i < 32 * pieces; i += LD_THREADS) {
            const int r = i / pieces, c8 = i - r * pieces, j = kb * 32 + r;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (j <= pos && j >= lo) v = *reinterpret_cast<const uint4*>(p.cache + gb_kv_offset(trow, p.ring_pages, j, 0, 1, HDK) + 8 * c8);
            *reinterpret_cast<uint4*>(kt + r * KS + 8 * c8) = v;
        }
        __syncthreads();
        const bool valid = kb * 32 + lane <= pos && kb * 32 + lane >= lo;
#pragma unroll
        for (int hi = 0; hi < LD_HW; ++hi) {
            const int h = warp + LD_WARPS * hi;
            if (h >= H) break;
            const float* qh = qs + size_t(h) * HDK;
            const __nv_bfloat16* kr = kt + lane * KS;
            float d0 = 0.f, d1 = 0.f;
            for (int c8 = 0; c8 < pieces; ++c8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(kr + 8 * c8);
                const float4 qa = *reinterpret_cast<const float4*>(qh + 8 * c8), qb = *reinterpret_cast<const float4*>(qh + 8 * c8 + 4);
                const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
                const float2 k0 = __bfloat1622float2(k2[0]), k1 = __bfloat1622float2(k2[1]);
                const float2 k2f = __bfloat1622float2(k2[2]), k3 = __bfloat1622float2(k2[3]);
                d0 = fmaf(qa.x, k0.x, d0); d1 = fmaf(qa.y, k0.y, d1);
                d0 = fmaf(qa.z, k1.x, d0); d1 = fmaf(qa.w, k1.y, d1);
                d0 = fmaf(qb.x, k2f.x, d0); d1 = fmaf(qb.y, k2f.y, d1);
                d0 = fmaf(qb.z, k3.x, d0); d1 = fmaf(qb.w, k3.y, d1);
            }
            const float s = valid ? (d0 + d1) * p.scale : -INFINITY;
            const float m_new = fmaxf(m[hi], gb_warp_max(s));
            const float alpha = m[hi] == -INFINITY ? 0.f : expf(m[hi] - m_new);
            const float pj = valid ? expf(s - m_new) : 0.f;
            l[hi] = l[hi] * alpha + gb_warp_sum(pj);
            m[hi] = m_new;
#pragma unroll
            for (int c = 0; c < 2 * LD_PAIRS; ++c) acc[hi][c] *= alpha;
            for (int r = 0; r < 32; ++r) {
                const float pr = __shfl_sync(0xffffffffu, pj, r);
                if (pr == 0.f) continue;                     // uniform over the warp
                const __nv_bfloat162* vr = reinterpret_cast<const __nv_bfloat162*>(kt + r * KS);
#pragma unroll
                for (int cp = 0; cp < LD_PAIRS; ++cp) {
                    if (64 * cp + 2 * lane < C) {
                        const float2 vv = __bfloat1622float2(vr[32 * cp + lane]);
                        acc[hi][2 * cp] = fmaf(pr, vv.x, acc[hi][2 * cp]);
                        acc[hi][2 * cp + 1] = fmaf(pr, vv.y, acc[hi][2 * cp + 1]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int hi = 0; hi < LD_HW; ++hi) {
        const int h = warp + LD_WARPS * hi;
        if (h >= H) break;
        float* o = p.scratch + ((size_t(t) * H + h) * p.splits + split) * (C + 2);
#pragma unroll
        for (int cp = 0; cp < LD_PAIRS; ++cp) {
            const int c = 64 * cp + 2 * lane;
            if (c < C) {
                o[c] = acc[hi][2 * cp];
                o[c + 1] = acc[hi][2 * cp + 1];
            }
        }
        if (lane == 0) {
            o[C] = m[hi];
            o[C + 1] = l[hi];
        }
    }
}

// ---------------------------------------------------------------- the same on the tensor cores
// The heads of a token are the 16 rows of mma.sync m16n8k16 tiles (heads beyond H are rows of zeros).  Four
// warps: each computes all scores of the 32 keys (S = Q K^T over the C + R entries: cheap, and it spares an
// exchange), does the softmax of its two rows per thread in registers, and multiplies the weights with its own
// quarter of the value columns.  The weights stay 32-bit: each is split into three bfloat16 terms (hi + mid +
// lo = the float exactly), three products with the same V fragments, sums in 32-bit.  Scores are 32-bit sums of
// exact products of bfloat16 q and rows.  Needs (C + R) % 16 == 0 and C % 64 == 0.
constexpr int LM_THREADS = 128;
constexpr int LM_MAX_OT = LD_MAX_C / 4 / 8;          // value tiles of 8 columns per warp

__device__ __forceinline__ void lm_ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned a = unsigned(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void lm_ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned a = unsigned(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void lm_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned lm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void lm_split3(float p, float& hi, float& mid, float& lo) {
    hi = __bfloat162float(__float2bfloat16_rn(p));
    const float r1 = p - hi;
    mid = __bfloat162float(__float2bfloat16_rn(r1));
    lo = r1 - mid;
}

__global__ void __launch_bounds__(LM_THREADS) latent_decode_mma_kernel(const LdParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int t = blockIdx.x, split = blockIdx.y;
    const int b = p.seq_of[t];
    if (b < 0) return;
    const int H = p.H, C = p.C, HDK = p.C + p.R, KS = ld_row_stride(HDK);
    __nv_bfloat16* qt = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [16][KS]: the heads' queries
    __nv_bfloat16* kt = qt + 16 * KS;                                          // [32][KS]: 32 cached rows
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = p.pos[t];
    const int lo = gb_first_visible(pos, p.window, 0);
    const int kbf = lo >> 5, nkb = (pos >> 5) - kbf + 1;      // blocks of 32 keys from the first one seen up to the token's own
    const int per = (nkb + p.splits - 1) / p.splits;
    const int kb0 = kbf + split * per, kb1 = min(kbf + nkb, kb0 + per);
    const int* trow = p.table + size_t(b) * p.table_width;
    const int pieces = HDK / 8;
    for (int i = threadIdx.x; i < 16 * pieces; i += LM_THREADS) {
        const int r = i / pieces, c8 = i - r * pieces;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < H) v = *reinterpret_cast<const uint4*>(p.q + size_t(t) * p.ldq + size_t(r) * HDK + 8 * c8);
        *reinterpret_cast<uint4*>(qt + r * KS + 8 * c8) = v;
    }
    const int CW = C / 4, ot = CW / 8;                 // this warp's value columns [warp * CW, +CW): ot tiles of 8
    const float sl2 = p.scale * 1.4426950408889634f;
    float o[LM_MAX_OT][4];
#pragma unroll
    for (int i = 0; i < LM_MAX_OT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int kb = kb0; kb < kb1; ++kb) {
        __syncthreads();
        for (int i = threadIdx.x; i < 32 * pieces; i += LM_THREADS) {
            const int r = i / pieces, c8 = i - r * pieces, j = kb * 32 + r;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (j <= pos && j >= lo) v = *reinterpret_cast<const uint4*>(p.cache + gb_kv_offset(trow, p.ring_pages, j, 0, 1, HDK) + 8 * c8);
            *reinterpret_cast<uint4*>(kt + r * KS + 8 * c8) = v;
        }
        __syncthreads();
        // ---- S = Q K^T: 16 heads x 32 keys, as four tiles of 8 keys
        float s[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        for (int k = 0; k < HDK / 16; ++k) {
            unsigned qf[4];
            lm_ldmatrix_x4(qf[0], qf[1], qf[2], qf[3], qt + (lane & 15) * KS + 16 * k + 8 * (lane >> 4));
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2) {
                unsigned b0, b1, b2, b3;
                lm_ldmatrix_x4(b0, b1, b2, b3, kt + (j2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * KS + 16 * k + 8 * ((lane >> 3) & 1));
                lm_mma(s[2 * j2], qf[0], qf[1], qf[2], qf[3], b0, b1);
                lm_mma(s[2 * j2 + 1], qf[0], qf[1], qf[2], qf[3], b2, b3);
            }
        }
        // ---- mask and running softmax: this thread's rows are heads lane / 4 and lane / 4 + 8
        const int key0 = kb * 32 + 2 * (lane & 3);
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int ka = key0 + 8 * j;
            if (ka > pos || ka < lo) s[j][0] = s[j][2] = -INFINITY;
            if (ka + 1 > pos || ka + 1 < lo) s[j][1] = s[j][3] = -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);       // finite: key kb * 32 is never masked
        const float a0 = m0 == -INFINITY ? 0.f : exp2f((m0 - mn0) * sl2), a1 = m1 == -INFINITY ? 0.f : exp2f((m1 - mn1) * sl2);
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            s[j][0] = exp2f((s[j][0] - mn0) * sl2); s[j][1] = exp2f((s[j][1] - mn0) * sl2);
            s[j][2] = exp2f((s[j][2] - mn1) * sl2); s[j][3] = exp2f((s[j][3] - mn1) * sl2);
            sum0 += s[j][0] + s[j][1];
            sum1 += s[j][2] + s[j][3];
        }
        l0 = l0 * a0 + sum0;
        l1 = l1 * a1 + sum1;
        m0 = mn0;
        m1 = mn1;
#pragma unroll
        for (int i = 0; i < LM_MAX_OT; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
        // ---- O += P V over this warp's columns; the weights as three bfloat16 terms, smallest first
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            unsigned ph[4], pm[4], pl[4];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float h4[4], m4[4], l4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) lm_split3(s[2 * kk + half][e], h4[e], m4[e], l4[e]);
                ph[2 * half] = lm_pack(h4[0], h4[1]); ph[2 * half + 1] = lm_pack(h4[2], h4[3]);
                pm[2 * half] = lm_pack(m4[0], m4[1]); pm[2 * half + 1] = lm_pack(m4[2], m4[3]);
                pl[2 * half] = lm_pack(l4[0], l4[1]); pl[2 * half + 1] = lm_pack(l4[2], l4[3]);
            }
#pragma unroll
            for (int i2 = 0; i2 < LM_MAX_OT / 2; ++i2) {
                if (2 * i2 < ot) {
                    unsigned b0, b1, b2, b3;
                    lm_ldmatrix_x4_trans(b0, b1, b2, b3, kt + (kk * 16 + (lane & 15)) * KS + warp * CW + 16 * i2 + 8 * (lane >> 4));
                    lm_mma(o[2 * i2], pl[0], pl[1], pl[2], pl[3], b0, b1);
                    lm_mma(o[2 * i2 + 1], pl[0], pl[1], pl[2], pl[3], b2, b3);
                    lm_mma(o[2 * i2], pm[0], pm[1], pm[2], pm[3], b0, b1);
                    lm_mma(o[2 * i2 + 1], pm[0], pm[1], pm[2], pm[3], b2, b3);
                    lm_mma(o[2 * i2], ph[0], ph[1], ph[2], ph[3], b0, b1);
                    lm_mma(o[2 * i2 + 1], ph[0], ph[1], ph[2], ph[3], b2, b3);
                }
            }
        }
    }
    // ---- this split's unnormalised mix, maximum (in units of the exponent) and sum
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int h0 = lane >> 2, h1 = h0 + 8;
    float* o0 = p.scratch + ((size_t(t) * H + h0) * p.splits + split) * (C + 2);
    float* o1 = p.scratch + ((size_t(t) * H + h1) * p.splits + split) * (C + 2);
#pragma unroll
    for (int i = 0; i < LM_MAX_OT; ++i) {
        if (i < ot) {
            const int c = warp * CW + 8 * i + 2 * (lane & 3);
            if (h0 < H) { o0[c] = o[i][0]; o0[c + 1] = o[i][1]; }
            if (h1 < H) { o1[c] = o[i][2]; o1[c + 1] = o[i][3]; }
        }
    }
    if (warp == 0 && (lane & 3) == 0) {
        if (h0 < H) { o0[C] = m0 == -INFINITY ? -INFINITY : m0 * p.scale; o0[C + 1] = l0; }
        if (h1 < H) { o1[C] = m1 == -INFINITY ? -INFINITY : m1 * p.scale; o1[C + 1] = l1; }
    }
}

// out[t, h, :] = sum_s mix_s e^(m_s - M) / sum_s l_s e^(m_s - M), splits in order; padding tokens give zeros.  sink
// [H] (or null): the denominator also counts e^(sink_h - M), a key without a value.  gate [T, H] rows ldg apart (or
// null): the head's result is multiplied by sigmoid(gate).
__global__ void latent_decode_merge_kernel(const float* __restrict__ scratch, const int* __restrict__ seq_of,
                                           __nv_bfloat16* __restrict__ out, long long ldo, int H, int C, int splits,
                                           const float* __restrict__ sink, const __nv_bfloat16* __restrict__ gate, long long ldg) {
    const int t = blockIdx.x, h = blockIdx.y;
    __nv_bfloat16* o = out + size_t(t) * ldo + size_t(h) * C;
    if (seq_of[t] < 0) {
        for (int c = threadIdx.x; c < C; c += blockDim.x) o[c] = __float2bfloat16_rn(0.f);
        return;
    }
    const float* base = scratch + (size_t(t) * H + h) * splits * (C + 2);
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, base[size_t(s) * (C + 2) + C]);
    float L = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = base[size_t(s) * (C + 2) + C];
        if (ms != -INFINITY) L += base[size_t(s) * (C + 2) + C + 1] * expf(ms - M);
    }
    float f = 1.f;                       // what the sums are multiplied by: a sink above every score brings them down to its level
    if (sink && M != -INFINITY) {
        const float sv = sink[h];
        if (sv > M) {
            f = expf(M - sv);
            L = L * f + 1.f;
        } else {
            L += expf(sv - M);
        }
    }
    if (gate) f *= 1.f / (1.f + expf(-__bfloat162float(gate[size_t(t) * ldg + h])));
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = base[size_t(s) * (C + 2) + C];
            if (ms != -INFINITY) v += base[size_t(s) * (C + 2) + c] * expf(ms - M);
        }
        o[c] = __float2bfloat16_rn(v * f / L);
    }
}

}  // namespace

GB_API int gb_latent_decode_supported(int H, int C, int R, int q_dtype, int cache_dtype) {
    const size_t smem = size_t(H) * (C + R) * 4 + size_t(32) * ld_row_stride(C + R) * 2;
    return q_dtype == GB_BF16 && cache_dtype == GB_BF16 && H >= 1 && H <= LD_MAX_HEADS && C >= 2 && C <= LD_MAX_C && C % 2 == 0 &&
           (C + R) % 8 == 0 && smem <= 160 * 1024;
}

// The tensor-core kernel takes what the kernel above takes when also (C + R) % 16 == 0 and C % 64 == 0.
static bool latent_decode_mma_fits(int H, int C, int R) {
    return H <= 16 && (C + R) % 16 == 0 && C % 64 == 0 && C <= LD_MAX_C && size_t(48) * ld_row_stride(C + R) * 2 <= 96 * 1024;
}

static int g_latent_decode_mma = 1;
GB_API int gb_latent_decode_set_mma(int on) {
    g_latent_decode_mma = on;
    return 0;
}

GB_API long long gb_latent_decode_scratch_floats(int T, int H, int C, int splits) {
    return (long long)T * H * splits * (C + 2);
}

// q: [T, H*(C+R)] bf16 (each head: q' of C entries, then the rotated part); out: [T, H*C] bf16; cache: the latent
// rows, [pages, 1, 64, C+R] bf16.  splits: parts of each token's keys (blocks of 32 keys are shared out evenly).
// window > 0: the last `window` positions only; sink float [H] and gate bf16 [T, H] (rows ldg apart), each or null: see the merge.
GB_API int gb_latent_decode(const void* q, long long ldq, void* out, long long ldo, int T, int H, int C, int R,
                            const int* seq_of, const int* pos, const int* table, int table_width, int ring_pages,
                            const void* cache, float scale, int splits, float* scratch, int window, const float* sink,
                            const void* gate, long long ldg, cudaStream_t stream) {
    GB_REQUIRE(window >= 0, "gb_latent_decode: a negative window");
    GB_REQUIRE(gb_latent_decode_supported(H, C, R, GB_BF16, GB_BF16), "gb_latent_decode: sizes heads=%d kv_rank=%d rot_dim=%d are not supported", H, C, R);
    GB_REQUIRE(splits >= 1 && splits <= 65535 && scratch && table_width > 0 && ring_pages > 0, "gb_latent_decode: bad arguments");
    GB_REQUIRE((ldq % 2) == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(scratch) & 7) == 0,
               "gb_latent_decode: misaligned operands");
    if (T == 0) return 0;
    LdParams p;
    p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache; p.seq_of = seq_of; p.pos = pos; p.table = table;
    p.scratch = scratch; p.ldq = ldq; p.H = H; p.C = C; p.R = R; p.splits = splits; p.table_width = table_width;
    p.ring_pages = ring_pages; p.scale = scale; p.window = window;
    if (g_latent_decode_mma && latent_decode_mma_fits(H, C, R)) {
        const size_t smem_mma = size_t(48) * ld_row_stride(C + R) * 2;
        static bool configured_mma = false;
        if (smem_mma > 48 * 1024 && !configured_mma) {
            if (cudaFuncSetAttribute(latent_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess)
                return gb_fail("gb_latent_decode: cannot get %zu bytes of shared memory", smem_mma);
            configured_mma = true;
        }
        latent_decode_mma_kernel<<<dim3(T, splits), LM_THREADS, smem_mma, stream>>>(p);
        GB_LAUNCH_OK("gb_latent_decode (tensor cores)");
        latent_decode_merge_kernel<<<dim3(T, H), 128, 0, stream>>>(scratch, seq_of, (__nv_bfloat16*)out, ldo, H, C, splits, sink, (const __nv_bfloat16*)gate, ldg);
        GB_LAUNCH_OK("gb_latent_decode (merge)");
        return 0;
    }
    const size_t smem = size_t(H) * (C + R) * 4 + size_t(32) * ld_row_stride(C + R) * 2;
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        if (cudaFuncSetAttribute(latent_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
            return gb_fail("gb_latent_decode: cannot get %zu bytes of shared memory", smem);
        configured = 160 * 1024;
    }
    latent_decode_kernel<<<dim3(T, splits), LD_THREADS, smem, stream>>>(p);
    GB_LAUNCH_OK("gb_latent_decode");
    latent_decode_merge_kernel<<<dim3(T, H), 128, 0, stream>>>(scratch, seq_of, (__nv_bfloat16*)out, ldo, H, C, splits, sink, (const __nv_bfloat16*)gate, ldg);
    GB_LAUNCH_OK("gb_latent_decode (merge)");
    return 0;
}
