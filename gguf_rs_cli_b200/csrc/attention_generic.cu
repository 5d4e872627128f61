// Attention over the paged cache, one block per (token, query head), for every kind of
// step: whole prompts, continuation and single tokens.  It restates the reference's
// per-head loop (src/model/llama.rs:374-394, src/gpu/attention.glsl:14-77): query head
// h reads KV head h / (nh/nkv); scores q.k * scale over the positions the token may
// see (<= its own, and inside the window if there is one); softmax with the maximum
// subtracted; weighted sum of values.  All in 32-bit with expf.  Keys are taken in
// blocks of 32 absolute positions, warp w taking blocks w, w+8, ..., and the eight
// partial results are merged in warp order, so a token's result depends on nothing but
// its own query and keys.  It is the attention of the 32-bit mode, the twin of the
// faster kernels in tests, and the path for head sizes those refuse.  Options: the first
// keep_first positions of a sequence stay visible behind the window (their pages are the
// first head_pages entries of the page table, in front of the ring); the result is
// multiplied by sigmoid(gate) entry by entry, or by one number per head; the softmax's denominator may count one
// more key that has no value (a sink), of score 0 or of a learned score per head (not scaled).  Instead of a window
// the keys may come in chunks of `chunk` positions counted from the sequence's start: a token sees the earlier tokens of
// its own chunk only.
#include <math.h>

#include "common.cuh"

constexpr int AG_MID_HD = 640;
constexpr int AG_MAX_HD = 1152;          // a latent row of 1,024 entries and a rotated part of 128
constexpr int AG_WARPS = 8;

// hd: entries of a query and of a key; hdv: entries of a value (and of a head's result); a value row starts
// every v_row entries of the value storage, which lets the values be the first hdv entries of the key rows
// themselves (attention over one shared latent row per position).  MAX_HD bounds both sizes.
template <typename TC, int MAX_HD>
__global__ void __launch_bounds__(AG_WARPS * 32) attention_generic_kernel(
    const void* __restrict__ q, int q_dtype, long long ldq, void* __restrict__ out, int out_dtype, long long ldo,
    int nh, int nkv, int hd, int hdv, int v_row, const int* __restrict__ seq_of, const int* __restrict__ pos,
    const int* __restrict__ table, int table_width, int ring_pages, const TC* __restrict__ kc,
    const TC* __restrict__ vc, int window, float scale, int head_pages, int keep_first, const void* __restrict__ gate,
    int gate_dtype, long long ldg, int gate_per_head, int sink, const float* __restrict__ sink_values, int chunk) {
    int t = blockIdx.x, h = blockIdx.y;
    int b = seq_of[t];
    size_t orow = size_t(t) * ldo + size_t(h) * hdv;
    if (b < 0) {
        for (int d = threadIdx.x; d < hdv; d += blockDim.x) gb_store(out, out_dtype, orow + d, 0.f);
        return;
    }
    __shared__ float qs[MAX_HD];
    __shared__ float acc_s[AG_WARPS][MAX_HD];
    __shared__ float m_s[AG_WARPS], l_s[AG_WARPS];
    for (int d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = gb_load(q, q_dtype, size_t(t) * ldq + size_t(h) * hd + d);
    __syncthreads();

    int p = pos[t];
    const bool vec8 = hd % 8 == 0 && (reinterpret_cast<uintptr_t>(kc) & 15) == 0;     // key rows start on 16 bytes
    int lo = gb_first_visible(p, window, chunk);
    int g = h / (nh / nkv);
    const int* trow = table + size_t(b) * table_width;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int C = MAX_HD / 32;
    float acc[C];
#pragma unroll
    for (int c = 0; c < C; ++c) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;

    // bfloat16 rows that start on 16 bytes: the lanes share each key row in pieces of eight entries (pieces lane,
    // lane + 32, ...), so that a row is read once and contiguously; shuffles bring the partial sums together.
    // Other rows: each lane walks its own key's row.  Either way the order of the sums is fixed by the sizes alone.
    constexpr int QC = (MAX_HD / 8 + 31) / 32;
    const bool shared_rows = sizeof(TC) == 2 && vec8;
    const bool pairs = sizeof(TC) == 2 && hdv % 2 == 0 && v_row % 2 == 0 && (reinterpret_cast<uintptr_t>(vc) & 3) == 0;
    float qr[QC][8];
    if (shared_rows) {
#pragma unroll
        for (int c = 0; c < QC; ++c)
#pragma unroll
            for (int e = 0; e < 8; ++e) qr[c][e] = (lane + 32 * c) * 8 < hd ? qs[(lane + 32 * c) * 8 + e] : 0.f;
    }

    // The keys a token sees: the window [lo, p], and in front of it the sequence's first keep_first positions as far as
    // the window does not hold them, [0, kept).  Blocks of the kept keys come first in the warps' round.
    const int kept = min(keep_first, lo), kept_blocks = (kept + 31) >> 5;
    const int n_blocks = kept_blocks + (p >> 5) - (lo >> 5) + 1;
    for (int ib = warp; ib < n_blocks; ib += AG_WARPS) {
        const bool front = ib < kept_blocks;
        int j = (front ? ib : (lo >> 5) + ib - kept_blocks) * 32 + lane;
        bool valid = front ? j < kept : (j >= lo && j <= p);
        float s = -INFINITY;
        long long off = 0;
        if (valid) off = (long long)gb_kv_offset(trow, ring_pages, j, g, nkv, 1, head_pages);        // the position's row number
        if (shared_rows) {
            const unsigned live = __ballot_sync(0xffffffffu, valid);
            for (int jj = 0; jj < 32; jj += 2) {
                if (!((live >> jj) & 3u)) continue;                                       // neither key is seen (uniform)
                const long long o0 = __shfl_sync(0xffffffffu, off, jj), o1 = __shfl_sync(0xffffffffu, off, jj + 1);
                const uint4* k0 = reinterpret_cast<const uint4*>(kc + o0 * hd);
                const uint4* k1 = reinterpret_cast<const uint4*>(kc + o1 * hd);
                float d0 = 0.f, d1 = 0.f;
#pragma unroll
                for (int c = 0; c < QC; ++c) {
                    const int piece = lane + 32 * c;
                    if (piece * 8 < hd) {
                        const uint4 r0 = k0[piece], r1 = k1[piece];
                        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&r0);
                        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&r1);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 ka = __bfloat1622float2(a2[e]), kb2 = __bfloat1622float2(b2[e]);
                            d0 = fmaf(qr[c][2 * e], ka.x, d0);
                            d0 = fmaf(qr[c][2 * e + 1], ka.y, d0);
                            d1 = fmaf(qr[c][2 * e], kb2.x, d1);
                            d1 = fmaf(qr[c][2 * e + 1], kb2.y, d1);
                        }
                    }
                }
                d0 = gb_warp_sum(d0);
                d1 = gb_warp_sum(d1);
                if (lane == jj && valid) s = d0 * scale;
                if (lane == jj + 1 && valid) s = d1 * scale;
            }
        } else if (valid) {
            const TC* kr = kc + off * hd;
            float dot = 0.f;
            for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], gb_to_float(kr[d]), dot);
            s = dot * scale;
        }
        float m_new = fmaxf(m, gb_warp_max(s));
        float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        float pj = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + gb_warp_sum(pj);
#pragma unroll
        for (int c = 0; c < C; ++c) acc[c] *= alpha;
        for (int jj = 0; jj < 32; ++jj) {
            float pv = __shfl_sync(0xffffffffu, pj, jj);
            long long o = __shfl_sync(0xffffffffu, off, jj);
            if (pv != 0.f) {
                const TC* vr = vc + o * v_row;
                if (pairs) {
                    // two bfloat16 values per load: acc[2c], acc[2c+1] belong to entries 64c + 2 lane and the next
                    const __nv_bfloat162* vr2 = reinterpret_cast<const __nv_bfloat162*>(vr);
#pragma unroll
                    for (int c = 0; c < C / 2; ++c) {
                        if (64 * c + 2 * lane < hdv) {
                            const float2 vv = __bfloat1622float2(vr2[32 * c + lane]);
                            acc[2 * c] = fmaf(pv, vv.x, acc[2 * c]);
                            acc[2 * c + 1] = fmaf(pv, vv.y, acc[2 * c + 1]);
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < C; ++c) {
                        int d = lane + 32 * c;
                        if (d < hdv) acc[c] = fmaf(pv, gb_to_float(vr[d]), acc[c]);
                    }
                }
            }
        }
        m = m_new;
    }
#pragma unroll
    for (int c = 0; c < C; ++c) {
        int d = pairs ? 64 * (c >> 1) + 2 * lane + (c & 1) : lane + 32 * c;
        if (d < hdv) acc_s[warp][d] = acc[c];
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < AG_WARPS; ++w) M = fmaxf(M, m_s[w]);
    float L = 0.f, wgt[AG_WARPS];
    for (int w = 0; w < AG_WARPS; ++w) {
        wgt[w] = (m_s[w] == -INFINITY) ? 0.f : expf(m_s[w] - M);
        L += l_s[w] * wgt[w];
    }
    float down = 1.f;                    // a sink above every score: the sums are brought down to its level
    if (sink && M != -INFINITY) {
        const float sv = sink_values ? sink_values[h] : 0.f;
        if (sv > M) {
            down = expf(M - sv);
            L = L * down + 1.f;
        } else {
            L += expf(sv - M);
        }
    }
    for (int d = threadIdx.x; d < hdv; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < AG_WARPS; ++w) o += acc_s[w][d] * wgt[w];
        o = o * down / L;
        if (gate) o *= 1.f / (1.f + expf(-gb_load(gate, gate_dtype, size_t(t) * ldg + (gate_per_head ? size_t(h) : size_t(h) * hdv + d))));
        gb_store(out, out_dtype, orow + d, o);
    }
}

// q: [T, nh, hd] with rows ldq elements apart (already rotated); out: [T, nh*hdv] with rows ldo
// apart.  seq_of[t] is the token's row in the page table (or -1 for padding, which gives
// zeros), pos[t] its position.  window 0 means all earlier keys.  Keys [pages, nkv, PAGE, hd]; values
// [pages, nkv, PAGE, v_row] of which the first hdv entries count (hdv = v_row = hd for ordinary heads).
GB_API int gb_attention_generic(const void* q, int q_dtype, long long ldq, void* out, int out_dtype, long long ldo,
                                int T, int nh, int nkv, int hd, int hdv, int v_row, const int* seq_of, const int* pos,
                                const int* table, int table_width, int ring_pages, const void* kcache,
                                const void* vcache, int cache_dtype, int window, float scale, int head_pages, int keep_first,
                                const void* gate, int gate_dtype, long long ldg, int gate_per_head, int sink,
                                const float* sink_values, int chunk, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(q_dtype) && gb_is_dtype(out_dtype) && gb_is_dtype(cache_dtype), "gb_attention_generic: bad dtype");
    GB_REQUIRE(hd > 0 && hd <= AG_MAX_HD, "gb_attention_generic: head_dim %d is not in 1..%d", hd, AG_MAX_HD);
    GB_REQUIRE(hdv > 0 && hdv <= AG_MAX_HD && v_row >= hdv, "gb_attention_generic: value size %d (rows of %d) is not in 1..%d", hdv, v_row, AG_MAX_HD);
    GB_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "gb_attention_generic: %d heads are not a multiple of %d KV heads", nh, nkv);
    GB_REQUIRE(nh <= 65535, "gb_attention_generic: too many heads (%d)", nh);
    GB_REQUIRE(window >= 0 && ring_pages > 0 && table_width > 0 && head_pages >= 0, "gb_attention_generic: bad cache geometry");
    GB_REQUIRE(keep_first >= 0, "gb_attention_generic: a negative number of kept positions");
    GB_REQUIRE(chunk >= 0 && (chunk == 0 || (window == 0 && keep_first == 0)), "gb_attention_generic: chunks go with neither a window nor kept positions");
    GB_REQUIRE(!gate || gb_is_dtype(gate_dtype), "gb_attention_generic: bad gate dtype");
    if (T == 0) return 0;
    dim3 grid(T, nh);
#define AG_LAUNCH(TC, MAX_HD)                                                                                     \
    attention_generic_kernel<TC, MAX_HD><<<grid, AG_WARPS * 32, 0, stream>>>(                                     \
        q, q_dtype, ldq, out, out_dtype, ldo, nh, nkv, hd, hdv, v_row, seq_of, pos, table, table_width, ring_pages, \
        (const TC*)kcache, (const TC*)vcache, window, scale, head_pages, window > 0 ? keep_first : 0, gate, gate_dtype, ldg, gate_per_head, sink, sink_values, chunk)
    const bool small = hd <= 256 && hdv <= 256, mid = hd <= AG_MID_HD && hdv <= AG_MID_HD;
    if (cache_dtype == GB_F32) {
        if (small) AG_LAUNCH(float, 256);
        else if (mid) AG_LAUNCH(float, AG_MID_HD);
        else AG_LAUNCH(float, AG_MAX_HD);
    } else {
        if (small) AG_LAUNCH(__nv_bfloat16, 256);
        else if (mid) AG_LAUNCH(__nv_bfloat16, AG_MID_HD);
        else AG_LAUNCH(__nv_bfloat16, AG_MAX_HD);
    }
#undef AG_LAUNCH
    GB_LAUNCH_OK("gb_attention_generic");
    return 0;
}
