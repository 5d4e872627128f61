// What stands between the projections of an attention mixer and the attention kernel when it is more than
// a rotation: normalised queries and keys with a query temperature that grows with the position, and the
// preparation of latent attention (the normalised latent row and the shared rotated key part go into the
// cache; queries are brought into the latent's space by a product per head).  All in 32-bit.
#include <math.h>

#include "common.cuh"

// ---------------------------------------- unit-RMS q and k, query temperature
// One block per token; its warps take the token's heads in turn: q heads first (scaled in place), then k
// heads (into the cache), then v heads (copied into the cache).
//   q_h <- q_h / sqrt(mean(q_h^2) + eps) * temp(p),  temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)
//   k_g <- k_g / sqrt(mean(k_g^2) + eps)
// normalise 0 leaves the division out; coef 0 the temperature.  Keys have D entries, values Dv.
__global__ void qk_norm_kv_write_kernel(void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                                        int dtype, long long ld, int H, int G, int D, int Dv, int normalise, float eps,
                                        float coef, int every, const int* __restrict__ seq_of,
                                        const int* __restrict__ pos, const int* __restrict__ table, int table_width,
                                        int ring_pages, void* __restrict__ kcache, void* __restrict__ vcache,
                                        int cache_dtype) {
    const int t = blockIdx.x;
    const int b = seq_of[t];
    if (b < 0) return;
    const int p = pos[t];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const size_t row = size_t(t) * size_t(ld);
    const int* trow = table + size_t(b) * table_width;
    const float temp = coef != 0.f ? 1.f + coef * logf(float((p + 1) / every) + 1.f) : 1.f;
    const int total = k ? H + 2 * G : H;
    for (int item = warp; item < total; item += warps) {
        if (item < H + G) {
            const bool is_q = item < H;
            const void* src = is_q ? q : k;
            const size_t o = row + size_t(is_q ? item : item - H) * D;
            float f = is_q ? temp : 1.f;
            if (normalise) {
                float ss = 0.f;
                for (int d = lane; d < D; d += 32) {
                    const float x = gb_load(src, dtype, o + d);
                    ss = fmaf(x, x, ss);
                }
                f /= sqrtf(gb_warp_sum(ss) / float(D) + eps);
            }
            if (is_q) {
                for (int d = lane; d < D; d += 32) gb_store(q, dtype, o + d, gb_load(q, dtype, o + d) * f);
            } else {
                const size_t c = gb_kv_offset(trow, ring_pages, p, item - H, G, D);
                for (int d = lane; d < D; d += 32) gb_store(kcache, cache_dtype, c + d, gb_load(k, dtype, o + d) * f);
            }
        } else {
            const int g = item - H - G;
            const size_t o = row + size_t(g) * Dv;
            const size_t c = gb_kv_offset(trow, ring_pages, p, g, G, Dv);
            for (int d = lane; d < Dv; d += 32) gb_store(vcache, cache_dtype, c + d, gb_load(v, dtype, o + d));
        }
    }
}

// q [T, H*D] (scaled in place), k [T, G*D], v [T, G*Dv]: first elements of token 0's parts; rows `ld` apart.
// kcache [pages, G, PAGE, D], vcache [pages, G, PAGE, Dv].  k and v null: only q is treated.
GB_API int gb_qk_norm_kv_write(void* q, const void* k, const void* v, int dtype, long long ld, int T, int H, int G, int D,
                               int Dv, int normalise, float eps, float coef, int every, const int* seq_of, const int* pos,
                               const int* table, int table_width, int ring_pages, void* kcache, void* vcache,
                               int cache_dtype, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(cache_dtype), "gb_qk_norm_kv_write: bad dtype");
    GB_REQUIRE(H > 0 && G > 0 && D > 0 && Dv > 0, "gb_qk_norm_kv_write: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d", H, G, D, Dv);
    GB_REQUIRE(!normalise || eps > 0.f, "gb_qk_norm_kv_write: eps must be positive");
    GB_REQUIRE(coef == 0.f || every > 0, "gb_qk_norm_kv_write: the temperature's period must be positive, got %d", every);
    GB_REQUIRE((k == nullptr) == (v == nullptr), "gb_qk_norm_kv_write: k and v must both be given or both be null");
    GB_REQUIRE(!k || (table && kcache && vcache && ring_pages > 0 && table_width >= 1), "gb_qk_norm_kv_write: cache missing");
    if (T == 0) return 0;
    qk_norm_kv_write_kernel<<<T, 128, 0, stream>>>(q, k, v, dtype, ld, H, G, D, Dv, normalise, eps, coef, every > 0 ? every : 1,
                                                   seq_of, pos, table, table_width, ring_pages, kcache, vcache, cache_dtype);
    GB_LAUNCH_OK("gb_qk_norm_kv_write");
    return 0;
}

// ------------------------------------------------------- latent attention
// One block per token.  dkv [C + Rd]: the first C entries, divided by their root mean square and multiplied
// by w, are the latent row c; the last Rd are a key part that all heads share, rotated by the token's
// position.  Both go into the cache as one row [C + Rd] (and into row_out, a plain copy [T, C + Rd] of
// this step's rows, when given).  q [H, D + Rd]: the last Rd entries of each head are rotated likewise and
// written to qa, head h's part starting at entry h * qa_stride + qa_off of the token's row (qa may be q
// itself: the rotation is then done in place).
// Rotation: the first rot_dims entries of the part, pair (2i, 2i+1) by position * inv_freq[i], or with `halves` pair
// (i, i + rot_dims/2); the rest pass unchanged.
__global__ void latent_prep_kernel(const void* __restrict__ q, long long ldq, const void* __restrict__ dkv,
                                   long long ldd, int dtype, int H, int D, int Rd, int C, int rot_dims,
                                   const float* __restrict__ inv_freq, const void* __restrict__ w, int w_dtype, float eps,
                                   void* qa, long long lda, int qa_stride, int qa_off, void* __restrict__ row_out,
                                   const int* __restrict__ seq_of,
                                   const int* __restrict__ pos, const int* __restrict__ table, int table_width,
                                   int ring_pages, void* __restrict__ cache, int cache_dtype, int halves) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int b = seq_of[t];
    if (b < 0) return;
    const int p = pos[t];
    const size_t drow = size_t(t) * size_t(ldd);
    float ss = 0.f;
    for (int d = threadIdx.x; d < C; d += blockDim.x) {
        const float x = gb_load(dkv, dtype, drow + d);
        ss = fmaf(x, x, ss);
    }
    ss = gb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int wv = 0; wv < (blockDim.x >> 5); ++wv) tot += red[wv];
    const float f = 1.f / sqrtf(tot / float(C) + eps);
    const size_t crow = gb_kv_offset(table + size_t(b) * table_width, ring_pages, p, 0, 1, C + Rd);
    const size_t rrow = size_t(t) * (C + Rd);
    for (int d = threadIdx.x; d < C; d += blockDim.x) {
        const float cv = gb_load(dkv, dtype, drow + d) * f * gb_load(w, w_dtype, d);
        gb_store(cache, cache_dtype, crow + d, cv);
        if (row_out) gb_store(row_out, dtype, rrow + d, cv);
    }
    // rotated parts: item 0 is the shared key part, items 1..H the heads' query parts
    const int half = rot_dims / 2, pairs = Rd / 2;          // Rd even: checked by the caller
    for (int idx = threadIdx.x; idx < (H + 1) * pairs; idx += blockDim.x) {
        const int item = idx / pairs, i = idx - item * pairs;
        float sn = 0.f, cs = 1.f;
        if (i < half) sincosf(float(p) * inv_freq[i], &sn, &cs);
        // the pair that angle i turns: neighbours (2i, 2i+1), or with `halves` entries (i, i + half); pairs behind the
        // rotated entries pass unchanged either way
        const int d0 = halves && i < half ? i : 2 * i, d1 = halves && i < half ? i + half : 2 * i + 1;
        float x0, x1, y0, y1;
        if (item == 0) {
            x0 = gb_load(dkv, dtype, drow + C + d0);
            x1 = gb_load(dkv, dtype, drow + C + d1);
        } else {
            const size_t o = size_t(t) * ldq + size_t(item - 1) * (D + Rd) + D;
            x0 = gb_load(q, dtype, o + d0);
            x1 = gb_load(q, dtype, o + d1);
        }
        gb_rotate(x0, x1, cs, sn, y0, y1);
        if (item == 0) {
            gb_store(cache, cache_dtype, crow + C + d0, y0);
            gb_store(cache, cache_dtype, crow + C + d1, y1);
            if (row_out) {
                gb_store(row_out, dtype, rrow + C + d0, y0);
                gb_store(row_out, dtype, rrow + C + d1, y1);
            }
        } else {
            const size_t o = size_t(t) * lda + size_t(item - 1) * qa_stride + qa_off;
            gb_store(qa, dtype, o + d0, y0);
            gb_store(qa, dtype, o + d1, y1);
        }
    }
}

GB_API int gb_latent_prep(const void* q, long long ldq, const void* dkv, long long ldd, int dtype, int T, int H, int D, int Rd,
                          int C, int rot_dims, const float* inv_freq, const void* w, int w_dtype, float eps, void* qa,
                          long long lda, int qa_stride, int qa_off, void* row_out, const int* seq_of, const int* pos,
                          const int* table, int table_width, int ring_pages, void* cache, int cache_dtype, int halves,
                          cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(w_dtype) && gb_is_dtype(cache_dtype), "gb_latent_prep: bad dtype");
    GB_REQUIRE(H > 0 && D >= 0 && C > 0 && Rd >= 0 && Rd % 2 == 0 && rot_dims >= 0 && rot_dims <= Rd && rot_dims % 2 == 0,
               "gb_latent_prep: bad sizes heads=%d dim=%d rot_dim=%d kv_rank=%d rotated=%d", H, D, Rd, C, rot_dims);
    GB_REQUIRE(rot_dims == 0 || inv_freq, "gb_latent_prep: no table of frequencies");
    GB_REQUIRE(table && cache && ring_pages > 0 && table_width >= 1 && eps > 0.f, "gb_latent_prep: cache missing");
    if (T == 0) return 0;
    latent_prep_kernel<<<T, 128, 0, stream>>>(q, ldq, dkv, ldd, dtype, H, D, Rd, C, rot_dims, inv_freq, w, w_dtype, eps, qa, lda,
                                              qa_stride, qa_off, row_out, seq_of, pos, table, table_width, ring_pages, cache, cache_dtype, halves);
    GB_LAUNCH_OK("gb_latent_prep");
    return 0;
}

// Keys and values per head of a prompt, laid out as pages for the tiled attention kernel: for token t of
// sequence b at position p (page table[b][p / 64], place p % 64),
//   K[page, h, place, :] = [kv[t, h*D : (h+1)*D], row[t, C : C + Rd]]    (the head's own part, the shared rotated part)
//   V[page, h, place, :] = kv[t, H*D + h*Dv : H*D + (h+1)*Dv]
// kv [T, H*D + H*Dv] is the product of the latent rows with the two up-projections, row [T, C + Rd] the
// rows that latent_prep wrote.  One block per token.
__global__ void pack_latent_heads_kernel(const __nv_bfloat16* __restrict__ kv, long long ldkv,
                                         const __nv_bfloat16* __restrict__ row, int H, int D, int Rd, int Dv, int C,
                                         const int* __restrict__ seq_of, const int* __restrict__ pos,
                                         const int* __restrict__ table, int table_width, __nv_bfloat16* __restrict__ K,
                                         __nv_bfloat16* __restrict__ V) {
    const int t = blockIdx.x;
    const int b = seq_of[t];
    if (b < 0) return;
    const int p = pos[t];
    const int page = table[size_t(b) * table_width + (p >> GB_PAGE_SHIFT)], place = p & (GB_PAGE - 1);
    const int hk = D + Rd;
    const __nv_bfloat16* kvr = kv + size_t(t) * ldkv;
    const __nv_bfloat16* rr = row + size_t(t) * (C + Rd) + C;
    for (int idx = threadIdx.x; idx < H * hk; idx += blockDim.x) {
        const int h = idx / hk, d = idx - h * hk;
        K[((size_t(page) * H + h) * GB_PAGE + place) * hk + d] = d < D ? kvr[h * D + d] : rr[d - D];
    }
    for (int idx = threadIdx.x; idx < H * Dv; idx += blockDim.x) {
        const int h = idx / Dv, d = idx - h * Dv;
        V[((size_t(page) * H + h) * GB_PAGE + place) * Dv + d] = kvr[size_t(H) * D + idx];
    }
}

GB_API int gb_pack_latent_heads(const void* kv, long long ldkv, const void* row, int T, int H, int D, int Rd, int Dv, int C,
                                const int* seq_of, const int* pos, const int* table, int table_width, void* K, void* V,
                                cudaStream_t stream) {
    GB_REQUIRE(H > 0 && D > 0 && Rd >= 0 && Dv > 0 && C > 0 && table_width > 0, "gb_pack_latent_heads: bad sizes");
    if (T == 0) return 0;
    pack_latent_heads_kernel<<<T, 256, 0, stream>>>((const __nv_bfloat16*)kv, ldkv, (const __nv_bfloat16*)row, H, D, Rd, Dv, C,
                                                    seq_of, pos, table, table_width, (__nv_bfloat16*)K, (__nv_bfloat16*)V);
    GB_LAUNCH_OK("gb_pack_latent_heads");
    return 0;
}

// --------------------------------------------------- a product per head
// out[t, h*os + o] = sum_i x[t, h*xs + i] * W[h, i, o] for o < O: every head has a matrix [I, O] of its own
// (row-major, heads one after the other).  32-bit FMAs.  A block takes HM_TOKENS tokens, one head and 32
// output columns; its four warps take a quarter of the inputs each (in ascending i) and the quarters are
// added in warp order, so a token's result depends on neither the batch nor timing.
constexpr int HM_TOKENS = 8;

template <typename TX, typename TW>
__global__ void __launch_bounds__(128) head_matmul_kernel(const TX* __restrict__ x, long long ldx, int xs,
                                                          const TW* __restrict__ W, int I, int O, void* __restrict__ out,
                                                          int out_dtype, long long ldo, int os, int T) {
    extern __shared__ float xt[];                     // [HM_TOKENS][I], then [4][HM_TOKENS][32] partial sums
    float* part = xt + HM_TOKENS * I;
    const int t0 = blockIdx.x * HM_TOKENS, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int o = blockIdx.z * 32 + lane;
    const int nt = min(HM_TOKENS, T - t0);
    for (int idx = threadIdx.x; idx < HM_TOKENS * I; idx += 128) {
        const int tt = idx / I, i = idx - tt * I;
        xt[idx] = tt < nt ? gb_to_float(x[size_t(t0 + tt) * ldx + size_t(h) * xs + i]) : 0.f;
    }
    __syncthreads();
    float acc[HM_TOKENS];
#pragma unroll
    for (int tt = 0; tt < HM_TOKENS; ++tt) acc[tt] = 0.f;
    const int per = (I + 3) / 4, i0 = warp * per, i1 = min(I, i0 + per);
    if (o < O) {
        const TW* wp = W + size_t(h) * I * O + o;
        for (int i = i0; i < i1; ++i) {
            const float wv = gb_to_float(wp[size_t(i) * O]);
#pragma unroll
            for (int tt = 0; tt < HM_TOKENS; ++tt) acc[tt] = fmaf(xt[tt * I + i], wv, acc[tt]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < HM_TOKENS; ++tt) part[(warp * HM_TOKENS + tt) * 32 + lane] = acc[tt];
    __syncthreads();
    for (int idx = threadIdx.x; idx < HM_TOKENS * 32; idx += 128) {
        const int tt = idx >> 5, ol = idx & 31, oo = blockIdx.z * 32 + ol;
        if (tt < nt && oo < O) {
            const float v = ((part[(0 * HM_TOKENS + tt) * 32 + ol] + part[(1 * HM_TOKENS + tt) * 32 + ol]) +
                             part[(2 * HM_TOKENS + tt) * 32 + ol]) + part[(3 * HM_TOKENS + tt) * 32 + ol];
            gb_store(out, out_dtype, size_t(t0 + tt) * ldo + size_t(h) * os + oo, v);
        }
    }
}

// x: head h's I inputs start at column h*xs of a row (rows ldx apart); out: its O results start at column h*os.
GB_API int gb_head_matmul(const void* x, int x_dtype, long long ldx, int xs, const void* W, int w_dtype, int H, int I, int O,
                          void* out, int out_dtype, long long ldo, int os, int T, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(x_dtype) && gb_is_dtype(w_dtype) && gb_is_dtype(out_dtype), "gb_head_matmul: bad dtype");
    GB_REQUIRE(H > 0 && H <= 65535 && I > 0 && O > 0 && xs >= I && os >= O, "gb_head_matmul: bad sizes heads=%d in=%d out=%d", H, I, O);
    const size_t smem = (size_t(HM_TOKENS) * I + 4 * HM_TOKENS * 32) * sizeof(float);
    GB_REQUIRE(smem <= 48 * 1024, "gb_head_matmul: %d inputs per head exceed %d", I, (48 * 1024 / 4 - 4 * HM_TOKENS * 32) / HM_TOKENS);
    if (T == 0) return 0;
    dim3 grid((T + HM_TOKENS - 1) / HM_TOKENS, H, (O + 31) / 32);
    GB_REQUIRE(grid.z <= 65535, "gb_head_matmul: too many outputs per head (%d)", O);
#define HM_LAUNCH(TX, TW)                                                                                             \
    head_matmul_kernel<TX, TW><<<grid, 128, smem, stream>>>((const TX*)x, ldx, xs, (const TW*)W, I, O, out, out_dtype, ldo, os, T)
    if (x_dtype == GB_F32 && w_dtype == GB_F32) HM_LAUNCH(float, float);
    else if (x_dtype == GB_BF16 && w_dtype == GB_BF16) HM_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == GB_BF16 && w_dtype == GB_F32) HM_LAUNCH(__nv_bfloat16, float);
    else HM_LAUNCH(float, __nv_bfloat16);
#undef HM_LAUNCH
    GB_LAUNCH_OK("gb_head_matmul");
    return 0;
}

// ------------------------- per-head RMS norm with a weight, rotation, mixing of values, cache write
// One block per token; its warps take the token's heads in turn: q heads (treated in place), k heads (into the
// cache), v heads (into the cache).
//   q_h <- rot_p(q_h / sqrt(mean(q_h^2) + eps) * wq),  k_g likewise with wk       (wq, wk [D] serve all heads;
//                                                                                  null: no norm at all)
//   rot_p: the first rot_dims entries of a head in pairs, (i, i + rot_dims/2) or (2i, 2i+1), by the angle
//          p * inv_freq[i]; the other entries pass; inv_freq null: no rotation
//   v_g <- (1 - lambda) v_g + lambda v_first_g   when v_first is given (another layer's values of the same token);
//   first_out, when given, receives the token's own values as they came (for the layers that mix them in).
// A head lies in shared memory (32-bit) between the norm and the rotation.  Cache positions follow the page table
// with head_pages kept pages in front of the ring.
struct HeadPrepParams {
    void* q;
    const void *k, *v;
    long long ld;
    int dtype, H, G, D, Dv;
    const void *wq, *wk;
    int w_dtype;
    float eps;
    const float* inv_freq;
    int rot_dims, pairing;
    const void* v_first;
    long long ld_first;
    float lambda;
    void* first_out;
    long long ld_out;
    const int *seq_of, *pos, *table;
    int table_width, ring_pages, head_pages;
    void *kcache, *vcache;
    int cache_dtype;
};

__global__ void __launch_bounds__(128) head_prep_kv_write_kernel(const HeadPrepParams a) {
    extern __shared__ float hp_sm[];
    const int t = blockIdx.x;
    const int b = a.seq_of[t];
    if (b < 0) return;
    const int p = a.pos[t];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int H = a.H, G = a.G, D = a.D, Dv = a.Dv;
    float* buf = hp_sm + warp * D;
    const size_t row = size_t(t) * size_t(a.ld);
    const int* trow = a.table + size_t(b) * a.table_width;
    const int half = a.inv_freq ? a.rot_dims / 2 : 0;
    const int items = a.k ? H + 2 * G : H;          // a layer that reads another layer's keys and values prepares its queries only
    for (int item = warp; item < items; item += warps) {
        if (item < H + G) {
            const bool is_q = item < H;
            const void* src = is_q ? (const void*)a.q : a.k;
            const void* w = is_q ? a.wq : a.wk;
            const size_t o = row + size_t(is_q ? item : item - H) * D;
            float ss = 0.f;
            for (int d = lane; d < D; d += 32) {
                const float x = gb_load(src, a.dtype, o + d);
                buf[d] = x;
                ss = fmaf(x, x, ss);
            }
            if (w) {
                const float f = 1.f / sqrtf(gb_warp_sum(ss) / float(D) + a.eps);
                for (int d = lane; d < D; d += 32) buf[d] = buf[d] * f * gb_load(w, a.w_dtype, d);
            }
            __syncwarp();
            void* dst = is_q ? a.q : a.kcache;
            const int dt = is_q ? a.dtype : a.cache_dtype;
            const size_t c = is_q ? o : gb_kv_offset(trow, a.ring_pages, p, item - H, G, D, a.head_pages);
            for (int i = lane; i < half; i += 32) {
                const int d0 = a.pairing ? 2 * i : i, d1 = a.pairing ? 2 * i + 1 : i + half;
                float sn, cs, y0, y1;
                sincosf(float(p) * a.inv_freq[i], &sn, &cs);
                gb_rotate(buf[d0], buf[d1], cs, sn, y0, y1);
                gb_store(dst, dt, c + d0, y0);
                gb_store(dst, dt, c + d1, y1);
            }
            for (int d = 2 * half + lane; d < D; d += 32) gb_store(dst, dt, c + d, buf[d]);
            __syncwarp();
        } else {
            const int g = item - H - G;
            const size_t o = row + size_t(g) * Dv;
            const size_t c = gb_kv_offset(trow, a.ring_pages, p, g, G, Dv, a.head_pages);
            for (int d = lane; d < Dv; d += 32) {
                float x = gb_load(a.v, a.dtype, o + d);
                if (a.first_out) gb_store(a.first_out, a.dtype, size_t(t) * a.ld_out + size_t(g) * Dv + d, x);
                if (a.v_first) x = (1.f - a.lambda) * x + a.lambda * gb_load(a.v_first, a.dtype, size_t(t) * a.ld_first + size_t(g) * Dv + d);
                gb_store(a.vcache, a.cache_dtype, c + d, x);
            }
        }
    }
}

// q [T, H*D] (treated in place), k [T, G*D], v [T, G*Dv]: column slices of one row-major buffer, rows `ld` apart.
// kcache [pages, G, PAGE, D], vcache [pages, G, PAGE, Dv].  v_first, first_out: [T, G*Dv] with rows of their own.
GB_API int gb_head_prep_kv_write(void* q, const void* k, const void* v, int dtype, long long ld, int T, int H, int G, int D,
                                 int Dv, const void* wq, const void* wk, int w_dtype, float eps, const float* inv_freq,
                                 int rot_dims, int pairing, const void* v_first, long long ld_first, float lambda,
                                 void* first_out, long long ld_out, const int* seq_of, const int* pos, const int* table,
                                 int table_width, int ring_pages, int head_pages, void* kcache, void* vcache,
                                 int cache_dtype, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(cache_dtype), "gb_head_prep_kv_write: bad dtype");
    GB_REQUIRE(H > 0 && G > 0 && D > 0 && Dv > 0 && D <= 4096, "gb_head_prep_kv_write: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d", H, G, D, Dv);
    GB_REQUIRE((wq == nullptr) == (wk == nullptr) && (!wq || (gb_is_dtype(w_dtype) && eps > 0.f)), "gb_head_prep_kv_write: bad norm");
    GB_REQUIRE(!inv_freq || (rot_dims > 0 && rot_dims % 2 == 0 && rot_dims <= D), "gb_head_prep_kv_write: %d of %d entries cannot be rotated", rot_dims, D);
    GB_REQUIRE(q && table && ring_pages > 0 && head_pages >= 0 && table_width >= 1, "gb_head_prep_kv_write: arguments missing");
    GB_REQUIRE((k && v && kcache && vcache) || (!k && !v), "gb_head_prep_kv_write: keys and values come together with their caches, or not at all");
    if (T == 0) return 0;
    HeadPrepParams a;
    a.q = q; a.k = k; a.v = v; a.ld = ld; a.dtype = dtype; a.H = H; a.G = G; a.D = D; a.Dv = Dv; a.wq = wq; a.wk = wk;
    a.w_dtype = w_dtype; a.eps = eps; a.inv_freq = inv_freq; a.rot_dims = rot_dims; a.pairing = pairing; a.v_first = v_first;
    a.ld_first = ld_first; a.lambda = lambda; a.first_out = first_out; a.ld_out = ld_out; a.seq_of = seq_of; a.pos = pos;
    a.table = table; a.table_width = table_width; a.ring_pages = ring_pages; a.head_pages = head_pages; a.kcache = kcache;
    a.vcache = vcache; a.cache_dtype = cache_dtype;
    head_prep_kv_write_kernel<<<T, 128, size_t(4) * D * sizeof(float), stream>>>(a);
    GB_LAUNCH_OK("gb_head_prep_kv_write");
    return 0;
}
