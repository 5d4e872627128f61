// Routed experts for steps of many tokens, on the tensor cores (mma.sync m16n8k16, bfloat16 in, 32-bit sums).
//
// The step's (token, choice) pairs are sorted by expert on the device (one block: counts, offsets, a list of tiles of
// 64 pairs that never cross an expert), so that the host learns nothing and waits for nothing.  One kernel then serves
// both products of an expert: a CTA takes a tile of 64 pairs and 64 features, gathers the pairs' rows (the tokens'
// rows of h for gate and up, the pairs' own rows of unit outputs for down) and the expert's matrix rows into shared
// memory with cp.async, two stages of 64 entries of K, and multiplies.  Gate and up share the gathered rows and end
// in the clamped unit g' sigmoid(1.702 g') (u' + 1); down ends in 32-bit rows per pair, which a last kernel sums per
// token in the order of the choices with the router's weights (no atomics: the result does not depend on timing).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int MG_BM = 64;           // pairs per tile (128, two row fragments a warp: the same time, 0.82 + 0.48 ms at 8,192 pairs)
constexpr int MG_WM = MG_BM / 64;   // fragments of 16 rows per warp (four warps share a tile's rows)
constexpr int MG_STAGES = 3;
constexpr int MG_BN = 64;           // features per tile
constexpr int MG_BK = 32;           // entries of K per stage: 12 KB a stage with gate and up, so that five CTAs share an SM
constexpr int MG_CH = MG_BK / 8;    // 16-byte chunks per row of a stage
constexpr int MG_THREADS = 128;

__device__ __forceinline__ void mg_cp16(void* dst, const void* src, bool valid) {
    unsigned d = unsigned(__cvta_generic_to_shared(dst));
    int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void mg_ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned a = unsigned(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mg_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// element offset of (row, 16-byte chunk) in a tile of rows of 32 bfloat16 (four chunks); two rows fill the 128 bytes that
// the banks span, so the chunk is XOR-swizzled by the row pair: eight consecutive rows of one chunk fall into eight bank groups
__device__ __forceinline__ int mg_swz(int row, int chunk) { return row * MG_BK + ((chunk ^ ((row >> 1) & 3)) << 3); }

}  // namespace

// What an identity expert gives for a pair: the token's own row.
struct MoeIdentity {
    const int* ids;                 // [T, top]; null: no identity experts
    const void* h;                  // [T, N] rows ldh apart
    long long ldh;
    int n_real, h_dtype;
};

// ids [n_pairs] -> offsets [E + 1], perm [n_pairs] (pairs in the order of their experts), tiles [max_tiles][2] = (expert,
// first place in perm), n_tiles [1].  Places inside an expert's range are handed out by atomics on shared memory: their
// order is not fixed, and nothing depends on it (every pair's rows are computed for themselves).
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ ids, int n_pairs, int E, int* __restrict__ offsets,
                                                        int* __restrict__ perm, int* __restrict__ tiles, int* __restrict__ n_tiles,
                                                        int* __restrict__ place_of) {
    __shared__ int count[1024], cursor[1024], tile0[1025];
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&count[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, t = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = cursor[e] = at;
            tile0[e] = t;
            at += count[e];
            t += (count[e] + MG_BM - 1) / MG_BM;
        }
        offsets[E] = at;
        tile0[E] = t;
        n_tiles[0] = t;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x)
        for (int j = tile0[e]; j < tile0[e + 1]; ++j) {
            tiles[2 * j] = e;
            tiles[2 * j + 1] = cursor[e] + (j - tile0[e]) * MG_BM;
        }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int place = atomicAdd(&cursor[ids[i]], 1);
        perm[place] = i;
        if (place_of) place_of[i] = place;
    }
}

// rows[place, :] = h[perm[place] / top, :]: the tokens' rows in the order of their pairs' experts (16-byte pieces).
__global__ void moe_gather_rows_kernel(const uint4* __restrict__ h, long long ldh16, const int* __restrict__ perm, int top, int k16,
                                       uint4* __restrict__ rows, long long total) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long place = i / k16;
    const int c = int(i - place * k16);
    rows[i] = h[size_t(perm[place] / top) * ldh16 + c];
}

// out[t, n] (+)= sum_r weights[t, r] z[place_of[t * top + r], n], the choices in their order.
__global__ void moe_combine_sorted_kernel(const float* __restrict__ z, const int* __restrict__ place_of,
                                          const float* __restrict__ weights, int top, int N, float* __restrict__ out, int accumulate,
                                          long long total, const MoeIdentity id) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / N;
    const int n = int(i - t * N);
    float acc = 0.f;
    for (int r = 0; r < top; ++r) {
        const bool own = id.ids && id.ids[t * top + r] >= id.n_real;
        acc = fmaf(weights[t * top + r], own ? gb_load(id.h, id.h_dtype, size_t(t) * id.ldh + n) : z[size_t(place_of[t * top + r]) * N + n], acc);
    }
    out[i] = accumulate ? out[i] + acc : acc;
}

struct MgParams {
    const __nv_bfloat16* a;         // rows of K entries, lda apart: row pair / a_div of a pair
    const __nv_bfloat16 *w0, *w1;   // [E, N, K] each; w1 only with GLU
    void* out;                      // GLU: bfloat16 [n_pairs, N]; else float [n_pairs, N]
    const int *offsets, *perm, *tiles, *n_tiles;
    long long lda;
    int a_div, N, K;
    float limit;
    int n_real;                     // experts numbered n_real and above have no matrices (identity experts): their tiles are left out
};


template <bool GLU>
__global__ void __launch_bounds__(MG_THREADS, 5) moe_grouped_kernel(const MgParams p) {
    extern __shared__ __align__(128) unsigned char mg_smem[];
    constexpr int NB = GLU ? 2 : 1;
    constexpr int STAGE = (MG_BM + NB * MG_BN) * MG_BK;                 // elements per stage
    __nv_bfloat16* sm = reinterpret_cast<__nv_bfloat16*>(mg_smem);
    __shared__ int rows[MG_BM];
    // blockIdx.x (which varies fastest in the order CTAs start) is the slice of features, blockIdx.y the tile of pairs:
    // CTAs that run together share a tile's gathered rows and walk through one expert's matrix
    if (int(blockIdx.y) >= p.n_tiles[0]) return;
    const int e = p.tiles[2 * blockIdx.y], place0 = p.tiles[2 * blockIdx.y + 1];
    if (e >= p.n_real) return;
    const int n_rows = min(MG_BM, p.offsets[e + 1] - place0);
    const int n0 = blockIdx.x * MG_BN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < MG_BM; i += MG_THREADS) rows[i] = i < n_rows ? p.perm[place0 + i] : -1;
    __syncthreads();
    const __nv_bfloat16* w0 = p.w0 + size_t(e) * p.N * p.K;
    const __nv_bfloat16* w1 = GLU ? p.w1 + size_t(e) * p.N * p.K : nullptr;

    auto load = [&](int k0, int stage) {
        __nv_bfloat16* as = sm + stage * STAGE;
        for (int i = tid; i < MG_BM * MG_CH; i += MG_THREADS) {
            const int r = i / MG_CH, c = i % MG_CH;
            const int pair = rows[r];
            const bool ok = pair >= 0 && k0 + c * 8 < p.K;
            mg_cp16(as + mg_swz(r, c), p.a + size_t(ok ? pair / p.a_div : 0) * p.lda + (ok ? k0 + c * 8 : 0), ok);
        }
#pragma unroll
        for (int m = 0; m < NB; ++m) {
            __nv_bfloat16* bs = as + (MG_BM + m * MG_BN) * MG_BK;
            const __nv_bfloat16* w = m ? w1 : w0;
            for (int i = tid; i < MG_BN * MG_CH; i += MG_THREADS) {
                const int r = i / MG_CH, c = i % MG_CH;
                const bool ok = n0 + r < p.N && k0 + c * 8 < p.K;
                mg_cp16(bs + mg_swz(r, c), w + (ok ? size_t(n0 + r) * p.K + k0 + c * 8 : 0), ok);
            }
        }
    };

    float acc[NB][MG_WM][MG_BN / 8][4];
#pragma unroll
    for (int m = 0; m < NB; ++m)
#pragma unroll
        for (int mi = 0; mi < MG_WM; ++mi)
#pragma unroll
            for (int j = 0; j < MG_BN / 8; ++j) acc[m][mi][j][0] = acc[m][mi][j][1] = acc[m][mi][j][2] = acc[m][mi][j][3] = 0.f;

    const int k_steps = (p.K + MG_BK - 1) / MG_BK;
    load(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (k_steps > 1) load(MG_BK, 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int ks = 0; ks < k_steps; ++ks) {
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();                                     // stage ks has landed; everyone is done with stage ks - 1
        if (ks + 2 < k_steps) load((ks + 2) * MG_BK, (ks + 2) % MG_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const __nv_bfloat16* as = sm + (ks % MG_STAGES) * STAGE;
#pragma unroll
        for (int k = 0; k < MG_BK / 16; ++k) {
            unsigned af[MG_WM][4];
#pragma unroll
            for (int mi = 0; mi < MG_WM; ++mi)
                mg_ldmatrix_x4(af[mi][0], af[mi][1], af[mi][2], af[mi][3],
                               as + mg_swz(warp * 16 * MG_WM + mi * 16 + (lane & 15), 2 * k + (lane >> 4)));
#pragma unroll
            for (int m = 0; m < NB; ++m) {
                const __nv_bfloat16* bs = as + (MG_BM + m * MG_BN) * MG_BK;
#pragma unroll
                for (int j2 = 0; j2 < MG_BN / 16; ++j2) {
                    unsigned b0, b1, b2, b3;
                    mg_ldmatrix_x4(b0, b1, b2, b3, bs + mg_swz(j2 * 16 + (lane & 7) + ((lane >> 4) << 3), 2 * k + ((lane >> 3) & 1)));
#pragma unroll
                    for (int mi = 0; mi < MG_WM; ++mi) {
                        mg_mma(acc[m][mi][2 * j2], af[mi], b0, b1);
                        mg_mma(acc[m][mi][2 * j2 + 1], af[mi], b2, b3);
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

#pragma unroll
    for (int mi = 0; mi < MG_WM; ++mi) {
    const int r0 = warp * 16 * MG_WM + mi * 16 + (lane >> 2), r1 = r0 + 8;
    const int pair0 = rows[r0], pair1 = rows[r1];
#pragma unroll
    for (int j = 0; j < MG_BN / 8; ++j) {
        const int n = n0 + 8 * j + 2 * (lane & 3);
        if (n >= p.N) continue;
        const bool two = n + 1 < p.N;
        if (GLU) {
            __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(p.out);
            if (pair0 >= 0) {
                y[size_t(pair0) * p.N + n] = __float2bfloat16_rn(gb_act_glu_clamped(acc[0][mi][j][0], acc[NB - 1][mi][j][0], p.limit));
                if (two) y[size_t(pair0) * p.N + n + 1] = __float2bfloat16_rn(gb_act_glu_clamped(acc[0][mi][j][1], acc[NB - 1][mi][j][1], p.limit));
            }
            if (pair1 >= 0) {
                y[size_t(pair1) * p.N + n] = __float2bfloat16_rn(gb_act_glu_clamped(acc[0][mi][j][2], acc[NB - 1][mi][j][2], p.limit));
                if (two) y[size_t(pair1) * p.N + n + 1] = __float2bfloat16_rn(gb_act_glu_clamped(acc[0][mi][j][3], acc[NB - 1][mi][j][3], p.limit));
            }
        } else {
            float* z = reinterpret_cast<float*>(p.out);
            if (pair0 >= 0) {
                z[size_t(pair0) * p.N + n] = acc[0][mi][j][0];
                if (two) z[size_t(pair0) * p.N + n + 1] = acc[0][mi][j][1];
            }
            if (pair1 >= 0) {
                z[size_t(pair1) * p.N + n] = acc[0][mi][j][2];
                if (two) z[size_t(pair1) * p.N + n + 1] = acc[0][mi][j][3];
            }
        }
    }
    }
}

// out[t, n] (+)= sum_r weights[t, r] z[t * top + r, n], the choices in their order.
__global__ void moe_combine_kernel(const float* __restrict__ z, const float* __restrict__ weights, int top, int N,
                                   float* __restrict__ out, int accumulate, long long total, const MoeIdentity id) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / N;
    const int n = int(i - t * N);
    float acc = 0.f;
    for (int r = 0; r < top; ++r) {
        const bool own = id.ids && id.ids[t * top + r] >= id.n_real;
        acc = fmaf(weights[t * top + r], own ? gb_load(id.h, id.h_dtype, size_t(t) * id.ldh + n) : z[(t * top + r) * N + n], acc);
    }
    out[i] = accumulate ? out[i] + acc : acc;
}

GB_API int gb_moe_grouped_supported(int K, int F) { return K % 8 == 0 && F % 8 == 0; }

// ints of scratch for T tokens: offsets, perm, tiles, n_tiles
GB_API long long gb_moe_grouped_scratch_ints(int T, int top, int E) {
    const long long pairs = (long long)T * top;
    return (E + 1) + pairs + 2 * ((pairs + MG_BM - 1) / MG_BM + E) + 1;
}

// h bfloat16 [T, K] rows ldh apart; ids [T, top], weights [T, top]; wg, wu [E, F, K], wd [E, N, F] bfloat16 contiguous;
// y bfloat16 [T*top, F], z float [T*top, N] scratch; out float [T, N] (added to when accumulate).  E counts all experts
// that ids may name; those numbered n_real and above are identity experts without matrices (then N = K).
GB_API int gb_moe_grouped(const void* h, long long ldh, int T, int K, int F, int N, int E, int top, const int* ids,
                          const float* weights, const void* wg, const void* wu, const void* wd, float limit, void* y, float* z,
                          int* scratch, float* out, int accumulate, int n_real, cudaStream_t stream) {
    GB_REQUIRE(n_real > 0 && n_real <= E && (n_real == E || N == K), "gb_moe_grouped: %d of %d experts have matrices (rows of %d and %d)", n_real, E, K, N);
    GB_REQUIRE(gb_moe_grouped_supported(K, F), "gb_moe_grouped: sizes K=%d F=%d must be multiples of 8", K, F);
    GB_REQUIRE(E > 0 && E <= 1024 && top > 0 && N > 0 && limit > 0.f && (ldh % 8) == 0, "gb_moe_grouped: bad sizes");
    GB_REQUIRE(((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(wg) | reinterpret_cast<uintptr_t>(wu) |
                 reinterpret_cast<uintptr_t>(wd) | reinterpret_cast<uintptr_t>(y)) & 15) == 0, "gb_moe_grouped: misaligned operands");
    if (T == 0) return 0;
    const int pairs = T * top, max_tiles = (pairs + MG_BM - 1) / MG_BM + E;
    int* offsets = scratch;
    int* perm = offsets + E + 1;
    int* tiles = perm + pairs;
    int* n_tiles = tiles + 2 * max_tiles;
    moe_sort_kernel<<<1, 1024, 0, stream>>>(ids, pairs, E, offsets, perm, tiles, n_tiles, nullptr);
    GB_LAUNCH_OK("gb_moe_grouped (sort)");
    static bool configured = false;
    constexpr int SMEM_GLU = MG_STAGES * (MG_BM + 2 * MG_BN) * MG_BK * 2, SMEM_ONE = MG_STAGES * (MG_BM + MG_BN) * MG_BK * 2;
    if (!configured) {
        if (cudaFuncSetAttribute(moe_grouped_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_GLU) != cudaSuccess ||
            cudaFuncSetAttribute(moe_grouped_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ONE) != cudaSuccess)
            return gb_fail("gb_moe_grouped: cannot get %d bytes of shared memory", SMEM_GLU);
        configured = true;
    }
    GB_REQUIRE(max_tiles <= 65535, "gb_moe_grouped: %d tiles of pairs are too many for one launch", max_tiles);
    MgParams p;
    p.a = (const __nv_bfloat16*)h; p.w0 = (const __nv_bfloat16*)wg; p.w1 = (const __nv_bfloat16*)wu; p.out = y;
    p.offsets = offsets; p.perm = perm; p.tiles = tiles; p.n_tiles = n_tiles; p.lda = ldh; p.a_div = top; p.N = F; p.K = K;
    p.limit = limit; p.n_real = n_real;
    moe_grouped_kernel<true><<<dim3((F + MG_BN - 1) / MG_BN, max_tiles), MG_THREADS, SMEM_GLU, stream>>>(p);
    GB_LAUNCH_OK("gb_moe_grouped (gate, up)");
    p.a = (const __nv_bfloat16*)y; p.w0 = (const __nv_bfloat16*)wd; p.w1 = nullptr; p.out = z; p.lda = F; p.a_div = 1;
    p.N = N; p.K = F;
    moe_grouped_kernel<false><<<dim3((N + MG_BN - 1) / MG_BN, max_tiles), MG_THREADS, SMEM_ONE, stream>>>(p);
    GB_LAUNCH_OK("gb_moe_grouped (down)");
    const long long total = (long long)T * N;
    MoeIdentity id;
    id.ids = n_real < E ? ids : nullptr; id.h = h; id.ldh = ldh; id.n_real = n_real; id.h_dtype = GB_BF16;
    moe_combine_kernel<<<unsigned((total + 255) / 256), 256, 0, stream>>>(z, weights, top, N, out, accumulate, total, id);
    GB_LAUNCH_OK("gb_moe_grouped (sum)");
    return 0;
}

// The pieces of the path that runs every expert's products as ordinary products over its own rows (the caller reads the
// experts' offsets on the host and launches them): pairs sorted by expert (offsets [E + 1], perm and place_of [T * top]),
// the tokens' rows gathered in that order, and at the end the weighted sum per token over rows in that order.
GB_API int gb_moe_sort(const int* ids, int T, int top, int E, int* offsets, int* perm, int* place_of, int* tiles_scratch,
                       cudaStream_t stream) {
    GB_REQUIRE(E > 0 && E <= 1024 && top > 0 && T >= 0, "gb_moe_sort: bad sizes");
    if (T == 0) return 0;
    const int pairs = T * top, max_tiles = (pairs + MG_BM - 1) / MG_BM + E;
    moe_sort_kernel<<<1, 1024, 0, stream>>>(ids, pairs, E, offsets, perm, tiles_scratch, tiles_scratch + 2 * max_tiles, place_of);
    GB_LAUNCH_OK("gb_moe_sort");
    return 0;
}

GB_API int gb_moe_gather_rows(const void* h, long long ldh, int T, int K, int top, const int* perm, void* rows, cudaStream_t stream) {
    GB_REQUIRE(K % 8 == 0 && ldh % 8 == 0 && ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(rows)) & 15) == 0,
               "gb_moe_gather_rows: rows of %d bfloat16 entries must be multiples of 16 bytes and aligned", K);
    if (T == 0) return 0;
    const long long total = (long long)T * top * (K / 8);
    moe_gather_rows_kernel<<<unsigned((total + 255) / 256), 256, 0, stream>>>((const uint4*)h, ldh / 8, perm, top, K / 8, (uint4*)rows, total);
    GB_LAUNCH_OK("gb_moe_gather_rows");
    return 0;
}

// ids, n_real, h (rows ldh apart): pairs whose expert is numbered n_real or above take the token's row of h instead of a
// row of z (ids null: none do).
GB_API int gb_moe_combine_sorted(const float* z, const int* place_of, const float* weights, int T, int top, int N, float* out,
                                 int accumulate, const int* ids, int n_real, const void* h, int h_dtype, long long ldh,
                                 cudaStream_t stream) {
    if (T == 0) return 0;
    MoeIdentity id;
    id.ids = ids; id.h = h; id.ldh = ldh; id.n_real = n_real; id.h_dtype = h_dtype;
    const long long total = (long long)T * N;
    moe_combine_sorted_kernel<<<unsigned((total + 255) / 256), 256, 0, stream>>>(z, place_of, weights, top, N, out, accumulate, total, id);
    GB_LAUNCH_OK("gb_moe_combine_sorted");
    return 0;
}
