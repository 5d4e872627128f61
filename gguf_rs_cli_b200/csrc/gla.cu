// Gated linear attention: per sequence and head a matrix S [D, Dv] (key channel i, value column j) that every
// token first shrinks row by row and then adds an outer product to, and reads out with its query:
//   alpha_i = sigmoid(z_i)^(1/tau) = exp(-softplus(-z_i) / tau),  z = a + bias      (32-bit)
//   S_ij <- alpha_i S_ij + k_i v_j;   o_j = sum_i S_ij q_i
// Two kernels, as for the delta rule (delta_rule.cu).  The first computes, for all tokens at once, what does not
// depend on the state: scaled queries, keys, decays and values as 32-bit rows padded to a multiple of four
// entries.  The second walks the tokens: a block takes a slice of columns of one (sequence, head); a column is
// shared by R lanes of a warp (R a power of two), lane r holding the NR rows r*NR .. r*NR + NR - 1 in registers;
// the read-out's sum over i ends with shuffles over those lanes.  The prepared rows of a few tokens at a time
// are copied into shared memory with cp.async, the next chunk while this one is worked on.  The state is read
// once at the start and written once at the end.  A sequence that brings many tokens is cut into segments that are walked
// side by side: every segment from a zero state, then the states at the segments' starts by a short carry
// (S <- diag(product of the segment's decays) S + the segment's own state), then every segment again from its start.
// The walk serves every mixer whose state obeys S <- diag(decay) S + k v^T: its two options are reading the state before
// the token's own update instead of after it, and a number per (token, head) times the token's value added to what is read
// (a bonus for the current token, or a skip path); a mixer brings its own preparation kernel (linear_walk.h).
#include <math.h>

#include "common.cuh"
#include "linear_walk.h"

struct GlaPrepParams {
    const void *q, *k, *v;          // q, k [T, H*D], v [T, H*Dv]: column slices of one buffer, rows `ld` apart
    const void* a;                  // [T, H*D] before the bias, rows ld_a apart
    const void* bias;               // [H*D]
    float* qkg;                     // [T, H, 3, DA]: scaled q, k, decays
    float* vf;                      // [T, H, VA]
    long long ld, ld_a;
    int dtype, a_dtype, w_dtype, H, D, Dv, DA, VA;
    float q_scale, inv_tau;
};

// One warp per (token, head).
__global__ void __launch_bounds__(128) gla_prep_kernel(const GlaPrepParams p) {
    const int t = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= p.H) return;
    const int D = p.D, DA = p.DA;
    float* o = p.qkg + (size_t(t) * p.H + h) * 3 * DA;
    const size_t row = size_t(t) * p.ld + size_t(h) * D;
    for (int d = lane; d < DA; d += 32) {
        float qv = 0.f, kv = 0.f, gv = 0.f;
        if (d < D) {
            qv = gb_load(p.q, p.dtype, row + d) * p.q_scale;
            kv = gb_load(p.k, p.dtype, row + d);
            const float z = gb_load(p.a, p.a_dtype, size_t(t) * p.ld_a + size_t(h) * D + d) + gb_load(p.bias, p.w_dtype, size_t(h) * D + d);
            const float sp = -z > 20.f ? -z : log1pf(expf(-z));          // softplus(-z) = -ln sigmoid(z)
            gv = expf(-sp * p.inv_tau);
        }
        o[d] = qv;
        o[DA + d] = kv;
        o[2 * DA + d] = gv;
    }
    float* vo = p.vf + (size_t(t) * p.H + h) * p.VA;
    for (int d = lane; d < p.VA; d += 32) vo[d] = d < p.Dv ? gb_load(p.v, p.dtype, size_t(t) * p.ld + size_t(h) * p.Dv + d) : 0.f;
}

struct GlaWalkParams {
    const float *qkg, *vf;          // what gla_prep_kernel wrote
    float* state;                   // [slots, H, D, Dv]
    float* out;                     // [T, H*Dv], rows ldo apart
    const int *cu, *slots, *qlens;
    long long ldo;
    int H, D, Dv, DA, VA, R, TC;
    // Long sequences are cut into segments of seg_len tokens that are walked side by side (n_seg of them per sequence in
    // the grid).  mode 0: one walk per sequence, from and into `state`.  mode 1: every segment from a zero state into
    // seg_state [B * n_seg, H, D, Dv], nothing read out.  mode 2: every segment from the state in seg_state (by then the
    // state at its start), read out, no state written.
    int mode, seg_len, n_seg;
    float* seg_state;
    const float* bonus;             // [T, H, 4] (first entry counts) or null: out += bonus * v
};

__device__ __forceinline__ void gla_cp16(float* dst, const float* src) {
    unsigned d = unsigned(__cvta_generic_to_shared(dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

// Blocks of the walk that share an SM when a lane holds up to 32 rows of S: a thread's registers are bounded so that this
// many fit.  Unbounded, the instance that reads the state first takes 187 registers and two blocks fit, the other 168 and
// three; a prompt of 2,048 tokens, 16 heads of 128 x 128, both passes: 0.77 ms with two blocks, 0.62 with three, 0.60 with four.
#define GLA_WALK_BLOCKS 4

// BEFORE: what a token reads is the state as the token before it left it (its own k v^T is not in it).
template <int NR, bool BEFORE>
__global__ void __launch_bounds__(128, NR <= 32 ? GLA_WALK_BLOCKS : 1) gla_walk_kernel(const GlaWalkParams p) {
    extern __shared__ __align__(16) float gla_sm[];
    float* sm = gla_sm;
    const int b = p.mode ? blockIdx.x / p.n_seg : blockIdx.x, seg = p.mode ? blockIdx.x % p.n_seg : 0, h = blockIdx.y;
    const int slot = p.slots[b], first = seg * p.seg_len;
    const int n = p.mode ? min(p.seg_len, p.qlens[b] - first) : p.qlens[b];
    if (slot < 0 || n <= 0) return;
    const int R = p.R, CW = 32 / R, CB = 4 * CW, D = p.D, Dv = p.Dv, DA = p.DA, TC = p.TC;
    const int RS = R * (NR + 4);                        // floats of one padded row of q, k or decays
    const int TOK = 3 * RS + CB + 4;                    // floats per token: q, k, decays, values of the slice, bonus
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane / CW, jj = lane - r * CW;
    const int col0 = blockIdx.z * CB;
    const int j = col0 + warp * CW + jj;
    const bool col_ok = j < Dv;
    float* sp = p.mode ? p.seg_state + (size_t(blockIdx.x) * p.H + h) * size_t(D) * Dv
                       : p.state + (size_t(slot) * p.H + h) * size_t(D) * Dv;
    float S[NR];
#pragma unroll
    for (int m = 0; m < NR; ++m) {
        const int i = r * NR + m;
        S[m] = (i < D && col_ok && p.mode != 1) ? sp[size_t(i) * Dv + j] : 0.f;
    }
    for (int i = threadIdx.x; i < 2 * TC * TOK; i += 128) sm[i] = 0.f;      // what no copy reaches stays zero
    __syncthreads();
    const int t0 = p.cu[b] + first;
    const int q4 = DA / 4, v4 = max(0, min(CB, p.VA - col0)) / 4;         // 16-byte pieces per row
    auto load_chunk = [&](int c0, int buf) {
        const int nt = min(TC, n - c0);
        float* base = sm + buf * TC * TOK;
        const int per = 3 * q4 + v4 + (p.bonus ? 1 : 0);
        for (int idx = threadIdx.x; idx < nt * per; idx += 128) {
            const int tt = idx / per, e = idx - tt * per;
            const size_t t = size_t(t0 + c0 + tt);
            float* row = base + tt * TOK;
            if (e == 3 * q4 + v4) {
                gla_cp16(row + 3 * RS + CB, p.bonus + (t * p.H + h) * 4);
            } else if (e < 3 * q4) {
                const int which = e / q4, k4 = e - which * q4, i = 4 * k4;
                gla_cp16(row + which * RS + (i / NR) * (NR + 4) + (i % NR), p.qkg + ((t * p.H + h) * 3 + which) * DA + i);
            } else {
                const int i = 4 * (e - 3 * q4);
                gla_cp16(row + 3 * RS + i, p.vf + (t * p.H + h) * p.VA + col0 + i);
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
            const float vj = row[3 * RS + warp * CW + jj];
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int m = 0; m < NR / 4; ++m) {
                const float4 gv = gg[m], kv = kk[m], qv = qq[m];
                if (BEFORE) {
                    o0 = fmaf(S[4 * m], qv.x, o0);     S[4 * m] = fmaf(kv.x, vj, S[4 * m] * gv.x);
                    o1 = fmaf(S[4 * m + 1], qv.y, o1); S[4 * m + 1] = fmaf(kv.y, vj, S[4 * m + 1] * gv.y);
                    o2 = fmaf(S[4 * m + 2], qv.z, o2); S[4 * m + 2] = fmaf(kv.z, vj, S[4 * m + 2] * gv.z);
                    o3 = fmaf(S[4 * m + 3], qv.w, o3); S[4 * m + 3] = fmaf(kv.w, vj, S[4 * m + 3] * gv.w);
                } else {
                    S[4 * m] = fmaf(kv.x, vj, S[4 * m] * gv.x);         o0 = fmaf(S[4 * m], qv.x, o0);
                    S[4 * m + 1] = fmaf(kv.y, vj, S[4 * m + 1] * gv.y); o1 = fmaf(S[4 * m + 1], qv.y, o1);
                    S[4 * m + 2] = fmaf(kv.z, vj, S[4 * m + 2] * gv.z); o2 = fmaf(S[4 * m + 2], qv.z, o2);
                    S[4 * m + 3] = fmaf(kv.w, vj, S[4 * m + 3] * gv.w); o3 = fmaf(S[4 * m + 3], qv.w, o3);
                }
            }
            float o = (o0 + o1) + (o2 + o3);
            for (int off = CW; off < 32; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
            if (p.bonus) o = fmaf(row[3 * RS + CB], vj, o);
            if (r == 0 && col_ok && p.mode != 1) p.out[size_t(t0 + c0 + tt) * p.ldo + size_t(h) * Dv + j] = o;
        }
        __syncthreads();                                   // this buffer is loaded again two chunks on
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (p.mode == 2) return;
#pragma unroll
    for (int m = 0; m < NR; ++m) {
        const int i = r * NR + m;
        if (i < D && col_ok) sp[size_t(i) * Dv + j] = S[m];
    }
}

// The product of a segment's decays per head and key channel: prod [B * n_seg, H, DA].
__global__ void __launch_bounds__(128) gla_decay_prod_kernel(const float* __restrict__ qkg, const int* __restrict__ cu,
                                                             const int* __restrict__ qlens, int H, int DA, int seg_len, int n_seg,
                                                             float* __restrict__ prod) {
    const int b = blockIdx.x / n_seg, seg = blockIdx.x % n_seg, h = blockIdx.y;
    const int first = seg * seg_len, n = min(seg_len, qlens[b] - first);
    if (n <= 0) return;
    const size_t t0 = size_t(cu[b] + first);
    for (int i = threadIdx.x; i < DA; i += blockDim.x) {
        float pr = 1.f;
        for (int t = 0; t < n; ++t) pr *= qkg[(((t0 + t) * H + h) * 3 + 2) * DA + i];
        prod[(size_t(blockIdx.x) * H + h) * DA + i] = pr;
    }
}

// From the segments' own states (walked from zero) to the states at their starts, in place, and the sequence's new state:
// S_0 = state; S_(s+1) = diag(prod_s) S_s + local_s.  One thread per entry of S.
__global__ void __launch_bounds__(256) gla_carry_kernel(float* __restrict__ state, float* __restrict__ seg_state,
                                                        const float* __restrict__ prod, const int* __restrict__ slots,
                                                        const int* __restrict__ qlens, int H, int D, int Dv, int DA, int seg_len,
                                                        int n_seg) {
    const int b = blockIdx.x, h = blockIdx.y;
    const int slot = slots[b], n = qlens[b];
    if (slot < 0 || n <= 0) return;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= D * Dv) return;
    const int i = e / Dv;
    float* sp = state + (size_t(slot) * H + h) * size_t(D) * Dv + e;
    float S = *sp;
    const int segs = (n + seg_len - 1) / seg_len;
    for (int s = 0; s < segs; ++s) {
        float* ls = seg_state + ((size_t(b) * n_seg + s) * H + h) * size_t(D) * Dv + e;
        const float local = *ls;
        *ls = S;
        S = fmaf(prod[((size_t(b) * n_seg + s) * H + h) * DA + i], S, local);
    }
    *sp = S;
}

// Rows per lane and lanes per column for key size D (the delta rule's shapes).
static void gla_shape(int D, int* nr, int* r) {
    int NR = D > 1024 ? 64 : D > 64 ? 32 : D > 32 ? 16 : 8, R = 1;
    while (R * NR < D) R <<= 1;
    *nr = NR;
    *r = R;
}

// Floats of scratch for the prepared rows of T tokens.
GB_API long long gb_gla_scratch_floats(int T, int H, int D, int Dv) {
    const long long DA = (D + 3) / 4 * 4, VA = (Dv + 3) / 4 * 4;
    return (long long)T * H * (3 * DA + VA);
}

// The same with room for a number per (token, head) behind the rows (four floats each).
GB_API long long gb_linear_walk_scratch_floats(int T, int H, int D, int Dv) {
    return gb_gla_scratch_floats(T, H, D, Dv) + (long long)T * H * 4;
}

// Sequences of more than GLA_SEG_FROM new tokens are walked in segments of GLA_SEG side by side: twice the arithmetic of one
// walk, on as many blocks as there are segments (a prompt of 2,048 tokens, 16 heads of 128 x 128: 1.02 ms as one walk).
constexpr int GLA_SEG = 128, GLA_SEG_FROM = 256;

// Floats of scratch for the segments' states and decay products of a step whose longest sequence brings max_qlen tokens
// (0: the step is walked sequence by sequence).
GB_API long long gb_gla_segment_floats(int B, int max_qlen, int H, int D, int Dv) {
    if (max_qlen <= GLA_SEG_FROM) return 0;
    const long long n_seg = (max_qlen + GLA_SEG - 1) / GLA_SEG, DA = (D + 3) / 4 * 4;
    return (long long)B * n_seg * H * ((long long)D * Dv + DA);
}

LinearWalkRows gb_linear_walk_rows(float* scratch, int T, int H, int D, int Dv, bool with_bonus) {
    LinearWalkRows r;
    r.DA = (D + 3) / 4 * 4;
    r.VA = (Dv + 3) / 4 * 4;
    r.qkg = scratch;
    r.vf = scratch + size_t(T) * H * 3 * r.DA;
    r.bonus = with_bonus ? r.vf + size_t(T) * H * r.VA : nullptr;
    return r;
}

int gb_linear_walk_launch(const LinearWalkRows& rows, bool before, float* state, float* out, long long ldo, const int* cu,
                          const int* slots, const int* qlens, int B, int H, int D, int Dv, int max_qlen, float* seg_scratch,
                          cudaStream_t stream, const char* who) {
    GB_REQUIRE(H > 0 && D > 0 && Dv > 0 && D <= 2048, "%s: bad sizes heads=%d dim=%d vdim=%d (dim up to 2048)", who, H, D, Dv);
    GB_REQUIRE(rows.qkg && (reinterpret_cast<uintptr_t>(rows.qkg) & 15) == 0, "%s: scratch missing or misaligned", who);
    const int DA = rows.DA, VA = rows.VA;
    GlaWalkParams p;
    p.qkg = rows.qkg; p.vf = rows.vf; p.bonus = rows.bonus; p.state = state; p.out = out; p.cu = cu; p.slots = slots; p.qlens = qlens;
    p.ldo = ldo; p.H = H; p.D = D; p.Dv = Dv; p.DA = DA; p.VA = VA;
    int NR, R;
    gla_shape(D, &NR, &R);
    const int CB = 4 * (32 / R);
    const int per_token = 4 * (3 * R * (NR + 4) + CB + 4);
    int TC = (20 * 1024) / per_token;                    // two buffers of at most 20 KB each
    TC = TC < 1 ? 1 : (TC > 16 ? 16 : TC);
    p.R = R; p.TC = TC;
    const size_t smem = size_t(2) * TC * per_token;
    GB_REQUIRE(smem <= 64 * 1024, "%s: key size %d needs %zu bytes of shared memory", who, D, smem);
    if (smem > 48 * 1024) {
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(gla_walk_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess ||
                cudaFuncSetAttribute(gla_walk_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess)
                return gb_fail("%s: cannot get %zu bytes of shared memory", who, smem);
            configured = true;
        }
    }
    dim3 grid(B, H, (Dv + CB - 1) / CB);
    GB_REQUIRE(grid.z <= 65535 && H <= 65535, "%s: too many heads or value columns", who);
    auto walk = [&](const GlaWalkParams& w, dim3 g) {
        if (before) {
            if (NR == 8) gla_walk_kernel<8, true><<<g, 128, smem, stream>>>(w);
            else if (NR == 16) gla_walk_kernel<16, true><<<g, 128, smem, stream>>>(w);
            else if (NR == 32) gla_walk_kernel<32, true><<<g, 128, smem, stream>>>(w);
            else gla_walk_kernel<64, true><<<g, 128, smem, stream>>>(w);
        } else {
            if (NR == 8) gla_walk_kernel<8, false><<<g, 128, smem, stream>>>(w);
            else if (NR == 16) gla_walk_kernel<16, false><<<g, 128, smem, stream>>>(w);
            else if (NR == 32) gla_walk_kernel<32, false><<<g, 128, smem, stream>>>(w);
            else gla_walk_kernel<64, false><<<g, 128, smem, stream>>>(w);
        }
    };
    p.mode = 0; p.seg_len = 0; p.n_seg = 1; p.seg_state = nullptr;
    if (max_qlen <= GLA_SEG_FROM || !seg_scratch) {
        walk(p, grid);
        GB_LAUNCH_OK(who);
        return 0;
    }
    const int n_seg = (max_qlen + GLA_SEG - 1) / GLA_SEG;
    float* prod = seg_scratch + size_t(B) * n_seg * H * size_t(D) * Dv;
    p.seg_len = GLA_SEG; p.n_seg = n_seg; p.seg_state = seg_scratch;
    dim3 seg_grid(B * n_seg, H, grid.z);
    p.mode = 1;
    walk(p, seg_grid);
    GB_LAUNCH_OK(who);
    gla_decay_prod_kernel<<<dim3(B * n_seg, H), 128, 0, stream>>>(p.qkg, cu, qlens, H, DA, GLA_SEG, n_seg, prod);
    GB_LAUNCH_OK(who);
    GB_REQUIRE((D * Dv + 255) / 256 <= 65535, "%s: state too large", who);
    gla_carry_kernel<<<dim3(B, H, (D * Dv + 255) / 256), 256, 0, stream>>>(state, seg_scratch, prod, slots, qlens, H, D, Dv, DA, GLA_SEG, n_seg);
    GB_LAUNCH_OK(who);
    p.mode = 2;
    walk(p, seg_grid);
    GB_LAUNCH_OK(who);
    return 0;
}

// q, k [T, H*D] and v [T, H*Dv]: column slices of one buffer with rows ld apart; a [T, H*D] the decay's
// projection before its bias [H*D]; state [slots, H, D, Dv] float32, read and renewed; out float32 [T, H*Dv].
GB_API int gb_gla(const void* q, const void* k, const void* v, int dtype, long long ld, const void* a, int a_dtype,
                  long long ld_a, const void* bias, int w_dtype, float inv_tau, float q_scale, float* state, float* out,
                  long long ldo, const int* cu, const int* slots, const int* qlens, int T, int B, int H, int D, int Dv,
                  float* scratch, int max_qlen, float* seg_scratch, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(a_dtype) && gb_is_dtype(w_dtype), "gb_gla: bad dtype");
    GB_REQUIRE(H > 0 && D > 0 && Dv > 0 && D <= 2048, "gb_gla: bad sizes heads=%d dim=%d vdim=%d (dim up to 2048)", H, D, Dv);
    GB_REQUIRE(inv_tau > 0.f, "gb_gla: the decay's exponent must be positive");
    GB_REQUIRE(scratch && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0, "gb_gla: scratch missing or misaligned");
    if (B == 0 || T == 0) return 0;
    const LinearWalkRows rows = gb_linear_walk_rows(scratch, T, H, D, Dv, false);
    GlaPrepParams pp;
    pp.q = q; pp.k = k; pp.v = v; pp.a = a; pp.bias = bias; pp.qkg = rows.qkg; pp.vf = rows.vf;
    pp.ld = ld; pp.ld_a = ld_a; pp.dtype = dtype; pp.a_dtype = a_dtype; pp.w_dtype = w_dtype; pp.H = H; pp.D = D; pp.Dv = Dv;
    pp.DA = rows.DA; pp.VA = rows.VA; pp.q_scale = q_scale; pp.inv_tau = inv_tau;
    GB_REQUIRE((H + 3) / 4 <= 65535, "gb_gla: too many heads (%d)", H);
    gla_prep_kernel<<<dim3(T, (H + 3) / 4), 128, 0, stream>>>(pp);
    GB_LAUNCH_OK("gb_gla (prepare)");
    return gb_linear_walk_launch(rows, false, state, out, ldo, cu, slots, qlens, B, H, D, Dv, max_qlen, seg_scratch, stream, "gb_gla");
}
