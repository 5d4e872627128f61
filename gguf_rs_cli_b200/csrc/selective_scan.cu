// The recurrence of a selective state-space mixer whose decay differs per channel AND per state entry (the selective
// scan of Mamba): per channel c and state entry n, with A = -exp(A_log),
//   dt_c = softplus(dt_raw_c + dt_bias_c);   S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;
//   y_c = sum_n S[c, n] C_n + D_c x_c;       out_c = y_c * silu(z_c)
// B and C [N] are shared by all channels of a token.  The state S [inner, N] lives in 32-bit floats per sequence and is
// carried from step to step; step sizes, their softplus, the decays' exponentials and every sum are 32-bit.
//
// A channel's N state entries are spread over `lpc` neighbouring lanes (a power of two) of SS_NS entries each, which
// stay in registers for the whole step; a token costs each lane SS_NS exponentials (exp2f of the step size times A log2 e:
// 481 instructions per token and channel with expf at 16 state entries) and 2 SS_NS multiply-adds, and the
// lanes of a channel add their shares of y by shuffles.  A block serves 128 / lpc channels of one sequence and walks the
// step's tokens in chunks of SS_CH: the chunk's B and C rows and the block's columns of dt, x and z are brought into
// shared memory together, so that the walk itself waits for no global load.
//
// Long prompts: the sequence is cut into segments that run side by side (gb_selective_scan with seg_scratch).  A first
// pass walks every segment from a zero state and keeps what it ends with and the sum of its step sizes; because the decay
// over a stretch of tokens is exp(A * sum of dt), the state in front of each segment follows by a short walk over the
// segments; the second pass then walks every segment from its true state and writes the results.
#include <math.h>

#include "common.cuh"

constexpr int SS_NS = 16;        // state entries per lane
constexpr int SS_CH = 16;        // tokens per chunk
constexpr int SS_THREADS = 128;
constexpr int SS_MAX_STATE = 256;
constexpr int SS_SEGMENT = 128;  // tokens per segment of a long prompt

struct ScanParams {
    const void *x, *z;            // [T, inner] each: the inputs behind convolution and activation, and the gate's rows
    long long ldx, ldz;
    const void* low;              // [T, R + 2N] of low_dtype: B from column R on, C from column R + N on
    long long ldl;
    const float* dt;              // [T, inner] float32, before bias and softplus
    long long lddt;
    const float *dt_bias, *a_log, *skip;     // [inner], [inner, N], [inner] float32
    float* state;                 // [slots, inner, N]
    void* out;                    // [T, inner]
    long long ldo;
    const int *cu, *slots, *qlens;
    float* seg;                   // segments of long prompts: per (sequence, segment) S_end [inner, N], then sum of dt [inner]
    int dtype, low_dtype, out_dtype, inner, N, R, lpc;
    int mode;                     // 0: whole sequences; 1: segments from zero, keep end state and sum of dt; 2: segments from their true state
    int max_segments;
};

__device__ __forceinline__ float ss_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// FULL: the state has a whole number of lanes' shares (N % SS_NS == 0): no entry is left out, and a lane reads its B and C
// entries of a token as four 16-byte pieces each.
template <bool FULL>
__global__ void __launch_bounds__(SS_THREADS) selective_scan_kernel(const ScanParams p) {
    extern __shared__ __align__(16) float ss_sm[];
    const int b = blockIdx.y;
    const int slot = p.slots[b];
    if (slot < 0) return;
    const int N = p.N, lpc = p.lpc, cpb = SS_THREADS / lpc;
    int first = p.cu[b], n_tok = p.qlens[b];
    const int seg = blockIdx.z;
    float* seg_rows = nullptr;
    if (p.mode != 0) {
        const int n_seg = (n_tok + SS_SEGMENT - 1) / SS_SEGMENT;
        if (seg >= n_seg) return;
        first += seg * SS_SEGMENT;
        n_tok = min(SS_SEGMENT, n_tok - seg * SS_SEGMENT);
        seg_rows = p.seg + (size_t(b) * p.max_segments + seg) * size_t(p.inner) * (N + 1);
    }
    float* bs = ss_sm;                         // [SS_CH][N]
    float* cs = bs + SS_CH * N;                // [SS_CH][N]
    float* dts = cs + SS_CH * N;               // [SS_CH][cpb]
    float* xs = dts + SS_CH * cpb;
    float* zs = xs + SS_CH * cpb;
    const int c0 = blockIdx.x * cpb;
    const int cl = threadIdx.x / lpc, part = threadIdx.x % lpc, n0 = part * SS_NS;
    const int c = c0 + cl;
    const bool live = c < p.inner;
    float A[SS_NS], S[SS_NS];
    float* srow = p.state + (size_t(slot) * p.inner + (live ? c : 0)) * N;
#pragma unroll
    for (int k = 0; k < SS_NS; ++k) {
        const bool in = live && n0 + k < N;
        A[k] = in ? -expf(p.a_log[size_t(c) * N + n0 + k]) * 1.4426950408889634f : 0.f;     // times log2(e): decays as powers of two
        S[k] = 0.f;
        if (in && p.mode == 0) S[k] = srow[n0 + k];
        // a segment's true start: the sequence's carried state for the first, else what the walk over the segments left
        if (in && p.mode == 2) S[k] = seg_rows[size_t(c) * N + n0 + k];
    }
    const float skip = live ? p.skip[c] : 0.f;
    float dt_sum = 0.f;
    for (int t0 = 0; t0 < n_tok; t0 += SS_CH) {
        const int n = min(SS_CH, n_tok - t0);
        __syncthreads();
        for (int j = 0; j < n; ++j) {
            const size_t t = size_t(first + t0 + j);
            const size_t row = t * p.ldl + p.R;
            for (int e = threadIdx.x; e < N; e += SS_THREADS) {
                bs[j * N + e] = gb_load(p.low, p.low_dtype, row + e);
                cs[j * N + e] = gb_load(p.low, p.low_dtype, row + N + e);
            }
            for (int i = threadIdx.x; i < cpb; i += SS_THREADS) {
                const int cc = c0 + i;
                const bool in = cc < p.inner;
                dts[j * cpb + i] = in ? ss_softplus(p.dt[t * p.lddt + cc] + p.dt_bias[cc]) : 0.f;
                xs[j * cpb + i] = in ? gb_load(p.x, p.dtype, t * p.ldx + cc) : 0.f;
                zs[j * cpb + i] = in && p.mode != 1 ? gb_load(p.z, p.dtype, t * p.ldz + cc) : 0.f;
            }
        }
        __syncthreads();
        for (int j = 0; j < n; ++j) {
            const float dtv = dts[j * cpb + cl], xv = xs[j * cpb + cl];
            const float dx = dtv * xv;
            const float* bj = bs + j * N + n0;
            const float* cj = cs + j * N + n0;
            float y = 0.f;
            if (FULL) {
                float ys[4] = {0.f, 0.f, 0.f, 0.f};          // four sums side by side, added in a fixed order
#pragma unroll
                for (int k4 = 0; k4 < SS_NS / 4; ++k4) {
                    const float4 b4 = reinterpret_cast<const float4*>(bj)[k4], c4 = reinterpret_cast<const float4*>(cj)[k4];
                    const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, cc4[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int k = 4 * k4 + e;
                        S[k] = fmaf(exp2f(dtv * A[k]), S[k], dx * bb[e]);
                        ys[e] = fmaf(S[k], cc4[e], ys[e]);
                    }
                }
                y = (ys[0] + ys[1]) + (ys[2] + ys[3]);
            } else {
#pragma unroll
                for (int k = 0; k < SS_NS; ++k) {
                    if (n0 + k < N) {
                        S[k] = fmaf(exp2f(dtv * A[k]), S[k], dx * bj[k]);
                        y = fmaf(S[k], cj[k], y);
                    }
                }
            }
            dt_sum += dtv;
            if (p.mode == 1) continue;
            for (int o = lpc >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (part == 0 && live) {
                const float zv = zs[j * cpb + cl];
                y = fmaf(skip, xv, y);
                gb_store(p.out, p.out_dtype, size_t(first + t0 + j) * p.ldo + c, y * (zv / (1.f + expf(-zv))));
            }
        }
    }
    if (!live) return;
    if (p.mode == 1) {
        // what the segment ends with from a zero state, and the sum of its step sizes
        float* e = seg_rows + size_t(p.inner) * N;
#pragma unroll
        for (int k = 0; k < SS_NS; ++k)
            if (n0 + k < N) seg_rows[size_t(c) * N + n0 + k] = S[k];
        if (part == 0) e[c] = dt_sum;
        return;
    }
    const bool last = p.mode == 0 || seg == (p.qlens[b] + SS_SEGMENT - 1) / SS_SEGMENT - 1;
    if (last) {
#pragma unroll
        for (int k = 0; k < SS_NS; ++k)
            if (n0 + k < N) srow[n0 + k] = S[k];
    }
}

// The walk over the segments of every sequence: segment g's true start is start(g - 1) * exp(A * sum of dt of g - 1) + what
// g - 1 ended with from zero; start(0) is the sequence's carried state.  In place: a segment's rows receive its start.
__global__ void __launch_bounds__(128) selective_scan_carry_kernel(const ScanParams p) {
    const int b = blockIdx.y;
    const int slot = p.slots[b];
    if (slot < 0) return;
    const int N = p.N;
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= (long long)p.inner * N) return;
    const int c = int(i / N);
    const int n_seg = (p.qlens[b] + SS_SEGMENT - 1) / SS_SEGMENT;
    const float a = -expf(p.a_log[i]);
    float s = p.state[size_t(slot) * p.inner * N + i];
    for (int g = 0; g < n_seg; ++g) {
        float* rows = p.seg + (size_t(b) * p.max_segments + g) * size_t(p.inner) * (N + 1);
        const float end = rows[i], sum = rows[size_t(p.inner) * N + c];
        rows[i] = s;
        s = fmaf(expf(a * sum), s, end);
    }
}

GB_API long long gb_selective_scan_segment_floats(int B, int max_qlen, int inner, int N) {
    if (max_qlen <= 2 * SS_SEGMENT) return 0;
    const long long n_seg = (max_qlen + SS_SEGMENT - 1) / SS_SEGMENT;
    return (long long)B * n_seg * inner * (N + 1);
}

// x, z [T, inner] (dtype, rows ldx / ldz apart); low [T, R + 2N] of low_dtype; dt float32 [T, inner]; dt_bias [inner], a_log
// [inner, N], skip [inner] float32; state float32 [slots, inner, N], read and renewed; out [T, inner] of out_dtype.
// seg_scratch: gb_selective_scan_segment_floats(B, max_qlen, inner, N) floats, or null (sequences walked whole).
GB_API int gb_selective_scan(const void* x, long long ldx, const void* z, long long ldz, int dtype, const void* low, int low_dtype,
                             long long ldl, int R, int N, const float* dt, long long lddt, const float* dt_bias, const float* a_log,
                             const float* skip, float* state, void* out, long long ldo, int out_dtype, const int* cu,
                             const int* slots, const int* qlens, int T, int B, int inner, int max_qlen, float* seg_scratch,
                             cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(out_dtype) && gb_is_dtype(low_dtype), "gb_selective_scan: bad dtype");
    GB_REQUIRE(inner > 0 && N > 0 && N <= SS_MAX_STATE && R >= 0, "gb_selective_scan: bad sizes inner=%d state=%d (1..%d)", inner, N, SS_MAX_STATE);
    GB_REQUIRE(x && z && low && dt && dt_bias && a_log && skip && state && out && cu && slots && qlens, "gb_selective_scan: arguments missing");
    if (B == 0 || T == 0) return 0;
    int lpc = 1;
    while (lpc * SS_NS < N) lpc *= 2;
    const int cpb = SS_THREADS / lpc;
    ScanParams p;
    p.x = x; p.z = z; p.ldx = ldx; p.ldz = ldz; p.low = low; p.ldl = ldl; p.dt = dt; p.lddt = lddt; p.dt_bias = dt_bias;
    p.a_log = a_log; p.skip = skip; p.state = state; p.out = out; p.ldo = ldo; p.cu = cu; p.slots = slots; p.qlens = qlens;
    p.seg = seg_scratch; p.dtype = dtype; p.low_dtype = low_dtype; p.out_dtype = out_dtype; p.inner = inner; p.N = N; p.R = R; p.lpc = lpc;
    p.max_segments = (max_qlen + SS_SEGMENT - 1) / SS_SEGMENT;
    const size_t smem = size_t(SS_CH) * (2 * N + 3 * cpb) * sizeof(float);
    const bool full = N % SS_NS == 0;
    const unsigned blocks = unsigned((inner + cpb - 1) / cpb);
    GB_REQUIRE(B <= 65535 && p.max_segments <= 65535, "gb_selective_scan: too many sequences or segments");
    if (!seg_scratch || max_qlen <= 2 * SS_SEGMENT) {
        p.mode = 0;
        if (full) selective_scan_kernel<true><<<dim3(blocks, B, 1), SS_THREADS, smem, stream>>>(p);
        else selective_scan_kernel<false><<<dim3(blocks, B, 1), SS_THREADS, smem, stream>>>(p);
        GB_LAUNCH_OK("gb_selective_scan");
        return 0;
    }
    p.mode = 1;
    if (full) selective_scan_kernel<true><<<dim3(blocks, B, p.max_segments), SS_THREADS, smem, stream>>>(p);
    else selective_scan_kernel<false><<<dim3(blocks, B, p.max_segments), SS_THREADS, smem, stream>>>(p);
    GB_LAUNCH_OK("gb_selective_scan (segments from zero)");
    const long long cells = (long long)inner * N;
    selective_scan_carry_kernel<<<dim3(unsigned((cells + 127) / 128), B), 128, 0, stream>>>(p);
    GB_LAUNCH_OK("gb_selective_scan (carry)");
    p.mode = 2;
    if (full) selective_scan_kernel<true><<<dim3(blocks, B, p.max_segments), SS_THREADS, smem, stream>>>(p);
    else selective_scan_kernel<false><<<dim3(blocks, B, p.max_segments), SS_THREADS, smem, stream>>>(p);
    GB_LAUNCH_OK("gb_selective_scan (segments)");
    return 0;
}
