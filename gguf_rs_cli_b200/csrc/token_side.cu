// A per-layer input that depends on the token alone: every layer owns a slice of `dim` columns of a table with a row
// per token; the slice gates a low-rank view of the residual stream,
//   g[t, j] = act(a[t, j]) * table[token_t, offset + j],     j < dim,
// where a = W_gate x is the caller's product and act GELU in its tanh form (or SiLU).  The caller then projects g back to
// the model's width and norms it into the stream.  32-bit arithmetic.
#include "common.cuh"

__global__ void token_side_gate_kernel(const void* __restrict__ a, int a_dtype, long long lda, const void* __restrict__ table,
                                       int table_dtype, long long ldt, int offset, const int* __restrict__ tokens, int V,
                                       int dim, int act, void* __restrict__ out, int out_dtype, long long ldo, long long total) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / dim;
    const int j = int(i - t * dim);
    const int tok = tokens[t];
    float v = 0.f;
    if (tok >= 0 && tok < V)
        v = gb_gate_act(gb_load(a, a_dtype, size_t(t) * lda + j), act) * gb_load(table, table_dtype, size_t(tok) * ldt + offset + j);
    gb_store(out, out_dtype, size_t(t) * ldo + j, v);
}

// a [T, dim] rows lda apart; table [V, ldt] (the layer's slice starts at column `offset`); out [T, dim] rows ldo apart.
GB_API int gb_token_side_gate(const void* a, int a_dtype, long long lda, const void* table, int table_dtype, long long ldt,
                              int offset, const int* tokens, int V, int T, int dim, int act, void* out, int out_dtype,
                              long long ldo, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(a_dtype) && gb_is_dtype(table_dtype) && gb_is_dtype(out_dtype), "gb_token_side_gate: bad dtype");
    GB_REQUIRE(dim > 0 && offset >= 0 && offset + dim <= ldt && V > 0 && (act == GB_ACT_SILU || act == GB_ACT_GELU_TANH),
               "gb_token_side_gate: bad sizes dim=%d offset=%d row=%lld", dim, offset, ldt);
    if (T == 0) return 0;
    const long long total = (long long)T * dim;
    token_side_gate_kernel<<<unsigned((total + 255) / 256), 256, 0, stream>>>(a, a_dtype, lda, table, table_dtype, ldt, offset, tokens,
                                                                              V, dim, act, out, out_dtype, ldo, total);
    GB_LAUNCH_OK("gb_token_side_gate");
    return 0;
}
