// Token embedding plus a hashed embedding of the pair (previous token, token):
//   x[t,:] = table[token,:] * scale + pairs[row,:],
//   row = (previous * mul_prev + token * mul_cur) mod buckets, and row `buckets` (the table's last) for a sequence's first token.
// The previous token of a step's first token is per-sequence state (one int32 per slot), renewed with the step's last token
// by the block that read it.  The row arithmetic is 64-bit.  copy, when given, receives x once more (for models that add the
// embedding's result to the stream again later).
#include "common.cuh"

__global__ void __launch_bounds__(256) embed_bigram_kernel(const void* __restrict__ table, int table_dtype,
                                                           const void* __restrict__ pairs, int pairs_dtype,
                                                           const int* __restrict__ tokens, const int* __restrict__ pos,
                                                           const int* __restrict__ seq_of, const int* __restrict__ cu,
                                                           const int* __restrict__ slots, const int* __restrict__ qlens,
                                                           int* __restrict__ prev_token, int E, int V, int buckets,
                                                           long long mul_prev, long long mul_cur, float scale,
                                                           float* __restrict__ out, float* __restrict__ copy) {
    __shared__ int row_s;
    const int t = blockIdx.x, b = seq_of[t];
    const int tok = tokens[t];
    float* o = out + size_t(t) * E;
    float* c = copy ? copy + size_t(t) * E : nullptr;
    if (b < 0 || tok < 0 || tok >= V) {
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            o[i] = 0.f;
            if (c) c[i] = 0.f;
        }
        return;
    }
    if (threadIdx.x == 0) {
        const int first = cu[b];
        int prev;
        if (t == first) {
            int* keep = prev_token + slots[b];
            prev = *keep;
            *keep = tokens[first + qlens[b] - 1];
        } else {
            prev = tokens[t - 1];
        }
        long long r = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
        if (r < 0) r += buckets;
        row_s = pos[t] == 0 ? buckets : int(r);
    }
    __syncthreads();
    const size_t base = size_t(tok) * E, pbase = size_t(row_s) * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        const float v = gb_load(table, table_dtype, base + i) * scale + gb_load(pairs, pairs_dtype, pbase + i);
        o[i] = v;
        if (c) c[i] = v;
    }
}

// table [V, E]; pairs [buckets + 1, E]; prev_token int32 [slots]; out, copy float32 [T, E] (copy may be null).
GB_API int gb_embed_bigram(const void* table, int table_dtype, const void* pairs, int pairs_dtype, const int* tokens,
                           const int* pos, const int* seq_of, const int* cu, const int* slots, const int* qlens,
                           int* prev_token, int T, int E, int V, int buckets, long long mul_prev, long long mul_cur,
                           float scale, float* out, float* copy, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(table_dtype) && gb_is_dtype(pairs_dtype), "gb_embed_bigram: bad dtype");
    GB_REQUIRE(T >= 0 && E > 0 && V > 0 && buckets > 0 && prev_token, "gb_embed_bigram: bad sizes T=%d E=%d V=%d buckets=%d", T, E, V, buckets);
    if (T == 0) return 0;
    embed_bigram_kernel<<<T, 256, 0, stream>>>(table, table_dtype, pairs, pairs_dtype, tokens, pos, seq_of, cu, slots, qlens,
                                               prev_token, E, V, buckets, mul_prev, mul_cur, scale, out, copy);
    GB_LAUNCH_OK("gb_embed_bigram");
    return 0;
}
