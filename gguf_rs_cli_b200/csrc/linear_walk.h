// The walk over tokens that every mixer with a state S <- diag(decay) S + k v^T shares (gla.cu).  A mixer's own
// preparation kernel writes, for every (token, head), 32-bit rows padded to multiples of four entries: what reads
// the state (q), what is written into it (k), the decays per key channel and the values; optionally one number
// whose product with the token's value is added to what the state gives.  Then gb_linear_walk_launch walks them.
#pragma once
#include "common.cuh"

struct LinearWalkRows {
    float* qkg;      // [T, H, 3, DA]: q, k, decays
    float* vf;       // [T, H, VA]
    float* bonus;    // [T, H, 4] (first entry counts), or null
    int DA, VA;
};

// Places of the rows in a scratch buffer of gb_linear_walk_scratch_floats(T, H, D, Dv) floats (16-byte aligned).
LinearWalkRows gb_linear_walk_rows(float* scratch, int T, int H, int D, int Dv, bool with_bonus);

// before: a token reads the state as the token before it left it.  state [slots, H, D, Dv] is read and renewed;
// out [T, H*Dv] float32 with rows ldo apart.  seg_scratch (gb_gla_segment_floats) lets long sequences be walked in
// segments side by side.  `who` names the caller in error messages.
int gb_linear_walk_launch(const LinearWalkRows& rows, bool before, float* state, float* out, long long ldo, const int* cu,
                          const int* slots, const int* qlens, int B, int H, int D, int Dv, int max_qlen, float* seg_scratch,
                          cudaStream_t stream, const char* who);
