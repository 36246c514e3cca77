// What the kernels of the difference-of-two-maps attention take (diffattn.cu, diffattn_mma.cu); the Python binding
// fills the same record (kernels._DiffAttnArgs).
#pragma once

struct DiffAttnArgs {
    void* ctx;                   // [T][ldc]: H heads of DV channels
    long long ldc;
    const void* q;               // [T][ldq]: H heads of [map 1 | map 2], D channels each
    long long ldq;
    const void* gate;            // [T][ldg]: a logit per head, or null
    long long ldg;
    const void* pool;
    long long pages;
    const int* ptab;
    long long ptab_stride;
    const int *tok_seq, *tok_pos, *seq_start, *seq_pos0, *seq_slot;
    int T, B, H, G, D, DV, HDC, window, keep;
    float scale, lambda, out_scale, eps;
};
