// What the kernels of the mixers with a matrix state take (recurrent.cu, lightning.cu); the Python binding fills the
// same record (kernels._ScanArgs).
#pragma once
#include <cuda_runtime.h>

struct ScanArgs {
    const void *q, *k, *v, *g;        // query (or receptance), key, value, output-gate pre-activation: activation rows
    long long ldq, ldk, ldv, ldg;     // row pitches, elements
    const float* decay;               // MODE 0: [rows][H * D] per-channel decay;  MODE 1: [rows][2 H] log gates (i, then f)
    const float* bonus;               // MODE 0: [H][D]
    const float* norm_w;              // [H * DV]
    void* out;                        // [rows][H * DV], pitch ldo
    long long ldo;
    float* state;                     // [slots][state_stride]; this mixer's part starts at state_offset
    long long state_stride, state_offset;
    const void* shift_src;            // MODE 0: the mixer's input rows [rows][W]; the last one is kept as the next step's
    int W;                            //         previous input, at the head of the state row (null: nothing kept)
    const int *seq_start, *seq_slot;
    int H, D, DV, KS;
    float q_scale, eps;
    float* raw;                       // [rows][H * DV] float: the heads' outputs before norm and gate
    long long rows;
    int qkv_act;                      // MODE 2: 1 = q, k and v pass through silu (in float) as they are staged
    int norm_all_heads;               // 1: the unit norm runs over all heads of a row together, not head by head
};

// The unit norm, channel weights and gate over a.raw (recurrent.cu): act 0 silu, 1 sigmoid.
int cm_scan_norm_gate(int dt, int act, const ScanArgs& a, cudaStream_t st);
