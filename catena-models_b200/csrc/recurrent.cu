// Mixers with a matrix-valued state per head that is carried from token to token:
//
//   decay mix      o_t = (S + diag(u) k_t v_t^T)^T r_t ;  S <- diag(w_t) S + k_t v_t^T
//                  (per-channel decay w_t in (0, 1) that depends on the token, bonus u for the present token)
//   matrix memory  m' = max(f + m, i) ;  S <- e^(f + m - m') S + e^(i - m') k v^T ;  n likewise with k alone ;
//                  o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)         (log-domain gates i, f with a running maximum m)
//
// followed, in the same kernel, by the unit norm of each head's output, the channel weights and the output
// gate.  State, gates, decays and all sums are float whatever the activation type.  The state lives in
// per-slot rows of a float array; a step starts from what is stored there (zeros for a new sequence) and
// leaves its last state, so whole prompts, portions of prompts and single tokens run the same code and
// give the same numbers.  One block owns one head of one sequence and walks the sequence's rows of the
// step in order; rows that belong to no sequence (padding) are never touched.
//
// Beside it: the token shift (each projection reads its own blend of the present and the previous
// token's input), the low-rank decay network, and the capped gate pre-activations.
#include "common.cuh"
#include <math.h>

// ------------------------------------------------------------------------------ token shift
// out[s][t] = T(h[t] + (prev[t] - h[t]) * mu[s]) for s < S, prev[t] = h[t - 1] within a sequence's rows of
// the step, and the stored previous input (the head of the sequence's state row) for its first row.
template <typename T>
__global__ void shift_mix_kernel(T* __restrict__ out, const T* __restrict__ h, const float* __restrict__ mu,
                                 const float* __restrict__ state, long long state_stride,
                                 const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                 const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot, int S,
                                 long long rows, int W) {
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.x;
    const int b = tok_seq[t];
    if (b < 0) return;
    const bool first = tok_pos[t] == seq_pos0[b];
    const float* sp = state + (long long)seq_slot[b] * state_stride;
    const T* hp = h + (t - 1) * W;
    const T* hr = h + t * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float x = to_f32(hr[c]);
        const float d = (first ? sp[c] : to_f32(hp[c])) - x;
        for (int s = 0; s < S; ++s) out[((long long)s * rows + t) * W + c] = from_f32<T>(fmaf(d, mu[(long long)s * W + c], x));
    }
}

extern "C" int cm_shift_mix(int dt, void* out, const void* h, const float* mu, const float* state,
                            long long state_stride, const int* tok_seq, const int* tok_pos, const int* seq_pos0,
                            const int* seq_slot, int S, long long rows, int W, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    const int threads = W >= 1024 ? 256 : 128;
    if (dt == DT_F32)
        cm_launch(shift_mix_kernel<float>, (unsigned)rows, threads, 0, st, (float*)out, (const float*)h, mu, state,
                  state_stride, tok_seq, tok_pos, seq_pos0, seq_slot, S, rows, W);
    else if (dt == DT_BF16)
        cm_launch(shift_mix_kernel<bf16>, (unsigned)rows, threads, 0, st, (bf16*)out, (const bf16*)h, mu, state,
                  state_stride, tok_seq, tok_pos, seq_pos0, seq_slot, S, rows, W);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ------------------------------------------------------------------------- small row products
// A warp's dot products of one weight row with RT rows of x (float sums, lanes stride the columns).
#define RP_ROWS 4
#define RP_THREADS 256
template <typename T>
__device__ __forceinline__ void warp_row_dots(const T* __restrict__ wrow, const T* __restrict__ x, long long ldx,
                                              int n_rows, int W, float* acc) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int r = 0; r < RP_ROWS; ++r) acc[r] = 0.f;
    for (int c = lane; c < W; c += 32) {
        const float wv = to_f32(wrow[c]);
#pragma unroll
        for (int r = 0; r < RP_ROWS; ++r)
            if (r < n_rows) acc[r] = fmaf(wv, to_f32(x[r * ldx + c]), acc[r]);
    }
#pragma unroll
    for (int r = 0; r < RP_ROWS; ++r) acc[r] = warp_sum(acc[r]);
}

// Decay of the decay mix: w = exp(-exp(W2 tanh(W1 x) + w0)), per token and channel, in float.
// x [rows][W], W1 [R][W], W2 [C][R], w0 [C]; out [rows][C] float.
template <typename T>
__global__ void __launch_bounds__(RP_THREADS)
lowrank_decay_kernel(float* __restrict__ out, const T* __restrict__ x, const T* __restrict__ w1,
                     const T* __restrict__ w2, const float* __restrict__ w0, long long rows, int W, int R, int C) {
    extern __shared__ float th[];                     // [RP_ROWS][R]
    pdl_trigger();
    pdl_wait();
    const long long row0 = (long long)blockIdx.x * RP_ROWS;
    const int n_rows = (int)min((long long)RP_ROWS, rows - row0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < R; r += RP_THREADS / 32) {
        float acc[RP_ROWS];
        warp_row_dots<T>(w1 + (long long)r * W, x + row0 * W, W, n_rows, W, acc);
        if (lane == 0)
            for (int i = 0; i < RP_ROWS; ++i) th[i * R + r] = tanhf(acc[i]);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_rows * C; e += RP_THREADS) {
        const int i = e / C, c = e - i * C;
        float z = 0.f;
        const T* wr = w2 + (long long)c * R;
        for (int r = 0; r < R; ++r) z = fmaf(to_f32(wr[r]), th[i * R + r], z);
        out[(row0 + i) * C + c] = expf(-expf(z + w0[c]));
    }
}

extern "C" int cm_lowrank_decay(int dt, float* out, const void* x, const void* w1, const void* w2, const float* w0,
                                long long rows, int W, int R, int C, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    const size_t smem = (size_t)RP_ROWS * R * sizeof(float);
    if (smem > 48 * 1024) CM_REFUSE("lowrank_decay: rank %d is too large", R);
    const unsigned grid = (unsigned)((rows + RP_ROWS - 1) / RP_ROWS);
    if (dt == DT_F32)
        cm_launch(lowrank_decay_kernel<float>, grid, RP_THREADS, smem, st, out, (const float*)x, (const float*)w1,
                  (const float*)w2, w0, rows, W, R, C);
    else if (dt == DT_BF16)
        cm_launch(lowrank_decay_kernel<bf16>, grid, RP_THREADS, smem, st, out, (const bf16*)x, (const bf16*)w1,
                  (const bf16*)w2, w0, rows, W, R, C);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

__device__ __forceinline__ float log_sigmoid_f32(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// Capped gate pre-activations of the matrix memory: z = W h + b for 2 * H rows of W (input gates, then
// forget gates); out[t][o] = cap * tanh(z / cap), and the logarithm of its sigmoid for the forget gates.
template <typename T>
__global__ void __launch_bounds__(RP_THREADS)
capped_gates_kernel(float* __restrict__ out, const T* __restrict__ x, const T* __restrict__ w,
                    const float* __restrict__ bias, float cap, long long rows, int W, int H) {
    pdl_trigger();
    pdl_wait();
    const long long row0 = (long long)blockIdx.x * RP_ROWS;
    const int n_rows = (int)min((long long)RP_ROWS, rows - row0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int o = warp; o < 2 * H; o += RP_THREADS / 32) {
        float acc[RP_ROWS];
        warp_row_dots<T>(w + (long long)o * W, x + row0 * W, W, n_rows, W, acc);
        if (lane == 0)
            for (int i = 0; i < n_rows; ++i) {
                float g = cap * tanhf((acc[i] + bias[o]) / cap);
                if (o >= H) g = log_sigmoid_f32(g);
                out[(row0 + i) * 2 * H + o] = g;
            }
    }
}

extern "C" int cm_capped_gates(int dt, float* out, const void* x, const void* w, const float* bias, float cap,
                               long long rows, int W, int H, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    const unsigned grid = (unsigned)((rows + RP_ROWS - 1) / RP_ROWS);
    if (dt == DT_F32)
        cm_launch(capped_gates_kernel<float>, grid, RP_THREADS, 0, st, out, (const float*)x, (const float*)w, bias, cap, rows, W, H);
    else if (dt == DT_BF16)
        cm_launch(capped_gates_kernel<bf16>, grid, RP_THREADS, 0, st, out, (const bf16*)x, (const bf16*)w, bias, cap, rows, W, H);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ------------------------------------------------------------------------------ the scan
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
};

// MODE 0: decay mix.  MODE 1: matrix memory.  Thread (j, ks) owns column j of S for the key channels
// ks, ks + KS, ...; the KS partial outputs of a column are added in index order.
template <typename T, int MODE>
__global__ void matrix_scan_kernel(const ScanArgs a) {
    extern __shared__ float sm[];
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int hd = blockIdx.x, b = blockIdx.y;
    const int s0 = a.seq_start[b], s1 = a.seq_start[b + 1];
    if (s1 <= s0) return;
    const int D = a.D, DV = a.DV, KS = a.KS, H = a.H;
    float* S = sm;                       // [D][DV]
    float* qv = S + D * DV;              // [D] query / receptance
    float* kv = qv + D;                  // [D] key
    float* wv = kv + D;                  // [D] decay (MODE 0) / normaliser n (MODE 1)
    float* uv = wv + D;                  // [D] bonus (MODE 0)
    float* part = uv + D;                // [KS][DV]
    const int tid = threadIdx.x, nt = blockDim.x;
    const int j = tid % DV, ks = tid / DV;
    const bool active = ks < KS;
    const long long per_head = (long long)D * DV + (MODE == 1 ? D + 1 : 0);
    float* st = a.state + (long long)a.seq_slot[b] * a.state_stride + a.state_offset + hd * per_head;
    for (int e = tid; e < D * DV; e += nt) S[e] = st[e];
    float m = 0.f;
    if (MODE == 1) {
        for (int e = tid; e < D; e += nt) wv[e] = st[D * DV + e];
        m = st[D * DV + D];
    } else {
        for (int e = tid; e < D; e += nt) uv[e] = a.bonus[hd * D + e];
    }
    const T* Q = (const T*)a.q + (long long)hd * D;
    const T* K = (const T*)a.k + (long long)hd * D;
    const T* V = (const T*)a.v + (long long)hd * DV;
    const T* G = (const T*)a.g + (long long)hd * DV;
    T* O = (T*)a.out + (long long)hd * DV;
    const float nw = active && ks == 0 ? a.norm_w[hd * DV + j] : 0.f;
    for (long long t = s0; t < s1; ++t) {
        __syncthreads();                 // the vectors of the row before are no longer read; S and n are loaded
        for (int e = tid; e < D; e += nt) {
            qv[e] = to_f32(Q[t * a.ldq + e]) * a.q_scale;
            kv[e] = to_f32(K[t * a.ldk + e]);
            if (MODE == 0) wv[e] = a.decay[t * ((long long)H * D) + hd * D + e];
        }
        const float vj = active ? to_f32(V[t * a.ldv + j]) : 0.f;
        float af = 1.f, bi = 1.f;
        if (MODE == 1) {
            const float ig = a.decay[t * 2 * H + hd], fg = a.decay[t * 2 * H + H + hd];
            const float m_new = fmaxf(fg + m, ig);
            af = expf(fg + m - m_new);
            bi = expf(ig - m_new);
            m = m_new;
        }
        __syncthreads();
        float acc = 0.f;
        if (active) {
            for (int i = ks; i < D; i += KS) {
                const float s = S[i * DV + j], x = kv[i] * vj;
                if (MODE == 0) {
                    acc = fmaf(fmaf(uv[i], x, s), qv[i], acc);
                    S[i * DV + j] = fmaf(wv[i], s, x);
                } else {
                    const float s2 = fmaf(af, s, bi * x);
                    S[i * DV + j] = s2;
                    acc = fmaf(s2, qv[i], acc);
                }
            }
            part[ks * DV + j] = acc;
        }
        float den = 1.f;
        if (MODE == 1) {
            // n <- a n + b k, then n . q over the block in a fixed order
            float dot = 0.f;
            for (int e = tid; e < D; e += nt) {
                const float n2 = fmaf(af, wv[e], bi * kv[e]);
                wv[e] = n2;
                dot = fmaf(n2, qv[e], dot);
            }
            dot = block_sum(dot, scratch);
            den = fmaxf(fabsf(dot), expf(-m)) + 1e-6f;
        } else {
            __syncthreads();
        }
        float o = 0.f;
        if (active && ks == 0) {
            for (int x = 0; x < KS; ++x) o += part[x * DV + j];
            o /= den;
        }
        const float ss = block_sum(o * o, scratch);
        if (active && ks == 0) {
            const float inv = 1.f / sqrtf(ss / (float)DV + a.eps);
            const float gz = to_f32(G[t * a.ldg + j]);
            const float act = MODE == 0 ? gz * sigmoid_f32(gz) : sigmoid_f32(gz);
            O[t * a.ldo + j] = from_f32<T>(((o * inv) * nw) * act);
        }
    }
    __syncthreads();
    for (int e = tid; e < D * DV; e += nt) st[e] = S[e];
    if (MODE == 1) {
        for (int e = tid; e < D; e += nt) st[D * DV + e] = wv[e];
        if (tid == 0) st[D * DV + D] = m;
    } else if (hd == 0 && a.shift_src) {
        const T* last = (const T*)a.shift_src + (long long)(s1 - 1) * a.W;
        float* keep = a.state + (long long)a.seq_slot[b] * a.state_stride;
        for (int e = tid; e < a.W; e += nt) keep[e] = to_f32(last[e]);
    }
}

// mode 0: decay mix, mode 1: matrix memory.  B sequences; rows of the step are found through seq_start.
extern "C" int cm_matrix_scan(int dt, int mode, const ScanArgs* args, int B, cudaStream_t st) {
    ScanArgs a = *args;
    if (B <= 0) return CM_OK;
    if (a.D <= 0 || a.DV <= 0 || a.DV > 1024) CM_REFUSE("matrix_scan: head sizes %d x %d (values up to 1024)", a.D, a.DV);
    int ks = 256 / a.DV;
    if (ks < 1) ks = 1;
    if (ks > a.D) ks = a.D;
    a.KS = ks;
    const int threads = (a.DV * ks + 31) / 32 * 32;
    const size_t smem = ((size_t)a.D * a.DV + 4 * (size_t)a.D + (size_t)ks * a.DV) * sizeof(float);
    if (smem > 200 * 1024) CM_REFUSE("matrix_scan: a state of %d x %d floats does not fit shared memory", a.D, a.DV);
    dim3 grid(a.H, B);
#define SCAN_LAUNCH(TT, M)                                                                                      \
    do {                                                                                                        \
        if (smem > 48 * 1024)                                                                                   \
            cudaFuncSetAttribute(matrix_scan_kernel<TT, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        cm_launch(matrix_scan_kernel<TT, M>, grid, threads, smem, st, a);                                       \
    } while (0)
    if (dt == DT_F32 && mode == 0) SCAN_LAUNCH(float, 0);
    else if (dt == DT_F32 && mode == 1) SCAN_LAUNCH(float, 1);
    else if (dt == DT_BF16 && mode == 0) SCAN_LAUNCH(bf16, 0);
    else if (dt == DT_BF16 && mode == 1) SCAN_LAUNCH(bf16, 1);
    else return CM_ERR_DTYPE;
#undef SCAN_LAUNCH
    CM_CHECK_LAUNCH();
    return CM_OK;
}
