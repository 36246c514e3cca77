// Prompt form of the mixer with one constant decay per head (recurrent.cu, mode 2): the same sums, regrouped so that
// only the state's step from chunk to chunk is serial.  With chunks of LC rows of a sequence, n rows in a chunk, w the
// head's decay and S the state before the chunk:
//
//   pass 1  KV = sum_s w^(n-1-s) k_s v_s^T                                  per chunk, all chunks side by side
//   pass 2  S_before(chunk) = S ;  S <- w^n S + KV                           per state element, chunk after chunk
//   pass 3  o_t = w^(t+1) S_before^T q_t + sum_(s<=t) w^(t-s) (q_t . k_s) v_s   per chunk, all chunks side by side
//
// (t, s count rows within the chunk), then the unit norm, channel weights and gate (cm_scan_norm_gate).  Everything
// is float on the CUDA cores: products of 4 x 4 register tiles out of shared memory.  q, k and v may pass through
// silu as they are staged.  The chunks' states go through `scratch` [B][chunks][H][D][DV]; the sequence's state row
// receives the last one.  Rows of padding belong to no sequence and are never touched.
#include "common.cuh"
#include "recurrent.h"
#include <math.h>

#define LC 64                    // rows of a chunk
#define LT 256                   // threads of a block

struct ChunkGeom {
    int D4, DV4;                 // D and DV rounded up to multiples of 4: pitches of the staged operands
    int chunks;                  // chunks per sequence that the launch provides for
};

template <typename T>
__device__ __forceinline__ float lc_in(const T* p, bool act) {
    const float x = to_f32(*p);
    return act ? x * sigmoid_f32(x) : x;
}

// rows [t0, t0 + n) of operand `src` (row pitch ld, head offset applied) as floats into dst[r * pitch + c]; columns
// from `width` to `pitch` and rows from n to LC hold zeros.  `scale_rows`: row r is multiplied by pw[n - 1 - r].
template <typename T>
__device__ __forceinline__ bool lc_vec8(const T* src, long long ld, int width) {
    return width % 8 == 0 && ld % 8 == 0 && (((uintptr_t)src) & 15) == 0;
}

template <typename T>
__device__ __forceinline__ void lc_stage(float* dst, int pitch, const T* src, long long ld, int n, int width, bool act,
                                         const float* pw, bool scale_rows) {
    if (lc_vec8<T>(src, ld, width)) {            // 16-byte loads: width = pitch here (a multiple of 8)
        const int w8 = width >> 3;
        for (int e = threadIdx.x; e < LC * w8; e += LT) {
            const int r = e / w8, c = (e - r * w8) << 3;
            float x[8] = {};
            if (r < n) {
                load8f<T>(src + r * ld + c, x);
                const float f = scale_rows ? pw[n - 1 - r] : 1.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = (act ? x[i] * sigmoid_f32(x[i]) : x[i]) * f;
            }
            store8f<float>(dst + r * pitch + c, x);
        }
        return;
    }
    for (int e = threadIdx.x; e < LC * pitch; e += LT) {
        const int r = e / pitch, c = e - r * pitch;
        float x = 0.f;
        if (r < n && c < width) {
            x = lc_in<T>(src + r * ld + c, act);
            if (scale_rows) x *= pw[n - 1 - r];
        }
        dst[e] = x;
    }
}

// the same, transposed: dst[c * LC + r]; neighbouring threads take neighbouring rows
template <typename T>
__device__ __forceinline__ void lc_stage_t(float* dst, int pitch, const T* src, long long ld, int n, int width, bool act) {
    if (lc_vec8<T>(src, ld, width)) {            // a thread takes eight channels of its row; a warp's stores go to 32 banks
        for (int e = threadIdx.x; e < LC * (width >> 3); e += LT) {
            const int c = (e / LC) << 3, r = e % LC;
            float x[8] = {};
            if (r < n) {
                load8f<T>(src + r * ld + c, x);
                if (act) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) x[i] *= sigmoid_f32(x[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[(c + i) * LC + r] = x[i];
        }
        return;
    }
    for (int e = threadIdx.x; e < LC * pitch; e += LT) {
        const int c = e / LC, r = e - c * LC;
        dst[e] = (r < n && c < width) ? lc_in<T>(src + r * ld + c, act) : 0.f;
    }
}

__device__ __forceinline__ void lc_powers(float* pw, float w) {
    for (int i = threadIdx.x; i <= LC; i += LT) pw[i] = powf(w, (float)i);
}

// pass 1: grid (chunk, head, sequence)
template <typename T>
__global__ void __launch_bounds__(LT)
lightning_kv_kernel(const ScanArgs a, ChunkGeom geo, float* __restrict__ scratch) {
    extern __shared__ __align__(16) float lsm[];
    pdl_trigger();
    pdl_wait();
    const int j = blockIdx.x, hd = blockIdx.y, b = blockIdx.z;
    const int s0 = a.seq_start[b], len = a.seq_start[b + 1] - s0;
    if (j * LC >= len) return;
    const int n = min(LC, len - j * LC), D = a.D, DV = a.DV, D4 = geo.D4, DV4 = geo.DV4;
    float* pw = lsm;                             // [LC + 4]
    float* sk = pw + LC + 4;                     // [LC][D4], row r times w^(n - 1 - r)
    float* sv = sk + LC * D4;                    // [LC][DV4]
    lc_powers(pw, a.decay[hd]);
    __syncthreads();
    const long long row0 = (long long)s0 + j * LC;
    lc_stage<T>(sk, D4, (const T*)a.k + row0 * a.ldk + (long long)hd * D, a.ldk, n, D, a.qkv_act, pw, true);
    lc_stage<T>(sv, DV4, (const T*)a.v + row0 * a.ldv + (long long)hd * DV, a.ldv, n, DV, a.qkv_act, pw, false);
    __syncthreads();
    float* out = scratch + (((long long)b * geo.chunks + j) * a.H + hd) * D * DV;
    const int tiles_c = DV4 >> 2, tiles = (D4 >> 2) * tiles_c;
    for (int tile = threadIdx.x; tile < tiles; tile += LT) {
        const int d0 = (tile / tiles_c) << 2, c0 = (tile - (tile / tiles_c) * tiles_c) << 2;
        float acc[4][4] = {};
        for (int s = 0; s < n; ++s) {
            const float4 kv = *reinterpret_cast<const float4*>(sk + s * D4 + d0);
            const float4 vv = *reinterpret_cast<const float4*>(sv + s * DV4 + c0);
            const float kk[4] = {kv.x, kv.y, kv.z, kv.w}, vs[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(kk[x], vs[y], acc[x][y]);
        }
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y)
                if (d0 + x < D && c0 + y < DV) out[(long long)(d0 + x) * DV + c0 + y] = acc[x][y];
    }
}

// pass 2: a thread per state element of a head and sequence walks the chunks; scratch[chunk] <- the state before it
__global__ void __launch_bounds__(LT)
lightning_carry_kernel(const ScanArgs a, ChunkGeom geo, float* __restrict__ scratch) {
    pdl_trigger();
    pdl_wait();
    const int hd = blockIdx.y, b = blockIdx.z;
    const long long per = (long long)a.D * a.DV;
    const long long e = (long long)blockIdx.x * LT + threadIdx.x;
    const int len = a.seq_start[b + 1] - a.seq_start[b];
    if (e >= per || len <= 0) return;
    float* st = a.state + (long long)a.seq_slot[b] * a.state_stride + a.state_offset + hd * per + e;
    const float w = a.decay[hd], w_full = powf(w, (float)LC);
    float S = *st;
    const long long step = (long long)a.H * per;                    // from a chunk's slot to the next chunk's
    float* slot = scratch + ((long long)b * geo.chunks * a.H + hd) * per + e;
    const int n_chunks = (len + LC - 1) / LC;
    for (int j0 = 0; j0 < n_chunks; j0 += 8) {                      // eight chunks' sums are asked for at once
        float kv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) kv[u] = j0 + u < n_chunks ? slot[(j0 + u) * step] : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (j0 + u < n_chunks) {
                slot[(j0 + u) * step] = S;
                const int n = min(LC, len - (j0 + u) * LC);
                S = fmaf(n == LC ? w_full : powf(w, (float)n), S, kv[u]);
            }
        }
    }
    *st = S;
}

// pass 3: grid (chunk, head, sequence)
template <typename T>
__global__ void __launch_bounds__(LT)
lightning_out_kernel(const ScanArgs a, ChunkGeom geo, const float* __restrict__ scratch) {
    extern __shared__ __align__(16) float lsm[];
    pdl_trigger();
    pdl_wait();
    const int j = blockIdx.x, hd = blockIdx.y, b = blockIdx.z;
    const int s0 = a.seq_start[b], len = a.seq_start[b + 1] - s0;
    if (j * LC >= len) return;
    const int n = min(LC, len - j * LC), D = a.D, DV = a.DV, D4 = geo.D4, DV4 = geo.DV4;
    float* pw = lsm;                             // [LC + 4]
    float* qT = pw + LC + 4;                     // [D4][LC]
    float* kT = qT + D4 * LC;                    // [D4][LC]
    float* sv = kT + D4 * LC;                    // [LC][DV4]
    float* aT = sv + LC * DV4;                   // [LC (s)][LC (t)]: w^(t - s) (q_t . k_s) for s <= t, else 0
    lc_powers(pw, a.decay[hd]);
    const long long row0 = (long long)s0 + j * LC;
    lc_stage_t<T>(qT, D4, (const T*)a.q + row0 * a.ldq + (long long)hd * D, a.ldq, n, D, a.qkv_act);
    lc_stage_t<T>(kT, D4, (const T*)a.k + row0 * a.ldk + (long long)hd * D, a.ldk, n, D, a.qkv_act);
    lc_stage<T>(sv, DV4, (const T*)a.v + row0 * a.ldv + (long long)hd * DV, a.ldv, n, DV, a.qkv_act, pw, false);
    __syncthreads();
    // the chunk's own scores: LC / 4 x LC / 4 tiles of 4 x 4, one per thread (LT = 256)
    {
        const int t0 = (threadIdx.x >> 4) << 2, k0 = (threadIdx.x & 15) << 2;
        float acc[4][4] = {};
        if (k0 <= t0 + 3) {
            for (int d = 0; d < D; ++d) {
                const float4 qv = *reinterpret_cast<const float4*>(qT + d * LC + t0);
                const float4 kv = *reinterpret_cast<const float4*>(kT + d * LC + k0);
                const float qq[4] = {qv.x, qv.y, qv.z, qv.w}, kk[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                for (int x = 0; x < 4; ++x)
#pragma unroll
                    for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(qq[x], kk[y], acc[x][y]);
            }
        }
#pragma unroll
        for (int y = 0; y < 4; ++y)
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int t = t0 + x, s = k0 + y;
                aT[s * LC + t] = s <= t ? acc[x][y] * pw[t - s] : 0.f;
            }
    }
    __syncthreads();
    const float* Sb = scratch + (((long long)b * geo.chunks + j) * a.H + hd) * D * DV;
    float* R = a.raw + row0 * ((long long)a.H * DV) + (long long)hd * DV;
    const int tiles_c = DV4 >> 2, tiles = (LC >> 2) * tiles_c;
    const bool vec = DV % 4 == 0 && (((uintptr_t)scratch) & 15) == 0;
    for (int tile = threadIdx.x; tile < tiles; tile += LT) {
        const int t0 = (tile / tiles_c) << 2, c0 = (tile - (tile / tiles_c) * tiles_c) << 2;
        if (t0 >= n) continue;
        float own[4][4] = {}, old[4][4] = {};
        const int s_end = min(n, t0 + 4);
        for (int s = 0; s < s_end; ++s) {
            const float4 av = *reinterpret_cast<const float4*>(aT + s * LC + t0);
            const float4 vv = *reinterpret_cast<const float4*>(sv + s * DV4 + c0);
            const float aa[4] = {av.x, av.y, av.z, av.w}, vs[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) own[x][y] = fmaf(aa[x], vs[y], own[x][y]);
        }
        for (int d = 0; d < D; ++d) {
            const float4 qv = *reinterpret_cast<const float4*>(qT + d * LC + t0);
            float ss[4];
            if (vec) {
                const float4 sv4 = *reinterpret_cast<const float4*>(Sb + (long long)d * DV + c0);
                ss[0] = sv4.x; ss[1] = sv4.y; ss[2] = sv4.z; ss[3] = sv4.w;
            } else {
#pragma unroll
                for (int y = 0; y < 4; ++y) ss[y] = c0 + y < DV ? Sb[(long long)d * DV + c0 + y] : 0.f;
            }
            const float qq[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) old[x][y] = fmaf(qq[x], ss[y], old[x][y]);
        }
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y)
                if (t0 + x < n && c0 + y < DV)
                    R[(long long)(t0 + x) * a.H * DV + c0 + y] = fmaf(pw[t0 + x + 1], old[x][y], own[x][y]) * a.q_scale;
    }
}

// The shared memory the two chunk kernels need for heads of D x DV, in bytes (the larger of the two).
extern "C" long long cm_lightning_chunked_smem(int D, int DV) {
    const long long D4 = (D + 3) / 4 * 4, DV4 = (DV + 3) / 4 * 4;
    return (long long)sizeof(float) * (LC + 4 + 2 * D4 * LC + LC * DV4 + LC * LC);
}

extern "C" int cm_lightning_chunk_rows() { return LC; }

// The prompt form: B sequences of up to max_len rows each (found through seq_start); scratch holds at least
// B * ceil(max_len / 64) * H * D * DV floats.  Ends with the unit norm, channel weights and sigmoid gate.
extern "C" int cm_lightning_chunked(int dt, const ScanArgs* args, int B, int max_len, float* scratch, cudaStream_t st) {
    ScanArgs a = *args;
    if (B <= 0 || a.rows <= 0 || max_len <= 0) return CM_OK;
    if (a.D <= 0 || a.DV <= 0 || !a.raw || !scratch || !a.decay) CM_REFUSE("lightning_chunked: head sizes %d x %d, or a buffer is missing", a.D, a.DV);
    const long long smem = cm_lightning_chunked_smem(a.D, a.DV);
    if (smem > 200 * 1024) CM_REFUSE("lightning_chunked: heads of %d x %d do not fit shared memory", a.D, a.DV);
    ChunkGeom geo;
    geo.D4 = (a.D + 3) / 4 * 4;
    geo.DV4 = (a.DV + 3) / 4 * 4;
    geo.chunks = (max_len + LC - 1) / LC;
    const size_t smem1 = sizeof(float) * (LC + 4 + (size_t)LC * geo.D4 + (size_t)LC * geo.DV4);
    dim3 grid(geo.chunks, a.H, B), cgrid((unsigned)(((long long)a.D * a.DV + LT - 1) / LT), a.H, B);
#define LC_RUN(TT)                                                                                                       \
    do {                                                                                                                 \
        if (smem1 > 48 * 1024) cudaFuncSetAttribute(lightning_kv_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1); \
        if (smem > 48 * 1024) cudaFuncSetAttribute(lightning_out_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        cm_launch(lightning_kv_kernel<TT>, grid, LT, smem1, st, a, geo, scratch);                                        \
        CM_CHECK_LAUNCH();                                                                                               \
        cm_launch(lightning_carry_kernel, cgrid, LT, 0, st, a, geo, scratch);                                            \
        CM_CHECK_LAUNCH();                                                                                               \
        cm_launch(lightning_out_kernel<TT>, grid, LT, (size_t)smem, st, a, geo, (const float*)scratch);                  \
        CM_CHECK_LAUNCH();                                                                                               \
    } while (0)
    if (dt == DT_F32) LC_RUN(float);
    else if (dt == DT_BF16) LC_RUN(bf16);
    else return CM_ERR_DTYPE;
#undef LC_RUN
    return cm_scan_norm_gate(dt, 1, a, st);
}
