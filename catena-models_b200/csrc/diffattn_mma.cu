// The tiles form of the difference-of-two-maps attention (diffattn.cu) on the tensor cores, for bfloat16 prompt
// steps: mma.sync m16n8k16 for q k^T of both maps and for the two probability-value products.
//
// One block = 64 queries of one head of one sequence, 16 per warp; keys come a cache page (64 positions) at a
// time, so a tile of keys is one contiguous piece of the layer's pages; the next page is copied (cp.async, two
// buffers) while the present one is multiplied.  Scores, maxima, exponentials and sums
// are float.  The probabilities stay 32-bit values on their way into the value product: p is cut into
// bfloat16(p) and bfloat16(p - bfloat16(p)), two products are issued, and their float sums carry p to within
// 2^-17 of its value (the values themselves are stored as bfloat16, so their side of the product is exact).
// Both maps keep an output tile in registers until the last key tile; then o = a1 - lambda a2, the unit norm
// over the head, the constant factor and the gate, as in the other forms.
//
// Head sizes: D and DV multiples of 16 up to 128; cache entries (HDC) and row pitches multiples of 8 elements.
#include "common.cuh"
#include <math.h>

#include "diffattn.h"

#define DM_BQ 64
#define DM_BK 64
#define DM_THREADS 128
#define DM_PAD 8

__device__ __forceinline__ void dm_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void dm_ldsm_x4_trans(uint32_t* r, const bf16* p) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// 16 bytes from global to shared memory without passing registers; `bytes` = 0 stores zeros instead
__device__ __forceinline__ void dm_copy16(bf16* dst, const bf16* src, int bytes) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(addr), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void dm_copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void dm_copy_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

__device__ __forceinline__ uint32_t dm_pack(float x, float y) {
    __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float dm_quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float dm_quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// One page of keys against a warp's 16 queries, both maps: scores, the maps' running maxima and sums, and the value
// products into the maps' output tiles.
template <int NV>
__device__ __forceinline__ void dm_tile(const DiffAttnArgs& a, const bf16* Qs, const bf16* Ks, const bf16* Vs, int ldk, int ldv,
                                        int k_now, int len, int q_lo, int q_hi, int q_last, float scale2, int warp, int gr,
                                        int tq, int lane, float (*mx)[2], float (*ls)[2], float (*O1)[4], float (*O2)[4]) {
    const int D = a.D, DV = a.DV;
        const bool all_seen = k_now + DM_BK - 1 <= q_lo && k_now + DM_BK - 1 < len && q_hi <= q_last &&
                              (a.window <= 0 || q_hi - k_now < a.window || k_now + DM_BK - 1 < a.keep);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float S[8][4];
#pragma unroll
            for (int n = 0; n < 8; ++n) S[n][0] = S[n][1] = S[n][2] = S[n][3] = 0.f;
            const bf16* qb = Qs + (warp * 16 + gr) * ldk + m * D + 2 * tq;
            const bf16* kb = Ks + gr * ldk + m * D + 2 * tq;
            for (int kd = 0; kd < D; kd += 16) {
                uint32_t af[4];
                af[0] = *reinterpret_cast<const uint32_t*>(qb + kd);
                af[1] = *reinterpret_cast<const uint32_t*>(qb + 8 * ldk + kd);
                af[2] = *reinterpret_cast<const uint32_t*>(qb + kd + 8);
                af[3] = *reinterpret_cast<const uint32_t*>(qb + 8 * ldk + kd + 8);
#pragma unroll
                for (int n = 0; n < 8; ++n) {
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kb + n * 8 * ldk + kd);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kb + n * 8 * ldk + kd + 8);
                    dm_mma(S[n], af, b0, b1);
                }
            }
            // scores in units of log2, masked by selection; the rows' maxima
            float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
            for (int n = 0; n < 8; ++n)
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    float s = S[n][x] * scale2;
                    if (!all_seen) {
                        const int kpos = k_now + n * 8 + 2 * tq + (x & 1), qpos = q_lo + gr + (x >> 1) * 8;
                        const bool vis = qpos <= q_last && kpos < len && kpos <= qpos &&
                                         (a.window <= 0 || qpos - kpos < a.window || kpos < a.keep);
                        s = vis ? s : -INFINITY;
                    }
                    S[n][x] = s;
                    if (x < 2) t0 = fmaxf(t0, s);
                    else t1 = fmaxf(t1, s);
                }
            const float n0 = fmaxf(mx[m][0], dm_quad_max(t0)), n1 = fmaxf(mx[m][1], dm_quad_max(t1));
            // a row that has seen nothing yet keeps zeros and a factor of one
            const float r0 = n0 == -INFINITY ? 0.f : n0, r1 = n1 == -INFINITY ? 0.f : n1;
            const float f0 = exp2f(mx[m][0] - r0), f1 = exp2f(mx[m][1] - r1);
            mx[m][0] = n0;
            mx[m][1] = n1;
            float add0 = 0.f, add1 = 0.f;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                S[n][0] = exp2f(S[n][0] - r0);
                S[n][1] = exp2f(S[n][1] - r0);
                S[n][2] = exp2f(S[n][2] - r1);
                S[n][3] = exp2f(S[n][3] - r1);
                add0 += S[n][0] + S[n][1];
                add1 += S[n][2] + S[n][3];
            }
            ls[m][0] = ls[m][0] * f0 + add0;
            ls[m][1] = ls[m][1] * f1 + add1;
            float (*O)[4] = m == 0 ? O1 : O2;
#pragma unroll
            for (int n = 0; n < NV; ++n) {
                O[n][0] *= f0;
                O[n][1] *= f0;
                O[n][2] *= f1;
                O[n][3] *= f1;
            }
            // O += P V with P as two bfloat16 terms; V's fragments through transposing matrix loads
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float pa = S[2 * kk + (x >> 1)][(x & 1) * 2], pb = S[2 * kk + (x >> 1)][(x & 1) * 2 + 1];
                    const __nv_bfloat162 hv = __floats2bfloat162_rn(pa, pb);
                    hi[x] = *reinterpret_cast<const uint32_t*>(&hv);
                    lo[x] = dm_pack(pa - __low2float(hv), pb - __high2float(hv));
                }
                const bf16* vb = Vs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + (lane >> 4) * 8;
#pragma unroll
                for (int n = 0; n < NV; n += 2) {
                    if (n * 8 < DV) {
                        uint32_t vf[4];
                        dm_ldsm_x4_trans(vf, vb + n * 8);
                        dm_mma(O[n], hi, vf[0], vf[1]);
                        dm_mma(O[n + 1], hi, vf[2], vf[3]);
                        dm_mma(O[n], lo, vf[0], vf[1]);
                        dm_mma(O[n + 1], lo, vf[2], vf[3]);
                    }
                }
            }
        }
}

// NV: n-tiles of 8 value channels that the output tiles are sized for (DV <= 8 NV).
template <int NV>
__global__ void __launch_bounds__(DM_THREADS, 1)
diff_attn_mma_kernel(const DiffAttnArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char dm_smem[];
    const int D = a.D, D2 = 2 * a.D, DV = a.DV, ldk = D2 + DM_PAD, ldv = DV + DM_PAD;
    bf16* Qs = reinterpret_cast<bf16*>(dm_smem);        // [64][2D + 8]
    bf16* Kb = Qs + DM_BQ * ldk;                         // two buffers of [64][2D + 8]
    bf16* Vb = Kb + 2 * DM_BK * ldk;                     // two buffers of [64][DV + 8]
    const int b = blockIdx.z, h = blockIdx.y, g = h / (a.H / a.G);
    const int s0 = a.seq_start[b], n_new = a.seq_start[b + 1] - s0;
    const int p0 = a.seq_pos0[b], len = p0 + n_new;
    const int q0 = p0 + blockIdx.x * DM_BQ;
    if (q0 >= len) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gr = lane >> 2, tq = lane & 3;
    const int nq = min(DM_BQ, len - q0), q_last = q0 + nq - 1;
    const int* prow = a.ptab + (long long)a.seq_slot[b] * a.ptab_stride;
    const bf16* Q = (const bf16*)a.q;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    {
        const int c8n = D2 >> 3;
        for (int e = threadIdx.x; e < DM_BQ * c8n; e += DM_THREADS) {
            const int r = e / c8n, c = (e - r * c8n) << 3;
            uint4 v = zero4;
            if (r < nq) v = *reinterpret_cast<const uint4*>(Q + (long long)(s0 + q0 - p0 + r) * a.ldq + (long long)h * D2 + c);
            *reinterpret_cast<uint4*>(Qs + r * ldk + c) = v;
        }
    }
    float O1[NV][4], O2[NV][4];
#pragma unroll
    for (int n = 0; n < NV; ++n)
#pragma unroll
        for (int x = 0; x < 4; ++x) O1[n][x] = O2[n][x] = 0.f;
    float mx[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}};     // [map][row g, row g + 8], in units of log2
    float ls[2][2] = {{0.f, 0.f}, {0.f, 0.f}};                              // this thread's share of the rows' sums
    const float scale2 = a.scale * 1.4426950408889634f;
    const int q_lo = q0 + warp * 16, q_hi = q_lo + 15;
    const int win_first = a.window > 0 ? max(0, q0 - a.window + 1) : 0;
    const int kept_end = a.window > 0 ? min(a.keep, q_last + 1) : 0;
    const int win_k0 = win_first / DM_BK * DM_BK;
    // a page's keys and values on their way into buffer `buf` (rows past the sequence's end arrive as zeros: a
    // probability of exactly zero times whatever an unwritten entry holds would not be zero)
    auto copy_page = [&](int k0, int buf) {
        const int page = prow[k0 / PAGE_TOKENS];
        const bf16* kt = kv_tile((const bf16*)a.pool, 0, a.pages, page, g, a.G, a.HDC);
        const bf16* vt = kv_tile((const bf16*)a.pool, 1, a.pages, page, g, a.G, a.HDC);
        bf16* Kd = Kb + buf * DM_BK * ldk;
        bf16* Vd = Vb + buf * DM_BK * ldv;
        const int c8k = D2 >> 3, c8v = DV >> 3;
        for (int e = threadIdx.x; e < DM_BK * c8k; e += DM_THREADS) {
            const int r = e / c8k, c = (e - r * c8k) << 3;
            dm_copy16(Kd + r * ldk + c, kt + (long long)r * a.HDC + c, k0 + r < len ? 16 : 0);
        }
        for (int e = threadIdx.x; e < DM_BK * c8v; e += DM_THREADS) {
            const int r = e / c8v, c = (e - r * c8v) << 3;
            dm_copy16(Vd + r * ldv + c, vt + (long long)r * a.HDC + c, k0 + r < len ? 16 : 0);
        }
    };
    // the pages that some query of the block sees: those with kept tokens, then from the first window's page on
    auto next_page = [&](int k0) {
        k0 += DM_BK;
        return (k0 >= kept_end && k0 < win_k0) ? win_k0 : k0;
    };
    int buf = 0;
    const int first = kept_end > 0 ? 0 : win_k0;
    copy_page(first, 0);
    dm_copy_commit();
    for (int k0 = first; k0 <= q_last; buf ^= 1) {
        const int k_now = k0;
        k0 = next_page(k0);
        if (k0 <= q_last) copy_page(k0, buf ^ 1);            // the next page travels while this one is multiplied
        dm_copy_commit();
        dm_copy_wait_all_but_one();
        __syncthreads();
        const bf16* Ks = Kb + buf * DM_BK * ldk;
        const bf16* Vs = Vb + buf * DM_BK * ldv;
        const bool skip = k_now > q_hi ||                                     // above the diagonal for this warp
                          (a.window > 0 && q_lo - (k_now + DM_BK - 1) >= a.window && k_now >= a.keep);   // before all its windows
        if (!skip) dm_tile<NV>(a, Qs, Ks, Vs, ldk, ldv, k_now, len, q_lo, q_hi, q_last, scale2, warp, gr, tq, lane, mx, ls, O1, O2);
        __syncthreads();                                     // the buffer is free for the copy after next
    }
    // the rows' sums, the difference of the maps, the head's unit norm, factor and gate
    float inv[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int r = 0; r < 2; ++r) inv[m][r] = 1.f / dm_quad_sum(ls[m][r]);
    float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
    for (int n = 0; n < NV; ++n) {
        if (n * 8 < DV) {
            O1[n][0] = O1[n][0] * inv[0][0] - a.lambda * (O2[n][0] * inv[1][0]);
            O1[n][1] = O1[n][1] * inv[0][0] - a.lambda * (O2[n][1] * inv[1][0]);
            O1[n][2] = O1[n][2] * inv[0][1] - a.lambda * (O2[n][2] * inv[1][1]);
            O1[n][3] = O1[n][3] * inv[0][1] - a.lambda * (O2[n][3] * inv[1][1]);
            ss0 += O1[n][0] * O1[n][0] + O1[n][1] * O1[n][1];
            ss1 += O1[n][2] * O1[n][2] + O1[n][3] * O1[n][3];
        }
    }
    ss0 = dm_quad_sum(ss0);
    ss1 = dm_quad_sum(ss1);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int qi = warp * 16 + gr + r * 8;
        if (qi >= nq) continue;
        const long long t = (long long)s0 + q0 - p0 + qi;
        float f = a.out_scale / sqrtf((r ? ss1 : ss0) / (float)DV + a.eps);
        if (a.gate) f *= sigmoid_f32(to_f32(((const bf16*)a.gate)[t * a.ldg + h]));
        bf16* out = (bf16*)a.ctx + t * a.ldc + (long long)h * DV + 2 * tq;
#pragma unroll
        for (int n = 0; n < NV; ++n)
            if (n * 8 < DV)
                *reinterpret_cast<__nv_bfloat162*>(out + n * 8) = __floats2bfloat162_rn(O1[n][2 * r] * f, O1[n][2 * r + 1] * f);
    }
}

template <int NV>
static int dm_launch(const DiffAttnArgs& a, int max_len, cudaStream_t st) {
    const size_t smem = ((size_t)(DM_BQ + 2 * DM_BK) * (2 * a.D + DM_PAD) + (size_t)2 * DM_BK * (a.DV + DM_PAD)) * sizeof(bf16);
    if (smem > 48 * 1024) cudaFuncSetAttribute(diff_attn_mma_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cm_launch(diff_attn_mma_kernel<NV>, dim3((max_len + DM_BQ - 1) / DM_BQ, a.H, a.B), DM_THREADS, smem, st, a);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// bfloat16 only.  Launched for sequences of up to max_len new tokens.
extern "C" int cm_diff_attn_mma(const DiffAttnArgs* args, int max_len, cudaStream_t st) {
    const DiffAttnArgs a = *args;
    if (a.T <= 0 || a.B <= 0 || max_len <= 0) return CM_OK;
    if (a.D % 16 || a.DV % 16 || a.D <= 0 || a.DV <= 0 || a.D > 128 || a.DV > 128)
        CM_REFUSE("diff_attn_mma: heads of 2 x %d and %d channels (multiples of 16 up to 128)", a.D, a.DV);
    if (a.HDC % 8 || 2 * a.D > a.HDC || a.DV > a.HDC || a.ldq % 8 || a.ldc % 2 || (((uintptr_t)a.q | (uintptr_t)a.pool) & 15) ||
        ((uintptr_t)a.ctx & 3))
        CM_REFUSE("diff_attn_mma: rows, cache entries (%d) or pointers are not aligned for 16-byte accesses", a.HDC);
    if (a.G <= 0 || a.H % a.G) CM_REFUSE("diff_attn_mma: %d query heads over %d key heads", a.H, a.G);
    if (a.DV <= 32) return dm_launch<4>(a, max_len, st);
    if (a.DV <= 64) return dm_launch<8>(a, max_len, st);
    if (a.DV <= 96) return dm_launch<12>(a, max_len, st);
    return dm_launch<16>(a, max_len, st);
}
