// Flat streaming kernels for ANY sequence length (fp32, 16-byte aligned tensor base): the same
// memcpy-like sweep and CTA-wide span scan as scan_flat.cuh, with row boundaries tracked per
// element instead of per float4, so that T need not be a multiple of 4.
//
// A unit of work is a run of whole rows (short rows) or one row (long rows); it covers the
// elements [E0, E1) of the flat tensor.  The CTA reads the aligned float4s that cover that
// range; the up to three elements before E0 and after E1 that share a float4 with it belong to
// other units: they are turned into identity maps on the way in and are not written on the way
// out (boundary float4s are written element by element, interior ones as one 16-byte store).
// An element is a row start when its offset from E0 is a multiple of T; its gate is zeroed in
// the recurrence exactly as in scan_flat.cuh.  The tensor's very last float4 may stick out past
// the allocation when rows*T is not a multiple of 4: it is read and written element by element.
#pragma once

#include "scan_common.cuh"

namespace ssb {
namespace flat_any {

struct Unit {
    int64_t e0, e1;      // element range of the unit in the flat tensor
    int64_t first_row;   // row index of element e0
};

template <int CAP>
__device__ __forceinline__ Unit unit_of(int64_t u, int64_t rows, int64_t T, int64_t rows_per_unit) {
    Unit x;
    x.first_row = u * rows_per_unit;
    const int64_t r1 = x.first_row + rows_per_unit < rows ? x.first_row + rows_per_unit : rows;
    x.e0 = x.first_row * T;
    x.e1 = r1 * T;
    return x;
}

// Rows per unit: as many whole rows as fit a span with room for 3 slack elements on each side.
template <int CAP>
__host__ __device__ inline int64_t rows_per_unit(int64_t T) {
    const int64_t fit = ((int64_t)CAP * 4 - 6) / T;
    return fit < 1 ? 1 : fit;
}

__device__ __forceinline__ float4 load4_guarded(const float *base, int64_t e4, int64_t n_total) {
    if (!SSB_INDEX_OK(e4, n_total + 3, 80)) return make_float4(0.f, 0.f, 0.f, 0.f);  // e4 may trail the end by up to 3 slack elements
    if (e4 + 4 <= n_total) return __ldcs(reinterpret_cast<const float4 *>(base + e4));
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    if (e4 < n_total) r.x = base[e4];
    if (e4 + 1 < n_total) r.y = base[e4 + 1];
    if (e4 + 2 < n_total) r.z = base[e4 + 2];
    return r;
}

__device__ __forceinline__ void store4_masked(float *base, int64_t e4, float4 v, unsigned ok) {
    if ((ok & 15u) == 15u) {
        __stcs(reinterpret_cast<float4 *>(base + e4), v);
    } else {
        if (ok & 1u) base[e4] = v.x;
        if (ok & 2u) base[e4 + 1] = v.y;
        if (ok & 4u) base[e4 + 2] = v.z;
        if (ok & 8u) base[e4 + 3] = v.w;
    }
}

// Per-float4 bookkeeping, packed in one word: bits 0-3 element belongs to the unit, bits 4-7
// element starts a row, bits 8-11 element ends a row.  `rel0` is the offset of the float4's first
// element from the unit's first element (-3 .. unit length), `len` the unit's length in elements;
// both fit 32 bits because a unit is at most one row or one span long.
__device__ __forceinline__ unsigned marks_of(int rel0, int len, uint32_t T) {
    unsigned m = 0u;
    uint32_t pos = rel0 >= 0 ? (uint32_t)rel0 % T : 0u;  // position of element 0 inside its row
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int rel = rel0 + j;
        if (rel >= 0) {
            if (rel < len) {
                m |= 1u << j;
                if (pos == 0u) m |= 16u << j;
                if (pos == T - 1u) m |= 256u << j;
            }
            pos++;
            if (pos == T) pos = 0u;
        }
    }
    return m;
}

__device__ __forceinline__ bool mk_ok(unsigned m, int k) { return (m >> k) & 1u; }
__device__ __forceinline__ bool mk_start(unsigned m, int k) { return (m >> (4 + k)) & 1u; }
__device__ __forceinline__ bool mk_end(unsigned m, int k) { return (m >> (8 + k)) & 1u; }
__device__ __forceinline__ bool mk_all(unsigned m) { return (m & 15u) == 15u; }
// Row of element e4+k (called only for row starts / ends when the caller passed per-row carries).
__device__ __forceinline__ int64_t row_of(int64_t e4, int k, const Unit &u, int64_t T) {
    return u.first_row + (e4 + k - u.e0) / T;
}

template <int THREADS, int U>
__global__ void __launch_bounds__(THREADS)
flat_any_fwd_kernel(const float *__restrict__ gate, const float *__restrict__ value, float *__restrict__ out,
                    int64_t rows, int64_t T, const float *__restrict__ h_in) {
    constexpr int NW = THREADS / 32;
    constexpr int NE = NW * U;
    static_assert(NE <= 32, "second-level scan is one warp wide");
    constexpr int CAP = THREADS * U;
    __shared__ float2 s_tot[2][NE];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t n_total = rows * T;
    const int64_t rpu = rows_per_unit<CAP>(T);
    const int64_t n_units = (rows + rpu - 1) / rpu;
    int buf = 0;

    for (int64_t un = blockIdx.x; un < n_units; un += gridDim.x) {
        const Unit u = unit_of<CAP>(un, rows, T, rpu);
        const int64_t v_lo = u.e0 / 4, v_hi = (u.e1 + 3) / 4;
        float carry = 0.f;
        for (int64_t first_vec = v_lo; first_vec < v_hi; first_vec += CAP) {
            const int n_vec = (int)(v_hi - first_vec < CAP ? v_hi - first_vec : CAP);
            float4 a[U], b[U];
            unsigned mk[U];
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int o = j * THREADS + tid;
                if (o < n_vec) {
                    const int64_t e4 = (first_vec + o) * 4;
                    a[j] = load4_guarded(gate, e4, n_total);
                    b[j] = load4_guarded(value, e4, n_total);
                    mk[j] = marks_of((int)(e4 - u.e0), (int)(u.e1 - u.e0), (uint32_t)T);
                } else {
                    a[j] = make_float4(1.f, 1.f, 1.f, 1.f);
                    b[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    mk[j] = 0u;
                }
            }
#pragma unroll
            for (int j = 0; j < U; j++) {
                float *av = reinterpret_cast<float *>(&a[j]), *bv = reinterpret_cast<float *>(&b[j]);
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    if (!mk_ok(mk[j], k)) { av[k] = 1.f; bv[k] = 0.f; }
                    if (mk_start(mk[j], k)) {
                        if (h_in != nullptr)
                            bv[k] = fmaf(av[k], h_in[row_of((first_vec + j * THREADS + tid) * 4, k, u, T)], bv[k]);
                        av[k] = 0.f;
                    }
                }
            }
            float A[U], B[U];
#pragma unroll
            for (int j = 0; j < U; j++) {
                B[j] = fmaf(a[j].y, b[j].x, b[j].y);
                B[j] = fmaf(a[j].z, B[j], b[j].z);
                B[j] = fmaf(a[j].w, B[j], b[j].w);
                A[j] = (a[j].x * a[j].y) * (a[j].z * a[j].w);
            }
#pragma unroll
            for (int j = 0; j < U; j++) warp_scan_forward<float>(A[j], B[j], lane);
            if (lane == 31) {
#pragma unroll
                for (int j = 0; j < U; j++) s_tot[buf][j * NW + warp] = make_float2(A[j], B[j]);
            }
            __syncthreads();
            float tA = 1.f, tB = 0.f;
            if (lane < NE) {
                const float2 t = s_tot[buf][lane];
                tA = t.x;
                tB = t.y;
            }
            warp_scan_forward<float>(tA, tB, lane);
            const float span_A = __shfl_sync(kFullMask, tA, NE - 1);
            const float span_B = __shfl_sync(kFullMask, tB, NE - 1);
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int q = j * NW + warp;
                float pA = __shfl_sync(kFullMask, tA, q > 0 ? q - 1 : 0);
                float pB = __shfl_sync(kFullMask, tB, q > 0 ? q - 1 : 0);
                if (q == 0) { pA = 1.f; pB = 0.f; }
                const float warp_start = fmaf(pA, carry, pB);
                float lA = __shfl_up_sync(kFullMask, A[j], 1);
                float lB = __shfl_up_sync(kFullMask, B[j], 1);
                if (lane == 0) { lA = 1.f; lB = 0.f; }
                float h = fmaf(lA, warp_start, lB);
                float4 o4;
                h = fmaf(a[j].x, h, b[j].x); o4.x = h;
                h = fmaf(a[j].y, h, b[j].y); o4.y = h;
                h = fmaf(a[j].z, h, b[j].z); o4.z = h;
                h = fmaf(a[j].w, h, b[j].w); o4.w = h;
                const int o = j * THREADS + tid;
                if (o < n_vec && SSB_INDEX_OK((first_vec + o) * 4, n_total + 3, 81)) store4_masked(out, (first_vec + o) * 4, o4, mk[j]);
            }
            carry = fmaf(span_A, carry, span_B);
            buf ^= 1;
        }
    }
}

template <int THREADS, int U>
__global__ void __launch_bounds__(THREADS)
flat_any_bwd_kernel(const float *__restrict__ gate, const float *__restrict__ hout, const float *__restrict__ gout,
                    float *__restrict__ ggate, float *__restrict__ gvalue, int64_t rows, int64_t T,
                    const float *__restrict__ c_in, const float *__restrict__ h_prev) {
    constexpr int NW = THREADS / 32;
    constexpr int NE = NW * U;
    static_assert(NE <= 32, "second-level scan is one warp wide");
    constexpr int CAP = THREADS * U;
    __shared__ float2 s_tot[2][NE];
    __shared__ float s_hw[2][NE];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t n_total = rows * T;
    const int64_t rpu = rows_per_unit<CAP>(T);
    const int64_t n_units = (rows + rpu - 1) / rpu;
    int buf = 0;

    for (int64_t un = blockIdx.x; un < n_units; un += gridDim.x) {
        const Unit u = unit_of<CAP>(un, rows, T, rpu);
        const int64_t v_lo = u.e0 / 4, v_hi = (u.e1 + 3) / 4;
        const int64_t n_pieces = (v_hi - v_lo + CAP - 1) / CAP;
        float carry = 0.f;
        for (int64_t piece = n_pieces - 1; piece >= 0; piece--) {
            const int64_t first_vec = v_lo + piece * CAP;
            const int n_vec = (int)(v_hi - first_vec < CAP ? v_hi - first_vec : CAP);
            float4 a[U], g[U], h[U];
            unsigned mk[U];
            // h just left of the piece (thread 0 only); a piece never starts at element 0 of the
            // tensor unless that element is a row start, in which case the value is not used
            float edge = 0.f;
            if (tid == 0 && first_vec > 0) edge = hout[first_vec * 4 - 1];
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int o = j * THREADS + tid;
                if (o < n_vec) {
                    const int64_t e4 = (first_vec + o) * 4;
                    a[j] = load4_guarded(gate, e4, n_total);
                    g[j] = load4_guarded(gout, e4, n_total);
                    h[j] = load4_guarded(hout, e4, n_total);
                    mk[j] = marks_of((int)(e4 - u.e0), (int)(u.e1 - u.e0), (uint32_t)T);
                } else {
                    a[j] = make_float4(1.f, 1.f, 1.f, 1.f);
                    g[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    h[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    mk[j] = 0u;
                }
            }
            float hb[U][4];  // for row starts: the caller's h just before the row (or 0)
#pragma unroll
            for (int j = 0; j < U; j++) {
                float *av = reinterpret_cast<float *>(&a[j]), *gv = reinterpret_cast<float *>(&g[j]);
                const int64_t e4 = (first_vec + j * THREADS + tid) * 4;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    hb[j][k] = 0.f;
                    if (!mk_ok(mk[j], k)) { av[k] = 1.f; gv[k] = 0.f; }
                    if (mk_end(mk[j], k) && c_in != nullptr) gv[k] += c_in[row_of(e4, k, u, T)];
                    if (mk_start(mk[j], k)) {
                        av[k] = 0.f;
                        if (h_prev != nullptr) hb[j][k] = h_prev[row_of(e4, k, u, T)];
                    }
                }
            }
            float A[U], D[U];
#pragma unroll
            for (int j = 0; j < U; j++) {
                D[j] = a[j].w * g[j].w;
                D[j] = a[j].z * (g[j].z + D[j]);
                D[j] = a[j].y * (g[j].y + D[j]);
                D[j] = a[j].x * (g[j].x + D[j]);
                A[j] = (a[j].x * a[j].y) * (a[j].z * a[j].w);
            }
#pragma unroll
            for (int j = 0; j < U; j++) warp_scan_reverse<float>(A[j], D[j], lane);
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < U; j++) s_tot[buf][j * NW + warp] = make_float2(A[j], D[j]);
            }
            if (lane == 31) {
#pragma unroll
                for (int j = 0; j < U; j++) s_hw[buf][j * NW + warp] = h[j].w;
            }
            __syncthreads();
            float tA = 1.f, tD = 0.f;
            if (lane < NE) {
                const float2 t = s_tot[buf][lane];
                tA = t.x;
                tD = t.y;
            }
            warp_scan_reverse<float>(tA, tD, lane);
            const float span_A = __shfl_sync(kFullMask, tA, 0);
            const float span_D = __shfl_sync(kFullMask, tD, 0);
#pragma unroll
            for (int j = U - 1; j >= 0; j--) {
                const int q = j * NW + warp;
                float pA = __shfl_sync(kFullMask, tA, q < 31 ? q + 1 : 31);
                float pD = __shfl_sync(kFullMask, tD, q < 31 ? q + 1 : 31);
                if (q == NE - 1) { pA = 1.f; pD = 0.f; }
                const float warp_start = fmaf(pA, carry, pD);
                float lA = __shfl_down_sync(kFullMask, A[j], 1);
                float lD = __shfl_down_sync(kFullMask, D[j], 1);
                if (lane == 31) { lA = 1.f; lD = 0.f; }
                float c = fmaf(lA, warp_start, lD);
                float hl = __shfl_up_sync(kFullMask, h[j].w, 1);
                if (lane == 0) hl = q > 0 ? s_hw[buf][q - 1] : edge;
                const float left[4] = {mk_start(mk[j], 0) ? hb[j][0] : hl, mk_start(mk[j], 1) ? hb[j][1] : h[j].x,
                                       mk_start(mk[j], 2) ? hb[j][2] : h[j].y, mk_start(mk[j], 3) ? hb[j][3] : h[j].z};
                float4 oa, og;
                float gb;
                gb = g[j].w + c; c = a[j].w * gb; og.w = gb; oa.w = gb * left[3];
                gb = g[j].z + c; c = a[j].z * gb; og.z = gb; oa.z = gb * left[2];
                gb = g[j].y + c; c = a[j].y * gb; og.y = gb; oa.y = gb * left[1];
                gb = g[j].x + c; og.x = gb; oa.x = gb * left[0];
                const int o = j * THREADS + tid;
                if (o < n_vec && SSB_INDEX_OK((first_vec + o) * 4, n_total + 3, 82)) {
                    store4_masked(ggate, (first_vec + o) * 4, oa, mk[j]);
                    store4_masked(gvalue, (first_vec + o) * 4, og, mk[j]);
                }
            }
            carry = fmaf(span_A, carry, span_D);
            buf ^= 1;
        }
    }
}

}  // namespace flat_any
}  // namespace ssb
