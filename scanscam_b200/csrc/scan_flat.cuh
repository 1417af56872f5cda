// "Flat" streaming kernels for the aligned fp32 rows layout (T % 4 == 0, 16-byte aligned).
//
// The [rows, T] matrix is swept like a memcpy sweeps a flat array: a CTA takes a span of
// consecutive float4s, thread i of the CTA loads float4 number j*THREADS + i of the span
// (j = 0..U-1), so every warp-wide load covers 512 contiguous bytes, a CTA covers a contiguous
// 16 KB per tensor, and the CTAs of the grid cover one contiguous window of memory at a time.
// That is the access pattern under which HBM delivers its best mixed read/write bandwidth.
//
// Row boundaries need no segment logic.  The scan is a fold of affine maps x -> a*x + b, and a
// map with a = 0 forgets everything to its left; setting the gate of the first element of
// every row to zero (and folding a caller-supplied carry into that element's value) turns the
// whole span into one ordinary scan.  A span is either a whole number of rows (T <= span
// capacity), or a piece of one long row walked left to right by the same CTA with the carry in
// a register.
//
// Inside a span: each thread folds its 4 elements, a shuffle scan composes the 32 lanes, the
// U*WARPS warp totals (at most 32) go through shared memory and are scanned once more by
// every warp redundantly (one __syncthreads per span), and each thread replays its 4 elements
// from its now-known starting value.
#pragma once

#include "scan_common.cuh"

namespace ssb {
namespace flat {

// Logistic function, for the entry points that take gate LOGITS: a = 1 / (1 + 2^(-z*log2(e))),
// as two special-function instructions (ex2.approx, rcp.approx; relative error ~2^-22) and two
// FP32 operations.  The span kernels have no slack for more arithmetic: with expf() and a true
// division the forward took 0.22 ms instead of 0.125 ms on 67 M elements, and __expf/__fdividef
// (which add range handling) were hardly better.
__device__ __forceinline__ float sigmoidf(float z) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
    return r;
}
__device__ __forceinline__ float4 sigmoid4(float4 z) {
    return make_float4(sigmoidf(z.x), sigmoidf(z.y), sigmoidf(z.z), sigmoidf(z.w));
}

// ---------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------
// SIGMOID: `gate` holds logits z and the gate is sigmoid(z), computed on the fly.
template <int THREADS, int U, bool SIGMOID = false>
__global__ void __launch_bounds__(THREADS)
flat_fwd_kernel(const float4 *__restrict__ gate, const float4 *__restrict__ value,
                float4 *__restrict__ out, int64_t rows, int64_t T4,
                const float *__restrict__ h_in) {
    constexpr int NW = THREADS / 32;
    constexpr int NE = NW * U;  // warp totals per span
    static_assert(NE <= 32, "second-level scan is one warp wide");
    constexpr int CAP = THREADS * U;  // span capacity in float4s
    __shared__ float2 s_tot[2][NE];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool long_rows = T4 > CAP;
    // Short rows: a span is `rps` whole rows.  Long rows: a span is a CAP-sized piece of a row.
    const int64_t rps = long_rows ? 1 : CAP / T4;
    const int64_t pieces = long_rows ? (T4 + CAP - 1) / CAP : 1;
    const int64_t n_units = long_rows ? rows : (rows + rps - 1) / rps;  // units handed to CTAs
    [[maybe_unused]] const int64_t extent = rows * T4;  // float4s per tensor: what a checked build tests indices against
    int buf = 0;

    for (int64_t unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
        float carry = 0.f;  // h at the end of the previous piece of a long row
        for (int64_t piece = 0; piece < pieces; piece++) {
            int64_t first_vec;
            int n_vec;
            if (long_rows) {
                first_vec = unit * T4 + piece * CAP;
                const int64_t left = T4 - piece * CAP;
                n_vec = (int)(left < CAP ? left : CAP);
            } else {
                first_vec = unit * rps * T4;
                const int64_t r_here = (rows - unit * rps) < rps ? (rows - unit * rps) : rps;
                n_vec = (int)(r_here * T4);
            }
            float4 a[U], b[U];
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int o = j * THREADS + tid;
                if (o < n_vec && SSB_INDEX_OK(first_vec + o, extent, 10)) {
                    a[j] = __ldcs(gate + first_vec + o);
                    if (SIGMOID) a[j] = sigmoid4(a[j]);
                    b[j] = __ldcs(value + first_vec + o);
                } else {
                    a[j] = make_float4(1.f, 1.f, 1.f, 1.f);
                    b[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            // Row starts: forget the left, fold the caller's carry into the first value.
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int o = j * THREADS + tid;
                if (o < n_vec) {
                    bool start;
                    int64_t row;
                    if (long_rows) {
                        start = (piece == 0 && o == 0);
                        row = unit;
                    } else {
                        const uint32_t p = (uint32_t)o % (uint32_t)T4;
                        start = (p == 0);
                        row = unit * rps + (uint32_t)o / (uint32_t)T4;
                    }
                    if (start) {
                        if (h_in != nullptr) b[j].x = fmaf(a[j].x, h_in[row], b[j].x);
                        a[j].x = 0.f;
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
            // Second level: every warp scans the NE warp totals (sequence order: j major).
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
                // exclusive prefix of warp totals before (j, warp)
                float pA = __shfl_sync(kFullMask, tA, q > 0 ? q - 1 : 0);
                float pB = __shfl_sync(kFullMask, tB, q > 0 ? q - 1 : 0);
                if (q == 0) { pA = 1.f; pB = 0.f; }
                const float warp_start = fmaf(pA, carry, pB);
                // exclusive prefix of lanes before this one inside the warp
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
                if (o < n_vec && SSB_INDEX_OK(first_vec + o, extent, 11)) __stcs(out + first_vec + o, o4);
            }
            carry = fmaf(span_A, carry, span_B);
            buf ^= 1;  // the next span writes the other buffer: one barrier per span suffices
        }
    }
}

// ---------------------------------------------------------------------------------------
// Fused backward: c_t = a_t*(g_t + c_{t+1}) folded from the right, gb_t = g_t + c_{t+1},
// ga_t = gb_t*h_{t-1}.  The gate of every row's first element is zeroed in the recurrence so
// that nothing leaks into the previous row; long rows are walked right to left.
// ---------------------------------------------------------------------------------------
// SIGMOID: `gate` holds logits z; the first output is the gradient with respect to z,
// grad_gate * a * (1 - a) with a = sigmoid(z).
template <int THREADS, int U, int MIN_CTAS = 0, bool SIGMOID = false>  // MIN_CTAS 0: no register cap requested
__global__ void __launch_bounds__(THREADS, MIN_CTAS)
flat_bwd_kernel(const float4 *__restrict__ gate, const float4 *__restrict__ hout,
                const float4 *__restrict__ gout, float4 *__restrict__ ggate,
                float4 *__restrict__ gvalue, int64_t rows, int64_t T4,
                const float *__restrict__ c_in, const float *__restrict__ h_prev) {
    constexpr int NW = THREADS / 32;
    constexpr int NE = NW * U;
    static_assert(NE <= 32, "second-level scan is one warp wide");
    constexpr int CAP = THREADS * U;
    __shared__ float2 s_tot[2][NE];
    __shared__ float s_hw[2][NE];  // last h of every warp's float4 row: the halo of the next warp

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool long_rows = T4 > CAP;
    const int64_t rps = long_rows ? 1 : CAP / T4;
    const int64_t pieces = long_rows ? (T4 + CAP - 1) / CAP : 1;
    const int64_t n_units = long_rows ? rows : (rows + rps - 1) / rps;
    [[maybe_unused]] const int64_t extent = rows * T4;  // float4s per tensor (checked builds)
    const float *h_scalar = reinterpret_cast<const float *>(hout);
    int buf = 0;

    for (int64_t unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
        float carry = 0.f;  // c entering this piece from the right
        for (int64_t piece = pieces - 1; piece >= 0; piece--) {
            int64_t first_vec;
            int n_vec;
            if (long_rows) {
                first_vec = unit * T4 + piece * CAP;
                const int64_t left = T4 - piece * CAP;
                n_vec = (int)(left < CAP ? left : CAP);
            } else {
                first_vec = unit * rps * T4;
                const int64_t r_here = (rows - unit * rps) < rps ? (rows - unit * rps) : rps;
                n_vec = (int)(r_here * T4);
            }
            float4 a[U], g[U], h[U];
            // h just left of the span: only thread 0 needs it, and only inside a long row; the
            // load is issued before the bulk loads so that it never sits on the critical path.
            float edge = 0.f;
            if (long_rows && tid == 0 && piece > 0 && SSB_INDEX_OK(first_vec * 4 - 1, extent * 4, 12)) edge = h_scalar[first_vec * 4 - 1];
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int o = j * THREADS + tid;
                if (o < n_vec && SSB_INDEX_OK(first_vec + o, extent, 10)) {
                    a[j] = __ldcs(gate + first_vec + o);
                    if (SIGMOID) a[j] = sigmoid4(a[j]);
                    g[j] = __ldcs(gout + first_vec + o);
                    h[j] = __ldcs(hout + first_vec + o);
                } else {
                    a[j] = make_float4(1.f, 1.f, 1.f, 1.f);
                    g[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    h[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            bool is_start[U];
            float h_before[U];  // for a row start: the caller's h just before the row (or 0)
            float a_first[U];   // the gate of the float4's first element before a row start zeroes it
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int o = j * THREADS + tid;
                is_start[j] = false;
                h_before[j] = 0.f;
                a_first[j] = a[j].x;
                if (o < n_vec) {
                    bool end;
                    int64_t row;
                    if (long_rows) {
                        is_start[j] = (piece == 0 && o == 0);
                        end = (piece == pieces - 1 && o == n_vec - 1);
                        row = unit;
                    } else {
                        const uint32_t p = (uint32_t)o % (uint32_t)T4;
                        is_start[j] = (p == 0);
                        end = (p == (uint32_t)T4 - 1);
                        row = unit * rps + (uint32_t)o / (uint32_t)T4;
                    }
                    if (is_start[j]) {
                        a[j].x = 0.f;
                        if (h_prev != nullptr) h_before[j] = h_prev[row];
                    }
                    if (end && c_in != nullptr) g[j].w += c_in[row];
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
            warp_scan_reverse<float>(tA, tD, lane);  // lanes >= NE hold the identity
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
                // h just left of this float4: the lane to the left, the previous warp's last lane
                // (through shared memory), or, for the span's very first float4, `edge`.
                float hl = __shfl_up_sync(kFullMask, h[j].w, 1);
                if (lane == 0) hl = q > 0 ? s_hw[buf][q - 1] : edge;
                if (is_start[j]) hl = h_before[j];
                float4 oa, og;
                float gb;
                gb = g[j].w + c; c = a[j].w * gb; og.w = gb; oa.w = gb * h[j].z;
                gb = g[j].z + c; c = a[j].z * gb; og.z = gb; oa.z = gb * h[j].y;
                gb = g[j].y + c; c = a[j].y * gb; og.y = gb; oa.y = gb * h[j].x;
                gb = g[j].x + c; og.x = gb; oa.x = gb * hl;
                if (SIGMOID) {  // chain rule through a = sigmoid(z): d a / d z = a (1 - a)
                    oa.x *= a_first[j] * (1.f - a_first[j]);
                    oa.y *= a[j].y * (1.f - a[j].y);
                    oa.z *= a[j].z * (1.f - a[j].z);
                    oa.w *= a[j].w * (1.f - a[j].w);
                }
                const int o = j * THREADS + tid;
                if (o < n_vec && SSB_INDEX_OK(first_vec + o, extent, 13)) {
                    __stcs(ggate + first_vec + o, oa);
                    __stcs(gvalue + first_vec + o, og);
                }
            }
            carry = fmaf(span_A, carry, span_D);
            buf ^= 1;
        }
    }
}

}  // namespace flat
}  // namespace ssb
