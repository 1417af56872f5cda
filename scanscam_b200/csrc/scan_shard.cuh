// Row maps of one shard of a sequence that is split along T across devices.
//
// A shard of a row is the affine map h_end = A*h_start + B (forward) or c_first = A*c_in + D
// (the reverse recurrence c_t = a_t*(g_t + c_{t+1})).  The map is needed only by the OTHER
// shards, as the state their part of the row starts from, so it has to exist before the exchange;
// the shard's own scan comes after it.  Computing the map by folding the whole shard would read
// two tensors once more (8 bytes per element on top of the scan's 12 or 20).
//
// This kernel folds the shard from the far end instead -- the forward map from the shard's LAST
// element towards its first, the reverse map from the FIRST element towards the last -- and keeps
// the running map S = (sA, sB) of what it has walked so far.  What is still unwalked enters the
// result only through the factor sA (the product of the walked gates).  As soon as |sA| <= cut the
// walk stops: the unwalked part could change the result by at most cut * |state entering the walked
// part|, i.e. by at most `cut` relative to the largest value of the scan.  With cut = 0 the walk
// stops only when the product has become exactly zero (an exact-zero gate, or a product that
// underflowed), and the result equals the full fold up to reassociation; a negative cut never
// stops early.  Rows whose product stays above the cut are walked in full, so the kernel is
// correct for any gates; it is cheap for gates below one, whose products vanish after a few
// thousand steps (0.995^t drops below 2^-40 after 5.5 K steps and to zero after 20.6 K).
//
// One CTA per row; a chunk of THREADS*U float4s per iteration with the span arithmetic of the
// look-back family (per-float4 maps, shuffle scan across the warp, second level through shared
// memory, one barrier per chunk).
#pragma once

#include "scan_common.cuh"

namespace ssb {
namespace shard {

template <int THREADS, int U, bool BWD>
__global__ void __launch_bounds__(THREADS)
tail_map_kernel(const float4 *__restrict__ gate, const float4 *__restrict__ in1,  // value | gout
                int64_t rows, int64_t T4, float cut, float *__restrict__ agg,     // [rows][2]
                unsigned long long *__restrict__ walked) {                         // optional: += elements read per tensor
    constexpr int NW = THREADS / 32;
    constexpr int NE = NW * U;
    static_assert(NE <= 32, "second-level scan is one warp wide");
    constexpr int CAP = THREADS * U;
    __shared__ float2 s_tot[2][NE];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t n_chunks = (T4 + CAP - 1) / CAP;
    int buf = 0;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        float sA = 1.f, sB = 0.f;
        int64_t k = 0;
        while (k < n_chunks) {
            // chunk k in walking order: counted from the row's end (forward map) or start (reverse map)
            int64_t lo, n;
            if (!BWD) {
                const int64_t hi = T4 - k * CAP;
                lo = hi > CAP ? hi - CAP : 0;
                n = hi - lo;
            } else {
                lo = k * CAP;
                n = T4 - lo < CAP ? T4 - lo : CAP;
            }
            const float4 *ga = gate + row * T4 + lo, *xa = in1 + row * T4 + lo;
            float A[U], B[U];
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int o = j * THREADS + tid;
                float4 a = make_float4(1.f, 1.f, 1.f, 1.f), x = make_float4(0.f, 0.f, 0.f, 0.f);
                if (o < n && SSB_INDEX_OK(row * T4 + lo + o, rows * T4, 30)) {
                    a = __ldcs(ga + o);
                    x = __ldcs(xa + o);
                }
                if (!BWD) {
                    B[j] = fmaf(a.y, x.x, x.y);
                    B[j] = fmaf(a.z, B[j], x.z);
                    B[j] = fmaf(a.w, B[j], x.w);
                } else {
                    B[j] = a.w * x.w;
                    B[j] = a.z * (x.z + B[j]);
                    B[j] = a.y * (x.y + B[j]);
                    B[j] = a.x * (x.x + B[j]);
                }
                A[j] = (a.x * a.y) * (a.z * a.w);
            }
#pragma unroll
            for (int j = 0; j < U; j++) {
                if (!BWD) warp_scan_forward<float>(A[j], B[j], lane);
                else warp_scan_reverse<float>(A[j], B[j], lane);
            }
            if (lane == (BWD ? 0 : 31)) {
#pragma unroll
                for (int j = 0; j < U; j++) s_tot[buf][j * NW + warp] = make_float2(A[j], B[j]);
            }
            __syncthreads();
            // every warp composes the chunk's map for itself (NE entries): no second barrier
            float tA = 1.f, tB = 0.f;
            if (lane < NE) {
                const float2 tt = s_tot[buf][lane];
                tA = tt.x;
                tB = tt.y;
            }
            if (!BWD) warp_scan_forward<float>(tA, tB, lane);
            else warp_scan_reverse<float>(tA, tB, lane);
            const float cA = __shfl_sync(kFullMask, tA, BWD ? 0 : NE - 1);
            const float cB = __shfl_sync(kFullMask, tB, BWD ? 0 : NE - 1);
            // the chunk lies before (forward) / after (reverse) everything walked so far
            sB = fmaf(sA, cB, sB);
            sA *= cA;
            buf ^= 1;
            k++;
            if (fabsf(sA) <= cut) break;  // uniform: every thread holds the same sA
        }
        if (tid == 0) {
            agg[2 * row] = sA;
            agg[2 * row + 1] = sB;
            if (walked != nullptr) {
                const int64_t vecs = k * CAP < T4 ? k * CAP : T4;
                atomicAdd(walked, (unsigned long long)(vecs * 4));
            }
        }
    }
}

// Adds `n` to a device counter (the traffic account of the shapes that fall back to a full reduction).
__global__ void add_counter_kernel(unsigned long long *counter, unsigned long long n) { atomicAdd(counter, n); }

}  // namespace shard
}  // namespace ssb
