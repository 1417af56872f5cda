// Channels-last kernels: dense [N, T, C], scan over T, channel innermost.
//
// A lane owns one channel, a warp 32 adjacent channels (one coalesced 128-byte line per time
// step), and the WS warps of a CTA own WS consecutive segments of L time steps: a CTA tile is
// WS*L steps of 32 channels.  Each thread keeps its L steps in registers (2L or 3L independent
// loads in flight), folds them into one affine map, the CTA composes the WS maps of every
// channel through shared memory, and each thread re-runs its L steps from the value it now
// knows it starts at.  The CTA walks T tile by tile with the channel's carry in shared memory.
//
// Replaces the reference's transposed kernels (src/scanscam_cuda.cu:471-554 and :584-685).
#pragma once

#include "scan_common.cuh"

namespace ssb {

template <typename real, int WS, int L>
__global__ void __launch_bounds__(WS * 32)
cl_fwd_kernel(const real *__restrict__ gate, const real *__restrict__ value,
              real *__restrict__ out, int64_t N, int64_t T, int64_t C) {
    __shared__ real sA[WS][32], sB[WS][32], sCarry[32];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t cblocks = (C + 31) / 32;
    const int64_t n = blockIdx.x / cblocks;
    const int64_t c = (blockIdx.x % cblocks) * 32 + lane;
    const bool c_ok = c < C;
    const int64_t base = n * T * C + (c_ok ? c : 0);
    if (warp == 0) sCarry[lane] = real(0);
    __syncthreads();
    for (int64_t t0 = 0; t0 < T; t0 += (int64_t)WS * L) {
        const int64_t tb = t0 + (int64_t)warp * L;
        real a[L], b[L];
#pragma unroll
        for (int k = 0; k < L; k++) {
            const int64_t t = tb + k;
            if (c_ok && t < T && SSB_INDEX_OK(base + t * C, N * T * C, 50)) {
                a[k] = __ldcs(gate + base + t * C);
                b[k] = __ldcs(value + base + t * C);
            } else {
                a[k] = real(1);
                b[k] = real(0);
            }
        }
        real A = a[0], B = b[0];
#pragma unroll
        for (int k = 1; k < L; k++) {
            B = fma_<real>(a[k], B, b[k]);
            A *= a[k];
        }
        sA[warp][lane] = A;
        sB[warp][lane] = B;
        __syncthreads();
        real h = sCarry[lane];
        for (int j = 0; j < warp; j++) h = fma_<real>(sA[j][lane], h, sB[j][lane]);
#pragma unroll
        for (int k = 0; k < L; k++) {
            h = fma_<real>(a[k], h, b[k]);
            const int64_t t = tb + k;
            if (c_ok && t < T && SSB_INDEX_OK(base + t * C, N * T * C, 51)) __stcs(out + base + t * C, h);
        }
        __syncthreads();  // all warps have read the carry and the maps of this tile
        if (warp == WS - 1) sCarry[lane] = h;
    }
}

// Backward, tiles visited right to left; h_{t-1} is simply the line above in memory.
template <typename real, int WS, int L>
__global__ void __launch_bounds__(WS * 32)
cl_bwd_kernel(const real *__restrict__ gate, const real *__restrict__ hout,
              const real *__restrict__ gout, real *__restrict__ ggate,
              real *__restrict__ gvalue, int64_t N, int64_t T, int64_t C) {
    __shared__ real sA[WS][32], sD[WS][32], sCarry[32];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t cblocks = (C + 31) / 32;
    const int64_t n = blockIdx.x / cblocks;
    const int64_t c = (blockIdx.x % cblocks) * 32 + lane;
    const bool c_ok = c < C;
    const int64_t base = n * T * C + (c_ok ? c : 0);
    constexpr int64_t TILE_T = (int64_t)WS * L;
    if (warp == 0) sCarry[lane] = real(0);
    __syncthreads();
    const int64_t n_tiles = (T + TILE_T - 1) / TILE_T;
    for (int64_t t0 = (n_tiles - 1) * TILE_T; t0 >= 0; t0 -= TILE_T) {
        const int64_t tb = t0 + (int64_t)warp * L;
        real a[L], g[L], hp[L];
#pragma unroll
        for (int k = 0; k < L; k++) {
            const int64_t t = tb + k;
            if (c_ok && t < T && SSB_INDEX_OK(base + t * C, N * T * C, 52)) {
                a[k] = __ldcs(gate + base + t * C);
                g[k] = __ldcs(gout + base + t * C);
                hp[k] = t > 0 ? __ldcs(hout + base + (t - 1) * C) : real(0);
            } else {
                a[k] = real(1);
                g[k] = real(0);
                hp[k] = real(0);
            }
        }
        real A = real(1), D = real(0);
#pragma unroll
        for (int k = L - 1; k >= 0; k--) {
            D = a[k] * (g[k] + D);
            A *= a[k];
        }
        sA[warp][lane] = A;
        sD[warp][lane] = D;
        __syncthreads();
        real cc = sCarry[lane];
        for (int j = WS - 1; j > warp; j--) cc = fma_<real>(sA[j][lane], cc, sD[j][lane]);
#pragma unroll
        for (int k = L - 1; k >= 0; k--) {
            const real gb = g[k] + cc;
            cc = a[k] * gb;
            const int64_t t = tb + k;
            if (c_ok && t < T && SSB_INDEX_OK(base + t * C, N * T * C, 53)) {
                __stcs(gvalue + base + t * C, gb);
                __stcs(ggate + base + t * C, gb * hp[k]);
            }
        }
        __syncthreads();
        if (warp == 0) sCarry[lane] = cc;
    }
}

}  // namespace ssb
