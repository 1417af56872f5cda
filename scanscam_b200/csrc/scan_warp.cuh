// Warp-per-row kernels: the general-shape family (any T, any alignment, fp32 and fp64).
//
// One warp owns one row at a time and walks it in chunks of 32*VEC*U elements.  Loads are
// "striped": in sub-chunk u, lane l reads the VEC consecutive elements starting at
// (u*32 + l)*VEC, so a warp-wide load instruction covers one contiguous 32*VEC*sizeof(real)
// byte span.  Each lane folds its VEC elements into one affine map, a shuffle scan composes
// the 32 maps of a sub-chunk, the running carry of the row is applied, and the lane re-runs
// the recurrence over its own elements from its now-known starting value.  The carry from
// sub-chunk to sub-chunk is one FMA, so nothing serialises across chunks but that FMA.
//
// The forward kernel replaces the reference's blocked/vectorised/simple/coalesced forward
// kernels (src/scanscam_cuda.cu:21-36,61-119,144-258); the backward kernel replaces
// :309-332 and :366-425.  With REDUCE the kernels only emit each row's aggregate map
// (used to shard a sequence across GPUs).
#pragma once

#include "scan_common.cuh"

namespace ssb {

constexpr int kWarpKernelWarps = 8;  // warps per CTA

// io_t is the storage type of the tensors (real itself, or bf16 / fp16 with real = float: the
// arithmetic and the per-row carries stay in fp32).
template <typename real, int VEC, int U, bool REDUCE, typename io_t = real>
__global__ void __launch_bounds__(kWarpKernelWarps * 32)
warp_rows_fwd_kernel(const io_t *__restrict__ gate, const io_t *__restrict__ value,
                     io_t *__restrict__ out, int64_t rows, int64_t T,
                     const real *__restrict__ h_in, real *__restrict__ agg) {
    constexpr int CH = 32 * VEC * U;
    const int lane = threadIdx.x & 31;
    const int64_t n_warps = (int64_t)gridDim.x * kWarpKernelWarps;
    // Interleave so that consecutive rows land on different CTAs.
    for (int64_t row = (int64_t)(threadIdx.x >> 5) * gridDim.x + blockIdx.x; row < rows;
         row += n_warps) {
        const io_t *g = gate + row * T;
        const io_t *v = value + row * T;
        real carry = (!REDUCE && h_in != nullptr) ? h_in[row] : real(0);
        real a_row = real(1);
        for (int64_t t0 = 0; t0 < T; t0 += CH) {
            Pack<real, VEC> a[U], b[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int64_t idx = t0 + (int64_t)(u * 32 + lane) * VEC;
                if (idx < T && SSB_INDEX_OK(row * T + idx, rows * T, 40)) {  // T % VEC == 0 whenever VEC > 1, so a pack is all in or all out
                    a[u] = load_stream_io<real, io_t, VEC>(g + idx);
                    b[u] = load_stream_io<real, io_t, VEC>(v + idx);
                } else {
#pragma unroll
                    for (int k = 0; k < VEC; k++) { a[u].v[k] = real(1); b[u].v[k] = real(0); }
                }
            }
            real A[U], B[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                A[u] = a[u].v[0];
                B[u] = b[u].v[0];
#pragma unroll
                for (int k = 1; k < VEC; k++) {
                    B[u] = fma_<real>(a[u].v[k], B[u], b[u].v[k]);
                    A[u] *= a[u].v[k];
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) warp_scan_forward<real>(A[u], B[u], lane);
#pragma unroll
            for (int u = 0; u < U; u++) {
                real Ae = __shfl_up_sync(kFullMask, A[u], 1);
                real Be = __shfl_up_sync(kFullMask, B[u], 1);
                if (lane == 0) { Ae = real(1); Be = real(0); }
                const real At = __shfl_sync(kFullMask, A[u], 31);
                const real Bt = __shfl_sync(kFullMask, B[u], 31);
                if constexpr (!REDUCE) {
                    real h = fma_<real>(Ae, carry, Be);
                    Pack<real, VEC> o;
#pragma unroll
                    for (int k = 0; k < VEC; k++) {
                        h = fma_<real>(a[u].v[k], h, b[u].v[k]);
                        o.v[k] = h;
                    }
                    const int64_t idx = t0 + (int64_t)(u * 32 + lane) * VEC;
                    if (idx < T && SSB_INDEX_OK(row * T + idx, rows * T, 41)) store_stream_io<real, io_t, VEC>(out + row * T + idx, o);
                } else {
                    a_row *= At;
                }
                carry = fma_<real>(At, carry, Bt);
            }
        }
        if constexpr (REDUCE) {
            if (lane == 0) {
                agg[2 * row] = a_row;
                agg[2 * row + 1] = carry;
            }
        }
    }
}

// Backward.  With c_t = a_t * gb_t (the gradient leaving step t towards step t-1) the
// recurrence is  gb_t = g_t + c_{t+1},  c_t = a_t * gb_t,  i.e. the map c -> a_t*c + a_t*g_t,
// folded from the right; ga_t = gb_t * h_{t-1}.  This is the order of operations of the
// reference's sequential loop (src/scanscam_cpu.hpp:64-77).
template <typename real, int VEC, int U, bool REDUCE, typename io_t = real>
__global__ void __launch_bounds__(kWarpKernelWarps * 32)
warp_rows_bwd_kernel(const io_t *__restrict__ gate, const io_t *__restrict__ hout,
                     const io_t *__restrict__ gout, io_t *__restrict__ ggate,
                     io_t *__restrict__ gvalue, int64_t rows, int64_t T,
                     const real *__restrict__ c_in, const real *__restrict__ h_prev,
                     real *__restrict__ agg) {
    constexpr int CH = 32 * VEC * U;
    const int lane = threadIdx.x & 31;
    const int64_t n_warps = (int64_t)gridDim.x * kWarpKernelWarps;
    const int64_t n_chunks = (T + CH - 1) / CH;
    for (int64_t row = (int64_t)(threadIdx.x >> 5) * gridDim.x + blockIdx.x; row < rows;
         row += n_warps) {
        const io_t *ga_ = gate + row * T;
        const io_t *gg_ = gout + row * T;
        const io_t *hh_ = REDUCE ? nullptr : hout + row * T;
        real carry = (!REDUCE && c_in != nullptr) ? c_in[row] : real(0);
        real a_row = real(1);
        for (int64_t t0 = (n_chunks - 1) * CH; t0 >= 0; t0 -= CH) {
            Pack<real, VEC> a[U], g[U], h[U];
            real edge = real(0);  // h just left of this chunk
            if constexpr (!REDUCE) {
                if (t0 > 0 && SSB_INDEX_OK(row * T + t0 - 1, rows * T, 42)) edge = widen<real, io_t>(hh_[t0 - 1]);
                else if (h_prev != nullptr) edge = h_prev[row];
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int64_t idx = t0 + (int64_t)(u * 32 + lane) * VEC;
                if (idx < T && SSB_INDEX_OK(row * T + idx, rows * T, 43)) {
                    a[u] = load_stream_io<real, io_t, VEC>(ga_ + idx);
                    g[u] = load_stream_io<real, io_t, VEC>(gg_ + idx);
                    if constexpr (!REDUCE) h[u] = load_stream_io<real, io_t, VEC>(hh_ + idx);
                } else {
#pragma unroll
                    for (int k = 0; k < VEC; k++) {
                        a[u].v[k] = real(1); g[u].v[k] = real(0); h[u].v[k] = real(0);
                    }
                }
            }
            real A[U], D[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                A[u] = real(1);
                D[u] = real(0);
#pragma unroll
                for (int k = VEC - 1; k >= 0; k--) {
                    D[u] = a[u].v[k] * (g[u].v[k] + D[u]);
                    A[u] *= a[u].v[k];
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) warp_scan_reverse<real>(A[u], D[u], lane);
#pragma unroll
            for (int u = U - 1; u >= 0; u--) {
                real Ae = __shfl_down_sync(kFullMask, A[u], 1);
                real De = __shfl_down_sync(kFullMask, D[u], 1);
                if (lane == 31) { Ae = real(1); De = real(0); }
                const real At = __shfl_sync(kFullMask, A[u], 0);
                const real Dt = __shfl_sync(kFullMask, D[u], 0);
                if constexpr (!REDUCE) {
                    // h just left of this lane's first element
                    real left = __shfl_up_sync(kFullMask, h[u].v[VEC - 1], 1);
                    if (u > 0) {
                        const real wrap = __shfl_sync(kFullMask, h[u > 0 ? u - 1 : 0].v[VEC - 1], 31);
                        if (lane == 0) left = wrap;
                    } else if (lane == 0) {
                        left = edge;
                    }
                    real c = fma_<real>(Ae, carry, De);
                    Pack<real, VEC> oa, ob;
#pragma unroll
                    for (int k = VEC - 1; k >= 0; k--) {
                        const real gb = g[u].v[k] + c;
                        c = a[u].v[k] * gb;
                        ob.v[k] = gb;
                        oa.v[k] = gb * (k > 0 ? h[u].v[k > 0 ? k - 1 : 0] : left);
                    }
                    const int64_t idx = t0 + (int64_t)(u * 32 + lane) * VEC;
                    if (idx < T && SSB_INDEX_OK(row * T + idx, rows * T, 44)) {
                        store_stream_io<real, io_t, VEC>(ggate + row * T + idx, oa);
                        store_stream_io<real, io_t, VEC>(gvalue + row * T + idx, ob);
                    }
                } else {
                    a_row *= At;
                }
                carry = fma_<real>(At, carry, Dt);
            }
        }
        if constexpr (REDUCE) {
            if (lane == 0) {
                agg[2 * row] = a_row;
                agg[2 * row + 1] = carry;
            }
        }
    }
}

// Folds the per-shard aggregate maps of a T-sharded sequence into the carry one shard
// starts from.  aggs is [n_shards, rows, 2].  Forward: shards 0..shard-1, left to right.
// Reverse: shards n_shards-1..shard+1, right to left.  One thread per row.
template <typename real>
__global__ void shard_carry_kernel(const real *__restrict__ aggs, int n_shards, int shard,
                                   int reverse, int64_t rows, real *__restrict__ carry) {
    const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    real x = real(0);
    if (!reverse) {
        for (int s = 0; s < shard; s++) {
            const real *p = aggs + ((int64_t)s * rows + r) * 2;
            x = fma_<real>(p[0], x, p[1]);
        }
    } else {
        for (int s = n_shards - 1; s > shard; s--) {
            const real *p = aggs + ((int64_t)s * rows + r) * 2;
            x = fma_<real>(p[0], x, p[1]);
        }
    }
    carry[r] = x;
}

}  // namespace ssb
