// Channels-last kernels for NARROW tensors: dense fp32 [N, T, C] with C = 4, 8 or 16 channels
// (16-byte aligned base), scan over T.  A time step of such a tensor is 16-64 bytes; the kernels
// that give a CTA a block of 32 channels (scan_cl_stream.cuh, scan_cl.cuh) would touch one sector
// per step and leave three quarters of every lane group idle.  The reference's test grid has such
// a shape, (512, 4096, 8) (scanscam/cuda_test.py:132).
//
//   * A unit of work is one batch element with ALL of its channels: the [T, C] slab of a batch
//     element is one contiguous run of bytes, so a tile of TT steps is TT*C*4 contiguous bytes and
//     moves with ONE untiled bulk copy per tensor (`cp.async.bulk`, mbarrier completion) into a
//     ring of shared-memory stages, and the results leave with one bulk store per tensor.
//   * Thread (seg, cg) owns 4 adjacent channels (one float4 per step) of the seg-th run of TS
//     consecutive steps.  TS is odd: the runs of the 8/CG segments that share a quarter warp then
//     start in different 16*CG-byte slots of a 128-byte bank row, and the float4 reads and writes
//     of a warp are conflict-free without any swizzle.
//   * A thread folds its run, the runs of a warp are composed with shuffles, the warps' totals
//     cross through shared memory (one barrier), and the thread replays its run from its
//     now-known starting value; the carry from tile to tile is a float4 in registers.
//   * The backward fetches h one step earlier (the copy starts one row before the tile; at the
//     first step of the sequence there is nothing before it and the owning thread uses 0).
//   * The last tile of a sequence may be partial: the copies are sized to what exists and the
//     steps beyond it are masked to the identity (a = 1, b = g = 0), so stale shared memory never
//     enters the backward's right-to-left recurrence.
//
// Every mbarrier wait is bounded; a wait that runs out is reported through the status word.
#pragma once

#include "scan_cl_stream.cuh"
#include "scan_common.cuh"
#include "scan_tma.cuh"

namespace ssb {
namespace cln {

using cls::add4;
using cls::fma4;
using cls::Map4;
using cls::mul4;
using cls::shfl4;

// Untiled bulk copies: both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void bulk_store(void *dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}

template <int CG, int TS, int WARPS, int STAGES, int OUTBUF, bool BWD>
struct Config {
    static constexpr int C = 4 * CG;           // channels of the tensor (exactly)
    static constexpr int ROW = 16 * CG;        // bytes of one time step
    static constexpr int SPW = 32 / CG;        // segments (runs) per warp
    static constexpr int SEGS = WARPS * SPW;
    static constexpr int TT = SEGS * TS;       // steps per tile
    static constexpr int THREADS = WARPS * 32;
    static constexpr int N_IN = BWD ? 3 : 2;
    static constexpr int N_OUT = BWD ? 2 : 1;
    static constexpr int TILE = TT * ROW;
    static constexpr int SMEM_BYTES = (STAGES * N_IN + OUTBUF * N_OUT) * TILE + 128;
    static_assert(CG == 1 || CG == 2 || CG == 4, "4, 8 or 16 channels");
    static_assert(TS % 2 == 1, "an odd run length keeps the shared-memory accesses conflict-free");
    static_assert(STAGES >= 1 && OUTBUF >= 1 && SMEM_BYTES <= 227 * 1024, "ring sizes");
};

template <int CG, int TS, int WARPS, int STAGES, int OUTBUF, bool BWD>
__global__ void __launch_bounds__(WARPS * 32)
cl_narrow_kernel(const float *__restrict__ gate, const float *__restrict__ in1,  // value | h
                 const float *__restrict__ in2,                                   // unused | gout
                 float *__restrict__ out1, float *__restrict__ out2,              // h | ggate, gvalue
                 int64_t N, int64_t T) {
    using Cfg = Config<CG, TS, WARPS, STAGES, OUTBUF, BWD>;
    constexpr int SPW = Cfg::SPW, NW = WARPS, N_IN = Cfg::N_IN, N_OUT = Cfg::N_OUT, TILE = Cfg::TILE, ROW = Cfg::ROW,
                  TT = Cfg::TT, C = Cfg::C;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[STAGES];
    __shared__ float4 s_tot[2][NW][CG][2];  // per warp and channel group: the warp's composed map (A, B)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cg = lane % CG, seg_in_warp = lane / CG, seg = warp * SPW + seg_in_warp;
    const uint32_t smem0 = (tma::smem_u32(smem_raw) + 127u) & ~127u;
    const uint32_t out_base = smem0 + STAGES * N_IN * TILE;
    const uint32_t bar0 = tma::smem_u32(&full_bar[0]);
    const int64_t n_tiles = (T + TT - 1) / TT;
    const int64_t my_units = (int64_t)blockIdx.x < N ? (N - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int64_t n_items = my_units * n_tiles;
    const uint32_t my_off = (uint32_t)(seg * TS * ROW + cg * 16);  // this thread's float4 at its first step inside a tile

    // item i of this CTA: tile (forward: i % n_tiles, backward: counted from the end) of batch element blockIdx.x + (i / n_tiles) * gridDim.x
    auto coords = [&](int64_t i, int64_t &n, int64_t &t0, int &steps) {
        n = blockIdx.x + (i / n_tiles) * (int64_t)gridDim.x;
        const int64_t tile = BWD ? n_tiles - 1 - (i % n_tiles) : (i % n_tiles);
        t0 = tile * TT;
        steps = (int)(T - t0 < TT ? T - t0 : TT);
    };
    auto issue = [&](int64_t i) {  // thread 0: bulk loads of item i into stage i % STAGES
        const int stage = (int)(i % STAGES);
        int64_t n, t0;
        int steps;
        coords(i, n, t0, steps);
        const uint32_t bar = bar0 + 8 * stage, dst = smem0 + stage * N_IN * TILE;
        const uint32_t bytes = (uint32_t)steps * ROW;
        const int64_t first = (n * T + t0) * C;  // element offset of the tile
        // backward: h arrives one step early; at t0 == 0 the row before the tile does not exist
        const uint32_t h_bytes = !BWD ? bytes : (t0 > 0 ? bytes : bytes - ROW);
        tma::mbar_expect_tx(bar, bytes + h_bytes + (BWD ? bytes : 0u));
        bulk_load(dst, gate + first, bytes, bar);
        if (!BWD) {
            bulk_load(dst + TILE, in1 + first, bytes, bar);
        } else {
            if (t0 > 0) bulk_load(dst + TILE, in1 + first - C, bytes, bar);
            else if (h_bytes > 0) bulk_load(dst + TILE + ROW, in1 + first, h_bytes, bar);
            bulk_load(dst + 2 * TILE, in2 + first, bytes, bar);
        }
    };

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) tma::mbar_init(bar0 + 8 * s, 1);
        tma::fence_mbar_init();
        for (int64_t i = 0; i < STAGES && i < n_items; i++) issue(i);
    }
    __syncthreads();

    bool timed_out = false;
    unsigned phase_bits = 0u;
    int out_slot = 0, buf = 0;
    const float4 one4 = make_float4(1.f, 1.f, 1.f, 1.f), zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 carry = zero4;  // state entering the tile, for this thread's 4 channels

    for (int64_t i = 0; i < n_items; i++) {
        const int stage = (int)(i % STAGES);
        const uint32_t in0 = smem0 + stage * N_IN * TILE + my_off;
        int64_t n, t0;
        int steps;
        coords(i, n, t0, steps);
        if (i % n_tiles == 0) carry = zero4;  // a new batch element starts
        if (!tma::mbar_wait_bounded(bar0 + 8 * stage, (phase_bits >> stage) & 1u)) timed_out = true;
        phase_bits ^= 1u << stage;

        float4 a[TS], x[TS], y[TS];  // x: value | h one step earlier ; y: unused | gout
#pragma unroll
        for (int k = 0; k < TS; k++) {
            const int r = seg * TS + k;  // step inside the tile
            if (r < steps) {
                a[k] = tma::lds128(in0 + k * ROW);
                x[k] = tma::lds128(in0 + TILE + k * ROW);
                if (BWD) {
                    y[k] = tma::lds128(in0 + 2 * TILE + k * ROW);
                    if (t0 == 0 && r == 0) x[k] = zero4;  // h before the first step
                }
            } else {  // beyond the end of the sequence: the identity
                a[k] = one4;
                x[k] = zero4;
                y[k] = zero4;
            }
        }
        Map4 m;
        if (!BWD) {
            m.A = a[0]; m.B = x[0];
#pragma unroll
            for (int k = 1; k < TS; k++) { m.B = fma4(a[k], m.B, x[k]); m.A = mul4(m.A, a[k]); }
        } else {
            m.A = one4; m.B = zero4;
#pragma unroll
            for (int k = TS - 1; k >= 0; k--) { m.B = mul4(a[k], add4(y[k], m.B)); m.A = mul4(m.A, a[k]); }
        }
#pragma unroll
        for (int d = 1; d < SPW; d <<= 1) {
            const float4 pA = shfl4(m.A, d * CG, !BWD), pB = shfl4(m.B, d * CG, !BWD);
            const bool has = BWD ? (seg_in_warp + d < SPW) : (seg_in_warp >= d);
            if (has) { m.B = fma4(m.A, pB, m.B); m.A = mul4(m.A, pA); }
        }
        if (seg_in_warp == (BWD ? 0 : SPW - 1)) {
            s_tot[buf][warp][cg][0] = m.A;
            s_tot[buf][warp][cg][1] = m.B;
        }
        if (tid == 0) tma::store_wait_read<OUTBUF - 1>();  // the staging slot about to be reused is free
        __syncthreads();
        // Every thread holds its tile data in registers: this very stage can be refilled now.
        if (tid == 0 && i + STAGES < n_items) issue(i + STAGES);

        // State entering this warp's runs, and the state leaving the tile (the next carry).
        float4 s = carry, run = carry;
#pragma unroll
        for (int q = 0; q < NW; q++) {
            const int w = BWD ? NW - 1 - q : q;
            const float4 tA = s_tot[buf][w][cg][0], tB = s_tot[buf][w][cg][1];
            if (w == warp) s = run;
            run = fma4(tA, run, tB);
        }
        carry = run;
        {  // ... and this thread's own run: the exclusive prefix inside the warp
            float4 eA = shfl4(m.A, CG, !BWD), eB = shfl4(m.B, CG, !BWD);
            if (seg_in_warp == (BWD ? SPW - 1 : 0)) { eA = one4; eB = zero4; }
            s = fma4(eA, s, eB);
        }

        const uint32_t ob = out_base + out_slot * N_OUT * TILE + my_off;
        if (!BWD) {
#pragma unroll
            for (int k = 0; k < TS; k++) {
                s = fma4(a[k], s, x[k]);
                tma::sts128(ob + k * ROW, s);
            }
        } else {
#pragma unroll
            for (int k = TS - 1; k >= 0; k--) {
                const float4 gb = add4(y[k], s);
                s = mul4(a[k], gb);
                tma::sts128(ob + k * ROW, mul4(gb, x[k]));  // grad of gate = gb_t * h_{t-1}
                tma::sts128(ob + TILE + k * ROW, gb);        // grad of value
            }
        }
        tma::fence_async_smem();
        __syncthreads();
        if (tid == 0) {
            const int64_t first = (n * T + t0) * C;
            const uint32_t bytes = (uint32_t)steps * ROW;
            bulk_store(out1 + first, ob - my_off, bytes);
            if (BWD) bulk_store(out2 + first, ob - my_off + TILE, bytes);
            tma::store_commit();
        }
        out_slot = (out_slot + 1 == OUTBUF) ? 0 : out_slot + 1;
        buf ^= 1;
    }
    if (tid == 0) tma::store_wait_read<0>();
    if (timed_out && lane == 0) report_device_wait(8);
}

}  // namespace cln
}  // namespace ssb
