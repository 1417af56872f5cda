// TMA-staged flat sweep for the aligned fp32 rows layout with power-of-two rows that fit a span
// (T = 32 ... 32*LINES, T a power of two): the access pattern of scan_flat.cuh -- CTAs sweep
// memory in consecutive spans of whole rows -- with the data movement of scan_tma.cuh.
//
//   * A span is LINES consecutive 128-byte lines (LINES*32 elements): R = LINES/(T/32) whole rows.
//     The tensor is described to the TMA as [rows][T/32][32]; one `cp.async.bulk.tensor.3d` box
//     {32, T/32, R} per input tensor brings a span into a ring stage (mbarrier completion,
//     128-byte swizzle), up to STAGES-1 spans ahead of the arithmetic.
//   * Thread t of the CTA owns line t: 32 consecutive elements, read as 8 conflict-free float4s.
//     It folds them sequentially (no shuffles), a 5-step shuffle scan composes the 32 lines of a
//     warp, the warps' totals cross through shared memory (one barrier), and the thread replays
//     its 32 elements.  That is ~6 instructions per element against ~14 in the register kernels.
//   * Results go to a swizzled staging tile and leave through one bulk tensor store per span.
//   * Row starts are line starts (T % 32 == 0): the first gate of a row's first line is zeroed
//     in the recurrence, exactly as in the other families.  The backward reads h_{t-1} of a
//     line's first element straight from the h tile in shared memory.
//
// Storage type IO: float, or a 16-bit type (bf16 / fp16) with fp32 arithmetic.  With 16-bit
// storage a 128-byte line holds 64 elements and two threads share it: a thread still owns 32
// consecutive elements (a "unit", four 16-byte chunks of 8), the tensor is described as
// [rows][T/64][64], and everything between the unpack after the shared-memory read and the pack
// before the shared-memory write is the fp32 code.  "Line" below means unit where it describes
// what a thread owns.
//
// Every mbarrier wait is bounded; a wait that runs out is reported through the status word.
#pragma once

#include <cuda.h>

#include "scan_common.cuh"
#include "scan_flat.cuh"
#include "scan_tma.cuh"

namespace ssb {
namespace tmaflat {

template <int LINES, int STAGES, int OUTBUF, bool BWD, typename IO = float>
struct Config {
    static constexpr int TPL = 4 / (int)sizeof(IO);  // threads per 128-byte line
    static constexpr int THREADS = LINES * TPL;
    static constexpr int N_IN = BWD ? 3 : 2;
    static constexpr int N_OUT = BWD ? 2 : 1;
    static constexpr int TILE = LINES * 128;
    static constexpr int SMEM_BYTES = (STAGES * N_IN + OUTBUF * N_OUT) * TILE + 1024;
    static_assert(sizeof(IO) == 4 || sizeof(IO) == 2, "fp32 or 16-bit storage");
    static_assert(THREADS % 32 == 0 && LINES % 8 == 0 && LINES <= 256 && THREADS <= 512,
                  "a span is whole warps of units, whole swizzle atoms, and fits a TMA box");
};

// Swizzled byte offset of float4 `j` (0..7) of line `t` inside a 1024-byte aligned tile.
__device__ __forceinline__ uint32_t chunk_offset(int t, int j) { return (uint32_t)((t << 7) | ((j ^ (t & 7)) << 4)); }
// Swizzled byte offset of 16-byte chunk `j` of the 32 elements thread `t` owns (j < 8 for fp32,
// j < 4 for 16-bit storage, where threads 2l and 2l+1 share line l).
template <typename IO>
__device__ __forceinline__ uint32_t unit_chunk_offset(int t, int j) {
    if constexpr (sizeof(IO) == 4) return chunk_offset(t, j);
    else return chunk_offset(t >> 1, ((t & 1) << 2) | j);
}

// SIGMOID: the gate tensor holds logits z; the gate is sigmoid(z) (flat::sigmoidf) and the
// backward's first output is the gradient with respect to z.
// RECOMPUTE (backward only): the second input is the forward's value tensor b instead of its output
// h; the kernel rebuilds h for the span with a forward scan of (a, b) -- both scans share the one
// barrier -- so a caller need not keep h between the passes.  carry_b is then the h entering each
// row (the forward's h_in).
// LONG: rows longer than a span (T a multiple of the span's 32*threads elements).  A span is then one
// piece of one row (the tensor maps' boxes are {line, LINES, 1}); a CTA walks the `pieces` pieces of a
// row one after the other -- forward from the first, backward from the last -- and hands the state
// from piece to piece through one float in shared memory, using the row-start / row-end carry
// mechanism of the short-row case.  The backward's h just before a piece comes from `h_rows`.
template <int LINES, int STAGES, int OUTBUF, bool BWD, bool SIGMOID = false, bool RECOMPUTE = false, typename IO = float,
          bool LONG = false>
__global__ void __launch_bounds__(LINES * (4 / (int)sizeof(IO)))
tma_flat_kernel(const __grid_constant__ CUtensorMap map_gate, const __grid_constant__ CUtensorMap map_in1,
                const __grid_constant__ CUtensorMap map_in2, const __grid_constant__ CUtensorMap map_out1,
                const __grid_constant__ CUtensorMap map_out2, int64_t rows, int lines_per_row,
                const float *__restrict__ carry_a,   // fwd: h_in | bwd: c_in
                const float *__restrict__ carry_b,   // bwd: h_prev
                int pieces,                          // LONG: spans per row (1 otherwise)
                const IO *__restrict__ h_rows) {     // LONG backward: the h tensor (NULL otherwise)
    using Cfg = Config<LINES, STAGES, OUTBUF, BWD, IO>;
    constexpr int N_IN = Cfg::N_IN, N_OUT = Cfg::N_OUT, TILE = Cfg::TILE, NW = Cfg::THREADS / 32;
    constexpr bool F32 = sizeof(IO) == 4;
    constexpr int NCH = F32 ? 8 : 4;  // 16-byte chunks per thread
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[STAGES];
    __shared__ float2 s_tot[2][NW];
    __shared__ float2 s_fwd[RECOMPUTE ? 2 : 1][NW];  // RECOMPUTE: the forward scan's warp totals
    static_assert(BWD || !RECOMPUTE, "only the backward recomputes");
    static_assert(!(LONG && RECOMPUTE), "recomputing h needs the row inside one span");
    __shared__ float s_chain;  // LONG: the state handed from one piece of a row to the next

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t smem0 = (tma::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t out_base = smem0 + STAGES * N_IN * TILE;
    const uint32_t bar0 = tma::smem_u32(&full_bar[0]);
    const int rows_per_span = Cfg::THREADS / lines_per_row;  // lines_per_row: 32-element units per row (LONG: per piece)
    const int64_t n_spans = LONG ? rows : (rows + rows_per_span - 1) / rows_per_span;  // LONG: counted in rows here
    const int64_t my_spans = ((int64_t)blockIdx.x < n_spans ? (n_spans - blockIdx.x + gridDim.x - 1) / gridDim.x : 0) *
                             (LONG ? pieces : 1);
    // LONG: item i of this CTA is piece i % pieces (counted from the end, backward) of row blockIdx.x + (i / pieces) * gridDim.x
    auto long_row = [&](int64_t i) { return blockIdx.x + (i / pieces) * (int64_t)gridDim.x; };
    auto long_piece = [&](int64_t i) { return BWD ? pieces - 1 - (int)(i % pieces) : (int)(i % pieces); };
    // line of this thread inside its row, and whether it starts / ends a row
    const int line_in_row = tid & (lines_per_row - 1);  // lines_per_row is a power of two
    const bool row_start = line_in_row == 0, row_end = line_in_row == lines_per_row - 1;
    const int row_in_span = tid / lines_per_row;

    auto issue = [&](int64_t i) {  // thread 0: loads of this CTA's i-th span into stage i % STAGES
        const int stage = (int)(i % STAGES);
        const int64_t span = blockIdx.x + i * (int64_t)gridDim.x;
        const int row0 = LONG ? (int)long_row(i) : (int)(span * rows_per_span);
        const int line0 = LONG ? long_piece(i) * LINES : 0;
        const uint32_t bar = bar0 + 8 * stage, dst = smem0 + stage * N_IN * TILE;
        tma::mbar_expect_tx(bar, N_IN * TILE);
        tma::load_box(dst, &map_gate, 0, line0, row0, bar);
        tma::load_box(dst + TILE, &map_in1, 0, line0, row0, bar);
        if (BWD) tma::load_box(dst + 2 * TILE, &map_in2, 0, line0, row0, bar);
    };

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) tma::mbar_init(bar0 + 8 * s, 1);
        tma::fence_mbar_init();
    }
    // Every CTA of this grid is resident by now (persistent grid): the next kernel in the stream may
    // be scheduled onto SMs as they free up.  This kernel itself touches global memory only after
    // the kernel before it has completed.
    grid_dependents_may_launch();
    grid_dependency_wait();
    if (tid == 0)
        for (int64_t i = 0; i < STAGES - 1 && i < my_spans; i++) issue(i);
    __syncthreads();

    uint32_t off[NCH];
#pragma unroll
    for (int j = 0; j < NCH; j++) off[j] = unit_chunk_offset<IO>(tid, j);
    bool timed_out = false;
    unsigned phase_bits = 0u;
    int out_slot = 0, buf = 0;

    for (int64_t i = 0; i < my_spans; i++) {
        const int stage = (int)(i % STAGES);
        const int64_t span = blockIdx.x + i * (int64_t)gridDim.x;
        const int64_t row = LONG ? long_row(i) : span * rows_per_span + row_in_span;
        const int piece = LONG ? long_piece(i) : 0;
        const bool first_piece = !LONG || i % pieces == 0;  // of the row, in processing order
        const uint32_t in0 = smem0 + stage * N_IN * TILE;
        // LONG backward: h just before the piece, for thread 0 (issued before the wait to overlap with it)
        float h_before_piece = 0.f;
        if (LONG && BWD && tid == 0 && piece > 0)
            h_before_piece = widen<float, IO>(h_rows[row * ((int64_t)pieces * Cfg::THREADS * 32) + (int64_t)piece * Cfg::THREADS * 32 - 1]);
        if (!tma::mbar_wait_bounded(bar0 + 8 * stage, (phase_bits >> stage) & 1u)) timed_out = true;
        phase_bits ^= 1u << stage;

        float a[32], x[32], y[32];  // x: value | h ; y: unused | gout
        if constexpr (!F32) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float4 va = tma::lds128(in0 + off[j]), vx = tma::lds128(in0 + TILE + off[j]);
                const float wa[4] = {va.x, va.y, va.z, va.w}, wx[4] = {vx.x, vx.y, vx.z, vx.w};
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    unpack2<IO>(__float_as_uint(wa[k]), a[8 * j + 2 * k], a[8 * j + 2 * k + 1]);
                    unpack2<IO>(__float_as_uint(wx[k]), x[8 * j + 2 * k], x[8 * j + 2 * k + 1]);
                }
                if (SIGMOID) {
#pragma unroll
                    for (int k = 0; k < 8; k++) a[8 * j + k] = flat::sigmoidf(a[8 * j + k]);
                }
                if (BWD) {
                    const float4 vy = tma::lds128(in0 + 2 * TILE + off[j]);
                    const float wy[4] = {vy.x, vy.y, vy.z, vy.w};
#pragma unroll
                    for (int k = 0; k < 4; k++) unpack2<IO>(__float_as_uint(wy[k]), y[8 * j + 2 * k], y[8 * j + 2 * k + 1]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < (F32 ? 8 : 0); j++) {
            const float4 va = tma::lds128(in0 + off[j]), vx = tma::lds128(in0 + TILE + off[j]);
            a[4 * j] = va.x; a[4 * j + 1] = va.y; a[4 * j + 2] = va.z; a[4 * j + 3] = va.w;
            if (SIGMOID) {
#pragma unroll
                for (int k = 0; k < 4; k++) a[4 * j + k] = flat::sigmoidf(a[4 * j + k]);
            }
            x[4 * j] = vx.x; x[4 * j + 1] = vx.y; x[4 * j + 2] = vx.z; x[4 * j + 3] = vx.w;
            if (BWD) {
                const float4 vy = tma::lds128(in0 + 2 * TILE + off[j]);
                y[4 * j] = vy.x; y[4 * j + 1] = vy.y; y[4 * j + 2] = vy.z; y[4 * j + 3] = vy.w;
            }
        }
        float h_left = 0.f;  // backward: h just before this line's first element
        if (BWD) {
            if (row_start) {
                if (LONG && piece > 0) h_left = h_before_piece;
                else if (carry_b != nullptr && row < rows) h_left = carry_b[row];
            } else if (!RECOMPUTE) {
                if constexpr (F32) {
                    h_left = tma::lds32(in0 + TILE + chunk_offset(tid - 1, 7) + 12);
                } else {  // the word that holds the previous unit's last two elements
                    float before;
                    unpack2<IO>(__float_as_uint(tma::lds32(in0 + TILE + unit_chunk_offset<IO>(tid - 1, 3) + 12)), before, h_left);
                }
            }
        }
        const float a_first = a[0];  // the line's first gate before a row start zeroes it
        // Row boundaries and caller-supplied carries.
        if (!BWD) {
            if (row_start) {
                if (!first_piece) x[0] = fmaf(a[0], s_chain, x[0]);
                else if (carry_a != nullptr && row < rows) x[0] = fmaf(a[0], carry_a[row], x[0]);
                a[0] = 0.f;
            }
        } else {
            if (RECOMPUTE && row_start) x[0] = fmaf(a[0], h_left, x[0]);
            if (row_start) a[0] = 0.f;
            if (row_end && !first_piece) y[31] += s_chain;
            else if (row_end && carry_a != nullptr && row < rows) y[31] += carry_a[row];
            if (row >= rows) {  // rows past the end arrive as zeros; keep them inert
#pragma unroll
                for (int k = 0; k < 32; k++) a[k] = 0.f;
            }
        }
        float A, B;
        float FA = 1.f, FB = 0.f;  // RECOMPUTE: this line's map in the forward direction
        if (RECOMPUTE) {
            FA = a[0]; FB = x[0];
#pragma unroll
            for (int k = 1; k < 32; k++) { FB = fmaf(a[k], FB, x[k]); FA *= a[k]; }
            warp_scan_forward<float>(FA, FB, lane);
            if (lane == 31) s_fwd[buf][warp] = make_float2(FA, FB);
        }
        if (!BWD) {
            A = a[0]; B = x[0];
#pragma unroll
            for (int k = 1; k < 32; k++) { B = fmaf(a[k], B, x[k]); A *= a[k]; }
            warp_scan_forward<float>(A, B, lane);
        } else {
            A = 1.f; B = 0.f;
#pragma unroll
            for (int k = 31; k >= 0; k--) { B = a[k] * (y[k] + B); A *= a[k]; }
            warp_scan_reverse<float>(A, B, lane);
        }
        if (lane == (BWD ? 0 : 31)) s_tot[buf][warp] = make_float2(A, B);
        if (tid == 0) tma::store_wait_read<OUTBUF - 1>();  // the staging slot about to be reused is free
        __syncthreads();
        // Every thread holds its span data in registers: the stage can be refilled now.  (Refilling
        // the stage just read instead, one span deeper, measured 1-2 % slower.)
        if (tid == 0 && i + STAGES - 1 < my_spans) issue(i + STAGES - 1);

        // Start value of this warp (maps of the warps processed before it) and of this lane.
        float wA = 1.f, wB = 0.f;
        if (!BWD) {
            for (int w = 0; w < warp; w++) { const float2 t = s_tot[buf][w]; wB = fmaf(t.x, wB, t.y); wA *= t.x; }
        } else {
            for (int w = NW - 1; w > warp; w--) { const float2 t = s_tot[buf][w]; wB = fmaf(t.x, wB, t.y); wA *= t.x; }
        }
        float lA = BWD ? __shfl_down_sync(kFullMask, A, 1) : __shfl_up_sync(kFullMask, A, 1);
        float lB = BWD ? __shfl_down_sync(kFullMask, B, 1) : __shfl_up_sync(kFullMask, B, 1);
        if (lane == (BWD ? 31 : 0)) { lA = 1.f; lB = 0.f; }
        float s = fmaf(lA, wB, lB);  // the span starts from 0: it begins at a row start
        if (RECOMPUTE) {  // turn x from b into h: h just before this line, then the line itself
            float fB = 0.f;
            for (int w = 0; w < warp; w++) { const float2 t = s_fwd[buf][w]; fB = fmaf(t.x, fB, t.y); }
            float pA = __shfl_up_sync(kFullMask, FA, 1), pB = __shfl_up_sync(kFullMask, FB, 1);
            if (lane == 0) { pA = 1.f; pB = 0.f; }
            float hp = fmaf(pA, fB, pB);
            if (!row_start) h_left = hp;
#pragma unroll
            for (int k = 0; k < 32; k++) { hp = fmaf(a[k], hp, x[k]); x[k] = hp; }
        }

        const uint32_t ob = out_base + out_slot * N_OUT * TILE;
        if constexpr (!F32) {
            // In place: forward x <- h; backward y <- grad of value, a <- grad of gate.  Then pack.
            if (!BWD) {
#pragma unroll
                for (int k = 0; k < 32; k++) { s = fmaf(a[k], s, x[k]); x[k] = s; }
            } else {
#pragma unroll
                for (int k = 31; k >= 0; k--) {
                    const float gb = y[k] + s, ak = (k == 0) ? a_first : a[k];
                    s = (LONG && k == 0 ? a_first : a[k]) * gb;
                    y[k] = gb;
                    a[k] = gb * (k > 0 ? x[k > 0 ? k - 1 : 0] : h_left);
                    if (SIGMOID) a[k] *= ak * (1.f - ak);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float *src = BWD ? a : x;
                float4 o;
                o.x = __uint_as_float(pack2<IO>(src[8 * j], src[8 * j + 1]));
                o.y = __uint_as_float(pack2<IO>(src[8 * j + 2], src[8 * j + 3]));
                o.z = __uint_as_float(pack2<IO>(src[8 * j + 4], src[8 * j + 5]));
                o.w = __uint_as_float(pack2<IO>(src[8 * j + 6], src[8 * j + 7]));
                tma::sts128(ob + off[j], o);
                if (BWD) {
                    o.x = __uint_as_float(pack2<IO>(y[8 * j], y[8 * j + 1]));
                    o.y = __uint_as_float(pack2<IO>(y[8 * j + 2], y[8 * j + 3]));
                    o.z = __uint_as_float(pack2<IO>(y[8 * j + 4], y[8 * j + 5]));
                    o.w = __uint_as_float(pack2<IO>(y[8 * j + 6], y[8 * j + 7]));
                    tma::sts128(ob + TILE + off[j], o);
                }
            }
        } else if (!BWD) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float4 o;
                s = fmaf(a[4 * j], s, x[4 * j]); o.x = s;
                s = fmaf(a[4 * j + 1], s, x[4 * j + 1]); o.y = s;
                s = fmaf(a[4 * j + 2], s, x[4 * j + 2]); o.z = s;
                s = fmaf(a[4 * j + 3], s, x[4 * j + 3]); o.w = s;
                tma::sts128(ob + off[j], o);
            }
        } else {
#pragma unroll
            for (int j = 7; j >= 0; j--) {
                float4 oa, og;
                float gb;
                gb = y[4 * j + 3] + s; s = a[4 * j + 3] * gb; og.w = gb; oa.w = gb * x[4 * j + 2];
                gb = y[4 * j + 2] + s; s = a[4 * j + 2] * gb; og.z = gb; oa.z = gb * x[4 * j + 1];
                gb = y[4 * j + 1] + s; s = a[4 * j + 1] * gb; og.y = gb; oa.y = gb * x[4 * j];
                gb = y[4 * j] + s; s = a[4 * j] * gb; og.x = gb;
                if (LONG && j == 0) s = a_first * gb;  // what leaves the piece towards the one before it
                oa.x = gb * (j > 0 ? x[j > 0 ? 4 * j - 1 : 0] : h_left);
                if (SIGMOID) {  // d sigmoid(z) / dz = a (1 - a)
                    const float a0 = j > 0 ? a[4 * j] : a_first;
                    oa.x *= a0 * (1.f - a0);
                    oa.y *= a[4 * j + 1] * (1.f - a[4 * j + 1]);
                    oa.z *= a[4 * j + 2] * (1.f - a[4 * j + 2]);
                    oa.w *= a[4 * j + 3] * (1.f - a[4 * j + 3]);
                }
                tma::sts128(ob + off[j], oa);
                tma::sts128(ob + TILE + off[j], og);
            }
        }
        if (LONG && tid == (BWD ? 0 : Cfg::THREADS - 1)) s_chain = s;  // read by the next piece after the barrier below
        tma::fence_async_smem();
        __syncthreads();
        if (tid == 0) {
            const int row0 = LONG ? (int)row : (int)(span * rows_per_span);
            const int line0 = LONG ? piece * LINES : 0;
            tma::store_box(&map_out1, 0, line0, row0, ob);
            if (BWD) tma::store_box(&map_out2, 0, line0, row0, ob + TILE);
            tma::store_commit();
        }
        out_slot = (out_slot + 1 == OUTBUF) ? 0 : out_slot + 1;
        buf ^= 1;
    }
    if (tid == 0) tma::store_wait_read<0>();
    if (timed_out && lane == 0) report_device_wait(6);
}

}  // namespace tmaflat
}  // namespace ssb
