// Channels-last streaming kernels: dense fp32 [N, T, C] (C % 4 == 0, 16-byte aligned base), scan
// over T, for problems with enough independent (batch element, channel block) pairs to fill the
// GPU without splitting T.  Replaces the reference's transposed kernels
// (src/scanscam_cuda.cu:471-723) on such shapes.
//
//   * A unit of work is one batch element and CC adjacent channels; a CTA owns a unit and walks
//     its T steps in tiles of TT steps, forward kernels from step 0 up, backward kernels from the
//     last step down.  The carry from tile to tile is a float4 in registers: no workspace, no
//     handshake between CTAs.
//   * The tensor is described to the TMA as {C, T, N}; one `cp.async.bulk.tensor.3d` box
//     {CC, TT, 1} per input brings a tile into a ring of shared-memory stages (mbarrier
//     completion), STAGES tiles ahead of the arithmetic and across unit boundaries.  Steps past
//     T and channels past C arrive as zeros and are clipped on the way out.  The backward fetches
//     h with a box that starts one step earlier (h_{t-1}; step -1 reads the fill value 0).
//   * Thread (seg, cg) owns 4 adjacent channels (one float4 per step) and the seg-th run of
//     TS = TT/SEG steps.  It folds its run sequentially, the runs of a warp are composed with
//     shuffles, the warps' totals cross through shared memory (one barrier), and the thread
//     replays its run from its now-known starting value: ~5 instructions per element.
//     The 8 (or 16) threads of a quarter warp read one contiguous 128-byte row: no bank conflicts.
//   * Results go to a staging tile and leave through one bulk tensor store per tile.
//   * With few (batch element, channel block) pairs the time axis is cut into `chunks` pieces that
//     run as units of their own, in two passes: cl_tail_map_kernel composes each chunk's map as
//     far as the gate products need (2*CC floats per chunk), and this kernel starts each chunk
//     from the fold of the maps of the chunks before it (after it, for the backward), which every
//     CTA computes for itself at the start of a unit.
//     That launch may be a programmatic dependent launch: the CTAs set up and issue their first
//     tile loads while the map kernel drains, and wait for it (griddepcontrol.wait) only before
//     they read the maps.
//
//   * Storage type IO: float, or bf16 / fp16 with fp32 arithmetic.  A thread still owns 4 adjacent
//     channels; with 16-bit storage they are 8 bytes (one 64-bit shared-memory access), a tile row
//     of CC channels is CC*2 bytes, and the 16 threads of a half warp cover a 128-byte row.
//     Chunk maps and carries stay fp32.
//   * SIGMOID: the gate tensor holds logits z; the gate is sigmoid(z) (flat::sigmoidf) and the
//     backward's first output is the gradient with respect to z.
//
// Every mbarrier wait is bounded; a wait that runs out is reported through the status word.
#pragma once

#include <cuda.h>

#include "scan_common.cuh"
#include "scan_flat.cuh"
#include "scan_tma.cuh"

namespace ssb {
namespace cls {

template <int CC, int TT, int SEG, int STAGES, int OUTBUF, bool BWD, typename IO = float>
struct Config {
    static constexpr int ROW = CC * (int)sizeof(IO);  // bytes of one tile row
    static constexpr int CG = CC / 4;            // float4 channel groups per tile row
    static constexpr int THREADS = CG * SEG;
    static constexpr int TS = TT / SEG;          // steps per thread
    static constexpr int SPW = 32 / CG;          // segments per warp
    static constexpr int NW = THREADS / 32;
    static constexpr int N_IN = BWD ? 3 : 2;
    static constexpr int N_OUT = BWD ? 2 : 1;
    static constexpr int TILE = TT * ROW;
    static constexpr int SMEM_BYTES = (STAGES * N_IN + OUTBUF * N_OUT) * TILE + 128;
    static_assert(CC == 32 || CC == 64 || CC == 128, "a tile row is 8, 16 or 32 groups of 4 channels");
    static_assert(ROW % 128 == 0, "a tile row is whole 128-byte lines (conflict-free shared-memory access)");
    static_assert(TT % SEG == 0 && THREADS % 32 == 0 && THREADS <= 1024 && TT <= 256, "tile shape");
    static_assert(STAGES >= 1 && OUTBUF >= 1, "ring sizes");
};

struct Map4 {  // four affine maps x -> A*x + B, one per channel of a float4
    float4 A, B;
};

__device__ __forceinline__ float4 fma4(float4 a, float4 x, float4 b) {
    return make_float4(fmaf(a.x, x.x, b.x), fmaf(a.y, x.y, b.y), fmaf(a.z, x.z, b.z), fmaf(a.w, x.w, b.w));
}
__device__ __forceinline__ float4 mul4(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 shfl4(float4 v, int delta, bool up) {
    float4 r;
    if (up) {
        r.x = __shfl_up_sync(kFullMask, v.x, delta); r.y = __shfl_up_sync(kFullMask, v.y, delta);
        r.z = __shfl_up_sync(kFullMask, v.z, delta); r.w = __shfl_up_sync(kFullMask, v.w, delta);
    } else {
        r.x = __shfl_down_sync(kFullMask, v.x, delta); r.y = __shfl_down_sync(kFullMask, v.y, delta);
        r.z = __shfl_down_sync(kFullMask, v.z, delta); r.w = __shfl_down_sync(kFullMask, v.w, delta);
    }
    return r;
}

// n_units = N * cblocks * chunks; unit u is chunk u % chunks of (batch element, channel block)
// u / chunks and covers `pieces` tiles.  maps (NULL when chunks == 1): [n_units][2][CC], the chunk
// maps (A, B) a preceding kernel wrote; a unit starts from the fold of the maps of its pair's
// earlier (backward: later) chunks.
// Four adjacent channels of one step, shared memory <-> fp32 registers.
template <typename IO>
__device__ __forceinline__ float4 lds_vec4(uint32_t addr) {
    if constexpr (sizeof(IO) == 4) {
        return tma::lds128(addr);
    } else {
        uint32_t lo, hi;
        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(addr));
        float4 r;
        unpack2<IO>(lo, r.x, r.y);
        unpack2<IO>(hi, r.z, r.w);
        return r;
    }
}
template <typename IO>
__device__ __forceinline__ void sts_vec4(uint32_t addr, float4 v) {
    if constexpr (sizeof(IO) == 4) {
        tma::sts128(addr, v);
    } else {
        const uint32_t lo = pack2<IO>(v.x, v.y), hi = pack2<IO>(v.z, v.w);
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(lo), "r"(hi) : "memory");
    }
}

__device__ __forceinline__ float4 sigmoid4(float4 z) {
    return make_float4(flat::sigmoidf(z.x), flat::sigmoidf(z.y), flat::sigmoidf(z.z), flat::sigmoidf(z.w));
}
__device__ __forceinline__ float4 dsigmoid4(float4 a) {  // a (1 - a), the derivative of the sigmoid at its output a
    return make_float4(a.x * (1.f - a.x), a.y * (1.f - a.y), a.z * (1.f - a.z), a.w * (1.f - a.w));
}

template <int CC, int TT, int SEG, int STAGES, int OUTBUF, bool BWD, typename IO = float, bool SIGMOID = false>
__global__ void __launch_bounds__(CC / 4 * SEG)
cl_stream_kernel(const __grid_constant__ CUtensorMap map_gate, const __grid_constant__ CUtensorMap map_in1,
                 const __grid_constant__ CUtensorMap map_in2, const __grid_constant__ CUtensorMap map_out1,
                 const __grid_constant__ CUtensorMap map_out2, int64_t n_units, int cblocks, int pieces, int chunks,
                 const float *__restrict__ maps) {
    using Cfg = Config<CC, TT, SEG, STAGES, OUTBUF, BWD, IO>;
    constexpr int CG = Cfg::CG, TS = Cfg::TS, SPW = Cfg::SPW, NW = Cfg::NW, N_IN = Cfg::N_IN, N_OUT = Cfg::N_OUT,
                  TILE = Cfg::TILE, ROW = Cfg::ROW;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[STAGES];
    __shared__ float4 s_tot[2][NW][CG][2];  // per warp and channel group: the warp's composed map (A, B)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cg = tid % CG, seg = tid / CG;       // seg = warp * SPW + (lane / CG)
    const int seg_in_warp = lane / CG;
    const uint32_t smem0 = (tma::smem_u32(smem_raw) + 127u) & ~127u;
    const uint32_t out_base = smem0 + STAGES * N_IN * TILE;
    const uint32_t bar0 = tma::smem_u32(&full_bar[0]);
    const int64_t my_units = (int64_t)blockIdx.x < n_units ? (n_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int64_t n_items = my_units * pieces;
    // byte offset of this thread's float4 at its first step inside a tile
    const uint32_t my_off = (uint32_t)(seg * TS * ROW + cg * 4 * (int)sizeof(IO));

    auto coords = [&](int64_t i, int &c0, int &t0, int &n) {
        const int64_t unit = blockIdx.x + (i / pieces) * (int64_t)gridDim.x;
        const int piece = (int)(i % pieces), chunk = (int)(unit % chunks);
        const int64_t pair = unit / chunks;
        n = (int)(pair / cblocks);
        c0 = (int)(pair % cblocks) * CC;
        t0 = (chunk * pieces + (BWD ? pieces - 1 - piece : piece)) * TT;
    };
    auto issue = [&](int64_t i) {  // thread 0: loads of this CTA's i-th tile into stage i % STAGES
        const int stage = (int)(i % STAGES);
        int c0, t0, n;
        coords(i, c0, t0, n);
        const uint32_t bar = bar0 + 8 * stage, dst = smem0 + stage * N_IN * TILE;
        tma::mbar_expect_tx(bar, N_IN * TILE);
        tma::load_box(dst, &map_gate, c0, t0, n, bar);
        tma::load_box(dst + TILE, &map_in1, c0, BWD ? t0 - 1 : t0, n, bar);  // backward: h one step earlier
        if (BWD) tma::load_box(dst + 2 * TILE, &map_in2, c0, t0, n, bar);
    };

    // The scan pass of the chunked form is launched as a programmatic dependent of the map kernel: it
    // issues its first tile loads at once (the map kernel only reads the same inputs) and waits
    // before it reads the maps.  The other uses are ordinary launches: started early behind a kernel of
    // this kind they lost 1-12 % on shapes whose units take several rounds (measured on B200).
    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) tma::mbar_init(bar0 + 8 * s, 1);
        tma::fence_mbar_init();
        for (int64_t i = 0; i < STAGES && i < n_items; i++) issue(i);
    }
    __syncthreads();

    bool timed_out = false, maps_ready = false;
    unsigned phase_bits = 0u;
    int out_slot = 0, buf = 0;
    float4 carry = make_float4(0.f, 0.f, 0.f, 0.f);  // state entering the tile, for this thread's 4 channels
    const float4 one4 = make_float4(1.f, 1.f, 1.f, 1.f), zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

    for (int64_t i = 0; i < n_items; i++) {
        const int stage = (int)(i % STAGES);
        const uint32_t in0 = smem0 + stage * N_IN * TILE + my_off;
        if (i % pieces == 0) {  // a new unit starts
            carry = zero4;
            if (maps != nullptr) {
                if (!maps_ready) {  // the maps come from the kernel before this one
                    grid_dependency_wait();
                    maps_ready = true;
                }
                const int64_t unit = blockIdx.x + (i / pieces) * (int64_t)gridDim.x;
                const int chunk = (int)(unit % chunks);
                const float *m = maps + (unit - chunk) * 2 * CC + cg * 4;  // the pair's first chunk
                const int n_before = BWD ? chunks - 1 - chunk : chunk;
#pragma unroll 4
                for (int q = 0; q < n_before; q++) {
                    const int k = BWD ? chunks - 1 - q : q;
                    const float4 mA = __ldcg(reinterpret_cast<const float4 *>(m + (int64_t)k * 2 * CC));
                    const float4 mB = __ldcg(reinterpret_cast<const float4 *>(m + ((int64_t)k * 2 + 1) * CC));
                    carry = fma4(mA, carry, mB);
                }
            }
        }
        if (!tma::mbar_wait_bounded(bar0 + 8 * stage, (phase_bits >> stage) & 1u)) timed_out = true;
        phase_bits ^= 1u << stage;

        float4 a[TS], x[TS], y[TS];  // x: value | h one step earlier ; y: unused | gout
#pragma unroll
        for (int k = 0; k < TS; k++) {
            a[k] = lds_vec4<IO>(in0 + k * ROW);
            if (SIGMOID) a[k] = sigmoid4(a[k]);
            x[k] = lds_vec4<IO>(in0 + TILE + k * ROW);
            if (BWD) y[k] = lds_vec4<IO>(in0 + 2 * TILE + k * ROW);
        }
        // This thread's run as one map, then the runs of the warp composed (forward: left to
        // right, lower segments first; backward: right to left).
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
        // ... and this thread's own run: the exclusive prefix inside the warp
        {
            float4 eA = shfl4(m.A, CG, !BWD), eB = shfl4(m.B, CG, !BWD);
            if (seg_in_warp == (BWD ? SPW - 1 : 0)) { eA = one4; eB = zero4; }
            s = fma4(eA, s, eB);
        }

        const uint32_t ob = out_base + out_slot * N_OUT * TILE + my_off;
        if (!BWD) {
#pragma unroll
            for (int k = 0; k < TS; k++) {
                s = fma4(a[k], s, x[k]);
                sts_vec4<IO>(ob + k * ROW, s);
            }
        } else {
#pragma unroll
            for (int k = TS - 1; k >= 0; k--) {
                const float4 gb = add4(y[k], s);
                s = mul4(a[k], gb);
                float4 dgate = mul4(gb, x[k]);  // grad of gate = gb_t * h_{t-1}
                if (SIGMOID) dgate = mul4(dgate, dsigmoid4(a[k]));
                sts_vec4<IO>(ob + k * ROW, dgate);
                sts_vec4<IO>(ob + TILE + k * ROW, gb);        // grad of value
            }
        }
        tma::fence_async_smem();
        __syncthreads();
        if (tid == 0) {
            int c0, t0, n;
            coords(i, c0, t0, n);
            tma::store_box(&map_out1, c0, t0, n, ob - my_off);
            if (BWD) tma::store_box(&map_out2, c0, t0, n, ob - my_off + TILE);
            tma::store_commit();
        }
        out_slot = (out_slot + 1 == OUTBUF) ? 0 : out_slot + 1;
        buf ^= 1;
    }
    if (tid == 0) tma::store_wait_read<0>();
    if (timed_out && lane == 0) report_device_wait(7);
}

// The chunk maps of the two-pass form without reading whole chunks (`maps` as the kernel above reads
// it: [unit][2][CC], A then B), folded from the end of the chunk that the NEXT
// chunk depends on -- the forward map from the chunk's last step towards its first, the reverse map
// from its first step towards the last -- in tiles of SEG*TS steps, and abandoned as soon as the
// product of the gates walked so far has dropped to |A| <= cut in every one of the unit's 32
// channels: what was not walked could change B by at most cut times the state entering the walked
// part.  cut = 0 stops only at exactly-zero products; rows whose products stay above the cut are
// walked in full.  Plain vector loads (the walk's length is not known in advance, so nothing is
// prefetched past it): thread (seg, cg) reads 4 adjacent channels of TS consecutive steps, the 8
// threads of a quarter warp one 128-byte row.  Blocks of 128 bytes of channels (32 fp32, 64 bf16 /
// fp16: the 16 threads of a half warp read one row, 8 bytes each), C % 4 == 0; fp32 arithmetic.
template <typename IO>
__device__ __forceinline__ float4 ldcs_vec4(const IO *p) {  // four adjacent channels of one step, streamed
    if constexpr (sizeof(IO) == 4) {
        return __ldcs(reinterpret_cast<const float4 *>(p));
    } else {
        const uint2 v = __ldcs(reinterpret_cast<const uint2 *>(p));
        float4 r;
        unpack2<IO>(v.x, r.x, r.y);
        unpack2<IO>(v.y, r.z, r.w);
        return r;
    }
}

template <int SEG, int TS, bool BWD, bool SIGMOID = false, typename IO = float>
__global__ void __launch_bounds__(32 / (int)sizeof(IO) * SEG)
cl_tail_map_kernel(const IO *__restrict__ gate, const IO *__restrict__ in1,  // value | gout
                   int64_t T, int64_t C, int64_t n_units, int cblocks, int64_t chunk_steps, int chunks, float cut,
                   float *__restrict__ maps) {
    constexpr int CC = 128 / (int)sizeof(IO), CG = CC / 4, THREADS = CG * SEG, NW = THREADS / 32, SPW = 32 / CG, TT = SEG * TS;
    static_assert(THREADS % 32 == 0 && THREADS <= 1024, "whole warps");
    __shared__ float4 s_tot[NW][CG][2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cg = tid % CG, seg = tid / CG, seg_in_warp = lane / CG;
    const float4 one4 = make_float4(1.f, 1.f, 1.f, 1.f), zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    grid_dependents_may_launch();  // the scan pass may set up beside this grid; it waits before it reads `maps`
    for (int64_t unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
        const int chunk = (int)(unit % chunks);
        const int64_t pair = unit / chunks;
        const int64_t n = pair / cblocks;
        const int c = (int)(pair % cblocks) * CC + cg * 4;
        const bool c_ok = c < C;  // C % 4 == 0: a float4 is all in or all out
        const int64_t lo = (int64_t)chunk * chunk_steps, hi = lo + chunk_steps < T ? lo + chunk_steps : T;
        const IO *ga = gate + n * T * C + c, *xa = in1 + n * T * C + c;
        float4 sA = one4, sB = zero4;
        for (int64_t walked = 0; walked < hi - lo; walked += TT) {
            // this thread's TS steps of the tile; steps outside the chunk are the identity
            const int64_t t0 = (BWD ? lo + walked : hi - walked - TT) + (int64_t)seg * TS;
            float4 a[TS], x[TS];
#pragma unroll
            for (int k = 0; k < TS; k++) {
                const int64_t t = t0 + k;
                if (c_ok && t >= lo && t < hi && SSB_INDEX_OK(n * T * C + c + t * C, (n_units / chunks / cblocks) * T * C, 70)) {
                    a[k] = ldcs_vec4<IO>(ga + t * C);
                    x[k] = ldcs_vec4<IO>(xa + t * C);
                    if (SIGMOID) a[k] = sigmoid4(a[k]);
                } else {
                    a[k] = one4;
                    x[k] = zero4;
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
                for (int k = TS - 1; k >= 0; k--) { m.B = mul4(a[k], add4(x[k], m.B)); m.A = mul4(m.A, a[k]); }
            }
#pragma unroll
            for (int d = 1; d < SPW; d <<= 1) {
                const float4 pA = shfl4(m.A, d * CG, !BWD), pB = shfl4(m.B, d * CG, !BWD);
                const bool has = BWD ? (seg_in_warp + d < SPW) : (seg_in_warp >= d);
                if (has) { m.B = fma4(m.A, pB, m.B); m.A = mul4(m.A, pA); }
            }
            if (seg_in_warp == (BWD ? 0 : SPW - 1)) {
                s_tot[warp][cg][0] = m.A;
                s_tot[warp][cg][1] = m.B;
            }
            __syncthreads();
            float4 tA = one4, tB = zero4;  // the tile's map for this thread's 4 channels
#pragma unroll
            for (int q = 0; q < NW; q++) {
                const int w = BWD ? NW - 1 - q : q;
                const float4 wA = s_tot[w][cg][0], wB = s_tot[w][cg][1];
                tB = fma4(wA, tB, wB);
                tA = mul4(tA, wA);
            }
            // the tile lies before (forward) / after (reverse) everything walked so far
            sB = fma4(sA, tB, sB);
            sA = mul4(sA, tA);
            const bool small = fabsf(sA.x) <= cut && fabsf(sA.y) <= cut && fabsf(sA.z) <= cut && fabsf(sA.w) <= cut;
            if (__syncthreads_and(small || !c_ok)) break;  // also the barrier that frees s_tot for the next tile
        }
        if (seg == 0) {
            *reinterpret_cast<float4 *>(maps + (unit * 2) * CC + cg * 4) = sA;
            *reinterpret_cast<float4 *>(maps + (unit * 2 + 1) * CC + cg * 4) = sB;
        }
    }
}

}  // namespace cls
}  // namespace ssb
