// Channels-last kernels with TMA-staged tiles: dense fp32 [N, T, C] (C % 4 == 0, 16-byte aligned
// base), scan over T.  Same tile decomposition, ticket order and look-back protocol as
// scan_cl_lookback.cuh; what changes is where a tile lives while it is processed.
//
//   * The tensor is described to the TMA as a 3-D array {C, T, N}; a box of {CC, TT, 1} is TT
//     time steps of CC adjacent channels of one batch element.  One thread issues
//     `cp.async.bulk.tensor.3d` loads for the tile that will be processed STAGES-1 tiles from
//     now into a ring of shared-memory stages (mbarrier completion), so the bytes in flight do
//     not depend on registers or occupancy and the look-back latency of one tile overlaps with
//     the loads of the next ones.  Out-of-range time steps and channels arrive as zeros and are
//     clipped on the way out by the TMA; the backward fetches h shifted by one time step with a
//     box that starts at t0-1 (coordinate -1 reads the fill value 0 = h before the first step).
//   * Thread (seg, c) owns channel c of the tile and the seg-th run of TT/SEG time steps; it
//     reads its elements from shared memory twice (fold, replay) instead of keeping them in
//     registers.  Adjacent threads read adjacent floats: no bank conflicts, no swizzle needed.
//   * Results are written to a shared-memory tile and leave through a bulk tensor store.
//
// Every wait (mbarrier, look-back flag) is bounded and reports through the device status word.
#pragma once

#include <cuda.h>

#include "scan_cl_lookback.cuh"
#include "scan_tma.cuh"

namespace ssb {
namespace cl3 {

using cl2::Geometry;

template <int CC, int TT, int STAGES, int OUTBUF, bool BWD>
struct Config {
    static constexpr int THREADS = 256;
    static constexpr int SEG = THREADS / CC;       // time segments per tile
    static constexpr int SPT = TT / SEG;           // steps per thread
    static constexpr int N_IN = BWD ? 3 : 2;
    static constexpr int N_OUT = BWD ? 2 : 1;
    static constexpr int TILE_BYTES = TT * CC * 4;
    static constexpr int SMEM_BYTES = (STAGES * N_IN + OUTBUF * N_OUT) * TILE_BYTES + 128;
    static_assert(THREADS % CC == 0 && TT % SEG == 0, "tile shape must divide evenly among the threads");
    static_assert(CC % 32 == 0 && CC * 4 % 16 == 0, "a tile row is whole warps wide");
};

// Record sections of the workspace (same scheme as cl2, CC channels per tile).
__host__ __device__ inline size_t maps_offset(int64_t n_tiles) { return cl2::flags_offset() + cl2::round256((size_t)n_tiles * 4); }
__host__ __device__ inline size_t values_offset(int64_t n_tiles, int cc) {
    return maps_offset(n_tiles) + cl2::round256((size_t)n_tiles * 2 * cc * 4);
}
__host__ __device__ inline size_t workspace_bytes(int64_t n_tiles, int cc) {
    return values_offset(n_tiles, cc) + cl2::round256((size_t)n_tiles * cc * 4);
}

__device__ __forceinline__ float ld_relaxed_f32(const float *p) {
    float v;
    asm volatile("ld.relaxed.gpu.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

template <int CC, int TT, int STAGES, int OUTBUF, bool BWD>
__global__ void __launch_bounds__(256, 1)
cl_tma_kernel(const __grid_constant__ CUtensorMap map_gate, const __grid_constant__ CUtensorMap map_in1,
              const __grid_constant__ CUtensorMap map_in2, const __grid_constant__ CUtensorMap map_out1,
              const __grid_constant__ CUtensorMap map_out2, Geometry geo, lookback::Order order,
              unsigned char *__restrict__ workspace) {
    using Cfg = Config<CC, TT, STAGES, OUTBUF, BWD>;
    constexpr int SEG = Cfg::SEG, SPT = Cfg::SPT, N_IN = Cfg::N_IN, N_OUT = Cfg::N_OUT, TILE = Cfg::TILE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[STAGES];
    __shared__ float s_mapA[2][SEG][CC], s_mapB[2][SEG][CC];
    __shared__ float s_lbA[SEG][CC], s_lbB[SEG][CC];
    __shared__ int s_kind[SEG][CC / 32];
    __shared__ float s_carry[CC];
    __shared__ int s_found;
    __shared__ int64_t s_queue[STAGES];

    unsigned long long *ticket = reinterpret_cast<unsigned long long *>(workspace);
    unsigned *flags = reinterpret_cast<unsigned *>(workspace + cl2::flags_offset());
    float *maps = reinterpret_cast<float *>(workspace + maps_offset(geo.n_tiles));
    float *values = reinterpret_cast<float *>(workspace + values_offset(geo.n_tiles, CC));

    const int tid = threadIdx.x, lane = tid & 31;
    const int c = tid % CC, seg = tid / CC, sub = (tid % CC) / 32;  // sub: which warp of the segment
    const int ord = BWD ? SEG - 1 - seg : seg;
    const uint32_t smem0 = (tma::smem_u32(smem_raw) + 127u) & ~127u;
    const uint32_t in_base = smem0, out_base = smem0 + STAGES * N_IN * TILE;
    const uint32_t bar0 = tma::smem_u32(&full_bar[0]);
    const int64_t n_tickets = order.tickets();
    bool timed_out = false;

    auto issue_loads = [&](int64_t tk, int stage) {  // thread 0 only
        int64_t group, seq;
        if (tk >= n_tickets || !order.decode(tk, group, seq)) return;
        const int64_t n = group / geo.cgroups, cg = group - n * geo.cgroups;
        const int64_t piece = BWD ? geo.pieces - 1 - seq : seq;
        const int c0 = (int)(cg * CC), t0 = (int)(piece * TT);
        const uint32_t bar = bar0 + 8 * stage;
        const uint32_t dst = in_base + stage * N_IN * TILE;
        tma::mbar_expect_tx(bar, N_IN * TILE);
        tma::load_box(dst, &map_gate, c0, t0, (int)n, bar);
        if (!BWD) {
            tma::load_box(dst + TILE, &map_in1, c0, t0, (int)n, bar);
        } else {
            tma::load_box(dst + TILE, &map_in1, c0, t0 - 1, (int)n, bar);  // h shifted by one step
            tma::load_box(dst + 2 * TILE, &map_in2, c0, t0, (int)n, bar);
        }
    };

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) tma::mbar_init(bar0 + 8 * s, 1);
        tma::fence_mbar_init();
        for (int s = 0; s < STAGES - 1; s++) {
            const int64_t tk = (int64_t)atomicAdd(ticket, 1ull);
            s_queue[s] = tk;
            issue_loads(tk, s);
        }
    }
    __syncthreads();

    unsigned phase_bits = 0u;  // parity of each stage's mbarrier, one bit per stage
    int out_slot = 0;
    int buf = 0;
    for (int64_t pos = 0;; pos++) {
        const int stage = (int)(pos % STAGES);
        const int64_t t = s_queue[stage];
        // Reserve the tile that will be processed STAGES-1 iterations from now.
        int64_t t_ahead = 0;
        const int stage_ahead = (int)((pos + STAGES - 1) % STAGES);
        if (tid == 0) t_ahead = (int64_t)atomicAdd(ticket, 1ull);
        if (t >= n_tickets) break;
        int64_t group, seq;
        const bool real = order.decode(t, group, seq);
        if (!real) {
            __syncthreads();  // everyone has read s_queue[stage]; previous tile fully consumed
            if (tid == 0) {
                s_queue[stage_ahead] = t_ahead;
                issue_loads(t_ahead, stage_ahead);
            }
            __syncthreads();
            continue;
        }
        const int64_t n = group / geo.cgroups, cg = group - n * geo.cgroups;
        const int64_t piece = BWD ? geo.pieces - 1 - seq : seq;
        const int64_t rec = group * geo.pieces + seq;
        const int c0 = (int)(cg * CC), t0 = (int)(piece * TT);

        // Early, non-blocking look at the predecessor this segment will read on its first look-back pass.
        unsigned early_flag = 0u;
        float early_val = 0.f;
        if (seg < seq) {  // lane 0 acquires, the warp barrier orders the other lanes' record loads after it
            if (lane == 0) early_flag = cl2::ld_acquire_u32(flags + rec - 1 - seg);
            early_flag = __shfl_sync(kFullMask, early_flag, 0);
            __syncwarp();
            if (early_flag == 2u) early_val = ld_relaxed_f32(values + (rec - 1 - seg) * CC + c);
        }

        // Wait for this tile's loads.
        const uint32_t parity = (phase_bits >> stage) & 1u;
        if (!tma::mbar_wait_bounded(bar0 + 8 * stage, parity)) timed_out = true;
        phase_bits ^= 1u << stage;
        const uint32_t in0 = in_base + stage * N_IN * TILE;
        const uint32_t my_col = (uint32_t)c * 4;

        // Fold this thread's steps into one map.
        float A = 1.f, B = 0.f;
        if (!BWD) {
#pragma unroll
            for (int k = 0; k < SPT; k++) {
                const uint32_t off = (uint32_t)((seg * SPT + k) * CC) * 4 + my_col;
                const float a = tma::lds32(in0 + off), x = tma::lds32(in0 + TILE + off);
                B = fmaf(a, B, x);
                A *= a;
            }
        } else {
#pragma unroll
            for (int k = SPT - 1; k >= 0; k--) {
                const int step = seg * SPT + k;
                const uint32_t off = (uint32_t)(step * CC) * 4 + my_col;
                float a = tma::lds32(in0 + off);
                const float g = tma::lds32(in0 + 2 * TILE + off);
                if ((int64_t)t0 + step >= geo.T) a = 1.f;  // zero fill beyond T must act as the identity
                B = a * (g + B);
                A *= a;
            }
        }
        s_mapA[buf][ord][c] = A;
        s_mapB[buf][ord][c] = B;
        if (tid == 0) tma::store_wait_read<OUTBUF - 1>();  // the out slot about to be reused is free
        __syncthreads();
        if (tid == 0) {  // every thread is past the previous tile: its stage can be refilled
            s_queue[stage_ahead] = t_ahead;
            issue_loads(t_ahead, stage_ahead);
        }

        float pA = 1.f, pB = 0.f;  // exclusive prefix over the segments processed before this one
        for (int j = 0; j < ord; j++) {
            const float qa = s_mapA[buf][j][c], qb = s_mapB[buf][j][c];
            pB = fmaf(qa, pB, qb);
            pA *= qa;
        }
        float totA = 1.f, totB = 0.f;
        if (seg == 0) {
            for (int j = 0; j < SEG; j++) {
                const float qa = s_mapA[buf][j][c], qb = s_mapB[buf][j][c];
                totB = fmaf(qa, totB, qb);
                totA *= qa;
            }
            if (seq > 0) {
                maps[rec * (2 * CC) + c] = totA;
                maps[rec * (2 * CC) + CC + c] = totB;
            } else {
                values[rec * CC + c] = totB;
            }
        }
        float carry = 0.f;
        if (seq > 0) {  // uniform for the CTA
            __syncthreads();  // all record stores of segment 0 happen-before the release below
            if (tid == 0) cl2::st_release_u32(flags + rec, 1u);
            float lbA = 1.f, lbB = 0.f;
            for (int64_t round = 0;; round++) {
                const int64_t back = round * SEG + seg;
                int kind = 0;
                float ra = 1.f, rb = 0.f;
                if (back < seq) {
                    const int64_t r = rec - 1 - back;
                    unsigned f = (round == 0 && early_flag == 2u) ? 2u : 0u;
                    if (lane == 0 && f == 0u) {
                        f = cl2::ld_acquire_u32(flags + r);
                        if (f == 0u) {
                            const uint64_t w0 = lookback::now_ns();
                            while ((f = cl2::ld_acquire_u32(flags + r)) == 0u) {
                                if (lookback::now_ns() - w0 > 1000000000ull) { f = 3u; break; }
                            }
                        }
                    }
                    f = __shfl_sync(kFullMask, f, 0);
                    __syncwarp();
                    if (f == 2u) {
                        kind = 2;
                        ra = 0.f;
                        rb = (round == 0 && early_flag == 2u) ? early_val : ld_relaxed_f32(values + r * CC + c);
                    } else if (f == 1u) {
                        kind = 1;
                        ra = ld_relaxed_f32(maps + r * (2 * CC) + c);
                        rb = ld_relaxed_f32(maps + r * (2 * CC) + CC + c);
                    } else {
                        timed_out = true;
                        kind = 2;
                        ra = 0.f;
                    }
                } else if (back == seq) {
                    kind = 2;
                    ra = 0.f;
                }
                s_lbA[seg][c] = ra;
                s_lbB[seg][c] = rb;
                if (lane == 0) s_kind[seg][sub] = kind;
                __syncthreads();
                if (seg == 0) {
                    int found = 0;
                    for (int j = 0; j < SEG && !found; j++) {
                        int kj = s_kind[j][0];
#pragma unroll
                        for (int w = 1; w < CC / 32; w++) kj = min(kj, s_kind[j][w]);  // a record counts as final only if every warp saw it final
                        if (kj == 0) break;
                        const float qa = s_lbA[j][c], qb = s_lbB[j][c];
                        lbB = fmaf(lbA, qb, lbB);
                        lbA *= qa;
                        if (kj == 2) found = 1;
                    }
                    if (found) {
                        s_carry[c] = lbB;
                        values[rec * CC + c] = fmaf(totA, lbB, totB);
                    }
                    if (tid == 0) s_found = found;
                }
                __syncthreads();
                if (s_found) break;
            }
            if (tid == 0) cl2::st_release_u32(flags + rec, 2u);  // after the barrier: all value stores are ordered before it
            carry = s_carry[c];
        } else {
            __syncthreads();
            if (tid == 0) cl2::st_release_u32(flags + rec, 2u);
        }

        // Replay from shared memory into the output tile(s).
        const uint32_t ob = out_base + out_slot * N_OUT * TILE;
        float h = fmaf(pA, carry, pB);
        if (!BWD) {
#pragma unroll
            for (int k = 0; k < SPT; k++) {
                const uint32_t off = (uint32_t)((seg * SPT + k) * CC) * 4 + my_col;
                const float a = tma::lds32(in0 + off), x = tma::lds32(in0 + TILE + off);
                h = fmaf(a, h, x);
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(ob + off), "f"(h) : "memory");
            }
        } else {
#pragma unroll
            for (int k = SPT - 1; k >= 0; k--) {
                const int step = seg * SPT + k;
                const uint32_t off = (uint32_t)(step * CC) * 4 + my_col;
                float a = tma::lds32(in0 + off);
                const float hp = tma::lds32(in0 + TILE + off), g = tma::lds32(in0 + 2 * TILE + off);
                if ((int64_t)t0 + step >= geo.T) a = 1.f;
                const float gb = g + h;
                h = a * gb;
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(ob + off), "f"(gb * hp) : "memory");
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(ob + TILE + off), "f"(gb) : "memory");
            }
        }
        tma::fence_async_smem();
        __syncthreads();
        if (tid == 0) {
            tma::store_box(&map_out1, c0, t0, (int)n, ob);
            if (BWD) tma::store_box(&map_out2, c0, t0, (int)n, ob + TILE);
            tma::store_commit();
        }
        out_slot = (out_slot + 1 == OUTBUF) ? 0 : out_slot + 1;
        buf ^= 1;
    }
    if (tid == 0) tma::store_wait_read<0>();
    if (timed_out && lane == 0) report_device_wait(5);
}

}  // namespace cl3
}  // namespace ssb
