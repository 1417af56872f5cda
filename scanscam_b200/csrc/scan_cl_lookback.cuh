// Channels-last kernels with the time axis split across CTAs: dense [N, T, C] fp32, scan over T.
//
// A tile is W*L consecutive time steps of one group of 32*VEC adjacent channels of one batch
// element.  A lane owns VEC adjacent channels (one 16-byte load per time step when VEC = 4), a
// warp owns L consecutive steps of the tile, so every load instruction of a warp covers
// 128*VEC contiguous bytes and a thread keeps 2L (forward) or 3L (backward) independent loads
// in flight.  Each thread folds its L steps into one affine map per channel, the W warps of the
// CTA compose their maps through shared memory, and every thread replays its steps from the
// value it starts at.
//
// Tiles of one channel group that follow each other in time are processed by DIFFERENT CTAs at
// the same time.  The per-channel carry crosses tiles through global memory with decoupled
// look-back: a tile first publishes its own map (flag 1), reads its predecessors' records --
// W of them per round, one per warp -- until it meets one whose inclusive value is known
// (flag 2), and then publishes its own inclusive value.  Tiles are handed out by an atomic
// ticket in the same wave order as the rows-layout look-back kernels (scan_lookback.cuh), so a
// tile only ever waits for tiles with smaller tickets and the grid is full however few channel
// groups there are.  Polls are bounded (~1 s) and report through the device status word.
//
// Replaces the reference's transposed kernels (src/scanscam_cuda.cu:471-554, 584-685), whose
// parallelism is limited to N * C/32 blocks.
#pragma once

#include "scan_common.cuh"
#include "scan_lookback.cuh"

namespace ssb {
namespace cl2 {

struct Geometry {
    int64_t N, T, C;
    int64_t cgroups;   // channel groups per batch element
    int64_t pieces;    // tiles along T
    int64_t n_tiles;   // N * cgroups * pieces
};

// Workspace layout: [ticket | flags (4 B per tile) | own maps (2*32*VEC floats per tile) |
// inclusive values (32*VEC floats per tile)], each section 256-byte aligned.
__host__ __device__ inline size_t round256(size_t x) { return (x + 255) & ~(size_t)255; }
__host__ __device__ inline size_t flags_offset() { return lookback::kHeaderBytes; }
__host__ __device__ inline size_t maps_offset(int64_t n_tiles) { return flags_offset() + round256((size_t)n_tiles * 4); }
__host__ __device__ inline size_t values_offset(int64_t n_tiles, int vec) {
    return maps_offset(n_tiles) + round256((size_t)n_tiles * 64 * vec * 4);
}
__host__ __device__ inline size_t workspace_bytes(int64_t n_tiles, int vec) {
    return values_offset(n_tiles, vec) + round256((size_t)n_tiles * 32 * vec * 4);
}
// Only the ticket and the flags have to start at zero.
__host__ __device__ inline size_t bytes_to_clear(int64_t n_tiles) { return maps_offset(n_tiles); }

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_u32(unsigned *p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Coherent (L1-bypassing) load of one lane's channels from a record another CTA has written.
template <int VEC>
__device__ __forceinline__ Pack<float, VEC> load_record_pack(const float *p) {
    Pack<float, VEC> r;
    if constexpr (VEC == 4) {
        asm volatile("ld.relaxed.gpu.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3])
                     : "l"(p)
                     : "memory");
    } else {
        static_assert(VEC == 1, "unsupported pack width");
        asm volatile("ld.relaxed.gpu.global.f32 %0, [%1];" : "=f"(r.v[0]) : "l"(p) : "memory");
    }
    return r;
}

template <int VEC, int W, int L, bool BWD>
__global__ void __launch_bounds__(W * 32)
cl_lookback_kernel(const float *__restrict__ gate, const float *__restrict__ in1,  // value | h
                   const float *__restrict__ in2,                                    // unused | gout
                   float *__restrict__ out1, float *__restrict__ out2,              // h | ggate, gvalue
                   Geometry geo, lookback::Order order, unsigned char *__restrict__ workspace) {
    using P = Pack<float, VEC>;
    constexpr int TILE_T = W * L;
    __shared__ P s_mapA2[2][W][32], s_mapB2[2][W][32];   // per-warp maps of this tile (double-buffered)
    __shared__ P s_lbA[W][32], s_lbB[W][32];     // predecessors' records of one look-back round
    __shared__ int s_kind[W];                    // 0 none, 1 own map, 2 inclusive value
    __shared__ P s_carry[32];
    __shared__ int s_found;
    __shared__ int64_t s_ticket[2];

    unsigned long long *ticket = reinterpret_cast<unsigned long long *>(workspace);
    unsigned *flags = reinterpret_cast<unsigned *>(workspace + flags_offset());
    float *maps = reinterpret_cast<float *>(workspace + maps_offset(geo.n_tiles));
    float *values = reinterpret_cast<float *>(workspace + values_offset(geo.n_tiles, VEC));

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ord = BWD ? W - 1 - warp : warp;  // position of this warp in processing order
    const int64_t n_tickets = order.tickets();
    int buf = 0;
    bool timed_out = false;

    if (tid == 0) s_ticket[0] = (int64_t)atomicAdd(ticket, 1ull);
    __syncthreads();
    int64_t t = s_ticket[0];

    while (t < n_tickets) {
        if (tid == 0) s_ticket[buf ^ 1] = (int64_t)atomicAdd(ticket, 1ull);
        int64_t group, seq;
        const bool real = order.decode(t, group, seq);
        if (!real) {
            __syncthreads();
            t = s_ticket[buf ^ 1];
            buf ^= 1;
            continue;
        }
        const int64_t n = group / geo.cgroups, cg = group - n * geo.cgroups;
        const int64_t piece = BWD ? geo.pieces - 1 - seq : seq;
        const int64_t c0 = cg * (32 * VEC) + lane * VEC;
        const bool c_ok = c0 < geo.C;  // C % VEC == 0 whenever VEC > 1: a pack is all in or all out
        const int64_t t_first = piece * TILE_T + (int64_t)warp * L;
        const int64_t base = n * geo.T * geo.C + c0;
        const int64_t rec = group * geo.pieces + seq;  // record index; predecessors are rec-1, rec-2, ...

        // Early, non-blocking look at this warp's predecessor of the first round: when channel
        // groups outnumber CTAs it finished a wave ago, and its inclusive value is fetched while
        // the tile's own loads are in flight.
        unsigned early_flag = 0u;
        P early_val;
#pragma unroll
        for (int v = 0; v < VEC; v++) early_val.v[v] = 0.f;
        if (warp < seq) {  // lane 0 acquires, the warp barrier orders the other lanes' record loads after it
            if (lane == 0) early_flag = ld_acquire_u32(flags + rec - 1 - warp);
            early_flag = __shfl_sync(kFullMask, early_flag, 0);
            __syncwarp();
            if (early_flag == 2u) early_val = load_record_pack<VEC>(values + (rec - 1 - warp) * (32 * VEC) + lane * VEC);
        }

        P a[L], x[L], y[L];
#pragma unroll
        for (int k = 0; k < L; k++) {
            const int64_t tt = t_first + k;
            if (c_ok && tt < geo.T && SSB_INDEX_OK(base + tt * geo.C, geo.N * geo.T * geo.C, 60)) {
                a[k] = load_stream<float, VEC>(gate + base + tt * geo.C);
                if (!BWD) {
                    x[k] = load_stream<float, VEC>(in1 + base + tt * geo.C);
                } else {
                    y[k] = load_stream<float, VEC>(in2 + base + tt * geo.C);
                    if (tt > 0) {
                        x[k] = load_stream<float, VEC>(in1 + base + (tt - 1) * geo.C);  // h_{t-1}
                    } else {
#pragma unroll
                        for (int v = 0; v < VEC; v++) x[k].v[v] = 0.f;
                    }
                }
            } else {
#pragma unroll
                for (int v = 0; v < VEC; v++) { a[k].v[v] = 1.f; x[k].v[v] = 0.f; y[k].v[v] = 0.f; }
            }
        }
        // This thread's L steps as one map per channel.
        P mA, mB;
#pragma unroll
        for (int v = 0; v < VEC; v++) {
            float A = 1.f, B = 0.f;
            if (!BWD) {
#pragma unroll
                for (int k = 0; k < L; k++) { B = fmaf(a[k].v[v], B, x[k].v[v]); A *= a[k].v[v]; }
            } else {
#pragma unroll
                for (int k = L - 1; k >= 0; k--) { B = a[k].v[v] * (y[k].v[v] + B); A *= a[k].v[v]; }
            }
            mA.v[v] = A;
            mB.v[v] = B;
        }
        P (*s_mapA)[32] = s_mapA2[buf];
        P (*s_mapB)[32] = s_mapB2[buf];
        s_mapA[ord][lane] = mA;
        s_mapB[ord][lane] = mB;
        __syncthreads();
        const int64_t t_next = s_ticket[buf ^ 1];

        // Exclusive prefix over the warps processed before this one.
        P pA, pB;
#pragma unroll
        for (int v = 0; v < VEC; v++) { pA.v[v] = 1.f; pB.v[v] = 0.f; }
        for (int j = 0; j < ord; j++) {
            const P qa = s_mapA[j][lane], qb = s_mapB[j][lane];
#pragma unroll
            for (int v = 0; v < VEC; v++) {
                pB.v[v] = fmaf(qa.v[v], pB.v[v], qb.v[v]);
                pA.v[v] *= qa.v[v];
            }
        }
        // Warp 0 also forms the whole tile's map and publishes it.
        P totA, totB;
        if (warp == 0) {
#pragma unroll
            for (int v = 0; v < VEC; v++) { totA.v[v] = 1.f; totB.v[v] = 0.f; }
            for (int j = 0; j < W; j++) {
                const P qa = s_mapA[j][lane], qb = s_mapB[j][lane];
#pragma unroll
                for (int v = 0; v < VEC; v++) {
                    totB.v[v] = fmaf(qa.v[v], totB.v[v], qb.v[v]);
                    totA.v[v] *= qa.v[v];
                }
            }
            if (seq > 0) {
                float *m = maps + rec * (64 * VEC) + lane * VEC;
                *reinterpret_cast<P *>(m) = totA;
                *reinterpret_cast<P *>(m + 32 * VEC) = totB;
                __syncwarp();  // all lanes' record stores happen-before lane 0's release store
                if (lane == 0) st_release_u32(flags + rec, 1u);
            } else {
                *reinterpret_cast<P *>(values + rec * (32 * VEC) + lane * VEC) = totB;  // starts from 0
                __syncwarp();  // all lanes' record stores happen-before lane 0's release store
                if (lane == 0) st_release_u32(flags + rec, 2u);
            }
        }

        P carry;
#pragma unroll
        for (int v = 0; v < VEC; v++) carry.v[v] = 0.f;
        if (seq > 0) {  // uniform for the CTA
            P lbA, lbB;  // warp 0: composition of the predecessors inspected so far
#pragma unroll
            for (int v = 0; v < VEC; v++) { lbA.v[v] = 1.f; lbB.v[v] = 0.f; }
            for (int64_t round = 0;; round++) {
                const int64_t back = round * W + warp;  // this warp reads the (back+1)-th predecessor
                int kind = 0;
                P ra, rb;
#pragma unroll
                for (int v = 0; v < VEC; v++) { ra.v[v] = 1.f; rb.v[v] = 0.f; }
                if (back < seq) {
                    const int64_t r = rec - 1 - back;
                    // Lane 0 polls the tile's flag; the outcome is shared so that all channels of
                    // the tile take the same decision, then every lane reads its channels.
                    unsigned f = (round == 0 && early_flag == 2u) ? 2u : 0u;
                    if (lane == 0 && f == 0u) {
                        f = ld_acquire_u32(flags + r);
                        if (f == 0u) {
                            const uint64_t t0 = lookback::now_ns();
                            while ((f = ld_acquire_u32(flags + r)) == 0u) {
                                if (lookback::now_ns() - t0 > 1000000000ull) { f = 3u; break; }
                            }
                        }
                    }
                    f = __shfl_sync(kFullMask, f, 0);
                    __syncwarp();
                    if (f == 2u) {
                        kind = 2;
                        rb = (round == 0 && early_flag == 2u) ? early_val
                                                              : load_record_pack<VEC>(values + r * (32 * VEC) + lane * VEC);
#pragma unroll
                        for (int v = 0; v < VEC; v++) ra.v[v] = 0.f;
                    } else if (f == 1u) {
                        kind = 1;
                        const float *m = maps + r * (64 * VEC) + lane * VEC;
                        ra = load_record_pack<VEC>(m);
                        rb = load_record_pack<VEC>(m + 32 * VEC);
                    } else {  // timed out: treat as the start of the sequence
                        timed_out = true;
                        kind = 2;
#pragma unroll
                        for (int v = 0; v < VEC; v++) { ra.v[v] = 0.f; rb.v[v] = 0.f; }
                    }
                } else if (back == seq) {  // just before the first tile: the scan starts from 0
                    kind = 2;
#pragma unroll
                    for (int v = 0; v < VEC; v++) { ra.v[v] = 0.f; rb.v[v] = 0.f; }
                }
                s_lbA[warp][lane] = ra;
                s_lbB[warp][lane] = rb;
                if (lane == 0) s_kind[warp] = kind;
                __syncthreads();
                if (warp == 0) {
                    int found = 0;
                    for (int j = 0; j < W && !found; j++) {
                        const int kj = s_kind[j];
                        if (kj == 0) break;
                        const P qa = s_lbA[j][lane], qb = s_lbB[j][lane];
#pragma unroll
                        for (int v = 0; v < VEC; v++) {  // farther record applies first
                            lbB.v[v] = fmaf(lbA.v[v], qb.v[v], lbB.v[v]);
                            lbA.v[v] *= qa.v[v];
                        }
                        if (kj == 2) found = 1;
                    }
                    if (found) {
                        s_carry[lane] = lbB;
                        P incl;
#pragma unroll
                        for (int v = 0; v < VEC; v++) incl.v[v] = fmaf(totA.v[v], lbB.v[v], totB.v[v]);
                        *reinterpret_cast<P *>(values + rec * (32 * VEC) + lane * VEC) = incl;
                        __syncwarp();
                        if (lane == 0) st_release_u32(flags + rec, 2u);
                    }
                    if (lane == 0) s_found = found;
                }
                __syncthreads();
                if (s_found) break;
            }
            carry = s_carry[lane];
        }

        // Replay this thread's steps from its starting value.
        P start;
#pragma unroll
        for (int v = 0; v < VEC; v++) start.v[v] = fmaf(pA.v[v], carry.v[v], pB.v[v]);
        if (!BWD) {
#pragma unroll
            for (int k = 0; k < L; k++) {
                P o;
#pragma unroll
                for (int v = 0; v < VEC; v++) {
                    start.v[v] = fmaf(a[k].v[v], start.v[v], x[k].v[v]);
                    o.v[v] = start.v[v];
                }
                const int64_t tt = t_first + k;
                if (c_ok && tt < geo.T && SSB_INDEX_OK(base + tt * geo.C, geo.N * geo.T * geo.C, 61)) store_stream<float, VEC>(out1 + base + tt * geo.C, o);
            }
        } else {
#pragma unroll
            for (int k = L - 1; k >= 0; k--) {
                P oa, og;
#pragma unroll
                for (int v = 0; v < VEC; v++) {
                    const float gb = y[k].v[v] + start.v[v];
                    start.v[v] = a[k].v[v] * gb;
                    og.v[v] = gb;
                    oa.v[v] = gb * x[k].v[v];
                }
                const int64_t tt = t_first + k;
                if (c_ok && tt < geo.T && SSB_INDEX_OK(base + tt * geo.C, geo.N * geo.T * geo.C, 62)) {
                    store_stream<float, VEC>(out1 + base + tt * geo.C, oa);
                    store_stream<float, VEC>(out2 + base + tt * geo.C, og);
                }
            }
        }
        t = t_next;
        buf ^= 1;
    }
    if (timed_out && lane == 0) report_device_wait(4);
}

}  // namespace cl2
}  // namespace ssb
