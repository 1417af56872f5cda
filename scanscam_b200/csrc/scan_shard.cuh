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

// ---------------------------------------------------------------------------------------------
// Exchange of the shard maps through peer memory (one process per GPU, every GPU of the node can
// store into every other's buffer over NVLink).  Every rank owns one exchange buffer:
//   data  [direction 2][generation 2][source rank world][rows][2] floats   -- the maps, as
//         ssb_shard_carry_f32 reads them ([n_shards, rows, 2])
//   flags [direction 2][generation 2][source rank world] 32-bit epochs
//   done  [direction 2] 32-bit CTA counters (local use)
// The map kernel of rank r stores each row's (A, B) into slot [dir][gen][r] of EVERY rank's buffer
// (plain stores), and the last CTA to finish publishes flag [dir][gen][r] = epoch at every rank
// after a system-wide fence.  The carry kernel of each rank waits -- bounded, about a second --
// until ALL `world` flags of its own buffer have reached the epoch, then folds the maps it needs.
// Because every rank waits for every rank, no rank can be more than one call ahead of another, and
// two generations of slots (epoch parity) are enough: a slot is overwritten only by a call two
// epochs later, which its writer can reach only after the reader's previous wait has been served.
// ---------------------------------------------------------------------------------------------
constexpr int kMaxPeers = 8;
struct PeerExchange {
    int world, rank;
    int64_t rows;
    unsigned char *buf[kMaxPeers];
};
__host__ __device__ inline size_t px_round256(size_t x) { return (x + 255) & ~(size_t)255; }
__host__ __device__ inline size_t px_slot_bytes(int64_t rows) { return (size_t)rows * 2 * sizeof(float); }
__host__ __device__ inline size_t px_data_offset(int world, int64_t rows, int dir, int gen, int src) {
    return ((size_t)((dir * 2 + gen) * world + src)) * px_slot_bytes(rows);
}
__host__ __device__ inline size_t px_flags_offset(int world, int64_t rows) { return px_round256(px_data_offset(world, rows, 2, 0, 0)); }
__host__ __device__ inline size_t px_flag_offset(int world, int64_t rows, int dir, int gen, int src) {
    return px_flags_offset(world, rows) + ((size_t)((dir * 2 + gen) * world + src)) * sizeof(unsigned);
}
__host__ __device__ inline size_t px_done_offset(int world, int64_t rows, int dir) {
    return px_flags_offset(world, rows) + px_round256((size_t)4 * kMaxPeers * sizeof(unsigned)) + (size_t)dir * sizeof(unsigned);
}
__host__ __device__ inline size_t px_total_bytes(int world, int64_t rows) { return px_done_offset(world, rows, 0) + 256; }

__device__ __forceinline__ void st_release_sys_u32(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// PUBLISH: besides (or instead of) `agg`, every row's map goes into slot [dir][gen][px.rank] of every
// rank's exchange buffer, and the CTA that finishes last raises the flags (see above).
template <int THREADS, int U, bool BWD, bool PUBLISH = false>
__global__ void __launch_bounds__(THREADS)
tail_map_kernel(const float4 *__restrict__ gate, const float4 *__restrict__ in1,  // value | gout
                int64_t rows, int64_t T4, float cut, float *__restrict__ agg,     // [rows][2] (PUBLISH: may be NULL)
                unsigned long long *__restrict__ walked,                           // optional: += elements read per tensor
                PeerExchange px, int gen, unsigned epoch) {                      // PUBLISH only (else ignored)
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
            if (agg != nullptr) {
                agg[2 * row] = sA;
                agg[2 * row + 1] = sB;
            }
            if (PUBLISH) {
                const size_t off = px_data_offset(px.world, px.rows, BWD ? 1 : 0, gen, px.rank) + (size_t)row * sizeof(float2);
                for (int p = 0; p < px.world; p++) *reinterpret_cast<float2 *>(px.buf[p] + off) = make_float2(sA, sB);
            }
            if (walked != nullptr) {
                const int64_t vecs = k * CAP < T4 ? k * CAP : T4;
                atomicAdd(walked, (unsigned long long)(vecs * 4));
            }
        }
    }
    if (PUBLISH && tid == 0) {
        // this CTA's stores to the peers are ordered before its ticket; the CTA that draws the last
        // ticket has therefore (transitively) every CTA's stores before its flag stores
        unsigned *done = reinterpret_cast<unsigned *>(px.buf[px.rank] + px_done_offset(px.world, px.rows, BWD ? 1 : 0));
        __threadfence_system();
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            atomicExch(done, 0u);  // ready for the next call (stream order keeps calls of one direction apart)
            __threadfence_system();
            const size_t foff = px_flag_offset(px.world, px.rows, BWD ? 1 : 0, gen, px.rank);
            for (int p = 0; p < px.world; p++) st_release_sys_u32(reinterpret_cast<unsigned *>(px.buf[p] + foff), epoch);
        }
    }
}

// The consumer side of the exchange: waits (bounded) until every rank's flag of this direction and
// generation has reached `epoch`, then folds the maps of the shards before (forward) or after
// (reverse) this rank's own into the state its shard starts from -- shard_carry_kernel on the maps
// the peers stored into this rank's buffer.  One thread per row; every CTA polls for itself.
__global__ void peer_carry_kernel(PeerExchange px, int dir, int gen, unsigned epoch, float *__restrict__ carry) {
    __shared__ int s_timed_out;
    if (threadIdx.x == 0) s_timed_out = 0;
    __syncthreads();
    if ((int)threadIdx.x < px.world) {
        const unsigned *flag = reinterpret_cast<const unsigned *>(px.buf[px.rank] + px_flag_offset(px.world, px.rows, dir, gen, (int)threadIdx.x));
        if ((int)(ld_acquire_sys_u32(flag) - epoch) < 0) {
            uint64_t t0;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
            while ((int)(ld_acquire_sys_u32(flag) - epoch) < 0) {
                uint64_t t1;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                if (t1 - t0 > 1000000000ull) { s_timed_out = 1; break; }
            }
        }
    }
    __syncthreads();  // the pollers' acquire loads happen-before every thread's reads of the maps
    if (s_timed_out && threadIdx.x == 0) report_device_wait(9);
    const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= px.rows) return;
    const unsigned char *base = px.buf[px.rank];
    float x = 0.f;
    if (dir == 0) {
        for (int s = 0; s < px.rank; s++) {
            const float2 m = reinterpret_cast<const float2 *>(base + px_data_offset(px.world, px.rows, 0, gen, s))[r];
            x = fmaf(m.x, x, m.y);
        }
    } else {
        for (int s = px.world - 1; s > px.rank; s--) {
            const float2 m = reinterpret_cast<const float2 *>(base + px_data_offset(px.world, px.rows, 1, gen, s))[r];
            x = fmaf(m.x, x, m.y);
        }
    }
    carry[r] = x;
}

// Adds `n` to a device counter (the traffic account of the shapes that fall back to a full reduction).
__global__ void add_counter_kernel(unsigned long long *counter, unsigned long long n) { atomicAdd(counter, n); }

}  // namespace shard
}  // namespace ssb
