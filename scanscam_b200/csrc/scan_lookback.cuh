// Long-sequence kernels: rows that are longer than one span are split into spans that
// DIFFERENT CTAs process concurrently, and the carry travels from span to span through global
// memory with decoupled look-back (Merrill & Garland's single-pass scan, applied to the affine
// maps of this recurrence).  Same span arithmetic as the flat family (scan_flat.cuh); what
// differs is who processes which span and where the carry comes from.
//
// Scheduling.  Spans are handed out by an atomic ticket, so a span is only ever owned by a CTA
// that is already running, and every span depends only on spans with smaller tickets: the
// scheme cannot deadlock, whatever the number of resident CTAs.  Tickets are ordered so that the
// spans in flight at any time are K consecutive pieces of every row (K = CTAs / rows, at least
// 1): a span's predecessor is then at most K-1 tickets away or belongs to the previous wave,
// which keeps the look-back short, and all CTAs stay busy however few rows there are.
//
// Per-span record in the workspace: 16 bytes, written and read as one scalar 128-bit unit (see Record).  A map
// with A == 0 is as good as a prefix (it forgets its input), so exact-zero gates cut the
// look-back short.  Every poll loop gives up after about a second, reports through the device
// status word and lets the kernel run to completion.
#pragma once

#include "scan_common.cuh"

namespace ssb {
namespace lookback {

// One 16-byte record per span: {x, y, flag, unused}.  flag 1: (x, y) = (A, B), the span's own
// map.  flag 2: x = P, the scan value at the span's end with everything before it applied.
// A record is written with ONE 128-bit store and read with ONE 128-bit load, both of the scalar
// `.b128` type (PTX ISA 8.3): a scalar access is single-copy atomic, so a reader that sees the
// flag sees the data stored with it.  (The vector forms `.v4.b32` are, in the memory model, four
// separate 32-bit accesses and would promise no such thing.)  The flag of a record only ever
// moves 0 -> 1 -> 2 and every state carries all the data its readers need, so relaxed ordering
// is enough: nothing else is published through the record.
struct alignas(16) Record {
    float x, y;
    unsigned flag, unused;
};

constexpr unsigned kFlagAgg = 1u, kFlagPrefix = 2u;
constexpr size_t kHeaderBytes = 256;  // ticket counter, padded

__device__ __forceinline__ Record load_record(const Record *p) {
    unsigned long long lo, hi;
    asm volatile("{\n\t.reg .b128 r;\n\tld.relaxed.gpu.global.b128 r, [%2];\n\tmov.b128 {%0, %1}, r;\n\t}"
                 : "=l"(lo), "=l"(hi)
                 : "l"(p)
                 : "memory");
    Record r;
    r.x = __uint_as_float((unsigned)lo);
    r.y = __uint_as_float((unsigned)(lo >> 32));
    r.flag = (unsigned)hi;
    r.unused = (unsigned)(hi >> 32);
    return r;
}

__device__ __forceinline__ void store_record(Record *p, float x, float y, unsigned flag) {
    const unsigned long long lo = (unsigned long long)__float_as_uint(x) | ((unsigned long long)__float_as_uint(y) << 32);
    const unsigned long long hi = (unsigned long long)flag;
    asm volatile("{\n\t.reg .b128 r;\n\tmov.b128 r, {%1, %2};\n\tst.relaxed.gpu.global.b128 [%0], r;\n\t}" ::"l"(p), "l"(lo), "l"(hi)
                 : "memory");
}

__device__ __forceinline__ uint64_t now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Decodes a ticket into (row, piece).  Returns false for the padding tickets of a last,
// partial wave.
struct Order {
    int64_t rows, pieces, k, wave;  // wave = rows * k tickets
    __device__ __forceinline__ bool decode(int64_t t, int64_t &row, int64_t &piece) const {
        const int64_t w = t / wave, i = t - w * wave;
        row = i / k;
        piece = w * k + (i - row * k);
        return piece < pieces;
    }
    __device__ __forceinline__ int64_t tickets() const { return ((pieces + k - 1) / k) * wave; }
};

// Warp-wide look-back (all 32 lanes of one warp call it).  `rec` points at the record of the
// nearest predecessor, `count` predecessors exist (records rec[0], rec[-1], ...).  `early` is
// what this lane read from its record of the first window before the span's arithmetic began
// (flag 0 if it was not ready then, or if the lane has no record).  Returns the carry: the scan
// value just before the calling span, the sequence starting from 0 before the farthest
// predecessor.
__device__ __forceinline__ float look_back(const Record *rec, int64_t count, int lane, Record early,
                                           bool &timed_out) {
    float mA = 1.f, mB = 0.f;  // composition of the predecessors inspected so far (nearest applied last)
    int64_t done = 0;
    while (true) {
        const int64_t mine = done + lane;
        float A = 1.f, B = 0.f;
        bool is_prefix = false;
        if (mine == count) {  // the virtual record before the first span: the scan starts from 0
            A = 0.f;
            is_prefix = true;
        } else if (mine < count) {
            Record r = early;
            if (done > 0 || r.flag == 0u) {
                r = load_record(rec - mine);
                if (r.flag == 0u) {
                    const uint64_t t0 = now_ns();
                    while ((r = load_record(rec - mine)).flag == 0u) {
                        if (now_ns() - t0 > 1000000000ull) { timed_out = true; break; }
                    }
                }
            }
            if (r.flag == kFlagPrefix) {
                A = 0.f; B = r.x; is_prefix = true;
            } else if (r.flag == kFlagAgg) {
                A = r.x; B = r.y; is_prefix = (A == 0.f);
            } else {  // timed out: pretend the sequence starts here
                A = 0.f; B = 0.f; is_prefix = true;
            }
        }
        const unsigned stops = __ballot_sync(kFullMask, is_prefix);
        const int stop_lane = stops ? __ffs(stops) - 1 : 32;
        if (lane > stop_lane) { A = 1.f; B = 0.f; }
        // suffix composition: lane 0 ends with map_0 o map_1 o ... (farthest applied first)
        warp_scan_reverse<float>(A, B, lane);
        const float wA = __shfl_sync(kFullMask, A, 0), wB = __shfl_sync(kFullMask, B, 0);
        // the window is farther than what was composed so far: total(x) = m(window(x))
        mB = fmaf(mA, wB, mB);
        mA *= wA;
        if (stops) break;
        done += 32;
    }
    return mB;  // mA is 0 here: the chain ended in a prefix
}

// ---------------------------------------------------------------------------------------
// Forward / backward scan over long rows.  BWD = false: h_t = a_t*h_{t-1} + b_t.
// BWD = true : c_t = a_t*(g_t + c_{t+1}) from the right, gb_t = g_t + c_{t+1}, ga_t = gb_t*h_{t-1};
//              `pieces` are then counted from the right end of the row.
// ---------------------------------------------------------------------------------------
template <int THREADS, int U, bool BWD>
__global__ void __launch_bounds__(THREADS)
lookback_kernel(const float4 *__restrict__ gate, const float4 *__restrict__ in1,  // value | h
                const float4 *__restrict__ in2,                                    // unused | gout
                float4 *__restrict__ out1, float4 *__restrict__ out2,              // h | ggate, gvalue
                int64_t T4, Order order, const float *__restrict__ carry_in,       // h_in | c_in
                const float *__restrict__ h_prev, unsigned char *__restrict__ workspace) {
    constexpr int NW = THREADS / 32;
    constexpr int NE = NW * U;
    static_assert(NE <= 32, "second-level scan is one warp wide");
    constexpr int CAP = THREADS * U;
    __shared__ float2 s_tot[2][NE];
    __shared__ float s_hw[2][NE];
    __shared__ int64_t s_ticket[2];

    unsigned long long *ticket = reinterpret_cast<unsigned long long *>(workspace);
    Record *records = reinterpret_cast<Record *>(workspace + kHeaderBytes);
    const float *h_scalar = reinterpret_cast<const float *>(in1);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t n_tickets = order.tickets();
    [[maybe_unused]] const int64_t extent = order.rows * T4;  // float4s per tensor (checked builds)
    int buf = 0;
    bool timed_out = false;

    if (tid == 0) s_ticket[0] = (int64_t)atomicAdd(ticket, 1ull);
    __syncthreads();
    int64_t t = s_ticket[0];

    while (t < n_tickets) {
        // Prefetch the next ticket; it is published by this span's first barrier.
        if (tid == 0) s_ticket[buf ^ 1] = (int64_t)atomicAdd(ticket, 1ull);
        int64_t row, seq;  // seq: position of the piece in processing order (0 = first processed)
        const bool real = order.decode(t, row, seq);
        if (!real) {  // padding ticket (uniform for the CTA)
            __syncthreads();
            t = s_ticket[buf ^ 1];
            buf ^= 1;
            continue;
        }
        const int64_t piece = BWD ? order.pieces - 1 - seq : seq;  // position in the row, left to right
        const int64_t first_vec = row * T4 + piece * CAP;
        const int64_t left = T4 - piece * CAP;
        const int n_vec = (int)(left < CAP ? left : CAP);
        Record *my_rec = records + row * order.pieces + seq;

        // Early, non-blocking look at the predecessors' records: when rows outnumber CTAs the
        // predecessor finished a whole wave ago and its prefix is already there, so the
        // look-back below costs no extra memory round trip.
        Record early;
        early.x = early.y = 0.f;
        early.flag = early.unused = 0u;
        if (lane < seq) early = load_record(my_rec - 1 - lane);

        float4 a[U], x[U], y[U];
        float edge = 0.f;
        if (BWD && tid == 0 && piece > 0 && SSB_INDEX_OK(first_vec * 4 - 1, extent * 4, 20)) edge = h_scalar[first_vec * 4 - 1];
#pragma unroll
        for (int j = 0; j < U; j++) {
            const int o = j * THREADS + tid;
            if (o < n_vec && SSB_INDEX_OK(first_vec + o, extent, 21)) {
                a[j] = __ldcs(gate + first_vec + o);
                x[j] = __ldcs(in1 + first_vec + o);
                if (BWD) y[j] = __ldcs(in2 + first_vec + o);
            } else {
                a[j] = make_float4(1.f, 1.f, 1.f, 1.f);
                x[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (BWD) y[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        // Row ends: the first element forgets the left; caller-supplied carries are folded in.
        if (!BWD) {
            if (piece == 0 && tid == 0) {
                if (carry_in != nullptr) x[0].x = fmaf(a[0].x, carry_in[row], x[0].x);
                a[0].x = 0.f;
            }
        } else {
            if (piece == 0 && tid == 0) {
                a[0].x = 0.f;
                edge = h_prev != nullptr ? h_prev[row] : 0.f;
            }
            if (seq == 0 && carry_in != nullptr) {
#pragma unroll
                for (int j = 0; j < U; j++)
                    if (j * THREADS + tid == n_vec - 1) y[j].w += carry_in[row];
            }
        }
        float A[U], B[U];
#pragma unroll
        for (int j = 0; j < U; j++) {
            if (!BWD) {
                B[j] = fmaf(a[j].y, x[j].x, x[j].y);
                B[j] = fmaf(a[j].z, B[j], x[j].z);
                B[j] = fmaf(a[j].w, B[j], x[j].w);
            } else {
                B[j] = a[j].w * y[j].w;
                B[j] = a[j].z * (y[j].z + B[j]);
                B[j] = a[j].y * (y[j].y + B[j]);
                B[j] = a[j].x * (y[j].x + B[j]);
            }
            A[j] = (a[j].x * a[j].y) * (a[j].z * a[j].w);
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
        if (BWD && lane == 31) {
#pragma unroll
            for (int j = 0; j < U; j++) s_hw[buf][j * NW + warp] = x[j].w;
        }
        __syncthreads();
        const int64_t t_next = s_ticket[buf ^ 1];
        float tA = 1.f, tB = 0.f;
        if (lane < NE) {
            const float2 tt = s_tot[buf][lane];
            tA = tt.x;
            tB = tt.y;
        }
        if (!BWD) warp_scan_forward<float>(tA, tB, lane);
        else warp_scan_reverse<float>(tA, tB, lane);
        const float span_A = __shfl_sync(kFullMask, tA, BWD ? 0 : NE - 1);
        const float span_B = __shfl_sync(kFullMask, tB, BWD ? 0 : NE - 1);

        // Carry entering the span.  Every warp performs the look-back for itself (the records are
        // a few hundred bytes and sit in L2), so no warp waits at a barrier for another one's
        // polling; only warp 0 publishes.  Warps may meet a predecessor in different states and
        // compose the same carry in a different order: equal up to rounding.
        float carry = 0.f;
        if (seq > 0) {  // uniform for the CTA
            if (tid == 0) store_record(my_rec, span_A, span_B, kFlagAgg);
            // Only the pieces of this row processed before this one are predecessors.
            carry = look_back(my_rec - 1, seq, lane, early, timed_out);
            if (tid == 0) store_record(my_rec, fmaf(span_A, carry, span_B), 0.f, kFlagPrefix);
        } else if (tid == 0) {
            store_record(my_rec, span_B, 0.f, kFlagPrefix);  // starts from 0: map(0) = B
        }

        if (!BWD) {
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int q = j * NW + warp;
                float pA = __shfl_sync(kFullMask, tA, q > 0 ? q - 1 : 0);
                float pB = __shfl_sync(kFullMask, tB, q > 0 ? q - 1 : 0);
                if (q == 0) { pA = 1.f; pB = 0.f; }
                const float warp_start = fmaf(pA, carry, pB);
                float lA = __shfl_up_sync(kFullMask, A[j], 1);
                float lB = __shfl_up_sync(kFullMask, B[j], 1);
                if (lane == 0) { lA = 1.f; lB = 0.f; }
                float h = fmaf(lA, warp_start, lB);
                float4 o4;
                h = fmaf(a[j].x, h, x[j].x); o4.x = h;
                h = fmaf(a[j].y, h, x[j].y); o4.y = h;
                h = fmaf(a[j].z, h, x[j].z); o4.z = h;
                h = fmaf(a[j].w, h, x[j].w); o4.w = h;
                const int o = j * THREADS + tid;
                if (o < n_vec && SSB_INDEX_OK(first_vec + o, extent, 22)) __stcs(out1 + first_vec + o, o4);
            }
        } else {
#pragma unroll
            for (int j = U - 1; j >= 0; j--) {
                const int q = j * NW + warp;
                float pA = __shfl_sync(kFullMask, tA, q < 31 ? q + 1 : 31);
                float pD = __shfl_sync(kFullMask, tB, q < 31 ? q + 1 : 31);
                if (q == NE - 1) { pA = 1.f; pD = 0.f; }
                const float warp_start = fmaf(pA, carry, pD);
                float lA = __shfl_down_sync(kFullMask, A[j], 1);
                float lD = __shfl_down_sync(kFullMask, B[j], 1);
                if (lane == 31) { lA = 1.f; lD = 0.f; }
                float c = fmaf(lA, warp_start, lD);
                float hl = __shfl_up_sync(kFullMask, x[j].w, 1);
                if (lane == 0) hl = q > 0 ? s_hw[buf][q - 1] : edge;
                float4 oa, og;
                float gb;
                gb = y[j].w + c; c = a[j].w * gb; og.w = gb; oa.w = gb * x[j].z;
                gb = y[j].z + c; c = a[j].z * gb; og.z = gb; oa.z = gb * x[j].y;
                gb = y[j].y + c; c = a[j].y * gb; og.y = gb; oa.y = gb * x[j].x;
                gb = y[j].x + c; og.x = gb; oa.x = gb * hl;
                const int o = j * THREADS + tid;
                if (o < n_vec && SSB_INDEX_OK(first_vec + o, extent, 23)) {
                    __stcs(out1 + first_vec + o, oa);
                    __stcs(out2 + first_vec + o, og);
                }
            }
        }
        t = t_next;
        buf ^= 1;
    }
    if (timed_out && lane == 0) report_device_wait(3);
}

// One warp runs the look-back on a single predecessor record that nobody will ever publish:
// the poll gives up after its time limit, the carry falls back to 0 and the device status word
// is set.  Used by the self-test entry point to exercise the give-up path without hanging.
__global__ void wait_probe_kernel(Record *rec, float *carry_out) {
    const int lane = threadIdx.x & 31;
    bool timed_out = false;
    Record none;
    none.x = none.y = 0.f;
    none.flag = none.unused = 0u;
    const float c = look_back(rec, 1, lane, none, timed_out);
    if (lane == 0) {
        *carry_out = c;
        if (timed_out) report_device_wait(3);
    }
}

// ---------------------------------------------------------------------------------------
// Row aggregates for sequence sharding, two launches and no waiting: every span writes its own
// map (A, B) to the workspace, then one warp per row folds the row's spans in order.
// BWD = false: maps of h_t = a_t*h_{t-1} + b_t.  BWD = true: maps of c_t = a_t*(g_t + c_{t+1}).
// ---------------------------------------------------------------------------------------
template <int THREADS, int U, bool BWD>
__global__ void __launch_bounds__(THREADS)
span_maps_kernel(const float4 *__restrict__ gate, const float4 *__restrict__ in1, int64_t rows, int64_t T4,
                 int64_t pieces, float2 *__restrict__ maps) {
    constexpr int NW = THREADS / 32;
    constexpr int NE = NW * U;
    static_assert(NE <= 32, "second-level scan is one warp wide");
    constexpr int CAP = THREADS * U;
    __shared__ float2 s_tot[2][NE];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t n_spans = rows * pieces;
    [[maybe_unused]] const int64_t extent = rows * T4;
    int buf = 0;
    // piece-major order: the spans in flight are the same piece of consecutive rows
    for (int64_t s = blockIdx.x; s < n_spans; s += gridDim.x) {
        const int64_t piece = s / rows, row = s - piece * rows;
        const int64_t first_vec = row * T4 + piece * CAP;
        const int64_t left = T4 - piece * CAP;
        const int n_vec = (int)(left < CAP ? left : CAP);
        float A[U], B[U];
#pragma unroll
        for (int j = 0; j < U; j++) {
            const int o = j * THREADS + tid;
            float4 a = make_float4(1.f, 1.f, 1.f, 1.f), x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (o < n_vec && SSB_INDEX_OK(first_vec + o, extent, 24)) {
                a = __ldcs(gate + first_vec + o);
                x = __ldcs(in1 + first_vec + o);
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
        if (warp == 0) {
            float tA = 1.f, tB = 0.f;
            if (lane < NE) {
                const float2 tt = s_tot[buf][lane];
                tA = tt.x;
                tB = tt.y;
            }
            if (!BWD) warp_scan_forward<float>(tA, tB, lane);
            else warp_scan_reverse<float>(tA, tB, lane);
            if (lane == (BWD ? 0 : NE - 1)) maps[row * pieces + piece] = make_float2(tA, tB);
        }
        buf ^= 1;
    }
}

// One warp per row: folds the row's `pieces` span maps into the row's map (A, B).
template <bool BWD>
__global__ void fold_maps_kernel(const float2 *__restrict__ maps, int64_t rows, int64_t pieces,
                                 float *__restrict__ agg) {
    const int lane = threadIdx.x & 31;
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= rows) return;
    float rA = 1.f, rB = 0.f;
    const float2 *m = maps + row * pieces;
    for (int64_t base = 0; base < pieces; base += 32) {
        // forward: pieces left to right; backward: right to left (the rightmost applies first)
        const int64_t i = base + lane;
        const int64_t idx = BWD ? pieces - 1 - i : i;
        float A = 1.f, B = 0.f;
        if (i < pieces) {
            const float2 v = m[idx];
            A = v.x;
            B = v.y;
        }
        warp_scan_forward<float>(A, B, lane);  // lane 31: window composed in processing order
        const float wA = __shfl_sync(kFullMask, A, 31), wB = __shfl_sync(kFullMask, B, 31);
        rB = fmaf(wA, rB, wB);  // the window applies after what was folded so far
        rA *= wA;
    }
    if (lane == 0) {
        agg[2 * row] = rA;
        agg[2 * row + 1] = rB;
    }
}

// Two-pass form for a few very long rows: every row is cut into K chunks that are scanned as rows
// of their own.  Given the chunks' maps ([rows*K][2], forward or reverse recurrence) this kernel
// writes the state entering every chunk (carry [rows*K]); the caller's per-row carry0 (may be NULL)
// enters the first chunk processed.  One warp per row walks the maps 32 at a time, the next 32
// already in flight while the current ones are composed.
template <bool BWD, typename real>
__global__ void chunk_carry_kernel(const real *__restrict__ maps, int64_t rows, int64_t K,
                                   const real *__restrict__ carry0, real *__restrict__ carry) {
    const int lane = threadIdx.x & 31;
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= rows) return;
    real run = carry0 != nullptr ? carry0[row] : real(0);
    real nA, nB;
    auto fetch = [&](int64_t base) {
        const int64_t i = base + lane;  // position in processing order; chunk index is K-1-i backward
        nA = real(1);
        nB = real(0);
        if (i < K) {
            const real *m = maps + 2 * (row * K + (BWD ? K - 1 - i : i));
            nA = m[0];
            nB = m[1];
        }
    };
    fetch(0);
    for (int64_t base = 0; base < K; base += 32) {
        real A = nA, B = nB;
        fetch(base + 32);
        warp_scan_forward<real>(A, B, lane);
        real eA = __shfl_up_sync(kFullMask, A, 1), eB = __shfl_up_sync(kFullMask, B, 1);
        if (lane == 0) { eA = real(1); eB = real(0); }
        const int64_t i = base + lane;
        if (i < K) carry[row * K + (BWD ? K - 1 - i : i)] = fma_<real>(eA, run, eB);
        run = fma_<real>(__shfl_sync(kFullMask, A, 31), run, __shfl_sync(kFullMask, B, 31));
    }
}

// h just before each chunk of the [rows*K, chunk_len] view (the backward's h_prev): the element
// preceding the chunk in memory, or the caller's h_prev0 / 0 at a row start.  One thread per chunk.
template <typename real>
__global__ void chunk_h_prev_kernel(const real *__restrict__ h, int64_t rows, int64_t K, int64_t chunk_len,
                                    const real *__restrict__ h_prev0, real *__restrict__ h_prev_view) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= rows * K) return;
    h_prev_view[v] = ((v % K) > 0 && SSB_INDEX_OK(v * chunk_len - 1, rows * K * chunk_len, 25))
                         ? h[v * chunk_len - 1]
                         : (h_prev0 != nullptr && (v % K) == 0 ? h_prev0[v / K] : real(0));
}

}  // namespace lookback
}  // namespace ssb
