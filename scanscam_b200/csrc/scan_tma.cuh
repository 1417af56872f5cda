// TMA-staged kernels for the aligned fp32 rows layout (T % 32 == 0, 16-byte aligned base).
//
// Data movement is done by the tensor memory accelerator, not by the threads:
//   * each [rows, T] tensor is described to the TMA as a 3-D array [rows][T/32][32 floats],
//     so a box of {32, L, 1} is L consecutive 128-byte lines of one row;
//   * every warp owns a private ring of STAGES shared-memory slots; one lane arms the slot's
//     mbarrier with the byte count and issues one `cp.async.bulk.tensor.3d` per input tensor,
//     up to STAGES chunks ahead of the arithmetic, so the bytes in flight per SM are set by
//     the ring depth and not by occupancy or registers;
//   * tiles land in shared memory with the 128-byte swizzle, under which "lane l reads its
//     own 16 (or 32) consecutive floats as float4s" is bank-conflict free;
//   * results are written back to a swizzled staging slot and leave through a bulk tensor
//     store, so the threads never issue a global memory instruction in the steady state.
// A warp walks its rows chunk by chunk with the row's carry in a register; chunks of one row
// are chained by a single FMA, rows are independent, and warps never synchronise with each
// other.  Every mbarrier wait is bounded (about one second); a wait that runs out sets the
// device status word and the warp drains and leaves.
//
// Same math and same entry points as the warp kernels; this is the fast path for the shapes
// the reference serves with its vectorised kernel (src/scanscam_cuda.cu:195-258,271-283) and
// its backward kernel (:366-425).
#pragma once

#include <cuda.h>

#include "scan_common.cuh"

namespace ssb {
namespace tma {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: gives up after about one second of wall time.
__device__ __forceinline__ bool mbar_wait_lane(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t_start = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++) {
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (global_ns() - t_start > 1000000000ull) return false;
    }
}

// Warp-wide bounded wait (all 32 lanes call it); the outcome is the same in every lane, so
// the callers' control flow stays convergent even when a wait gives up.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    return __all_sync(kFullMask, mbar_wait_lane(bar, parity)) != 0;
}

// Box load global -> shared (this CTA's own shared memory), completion counted on `bar`.
__device__ __forceinline__ void load_box(uint32_t dst, const CUtensorMap *map, int c0, int c1,
                                         int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}

// Box store shared -> global, tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void store_box(const CUtensorMap *map, int c0, int c1, int c2,
                                          uint32_t src) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::
                     "l"(map),
                 "r"(c0), "r"(c1), "r"(c2), "r"(src)
                 : "memory");
}

__device__ __forceinline__ void store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Orders this thread's shared-memory writes before later reads by the async (TMA) proxy.
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ float4 lds128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(addr));
    return v;
}

__device__ __forceinline__ void sts128(uint32_t addr, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y),
                 "f"(v.z), "f"(v.w)
                 : "memory");
}

__device__ __forceinline__ float lds32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

// Byte offset, inside a 1024-byte aligned tile, of the float4 that holds elements
// [e, e+4) (e % 4 == 0) under the 128-byte swizzle: the 16-byte chunk index within a
// 128-byte line is XORed with the line index modulo 8.
__device__ __forceinline__ uint32_t swizzled_offset(int e) {
    const int line = e >> 5;
    const int chunk = (e >> 2) & 7;
    return (uint32_t)((line << 7) | ((chunk ^ (line & 7)) << 4));
}

// Shared-memory bytes one warp needs.
template <int EPL, int STAGES, int N_IN, int N_OUT>
__host__ __device__ constexpr int warp_smem_bytes() {
    return (STAGES * N_IN + 2 * N_OUT) * (32 * EPL * 4);
}

// ---------------------------------------------------------------------------------------
// Forward.  EPL = elements per lane per chunk (16 or 32); a chunk is 32*EPL elements of a row.
// ---------------------------------------------------------------------------------------
template <int EPL, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1)
tma_rows_fwd_kernel(const __grid_constant__ CUtensorMap map_gate,
                    const __grid_constant__ CUtensorMap map_value,
                    const __grid_constant__ CUtensorMap map_out, int64_t rows, int64_t T,
                    const float *__restrict__ h_in) {
    constexpr int CH = 32 * EPL;
    constexpr int TILE = CH * 4;
    constexpr int LINES = CH / 32;
    constexpr int NV = EPL / 4;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[WARPS][STAGES];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t base = ((smem_u32(smem_raw) + 1023u) & ~1023u) +
                          (uint32_t)warp * warp_smem_bytes<EPL, STAGES, 2, 1>();
    const uint32_t out_base = base + STAGES * 2 * TILE;
    const uint32_t bar0 = smem_u32(&full_bar[warp][0]);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) mbar_init(bar0 + 8 * s, 1);
        fence_mbar_init();
    }
    __syncwarp();

    const int64_t n_warps = (int64_t)gridDim.x * WARPS;
    const int64_t first_row = (int64_t)warp * gridDim.x + blockIdx.x;
    const int cpr = (int)((T + CH - 1) / CH);  // chunks per row
    const int64_t my_rows = first_row < rows ? (rows - first_row + n_warps - 1) / n_warps : 0;
    const int64_t n_items = my_rows * cpr;

    uint32_t off[NV];
#pragma unroll
    for (int j = 0; j < NV; j++) off[j] = swizzled_offset(lane * EPL + 4 * j);

    // producer cursor (lane 0 only issues)
    int64_t p_item = 0, p_row = first_row;
    int p_chunk = 0;
    int p_stage = 0;
    auto issue = [&]() {
        const int s = p_stage;
        if (lane == 0) {
            const uint32_t bar = bar0 + 8 * s;
            mbar_expect_tx(bar, 2 * TILE);
            load_box(base + (2 * s) * TILE, &map_gate, 0, p_chunk * LINES, (int)p_row, bar);
            load_box(base + (2 * s + 1) * TILE, &map_value, 0, p_chunk * LINES, (int)p_row, bar);
        }
        p_item++;
        if (++p_stage == STAGES) p_stage = 0;
        if (++p_chunk == cpr) { p_chunk = 0; p_row += n_warps; }
    };
    for (int s = 0; s < STAGES && p_item < n_items; s++) issue();

    int64_t row = first_row;
    int chunk = 0;
    float carry = 0.f;
    bool ok = true;
    int64_t item = 0;
    int s = 0;
    uint32_t parity = 0;
    for (; item < n_items; item++) {
        if (chunk == 0) carry = h_in != nullptr ? h_in[row] : 0.f;
        if (!mbar_wait_bounded(bar0 + 8 * s, parity)) { ok = false; break; }
        float a[EPL], b[EPL];
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const float4 va = lds128(base + (2 * s) * TILE + off[j]);
            const float4 vb = lds128(base + (2 * s + 1) * TILE + off[j]);
            a[4 * j] = va.x; a[4 * j + 1] = va.y; a[4 * j + 2] = va.z; a[4 * j + 3] = va.w;
            b[4 * j] = vb.x; b[4 * j + 1] = vb.y; b[4 * j + 2] = vb.z; b[4 * j + 3] = vb.w;
        }
        __syncwarp();  // every lane has read the slot: it can be refilled
        if (p_item < n_items) issue();

        float A = a[0], B = b[0];
#pragma unroll
        for (int k = 1; k < EPL; k++) {
            B = fmaf(a[k], B, b[k]);
            A *= a[k];
        }
        warp_scan_forward<float>(A, B, lane);
        float Ae = __shfl_up_sync(kFullMask, A, 1);
        float Be = __shfl_up_sync(kFullMask, B, 1);
        if (lane == 0) { Ae = 1.f; Be = 0.f; }
        const float At = __shfl_sync(kFullMask, A, 31);
        const float Bt = __shfl_sync(kFullMask, B, 31);
        float h = fmaf(Ae, carry, Be);
        carry = fmaf(At, carry, Bt);

        // The staging slot used two chunks ago must have been read by its store.
        const uint32_t ob = out_base + (uint32_t)(item & 1) * TILE;
        if (lane == 0) store_wait_read<1>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < NV; j++) {
            float4 o;
            h = fmaf(a[4 * j], h, b[4 * j]); o.x = h;
            h = fmaf(a[4 * j + 1], h, b[4 * j + 1]); o.y = h;
            h = fmaf(a[4 * j + 2], h, b[4 * j + 2]); o.z = h;
            h = fmaf(a[4 * j + 3], h, b[4 * j + 3]); o.w = h;
            sts128(ob + off[j], o);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
            store_box(&map_out, 0, chunk * LINES, (int)row, ob);
            store_commit();
        }
        if (++chunk == cpr) { chunk = 0; row += n_warps; }
        if (++s == STAGES) { s = 0; parity ^= 1u; }
    }
    if (!ok) {
        if (lane == 0) report_device_wait(1);
        // Drain: loads still in flight target this CTA's shared memory.
        for (int64_t it = item; it < p_item; it++) {
            (void)mbar_wait_bounded(bar0 + 8 * (int)(it % STAGES), (uint32_t)((it / STAGES) & 1));
        }
    }
    if (lane == 0) store_wait_read<0>();
    __syncwarp();
}

// ---------------------------------------------------------------------------------------
// Fused backward: reads gate, h, gout once, writes grad_gate and grad_value.
// Chunks of a row are visited right to left.  h_{t-1} for a lane's first element comes from
// the lane to its left; for lane 0 it is the last element of the chunk to the left, which is
// the next item of the ring and therefore already in flight.
// ---------------------------------------------------------------------------------------
template <int EPL, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1)
tma_rows_bwd_kernel(const __grid_constant__ CUtensorMap map_gate,
                    const __grid_constant__ CUtensorMap map_h,
                    const __grid_constant__ CUtensorMap map_gout,
                    const __grid_constant__ CUtensorMap map_ggate,
                    const __grid_constant__ CUtensorMap map_gvalue, int64_t rows, int64_t T,
                    const float *__restrict__ c_in, const float *__restrict__ h_prev) {
    constexpr int CH = 32 * EPL;
    constexpr int TILE = CH * 4;
    constexpr int LINES = CH / 32;
    constexpr int NV = EPL / 4;
    static_assert(STAGES >= 2, "the h halo is read from the next ring slot");
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[WARPS][STAGES];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t base = ((smem_u32(smem_raw) + 1023u) & ~1023u) +
                          (uint32_t)warp * warp_smem_bytes<EPL, STAGES, 3, 2>();
    const uint32_t out_base = base + STAGES * 3 * TILE;
    const uint32_t bar0 = smem_u32(&full_bar[warp][0]);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) mbar_init(bar0 + 8 * s, 1);
        fence_mbar_init();
    }
    __syncwarp();

    const int64_t n_warps = (int64_t)gridDim.x * WARPS;
    const int64_t first_row = (int64_t)warp * gridDim.x + blockIdx.x;
    const int cpr = (int)((T + CH - 1) / CH);
    const int64_t my_rows = first_row < rows ? (rows - first_row + n_warps - 1) / n_warps : 0;
    const int64_t n_items = my_rows * cpr;

    uint32_t off[NV];
#pragma unroll
    for (int j = 0; j < NV; j++) off[j] = swizzled_offset(lane * EPL + 4 * j);
    const uint32_t last_off = swizzled_offset(CH - 4) + 12;  // element CH-1 of a tile

    int64_t p_item = 0, p_row = first_row;
    int p_chunk = cpr - 1;
    int p_stage = 0;
    auto issue = [&]() {
        const int s = p_stage;
        if (lane == 0) {
            const uint32_t bar = bar0 + 8 * s;
            mbar_expect_tx(bar, 3 * TILE);
            load_box(base + (3 * s) * TILE, &map_gate, 0, p_chunk * LINES, (int)p_row, bar);
            load_box(base + (3 * s + 1) * TILE, &map_h, 0, p_chunk * LINES, (int)p_row, bar);
            load_box(base + (3 * s + 2) * TILE, &map_gout, 0, p_chunk * LINES, (int)p_row, bar);
        }
        p_item++;
        if (++p_stage == STAGES) p_stage = 0;
        if (--p_chunk < 0) { p_chunk = cpr - 1; p_row += n_warps; }
    };
    for (int s = 0; s < STAGES && p_item < n_items; s++) issue();

    int64_t row = first_row;
    int chunk = cpr - 1;
    float carry = 0.f;
    bool ok = true;
    int64_t item = 0;
    int s = 0;
    uint32_t parity = 0;
    for (; item < n_items; item++) {
        if (chunk == cpr - 1) carry = c_in != nullptr ? c_in[row] : 0.f;
        if (!mbar_wait_bounded(bar0 + 8 * s, parity)) { ok = false; break; }
        float a[EPL], g[EPL], h[EPL];
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const float4 va = lds128(base + (3 * s) * TILE + off[j]);
            const float4 vh = lds128(base + (3 * s + 1) * TILE + off[j]);
            const float4 vg = lds128(base + (3 * s + 2) * TILE + off[j]);
            a[4 * j] = va.x; a[4 * j + 1] = va.y; a[4 * j + 2] = va.z; a[4 * j + 3] = va.w;
            h[4 * j] = vh.x; h[4 * j + 1] = vh.y; h[4 * j + 2] = vh.z; h[4 * j + 3] = vh.w;
            g[4 * j] = vg.x; g[4 * j + 1] = vg.y; g[4 * j + 2] = vg.z; g[4 * j + 3] = vg.w;
        }
        // Beyond the end of the row the TMA filled zeros; the reverse fold needs the identity
        // map there (gate 1, gradient 0) so that an incoming carry passes through.
        if (chunk == cpr - 1 && (int64_t)cpr * CH != T) {
            const int valid = (int)(T - (int64_t)chunk * CH) - lane * EPL;
#pragma unroll
            for (int k = 0; k < EPL; k++) {
                if (k >= valid) { a[k] = 1.f; g[k] = 0.f; }
            }
        }
        // h just left of the chunk: last element of the next item's h tile (same row).
        float edge = 0.f;
        if (chunk > 0) {
            const int s1 = (s + 1 == STAGES) ? 0 : s + 1;
            if (!mbar_wait_bounded(bar0 + 8 * s1, (s + 1 == STAGES) ? (parity ^ 1u) : parity)) {
                ok = false;
                break;
            }
            edge = lds32(base + (3 * s1 + 1) * TILE + last_off);
        } else if (h_prev != nullptr) {
            edge = h_prev[row];
        }
        __syncwarp();
        if (p_item < n_items) issue();

        float A = 1.f, D = 0.f;
#pragma unroll
        for (int k = EPL - 1; k >= 0; k--) {
            D = a[k] * (g[k] + D);
            A *= a[k];
        }
        warp_scan_reverse<float>(A, D, lane);
        float Ae = __shfl_down_sync(kFullMask, A, 1);
        float De = __shfl_down_sync(kFullMask, D, 1);
        if (lane == 31) { Ae = 1.f; De = 0.f; }
        const float At = __shfl_sync(kFullMask, A, 0);
        const float Dt = __shfl_sync(kFullMask, D, 0);
        float left = __shfl_up_sync(kFullMask, h[EPL - 1], 1);
        if (lane == 0) left = edge;
        float c = fmaf(Ae, carry, De);
        carry = fmaf(At, carry, Dt);

        const uint32_t ob = out_base + (uint32_t)(item & 1) * (2 * TILE);
        if (lane == 0) store_wait_read<1>();
        __syncwarp();
#pragma unroll
        for (int j = NV - 1; j >= 0; j--) {
            float4 oa, og;
            float gb;
            gb = g[4 * j + 3] + c; c = a[4 * j + 3] * gb; og.w = gb; oa.w = gb * h[4 * j + 2];
            gb = g[4 * j + 2] + c; c = a[4 * j + 2] * gb; og.z = gb; oa.z = gb * h[4 * j + 1];
            gb = g[4 * j + 1] + c; c = a[4 * j + 1] * gb; og.y = gb; oa.y = gb * h[4 * j];
            gb = g[4 * j] + c; c = a[4 * j] * gb; og.x = gb;
            oa.x = gb * (j > 0 ? h[j > 0 ? 4 * j - 1 : 0] : left);
            sts128(ob + off[j], oa);
            sts128(ob + TILE + off[j], og);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
            store_box(&map_ggate, 0, chunk * LINES, (int)row, ob);
            store_box(&map_gvalue, 0, chunk * LINES, (int)row, ob + TILE);
            store_commit();
        }
        if (--chunk < 0) { chunk = cpr - 1; row += n_warps; }
        if (++s == STAGES) { s = 0; parity ^= 1u; }
    }
    if (!ok) {
        if (lane == 0) report_device_wait(2);
        for (int64_t it = item; it < p_item; it++) {
            (void)mbar_wait_bounded(bar0 + 8 * (int)(it % STAGES), (uint32_t)((it / STAGES) & 1));
        }
    }
    if (lane == 0) store_wait_read<0>();
    __syncwarp();
}

}  // namespace tma
}  // namespace ssb
