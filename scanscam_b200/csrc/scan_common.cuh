// Shared device helpers for the gated-linear-scan kernels (sm_100a).
//
// The scan h_t = a_t*h_{t-1} + b_t is a fold of affine maps x -> a*x + b.  Maps compose
// associatively: applying (a1,b1) and then (a2,b2) is (a2*a1, a2*b1 + b2).  Every kernel
// here composes such pairs and never divides by a gate or goes through logarithms, so
// exact-zero gates ("resets") and gates with |a| > 1 are handled like any other value.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ssb {

constexpr unsigned kFullMask = 0xffffffffu;

// Device-side status word: [0] = ssb_status_t code (0 = ok), [1] = kernel-specific detail.
// Written by a kernel whose bounded wait gives up; read and cleared by ssb_device_status().
__device__ int g_status_word[2];

__device__ __forceinline__ void report_device_wait(int detail) {
    if (atomicCAS(&g_status_word[0], 0, 4 /* SSB_ERR_DEVICE_WAIT */) == 0) {
        g_status_word[1] = detail;
    }
}

// Checked build (-DSSB_CHECKED, `python -m scanscam_b200.build --checked`): every kernel that computes
// its own global addresses tests each index against the tensor's extent before the access.  An
// index outside [0, extent) is never dereferenced: the access is skipped (a load yields the
// identity element the kernel uses for padding), the status word is set to SSB_ERR_DEVICE_CHECK
// with the site's code, and the kernel runs on to its normal end -- no trap, no assert, the
// context stays usable.  The kernels that move data with bulk tensor copies need no such test:
// the copy engine clips every box against the extents in the tensor map.  In the ordinary build
// the test is the constant `true`.
__device__ __forceinline__ void report_device_check(int site) {
    if (atomicCAS(&g_status_word[0], 0, 7 /* SSB_ERR_DEVICE_CHECK */) == 0) {
        g_status_word[1] = site;
    }
}
#ifdef SSB_CHECKED
__device__ __forceinline__ bool index_in_range(int64_t index, int64_t extent, int site) {
    if (index >= 0 && index < extent) return true;
    report_device_check(site);
    return false;
}
#define SSB_INDEX_OK(index, extent, site) ::ssb::index_in_range((int64_t)(index), (int64_t)(extent), (site))
// Submits one index to the test without touching memory (the self-test of the reporting path).
__global__ void index_check_probe_kernel(int64_t index, int64_t extent) { (void)SSB_INDEX_OK(index, extent, 99); }
#else
#define SSB_INDEX_OK(index, extent, site) true
#endif

// A naturally aligned pack of VEC scalars; loads/stores of a 16-byte pack compile to one
// 128-bit memory instruction.
template <typename real, int VEC>
struct alignas(sizeof(real) * VEC) Pack {
    real v[VEC];
};

// Streaming (evict-first) global loads and stores: every byte is touched exactly once.
template <typename real, int VEC>
__device__ __forceinline__ Pack<real, VEC> load_stream(const real *p) {
    Pack<real, VEC> r;
    if constexpr (sizeof(real) * VEC == 16 && sizeof(real) == 4) {
        float4 t = __ldcs(reinterpret_cast<const float4 *>(p));
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else if constexpr (sizeof(real) * VEC == 16 && sizeof(real) == 8) {
        double2 t = __ldcs(reinterpret_cast<const double2 *>(p));
        r.v[0] = t.x; r.v[1] = t.y;
    } else {
        static_assert(VEC == 1, "unsupported pack width");
        r.v[0] = __ldcs(p);
    }
    return r;
}

template <typename real, int VEC>
__device__ __forceinline__ void store_stream(real *p, const Pack<real, VEC> &r) {
    if constexpr (sizeof(real) * VEC == 16 && sizeof(real) == 4) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(r.v[0], r.v[1], r.v[2], r.v[3]));
    } else if constexpr (sizeof(real) * VEC == 16 && sizeof(real) == 8) {
        __stcs(reinterpret_cast<double2 *>(p), make_double2(r.v[0], r.v[1]));
    } else {
        static_assert(VEC == 1, "unsupported pack width");
        __stcs(p, r.v[0]);
    }
}

// ---- programmatic dependent launch ----------------------------------------------------------
// A kernel launched with the attribute cudaLaunchAttributeProgrammaticStreamSerialization may
// start while the kernel before it in the stream is still running, once every CTA of that kernel
// has executed the trigger (or exited); the wait returns when the earlier kernel has completed
// and its writes are visible -- at once when the launch carried no such dependency.  A kernel that
// waits before its first access to global memory is therefore ordered exactly like an ordinary
// launch; what overlaps is its launch, its block scheduling and whatever set-up precedes the wait.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- 16-bit storage types (bf16 / fp16 in memory, fp32 arithmetic) -------------------------
// Two packed 16-bit values <-> two floats.  `lo` is the element at the lower address.
template <typename io_t>
__device__ __forceinline__ void unpack2(uint32_t w, float &lo, float &hi);
template <>
__device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t w, float &lo, float &hi) {
    lo = __uint_as_float(w << 16);  // a bf16 is the upper half of the fp32 with the same value
    hi = __uint_as_float(w & 0xffff0000u);
}
template <>
__device__ __forceinline__ void unpack2<__half>(uint32_t w, float &lo, float &hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w));
    lo = f.x;
    hi = f.y;
}
template <typename io_t>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);  // round to nearest even
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}
// One stored element as the arithmetic type (`real` itself, or a 16-bit type widened to float).
template <typename real, typename io_t>
__device__ __forceinline__ real widen(io_t x) {
    if constexpr (sizeof(io_t) == sizeof(real)) return x;
    else if constexpr (sizeof(io_t) == 2 && sizeof(real) == 4) { float lo, hi; unpack2<io_t>((uint32_t)*reinterpret_cast<const uint16_t *>(&x), lo, hi); return lo; }
}

// Loads VEC elements stored as io_t into a pack of `real`; io_t == real is the plain load above.
// For a 16-bit io_t, VEC is 1 (scalar) or 8 (one 16-byte load).
template <typename real, typename io_t, int VEC>
__device__ __forceinline__ Pack<real, VEC> load_stream_io(const io_t *p) {
    if constexpr (sizeof(io_t) == sizeof(real)) {
        return load_stream<real, VEC>(reinterpret_cast<const real *>(p));
    } else {
        static_assert(sizeof(io_t) == 2 && sizeof(real) == 4 && (VEC == 1 || VEC == 8), "16-bit storage, fp32 arithmetic");
        Pack<real, VEC> r;
        if constexpr (VEC == 1) {
            r.v[0] = widen<real, io_t>(*p);
        } else {
            const uint4 t = __ldcs(reinterpret_cast<const uint4 *>(p));
            unpack2<io_t>(t.x, r.v[0], r.v[1]);
            unpack2<io_t>(t.y, r.v[2], r.v[3]);
            unpack2<io_t>(t.z, r.v[4], r.v[5]);
            unpack2<io_t>(t.w, r.v[6], r.v[7]);
        }
        return r;
    }
}

template <typename real, typename io_t, int VEC>
__device__ __forceinline__ void store_stream_io(io_t *p, const Pack<real, VEC> &r) {
    if constexpr (sizeof(io_t) == sizeof(real)) {
        store_stream<real, VEC>(reinterpret_cast<real *>(p), r);
    } else {
        static_assert(sizeof(io_t) == 2 && sizeof(real) == 4 && (VEC == 1 || VEC == 8), "16-bit storage, fp32 arithmetic");
        if constexpr (VEC == 1) {
            *p = static_cast<io_t>(r.v[0]);
        } else {
            uint4 t;
            t.x = pack2<io_t>(r.v[0], r.v[1]);
            t.y = pack2<io_t>(r.v[2], r.v[3]);
            t.z = pack2<io_t>(r.v[4], r.v[5]);
            t.w = pack2<io_t>(r.v[6], r.v[7]);
            __stcs(reinterpret_cast<uint4 *>(p), t);
        }
    }
}

template <typename real>
__device__ __forceinline__ real fma_(real a, real b, real c);
template <>
__device__ __forceinline__ float fma_<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <>
__device__ __forceinline__ double fma_<double>(double a, double b, double c) { return fma(a, b, c); }

// Inclusive scan of affine maps across the lanes of a warp, left to right: afterwards lane l
// holds the composition of the maps of lanes 0..l (lane 0's applied first).
template <typename real>
__device__ __forceinline__ void warp_scan_forward(real &A, real &B, int lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        real Ap = __shfl_up_sync(kFullMask, A, d);
        real Bp = __shfl_up_sync(kFullMask, B, d);
        if (lane >= d) {
            B = fma_<real>(A, Bp, B);
            A *= Ap;
        }
    }
}

// Same, right to left: lane l ends with the composition of lanes 31..l (lane 31's first).
template <typename real>
__device__ __forceinline__ void warp_scan_reverse(real &A, real &B, int lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        real Ap = __shfl_down_sync(kFullMask, A, d);
        real Bp = __shfl_down_sync(kFullMask, B, d);
        if (lane + d < 32) {
            B = fma_<real>(A, Bp, B);
            A *= Ap;
        }
    }
}

}  // namespace ssb
