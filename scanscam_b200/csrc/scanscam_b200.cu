// C-ABI launch layer (see include/scanscam_b200.h).  One translation unit: the kernels are
// header templates instantiated here.  No torch, no allocation, no synchronisation except in
// ssb_device_status().
#include "../../include/scanscam_b200.h"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <limits>
#include <type_traits>

#include "scan_cl.cuh"
#include "scan_cl_lookback.cuh"
#include "scan_cl_narrow.cuh"
#include "scan_cl_stream.cuh"
#include "scan_cl_tma.cuh"
#include "scan_common.cuh"
#include "scan_flat.cuh"
#include "scan_flat_any.cuh"
#include "scan_lookback.cuh"
#include "scan_shard.cuh"
#include "scan_tma.cuh"
#include "scan_tma_flat.cuh"
#include "scan_warp.cuh"

namespace {

thread_local char t_last_error[512] = "";

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_last_error, sizeof(t_last_error), fmt, ap);
    va_end(ap);
    return status;
}

int check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        return fail(SSB_ERR_LAUNCH, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
    }
    return SSB_OK;
}

bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Validates a [rows, T] problem; *n receives rows*T.
int check_shape(int64_t rows, int64_t T, int64_t *n) {
    if (rows < 0 || T < 0) return fail(SSB_ERR_BAD_ARG, "negative size: rows=%lld T=%lld", (long long)rows, (long long)T);
    if (T > 0 && rows > std::numeric_limits<int64_t>::max() / 8 / T)
        return fail(SSB_ERR_BAD_ARG, "rows*T overflows: rows=%lld T=%lld", (long long)rows, (long long)T);
    *n = rows * T;
    return SSB_OK;
}

int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int v = cached[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

// ------------------------------------------------------------------------------------
// Warp-per-row family
// ------------------------------------------------------------------------------------
template <typename real>
constexpr int vec_width() { return 16 / (int)sizeof(real); }

int warp_grid(int64_t rows) {
    const int64_t want = (rows + ssb::kWarpKernelWarps - 1) / ssb::kWarpKernelWarps;
    const int64_t cap = (int64_t)sm_count() * 8;  // 8 CTAs of 8 warps fill an SM
    return (int)(want < cap ? want : cap);
}

template <typename real, bool REDUCE>
int launch_warp_fwd(const real *gate, const real *value, real *out, int64_t rows, int64_t T,
                    const real *h_in, real *agg, cudaStream_t st) {
    constexpr int V = vec_width<real>();
    const bool vec = (T % V == 0) && aligned_to(gate, 16) && aligned_to(value, 16) &&
                     (REDUCE || aligned_to(out, 16));
    const int grid = warp_grid(rows);
    const int block = ssb::kWarpKernelWarps * 32;
    if (vec) {
        ssb::warp_rows_fwd_kernel<real, V, 4, REDUCE><<<grid, block, 0, st>>>(gate, value, out, rows, T, h_in, agg);
    } else {
        ssb::warp_rows_fwd_kernel<real, 1, 4, REDUCE><<<grid, block, 0, st>>>(gate, value, out, rows, T, h_in, agg);
    }
    return check_launch("warp_rows_fwd_kernel");
}

template <typename real, bool REDUCE>
int launch_warp_bwd(const real *gate, const real *h, const real *gout, real *ggate, real *gvalue,
                    int64_t rows, int64_t T, const real *c_in, const real *h_prev, real *agg,
                    cudaStream_t st) {
    constexpr int V = vec_width<real>();
    const bool vec = (T % V == 0) && aligned_to(gate, 16) && aligned_to(gout, 16) &&
                     (REDUCE || (aligned_to(h, 16) && aligned_to(ggate, 16) && aligned_to(gvalue, 16)));
    const int grid = warp_grid(rows);
    const int block = ssb::kWarpKernelWarps * 32;
    if (vec) {
        ssb::warp_rows_bwd_kernel<real, V, 4, REDUCE><<<grid, block, 0, st>>>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, agg);
    } else {
        ssb::warp_rows_bwd_kernel<real, 1, 4, REDUCE><<<grid, block, 0, st>>>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, agg);
    }
    return check_launch("warp_rows_bwd_kernel");
}

// ------------------------------------------------------------------------------------
// TMA family
// ------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static std::atomic<void *> cached{nullptr};
    void *p = cached.load(std::memory_order_acquire);
    if (p == nullptr) {
        cudaDriverEntryPointQueryResult q;
        void *fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        cached.store(fn, std::memory_order_release);
        p = fn;
    }
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
}

// cuTensorMapEncodeTiled is a driver call and wants a context current on the calling thread.  A
// thread that has made no runtime call yet (an autograd worker reaching a launch function whose
// lookups are all cached) has none: bind the device's primary context and encode again.
template <typename... Args>
CUresult encode_tiled(PFN_cuTensorMapEncodeTiled_v12000 enc, Args... args) {
    CUresult r = enc(args...);
    if (r == CUDA_ERROR_INVALID_CONTEXT || r == CUDA_ERROR_NOT_INITIALIZED) {
        if (cudaFree(nullptr) != cudaSuccess) (void)cudaGetLastError();
        r = enc(args...);
    }
    return r;
}

bool tma_eligible(int64_t rows, int64_t T) {
    return T % 32 == 0 && T >= 32 && rows <= 0x7fffffffLL && T / 32 <= 0x7fffffffLL;
}

// Describes a dense fp32 [rows, T] matrix as [rows][T/32][32] with boxes of `lines` 128-byte
// lines of one row, 128-byte swizzle, zero fill outside.
int make_rows_map(CUtensorMap *map, const float *ptr, int64_t rows, int64_t T, int lines) {
    PFN_cuTensorMapEncodeTiled_v12000 enc = encode_fn();
    if (enc == nullptr) return fail(SSB_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {32, (cuuint64_t)(T / 32), (cuuint64_t)rows};
    cuuint64_t strides[2] = {128, (cuuint64_t)T * 4};
    cuuint32_t box[3] = {32, (cuuint32_t)lines, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_tiled(enc, map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(ptr), dims, strides, box,
                     estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SSB_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return SSB_OK;
}

template <int EPL, int STAGES, int WARPS>
int launch_tma_fwd(const float *gate, const float *value, float *out, int64_t rows, int64_t T,
                   const float *h_in, cudaStream_t st) {
    CUtensorMap mg, mv, mo;
    int rc;
    if ((rc = make_rows_map(&mg, gate, rows, T, EPL)) != SSB_OK) return rc;
    if ((rc = make_rows_map(&mv, value, rows, T, EPL)) != SSB_OK) return rc;
    if ((rc = make_rows_map(&mo, out, rows, T, EPL)) != SSB_OK) return rc;
    auto kern = ssb::tma::tma_rows_fwd_kernel<EPL, STAGES, WARPS>;
    const int smem = WARPS * ssb::tma::warp_smem_bytes<EPL, STAGES, 2, 1>() + 1024;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(tma_rows_fwd_kernel)");
    const int64_t want = (rows + WARPS - 1) / WARPS;
    const int grid = (int)(want < sm_count() ? want : sm_count());
    kern<<<grid, WARPS * 32, smem, st>>>(mg, mv, mo, rows, T, h_in);
    return check_launch("tma_rows_fwd_kernel");
}

template <int EPL, int STAGES, int WARPS>
int launch_tma_bwd(const float *gate, const float *h, const float *gout, float *ggate, float *gvalue,
                   int64_t rows, int64_t T, const float *c_in, const float *h_prev, cudaStream_t st) {
    CUtensorMap ma, mh, mg, mga, mgb;
    int rc;
    if ((rc = make_rows_map(&ma, gate, rows, T, EPL)) != SSB_OK) return rc;
    if ((rc = make_rows_map(&mh, h, rows, T, EPL)) != SSB_OK) return rc;
    if ((rc = make_rows_map(&mg, gout, rows, T, EPL)) != SSB_OK) return rc;
    if ((rc = make_rows_map(&mga, ggate, rows, T, EPL)) != SSB_OK) return rc;
    if ((rc = make_rows_map(&mgb, gvalue, rows, T, EPL)) != SSB_OK) return rc;
    auto kern = ssb::tma::tma_rows_bwd_kernel<EPL, STAGES, WARPS>;
    const int smem = WARPS * ssb::tma::warp_smem_bytes<EPL, STAGES, 3, 2>() + 1024;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(tma_rows_bwd_kernel)");
    const int64_t want = (rows + WARPS - 1) / WARPS;
    const int grid = (int)(want < sm_count() ? want : sm_count());
    kern<<<grid, WARPS * 32, smem, st>>>(ma, mh, mg, mga, mgb, rows, T, c_in, h_prev);
    return check_launch("tma_rows_bwd_kernel");
}

// ------------------------------------------------------------------------------------
// Flat streaming family
// ------------------------------------------------------------------------------------
bool flat_eligible(int64_t rows, int64_t T) {
    return T % 4 == 0 && T >= 4 && rows * (T / 4) < (int64_t)1 << 40;
}

// TAG makes one instantiation (and one cached occupancy) per kernel instantiation.
// Tuning override for the duration of one entry-point call: CTAs per SM (0 = as many as fit).
thread_local int t_grid_per_sm = 0;
struct GridScope {
    explicit GridScope(int per_sm) { t_grid_per_sm = per_sm; }
    ~GridScope() { t_grid_per_sm = 0; }
};

template <int TAG, typename K>
int persistent_grid(K kern, int threads, int64_t units) {
    static std::atomic<int> cached_occ{0};
    int occ = cached_occ.load(std::memory_order_relaxed);
    if (occ == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, threads, 0) != cudaSuccess || occ <= 0) {
            (void)cudaGetLastError();
            occ = 1;
        }
        cached_occ.store(occ, std::memory_order_relaxed);
    }
    const int per_sm = (t_grid_per_sm > 0 && t_grid_per_sm < occ) ? t_grid_per_sm : occ;
    const int64_t cap = (int64_t)sm_count() * per_sm;
    return (int)(units < cap ? (units > 0 ? units : 1) : cap);
}

// Launches `kern` as a programmatic dependent of the work ahead of it in `st`.  Only for kernels that
// execute griddepcontrol.wait before their first access to global memory: such a kernel is ordered
// like an ordinary launch, and its launch and set-up overlap the tail of the kernel ahead.  Used for
// the span sweep on bulk tensor copies (measured on B200, 2048 x 4096 forward + backward: 47.4 -> 43.3 us
// per step as stream launches, 42.8 -> 41.9 us inside a CUDA graph; no change on 16384 x 4096) and for
// the scan pass of the channels-last chunked form; NOT for the flat sweeps, whose thousands of small
// CTAs queue up behind the wait and cost more than the launch they hide (1024 x 1024: 9.3 -> 10.7 us
// per step), nor for the channels-last streaming kernels in general (-1 ... -12 %).
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kern)(KArgs...), int grid, int threads, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

int64_t flat_units(int64_t rows, int64_t T4, int cap) {
    if (T4 > cap) return rows;
    const int64_t rps = cap / T4;
    return (rows + rps - 1) / rps;
}

template <int THREADS, int U>
int launch_flat_fwd(const float *gate, const float *value, float *out, int64_t rows, int64_t T,
                    const float *h_in, cudaStream_t st) {
    auto kern = ssb::flat::flat_fwd_kernel<THREADS, U>;
    const int grid = persistent_grid<THREADS * 64 + U * 2>(kern, THREADS, flat_units(rows, T / 4, THREADS * U));
    kern<<<grid, THREADS, 0, st>>>(reinterpret_cast<const float4 *>(gate), reinterpret_cast<const float4 *>(value),
                                   reinterpret_cast<float4 *>(out), rows, T / 4, h_in);
    return check_launch("flat_fwd_kernel");
}

template <int THREADS, int U, int MIN_CTAS = 0>
int launch_flat_bwd(const float *gate, const float *h, const float *gout, float *ggate, float *gvalue,
                    int64_t rows, int64_t T, const float *c_in, const float *h_prev, cudaStream_t st) {
    auto kern = ssb::flat::flat_bwd_kernel<THREADS, U, MIN_CTAS>;
    const int grid = persistent_grid<THREADS * 64 + U * 2 + 1 + MIN_CTAS * 1000000>(kern, THREADS, flat_units(rows, T / 4, THREADS * U));
    kern<<<grid, THREADS, 0, st>>>(reinterpret_cast<const float4 *>(gate), reinterpret_cast<const float4 *>(h),
                                   reinterpret_cast<const float4 *>(gout), reinterpret_cast<float4 *>(ggate),
                                   reinterpret_cast<float4 *>(gvalue), rows, T / 4, c_in, h_prev);
    return check_launch("flat_bwd_kernel");
}

// Flat sweep with per-element row boundaries (any T).
bool flat_any_eligible(int64_t rows, int64_t T) { return T >= 1 && T <= 0x3ffffff0LL && rows * T < (int64_t)1 << 42; }

template <int THREADS, int U, bool BWD>
int launch_flat_any(const float *gate, const float *in1, const float *in2, float *out1, float *out2, int64_t rows,
                    int64_t T, const float *carry_a, const float *carry_b, cudaStream_t st) {
    const int64_t rpu = ssb::flat_any::rows_per_unit<THREADS * U>(T);
    const int64_t units = (rows + rpu - 1) / rpu;
    if constexpr (!BWD) {
        auto kern = ssb::flat_any::flat_any_fwd_kernel<THREADS, U>;
        const int grid = persistent_grid<400000 + THREADS * 64 + U * 2>(kern, THREADS, units);
        kern<<<grid, THREADS, 0, st>>>(gate, in1, out1, rows, T, carry_a);
    } else {
        auto kern = ssb::flat_any::flat_any_bwd_kernel<THREADS, U>;
        const int grid = persistent_grid<400000 + THREADS * 64 + U * 2 + 1>(kern, THREADS, units);
        kern<<<grid, THREADS, 0, st>>>(gate, in1, in2, out1, out2, rows, T, carry_a, carry_b);
    }
    return check_launch("flat_any_kernel");
}

// Tuning table of the flat family: id -> (threads per CTA, float4s per thread).
#define SSB_FLAT_CONFIGS(X) \
    X(0, 256, 4) X(1, 512, 2) X(2, 1024, 1) X(3, 256, 2) X(4, 128, 4) X(5, 512, 1) X(6, 128, 8) \
    X(7, 64, 16) X(8, 64, 8) X(9, 256, 1) X(10, 128, 2) X(11, 64, 4) X(12, 128, 1) X(13, 32, 16)

int dispatch_flat_fwd(int tuning, const float *gate, const float *value, float *out, int64_t rows,
                      int64_t T, const float *h_in, cudaStream_t st) {
    switch (tuning) {
#define X(ID, TH, UU) case ID: return launch_flat_fwd<TH, UU>(gate, value, out, rows, T, h_in, st);
        SSB_FLAT_CONFIGS(X)
#undef X
        default: return fail(SSB_ERR_UNSUPPORTED, "unknown forward flat tuning id %d", tuning);
    }
}

int dispatch_flat_bwd(int tuning, const float *gate, const float *h, const float *gout, float *ggate,
                      float *gvalue, int64_t rows, int64_t T, const float *c_in, const float *h_prev,
                      cudaStream_t st) {
    switch (tuning) {
#define X(ID, TH, UU) case ID: return launch_flat_bwd<TH, UU>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        SSB_FLAT_CONFIGS(X)
#undef X
        // the default span shape with the register budget capped so that 4 or 5 CTAs fit per SM
        case 14: return launch_flat_bwd<128, 8, 4>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 15: return launch_flat_bwd<128, 8, 5>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 16: return launch_flat_bwd<256, 4, 2>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        default: return fail(SSB_ERR_UNSUPPORTED, "unknown backward flat tuning id %d", tuning);
    }
}

// ------------------------------------------------------------------------------------
// Look-back family (long rows)
// ------------------------------------------------------------------------------------
// Tuning table: id -> (threads per CTA, float4s per thread); span capacity = product.
#define SSB_LOOKBACK_CONFIGS(X) X(0, 128, 8) X(1, 256, 4) X(2, 256, 2) X(3, 128, 4) X(4, 512, 2) X(5, 256, 1) X(6, 64, 16)

int lookback_cap(int tuning) {
    switch (tuning) {
#define X(ID, TH, UU) case ID: return TH * UU;
        SSB_LOOKBACK_CONFIGS(X)
#undef X
        default: return 0;
    }
}

bool lookback_eligible(int64_t rows, int64_t T, int tuning) {
    const int cap = lookback_cap(tuning);
    return cap > 0 && flat_eligible(rows, T) && T / 4 > cap;
}

// Tuning id 16 of the family: no look-back at all but two passes over chunks of T (few, very long
// rows, where the look-back chain of a row has too few CTAs behind it to hide its latency).
constexpr int kChunkedId = 16;
int64_t chunked_len(int64_t T) {  // a power of two that divides T: the chunks are rows of a [rows*K, len] view
    for (int64_t c = 4096; c >= 256; c >>= 1)
        if (T % c == 0 && T / c >= 2) return c;
    return 0;
}
size_t round256(size_t x) { return (x + 255) & ~(size_t)255; }
bool chunked_eligible(int64_t rows, int64_t T) {
    const int64_t len = chunked_len(T);
    return len > 0 && rows > 0 && T / len <= 0x7fffffffLL / rows;
}
size_t chunked_bytes(int64_t rows, int64_t T, size_t elem = 4) {  // maps [rows*K][2], carry [rows*K], h_prev [rows*K]
    if (!chunked_eligible(rows, T)) return 0;
    const size_t views = (size_t)rows * (size_t)(T / chunked_len(T));
    return round256(views * 2 * elem) + 2 * round256(views * elem);
}

// Tuning id 17 of the family: long chunks with early-terminated maps.  A row is cut into K chunks of
// whole 4096-element spans; pass 1 folds each chunk's map from the end its successor depends on and
// stops once the product of the gates walked so far has dropped to kChunkCut (scan_shard.cuh), so
// that gates below one cost a few thousand steps per chunk instead of a second pass over the
// tensor; then the carries are folded as for id 16 and the chunks run as rows of the span-by-span
// sweep.  K is the smallest divisor of T/4096 that gives at least kTailViews chunks in all (the
// sweep walks whole chunks per CTA and wants several per SM), chunks of at least two spans; rows too
// short for that get as many chunks as they have.
constexpr int kChunkedTailId = 17;
constexpr int kTailThreads = 256, kTailU = 2;  // map walk in 2048-element pieces: it overshoots the cut by half a piece on average
constexpr float kChunkCut = 9.094947017729282e-13f;  // 2^-40: far below fp32 rounding of the scan itself
constexpr int64_t kTailViews = 1024, kTailMinViews = 64;
constexpr int64_t kTailMaxRows = 256;  // the default up to this many rows (measured 1.5-2.2x look-back up to 96 rows, equal at 256)
int64_t tail_chunks(int64_t rows, int64_t T) {  // K, or 0 when the shape does not fit
    if (rows <= 0 || T % 4096 != 0) return 0;
    const int64_t n4 = T / 4096;
    int64_t enough = 0, most = 0;  // smallest K that reaches kTailViews chunks; largest K of all
    for (int64_t d = 1; d * d <= n4; d++) {
        if (n4 % d != 0) continue;
        for (int64_t k : {d, n4 / d}) {
            if (n4 / k < 2 || rows * k > 0x7fffffffLL) continue;
            if (rows * k >= kTailViews && (enough == 0 || k < enough)) enough = k;
            if (k > most) most = k;
        }
    }
    if (enough) return enough;
    return rows * most >= kTailMinViews ? most : 0;  // short rows: as many chunks as there are, if they can occupy the GPU at all
}
size_t chunked_tail_bytes(int64_t rows, int64_t T) {  // maps [views][2], carry [views], h_prev [views]
    const int64_t K = tail_chunks(rows, T);
    if (K == 0) return 0;
    const size_t views = (size_t)rows * (size_t)K;
    return round256(views * 8) + 2 * round256(views * 4);
}

size_t lookback_bytes(int64_t rows, int64_t T, int tuning) {
    if (tuning == kChunkedId) return chunked_bytes(rows, T);
    if (tuning == kChunkedTailId) return chunked_tail_bytes(rows, T);
    const int cap = lookback_cap(tuning);
    if (cap == 0 || T % 4 != 0) return 0;
    const int64_t pieces = (T / 4 + cap - 1) / cap;
    return ssb::lookback::kHeaderBytes + (size_t)rows * (size_t)pieces * sizeof(ssb::lookback::Record);
}

template <int THREADS, int U, bool BWD>
int launch_lookback(const float *gate, const float *in1, const float *in2, float *out1, float *out2, int64_t rows,
                    int64_t T, const float *carry_in, const float *h_prev, void *workspace, size_t need,
                    cudaStream_t st) {
    auto kern = ssb::lookback::lookback_kernel<THREADS, U, BWD>;
    const int64_t T4 = T / 4;
    ssb::lookback::Order order;
    order.rows = rows;
    order.pieces = (T4 + THREADS * U - 1) / (THREADS * U);
    const int grid_cap = persistent_grid<THREADS * 64 + U * 2 + (BWD ? 1 : 0) + 100000>(kern, THREADS, (int64_t)1 << 40);
    int64_t k = (grid_cap + rows - 1) / rows;
    if (k < 1) k = 1;
    if (k > order.pieces) k = order.pieces;
    order.k = k;
    order.wave = rows * k;
    const int64_t tickets = ((order.pieces + k - 1) / k) * order.wave;
    const int grid = (int)(tickets < grid_cap ? tickets : grid_cap);
    if (cudaMemsetAsync(workspace, 0, need, st) != cudaSuccess) return check_launch("cudaMemsetAsync(workspace)");
    kern<<<grid, THREADS, 0, st>>>(reinterpret_cast<const float4 *>(gate), reinterpret_cast<const float4 *>(in1),
                                   reinterpret_cast<const float4 *>(in2), reinterpret_cast<float4 *>(out1),
                                   reinterpret_cast<float4 *>(out2), T4, order, carry_in, h_prev,
                                   static_cast<unsigned char *>(workspace));
    return check_launch("lookback_kernel");
}

template <bool BWD, typename real = float>
int launch_chunked(const real *gate, const real *in1, const real *in2, real *out1, real *out2, int64_t rows, int64_t T,
                   const real *carry_in, const real *h_prev, void *workspace, size_t workspace_bytes, cudaStream_t st) {
    if (!chunked_eligible(rows, T))
        return fail(SSB_ERR_UNSUPPORTED, "the two-pass chunked scan needs T divisible by a power of two >= 256 (T=%lld)", (long long)T);
    const size_t need = chunked_bytes(rows, T, sizeof(real));
    if (workspace == nullptr || workspace_bytes < need || !aligned_to(workspace, 256))
        return fail(SSB_ERR_WORKSPACE, "the two-pass chunked scan needs a 256-byte aligned workspace of %zu bytes (got %zu)", need, workspace_bytes);
    const int64_t len = chunked_len(T), K = T / len, views = rows * K;
    char *ws = static_cast<char *>(workspace);
    real *maps = reinterpret_cast<real *>(ws);
    real *carry = reinterpret_cast<real *>(ws + round256((size_t)views * 2 * sizeof(real)));
    real *hprev = reinterpret_cast<real *>(ws + round256((size_t)views * 2 * sizeof(real)) + round256((size_t)views * sizeof(real)));
    // pass 1: the map of every chunk (two of the tensors read once)
    int rc;
    if constexpr (sizeof(real) == 4) {
        rc = BWD ? ssb_shard_reduce_bwd_f32(gate, in2, maps, views, len, nullptr, 0, st)
                 : ssb_shard_reduce_fwd_f32(gate, in1, maps, views, len, nullptr, 0, st);
    } else {
        rc = BWD ? launch_warp_bwd<real, true>(gate, nullptr, in2, nullptr, nullptr, views, len, nullptr, nullptr, maps, st)
                 : launch_warp_fwd<real, true>(gate, in1, nullptr, views, len, nullptr, maps, st);
    }
    if (rc != SSB_OK) return rc;
    const int64_t blocks = (rows * 32 + 255) / 256;
    ssb::lookback::chunk_carry_kernel<BWD, real><<<(int)blocks, 256, 0, st>>>(maps, rows, K, carry_in, carry);
    if ((rc = check_launch("chunk_carry_kernel")) != SSB_OK) return rc;
    if (BWD) {
        ssb::lookback::chunk_h_prev_kernel<real><<<(int)((views + 255) / 256), 256, 0, st>>>(in1, rows, K, len, h_prev, hprev);
        if ((rc = check_launch("chunk_h_prev_kernel")) != SSB_OK) return rc;
    }
    // pass 2: the chunks as rows of their own, each started from its entering state
    if constexpr (sizeof(real) == 4) {
        if (!BWD) return ssb_scan_fwd_f32_ex(gate, in1, out1, views, len, carry, SSB_VARIANT_AUTO, nullptr, 0, st);
        return ssb_scan_bwd_f32_ex(gate, in1, in2, out1, out2, views, len, carry, hprev, SSB_VARIANT_AUTO, nullptr, 0, st);
    } else {
        if (!BWD) return launch_warp_fwd<real, false>(gate, in1, out1, views, len, carry, nullptr, st);
        return launch_warp_bwd<real, false>(gate, in1, in2, out1, out2, views, len, carry, hprev, nullptr, st);
    }
}

template <bool BWD>
int launch_chunked_tail(const float *gate, const float *in1, const float *in2, float *out1, float *out2, int64_t rows, int64_t T,
                        const float *carry_in, const float *h_prev, void *workspace, size_t workspace_bytes, cudaStream_t st);

template <bool BWD>
int dispatch_lookback(int tuning, const float *gate, const float *in1, const float *in2, float *out1, float *out2,
                      int64_t rows, int64_t T, const float *carry_in, const float *h_prev, void *workspace,
                      size_t workspace_bytes, cudaStream_t st) {
    if (tuning == kChunkedId)
        return launch_chunked<BWD>(gate, in1, in2, out1, out2, rows, T, carry_in, h_prev, workspace, workspace_bytes, st);
    if (tuning == kChunkedTailId)
        return launch_chunked_tail<BWD>(gate, in1, in2, out1, out2, rows, T, carry_in, h_prev, workspace, workspace_bytes, st);
    if (!lookback_eligible(rows, T, tuning))
        return fail(SSB_ERR_UNSUPPORTED, "look-back kernels need 16-byte aligned tensors, T %% 4 == 0 and rows longer than one span (T=%lld)", (long long)T);
    const size_t need = lookback_bytes(rows, T, tuning);
    if (workspace == nullptr || workspace_bytes < need || !aligned_to(workspace, 256))
        return fail(SSB_ERR_WORKSPACE, "look-back needs a 256-byte aligned workspace of %zu bytes (got %zu)", need, workspace_bytes);
    switch (tuning) {
#define X(ID, TH, UU) case ID: return launch_lookback<TH, UU, BWD>(gate, in1, in2, out1, out2, rows, T, carry_in, h_prev, workspace, need, st);
        SSB_LOOKBACK_CONFIGS(X)
#undef X
        default: return fail(SSB_ERR_UNSUPPORTED, "unknown look-back tuning id %d", tuning);
    }
}

// Row aggregates through per-span maps in a workspace (long rows).
constexpr int kMapsThreads = 256, kMapsU = 4;

size_t span_maps_bytes(int64_t rows, int64_t T) {
    if (T % 4 != 0 || T / 4 <= kMapsThreads * kMapsU) return 0;
    const int64_t pieces = (T / 4 + kMapsThreads * kMapsU - 1) / (kMapsThreads * kMapsU);
    return (size_t)rows * (size_t)pieces * sizeof(float2);
}

template <bool BWD>
int launch_span_maps(const float *gate, const float *in1, float *agg, int64_t rows, int64_t T, void *workspace,
                     cudaStream_t st) {
    const int64_t T4 = T / 4;
    const int64_t pieces = (T4 + kMapsThreads * kMapsU - 1) / (kMapsThreads * kMapsU);
    auto kern = ssb::lookback::span_maps_kernel<kMapsThreads, kMapsU, BWD>;
    const int grid = persistent_grid<200000 + (BWD ? 1 : 0)>(kern, kMapsThreads, rows * pieces);
    kern<<<grid, kMapsThreads, 0, st>>>(reinterpret_cast<const float4 *>(gate), reinterpret_cast<const float4 *>(in1),
                                        rows, T4, pieces, static_cast<float2 *>(workspace));
    int rc = check_launch("span_maps_kernel");
    if (rc != SSB_OK) return rc;
    const int64_t blocks = (rows * 32 + 255) / 256;
    ssb::lookback::fold_maps_kernel<BWD><<<(int)blocks, 256, 0, st>>>(static_cast<const float2 *>(workspace), rows, pieces, agg);
    return check_launch("fold_maps_kernel");
}

// ------------------------------------------------------------------------------------
// TMA-staged flat sweep (power-of-two rows that fit a span); tuning ids 32 + k of the TMA family
// ------------------------------------------------------------------------------------
#define SSB_TMAFLAT_CONFIGS(X) /* id, lines, stages, out buffers (forward) | (backward) */ \
    X(0, 128, 2, 2, 128, 2, 1) X(1, 128, 3, 2, 128, 2, 2) X(2, 64, 3, 2, 64, 3, 2) X(3, 64, 4, 2, 64, 2, 2) \
    X(4, 128, 2, 1, 64, 2, 1) X(5, 256, 2, 1, 128, 3, 1) X(6, 32, 4, 2, 32, 4, 2)

// `elem_bytes`: 4 (fp32) or 2 (bf16 / fp16 storage); a 128-byte line holds 128 / elem_bytes elements.
constexpr int kTmaFlatLongId = 48;  // TMA family tuning id: the flat sweep over rows of several 4096-element spans
bool tmaflat_eligible(int64_t rows, int64_t T, int lines, int elem_bytes = 4) {
    const int per_line = 128 / elem_bytes;
    if (T % per_line != 0 || rows > 0x7fffffffLL) return false;
    const int64_t lpr = T / per_line;
    return lpr >= 1 && lpr <= lines && (lpr & (lpr - 1)) == 0;
}

template <typename IO> constexpr CUtensorMapDataType tensor_map_type();
template <> constexpr CUtensorMapDataType tensor_map_type<float>() { return CU_TENSOR_MAP_DATA_TYPE_FLOAT32; }
template <> constexpr CUtensorMapDataType tensor_map_type<__nv_bfloat16>() { return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; }
template <> constexpr CUtensorMapDataType tensor_map_type<__half>() { return CU_TENSOR_MAP_DATA_TYPE_FLOAT16; }

template <typename IO>
int make_span_map(CUtensorMap *map, const IO *ptr, int64_t rows, int64_t T, int lines) {
    PFN_cuTensorMapEncodeTiled_v12000 enc = encode_fn();
    if (enc == nullptr) return fail(SSB_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
    constexpr int per_line = 128 / (int)sizeof(IO);
    const int64_t lpr = T / per_line;
    cuuint64_t dims[3] = {(cuuint64_t)per_line, (cuuint64_t)lpr, (cuuint64_t)rows};
    cuuint64_t strides[2] = {128, (cuuint64_t)T * sizeof(IO)};
    cuuint32_t box[3] = {(cuuint32_t)per_line, (cuuint32_t)lpr, (cuuint32_t)(lines / lpr)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_tiled(enc, map, tensor_map_type<IO>(), 3, const_cast<IO *>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SSB_ERR_LAUNCH, "cuTensorMapEncodeTiled(span) failed with CUresult %d", (int)r);
    return SSB_OK;
}

template <typename T> struct as_given { using type = T; };  // keeps a parameter out of template deduction

// The same view with boxes of `lines` lines of one row (rows longer than a span).
template <typename IO>
int make_long_map(CUtensorMap *map, const IO *ptr, int64_t rows, int64_t T, int lines) {
    PFN_cuTensorMapEncodeTiled_v12000 enc = encode_fn();
    if (enc == nullptr) return fail(SSB_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
    constexpr int per_line = 128 / (int)sizeof(IO);
    cuuint64_t dims[3] = {(cuuint64_t)per_line, (cuuint64_t)(T / per_line), (cuuint64_t)rows};
    cuuint64_t strides[2] = {128, (cuuint64_t)T * sizeof(IO)};
    cuuint32_t box[3] = {(cuuint32_t)per_line, (cuuint32_t)lines, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_tiled(enc, map, tensor_map_type<IO>(), 3, const_cast<IO *>(ptr), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SSB_ERR_LAUNCH, "cuTensorMapEncodeTiled(long rows) failed with CUresult %d", (int)r);
    return SSB_OK;
}

// LONG: rows of a whole number of spans (T % (LINES * 128 / sizeof(IO)) == 0, more than one span):
// a CTA walks a row span by span and chains the state through shared memory.
template <int LINES, int STAGES, int OUTBUF, bool BWD, bool SIGMOID = false, bool RECOMPUTE = false, typename IO = float,
          bool LONG = false>
int launch_tmaflat(const IO *gate, const IO *in1, const typename as_given<IO>::type *in2, IO *out1,
                   typename as_given<IO>::type *out2, int64_t rows,
                   int64_t T, const float *carry_a, const float *carry_b, cudaStream_t st) {
    using Cfg = ssb::tmaflat::Config<LINES, STAGES, OUTBUF, BWD, IO>;
    static_assert(STAGES >= 2, "the ring needs a stage to refill while another is consumed");
    constexpr int per_line = 128 / (int)sizeof(IO);
    constexpr int64_t span_elems = (int64_t)LINES * per_line;
    if (LONG) {
        if (T % span_elems != 0 || T / span_elems < 2 || T / span_elems > 0x7fffffffLL || rows > 0x7fffffffLL)
            return fail(SSB_ERR_UNSUPPORTED, "the TMA flat sweep over long rows needs T to be a multiple (>= 2) of %lld (T=%lld)",
                        (long long)span_elems, (long long)T);
    } else if (!tmaflat_eligible(rows, T, LINES, (int)sizeof(IO))) {
        return fail(SSB_ERR_UNSUPPORTED, "the TMA flat sweep needs T = %d * 2^k <= %d (T=%lld)", per_line, LINES * per_line, (long long)T);
    }
    auto kern = ssb::tmaflat::tma_flat_kernel<LINES, STAGES, OUTBUF, BWD, SIGMOID, RECOMPUTE, IO, LONG>;
    CUtensorMap mg, m1, m2, mo1, mo2;
    int rc;
    auto make = [&](CUtensorMap *m, const IO *p) { return LONG ? make_long_map<IO>(m, p, rows, T, LINES) : make_span_map(m, p, rows, T, LINES); };
    if ((rc = make(&mg, gate)) != SSB_OK) return rc;
    if ((rc = make(&m1, in1)) != SSB_OK) return rc;
    if ((rc = make(&mo1, out1)) != SSB_OK) return rc;
    if (BWD) {
        if ((rc = make(&m2, in2)) != SSB_OK) return rc;
        if ((rc = make(&mo2, out2)) != SSB_OK) return rc;
    } else {  // the forward never touches them: any valid descriptor will do
        m2 = m1;
        mo2 = mo1;
    }
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(tma_flat_kernel)");
    static std::atomic<int> cached_occ{0};  // one per instantiation of this function template
    int occ = cached_occ.load(std::memory_order_relaxed);
    if (occ == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, Cfg::THREADS, Cfg::SMEM_BYTES) != cudaSuccess || occ <= 0) {
            (void)cudaGetLastError();
            occ = 1;
        }
        cached_occ.store(occ, std::memory_order_relaxed);
    }
    const int upr = LONG ? Cfg::THREADS : (int)(T / 32);  // 32-element units per row (LONG: per piece)
    const int64_t spans = LONG ? rows : (rows + Cfg::THREADS / upr - 1) / (Cfg::THREADS / upr);
    const int64_t cap = (int64_t)sm_count() * occ;
    int grid = (int)(spans < cap ? spans : cap);
    if (LONG && spans > cap) {  // whole rows per CTA: as few CTAs as give every CTA the same number of rows (+-1)
        const int64_t per_cta = (spans + cap - 1) / cap;
        grid = (int)((spans + per_cta - 1) / per_cta);
    }
    const int pieces = LONG ? (int)(T / span_elems) : 1;
    // a programmatic dependent of whatever precedes it in the stream: the kernel waits for that before
    // its first access to global memory, so only its launch and set-up overlap the predecessor's tail
    const IO *h_rows = (LONG && BWD) ? in1 : nullptr;
    if (launch_dependent(kern, grid, Cfg::THREADS, Cfg::SMEM_BYTES, st, mg, m1, m2, mo1, mo2, rows, upr, carry_a, carry_b, pieces,
                         h_rows) != cudaSuccess)
        return check_launch("tma_flat_kernel (dependent launch)");
    return check_launch("tma_flat_kernel");
}

template <bool BWD>
int launch_chunked_tail(const float *gate, const float *in1, const float *in2, float *out1, float *out2, int64_t rows, int64_t T,
                        const float *carry_in, const float *h_prev, void *workspace, size_t workspace_bytes, cudaStream_t st) {
    const int64_t K = tail_chunks(rows, T);
    if (K == 0 || encode_fn() == nullptr)
        return fail(SSB_ERR_UNSUPPORTED, "the long-chunk form needs T to be a multiple of 4096 with a divisor that yields at least %lld "
                    "chunks of two or more spans (rows=%lld T=%lld)", (long long)kTailViews, (long long)rows, (long long)T);
    const size_t need = chunked_tail_bytes(rows, T);
    if (workspace == nullptr || workspace_bytes < need || !aligned_to(workspace, 256))
        return fail(SSB_ERR_WORKSPACE, "the long-chunk form needs a 256-byte aligned workspace of %zu bytes (got %zu)", need, workspace_bytes);
    const int64_t views = rows * K, len = T / K;
    char *ws = static_cast<char *>(workspace);
    float *maps = reinterpret_cast<float *>(ws);
    float *carry = reinterpret_cast<float *>(ws + round256((size_t)views * 8));
    float *hprev = reinterpret_cast<float *>(ws + round256((size_t)views * 8) + round256((size_t)views * 4));
    // pass 1: every chunk's map, walked from the end the next chunk depends on, as far as the gate product needs
    auto mk = ssb::shard::tail_map_kernel<kTailThreads, kTailU, BWD>;
    const int grid = persistent_grid<600000 + (BWD ? 1 : 0)>(mk, kTailThreads, views);
    mk<<<grid, kTailThreads, 0, st>>>(reinterpret_cast<const float4 *>(gate), reinterpret_cast<const float4 *>(BWD ? in2 : in1), views,
                                      len / 4, kChunkCut, maps, nullptr, ssb::shard::PeerExchange(), 0, 0u);
    int rc = check_launch("tail_map_kernel");
    if (rc != SSB_OK) return rc;
    // pass 2: the state entering every chunk (one warp per row folds its K maps in order)
    ssb::lookback::chunk_carry_kernel<BWD, float><<<(int)((rows * 32 + 255) / 256), 256, 0, st>>>(maps, rows, K, carry_in, carry);
    if ((rc = check_launch("chunk_carry_kernel")) != SSB_OK) return rc;
    if (BWD) {
        ssb::lookback::chunk_h_prev_kernel<float><<<(int)((views + 255) / 256), 256, 0, st>>>(in1, rows, K, len, h_prev, hprev);
        if ((rc = check_launch("chunk_h_prev_kernel")) != SSB_OK) return rc;
    }
    // pass 3: the chunks as rows of the span-by-span sweep, each started from its entering state
    if (!BWD) return launch_tmaflat<128, 4, 2, false, false, false, float, true>(gate, in1, nullptr, out1, nullptr, views, len, carry, nullptr, st);
    return launch_tmaflat<128, 3, 1, true, false, false, float, true>(gate, in1, in2, out1, out2, views, len, carry, hprev, st);
}

// `variant` carries the family in its low byte and a tuning id in bits 8..15 (0 = default).
int family_of(int variant) { return variant & 0xff; }
int tuning_of(int variant) { return (variant >> 8) & 0xff; }
int grid_per_sm_of(int variant) { return (variant >> 16) & 0xff; }

int dispatch_tma_fwd(int tuning, const float *gate, const float *value, float *out, int64_t rows,
                     int64_t T, const float *h_in, cudaStream_t st) {
    switch (tuning) {
        case 0: return launch_tma_fwd<16, 4, 8>(gate, value, out, rows, T, h_in, st);
        case 1: return launch_tma_fwd<16, 2, 8>(gate, value, out, rows, T, h_in, st);
        case 2: return launch_tma_fwd<16, 3, 8>(gate, value, out, rows, T, h_in, st);
        case 3: return launch_tma_fwd<16, 6, 8>(gate, value, out, rows, T, h_in, st);
        case 4: return launch_tma_fwd<16, 4, 10>(gate, value, out, rows, T, h_in, st);
        case 5: return launch_tma_fwd<16, 8, 4>(gate, value, out, rows, T, h_in, st);
        case 6: return launch_tma_fwd<32, 2, 8>(gate, value, out, rows, T, h_in, st);
        case 7: return launch_tma_fwd<32, 4, 4>(gate, value, out, rows, T, h_in, st);
        case 8: return launch_tma_fwd<32, 2, 6>(gate, value, out, rows, T, h_in, st);
        case 9: return launch_tma_fwd<16, 4, 6>(gate, value, out, rows, T, h_in, st);
        case 10: return launch_tma_fwd<16, 2, 16>(gate, value, out, rows, T, h_in, st);
        case 11: return launch_tma_fwd<16, 3, 12>(gate, value, out, rows, T, h_in, st);
        default: return fail(SSB_ERR_UNSUPPORTED, "unknown forward TMA tuning id %d", tuning);
    }
}

int dispatch_tma_bwd(int tuning, const float *gate, const float *h, const float *gout, float *ggate,
                     float *gvalue, int64_t rows, int64_t T, const float *c_in, const float *h_prev,
                     cudaStream_t st) {
    switch (tuning) {
        case 0: return launch_tma_bwd<16, 3, 8>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 1: return launch_tma_bwd<16, 2, 8>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 2: return launch_tma_bwd<16, 2, 10>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 3: return launch_tma_bwd<16, 4, 6>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 4: return launch_tma_bwd<16, 5, 5>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 5: return launch_tma_bwd<16, 8, 4>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 6: return launch_tma_bwd<32, 2, 5>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 7: return launch_tma_bwd<32, 3, 4>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 8: return launch_tma_bwd<16, 3, 6>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 10: return launch_tma_bwd<16, 2, 11>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case 11: return launch_tma_bwd<16, 2, 12>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        default: return fail(SSB_ERR_UNSUPPORTED, "unknown backward TMA tuning id %d", tuning);
    }
}

// Default kernel choice, from sweeps on B200 over T = 64 .. 16M at 67 MB .. 4 GB per tensor
// (`python -m scanscam_b200.tune` reproduces them):
//   * aligned fp32, T = 32 * 2^k <= 4096 (every benchmark configuration but the long-context
//     one) -> the TMA-staged flat sweep: spans of whole rows brought in by bulk tensor copies,
//     32 elements per thread.  Same speed as the register version below within +-1 % (203-209
//     Gelem/s fwd+bwd on cfg2/4/5 either way), ~30 W less power, 10 % higher sustained SM clock.
//   * other aligned fp32 with T % 4 == 0, rows that fit a 16 KB span (T <= 4096) -> flat, 128
//     threads x 8 float4s: the best or within 2 % of the best in both directions at every T.
//   * longer rows: look-back (same span shape) when the caller can supply scratch -- within 3 %
//     of the best everywhere and the only family whose speed does not depend on the number of
//     rows; without scratch the flat family walks each row with one CTA.
//   * very long rows with 1024 or more of them: the TMA ring (one warp per row, 2-stage ring,
//     8 warps per CTA) is 3-7 % ahead of look-back there and needs no scratch.
//   * odd T on aligned tensors -> the per-element flat sweep or one warp per row, by length;
//     unaligned views and fp64 -> one warp per row.
int pick_variant(bool backward, int64_t rows, int64_t T, bool all_aligned16, bool workspace_ok = false) {
    // Many long rows of whole 4096-element spans: the flat sweep that walks a row span by span wins the
    // backward at every measured shape from 1024 x 65536 to 16384 x 16384 (+1-7 % over look-back, +0.5-4 %
    // over the per-warp ring) and the forward from 2048 rows up; below that the forward is left to the
    // rules that follow (per-warp ring for very long rows, look-back otherwise).  It needs no scratch.
    if (all_aligned16 && rows >= (backward ? 1024 : 2048) && T >= 16384 && T % 4096 == 0 && T / 4096 <= 0x7fffffffLL &&
        rows <= 0x7fffffffLL && encode_fn() != nullptr)
        return SSB_VARIANT_TMA | (kTmaFlatLongId << 8);
    // Forward, about a thousand long rows (too few for the sweep above): the per-warp ring of 16-warp
    // CTAs beats look-back by 4-6 % from 65536 steps up (6.46 / 6.61 against 6.10 / 6.30 TB/s at
    // 1024 x 65536 / 131072); at 1536 rows look-back is ahead again (6.1-6.3 against 5.9).
    if (!backward && all_aligned16 && tma_eligible(rows, T) && T >= 65536 && rows >= 1024 && rows < 1280 && encode_fn() != nullptr)
        return SSB_VARIANT_TMA | (10 << 8);
    if (all_aligned16 && tma_eligible(rows, T) && T >= 262144 && rows >= 1024) return SSB_VARIANT_TMA | (1 << 8);
    // A few very long rows: a row's look-back chain has too few CTAs behind it to hide its latency, and
    // two passes over 4096-step chunks (20 / 28 bytes per element) win by 10-35 % (measured at 4, 16 and
    // 64 rows; at 1-2 rows the serial carry pass over the chunks takes the gain back, from 96 rows up
    // look-back is at 3.5-6 TB/s and wins).
    if (workspace_ok && all_aligned16 && rows <= kTailMaxRows && T >= 65536 && tail_chunks(rows, T) != 0 && encode_fn() != nullptr)
        return SSB_VARIANT_LOOKBACK | (kChunkedTailId << 8);
    if (workspace_ok && all_aligned16 && rows >= 4 && rows <= 80 && T >= 65536 && chunked_len(T) == 4096 &&
        T / 4096 <= 4096 && chunked_eligible(rows, T) && encode_fn() != nullptr)
        return SSB_VARIANT_LOOKBACK | (kChunkedId << 8);
    // Look-back: rows longer than a span when there are too few of them to give every CTA a row of its own,
    // or when they are long (from 16384 steps).  Many rows just above a span (16384 x 4100: a full span and a
    // 4-element one per row) are left to the flat sweep below, which packs them better (6.3 against 4.2-4.7 TB/s).
    if (workspace_ok && all_aligned16 && lookback_eligible(rows, T, 0) && T > 4096 && (rows < 1024 || T >= 16384))
        return SSB_VARIANT_LOOKBACK;
    // Small problems (a few spans per SM at most, e.g. [4,256,1024]): the kernels are a few microseconds
    // long and what counts is how fast the grid gets going, not the steady state.  Power-of-two rows up
    // to 2048 steps: the TMA-staged sweep with 64-line spans, whose launch overlaps the tail of the
    // kernel ahead (programmatic dependent launch) -- on [1024,1024], forward + backward: 9.0 us inside
    // a CUDA graph, 9.6 us as stream launches, against 9.4 / 12.3 us for the choice below.  Other row
    // lengths: 512-element spans of 128 threads x 1 float4, which give every SM several CTAs at once.
    // (4096-step rows go to the general rule for power-of-two rows further down.)
    if (all_aligned16 && T <= 4096 && rows * T <= (int64_t)sm_count() * 4 * 4096) {
        const bool tma_ok = encode_fn() != nullptr;
        if (tma_ok && tmaflat_eligible(rows, T, 64)) return SSB_VARIANT_TMA | (34 << 8);
        if (flat_eligible(rows, T) && !(tma_ok && tmaflat_eligible(rows, T, 128))) return SSB_VARIANT_FLAT | (12 << 8);
    }
    if (all_aligned16 && tmaflat_eligible(rows, T, 128) && encode_fn() != nullptr) {
        // power-of-two rows that fit a span: the TMA-staged sweep (forward 128 lines x 2 stages;
        // backward 128 lines x 3 stages for 4096-step rows, 64 lines x 2 stages below)
        if (!backward) return SSB_VARIANT_TMA | (32 << 8);
        return SSB_VARIANT_TMA | ((T > 2048 ? 37 : 36) << 8);
    }
    if (all_aligned16 && flat_eligible(rows, T)) {
        // The default span holds 4096 elements: whole rows are packed into it, longer rows are walked
        // in 4096-element pieces.  When that leaves more than a fifth of the span's slots idle
        // (T = 2200: one row per span; T = 4100: a full piece and a 4-element one) the 2048-element
        // span of 128 threads x 4 float4s is 3-25 % faster (measured at T = 1500, 2200, 2600, 3000, 4100,
        // 5000; at T = 6000, two pieces and 73 % used, the large span still wins).
        const double used = T <= 4096 ? (double)((4096 / T) * T) / 4096.0 : (double)T / (double)(((T + 4095) / 4096) * 4096);
        if (used < (T <= 4096 ? 0.8 : 0.65)) return SSB_VARIANT_FLAT | (4 << 8);
        if (backward && T > 4096) return SSB_VARIANT_FLAT | (9 << 8);
        return SSB_VARIANT_FLAT | (6 << 8);
    }
    // Odd T: the per-element flat sweep (256 threads x 4 float4s) beats one warp per row for short
    // rows (a warp is mostly idle below ~384 steps) and for rows longer than a span; in between
    // the warp kernels are 10-30 % faster.
    if (all_aligned16 && flat_any_eligible(rows, T) && (T < 384 || T > 4608)) return SSB_VARIANT_FLAT_ANY | (1 << 8);
    return SSB_VARIANT_WARP;
}

// SSB_VARIANT_AUTO in the _ex entry points: the choice ssb_scan_recommend(..., can_provide_workspace = 1)
// reports when the caller's scratch is usable (256-byte aligned and large enough for that choice),
// else the choice made without scratch.
int pick_with_scratch(bool backward, int64_t rows, int64_t T, bool all_aligned16, const void *workspace, size_t workspace_bytes) {
    if (workspace != nullptr && aligned_to(workspace, 256)) {
        const int v = pick_variant(backward, rows, T, all_aligned16, true);
        if (family_of(v) != SSB_VARIANT_LOOKBACK || workspace_bytes >= lookback_bytes(rows, T, tuning_of(v))) return v;
    }
    return pick_variant(backward, rows, T, all_aligned16, false);
}

}  // namespace

extern "C" {

int ssb_version(void) { return 200; }

const char *ssb_status_string(int status) {
    switch (status) {
        case SSB_OK: return "ok";
        case SSB_ERR_BAD_ARG: return "bad argument";
        case SSB_ERR_ALIGNMENT: return "misaligned pointer";
        case SSB_ERR_LAUNCH: return "CUDA launch or driver error";
        case SSB_ERR_DEVICE_WAIT: return "device-side wait ran out";
        case SSB_ERR_WORKSPACE: return "workspace missing or too small";
        case SSB_ERR_UNSUPPORTED: return "variant does not support this shape";
        case SSB_ERR_DEVICE_CHECK: return "checked build: index outside its tensor";
        default: return "unknown status";
    }
}

const char *ssb_last_error(void) { return t_last_error; }

size_t ssb_scan_workspace_bytes(int64_t rows, int64_t T, int variant) {
    if (rows <= 0 || T <= 0 || family_of(variant) != SSB_VARIANT_LOOKBACK) return 0;
    return lookback_bytes(rows, T, tuning_of(variant));
}

int ssb_scan_recommend(int64_t rows, int64_t T, int backward, int aligned16, int can_provide_workspace) {
    if (rows <= 0 || T <= 0) return SSB_VARIANT_WARP;
    return pick_variant(backward != 0, rows, T, aligned16 != 0, can_provide_workspace != 0);
}

size_t ssb_shard_reduce_workspace_bytes(int64_t rows, int64_t T) {
    if (rows <= 0 || T <= 0) return 0;
    return span_maps_bytes(rows, T);
}

int ssb_scan_fwd_f32_ex(const float *gate, const float *value, float *out, int64_t rows, int64_t T,
                        const float *h_in, int variant, void *workspace, size_t workspace_bytes,
                        void *stream) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate || !value || !out) return fail(SSB_ERR_BAD_ARG, "ssb_scan_fwd_f32: NULL tensor pointer");
    if (!aligned_to(gate, 4) || !aligned_to(value, 4) || !aligned_to(out, 4) || !aligned_to(h_in, 4))
        return fail(SSB_ERR_ALIGNMENT, "ssb_scan_fwd_f32: pointers must be 4-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const GridScope grid_scope(grid_per_sm_of(variant));
    const bool al16 = aligned_to(gate, 16) && aligned_to(value, 16) && aligned_to(out, 16);
    if (family_of(variant) == SSB_VARIANT_AUTO) variant = pick_with_scratch(false, rows, T, al16, workspace, workspace_bytes);
    const int family = family_of(variant);
    switch (family) {
        case SSB_VARIANT_WARP:
            return launch_warp_fwd<float, false>(gate, value, out, rows, T, h_in, nullptr, st);
        case SSB_VARIANT_TMA:
            if (!al16 || !tma_eligible(rows, T))
                return fail(SSB_ERR_UNSUPPORTED, "TMA forward needs T %% 32 == 0 and 16-byte aligned tensors (T=%lld)", (long long)T);
            if (tuning_of(variant) == kTmaFlatLongId)  // four stages, one CTA per SM: every SM carries the same number of rows
                return launch_tmaflat<128, 4, 2, false, false, false, float, true>(gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr, st);
            if (tuning_of(variant) >= 32) {
                switch (tuning_of(variant) - 32) {
#define X(ID, FL, FS, FO, BL, BS, BO) case ID: return launch_tmaflat<FL, FS, FO, false>(gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr, st);
                    SSB_TMAFLAT_CONFIGS(X)
#undef X
                    default: return fail(SSB_ERR_UNSUPPORTED, "unknown TMA flat tuning id %d", tuning_of(variant));
                }
            }
            return dispatch_tma_fwd(tuning_of(variant), gate, value, out, rows, T, h_in, st);
        case SSB_VARIANT_FLAT:
            if (!al16 || !flat_eligible(rows, T))
                return fail(SSB_ERR_UNSUPPORTED, "flat forward needs T %% 4 == 0 and 16-byte aligned tensors (T=%lld)", (long long)T);
            return dispatch_flat_fwd(tuning_of(variant), gate, value, out, rows, T, h_in, st);
        case SSB_VARIANT_FLAT_ANY:
            if (!al16 || !flat_any_eligible(rows, T))
                return fail(SSB_ERR_UNSUPPORTED, "the any-T flat forward needs 16-byte aligned tensors");
            return tuning_of(variant) == 1 ? launch_flat_any<256, 4, false>(gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr, st)
                                           : launch_flat_any<128, 8, false>(gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr, st);
        case SSB_VARIANT_LOOKBACK:
            if (!al16) return fail(SSB_ERR_UNSUPPORTED, "look-back forward needs 16-byte aligned tensors");
            return dispatch_lookback<false>(tuning_of(variant), gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr,
                                            workspace, workspace_bytes, st);
        default:
            return fail(SSB_ERR_UNSUPPORTED, "forward variant %d is not available", variant);
    }
}

}  // extern "C"

// ---- built-in scratch for callers that cannot allocate --------------------------------------
namespace {

static_assert(SSB_STATIC_SCRATCH_BYTES ==
                  ssb::lookback::kHeaderBytes + SSB_STATIC_SCRATCH_SPANS * sizeof(ssb::lookback::Record),
              "the header's figures describe the look-back workspace layout");

// Lives in the library image: each GPU that loads the library carries these bytes until exit.
// In host code this name is only a handle for the runtime's symbol queries, never a device
// address; the launcher below asks the runtime for the address and hands that to the kernel.
static __device__ __align__(256) unsigned char g_static_scratch[SSB_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device, looked up once per device.
int static_scratch_address(void **out) {
    static std::atomic<void *> cached[64];
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(SSB_ERR_LAUNCH, "cudaGetDevice: %s", cudaGetErrorString(e));
    void *p = (dev >= 0 && dev < 64) ? cached[dev].load(std::memory_order_acquire) : nullptr;
    if (p == nullptr) {
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return fail(SSB_ERR_LAUNCH, "cudaGetSymbolAddress(built-in scratch) on device %d: %s", dev,
                        cudaGetErrorString(e));
        }
        if (dev >= 0 && dev < 64) cached[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return SSB_OK;
}

}  // namespace

extern "C" {

int ssb_scan_fwd_f32_static(const float *gate, const float *value, float *out, int64_t rows, int64_t T,
                            const float *h_in, void *stream) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate || !value || !out) return fail(SSB_ERR_BAD_ARG, "ssb_scan_fwd_f32_static: NULL tensor pointer");
    if (!aligned_to(gate, 16) || !aligned_to(value, 16) || !aligned_to(out, 16) || !aligned_to(h_in, 4))
        return fail(SSB_ERR_ALIGNMENT, "ssb_scan_fwd_f32_static: gate, value and out must be 16-byte aligned");
    if (!lookback_eligible(rows, T, 0))
        return fail(SSB_ERR_UNSUPPORTED,
                    "ssb_scan_fwd_f32_static serves rows longer than one 4096-element span with T %% 4 == 0 "
                    "(got T=%lld); other shapes need no scratch, call ssb_scan_fwd_f32",
                    (long long)T);
    const size_t need = lookback_bytes(rows, T, 0);
    if (need > (size_t)SSB_STATIC_SCRATCH_BYTES)
        return fail(SSB_ERR_WORKSPACE,
                    "problem needs %zu bytes of scratch (%lld rows x %lld spans) but the built-in scratch holds "
                    "%zu bytes (%d spans); pass your own workspace to ssb_scan_fwd_f32_ex instead",
                    need, (long long)rows, (long long)((T / 4 + 1023) / 1024), (size_t)SSB_STATIC_SCRATCH_BYTES,
                    SSB_STATIC_SCRATCH_SPANS);
    void *scratch = nullptr;
    if ((rc = static_scratch_address(&scratch)) != SSB_OK) return rc;
    // launch_lookback clears `need` bytes of the scratch on the stream (ticket counter and record
    // flags must start at zero; whatever the previous call left beyond that is never read).
    return launch_lookback<128, 8, false>(gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr, scratch, need,
                                          static_cast<cudaStream_t>(stream));
}

int ssb_scan_fwd_f32(const float *gate, const float *value, float *out, int64_t rows, int64_t T,
                     const float *h_in, void *stream) {
    return ssb_scan_fwd_f32_ex(gate, value, out, rows, T, h_in, SSB_VARIANT_AUTO, nullptr, 0, stream);
}

int ssb_scan_fwd_f64(const double *gate, const double *value, double *out, int64_t rows, int64_t T,
                     const double *h_in, void *stream) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate || !value || !out) return fail(SSB_ERR_BAD_ARG, "ssb_scan_fwd_f64: NULL tensor pointer");
    if (!aligned_to(gate, 8) || !aligned_to(value, 8) || !aligned_to(out, 8) || !aligned_to(h_in, 8))
        return fail(SSB_ERR_ALIGNMENT, "ssb_scan_fwd_f64: pointers must be 8-byte aligned");
    return launch_warp_fwd<double, false>(gate, value, out, rows, T, h_in, nullptr, static_cast<cudaStream_t>(stream));
}

int ssb_scan_bwd_f32_ex(const float *gate, const float *h, const float *gout, float *ggate, float *gvalue,
                        int64_t rows, int64_t T, const float *c_in, const float *h_prev, int variant,
                        void *workspace, size_t workspace_bytes, void *stream) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate || !h || !gout || !ggate || !gvalue) return fail(SSB_ERR_BAD_ARG, "ssb_scan_bwd_f32: NULL tensor pointer");
    if (!aligned_to(gate, 4) || !aligned_to(h, 4) || !aligned_to(gout, 4) || !aligned_to(ggate, 4) ||
        !aligned_to(gvalue, 4) || !aligned_to(c_in, 4) || !aligned_to(h_prev, 4))
        return fail(SSB_ERR_ALIGNMENT, "ssb_scan_bwd_f32: pointers must be 4-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const GridScope grid_scope(grid_per_sm_of(variant));
    const bool al16 = aligned_to(gate, 16) && aligned_to(h, 16) && aligned_to(gout, 16) &&
                      aligned_to(ggate, 16) && aligned_to(gvalue, 16);
    if (family_of(variant) == SSB_VARIANT_AUTO) variant = pick_with_scratch(true, rows, T, al16, workspace, workspace_bytes);
    const int family = family_of(variant);
    switch (family) {
        case SSB_VARIANT_WARP:
            return launch_warp_bwd<float, false>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, nullptr, st);
        case SSB_VARIANT_TMA:
            if (!al16 || !tma_eligible(rows, T))
                return fail(SSB_ERR_UNSUPPORTED, "TMA backward needs T %% 32 == 0 and 16-byte aligned tensors (T=%lld)", (long long)T);
            if (tuning_of(variant) == kTmaFlatLongId)
                return launch_tmaflat<128, 3, 1, true, false, false, float, true>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
            if (tuning_of(variant) >= 32) {
                switch (tuning_of(variant) - 32) {
#define X(ID, FL, FS, FO, BL, BS, BO) case ID: return launch_tmaflat<BL, BS, BO, true>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
                    SSB_TMAFLAT_CONFIGS(X)
#undef X
                    default: return fail(SSB_ERR_UNSUPPORTED, "unknown TMA flat tuning id %d", tuning_of(variant));
                }
            }
            return dispatch_tma_bwd(tuning_of(variant), gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case SSB_VARIANT_FLAT:
            if (!al16 || !flat_eligible(rows, T))
                return fail(SSB_ERR_UNSUPPORTED, "flat backward needs T %% 4 == 0 and 16-byte aligned tensors (T=%lld)", (long long)T);
            return dispatch_flat_bwd(tuning_of(variant), gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case SSB_VARIANT_FLAT_ANY:
            if (!al16 || !flat_any_eligible(rows, T))
                return fail(SSB_ERR_UNSUPPORTED, "the any-T flat backward needs 16-byte aligned tensors");
            return tuning_of(variant) == 1 ? launch_flat_any<256, 4, true>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st)
                                           : launch_flat_any<128, 8, true>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        case SSB_VARIANT_LOOKBACK:
            if (!al16) return fail(SSB_ERR_UNSUPPORTED, "look-back backward needs 16-byte aligned tensors");
            return dispatch_lookback<true>(tuning_of(variant), gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev,
                                           workspace, workspace_bytes, st);
        default:
            return fail(SSB_ERR_UNSUPPORTED, "backward variant %d is not available", variant);
    }
}

int ssb_scan_sigmoid_fwd_f32(const float *gate_logits, const float *value, float *out, int64_t rows, int64_t T,
                             const float *h_in, void *stream) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate_logits || !value || !out) return fail(SSB_ERR_BAD_ARG, "ssb_scan_sigmoid_fwd_f32: NULL tensor pointer");
    if (!aligned_to(gate_logits, 16) || !aligned_to(value, 16) || !aligned_to(out, 16) || !aligned_to(h_in, 4) ||
        !flat_eligible(rows, T))
        return fail(SSB_ERR_UNSUPPORTED, "ssb_scan_sigmoid_fwd_f32 needs T %% 4 == 0 and 16-byte aligned tensors (T=%lld)", (long long)T);
    if (tmaflat_eligible(rows, T, 128) && encode_fn() != nullptr)
        return launch_tmaflat<128, 2, 2, false, true>(gate_logits, value, nullptr, out, nullptr, rows, T, h_in, nullptr,
                                                      static_cast<cudaStream_t>(stream));
    auto kern = ssb::flat::flat_fwd_kernel<128, 8, true>;
    const int grid = persistent_grid<500000>(kern, 128, flat_units(rows, T / 4, 128 * 8));
    kern<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const float4 *>(gate_logits),
                                                             reinterpret_cast<const float4 *>(value),
                                                             reinterpret_cast<float4 *>(out), rows, T / 4, h_in);
    return check_launch("flat_fwd_kernel<sigmoid>");
}

int ssb_scan_sigmoid_bwd_f32(const float *gate_logits, const float *h, const float *gout, float *glogits, float *gvalue,
                             int64_t rows, int64_t T, const float *c_in, const float *h_prev, void *stream) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate_logits || !h || !gout || !glogits || !gvalue) return fail(SSB_ERR_BAD_ARG, "ssb_scan_sigmoid_bwd_f32: NULL tensor pointer");
    if (!aligned_to(gate_logits, 16) || !aligned_to(h, 16) || !aligned_to(gout, 16) || !aligned_to(glogits, 16) ||
        !aligned_to(gvalue, 16) || !aligned_to(c_in, 4) || !aligned_to(h_prev, 4) || !flat_eligible(rows, T))
        return fail(SSB_ERR_UNSUPPORTED, "ssb_scan_sigmoid_bwd_f32 needs T %% 4 == 0 and 16-byte aligned tensors (T=%lld)", (long long)T);
    if (tmaflat_eligible(rows, T, 128) && encode_fn() != nullptr) {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        return T > 2048 ? launch_tmaflat<128, 3, 1, true, true>(gate_logits, h, gout, glogits, gvalue, rows, T, c_in, h_prev, st)
                        : launch_tmaflat<64, 2, 1, true, true>(gate_logits, h, gout, glogits, gvalue, rows, T, c_in, h_prev, st);
    }
    auto kern = ssb::flat::flat_bwd_kernel<128, 8, 0, true>;
    const int grid = persistent_grid<500001>(kern, 128, flat_units(rows, T / 4, 128 * 8));
    kern<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4 *>(gate_logits), reinterpret_cast<const float4 *>(h),
        reinterpret_cast<const float4 *>(gout), reinterpret_cast<float4 *>(glogits), reinterpret_cast<float4 *>(gvalue),
        rows, T / 4, c_in, h_prev);
    return check_launch("flat_bwd_kernel<sigmoid>");
}

// ---- backward that recomputes h -----------------------------------------------------------
static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
static bool recompute_in_kernel(int64_t rows, int64_t T) { return tmaflat_eligible(rows, T, 128) && encode_fn() != nullptr; }

size_t ssb_scan_bwd_recompute_workspace_bytes(int64_t rows, int64_t T) {
    int64_t n;
    if (check_shape(rows, T, &n) != SSB_OK || n == 0 || recompute_in_kernel(rows, T)) return 0;
    const size_t fwd_ws = ssb_scan_workspace_bytes(rows, T, pick_variant(false, rows, T, true, true));
    const size_t bwd_ws = ssb_scan_workspace_bytes(rows, T, pick_variant(true, rows, T, true, true));
    return align256((size_t)rows * (size_t)T * 4) + (fwd_ws > bwd_ws ? fwd_ws : bwd_ws);
}

int ssb_scan_bwd_recompute_f32(const float *gate, const float *value, const float *gout, float *ggate, float *gvalue,
                               int64_t rows, int64_t T, const float *h_in, const float *c_in, void *workspace,
                               size_t workspace_bytes, void *stream) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate || !value || !gout || !ggate || !gvalue)
        return fail(SSB_ERR_BAD_ARG, "ssb_scan_bwd_recompute_f32: NULL tensor pointer");
    if (!aligned_to(gate, 16) || !aligned_to(value, 16) || !aligned_to(gout, 16) || !aligned_to(ggate, 16) ||
        !aligned_to(gvalue, 16) || !aligned_to(h_in, 4) || !aligned_to(c_in, 4))
        return fail(SSB_ERR_ALIGNMENT, "ssb_scan_bwd_recompute_f32: tensors must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (recompute_in_kernel(rows, T))
        return T > 2048 ? launch_tmaflat<128, 3, 1, true, false, true>(gate, value, gout, ggate, gvalue, rows, T, c_in, h_in, st)
                        : launch_tmaflat<64, 2, 1, true, false, true>(gate, value, gout, ggate, gvalue, rows, T, c_in, h_in, st);
    // Other shapes: the forward kernel rebuilds h into the workspace, the ordinary backward reads it.
    const size_t need = ssb_scan_bwd_recompute_workspace_bytes(rows, T);
    if (workspace == nullptr || workspace_bytes < need || !aligned_to(workspace, 256))
        return fail(SSB_ERR_WORKSPACE, "ssb_scan_bwd_recompute_f32 needs a 256-byte aligned workspace of %zu bytes (got %zu)",
                    need, workspace_bytes);
    float *h = static_cast<float *>(workspace);
    const size_t h_bytes = align256((size_t)n * 4);
    void *inner = static_cast<char *>(workspace) + h_bytes;
    const size_t inner_bytes = workspace_bytes - h_bytes;
    rc = ssb_scan_fwd_f32_ex(gate, value, h, rows, T, h_in, pick_variant(false, rows, T, true, true), inner, inner_bytes, stream);
    if (rc != SSB_OK) return rc;
    return ssb_scan_bwd_f32_ex(gate, h, gout, ggate, gvalue, rows, T, c_in, h_in, pick_variant(true, rows, T, true, true),
                               inner, inner_bytes, stream);
}

int ssb_scan_bwd_f32(const float *gate, const float *h, const float *gout, float *ggate, float *gvalue,
                     int64_t rows, int64_t T, const float *c_in, const float *h_prev, void *stream) {
    return ssb_scan_bwd_f32_ex(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, SSB_VARIANT_AUTO, nullptr, 0, stream);
}

int ssb_scan_bwd_f64(const double *gate, const double *h, const double *gout, double *ggate, double *gvalue,
                     int64_t rows, int64_t T, const double *c_in, const double *h_prev, void *stream) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate || !h || !gout || !ggate || !gvalue) return fail(SSB_ERR_BAD_ARG, "ssb_scan_bwd_f64: NULL tensor pointer");
    if (!aligned_to(gate, 8) || !aligned_to(h, 8) || !aligned_to(gout, 8) || !aligned_to(ggate, 8) ||
        !aligned_to(gvalue, 8) || !aligned_to(c_in, 8) || !aligned_to(h_prev, 8))
        return fail(SSB_ERR_ALIGNMENT, "ssb_scan_bwd_f64: pointers must be 8-byte aligned");
    return launch_warp_bwd<double, false>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, nullptr,
                                          static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ---- fp64 with scratch: a few long rows in two passes ------------------------------------------
namespace {
// One warp per row needs about a thousand rows to fill the GPU; below that, rows of whole 4096-step
// chunks run in the two-pass chunked form (40 / 56 bytes per element moved instead of 24 / 40).
// Measured: 16 rows x 2^21 steps 11.3 / 14.3 ms -> 0.25 / 0.33 ms, 512 rows 1.6x faster, 1024 rows slower.
constexpr int64_t kF64ChunkedRows = 768;
bool f64_chunked_applies(int64_t rows, int64_t T, const void *workspace, size_t workspace_bytes) {
    return rows < kF64ChunkedRows && T >= 16384 && chunked_len(T) == 4096 && chunked_eligible(rows, T) && workspace != nullptr &&
           aligned_to(workspace, 256) && workspace_bytes >= chunked_bytes(rows, T, 8);
}
}  // namespace

extern "C" {

size_t ssb_scan_f64_workspace_bytes(int64_t rows, int64_t T) {
    if (rows <= 0 || T <= 0 || rows >= kF64ChunkedRows || T < 16384 || chunked_len(T) != 4096) return 0;
    return chunked_bytes(rows, T, 8);
}

int ssb_scan_fwd_f64_ex(const double *gate, const double *value, double *out, int64_t rows, int64_t T, const double *h_in,
                        void *workspace, size_t workspace_bytes, void *stream) {
    int64_t n;
    if (check_shape(rows, T, &n) == SSB_OK && n > 0 && gate && value && out && aligned_to(gate, 8) && aligned_to(value, 8) &&
        aligned_to(out, 8) && aligned_to(h_in, 8) && f64_chunked_applies(rows, T, workspace, workspace_bytes))
        return launch_chunked<false, double>(gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr, workspace,
                                             workspace_bytes, static_cast<cudaStream_t>(stream));
    return ssb_scan_fwd_f64(gate, value, out, rows, T, h_in, stream);
}

int ssb_scan_bwd_f64_ex(const double *gate, const double *h, const double *gout, double *ggate, double *gvalue, int64_t rows,
                        int64_t T, const double *c_in, const double *h_prev, void *workspace, size_t workspace_bytes,
                        void *stream) {
    int64_t n;
    if (check_shape(rows, T, &n) == SSB_OK && n > 0 && gate && h && gout && ggate && gvalue && aligned_to(gate, 8) &&
        aligned_to(h, 8) && aligned_to(gout, 8) && aligned_to(ggate, 8) && aligned_to(gvalue, 8) && aligned_to(c_in, 8) &&
        aligned_to(h_prev, 8) && f64_chunked_applies(rows, T, workspace, workspace_bytes))
        return launch_chunked<true, double>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, workspace, workspace_bytes,
                                            static_cast<cudaStream_t>(stream));
    return ssb_scan_bwd_f64(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, stream);
}

}  // extern "C"

// ---- 16-bit storage (bf16 / fp16 in memory, fp32 arithmetic and carries) --------------------
namespace {

// SIGMOID / RECOMPUTE as in the fp32 entry points; those forms exist on the bulk-tensor sweep only
// (rows of T = 64 * 2^k <= 8192, for SIGMOID also larger multiples of 4096; 16-byte aligned), other
// shapes return SSB_ERR_UNSUPPORTED.
template <typename IO, bool SIGMOID = false>
int scan_fwd_h16(const void *gate_, const void *value_, void *out_, int64_t rows, int64_t T, const float *h_in,
                 void *stream, const char *who) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate_ || !value_ || !out_) return fail(SSB_ERR_BAD_ARG, "%s: NULL tensor pointer", who);
    if (!aligned_to(gate_, 2) || !aligned_to(value_, 2) || !aligned_to(out_, 2) || !aligned_to(h_in, 4))
        return fail(SSB_ERR_ALIGNMENT, "%s: tensors must be 2-byte aligned, carries 4-byte aligned", who);
    const IO *gate = static_cast<const IO *>(gate_), *value = static_cast<const IO *>(value_);
    IO *out = static_cast<IO *>(out_);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool al16 = aligned_to(gate, 16) && aligned_to(value, 16) && aligned_to(out, 16);
    if (al16 && encode_fn() != nullptr) {
        // configurations from a sweep on [16384,4096], [65536,2048], [524288,512] and [262144,64]
        if (tmaflat_eligible(rows, T, 64, 2))
            return T > 2048 ? launch_tmaflat<64, 2, 1, false, SIGMOID, false, IO>(gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr, st)
                            : launch_tmaflat<64, 2, 2, false, SIGMOID, false, IO>(gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr, st);
        if (tmaflat_eligible(rows, T, 128, 2))
            return launch_tmaflat<128, 2, 2, false, SIGMOID, false, IO>(gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr, st);
        // longer rows of whole spans: a CTA walks the row (8192-element spans, one CTA per SM with a deep
        // ring, measured 5-25 % ahead of 4096-element spans at four CTAs per SM where both apply)
        // (not with the sigmoid fused: that needs the four CTAs per SM to hide its arithmetic)
        if (!SIGMOID && T % 8192 == 0 && T > 8192)
            return launch_tmaflat<128, 4, 2, false, SIGMOID, false, IO, true>(gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr, st);
        if (T % 4096 == 0 && T > 8192)
            return launch_tmaflat<64, 2, 2, false, SIGMOID, false, IO, true>(gate, value, nullptr, out, nullptr, rows, T, h_in, nullptr, st);
    }
    if (SIGMOID)
        return fail(SSB_ERR_UNSUPPORTED, "%s needs T = 64 * 2^k <= 8192 (or, without recomputation, a larger multiple of 4096) and 16-byte aligned tensors (T=%lld)", who, (long long)T);
    const int grid = warp_grid(rows), block = ssb::kWarpKernelWarps * 32;
    if (al16 && T % 8 == 0)
        ssb::warp_rows_fwd_kernel<float, 8, 2, false, IO><<<grid, block, 0, st>>>(gate, value, out, rows, T, h_in, nullptr);
    else
        ssb::warp_rows_fwd_kernel<float, 1, 4, false, IO><<<grid, block, 0, st>>>(gate, value, out, rows, T, h_in, nullptr);
    return check_launch("warp_rows_fwd_kernel<16-bit>");
}

template <typename IO, bool SIGMOID = false, bool RECOMPUTE = false>
int scan_bwd_h16(const void *gate_, const void *h_, const void *gout_, void *ggate_, void *gvalue_, int64_t rows, int64_t T,
                 const float *c_in, const float *h_prev, void *stream, const char *who) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate_ || !h_ || !gout_ || !ggate_ || !gvalue_) return fail(SSB_ERR_BAD_ARG, "%s: NULL tensor pointer", who);
    if (!aligned_to(gate_, 2) || !aligned_to(h_, 2) || !aligned_to(gout_, 2) || !aligned_to(ggate_, 2) ||
        !aligned_to(gvalue_, 2) || !aligned_to(c_in, 4) || !aligned_to(h_prev, 4))
        return fail(SSB_ERR_ALIGNMENT, "%s: tensors must be 2-byte aligned, carries 4-byte aligned", who);
    const IO *gate = static_cast<const IO *>(gate_), *h = static_cast<const IO *>(h_), *gout = static_cast<const IO *>(gout_);
    IO *ggate = static_cast<IO *>(ggate_), *gvalue = static_cast<IO *>(gvalue_);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool al16 = aligned_to(gate, 16) && aligned_to(h, 16) && aligned_to(gout, 16) && aligned_to(ggate, 16) &&
                      aligned_to(gvalue, 16);
    if (al16 && encode_fn() != nullptr) {
        if (tmaflat_eligible(rows, T, 64, 2))
            return launch_tmaflat<64, 2, 1, true, SIGMOID, RECOMPUTE, IO>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        if (tmaflat_eligible(rows, T, 128, 2))
            return launch_tmaflat<128, 3, 1, true, SIGMOID, RECOMPUTE, IO>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        if constexpr (!RECOMPUTE) {
            if (!SIGMOID && T % 8192 == 0 && T > 8192)
                return launch_tmaflat<128, 3, 1, true, SIGMOID, false, IO, true>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
            if (T % 4096 == 0 && T > 8192)
                return launch_tmaflat<64, 2, 1, true, SIGMOID, false, IO, true>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, st);
        }
    }
    if (SIGMOID || RECOMPUTE)
        return fail(SSB_ERR_UNSUPPORTED, "%s needs T = 64 * 2^k <= 8192 (or, without recomputation, a larger multiple of 4096) and 16-byte aligned tensors (T=%lld)", who, (long long)T);
    const int grid = warp_grid(rows), block = ssb::kWarpKernelWarps * 32;
    if (al16 && T % 8 == 0)
        ssb::warp_rows_bwd_kernel<float, 8, 2, false, IO><<<grid, block, 0, st>>>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, nullptr);
    else
        ssb::warp_rows_bwd_kernel<float, 1, 4, false, IO><<<grid, block, 0, st>>>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, nullptr);
    return check_launch("warp_rows_bwd_kernel<16-bit>");
}

}  // namespace

extern "C" {

int ssb_scan_fwd_bf16(const void *gate, const void *value, void *out, int64_t rows, int64_t T, const float *h_in, void *stream) {
    return scan_fwd_h16<__nv_bfloat16>(gate, value, out, rows, T, h_in, stream, "ssb_scan_fwd_bf16");
}
int ssb_scan_fwd_f16(const void *gate, const void *value, void *out, int64_t rows, int64_t T, const float *h_in, void *stream) {
    return scan_fwd_h16<__half>(gate, value, out, rows, T, h_in, stream, "ssb_scan_fwd_f16");
}
int ssb_scan_bwd_bf16(const void *gate, const void *h, const void *gout, void *ggate, void *gvalue, int64_t rows, int64_t T,
                      const float *c_in, const float *h_prev, void *stream) {
    return scan_bwd_h16<__nv_bfloat16>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, stream, "ssb_scan_bwd_bf16");
}
int ssb_scan_bwd_f16(const void *gate, const void *h, const void *gout, void *ggate, void *gvalue, int64_t rows, int64_t T,
                     const float *c_in, const float *h_prev, void *stream) {
    return scan_bwd_h16<__half>(gate, h, gout, ggate, gvalue, rows, T, c_in, h_prev, stream, "ssb_scan_bwd_f16");
}
int ssb_scan_sigmoid_fwd_bf16(const void *gate_logits, const void *value, void *out, int64_t rows, int64_t T, const float *h_in,
                              void *stream) {
    return scan_fwd_h16<__nv_bfloat16, true>(gate_logits, value, out, rows, T, h_in, stream, "ssb_scan_sigmoid_fwd_bf16");
}
int ssb_scan_sigmoid_bwd_bf16(const void *gate_logits, const void *h, const void *gout, void *glogits, void *gvalue,
                              int64_t rows, int64_t T, const float *c_in, const float *h_prev, void *stream) {
    return scan_bwd_h16<__nv_bfloat16, true>(gate_logits, h, gout, glogits, gvalue, rows, T, c_in, h_prev, stream,
                                             "ssb_scan_sigmoid_bwd_bf16");
}
int ssb_scan_sigmoid_fwd_f16(const void *gate_logits, const void *value, void *out, int64_t rows, int64_t T, const float *h_in,
                             void *stream) {
    return scan_fwd_h16<__half, true>(gate_logits, value, out, rows, T, h_in, stream, "ssb_scan_sigmoid_fwd_f16");
}
int ssb_scan_sigmoid_bwd_f16(const void *gate_logits, const void *h, const void *gout, void *glogits, void *gvalue,
                             int64_t rows, int64_t T, const float *c_in, const float *h_prev, void *stream) {
    return scan_bwd_h16<__half, true>(gate_logits, h, gout, glogits, gvalue, rows, T, c_in, h_prev, stream,
                                      "ssb_scan_sigmoid_bwd_f16");
}
int ssb_scan_bwd_recompute_bf16(const void *gate, const void *value, const void *gout, void *ggate, void *gvalue, int64_t rows,
                                int64_t T, const float *h_in, const float *c_in, void *stream) {
    return scan_bwd_h16<__nv_bfloat16, false, true>(gate, value, gout, ggate, gvalue, rows, T, c_in, h_in, stream,
                                                    "ssb_scan_bwd_recompute_bf16");
}
int ssb_scan_bwd_recompute_f16(const void *gate, const void *value, const void *gout, void *ggate, void *gvalue, int64_t rows,
                               int64_t T, const float *h_in, const float *c_in, void *stream) {
    return scan_bwd_h16<__half, false, true>(gate, value, gout, ggate, gvalue, rows, T, c_in, h_in, stream,
                                             "ssb_scan_bwd_recompute_f16");
}

}  // extern "C"

// ---- channels-last ---------------------------------------------------------------------
namespace {
constexpr int kClWarps = 16;
constexpr int kClSteps = 8;

int check_cl(int64_t N, int64_t T, int64_t C, int64_t *n) {
    if (N < 0 || T < 0 || C < 0) return fail(SSB_ERR_BAD_ARG, "negative size: N=%lld T=%lld C=%lld", (long long)N, (long long)T, (long long)C);
    if (C > 0 && T > std::numeric_limits<int64_t>::max() / 8 / C) return fail(SSB_ERR_BAD_ARG, "T*C overflows");
    int rc = check_shape(N, T * C, n);
    if (rc != SSB_OK) return rc;
    const int64_t blocks = N * ((C + 31) / 32);
    if (blocks > 0x7fffffffLL) return fail(SSB_ERR_BAD_ARG, "N*ceil(C/32) exceeds the grid limit");
    return SSB_OK;
}

// Look-back channels-last kernels: W warps per CTA, L time steps per warp.  Tuning table:
// id -> (W, L forward, L backward); the smallest tile (W*L) of the table bounds the workspace.
#define SSB_CL2_CONFIGS(X) X(0, 8, 16, 16) X(1, 8, 16, 16) X(12, 8, 8, 4) X(2, 4, 4, 4) X(3, 8, 4, 2) X(4, 2, 16, 8) X(5, 4, 8, 8) X(6, 4, 8, 2) X(7, 4, 16, 8) \
    X(8, 8, 16, 8) X(9, 4, 8, 4) X(10, 8, 32, 16) X(11, 8, 24, 16)
constexpr int kCl2MinTile = 8;  // every instantiated tile (W*L) must cover at least this many steps

template <int VEC, int kCl2Warps, int L, bool BWD>
int launch_cl2(const float *gate, const float *in1, const float *in2, float *out1, float *out2, int64_t N, int64_t T,
               int64_t C, void *workspace, size_t workspace_bytes, cudaStream_t st) {
    static_assert(kCl2Warps * L >= kCl2MinTile, "ssb_scan_cl_workspace_bytes sizes the workspace for tiles of kCl2MinTile steps");
    auto kern = ssb::cl2::cl_lookback_kernel<VEC, kCl2Warps, L, BWD>;
    ssb::cl2::Geometry geo;
    geo.N = N; geo.T = T; geo.C = C;
    geo.cgroups = (C + 32 * VEC - 1) / (32 * VEC);
    geo.pieces = (T + kCl2Warps * L - 1) / (kCl2Warps * L);
    geo.n_tiles = N * geo.cgroups * geo.pieces;
    if (ssb::cl2::workspace_bytes(geo.n_tiles, VEC) > workspace_bytes)
        return fail(SSB_ERR_WORKSPACE, "channels-last look-back needs %zu bytes of workspace, got %zu",
                    ssb::cl2::workspace_bytes(geo.n_tiles, VEC), workspace_bytes);
    ssb::lookback::Order order;
    order.rows = N * geo.cgroups;
    order.pieces = geo.pieces;
    const int grid_cap = persistent_grid<300000 + VEC * 10000 + kCl2Warps * 1000 + L * 10 + (BWD ? 1 : 0)>(kern, kCl2Warps * 32, (int64_t)1 << 40);
    int64_t k = (grid_cap + order.rows - 1) / order.rows;
    if (k < 1) k = 1;
    if (k > order.pieces) k = order.pieces;
    order.k = k;
    order.wave = order.rows * k;
    const int64_t tickets = ((order.pieces + k - 1) / k) * order.wave;
    const int grid = (int)(tickets < grid_cap ? tickets : grid_cap);
    if (cudaMemsetAsync(workspace, 0, ssb::cl2::bytes_to_clear(geo.n_tiles), st) != cudaSuccess)
        return check_launch("cudaMemsetAsync(workspace)");
    kern<<<grid, kCl2Warps * 32, 0, st>>>(gate, in1, in2, out1, out2, geo, order, static_cast<unsigned char *>(workspace));
    return check_launch("cl_lookback_kernel");
}

// TMA-staged channels-last kernels.  Tuning ids 32 + k -> (CC, TT, stages, out buffers) forward | backward.
#define SSB_CL3_CONFIGS(X)                                                         \
    X(0, 64, 64, 3, 2, 64, 64, 2, 1) X(1, 64, 32, 3, 2, 64, 32, 3, 2) X(2, 128, 32, 3, 2, 128, 32, 2, 1) \
    X(3, 64, 128, 2, 1, 64, 64, 2, 2) X(4, 32, 64, 4, 2, 32, 64, 3, 2) X(5, 128, 64, 2, 1, 128, 32, 2, 2)
constexpr int kCl3MinTileElems = 32 * 64;  // smallest CC*TT of the table (bounds the workspace)

// What cuTensorMapEncodeTiled and the kernels' 32-bit box coordinates accept for a {C, T, N} view:
// pitches that are multiples of 16 bytes and below 2^40, extents below 2^31 with room for one tile.
bool cl3_eligible(int64_t N, int64_t T, int64_t C) {
    return C % 4 == 0 && N <= 0x7fffffffLL && T <= 0x7fffff00LL && C <= 0x7fffffffLL && T <= ((1LL << 40) - 1) / 4 / C;
}

template <typename IO>
int make_cl_map(CUtensorMap *map, const IO *ptr, int64_t N, int64_t T, int64_t C, int cc, int tt) {
    PFN_cuTensorMapEncodeTiled_v12000 enc = encode_fn();
    if (enc == nullptr) return fail(SSB_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {(cuuint64_t)C, (cuuint64_t)T, (cuuint64_t)N};
    cuuint64_t strides[2] = {(cuuint64_t)C * sizeof(IO), (cuuint64_t)T * (cuuint64_t)C * sizeof(IO)};
    cuuint32_t box[3] = {(cuuint32_t)cc, (cuuint32_t)tt, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_tiled(enc, map, tensor_map_type<IO>(), 3, const_cast<IO *>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SSB_ERR_LAUNCH, "cuTensorMapEncodeTiled([N,T,C]) failed with CUresult %d", (int)r);
    return SSB_OK;
}

// Channels-last streaming kernels (one CTA walks all of T for a block of channels, tiles through a
// TMA ring, no workspace).  Tuning ids 64 + k -> (CC, TT, segments, stages, out buffers) forward | backward.
// Ids 0 and 1 are the defaults for 32- and 64-channel blocks, picked from a sweep of 73 forward and
// 37 backward tile shapes on [8,4096,512], [64,4096,512], [16,2048,1024], [1,16384,8192] and
// [32,1024,2048]: large tiles win (the per-tile barriers and store hand-off are the fixed cost).
#define SSB_CLS_CONFIGS(X)                                                                   \
    X(0, 32, 256, 16, 2, 2, 32, 128, 16, 2, 1) X(1, 64, 256, 16, 1, 1, 64, 128, 8, 1, 1)     \
    X(2, 32, 128, 16, 2, 2, 32, 256, 16, 1, 1) X(3, 64, 128, 8, 2, 2, 64, 64, 8, 2, 1)       \
    X(4, 32, 64, 8, 2, 2, 32, 64, 16, 2, 1) X(5, 64, 64, 8, 2, 1, 64, 64, 4, 2, 1)           \
    X(6, 128, 32, 8, 3, 2, 128, 32, 8, 2, 1) X(7, 32, 128, 32, 2, 1, 32, 128, 32, 2, 1)

// `chunk_steps` = 0: a unit is all of T.  Otherwise (a multiple of TT) T is cut into chunks of that
// many steps, each a unit of its own that starts from the fold of maps[unit'][2][CC] over the chunks
// before it (written by cl_tail_map_kernel just ahead in the stream).
template <int CC, int TT, int SEG, int STAGES, int OUTBUF, bool BWD, typename IO = float, bool SIGMOID = false>
int launch_cls(const IO *gate, const typename as_given<IO>::type *in1, const typename as_given<IO>::type *in2,
               typename as_given<IO>::type *out1, typename as_given<IO>::type *out2, int64_t N, int64_t T,
               int64_t C, cudaStream_t st, int64_t chunk_steps = 0, const float *maps = nullptr) {
    using Cfg = ssb::cls::Config<CC, TT, SEG, STAGES, OUTBUF, BWD, IO>;
    auto kern = ssb::cls::cl_stream_kernel<CC, TT, SEG, STAGES, OUTBUF, BWD, IO, SIGMOID>;
    const int64_t cblocks = (C + CC - 1) / CC, tiles = (T + TT - 1) / TT;
    if (tiles > 0x7fffffffLL) return fail(SSB_ERR_UNSUPPORTED, "channels-last streaming kernels: T too large");
    if (chunk_steps % TT != 0) return fail(SSB_ERR_BAD_ARG, "channels-last streaming kernels: chunk of %lld steps, tiles of %d", (long long)chunk_steps, TT);
    const int64_t pieces = chunk_steps > 0 ? chunk_steps / TT : tiles;
    const int64_t chunks = (tiles + pieces - 1) / pieces;
    // tensors this launch does not touch still need a valid descriptor: describe a tensor it does
    const IO *p_in2 = BWD ? in2 : in1;
    IO *p_out2 = BWD ? out2 : out1;
    CUtensorMap mg, m1, m2, mo1, mo2;
    int rc;
    if ((rc = make_cl_map(&mg, gate, N, T, C, CC, TT)) != SSB_OK) return rc;
    if ((rc = make_cl_map(&m1, in1, N, T, C, CC, TT)) != SSB_OK) return rc;
    if ((rc = make_cl_map(&m2, p_in2, N, T, C, CC, TT)) != SSB_OK) return rc;
    if ((rc = make_cl_map(&mo1, out1, N, T, C, CC, TT)) != SSB_OK) return rc;
    if ((rc = make_cl_map(&mo2, p_out2, N, T, C, CC, TT)) != SSB_OK) return rc;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(cl_stream_kernel)");
    static std::atomic<int> cached_occ{0};  // one per instantiation of this function template
    int occ = cached_occ.load(std::memory_order_relaxed);
    if (occ == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, Cfg::THREADS, Cfg::SMEM_BYTES) != cudaSuccess || occ <= 0) {
            (void)cudaGetLastError();
            occ = 1;
        }
        cached_occ.store(occ, std::memory_order_relaxed);
    }
    const int64_t units = N * cblocks * chunks, cap = (int64_t)sm_count() * occ;
    const int grid = (int)(units < cap ? units : cap);
    if (maps != nullptr) {
        // the scan pass of the chunked form: it may start beside the map kernel it follows and waits
        // for it inside (griddepcontrol.wait) before the first read of `maps`
        if (launch_dependent(kern, grid, Cfg::THREADS, Cfg::SMEM_BYTES, st, mg, m1, m2, mo1, mo2, units, (int)cblocks, (int)pieces,
                             (int)chunks, maps) != cudaSuccess)
            return check_launch("cl_stream_kernel (dependent launch)");
        return check_launch("cl_stream_kernel");
    }
    kern<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(mg, m1, m2, mo1, mo2, units, (int)cblocks, (int)pieces, (int)chunks, maps);
    return check_launch("cl_stream_kernel");
}

// Two-pass form for shapes with few (batch element, channel block) pairs: chunk maps, carries, scan.
constexpr int kClsChunkTile = 256;   // chunk lengths are multiples of this (every tile height divides it)

// `cc`: channels per block (32 for fp32, 64 for 16-bit storage).  A chunk is p tiles; the scan pass
// gives every SM one chunk at a time, so its duration is rounds * (p + start-up) tile times with
// rounds = ceil(pairs * chunks / SMs), and the map pass walks about two tiles per chunk.  p is the
// value that minimises that estimate (e.g. 4 pairs x 1024 tiles: 37 chunks of 28 tiles = exactly
// one chunk per SM, instead of 47 chunks that need two rounds).
int64_t cls_chunk_steps(int64_t N, int64_t T, int64_t C, int cc = 32) {
    const int64_t pairs = N * ((C + cc - 1) / cc), tiles = (T + kClsChunkTile - 1) / kClsChunkTile;
    const int64_t slots = sm_count();
    int64_t best_p = tiles;
    double best_cost = 1e300;
    for (int64_t p = tiles < 4 ? tiles : 4; p <= tiles; p++) {
        const int64_t chunks = (tiles + p - 1) / p, units = pairs * chunks;
        if (units > 64 * slots) continue;
        const int64_t rounds = (units + slots - 1) / slots;
        const double cost = (double)rounds * ((double)p + 2.0) + (double)units * (p < 2 ? (double)p : 2.0) * 0.67 / (double)slots;
        if (cost < best_cost) { best_cost = cost; best_p = p; }
        if (chunks == 1) break;
    }
    return best_p * kClsChunkTile;
}
size_t cls_chunk_workspace_bytes(int64_t N, int64_t T, int64_t C, int cc = 32) {
    const int64_t steps = cls_chunk_steps(N, T, C, cc), chunks = (T + steps - 1) / steps;
    return (size_t)(N * ((C + cc - 1) / cc) * chunks) * 2 * cc * sizeof(float);  // (A, B) per unit and channel
}

template <bool BWD, typename IO = float, bool SIGMOID = false>
int launch_cls_chunked(const IO *gate, const typename as_given<IO>::type *in1, const typename as_given<IO>::type *in2,
                       typename as_given<IO>::type *out1, typename as_given<IO>::type *out2, int64_t N, int64_t T,
                       int64_t C, void *workspace, size_t workspace_bytes, cudaStream_t st) {
    constexpr int CC = 128 / (int)sizeof(IO);  // 128-byte tile rows
    const int64_t steps = cls_chunk_steps(N, T, C, CC), chunks = (T + steps - 1) / steps, pairs = N * ((C + CC - 1) / CC);
    if (workspace == nullptr || workspace_bytes < cls_chunk_workspace_bytes(N, T, C, CC))
        return fail(SSB_ERR_WORKSPACE, "channels-last chunked streaming needs %zu bytes of workspace, got %zu",
                    cls_chunk_workspace_bytes(N, T, C, CC), workspace_bytes);
    float *maps = static_cast<float *>(workspace);
    // pass 1 walks each chunk only as far as its gate products need (stops at 2^-40 in all of the block's channels)
    constexpr int kSeg = 256 / (CC / 4);  // 256 threads: 32 x 8 steps per tile for fp32, 16 x 8 for 16-bit storage
    auto mk = ssb::cls::cl_tail_map_kernel<kSeg, 8, BWD, SIGMOID, IO>;
    const int64_t units = pairs * chunks;
    const int grid = persistent_grid<700000 + (BWD ? 1 : 0) + (SIGMOID ? 2 : 0) + 4 * (int)sizeof(IO) +
                                     (std::is_same<IO, __half>::value ? 32 : 0)>(mk, 256, units);
    mk<<<grid, 256, 0, st>>>(gate, BWD ? in2 : in1, T, C, units, (int)((C + CC - 1) / CC), steps, (int)chunks, kChunkCut, maps);
    int rc = check_launch("cl_tail_map_kernel");
    if (rc != SSB_OK) return rc;
    // pass 2: the scan over the chunks; every unit folds the maps of its pair's chunks before it for itself
    if (!BWD) return launch_cls<CC, 256, 16, 2, 2, false, IO, SIGMOID>(gate, in1, nullptr, out1, nullptr, N, T, C, st, steps, maps);
    if constexpr (sizeof(IO) == 2)
        return launch_cls<CC, 256, 16, 1, 1, true, IO, SIGMOID>(gate, in1, in2, out1, out2, N, T, C, st, steps, maps);
    else
        return launch_cls<CC, 128, 16, 2, 1, true, IO, SIGMOID>(gate, in1, in2, out1, out2, N, T, C, st, steps, maps);
}

template <int CC, int TT, int STAGES, int OUTBUF, bool BWD>
int launch_cl3(const float *gate, const float *in1, const float *in2, float *out1, float *out2, int64_t N, int64_t T,
               int64_t C, void *workspace, size_t workspace_bytes, cudaStream_t st) {
    using Cfg = ssb::cl3::Config<CC, TT, STAGES, OUTBUF, BWD>;
    static_assert(CC * TT >= kCl3MinTileElems, "workspace bound assumes tiles of at least kCl3MinTileElems elements");
    static_assert(STAGES >= 2, "the ring needs a stage to refill while another is consumed");
    auto kern = ssb::cl3::cl_tma_kernel<CC, TT, STAGES, OUTBUF, BWD>;
    ssb::cl2::Geometry geo;
    geo.N = N; geo.T = T; geo.C = C;
    geo.cgroups = (C + CC - 1) / CC;
    geo.pieces = (T + TT - 1) / TT;
    geo.n_tiles = N * geo.cgroups * geo.pieces;
    const size_t need = ssb::cl3::workspace_bytes(geo.n_tiles, CC);
    if (need > workspace_bytes)
        return fail(SSB_ERR_WORKSPACE, "channels-last TMA kernels need %zu bytes of workspace, got %zu", need, workspace_bytes);
    CUtensorMap mg, m1, m2, mo1, mo2;
    int rc;
    if ((rc = make_cl_map(&mg, gate, N, T, C, CC, TT)) != SSB_OK) return rc;
    if ((rc = make_cl_map(&m1, in1, N, T, C, CC, TT)) != SSB_OK) return rc;
    if ((rc = make_cl_map(&m2, BWD ? in2 : in1, N, T, C, CC, TT)) != SSB_OK) return rc;
    if ((rc = make_cl_map(&mo1, out1, N, T, C, CC, TT)) != SSB_OK) return rc;
    if ((rc = make_cl_map(&mo2, BWD ? out2 : out1, N, T, C, CC, TT)) != SSB_OK) return rc;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(cl_tma_kernel)");
    static std::atomic<int> cached_occ{0};  // one per instantiation of this function template
    int occ = cached_occ.load(std::memory_order_relaxed);
    if (occ == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, Cfg::THREADS, Cfg::SMEM_BYTES) != cudaSuccess || occ <= 0) {
            (void)cudaGetLastError();
            occ = 1;
        }
        cached_occ.store(occ, std::memory_order_relaxed);
    }
    const int64_t grid_cap = (int64_t)sm_count() * occ;
    ssb::lookback::Order order;
    order.rows = N * geo.cgroups;
    order.pieces = geo.pieces;
    int64_t k = (grid_cap + order.rows - 1) / order.rows;
    if (k < 1) k = 1;
    if (k > order.pieces) k = order.pieces;
    order.k = k;
    order.wave = order.rows * k;
    const int64_t tickets = ((order.pieces + k - 1) / k) * order.wave;
    const int grid = (int)(tickets < grid_cap ? tickets : grid_cap);
    if (cudaMemsetAsync(workspace, 0, ssb::cl3::maps_offset(geo.n_tiles), st) != cudaSuccess)
        return check_launch("cudaMemsetAsync(workspace)");
    kern<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(mg, m1, m2, mo1, mo2, geo, order, static_cast<unsigned char *>(workspace));
    return check_launch("cl_tma_kernel");
}

// Narrow channels-last tensors (C = 4, 8 or 16): a CTA walks a whole batch element, tiles move as
// untiled bulk copies.  Forward: runs of 15 steps, two stages, two staging slots (180 KB); backward:
// runs of 11 steps, two stages, one staging slot (176 KB).
bool cl_narrow_eligible(int64_t N, int64_t T, int64_t C, bool all_aligned16) {
    return all_aligned16 && (C == 4 || C == 8 || C == 16) && N >= 1 && T >= 1 && N <= 0x7fffffffLL;
}

template <int CG, bool BWD>
int launch_cl_narrow_cg(const float *gate, const float *in1, const float *in2, float *out1, float *out2, int64_t N, int64_t T,
                        cudaStream_t st) {
    constexpr int TS = BWD ? 11 : 15, OUTBUF = BWD ? 1 : 2;
    using Cfg = ssb::cln::Config<CG, TS, 4, 2, OUTBUF, BWD>;
    auto kern = ssb::cln::cl_narrow_kernel<CG, TS, 4, 2, OUTBUF, BWD>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
        return check_launch("cudaFuncSetAttribute(cl_narrow_kernel)");
    static std::atomic<int> cached_occ{0};  // one per instantiation of this function template
    int occ = cached_occ.load(std::memory_order_relaxed);
    if (occ == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, Cfg::THREADS, Cfg::SMEM_BYTES) != cudaSuccess || occ <= 0) {
            (void)cudaGetLastError();
            occ = 1;
        }
        cached_occ.store(occ, std::memory_order_relaxed);
    }
    const int64_t cap = (int64_t)sm_count() * occ;
    kern<<<(int)(N < cap ? N : cap), Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(gate, in1, in2, out1, out2, N, T);
    return check_launch("cl_narrow_kernel");
}

template <bool BWD>
int launch_cl_narrow(const float *gate, const float *in1, const float *in2, float *out1, float *out2, int64_t N, int64_t T,
                     int64_t C, cudaStream_t st) {
    switch (C) {
        case 4: return launch_cl_narrow_cg<1, BWD>(gate, in1, in2, out1, out2, N, T, st);
        case 8: return launch_cl_narrow_cg<2, BWD>(gate, in1, in2, out1, out2, N, T, st);
        case 16: return launch_cl_narrow_cg<4, BWD>(gate, in1, in2, out1, out2, N, T, st);
        default: return fail(SSB_ERR_UNSUPPORTED, "the narrow channels-last kernels take C = 4, 8 or 16 (C=%lld)", (long long)C);
    }
}

template <typename real>
int cl_fwd(const real *gate, const real *value, real *out, int64_t N, int64_t T, int64_t C, void *stream) {
    int64_t n;
    int rc = check_cl(N, T, C, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate || !value || !out) return fail(SSB_ERR_BAD_ARG, "ssb_scan_cl_fwd: NULL tensor pointer");
    if (!aligned_to(gate, sizeof(real)) || !aligned_to(value, sizeof(real)) || !aligned_to(out, sizeof(real)))
        return fail(SSB_ERR_ALIGNMENT, "ssb_scan_cl_fwd: pointers must be aligned to the element size");
    const int grid = (int)(N * ((C + 31) / 32));
    ssb::cl_fwd_kernel<real, kClWarps, kClSteps><<<grid, kClWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(gate, value, out, N, T, C);
    return check_launch("cl_fwd_kernel");
}

template <typename real>
int cl_bwd(const real *gate, const real *h, const real *gout, real *ggate, real *gvalue, int64_t N, int64_t T,
           int64_t C, void *stream) {
    int64_t n;
    int rc = check_cl(N, T, C, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate || !h || !gout || !ggate || !gvalue) return fail(SSB_ERR_BAD_ARG, "ssb_scan_cl_bwd: NULL tensor pointer");
    if (!aligned_to(gate, sizeof(real)) || !aligned_to(h, sizeof(real)) || !aligned_to(gout, sizeof(real)) ||
        !aligned_to(ggate, sizeof(real)) || !aligned_to(gvalue, sizeof(real)))
        return fail(SSB_ERR_ALIGNMENT, "ssb_scan_cl_bwd: pointers must be aligned to the element size");
    const int grid = (int)(N * ((C + 31) / 32));
    ssb::cl_bwd_kernel<real, kClWarps, kClSteps><<<grid, kClWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(gate, h, gout, ggate, gvalue, N, T, C);
    return check_launch("cl_bwd_kernel");
}
}  // namespace

namespace {
int cl_family_of(int variant) { return variant & 0xff; }
int cl_tuning_of(int variant) { return (variant >> 8) & 0xff; }
bool cl_scalar_lanes(int variant) { return ((variant >> 16) & 1) != 0; }

// Whether the streaming kernels apply to this shape: they need a TMA-describable tensor, rows long
// enough to fill their 128-256 step tiles, and enough (batch element, 32-channel block) pairs to
// occupy the GPU without splitting T (measured on B200: from 96 pairs; below that the chunked and
// look-back forms win).
bool cl_stream_shape(int64_t N, int64_t T, int64_t C, bool all_aligned16) {
    return all_aligned16 && cl3_eligible(N, T, C) && T >= 128 && encode_fn() != nullptr && N * ((C + 31) / 32) >= 96;
}

// Which streaming tile shape (tuning id of SSB_CLS_CONFIGS) a direction gets, -1 = none.  A unit is
// all of T for one (batch element, channel block); units run in rounds over the resident CTAs and
// the last round is rarely full, so the choice goes by an estimate of rounds x cost of a round:
//   id 0  32-channel blocks, one CTA per SM;
//   id 1  64-channel blocks, one CTA per SM: half the units, a round costs 1.81 (forward) / 1.93
//         (backward) rounds of id 0 -- it wins when that halves the number of rounds;
//   id 2  32-channel blocks; forward: 128-step tiles, two CTAs per SM, used where one round of it
//         covers units that id 0 needs two rounds for (up to 1.5 units per SM); backward: 256-step
//         tiles, one stage: ahead of id 0 on every measured shape with more units than SMs.
// "Rounds" = the mean of units / slots and its ceiling: CTAs of a part-filled round run faster,
// they share the memory system with fewer others.  Fitted on [6...96, 2048...8192, 512...1024]
// (12 shapes, 96 ... 1536 units of 32 channels); the choice is the best or within 3 % of the best
// pinned id on each of them.
double cl_rounds(int64_t units, int64_t slots) {
    return 0.5 * ((double)units / (double)slots + (double)((units + slots - 1) / slots));
}
int cl_stream_id(bool backward, int64_t N, int64_t T, int64_t C, bool all_aligned16) {
    if (!cl_stream_shape(N, T, C, all_aligned16)) return -1;
    const int64_t sms = sm_count(), p32 = N * ((C + 31) / 32), p64 = N * ((C + 63) / 64);
    int id = (backward && p32 > sms) ? 2 : 0;
    double best = cl_rounds(p32, sms);
    if (!backward && p32 > sms && 2 * p32 <= 3 * sms && 1.72 * cl_rounds(p32, 2 * sms) < best) {
        best = 1.72 * cl_rounds(p32, 2 * sms);
        id = 2;
    }
    if (T >= 1024 && (C % 64 == 0 || C >= 512) && (backward ? 1.93 : 1.81) * cl_rounds(p64, sms) < best) id = 1;
    return id;
}

// Too few pairs for the above but long rows: the same kernels over chunks of T in two passes
// (measured 1.3-4x the look-back kernels from 2048 steps up).  Needs scratch.
bool cl_chunked_shape(int64_t N, int64_t T, int64_t C, bool all_aligned16) {
    return all_aligned16 && cl3_eligible(N, T, C) && T >= 2048 && encode_fn() != nullptr;
}

// Measured on B200: splitting T across CTAs pays when the plain kernels cannot fill the GPU
// (fewer than ~96 groups of 32 channels) or when there are at least 64 groups of 128 channels
// to keep the look-back chains short; with very few channels per row the 4-channel lanes of
// the look-back kernels are mostly idle and the plain kernels win.
bool cl_prefers_lookback(int64_t N, int64_t C) {
    if (C < 64) return false;
    const int64_t groups32 = N * ((C + 31) / 32), groups128 = N * ((C + 127) / 128);
    return groups128 >= 64 || groups32 < 96;
}

// Steps per tile of look-back tuning id `id` (0 = unknown id).
int cl2_tile_steps(int id, bool backward) {
    switch (id) {
#define X(ID, WW, LF, LB) case ID: return WW * (backward ? LB : LF);
        SSB_CL2_CONFIGS(X)
#undef X
        default: return 0;
    }
}
int cl3_tile_steps(int id, bool backward, int *cc) {
    switch (id) {
#define X(ID, FC, FT, FS, FO, BC, BT, BS, BO) case ID: *cc = backward ? BC : FC; return backward ? BT : FT;
        SSB_CL3_CONFIGS(X)
#undef X
        default: *cc = 0; return 0;
    }
}

// Scratch a look-back variant needs: one record per tile.
size_t cl2_need(int64_t N, int64_t T, int64_t C, int id, bool backward, bool vec) {
    const int steps = cl2_tile_steps(id, backward);
    if (steps == 0) return 0;
    const int v = vec ? 4 : 1;
    return ssb::cl2::workspace_bytes(N * ((C + 32 * v - 1) / (32 * v)) * ((T + steps - 1) / steps), v);
}
size_t cl3_need(int64_t N, int64_t T, int64_t C, int id, bool backward) {
    int cc = 0;
    const int steps = cl3_tile_steps(id, backward, &cc);
    if (steps == 0) return 0;
    return ssb::cl3::workspace_bytes(N * ((C + cc - 1) / cc) * ((T + steps - 1) / steps), cc);
}

// The choice SSB_CL_VARIANT_AUTO makes, given `ws_avail` bytes of usable scratch.
int cl_pick(bool backward, int64_t N, int64_t T, int64_t C, bool all_aligned16, size_t ws_avail) {
    // a handful of channels: whole batch elements per CTA, once there are enough of them to occupy the GPU
    if (cl_narrow_eligible(N, T, C, all_aligned16) && N >= 64 && T >= 64) return SSB_CL_VARIANT_NARROW;
    const int stream_id = cl_stream_id(backward, N, T, C, all_aligned16);
    if (stream_id >= 0) return SSB_CL_VARIANT_STREAM | (stream_id << 8);
    if (cl_chunked_shape(N, T, C, all_aligned16) && ws_avail >= cls_chunk_workspace_bytes(N, T, C)) return SSB_CL_VARIANT_CHUNKED;
    const bool vec = C % 4 == 0 && all_aligned16;
    if (cl_prefers_lookback(N, C) && ws_avail > 0 && ws_avail >= cl2_need(N, T, C, 0, backward, vec)) return SSB_CL_VARIANT_LOOKBACK;
    return SSB_CL_VARIANT_PLAIN;
}

template <bool BWD>
int cl_f32_ex(const float *gate, const float *in1, const float *in2, float *out1, float *out2, int64_t N, int64_t T, int64_t C,
              int variant, void *workspace, size_t workspace_bytes, void *stream, const char *who) {
    int64_t n;
    int rc = check_cl(N, T, C, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate || !in1 || !out1 || (BWD && (!in2 || !out2))) return fail(SSB_ERR_BAD_ARG, "%s: NULL tensor pointer", who);
    if (!aligned_to(gate, 4) || !aligned_to(in1, 4) || !aligned_to(in2, 4) || !aligned_to(out1, 4) || !aligned_to(out2, 4))
        return fail(SSB_ERR_ALIGNMENT, "%s: pointers must be 4-byte aligned", who);
    const bool al16 = aligned_to(gate, 16) && aligned_to(in1, 16) && aligned_to(in2, 16) && aligned_to(out1, 16) &&
                      aligned_to(out2, 16);
    const size_t ws_avail = (workspace != nullptr && aligned_to(workspace, 256)) ? workspace_bytes : 0;
    if (cl_family_of(variant) == SSB_CL_VARIANT_AUTO) variant = cl_pick(BWD, N, T, C, al16, ws_avail);
    const int id = cl_tuning_of(variant);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool tma_ok = al16 && cl3_eligible(N, T, C) && encode_fn() != nullptr;
    switch (cl_family_of(variant)) {
        case SSB_CL_VARIANT_PLAIN:
            if (!BWD) return cl_fwd<float>(gate, in1, out1, N, T, C, stream);
            return cl_bwd<float>(gate, in1, in2, out1, out2, N, T, C, stream);
        case SSB_CL_VARIANT_NARROW:
            if (!cl_narrow_eligible(N, T, C, al16))
                return fail(SSB_ERR_UNSUPPORTED, "%s: the narrow kernels need C = 4, 8 or 16 and 16-byte aligned tensors (C=%lld)", who, (long long)C);
            return launch_cl_narrow<BWD>(gate, in1, in2, out1, out2, N, T, C, st);
        case SSB_CL_VARIANT_STREAM:
            if (!tma_ok) return fail(SSB_ERR_UNSUPPORTED, "%s: the streaming kernels need C %% 4 == 0 and 16-byte aligned tensors", who);
            switch (id) {
#define X(ID, FC, FT, FG, FS, FO, BC, BT, BG, BS, BO)                                                              \
    case ID:                                                                                                        \
        if constexpr (!BWD) return launch_cls<FC, FT, FG, FS, FO, false>(gate, in1, nullptr, out1, nullptr, N, T, C, st); \
        else return launch_cls<BC, BT, BG, BS, BO, true>(gate, in1, in2, out1, out2, N, T, C, st);
                SSB_CLS_CONFIGS(X)
#undef X
                default: return fail(SSB_ERR_UNSUPPORTED, "%s: unknown streaming tuning id %d", who, id);
            }
        case SSB_CL_VARIANT_CHUNKED:
            if (!tma_ok) return fail(SSB_ERR_UNSUPPORTED, "%s: the chunked streaming form needs C %% 4 == 0 and 16-byte aligned tensors", who);
            if (ws_avail < cls_chunk_workspace_bytes(N, T, C))
                return fail(SSB_ERR_WORKSPACE, "%s: the chunked streaming form needs a 256-byte aligned workspace of %zu bytes (got %zu)",
                            who, cls_chunk_workspace_bytes(N, T, C), ws_avail);
            return launch_cls_chunked<BWD>(gate, in1, in2, out1, out2, N, T, C, workspace, workspace_bytes, st);
        case SSB_CL_VARIANT_LOOKBACK_TMA:
            if (!tma_ok) return fail(SSB_ERR_UNSUPPORTED, "%s: the TMA look-back kernels need C %% 4 == 0 and 16-byte aligned tensors", who);
            if (ws_avail == 0) return fail(SSB_ERR_WORKSPACE, "%s: look-back needs a 256-byte aligned workspace", who);
            switch (id) {
#define X(ID, FC, FT, FS, FO, BC, BT, BS, BO)                                                                                        \
    case ID:                                                                                                                          \
        if constexpr (!BWD) return launch_cl3<FC, FT, FS, FO, false>(gate, in1, nullptr, out1, nullptr, N, T, C, workspace, workspace_bytes, st); \
        else return launch_cl3<BC, BT, BS, BO, true>(gate, in1, in2, out1, out2, N, T, C, workspace, workspace_bytes, st);
                SSB_CL3_CONFIGS(X)
#undef X
                default: return fail(SSB_ERR_UNSUPPORTED, "%s: unknown TMA look-back tuning id %d", who, id);
            }
        case SSB_CL_VARIANT_LOOKBACK: {
            if (ws_avail == 0) return fail(SSB_ERR_WORKSPACE, "%s: look-back needs a 256-byte aligned workspace", who);
            const bool vec = C % 4 == 0 && al16 && !cl_scalar_lanes(variant);
            switch (id) {
#define X(ID, WW, LF, LB)                                                                                                          \
    case ID:                                                                                                                        \
        if constexpr (!BWD)                                                                                                         \
            return vec ? launch_cl2<4, WW, LF, false>(gate, in1, nullptr, out1, nullptr, N, T, C, workspace, workspace_bytes, st)   \
                       : launch_cl2<1, WW, LF, false>(gate, in1, nullptr, out1, nullptr, N, T, C, workspace, workspace_bytes, st);  \
        else                                                                                                                        \
            return vec ? launch_cl2<4, WW, LB, true>(gate, in1, in2, out1, out2, N, T, C, workspace, workspace_bytes, st)           \
                       : launch_cl2<1, WW, LB, true>(gate, in1, in2, out1, out2, N, T, C, workspace, workspace_bytes, st);
                SSB_CL2_CONFIGS(X)
#undef X
                default: return fail(SSB_ERR_UNSUPPORTED, "%s: unknown look-back tuning id %d", who, id);
            }
        }
        default:
            return fail(SSB_ERR_UNSUPPORTED, "%s: channels-last variant %d is not available", who, variant);
    }
}
}  // namespace

extern "C" {

int ssb_scan_cl_fwd_f32(const float *gate, const float *value, float *out, int64_t N, int64_t T, int64_t C, void *stream) {
    return cl_f32_ex<false>(gate, value, nullptr, out, nullptr, N, T, C, SSB_CL_VARIANT_AUTO, nullptr, 0, stream, "ssb_scan_cl_fwd_f32");
}

int ssb_scan_cl_recommend(int64_t N, int64_t T, int64_t C, int backward, int aligned16, int can_provide_workspace) {
    if (N <= 0 || T <= 0 || C <= 0) return SSB_CL_VARIANT_PLAIN;
    return cl_pick(backward != 0, N, T, C, aligned16 != 0, can_provide_workspace ? std::numeric_limits<size_t>::max() : 0);
}

size_t ssb_scan_cl_variant_workspace_bytes(int64_t N, int64_t T, int64_t C, int variant, int backward) {
    if (N <= 0 || T <= 0 || C <= 0) return 0;
    switch (cl_family_of(variant)) {
        case SSB_CL_VARIANT_CHUNKED: return C % 4 == 0 ? cls_chunk_workspace_bytes(N, T, C) : 0;
        case SSB_CL_VARIANT_LOOKBACK:  // the caller's alignment is unknown here: the larger of the two lane widths
            return std::max(cl2_need(N, T, C, cl_tuning_of(variant), backward != 0, false),
                            (C % 4 == 0 && !cl_scalar_lanes(variant)) ? cl2_need(N, T, C, cl_tuning_of(variant), backward != 0, true) : 0);
        case SSB_CL_VARIANT_LOOKBACK_TMA: return cl3_need(N, T, C, cl_tuning_of(variant), backward != 0);
        default: return 0;
    }
}

size_t ssb_scan_cl_workspace_bytes(int64_t N, int64_t T, int64_t C) {
    if (N <= 0 || T <= 0 || C <= 0) return 0;
    size_t need = 0;
    for (int vec : {1, 4}) {
        const int64_t tiles = N * ((C + 32 * vec - 1) / (32 * vec)) * ((T + kCl2MinTile - 1) / kCl2MinTile);
        const size_t b = ssb::cl2::workspace_bytes(tiles, vec);
        need = b > need ? b : need;
    }
    if (C % 4 == 0) {  // chunked streaming: maps and carries of every chunk
        const size_t b = cls_chunk_workspace_bytes(N, T, C);
        need = b > need ? b : need;
    }
    for (int cc : {32, 64, 128}) {  // TMA-staged tiles: at least kCl3MinTileElems elements each
        const int tt = kCl3MinTileElems / cc;
        const int64_t tiles = N * ((C + cc - 1) / cc) * ((T + tt - 1) / tt);
        const size_t b = ssb::cl3::workspace_bytes(tiles, cc);
        need = b > need ? b : need;
    }
    return need;
}

int ssb_scan_cl_fwd_f32_ex(const float *gate, const float *value, float *out, int64_t N, int64_t T, int64_t C, int variant,
                           void *workspace, size_t workspace_bytes, void *stream) {
    return cl_f32_ex<false>(gate, value, nullptr, out, nullptr, N, T, C, variant, workspace, workspace_bytes, stream,
                            "ssb_scan_cl_fwd_f32_ex");
}

int ssb_scan_cl_bwd_f32_ex(const float *gate, const float *h, const float *gout, float *ggate, float *gvalue, int64_t N,
                           int64_t T, int64_t C, int variant, void *workspace, size_t workspace_bytes, void *stream) {
    return cl_f32_ex<true>(gate, h, gout, ggate, gvalue, N, T, C, variant, workspace, workspace_bytes, stream,
                           "ssb_scan_cl_bwd_f32_ex");
}
}  // extern "C"

// ---- channels-last, 16-bit storage (bf16 / fp16 tensors, fp32 arithmetic) ---------------------
namespace {
bool cl_h16_eligible(int64_t N, int64_t T, int64_t C) {
    return C % 8 == 0 && N <= 0x7fffffffLL && T <= 0x7fffff00LL && C <= 0x7fffffffLL && T <= ((1LL << 40) - 1) / 2 / C;
}

// Whole-T units run in rounds over the resident CTAs, and the last round is rarely full.  The
// 256-step tiles (512 threads) keep one CTA per SM: rounds of 148.  The 128-step tiles (128 threads,
// half the shared memory) keep two: rounds of 296 that take 1.65-1.85 times as long (measured on
// 160 ... 1024 pairs of 64 channels: the factor is lower where the sigmoid adds arithmetic for the
// second CTA to hide).  Take the smaller estimate; beyond ~1200 pairs the difference is noise.
bool cl_h16_small_tiles(int64_t pairs, bool backward, bool sigmoid) {
    const int64_t sms = sm_count();
    if (pairs <= sms || pairs > 8 * sms) return false;
    const double factor = !sigmoid ? 1.85 : (backward ? 1.65 : 1.8);
    const double one = (double)((pairs + sms - 1) / sms), two = (double)((pairs + 2 * sms - 1) / (2 * sms)) * factor;
    return two < one;
}

template <typename IO, bool BWD, bool SIGMOID = false>
int cl_h16(const void *gate_, const void *in1_, const void *in2_, void *out1_, void *out2_, int64_t N, int64_t T, int64_t C,
           void *workspace, size_t workspace_bytes, void *stream, const char *who) {
    int64_t n;
    int rc = check_cl(N, T, C, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate_ || !in1_ || (BWD && !in2_) || !out1_ || (BWD && !out2_)) return fail(SSB_ERR_BAD_ARG, "%s: NULL tensor pointer", who);
    const bool al16 = aligned_to(gate_, 16) && aligned_to(in1_, 16) && aligned_to(in2_, 16) && aligned_to(out1_, 16) &&
                      aligned_to(out2_, 16);
    if (!al16 || !cl_h16_eligible(N, T, C) || encode_fn() == nullptr)
        return fail(SSB_ERR_UNSUPPORTED, "%s needs C %% 8 == 0 and 16-byte aligned tensors (C=%lld)", who, (long long)C);
    const IO *gate = static_cast<const IO *>(gate_), *in1 = static_cast<const IO *>(in1_), *in2 = static_cast<const IO *>(in2_);
    IO *out1 = static_cast<IO *>(out1_), *out2 = static_cast<IO *>(out2_);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t pairs = N * ((C + 63) / 64);
    if (pairs < 96 && T >= 2048 && workspace != nullptr && aligned_to(workspace, 256) &&
        workspace_bytes >= cls_chunk_workspace_bytes(N, T, C, 64))
        return launch_cls_chunked<BWD, IO, SIGMOID>(gate, in1, in2, out1, out2, N, T, C, workspace, workspace_bytes, st);
    if (cl_h16_small_tiles(pairs, BWD, SIGMOID)) {
        if (!BWD) return launch_cls<64, 128, 8, 2, 2, false, IO, SIGMOID>(gate, in1, nullptr, out1, nullptr, N, T, C, st);
        return launch_cls<64, 128, 8, 1, 1, true, IO, SIGMOID>(gate, in1, in2, out1, out2, N, T, C, st);
    }
    if (!BWD) return launch_cls<64, 256, 16, 2, 2, false, IO, SIGMOID>(gate, in1, nullptr, out1, nullptr, N, T, C, st);
    return launch_cls<64, 256, 16, 1, 1, true, IO, SIGMOID>(gate, in1, in2, out1, out2, N, T, C, st);  // from a sweep of 42 shapes
}
}  // namespace

extern "C" {

size_t ssb_scan_cl_h16_workspace_bytes(int64_t N, int64_t T, int64_t C) {
    if (N <= 0 || T <= 0 || C <= 0 || N * ((C + 63) / 64) >= 96 || T < 2048 || !cl_h16_eligible(N, T, C)) return 0;
    return cls_chunk_workspace_bytes(N, T, C, 64);
}
int ssb_scan_cl_fwd_bf16(const void *gate, const void *value, void *out, int64_t N, int64_t T, int64_t C, void *workspace,
                         size_t workspace_bytes, void *stream) {
    return cl_h16<__nv_bfloat16, false>(gate, value, nullptr, out, nullptr, N, T, C, workspace, workspace_bytes, stream,
                                        "ssb_scan_cl_fwd_bf16");
}
int ssb_scan_cl_bwd_bf16(const void *gate, const void *h, const void *gout, void *ggate, void *gvalue, int64_t N, int64_t T,
                         int64_t C, void *workspace, size_t workspace_bytes, void *stream) {
    return cl_h16<__nv_bfloat16, true>(gate, h, gout, ggate, gvalue, N, T, C, workspace, workspace_bytes, stream,
                                       "ssb_scan_cl_bwd_bf16");
}
int ssb_scan_cl_fwd_f16(const void *gate, const void *value, void *out, int64_t N, int64_t T, int64_t C, void *workspace,
                        size_t workspace_bytes, void *stream) {
    return cl_h16<__half, false>(gate, value, nullptr, out, nullptr, N, T, C, workspace, workspace_bytes, stream,
                                 "ssb_scan_cl_fwd_f16");
}
int ssb_scan_cl_bwd_f16(const void *gate, const void *h, const void *gout, void *ggate, void *gvalue, int64_t N, int64_t T,
                        int64_t C, void *workspace, size_t workspace_bytes, void *stream) {
    return cl_h16<__half, true>(gate, h, gout, ggate, gvalue, N, T, C, workspace, workspace_bytes, stream, "ssb_scan_cl_bwd_f16");
}

// Gate logits in, channels-last (the sigmoid and its derivative computed in the streaming kernels).
int ssb_scan_cl_sigmoid_fwd_bf16(const void *gate_logits, const void *value, void *out, int64_t N, int64_t T, int64_t C,
                                 void *workspace, size_t workspace_bytes, void *stream) {
    return cl_h16<__nv_bfloat16, false, true>(gate_logits, value, nullptr, out, nullptr, N, T, C, workspace, workspace_bytes,
                                              stream, "ssb_scan_cl_sigmoid_fwd_bf16");
}
int ssb_scan_cl_sigmoid_bwd_bf16(const void *gate_logits, const void *h, const void *gout, void *glogits, void *gvalue,
                                 int64_t N, int64_t T, int64_t C, void *workspace, size_t workspace_bytes, void *stream) {
    return cl_h16<__nv_bfloat16, true, true>(gate_logits, h, gout, glogits, gvalue, N, T, C, workspace, workspace_bytes, stream,
                                             "ssb_scan_cl_sigmoid_bwd_bf16");
}
int ssb_scan_cl_sigmoid_fwd_f16(const void *gate_logits, const void *value, void *out, int64_t N, int64_t T, int64_t C,
                                void *workspace, size_t workspace_bytes, void *stream) {
    return cl_h16<__half, false, true>(gate_logits, value, nullptr, out, nullptr, N, T, C, workspace, workspace_bytes, stream,
                                       "ssb_scan_cl_sigmoid_fwd_f16");
}
int ssb_scan_cl_sigmoid_bwd_f16(const void *gate_logits, const void *h, const void *gout, void *glogits, void *gvalue,
                                int64_t N, int64_t T, int64_t C, void *workspace, size_t workspace_bytes, void *stream) {
    return cl_h16<__half, true, true>(gate_logits, h, gout, glogits, gvalue, N, T, C, workspace, workspace_bytes, stream,
                                      "ssb_scan_cl_sigmoid_bwd_f16");
}

}  // extern "C"

namespace {
template <bool BWD>
int cl_sigmoid_f32(const float *gate, const float *in1, const float *in2, float *out1, float *out2, int64_t N, int64_t T,
                   int64_t C, void *workspace, size_t workspace_bytes, void *stream, const char *who) {
    int64_t n;
    int rc = check_cl(N, T, C, &n);
    if (rc != SSB_OK) return rc;
    if (n == 0) return SSB_OK;
    if (!gate || !in1 || (BWD && !in2) || !out1 || (BWD && !out2)) return fail(SSB_ERR_BAD_ARG, "%s: NULL tensor pointer", who);
    const bool al16 = aligned_to(gate, 16) && aligned_to(in1, 16) && aligned_to(in2, 16) && aligned_to(out1, 16) &&
                      aligned_to(out2, 16);
    if (!al16 || !cl3_eligible(N, T, C) || encode_fn() == nullptr)
        return fail(SSB_ERR_UNSUPPORTED, "%s needs C %% 4 == 0 and 16-byte aligned tensors (C=%lld)", who, (long long)C);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!cl_stream_shape(N, T, C, true) && cl_chunked_shape(N, T, C, true) && workspace != nullptr &&
        aligned_to(workspace, 256) && workspace_bytes >= cls_chunk_workspace_bytes(N, T, C))
        return launch_cls_chunked<BWD, float, true>(gate, in1, in2, out1, out2, N, T, C, workspace, workspace_bytes, st);
    switch (cl_stream_id(BWD, N, T, C, true)) {  // the tile shapes of SSB_CLS_CONFIGS ids 1, 2, 0
        case 1:
            if (!BWD) return launch_cls<64, 256, 16, 1, 1, false, float, true>(gate, in1, nullptr, out1, nullptr, N, T, C, st);
            return launch_cls<64, 128, 8, 1, 1, true, float, true>(gate, in1, in2, out1, out2, N, T, C, st);
        case 2:
            if (!BWD) return launch_cls<32, 128, 16, 2, 2, false, float, true>(gate, in1, nullptr, out1, nullptr, N, T, C, st);
            return launch_cls<32, 256, 16, 1, 1, true, float, true>(gate, in1, in2, out1, out2, N, T, C, st);
        default:
            if (!BWD) return launch_cls<32, 256, 16, 2, 2, false, float, true>(gate, in1, nullptr, out1, nullptr, N, T, C, st);
            return launch_cls<32, 128, 16, 2, 1, true, float, true>(gate, in1, in2, out1, out2, N, T, C, st);
    }
}
}  // namespace

extern "C" {

size_t ssb_scan_cl_sigmoid_workspace_bytes(int64_t N, int64_t T, int64_t C) {
    if (N <= 0 || T <= 0 || C <= 0 || cl_stream_shape(N, T, C, true) || !cl_chunked_shape(N, T, C, true)) return 0;
    return cls_chunk_workspace_bytes(N, T, C);
}

int ssb_scan_cl_sigmoid_fwd_f32(const float *gate_logits, const float *value, float *out, int64_t N, int64_t T, int64_t C,
                                void *workspace, size_t workspace_bytes, void *stream) {
    return cl_sigmoid_f32<false>(gate_logits, value, nullptr, out, nullptr, N, T, C, workspace, workspace_bytes, stream,
                                 "ssb_scan_cl_sigmoid_fwd_f32");
}
int ssb_scan_cl_sigmoid_bwd_f32(const float *gate_logits, const float *h, const float *gout, float *glogits, float *gvalue,
                                int64_t N, int64_t T, int64_t C, void *workspace, size_t workspace_bytes, void *stream) {
    return cl_sigmoid_f32<true>(gate_logits, h, gout, glogits, gvalue, N, T, C, workspace, workspace_bytes, stream,
                                "ssb_scan_cl_sigmoid_bwd_f32");
}

int ssb_scan_cl_fwd_f64(const double *gate, const double *value, double *out, int64_t N, int64_t T, int64_t C, void *stream) {
    return cl_fwd<double>(gate, value, out, N, T, C, stream);
}
int ssb_scan_cl_bwd_f32(const float *gate, const float *h, const float *gout, float *ggate, float *gvalue, int64_t N,
                        int64_t T, int64_t C, void *stream) {
    return cl_f32_ex<true>(gate, h, gout, ggate, gvalue, N, T, C, SSB_CL_VARIANT_AUTO, nullptr, 0, stream, "ssb_scan_cl_bwd_f32");
}
int ssb_scan_cl_bwd_f64(const double *gate, const double *h, const double *gout, double *ggate, double *gvalue,
                        int64_t N, int64_t T, int64_t C, void *stream) {
    return cl_bwd<double>(gate, h, gout, ggate, gvalue, N, T, C, stream);
}

// ---- sequence sharding -----------------------------------------------------------------
int ssb_shard_reduce_fwd_f32(const float *gate, const float *value, float *agg, int64_t rows, int64_t T,
                             void *workspace, size_t workspace_bytes, void *stream) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (rows == 0) return SSB_OK;
    if (!agg || (n > 0 && (!gate || !value))) return fail(SSB_ERR_BAD_ARG, "ssb_shard_reduce_fwd_f32: NULL pointer");
    if (!aligned_to(gate, 4) || !aligned_to(value, 4) || !aligned_to(agg, 4))
        return fail(SSB_ERR_ALIGNMENT, "ssb_shard_reduce_fwd_f32: pointers must be 4-byte aligned");
    const size_t need = span_maps_bytes(rows, T);
    if (workspace != nullptr && need > 0 && workspace_bytes >= need && aligned_to(workspace, 16) && aligned_to(gate, 16) &&
        aligned_to(value, 16))
        return launch_span_maps<false>(gate, value, agg, rows, T, workspace, static_cast<cudaStream_t>(stream));
    return launch_warp_fwd<float, true>(gate, value, nullptr, rows, T, nullptr, agg, static_cast<cudaStream_t>(stream));
}

int ssb_shard_reduce_bwd_f32(const float *gate, const float *gout, float *agg, int64_t rows, int64_t T,
                             void *workspace, size_t workspace_bytes, void *stream) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (rows == 0) return SSB_OK;
    if (!agg || (n > 0 && (!gate || !gout))) return fail(SSB_ERR_BAD_ARG, "ssb_shard_reduce_bwd_f32: NULL pointer");
    if (!aligned_to(gate, 4) || !aligned_to(gout, 4) || !aligned_to(agg, 4))
        return fail(SSB_ERR_ALIGNMENT, "ssb_shard_reduce_bwd_f32: pointers must be 4-byte aligned");
    const size_t need = span_maps_bytes(rows, T);
    if (workspace != nullptr && need > 0 && workspace_bytes >= need && aligned_to(workspace, 16) && aligned_to(gate, 16) &&
        aligned_to(gout, 16))
        return launch_span_maps<true>(gate, gout, agg, rows, T, workspace, static_cast<cudaStream_t>(stream));
    return launch_warp_bwd<float, true>(gate, nullptr, gout, nullptr, nullptr, rows, T, nullptr, nullptr, agg,
                                        static_cast<cudaStream_t>(stream));
}

int ssb_shard_carry_f32(const float *aggs, int n_shards, int shard, int reverse, int64_t rows, float *carry, void *stream) {
    if (rows < 0 || n_shards < 1 || shard < 0 || shard >= n_shards)
        return fail(SSB_ERR_BAD_ARG, "ssb_shard_carry_f32: bad shard %d of %d or rows=%lld", shard, n_shards, (long long)rows);
    if (rows == 0) return SSB_OK;
    if (!aggs || !carry) return fail(SSB_ERR_BAD_ARG, "ssb_shard_carry_f32: NULL pointer");
    const int block = 256;
    const int64_t grid = (rows + block - 1) / block;
    if (grid > 0x7fffffffLL) return fail(SSB_ERR_BAD_ARG, "ssb_shard_carry_f32: too many rows");
    ssb::shard_carry_kernel<float><<<(int)grid, block, 0, static_cast<cudaStream_t>(stream)>>>(aggs, n_shards, shard, reverse, rows, carry);
    return check_launch("shard_carry_kernel");
}

}  // extern "C"

namespace {

template <bool BWD>
int shard_map(const float *gate, const float *in1, float *agg, int64_t rows, int64_t T, float cut,
              unsigned long long *walked, void *stream, const char *who) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    if (rows == 0) return SSB_OK;
    if (!agg || (n > 0 && (!gate || !in1))) return fail(SSB_ERR_BAD_ARG, "%s: NULL pointer", who);
    if (!aligned_to(gate, 4) || !aligned_to(in1, 4) || !aligned_to(agg, 4) || !aligned_to(walked, 8))
        return fail(SSB_ERR_ALIGNMENT, "%s: tensors must be 4-byte aligned, the counter 8-byte aligned", who);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (T == 0 || T % 4 != 0 || !aligned_to(gate, 16) || !aligned_to(in1, 16)) {  // full reduction, one warp per row
        if (walked != nullptr && n > 0) {
            ssb::shard::add_counter_kernel<<<1, 1, 0, st>>>(walked, (unsigned long long)n);
            if ((rc = check_launch("add_counter_kernel")) != SSB_OK) return rc;
        }
        return BWD ? launch_warp_bwd<float, true>(gate, nullptr, in1, nullptr, nullptr, rows, T, nullptr, nullptr, agg, st)
                   : launch_warp_fwd<float, true>(gate, in1, nullptr, rows, T, nullptr, agg, st);
    }
    auto kern = ssb::shard::tail_map_kernel<kTailThreads, kTailU, BWD>;
    const int grid = persistent_grid<600000 + (BWD ? 1 : 0)>(kern, kTailThreads, rows);
    kern<<<grid, kTailThreads, 0, st>>>(reinterpret_cast<const float4 *>(gate), reinterpret_cast<const float4 *>(in1), rows,
                                        T / 4, cut, agg, walked, ssb::shard::PeerExchange(), 0, 0u);
    return check_launch("tail_map_kernel");
}
}  // namespace

extern "C" {

int ssb_shard_map_fwd_f32(const float *gate, const float *value, float *agg, int64_t rows, int64_t T, float cut,
                          unsigned long long *walked, void *stream) {
    return shard_map<false>(gate, value, agg, rows, T, cut, walked, stream, "ssb_shard_map_fwd_f32");
}

int ssb_shard_map_bwd_f32(const float *gate, const float *gout, float *agg, int64_t rows, int64_t T, float cut,
                          unsigned long long *walked, void *stream) {
    return shard_map<true>(gate, gout, agg, rows, T, cut, walked, stream, "ssb_shard_map_bwd_f32");
}

}  // extern "C"

namespace {
int to_peer_exchange(const ssb_peer_exchange_t *ex, ssb::shard::PeerExchange *px, const char *who) {
    if (ex == nullptr || ex->world < 1 || ex->world > ssb::shard::kMaxPeers || ex->rank < 0 || ex->rank >= ex->world || ex->rows < 0)
        return fail(SSB_ERR_BAD_ARG, "%s: bad exchange descriptor (world 1..%d, 0 <= rank < world)", who, ssb::shard::kMaxPeers);
    px->world = ex->world;
    px->rank = ex->rank;
    px->rows = ex->rows;
    for (int r = 0; r < ssb::shard::kMaxPeers; r++) {
        px->buf[r] = r < ex->world ? static_cast<unsigned char *>(ex->buffers[r]) : nullptr;
        if (r < ex->world && (px->buf[r] == nullptr || !aligned_to(px->buf[r], 256)))
            return fail(SSB_ERR_BAD_ARG, "%s: exchange buffer of rank %d is NULL or not 256-byte aligned", who, r);
    }
    return SSB_OK;
}

template <bool BWD>
int shard_map_publish(const float *gate, const float *in1, int64_t rows, int64_t T, float cut, const ssb::shard::PeerExchange &px,
                      unsigned epoch, unsigned long long *walked, cudaStream_t st) {
    auto kern = ssb::shard::tail_map_kernel<kTailThreads, kTailU, BWD, true>;
    const int grid = persistent_grid<610000 + (BWD ? 1 : 0)>(kern, kTailThreads, rows);
    kern<<<grid, kTailThreads, 0, st>>>(reinterpret_cast<const float4 *>(gate), reinterpret_cast<const float4 *>(in1), rows,
                                        T / 4, cut, nullptr, walked, px, (int)(epoch & 1u), epoch);
    return check_launch("tail_map_kernel<publish>");
}
}  // namespace

extern "C" {

size_t ssb_peer_exchange_bytes(int world, int64_t rows) {
    if (world < 1 || world > ssb::shard::kMaxPeers || rows <= 0) return 0;
    return ssb::shard::px_total_bytes(world, rows);
}

static_assert(sizeof(cudaIpcMemHandle_t) == SSB_IPC_HANDLE_BYTES, "the header's handle size is CUDA's");

int ssb_peer_buffer_create(size_t bytes, void **ptr, unsigned char handle[SSB_IPC_HANDLE_BYTES]) {
    if (ptr == nullptr || handle == nullptr || bytes == 0) return fail(SSB_ERR_BAD_ARG, "ssb_peer_buffer_create: NULL argument or zero size");
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return fail(SSB_ERR_LAUNCH, "cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
    cudaIpcMemHandle_t h;
    if ((e = cudaMemset(p, 0, bytes)) != cudaSuccess || (e = cudaDeviceSynchronize()) != cudaSuccess ||
        (e = cudaIpcGetMemHandle(&h, p)) != cudaSuccess) {
        (void)cudaFree(p);
        return fail(SSB_ERR_LAUNCH, "exchange buffer set-up: %s", cudaGetErrorString(e));
    }
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return SSB_OK;
}

int ssb_peer_buffer_open(const unsigned char handle[SSB_IPC_HANDLE_BYTES], void **ptr) {
    if (ptr == nullptr || handle == nullptr) return fail(SSB_ERR_BAD_ARG, "ssb_peer_buffer_open: NULL argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);  // mapped for the CURRENT device
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(SSB_ERR_LAUNCH, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    }
    *ptr = p;
    return SSB_OK;
}

int ssb_peer_buffer_close(void *ptr) {
    if (ptr == nullptr) return SSB_OK;
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(SSB_ERR_LAUNCH, "cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
    }
    return SSB_OK;
}

int ssb_peer_buffer_destroy(void *ptr) {
    if (ptr == nullptr) return SSB_OK;
    cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(SSB_ERR_LAUNCH, "cudaFree: %s", cudaGetErrorString(e));
    }
    return SSB_OK;
}

int ssb_shard_map_publish_f32(const float *gate, const float *other, int64_t rows, int64_t T, float cut, int backward,
                              const ssb_peer_exchange_t *exchange, unsigned epoch, unsigned long long *walked, void *stream) {
    int64_t n;
    int rc = check_shape(rows, T, &n);
    if (rc != SSB_OK) return rc;
    ssb::shard::PeerExchange px;
    if ((rc = to_peer_exchange(exchange, &px, "ssb_shard_map_publish_f32")) != SSB_OK) return rc;
    if (rows != px.rows || rows == 0) return fail(SSB_ERR_BAD_ARG, "ssb_shard_map_publish_f32: rows=%lld, the exchange was made for %lld", (long long)rows, (long long)px.rows);
    if (!gate || !other) return fail(SSB_ERR_BAD_ARG, "ssb_shard_map_publish_f32: NULL pointer");
    if (T == 0 || T % 4 != 0 || !aligned_to(gate, 16) || !aligned_to(other, 16) || !aligned_to(walked, 8))
        return fail(SSB_ERR_UNSUPPORTED, "ssb_shard_map_publish_f32 needs T %% 4 == 0 and 16-byte aligned tensors (T=%lld)", (long long)T);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return backward ? shard_map_publish<true>(gate, other, rows, T, cut, px, epoch, walked, st)
                    : shard_map_publish<false>(gate, other, rows, T, cut, px, epoch, walked, st);
}

int ssb_shard_carry_peer_f32(const ssb_peer_exchange_t *exchange, unsigned epoch, int backward, float *carry, void *stream) {
    ssb::shard::PeerExchange px;
    int rc = to_peer_exchange(exchange, &px, "ssb_shard_carry_peer_f32");
    if (rc != SSB_OK) return rc;
    if (px.rows == 0) return SSB_OK;
    if (!carry || !aligned_to(carry, 4)) return fail(SSB_ERR_BAD_ARG, "ssb_shard_carry_peer_f32: carry is NULL or misaligned");
    const int block = 256;
    const int64_t grid = (px.rows + block - 1) / block;
    if (grid > 0x7fffffffLL) return fail(SSB_ERR_BAD_ARG, "ssb_shard_carry_peer_f32: too many rows");
    ssb::shard::peer_carry_kernel<<<(int)grid, block, 0, static_cast<cudaStream_t>(stream)>>>(px, backward ? 1 : 0, (int)(epoch & 1u), epoch, carry);
    return check_launch("peer_carry_kernel");
}

int ssb_selftest_wait_timeout(void *scratch, size_t scratch_bytes, void *stream) {
    if (scratch == nullptr || scratch_bytes < 32 || !aligned_to(scratch, 16))
        return fail(SSB_ERR_WORKSPACE, "ssb_selftest_wait_timeout needs 32 bytes of 16-byte aligned device scratch");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(scratch, 0, 32, st) != cudaSuccess) return check_launch("cudaMemsetAsync(scratch)");
    auto *rec = static_cast<ssb::lookback::Record *>(scratch);
    ssb::lookback::wait_probe_kernel<<<1, 32, 0, st>>>(rec, reinterpret_cast<float *>(rec + 1));
    return check_launch("wait_probe_kernel");
}

int ssb_checked_build(void) {
#ifdef SSB_CHECKED
    return 1;
#else
    return 0;
#endif
}

int ssb_selftest_index_check(void *stream) {
#ifdef SSB_CHECKED
    ssb::index_check_probe_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(5, 4);
    return check_launch("index_check_probe_kernel");
#else
    (void)stream;
    return fail(SSB_ERR_UNSUPPORTED, "ssb_selftest_index_check: this is not the checked build");
#endif
}

int ssb_device_status(int *detail) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(SSB_ERR_LAUNCH, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    int word[2] = {0, 0};
    e = cudaMemcpyFromSymbol(word, ssb::g_status_word, sizeof(word));
    if (e != cudaSuccess) return fail(SSB_ERR_LAUNCH, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    if (detail) *detail = word[1];
    if (word[0] != 0) {
        const int zero[2] = {0, 0};
        (void)cudaMemcpyToSymbol(ssb::g_status_word, zero, sizeof(zero));
        return word[0] == SSB_ERR_DEVICE_CHECK
                   ? fail(word[0], "a kernel computed an index outside its tensor and skipped the access (site %d)", word[1])
                   : fail(word[0], "a device-side wait ran out (kernel code %d)", word[1]);
    }
    return SSB_OK;
}

}  // extern "C"
