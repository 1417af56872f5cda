/*
 * scanscam_b200 -- C-ABI launch layer of the B200 (sm_100a) gated linear scan.
 *
 *   forward :  h_t  = a_t * h_{t-1} + b_t           (a = gate, b = value, h = output)
 *   backward:  gb_t = g_t + a_{t+1} * gb_{t+1}      (g = upstream gradient)
 *              ga_t = gb_t * h_{t-1}
 *
 * Every entry point takes raw DEVICE pointers, 64-bit sizes and a CUDA stream
 * (a `cudaStream_t` passed as `void*`; NULL = the legacy default stream), enqueues
 * its kernels on that stream without synchronising, and returns an `ssb_status_t`.
 * Outputs are caller-allocated, as in the reference extension, whose functions all
 * have the shape `void f(Tensor inputs..., Tensor outputs...)`
 * (reference: src/scanscam_cuda.cu:725-737).  No compute entry point allocates device
 * memory; the ones that need scratch take it from the caller (see
 * ssb_scan_workspace_bytes).  (The set-up helpers ssb_peer_buffer_* of the multi-GPU
 * exchange are the exception, and say so.)  No torch types appear here: the PyTorch extension
 * `scanscam_ext` and any other FFI binding (ctypes, cgo, JNI ...) are equal clients.
 *
 * "rows" layout   : dense [rows, T], scan axis innermost and contiguous.
 * "cl" layout     : dense [N, T, C] (channels-last), scan over the middle axis.
 *
 * Thread safety: entry points may be called concurrently from several host threads
 * and on several streams.  The only process-wide state is a per-device status word
 * that device code sets when one of its bounded waits gives up (ssb_device_status).
 */
#ifndef SCANSCAM_B200_H
#define SCANSCAM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ssb_status {
    SSB_OK = 0,
    SSB_ERR_BAD_ARG = 1,     /* NULL where data is required, negative size, size overflow */
    SSB_ERR_ALIGNMENT = 2,   /* pointer not aligned to its element size */
    SSB_ERR_LAUNCH = 3,      /* the CUDA runtime or driver rejected a call; see ssb_last_error */
    SSB_ERR_DEVICE_WAIT = 4, /* a bounded device-side wait ran out (reported by ssb_device_status) */
    SSB_ERR_WORKSPACE = 5,   /* workspace missing or smaller than ssb_scan_workspace_bytes says */
    SSB_ERR_UNSUPPORTED = 6, /* the requested kernel variant cannot run this shape */
    SSB_ERR_DEVICE_CHECK = 7 /* checked build only: a kernel computed an index outside its tensor; the access was
                                skipped (reported by ssb_device_status) */
} ssb_status_t;

/* Kernel families, for callers that want to pin one (tests, tuning sweeps).
 * SSB_VARIANT_AUTO picks from (rows, T, alignment). */
typedef enum ssb_variant {
    SSB_VARIANT_AUTO = 0,
    SSB_VARIANT_WARP = 1,    /* one warp per row, register-resident, any T / any alignment */
    SSB_VARIANT_TMA = 2,     /* TMA-staged shared-memory tiles; needs T % 32 == 0, 16-B aligned base.  Tuning ids
                                0..31 per-warp rings, 32..38 the flat sweep for T = 32 * 2^k <= 4096, 48 the flat
                                sweep over rows that are a multiple (>= 2) of 4096 */
    SSB_VARIANT_LOOKBACK = 3, /* T split across CTAs with decoupled look-back; needs a workspace.  Tuning id 16
                                 (variant | 16 << 8): no look-back but two passes over 4096-step chunks of T
                                 run as rows of their own (chunk maps, carries, scan).  Tuning id 17: the same
                                 with long chunks whose maps are folded only as far as the gate product needs
                                 (it stops at 2^-40), then one sweep: for a few very long rows */
    SSB_VARIANT_FLAT = 4,    /* memcpy-like sweep, CTA-wide scan of 16 KB spans; needs T % 4 == 0, 16-B aligned base */
    SSB_VARIANT_FLAT_ANY = 5 /* the same sweep with per-element row boundaries: any T, 16-B aligned base */
} ssb_variant_t;

/* Library version (major*10000 + minor*100 + patch). */
int ssb_version(void);
/* Human-readable name of a status code (static storage). */
const char *ssb_status_string(int status);
/* Message of the last failure on the calling host thread (thread-local, never NULL). */
const char *ssb_last_error(void);

/* ------------------------------------------------------------------------------------
 * Forward scan, rows layout.
 * Replaces `blocked_linear_scan(gate, value, output)` (src/scanscam_cuda.cu:260-307,
 * kernels :144-258) and, behind the same math, `simple_linear_scan` (:38-59) and
 * `coalesced_linear_scan` (:121-142).
 *   gate, value, out : [rows, T]
 *   h_in             : optional [rows]; h just before step 0 (NULL = 0, the reference's case).
 *                      Used when this call is one shard of a longer sequence.
 * ---------------------------------------------------------------------------------- */
int ssb_scan_fwd_f32(const float *gate, const float *value, float *out, int64_t rows, int64_t T,
                     const float *h_in, void *stream);
int ssb_scan_fwd_f64(const double *gate, const double *value, double *out, int64_t rows,
                     int64_t T, const double *h_in, void *stream);
/* Same, with the kernel family pinned and an optional workspace (only SSB_VARIANT_LOOKBACK needs
 * one).  With SSB_VARIANT_AUTO the entry point makes the choice ssb_scan_recommend reports for
 * can_provide_workspace = 1 when `workspace` is 256-byte aligned and holds at least
 * ssb_scan_workspace_bytes() of that choice, and otherwise the choice made without scratch. */
int ssb_scan_fwd_f32_ex(const float *gate, const float *value, float *out, int64_t rows,
                        int64_t T, const float *h_in, int variant, void *workspace,
                        size_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------------------------
 * Fused backward, rows layout: one pass reads gate, h, gout and writes both gradients.
 * Replaces `blocked_linear_scan_backward(gate, output, outGrad, gateGradOut, valueGradOut)`
 * (src/scanscam_cuda.cu:427-469, kernel :366-425) and `simple_linear_scan_backward`
 * (:334-364).
 *   gate, h, gout, ggate, gvalue : [rows, T]   (h = the forward output)
 *   c_in   : optional [rows]; a_T * gb_T flowing in from the step after the last one (NULL = 0)
 *   h_prev : optional [rows]; h just before step 0, multiplies gb_0 into ga_0 (NULL = 0)
 * ---------------------------------------------------------------------------------- */
int ssb_scan_bwd_f32(const float *gate, const float *h, const float *gout, float *ggate,
                     float *gvalue, int64_t rows, int64_t T, const float *c_in,
                     const float *h_prev, void *stream);
int ssb_scan_bwd_f64(const double *gate, const double *h, const double *gout, double *ggate,
                     double *gvalue, int64_t rows, int64_t T, const double *c_in,
                     const double *h_prev, void *stream);
int ssb_scan_bwd_f32_ex(const float *gate, const float *h, const float *gout, float *ggate,
                        float *gvalue, int64_t rows, int64_t T, const float *c_in,
                        const float *h_prev, int variant, void *workspace,
                        size_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------------------------
 * Forward scan of long rows for callers that cannot hand over scratch memory.
 * (No counterpart in the reference: it never splits a row and so never needs scratch.)
 *
 * Some hosts of this library have nowhere to get device memory from at call time: an
 * inference server that reserved the whole GPU for its own pools at start-up and treats any
 * later cudaMalloc as a bug (it synchronises the device and can fail or fragment), a binding
 * from a language runtime that owns no CUDA allocator, code running between fixed-size
 * arenas.  For them this entry point runs the same look-back kernel as
 * ssb_scan_fwd_f32_ex(..., SSB_VARIANT_LOOKBACK, ...) on a scratch area that is built into the
 * library image: SSB_STATIC_SCRATCH_BYTES of device memory that every GPU holds from the
 * moment the library is loaded on it until the process exits.  The call itself allocates and
 * frees nothing, on the device or through any library.
 *
 * Limits and rules:
 *   - rows must be longer than one span (T > 4096), T % 4 == 0, all pointers 16-byte aligned;
 *     other shapes need no scratch: use ssb_scan_fwd_f32.
 *   - rows * ceil(T / 4096) must not exceed SSB_STATIC_SCRATCH_SPANS (65 536 spans, i.e. up to
 *     268 million elements); larger problems are refused with SSB_ERR_WORKSPACE and a message
 *     that names both sizes.
 *   - every call on a device uses the same scratch area, which still holds the previous
 *     call's records; the call clears, on `stream`, the part it is going to use before its
 *     kernel starts.  Two calls that can run on the GPU at the same time (different streams,
 *     different host threads) would overwrite each other's records: serialise them.
 *   - the first call on each device looks up the device address of the scratch area (a
 *     host-side query, done once per device with that device current).  Make that first call
 *     outside of any stream capture.
 * ---------------------------------------------------------------------------------- */
#define SSB_STATIC_SCRATCH_SPANS 65536
#define SSB_STATIC_SCRATCH_BYTES (256 + 16 * SSB_STATIC_SCRATCH_SPANS)
int ssb_scan_fwd_f32_static(const float *gate, const float *value, float *out, int64_t rows,
                            int64_t T, const float *h_in, void *stream);

/* ------------------------------------------------------------------------------------
 * Gate logits in, sigmoid fused (no counterpart in the reference, whose callers compute
 * gate = sigmoid(z) in a separate elementwise pass before `scan` and multiply by a(1-a) after
 * its backward).  h_t = sigmoid(z_t) * h_{t-1} + b_t.  The backward writes the gradient with
 * respect to z.  Saves one read and one write of a full tensor in each direction.
 * fp32, rows layout, T % 4 == 0 and 16-byte aligned tensors (SSB_ERR_UNSUPPORTED otherwise:
 * apply the sigmoid yourself and call ssb_scan_fwd_f32 / ssb_scan_bwd_f32).
 * ---------------------------------------------------------------------------------- */
int ssb_scan_sigmoid_fwd_f32(const float *gate_logits, const float *value, float *out, int64_t rows,
                             int64_t T, const float *h_in, void *stream);
int ssb_scan_sigmoid_bwd_f32(const float *gate_logits, const float *h, const float *gout,
                             float *glogits, float *gvalue, int64_t rows, int64_t T, const float *c_in,
                             const float *h_prev, void *stream);

/* ------------------------------------------------------------------------------------
 * 16-bit storage: bf16 or fp16 tensors in memory, fp32 arithmetic, fp32 per-row carries (no
 * counterpart in the reference, whose dispatch covers float and double only,
 * src/scanscam_cuda.cu:52, and raises for half types).  Halves the bytes the scan moves: forward
 * 6, backward 10 bytes per element.  Same meaning of every argument as ssb_scan_fwd_f32 /
 * ssb_scan_bwd_f32; tensor pointers address 16-bit elements and need 2-byte alignment (16-byte for
 * the fast kernels: rows of T = 64 * 2^k <= 8192, and longer rows that are a multiple of 4096, go
 * through the bulk-tensor sweep, other T % 8 == 0 through 16-byte loads, anything else element by
 * element).  Every output element is the fp32
 * result rounded to nearest-even once; the running state h is never rounded between steps.
 * ---------------------------------------------------------------------------------- */
int ssb_scan_fwd_bf16(const void *gate, const void *value, void *out, int64_t rows, int64_t T,
                      const float *h_in, void *stream);
int ssb_scan_bwd_bf16(const void *gate, const void *h, const void *gout, void *ggate, void *gvalue,
                      int64_t rows, int64_t T, const float *c_in, const float *h_prev, void *stream);
int ssb_scan_fwd_f16(const void *gate, const void *value, void *out, int64_t rows, int64_t T,
                     const float *h_in, void *stream);
int ssb_scan_bwd_f16(const void *gate, const void *h, const void *gout, void *ggate, void *gvalue,
                     int64_t rows, int64_t T, const float *c_in, const float *h_prev, void *stream);
/* The fused forms on 16-bit tensors: gate logits in (as ssb_scan_sigmoid_*_f32) and the backward
 * that recomputes h from (gate, value) (as ssb_scan_bwd_recompute_f32, no workspace).  Rows of
 * T = 64 * 2^k <= 8192 (the sigmoid forms also take longer rows that are a multiple of 4096) and
 * 16-byte aligned tensors only; SSB_ERR_UNSUPPORTED otherwise (compose them from the plain entry
 * points).  The recomputed h is the fp32 one, not its 16-bit rounding. */
int ssb_scan_sigmoid_fwd_bf16(const void *gate_logits, const void *value, void *out, int64_t rows,
                              int64_t T, const float *h_in, void *stream);
int ssb_scan_sigmoid_bwd_bf16(const void *gate_logits, const void *h, const void *gout, void *glogits,
                              void *gvalue, int64_t rows, int64_t T, const float *c_in,
                              const float *h_prev, void *stream);
int ssb_scan_sigmoid_fwd_f16(const void *gate_logits, const void *value, void *out, int64_t rows,
                             int64_t T, const float *h_in, void *stream);
int ssb_scan_sigmoid_bwd_f16(const void *gate_logits, const void *h, const void *gout, void *glogits,
                             void *gvalue, int64_t rows, int64_t T, const float *c_in,
                             const float *h_prev, void *stream);
int ssb_scan_bwd_recompute_bf16(const void *gate, const void *value, const void *gout, void *ggate,
                                void *gvalue, int64_t rows, int64_t T, const float *h_in,
                                const float *c_in, void *stream);
int ssb_scan_bwd_recompute_f16(const void *gate, const void *value, const void *gout, void *ggate,
                               void *gvalue, int64_t rows, int64_t T, const float *h_in,
                               const float *c_in, void *stream);

/* ------------------------------------------------------------------------------------
 * Backward that recomputes h (no counterpart in the reference, whose op.Scan.forward saves both
 * `gate` and `output` for the backward, scanscam/op.py:36).  Takes what the forward took --
 * gate a, value b, and the carry h_in entering each row (NULL = 0) -- plus gout and c_in, and
 * returns the same two gradients as ssb_scan_bwd_f32, so that a caller can drop h between the
 * passes (4 bytes per element of activation memory).
 *   - rows with T = 32 * 2^k <= 4096: one kernel rebuilds h for each span on the fly; it reads
 *     a, b, gout and writes the two gradients, the same 20 bytes per element as the ordinary
 *     backward.  No workspace.
 *   - any other shape: the forward kernel writes h into the caller's workspace and the ordinary
 *     backward reads it back (32 bytes per element in total); the workspace holds h for the
 *     duration of the call only.
 * fp32, rows layout, tensors 16-byte aligned.
 * ---------------------------------------------------------------------------------- */
size_t ssb_scan_bwd_recompute_workspace_bytes(int64_t rows, int64_t T);
int ssb_scan_bwd_recompute_f32(const float *gate, const float *value, const float *gout, float *ggate,
                               float *gvalue, int64_t rows, int64_t T, const float *h_in,
                               const float *c_in, void *workspace, size_t workspace_bytes, void *stream);

/* fp64 with scratch (an addition; same results as ssb_scan_fwd_f64 / ssb_scan_bwd_f64 up to fp64
 * reassociation).  The fp64 kernels give one warp a row, which needs about a thousand rows to fill
 * the GPU; with fewer than 768 rows of T >= 16384, T % 4096 == 0, and a workspace of
 * ssb_scan_f64_workspace_bytes(rows, T) bytes (256-byte aligned; 0 = this shape never uses one)
 * the rows are cut into 4096-step chunks and scanned in two passes.  NULL / too small a workspace
 * or any other shape behaves exactly like the plain entry points. */
size_t ssb_scan_f64_workspace_bytes(int64_t rows, int64_t T);
int ssb_scan_fwd_f64_ex(const double *gate, const double *value, double *out, int64_t rows, int64_t T,
                        const double *h_in, void *workspace, size_t workspace_bytes, void *stream);
int ssb_scan_bwd_f64_ex(const double *gate, const double *h, const double *gout, double *ggate,
                        double *gvalue, int64_t rows, int64_t T, const double *c_in,
                        const double *h_prev, void *workspace, size_t workspace_bytes, void *stream);

/* Bytes of scratch the given variant needs for a [rows, T] problem (0 = none).
 * The workspace must be 256-byte aligned; its contents need not be initialised (the entry
 * point clears what it needs on the stream it launches on).  A workspace must not be shared
 * by calls that can overlap on the GPU. */
size_t ssb_scan_workspace_bytes(int64_t rows, int64_t T, int variant);

/* The variant (family | tuning id << 8) the library would pick for this problem; the same
 * choice SSB_VARIANT_AUTO makes when `can_provide_workspace` is 0.  With a non-zero
 * `can_provide_workspace` the answer may be SSB_VARIANT_LOOKBACK (long rows: T > 4096), which
 * the caller then has to give ssb_scan_workspace_bytes() of scratch through the _ex entry
 * points.  `aligned16` says whether every tensor pointer is 16-byte aligned. */
int ssb_scan_recommend(int64_t rows, int64_t T, int backward, int aligned16, int can_provide_workspace);

/* ------------------------------------------------------------------------------------
 * Channels-last layout, [N, T, C] scanned over T.
 * Replace `transposed_linear_scan(gate, value, output, channelsPerBlock)`
 * (src/scanscam_cuda.cu:556-582, kernel :471-554) and
 * `transposed_linear_scan_backward(...)` (:687-723, kernel :584-685).  The reference's
 * `channelsPerBlock` is a tuning hint with no effect on results; it has no counterpart here.
 * ---------------------------------------------------------------------------------- */
int ssb_scan_cl_fwd_f32(const float *gate, const float *value, float *out, int64_t N, int64_t T,
                        int64_t C, void *stream);
int ssb_scan_cl_fwd_f64(const double *gate, const double *value, double *out, int64_t N,
                        int64_t T, int64_t C, void *stream);
int ssb_scan_cl_bwd_f32(const float *gate, const float *h, const float *gout, float *ggate,
                        float *gvalue, int64_t N, int64_t T, int64_t C, void *stream);
int ssb_scan_cl_bwd_f64(const double *gate, const double *h, const double *gout, double *ggate,
                        double *gvalue, int64_t N, int64_t T, int64_t C, void *stream);

/* Channels-last on 16-bit tensors (bf16 / fp16 storage, fp32 arithmetic; no counterpart in the
 * reference).  The streaming kernels with 64-channel blocks; C % 8 == 0 and 16-byte aligned
 * tensors, SSB_ERR_UNSUPPORTED otherwise.  `workspace` (ssb_scan_cl_h16_workspace_bytes, 256-byte
 * aligned, may be NULL) lets shapes with fewer than 96 (batch element, 64-channel block) pairs and
 * T >= 2048 run in the two-pass chunked form; without it one CTA walks all of T per pair.  The
 * query returns 0 for shapes that never use scratch. */
size_t ssb_scan_cl_h16_workspace_bytes(int64_t N, int64_t T, int64_t C);
int ssb_scan_cl_fwd_bf16(const void *gate, const void *value, void *out, int64_t N, int64_t T, int64_t C,
                         void *workspace, size_t workspace_bytes, void *stream);
int ssb_scan_cl_bwd_bf16(const void *gate, const void *h, const void *gout, void *ggate, void *gvalue,
                         int64_t N, int64_t T, int64_t C, void *workspace, size_t workspace_bytes,
                         void *stream);
int ssb_scan_cl_fwd_f16(const void *gate, const void *value, void *out, int64_t N, int64_t T, int64_t C,
                        void *workspace, size_t workspace_bytes, void *stream);
int ssb_scan_cl_bwd_f16(const void *gate, const void *h, const void *gout, void *ggate, void *gvalue,
                        int64_t N, int64_t T, int64_t C, void *workspace, size_t workspace_bytes,
                        void *stream);

/* Channels-last with gate logits in (sigmoid fused, as ssb_scan_sigmoid_*; no counterpart in the
 * reference), fp32 (C % 4 == 0) and 16-bit tensors (C % 8 == 0), 16-byte aligned; always the
 * streaming kernels.  `workspace`: ssb_scan_cl_sigmoid_workspace_bytes (fp32; 0 for shapes that
 * never use scratch) or ssb_scan_cl_h16_workspace_bytes (16-bit) bytes, may be NULL (then shapes
 * with few channel blocks run one CTA per block instead of the two-pass chunked form).
 * SSB_ERR_UNSUPPORTED for other channel counts or alignments: apply the sigmoid separately. */
size_t ssb_scan_cl_sigmoid_workspace_bytes(int64_t N, int64_t T, int64_t C);
int ssb_scan_cl_sigmoid_fwd_f32(const float *gate_logits, const float *value, float *out, int64_t N, int64_t T,
                                int64_t C, void *workspace, size_t workspace_bytes, void *stream);
int ssb_scan_cl_sigmoid_bwd_f32(const float *gate_logits, const float *h, const float *gout, float *glogits,
                                float *gvalue, int64_t N, int64_t T, int64_t C, void *workspace,
                                size_t workspace_bytes, void *stream);
int ssb_scan_cl_sigmoid_fwd_bf16(const void *gate_logits, const void *value, void *out, int64_t N, int64_t T,
                                 int64_t C, void *workspace, size_t workspace_bytes, void *stream);
int ssb_scan_cl_sigmoid_bwd_bf16(const void *gate_logits, const void *h, const void *gout, void *glogits,
                                 void *gvalue, int64_t N, int64_t T, int64_t C, void *workspace,
                                 size_t workspace_bytes, void *stream);
int ssb_scan_cl_sigmoid_fwd_f16(const void *gate_logits, const void *value, void *out, int64_t N, int64_t T,
                                int64_t C, void *workspace, size_t workspace_bytes, void *stream);
int ssb_scan_cl_sigmoid_bwd_f16(const void *gate_logits, const void *h, const void *gout, void *glogits,
                                void *gvalue, int64_t N, int64_t T, int64_t C, void *workspace,
                                size_t workspace_bytes, void *stream);

/* Channels-last with a selectable kernel family and optional scratch.  With scratch the time axis
 * can be split across CTAs (two-pass chunked streaming, or decoupled look-back), so the whole GPU
 * is busy even when N*C is small.  (No counterpart in the reference, whose one kernel per direction
 * gives a CTA a (batch element, channel block) pair for all of T, src/scanscam_cuda.cu:471-685.)
 *
 * `variant` = family | tuning id << 8 | (1 << 16 to force one channel per lane where the family
 * has a 4-channel form).  SSB_CL_VARIANT_AUTO chooses from the shape and from the scratch it was
 * given: shapes with at least 96 (batch element, 32-channel block) pairs, T >= 128, C % 4 == 0 and
 * 16-byte aligned tensors run the streaming kernels, which need no scratch -- the plain entry
 * points above choose them too -- with the tile shape (tuning id 0, 1 or 2) that an estimate of
 * rounds over the SMs favours for that direction, so the forward and the backward of one shape
 * may report different ids; with fewer pairs, T >= 2048 and enough scratch the same kernels run
 * over chunks of T in two passes; otherwise the look-back kernels when scratch is given and they
 * are faster, else the plain kernels.  A pinned family that cannot run the shape returns
 * SSB_ERR_UNSUPPORTED, one that is given too little scratch SSB_ERR_WORKSPACE.  Results do not
 * depend on the variant beyond fp32 reassociation.  There is no hidden state: every call names its
 * variant, and concurrent calls need only distinct workspaces. */
typedef enum ssb_cl_variant {
    SSB_CL_VARIANT_AUTO = 0,
    SSB_CL_VARIANT_PLAIN = 1,        /* a CTA walks all of T for 32 channels, lane = channel; any shape, no scratch */
    SSB_CL_VARIANT_LOOKBACK = 2,     /* tiles of one channel group on different CTAs, decoupled look-back; ids 0..12 */
    SSB_CL_VARIANT_LOOKBACK_TMA = 3, /* the same on tiles staged by bulk tensor copies; ids 0..5; C % 4 == 0 */
    SSB_CL_VARIANT_STREAM = 4,       /* a CTA walks all of T, tiles through a bulk-tensor ring; ids 0..7; no scratch */
    SSB_CL_VARIANT_CHUNKED = 5,      /* the streaming kernels over chunks of T in two passes (maps, then scan) */
    SSB_CL_VARIANT_NARROW = 6        /* C = 4, 8 or 16: a CTA walks a whole batch element, tiles are contiguous bytes
                                        moved by untiled bulk copies; no scratch; AUTO's choice from 64 batch elements up */
} ssb_cl_variant_t;

/* What SSB_CL_VARIANT_AUTO would run for this fp32 problem (`can_provide_workspace` != 0: assume
 * the caller can supply whatever ssb_scan_cl_variant_workspace_bytes asks for). */
int ssb_scan_cl_recommend(int64_t N, int64_t T, int64_t C, int backward, int aligned16, int can_provide_workspace);
/* Scratch that `variant` needs for this problem and direction: 0 for the plain and streaming
 * kernels, the chunk maps for the chunked form, one record per tile for look-back.
 * 256-byte aligned; contents need not be initialised. */
size_t ssb_scan_cl_variant_workspace_bytes(int64_t N, int64_t T, int64_t C, int variant, int backward);
/* An upper bound of the above over every variant and both directions, for callers that would
 * rather size one buffer once (it can be a third of a tensor; prefer the per-variant query). */
size_t ssb_scan_cl_workspace_bytes(int64_t N, int64_t T, int64_t C);
int ssb_scan_cl_fwd_f32_ex(const float *gate, const float *value, float *out, int64_t N, int64_t T,
                           int64_t C, int variant, void *workspace, size_t workspace_bytes, void *stream);
int ssb_scan_cl_bwd_f32_ex(const float *gate, const float *h, const float *gout, float *ggate,
                           float *gvalue, int64_t N, int64_t T, int64_t C, int variant, void *workspace,
                           size_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------------------------
 * Sequence (T) sharding.  The reference never splits a sequence; these three entry
 * points are the pieces a caller needs to do it: each shard is the affine map
 * h_end = A*h_in + B per row, maps compose associatively, and the composition of the
 * shards to the left (forward) or right (backward) is the carry a shard starts from.
 *
 * ssb_shard_reduce_fwd_f32: agg[r] = (A, B) with A = prod_t a_t and B = the scan's last
 *   value when started from 0.  Reads gate and value once, writes 8 bytes per row.
 * ssb_shard_reduce_bwd_f32: agg[r] = (A, D) of the reverse recurrence
 *   c_t = a_t * (g_t + c_{t+1}):  c_first = A * c_in + D.
 * ssb_shard_carry_f32: aggs is [n_shards, rows, 2] (every shard's pair, e.g. after an
 *   all-gather).  reverse == 0: carry[r] = h entering shard `shard` (fold of shards
 *   0..shard-1 from zero).  reverse != 0: carry[r] = c entering shard `shard` from the
 *   right (fold of shards n_shards-1 .. shard+1 from zero).
 * ---------------------------------------------------------------------------------- */
int ssb_shard_reduce_fwd_f32(const float *gate, const float *value, float *agg, int64_t rows,
                             int64_t T, void *workspace, size_t workspace_bytes, void *stream);
int ssb_shard_reduce_bwd_f32(const float *gate, const float *gout, float *agg, int64_t rows,
                             int64_t T, void *workspace, size_t workspace_bytes, void *stream);
/* Scratch the two reduce entry points can use (0 = they never use any for this shape).  With a
 * workspace of that size long rows are reduced by many CTAs per row; without one (NULL, 0) one
 * warp walks each row, which is slower for long rows and few of them. */
size_t ssb_shard_reduce_workspace_bytes(int64_t rows, int64_t T);
int ssb_shard_carry_f32(const float *aggs, int n_shards, int shard, int reverse, int64_t rows,
                        float *carry, void *stream);

/* The same two maps, computed by walking each row from the end that the map depends on most --
 * the forward map from the shard's last step towards its first, the reverse map from the first
 * step towards the last -- and stopping as soon as the product of the gates walked so far has
 * dropped to |A| <= cut.  What was not walked could change B (or D) by at most cut times the
 * state entering the walked part, i.e. by at most `cut` relative to the largest value of the scan.
 *   cut = 0 : stop only when the product is exactly zero (a zero gate, or underflow); the result
 *             equals ssb_shard_reduce_* up to reassociation.
 *   cut > 0 : e.g. 2^-40; gates in (0, 1) then cost a few thousand steps per row instead of the
 *             whole shard (8 bytes per element of the walked part only).
 *   cut < 0 : never stop early.
 * Rows whose product stays above the cut are walked in full, so the result is within the stated
 * bound for any gates.  `walked` (optional, device memory, 8-byte aligned) is incremented by the
 * number of elements read per tensor, for callers that account for the traffic.  No scratch.
 * T % 4 == 0 and 16-byte aligned tensors run one CTA per row; other shapes fall back to the full
 * reduction of ssb_shard_reduce_* without scratch. */
int ssb_shard_map_fwd_f32(const float *gate, const float *value, float *agg, int64_t rows, int64_t T,
                          float cut, unsigned long long *walked, void *stream);
int ssb_shard_map_bwd_f32(const float *gate, const float *gout, float *agg, int64_t rows, int64_t T,
                          float cut, unsigned long long *walked, void *stream);

/* ------------------------------------------------------------------------------------
 * The same exchange without a collective library: the map kernel stores its result straight into
 * every rank's buffer over NVLink (plain peer stores), and the carry kernel waits for them.
 * (No counterpart in the reference.)  For ONE process per GPU on one node with peer access
 * between all GPUs; the ranks call both entry points in the same order with the same `epoch`.
 *
 *   ssb_peer_exchange_t: `world` <= 8 ranks, this process's `rank`, `rows`, and for every rank r
 *     `buffers[r]` = the address, in THIS process, of rank r's exchange buffer of
 *     ssb_peer_exchange_bytes(world, rows) bytes (the rank's own from ssb_peer_buffer_create, the
 *     others' from ssb_peer_buffer_open, or any other zeroed allocation / peer mapping that kernels
 *     of this device can address).  Synchronise all ranks after mapping, before the first call.
 *   ssb_shard_map_publish_f32: as ssb_shard_map_fwd/bwd_f32 (`backward` selects the recurrence);
 *     every row's map goes to slot [direction][epoch & 1][rank] of every rank's buffer, and the
 *     last CTA to finish raises flag = epoch at every rank.  T % 4 == 0, 16-byte aligned tensors
 *     (SSB_ERR_UNSUPPORTED otherwise: use the collective path).
 *   ssb_shard_carry_peer_f32: waits until all `world` flags of this rank's buffer have reached
 *     `epoch` -- every wait is bounded at about a second, after which ssb_device_status() reports
 *     SSB_ERR_DEVICE_WAIT and the kernel ends -- then writes carry[rows]: the state this rank's
 *     shard starts from (fold of the ranks before it, or after it for the reverse recurrence).
 *   `epoch` starts at 1 and goes up by one per call and direction; the two directions have buffers
 *   and epochs of their own.  Because every rank waits for every rank, no rank runs more than one
 *   call ahead, and the two slot generations (epoch parity) never collide.
 * ---------------------------------------------------------------------------------- */
typedef struct ssb_peer_exchange {
    int world, rank;
    int64_t rows;
    void *buffers[8];
} ssb_peer_exchange_t;
size_t ssb_peer_exchange_bytes(int world, int64_t rows);
/* Set-up helpers for the exchange buffers (called once per job, not per step; these four are the
 * only entry points of the library that allocate or map device memory).
 *   ssb_peer_buffer_create: allocates `bytes` of zeroed device memory on the current device
 *     (cudaMalloc, so that the allocation is exportable as a whole) and writes its 64-byte CUDA IPC
 *     handle, to be sent to the other ranks by any means.
 *   ssb_peer_buffer_open: maps another process's buffer from its handle WITH THIS PROCESS'S OWN DEVICE
 *     CURRENT, which is what makes it addressable by kernels of this device (peer access between
 *     the two devices is switched on as needed); the two devices must be peer-capable.
 *   ssb_peer_buffer_close / ssb_peer_buffer_destroy: unmap a peer's buffer / free the own one. */
#define SSB_IPC_HANDLE_BYTES 64
int ssb_peer_buffer_create(size_t bytes, void **ptr, unsigned char handle[SSB_IPC_HANDLE_BYTES]);
int ssb_peer_buffer_open(const unsigned char handle[SSB_IPC_HANDLE_BYTES], void **ptr);
int ssb_peer_buffer_close(void *ptr);
int ssb_peer_buffer_destroy(void *ptr);
int ssb_shard_map_publish_f32(const float *gate, const float *other, int64_t rows, int64_t T, float cut, int backward,
                              const ssb_peer_exchange_t *exchange, unsigned epoch, unsigned long long *walked,
                              void *stream);
int ssb_shard_carry_peer_f32(const ssb_peer_exchange_t *exchange, unsigned epoch, int backward, float *carry,
                             void *stream);

/* Self-test of the bounded-wait machinery: launches one warp that looks back at a record which
 * is never published.  The kernel returns by itself after the poll's time limit (about one
 * second); afterwards ssb_device_status() reports SSB_ERR_DEVICE_WAIT once and the context
 * stays usable.  `scratch`: 32 bytes of 16-byte aligned device memory. */
int ssb_selftest_wait_timeout(void *scratch, size_t scratch_bytes, void *stream);

/* The checked build.  The same sources compiled with -DSSB_CHECKED (`python -m scanscam_b200.build
 * --checked` -> libscanscam_b200_checked.so) make every kernel that computes its own global
 * addresses test each index against its tensor's extent first; an index outside is not
 * dereferenced, the status word becomes SSB_ERR_DEVICE_CHECK with a code for the site, and the
 * kernel runs to its normal end: nothing traps, the context stays usable.  It stands in for a
 * memory checker where none can be run, at a few per cent of speed.  (The reference has neither.)
 * ssb_checked_build: 1 in that build, 0 in the ordinary one.
 * ssb_selftest_index_check: launches one thread that submits an out-of-range index VALUE to the
 * test (no memory is touched); afterwards ssb_device_status() reports SSB_ERR_DEVICE_CHECK once.
 * Returns SSB_ERR_UNSUPPORTED in the ordinary build. */
int ssb_checked_build(void);
int ssb_selftest_index_check(void *stream);

/* Synchronises the current device, returns and clears its device-side status word:
 * SSB_OK, SSB_ERR_DEVICE_WAIT if a kernel's bounded wait (mbarrier, look-back flag) gave up since
 * the last call, or SSB_ERR_DEVICE_CHECK from the checked build.  *detail (optional) receives the
 * kernel-specific code. */
int ssb_device_status(int *detail);

#ifdef __cplusplus
}
#endif
#endif /* SCANSCAM_B200_H */
