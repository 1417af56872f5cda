// PyTorch extension module `scanscam_ext`: the same function names, argument order and
// caller-allocated-output convention as the reference's extension
// (reference: src/scanscam_cuda.cu:725-737), implemented as thin calls into the C-ABI
// launch layer (include/scanscam_b200.h).  Differences from the reference, on purpose:
//   * kernels are enqueued on PyTorch's current stream of the tensors' device (the
//     reference uses the legacy default stream and no device guard);
//   * shapes, dtypes and devices are always checked (the reference's shape/dtype checks
//     are C asserts, compiled out in release builds, src/scanscam_cuda.cu:46-47);
//   * there are no CPU functions: this build has no CPU path.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "../../include/scanscam_b200.h"

namespace {

void check_tensor(const torch::Tensor &x, const char *name) {
    TORCH_CHECK(x.device().is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(x.is_contiguous(), name, " must be contiguous");
}

void check_same(const torch::Tensor &ref, const torch::Tensor &x, const char *name) {
    check_tensor(x, name);
    TORCH_CHECK(x.sizes() == ref.sizes(), name, " must have the same shape as gate");
    TORCH_CHECK(x.scalar_type() == ref.scalar_type(), name, " must have the same dtype as gate");
    TORCH_CHECK(x.device() == ref.device(), name, " must be on the same device as gate");
}

bool is_16bit(const torch::Tensor &x) { return x.scalar_type() == torch::kBFloat16 || x.scalar_type() == torch::kHalf; }

// `allow_16bit`: the rows-layout kernels also take bf16 / fp16 storage (an addition: the reference
// raises for them like for any other non-floating type).
void check_dtype(const torch::Tensor &x, const char *op, bool allow_16bit = false) {
    if (allow_16bit && is_16bit(x)) return;
    // Same wording as the dispatch macro the reference relies on.
    if (x.scalar_type() != torch::kFloat32 && x.scalar_type() != torch::kFloat64) {
        TORCH_CHECK_NOT_IMPLEMENTED(false, "\"", op, "\" not implemented for '", toString(x.scalar_type()), "'");
    }
}

void raise_on(int status, const char *op) {
    TORCH_CHECK(status == SSB_OK, op, " failed: ", ssb_status_string(status), ": ", ssb_last_error());
}

void *current_stream() { return static_cast<void *>(at::cuda::getCurrentCUDAStream().stream()); }

bool aligned16(const torch::Tensor &t) { return reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0; }

// Scratch for the kernels that want it, from PyTorch's caching allocator (stream-ordered, so
// the tensor may be released as soon as the launch has been enqueued on the current stream).
torch::Tensor scratch(size_t bytes, const torch::Tensor &like) {
    return torch::empty({static_cast<int64_t>(bytes)}, like.options().dtype(torch::kUInt8));
}

const void *opt_ptr(const c10::optional<torch::Tensor> &t, const torch::Tensor &like, int64_t rows, const char *name) {
    if (!t.has_value() || !t->defined()) return nullptr;
    check_tensor(*t, name);
    TORCH_CHECK(t->numel() == rows, name, " must have one element per row");
    // carries of 16-bit tensors are fp32
    const auto want = is_16bit(like) ? torch::kFloat32 : like.scalar_type();
    TORCH_CHECK(t->scalar_type() == want && t->device() == like.device(), name, " dtype/device mismatch");
    return t->data_ptr();
}

// ---- rows layout -----------------------------------------------------------------------
void scan_forward_impl(const torch::Tensor &gate, const torch::Tensor &value, torch::Tensor &output,
                       const c10::optional<torch::Tensor> &h_in, int64_t variant, const char *op) {
    check_tensor(gate, "gate");
    TORCH_CHECK(gate.dim() == 2, "gate must be 2-D [rows, T]");
    check_same(gate, value, "value");
    check_same(gate, output, "output");
    check_dtype(gate, op, true);
    const int64_t rows = gate.size(0), T = gate.size(1);
    c10::cuda::CUDAGuard guard(gate.device());
    const void *hin = opt_ptr(h_in, gate, rows, "h_in");
    int rc;
    if (is_16bit(gate)) {
        TORCH_CHECK(variant == SSB_VARIANT_AUTO, op, ": 16-bit tensors have no selectable kernel family");
        auto fn = gate.scalar_type() == torch::kBFloat16 ? ssb_scan_fwd_bf16 : ssb_scan_fwd_f16;
        rc = fn(gate.data_ptr(), value.data_ptr(), output.data_ptr(), rows, T, static_cast<const float *>(hin), current_stream());
    } else if (gate.scalar_type() == torch::kFloat32) {
        if (variant == SSB_VARIANT_AUTO)
            variant = ssb_scan_recommend(rows, T, 0, aligned16(gate) && aligned16(value) && aligned16(output), 1);
        const size_t ws_bytes = ssb_scan_workspace_bytes(rows, T, (int)variant);
        torch::Tensor ws;
        if (ws_bytes > 0) ws = scratch(ws_bytes, gate);
        rc = ssb_scan_fwd_f32_ex(gate.data_ptr<float>(), value.data_ptr<float>(), output.data_ptr<float>(), rows, T,
                                 static_cast<const float *>(hin), (int)variant, ws_bytes ? ws.data_ptr() : nullptr,
                                 ws_bytes, current_stream());
    } else {
        const size_t ws_bytes = ssb_scan_f64_workspace_bytes(rows, T);
        torch::Tensor ws;
        if (ws_bytes > 0) ws = scratch(ws_bytes, gate);
        rc = ssb_scan_fwd_f64_ex(gate.data_ptr<double>(), value.data_ptr<double>(), output.data_ptr<double>(), rows, T,
                                 static_cast<const double *>(hin), ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, current_stream());
    }
    raise_on(rc, op);
}

void scan_backward_impl(const torch::Tensor &gate, const torch::Tensor &output, const torch::Tensor &out_grad,
                        torch::Tensor &gate_grad, torch::Tensor &value_grad, const c10::optional<torch::Tensor> &c_in,
                        const c10::optional<torch::Tensor> &h_prev, int64_t variant, const char *op) {
    check_tensor(gate, "gate");
    TORCH_CHECK(gate.dim() == 2, "gate must be 2-D [rows, T]");
    check_same(gate, output, "output");
    check_same(gate, out_grad, "outGrad");
    check_same(gate, gate_grad, "gateGradOut");
    check_same(gate, value_grad, "valueGradOut");
    check_dtype(gate, op, true);
    const int64_t rows = gate.size(0), T = gate.size(1);
    c10::cuda::CUDAGuard guard(gate.device());
    const void *cin = opt_ptr(c_in, gate, rows, "c_in");
    const void *hp = opt_ptr(h_prev, gate, rows, "h_prev");
    int rc;
    if (is_16bit(gate)) {
        TORCH_CHECK(variant == SSB_VARIANT_AUTO, op, ": 16-bit tensors have no selectable kernel family");
        auto fn = gate.scalar_type() == torch::kBFloat16 ? ssb_scan_bwd_bf16 : ssb_scan_bwd_f16;
        rc = fn(gate.data_ptr(), output.data_ptr(), out_grad.data_ptr(), gate_grad.data_ptr(), value_grad.data_ptr(), rows, T,
                static_cast<const float *>(cin), static_cast<const float *>(hp), current_stream());
    } else if (gate.scalar_type() == torch::kFloat32) {
        if (variant == SSB_VARIANT_AUTO)
            variant = ssb_scan_recommend(rows, T, 1,
                                         aligned16(gate) && aligned16(output) && aligned16(out_grad) &&
                                             aligned16(gate_grad) && aligned16(value_grad), 1);
        const size_t ws_bytes = ssb_scan_workspace_bytes(rows, T, (int)variant);
        torch::Tensor ws;
        if (ws_bytes > 0) ws = scratch(ws_bytes, gate);
        rc = ssb_scan_bwd_f32_ex(gate.data_ptr<float>(), output.data_ptr<float>(), out_grad.data_ptr<float>(),
                                 gate_grad.data_ptr<float>(), value_grad.data_ptr<float>(), rows, T,
                                 static_cast<const float *>(cin), static_cast<const float *>(hp), (int)variant,
                                 ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, current_stream());
    } else {
        const size_t ws_bytes = ssb_scan_f64_workspace_bytes(rows, T);
        torch::Tensor ws;
        if (ws_bytes > 0) ws = scratch(ws_bytes, gate);
        rc = ssb_scan_bwd_f64_ex(gate.data_ptr<double>(), output.data_ptr<double>(), out_grad.data_ptr<double>(),
                                 gate_grad.data_ptr<double>(), value_grad.data_ptr<double>(), rows, T,
                                 static_cast<const double *>(cin), static_cast<const double *>(hp),
                                 ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, current_stream());
    }
    raise_on(rc, op);
}

// The three forward names of the reference differ only in kernel strategy; here they all run
// the same kernels (src/scanscam_cuda.cu:38-59, 121-142, 260-307).
void simple_linear_scan(torch::Tensor gate, torch::Tensor value, torch::Tensor output) {
    scan_forward_impl(gate, value, output, c10::nullopt, SSB_VARIANT_AUTO, "simple_linear_scan");
}
void coalesced_linear_scan(torch::Tensor gate, torch::Tensor value, torch::Tensor output) {
    scan_forward_impl(gate, value, output, c10::nullopt, SSB_VARIANT_AUTO, "coalesced_linear_scan");
}
void blocked_linear_scan(torch::Tensor gate, torch::Tensor value, torch::Tensor output) {
    scan_forward_impl(gate, value, output, c10::nullopt, SSB_VARIANT_AUTO, "blocked_linear_scan");
}
// src/scanscam_cuda.cu:334-364 and :427-469
void simple_linear_scan_backward(torch::Tensor gate, torch::Tensor output, torch::Tensor outGrad,
                                 torch::Tensor gateGradOut, torch::Tensor valueGradOut) {
    scan_backward_impl(gate, output, outGrad, gateGradOut, valueGradOut, c10::nullopt, c10::nullopt, SSB_VARIANT_AUTO,
                       "simple_linear_scan_backward");
}
void blocked_linear_scan_backward(torch::Tensor gate, torch::Tensor output, torch::Tensor outGrad,
                                  torch::Tensor gateGradOut, torch::Tensor valueGradOut) {
    scan_backward_impl(gate, output, outGrad, gateGradOut, valueGradOut, c10::nullopt, c10::nullopt, SSB_VARIANT_AUTO,
                       "blocked_linear_scan_backward");
}

// Extended entry points (not in the reference): pinned kernel family and shard carries.
void scan_forward_ex(torch::Tensor gate, torch::Tensor value, torch::Tensor output, c10::optional<torch::Tensor> h_in,
                     int64_t variant) {
    scan_forward_impl(gate, value, output, h_in, variant, "scan_forward_ex");
}
void scan_backward_ex(torch::Tensor gate, torch::Tensor output, torch::Tensor outGrad, torch::Tensor gateGradOut,
                      torch::Tensor valueGradOut, c10::optional<torch::Tensor> c_in, c10::optional<torch::Tensor> h_prev,
                      int64_t variant) {
    scan_backward_impl(gate, output, outGrad, gateGradOut, valueGradOut, c_in, h_prev, variant, "scan_backward_ex");
}

// ---- gate logits in, sigmoid fused (not in the reference) --------------------------------
void scan_sigmoid_forward(torch::Tensor logits, torch::Tensor value, torch::Tensor output) {
    check_tensor(logits, "gate_logits");
    TORCH_CHECK(logits.dim() == 2 && (logits.scalar_type() == torch::kFloat32 || is_16bit(logits)),
                "gate_logits must be 2-D float32, bfloat16 or float16");
    check_same(logits, value, "value");
    check_same(logits, output, "output");
    c10::cuda::CUDAGuard guard(logits.device());
    if (is_16bit(logits)) {
        auto fn = logits.scalar_type() == torch::kBFloat16 ? ssb_scan_sigmoid_fwd_bf16 : ssb_scan_sigmoid_fwd_f16;
        raise_on(fn(logits.data_ptr(), value.data_ptr(), output.data_ptr(), logits.size(0), logits.size(1), nullptr,
                    current_stream()),
                 "scan_sigmoid_forward");
        return;
    }
    raise_on(ssb_scan_sigmoid_fwd_f32(logits.data_ptr<float>(), value.data_ptr<float>(), output.data_ptr<float>(),
                                      logits.size(0), logits.size(1), nullptr, current_stream()),
             "scan_sigmoid_forward");
}

void scan_sigmoid_backward(torch::Tensor logits, torch::Tensor output, torch::Tensor outGrad, torch::Tensor logitsGradOut,
                           torch::Tensor valueGradOut) {
    check_tensor(logits, "gate_logits");
    TORCH_CHECK(logits.dim() == 2 && (logits.scalar_type() == torch::kFloat32 || is_16bit(logits)),
                "gate_logits must be 2-D float32, bfloat16 or float16");
    check_same(logits, output, "output");
    check_same(logits, outGrad, "outGrad");
    check_same(logits, logitsGradOut, "logitsGradOut");
    check_same(logits, valueGradOut, "valueGradOut");
    c10::cuda::CUDAGuard guard(logits.device());
    if (is_16bit(logits)) {
        auto fn = logits.scalar_type() == torch::kBFloat16 ? ssb_scan_sigmoid_bwd_bf16 : ssb_scan_sigmoid_bwd_f16;
        raise_on(fn(logits.data_ptr(), output.data_ptr(), outGrad.data_ptr(), logitsGradOut.data_ptr(),
                    valueGradOut.data_ptr(), logits.size(0), logits.size(1), nullptr, nullptr, current_stream()),
                 "scan_sigmoid_backward");
        return;
    }
    raise_on(ssb_scan_sigmoid_bwd_f32(logits.data_ptr<float>(), output.data_ptr<float>(), outGrad.data_ptr<float>(),
                                      logitsGradOut.data_ptr<float>(), valueGradOut.data_ptr<float>(), logits.size(0),
                                      logits.size(1), nullptr, nullptr, current_stream()),
             "scan_sigmoid_backward");
}

// ---- backward that recomputes h from (gate, value) (not in the reference) -----------------
void scan_backward_recompute(torch::Tensor gate, torch::Tensor value, torch::Tensor outGrad, torch::Tensor gateGradOut,
                             torch::Tensor valueGradOut) {
    check_tensor(gate, "gate");
    TORCH_CHECK(gate.dim() == 2 && (gate.scalar_type() == torch::kFloat32 || is_16bit(gate)),
                "gate must be 2-D float32, bfloat16 or float16");
    check_same(gate, value, "value");
    check_same(gate, outGrad, "outGrad");
    check_same(gate, gateGradOut, "gateGradOut");
    check_same(gate, valueGradOut, "valueGradOut");
    c10::cuda::CUDAGuard guard(gate.device());
    if (is_16bit(gate)) {
        auto fn = gate.scalar_type() == torch::kBFloat16 ? ssb_scan_bwd_recompute_bf16 : ssb_scan_bwd_recompute_f16;
        raise_on(fn(gate.data_ptr(), value.data_ptr(), outGrad.data_ptr(), gateGradOut.data_ptr(), valueGradOut.data_ptr(),
                    gate.size(0), gate.size(1), nullptr, nullptr, current_stream()),
                 "scan_backward_recompute");
        return;
    }
    const size_t ws_bytes = ssb_scan_bwd_recompute_workspace_bytes(gate.size(0), gate.size(1));
    torch::Tensor ws;
    if (ws_bytes > 0) ws = scratch(ws_bytes, gate);
    raise_on(ssb_scan_bwd_recompute_f32(gate.data_ptr<float>(), value.data_ptr<float>(), outGrad.data_ptr<float>(),
                                        gateGradOut.data_ptr<float>(), valueGradOut.data_ptr<float>(), gate.size(0),
                                        gate.size(1), nullptr, nullptr, ws_bytes ? ws.data_ptr() : nullptr, ws_bytes,
                                        current_stream()),
             "scan_backward_recompute");
}

// ---- channels-last ---------------------------------------------------------------------
void check_cpb(int64_t cpb) {
    // The reference asserts the same set (src/scanscam_cuda.cu:566); the value is a tuning hint
    // that does not change results and is not used by these kernels.
    TORCH_CHECK(cpb == 1 || cpb == 2 || cpb == 4 || cpb == 8 || cpb == 16 || cpb == 32,
                "channelsPerBlock must be one of 1, 2, 4, 8, 16, 32");
}

void transposed_linear_scan(torch::Tensor gate, torch::Tensor value, torch::Tensor output, int64_t channelsPerBlock) {
    check_tensor(gate, "gate");
    TORCH_CHECK(gate.dim() == 3, "gate must be 3-D [N, T, C]");
    check_same(gate, value, "value");
    check_same(gate, output, "output");
    // 16-bit storage is an addition, for channel counts the bulk-tensor kernels can describe
    check_dtype(gate, "transposed_linear_scan", gate.size(2) % 8 == 0);
    check_cpb(channelsPerBlock);
    c10::cuda::CUDAGuard guard(gate.device());
    int rc;
    if (is_16bit(gate)) {
        const size_t ws_bytes = ssb_scan_cl_h16_workspace_bytes(gate.size(0), gate.size(1), gate.size(2));
        torch::Tensor ws;
        if (ws_bytes > 0) ws = scratch(ws_bytes, gate);
        auto fn = gate.scalar_type() == torch::kBFloat16 ? ssb_scan_cl_fwd_bf16 : ssb_scan_cl_fwd_f16;
        rc = fn(gate.data_ptr(), value.data_ptr(), output.data_ptr(), gate.size(0), gate.size(1), gate.size(2),
                ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, current_stream());
    } else if (gate.scalar_type() == torch::kFloat32) {
        // the kernel that will run, and exactly the scratch it needs (none for the streaming kernels)
        const int variant = ssb_scan_cl_recommend(gate.size(0), gate.size(1), gate.size(2), 0,
                                                  aligned16(gate) && aligned16(value) && aligned16(output), 1);
        const size_t ws_bytes = ssb_scan_cl_variant_workspace_bytes(gate.size(0), gate.size(1), gate.size(2), variant, 0);
        torch::Tensor ws;
        if (ws_bytes > 0) ws = scratch(ws_bytes, gate);
        rc = ssb_scan_cl_fwd_f32_ex(gate.data_ptr<float>(), value.data_ptr<float>(), output.data_ptr<float>(),
                                    gate.size(0), gate.size(1), gate.size(2), variant, ws_bytes ? ws.data_ptr() : nullptr,
                                    ws_bytes, current_stream());
    } else {
        rc = ssb_scan_cl_fwd_f64(gate.data_ptr<double>(), value.data_ptr<double>(), output.data_ptr<double>(),
                                 gate.size(0), gate.size(1), gate.size(2), current_stream());
    }
    raise_on(rc, "transposed_linear_scan");
}

void transposed_linear_scan_backward(torch::Tensor gate, torch::Tensor output, torch::Tensor outGrad,
                                     torch::Tensor gateGradOut, torch::Tensor valueGradOut, int64_t channelsPerBlock) {
    check_tensor(gate, "gate");
    TORCH_CHECK(gate.dim() == 3, "gate must be 3-D [N, T, C]");
    check_same(gate, output, "output");
    check_same(gate, outGrad, "outGrad");
    check_same(gate, gateGradOut, "gateGradOut");
    check_same(gate, valueGradOut, "valueGradOut");
    check_dtype(gate, "transposed_linear_scan_backward", gate.size(2) % 8 == 0);
    check_cpb(channelsPerBlock);
    c10::cuda::CUDAGuard guard(gate.device());
    int rc;
    if (is_16bit(gate)) {
        const size_t ws_bytes = ssb_scan_cl_h16_workspace_bytes(gate.size(0), gate.size(1), gate.size(2));
        torch::Tensor ws;
        if (ws_bytes > 0) ws = scratch(ws_bytes, gate);
        auto fn = gate.scalar_type() == torch::kBFloat16 ? ssb_scan_cl_bwd_bf16 : ssb_scan_cl_bwd_f16;
        rc = fn(gate.data_ptr(), output.data_ptr(), outGrad.data_ptr(), gateGradOut.data_ptr(), valueGradOut.data_ptr(),
                gate.size(0), gate.size(1), gate.size(2), ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, current_stream());
    } else if (gate.scalar_type() == torch::kFloat32) {
        const int variant = ssb_scan_cl_recommend(gate.size(0), gate.size(1), gate.size(2), 1,
                                                  aligned16(gate) && aligned16(output) && aligned16(outGrad) &&
                                                      aligned16(gateGradOut) && aligned16(valueGradOut), 1);
        const size_t ws_bytes = ssb_scan_cl_variant_workspace_bytes(gate.size(0), gate.size(1), gate.size(2), variant, 1);
        torch::Tensor ws;
        if (ws_bytes > 0) ws = scratch(ws_bytes, gate);
        rc = ssb_scan_cl_bwd_f32_ex(gate.data_ptr<float>(), output.data_ptr<float>(), outGrad.data_ptr<float>(),
                                    gateGradOut.data_ptr<float>(), valueGradOut.data_ptr<float>(), gate.size(0),
                                    gate.size(1), gate.size(2), variant, ws_bytes ? ws.data_ptr() : nullptr, ws_bytes,
                                    current_stream());
    } else {
        rc = ssb_scan_cl_bwd_f64(gate.data_ptr<double>(), output.data_ptr<double>(), outGrad.data_ptr<double>(),
                                 gateGradOut.data_ptr<double>(), valueGradOut.data_ptr<double>(), gate.size(0),
                                 gate.size(1), gate.size(2), current_stream());
    }
    raise_on(rc, "transposed_linear_scan_backward");
}

// ---- channels-last with gate logits in (not in the reference) ------------------------------
void transposed_scan_sigmoid(torch::Tensor logits, torch::Tensor value, torch::Tensor output) {
    check_tensor(logits, "gate_logits");
    TORCH_CHECK(logits.dim() == 3 && (logits.scalar_type() == torch::kFloat32 || is_16bit(logits)),
                "gate_logits must be 3-D [N, T, C] float32, bfloat16 or float16");
    check_same(logits, value, "value");
    check_same(logits, output, "output");
    c10::cuda::CUDAGuard guard(logits.device());
    const int64_t N = logits.size(0), T = logits.size(1), C = logits.size(2);
    const size_t ws_bytes = is_16bit(logits) ? ssb_scan_cl_h16_workspace_bytes(N, T, C) : ssb_scan_cl_sigmoid_workspace_bytes(N, T, C);
    torch::Tensor ws;
    if (ws_bytes > 0) ws = scratch(ws_bytes, logits);
    void *wp = ws_bytes ? ws.data_ptr() : nullptr;
    int rc;
    if (logits.scalar_type() == torch::kFloat32)
        rc = ssb_scan_cl_sigmoid_fwd_f32(logits.data_ptr<float>(), value.data_ptr<float>(), output.data_ptr<float>(), N, T, C, wp,
                                         ws_bytes, current_stream());
    else
        rc = (logits.scalar_type() == torch::kBFloat16 ? ssb_scan_cl_sigmoid_fwd_bf16 : ssb_scan_cl_sigmoid_fwd_f16)(
            logits.data_ptr(), value.data_ptr(), output.data_ptr(), N, T, C, wp, ws_bytes, current_stream());
    raise_on(rc, "transposed_scan_sigmoid");
}

void transposed_scan_sigmoid_backward(torch::Tensor logits, torch::Tensor output, torch::Tensor outGrad,
                                      torch::Tensor logitsGradOut, torch::Tensor valueGradOut) {
    check_tensor(logits, "gate_logits");
    TORCH_CHECK(logits.dim() == 3 && (logits.scalar_type() == torch::kFloat32 || is_16bit(logits)),
                "gate_logits must be 3-D [N, T, C] float32, bfloat16 or float16");
    check_same(logits, output, "output");
    check_same(logits, outGrad, "outGrad");
    check_same(logits, logitsGradOut, "logitsGradOut");
    check_same(logits, valueGradOut, "valueGradOut");
    c10::cuda::CUDAGuard guard(logits.device());
    const int64_t N = logits.size(0), T = logits.size(1), C = logits.size(2);
    const size_t ws_bytes = is_16bit(logits) ? ssb_scan_cl_h16_workspace_bytes(N, T, C) : ssb_scan_cl_sigmoid_workspace_bytes(N, T, C);
    torch::Tensor ws;
    if (ws_bytes > 0) ws = scratch(ws_bytes, logits);
    void *wp = ws_bytes ? ws.data_ptr() : nullptr;
    int rc;
    if (logits.scalar_type() == torch::kFloat32)
        rc = ssb_scan_cl_sigmoid_bwd_f32(logits.data_ptr<float>(), output.data_ptr<float>(), outGrad.data_ptr<float>(),
                                         logitsGradOut.data_ptr<float>(), valueGradOut.data_ptr<float>(), N, T, C, wp, ws_bytes,
                                         current_stream());
    else
        rc = (logits.scalar_type() == torch::kBFloat16 ? ssb_scan_cl_sigmoid_bwd_bf16 : ssb_scan_cl_sigmoid_bwd_f16)(
            logits.data_ptr(), output.data_ptr(), outGrad.data_ptr(), logitsGradOut.data_ptr(), valueGradOut.data_ptr(), N, T, C,
            wp, ws_bytes, current_stream());
    raise_on(rc, "transposed_scan_sigmoid_backward");
}

// ---- sequence sharding (not in the reference) ------------------------------------------
void shard_reduce_forward(torch::Tensor gate, torch::Tensor value, torch::Tensor agg) {
    check_tensor(gate, "gate");
    TORCH_CHECK(gate.dim() == 2 && gate.scalar_type() == torch::kFloat32, "gate must be 2-D float32");
    check_same(gate, value, "value");
    check_tensor(agg, "agg");
    TORCH_CHECK(agg.scalar_type() == torch::kFloat32 && agg.numel() == 2 * gate.size(0), "agg must be float32 [rows, 2]");
    c10::cuda::CUDAGuard guard(gate.device());
    const size_t ws_bytes = ssb_shard_reduce_workspace_bytes(gate.size(0), gate.size(1));
    torch::Tensor ws;
    if (ws_bytes > 0) ws = scratch(ws_bytes, gate);
    raise_on(ssb_shard_reduce_fwd_f32(gate.data_ptr<float>(), value.data_ptr<float>(), agg.data_ptr<float>(),
                                      gate.size(0), gate.size(1), ws_bytes ? ws.data_ptr() : nullptr, ws_bytes,
                                      current_stream()),
             "shard_reduce_forward");
}

void shard_reduce_backward(torch::Tensor gate, torch::Tensor outGrad, torch::Tensor agg) {
    check_tensor(gate, "gate");
    TORCH_CHECK(gate.dim() == 2 && gate.scalar_type() == torch::kFloat32, "gate must be 2-D float32");
    check_same(gate, outGrad, "outGrad");
    check_tensor(agg, "agg");
    TORCH_CHECK(agg.scalar_type() == torch::kFloat32 && agg.numel() == 2 * gate.size(0), "agg must be float32 [rows, 2]");
    c10::cuda::CUDAGuard guard(gate.device());
    const size_t ws_bytes = ssb_shard_reduce_workspace_bytes(gate.size(0), gate.size(1));
    torch::Tensor ws;
    if (ws_bytes > 0) ws = scratch(ws_bytes, gate);
    raise_on(ssb_shard_reduce_bwd_f32(gate.data_ptr<float>(), outGrad.data_ptr<float>(), agg.data_ptr<float>(),
                                      gate.size(0), gate.size(1), ws_bytes ? ws.data_ptr() : nullptr, ws_bytes,
                                      current_stream()),
             "shard_reduce_backward");
}

// Row maps with early termination (see ssb_shard_map_*): `walked`, when given, is a one-element
// int64 CUDA tensor that accumulates the number of elements read per tensor.
void shard_map_impl(bool backward, const torch::Tensor &gate, const torch::Tensor &other, torch::Tensor &agg, double cut,
                    const c10::optional<torch::Tensor> &walked, const char *op) {
    check_tensor(gate, "gate");
    TORCH_CHECK(gate.dim() == 2 && gate.scalar_type() == torch::kFloat32, "gate must be 2-D float32");
    check_same(gate, other, backward ? "outGrad" : "value");
    check_tensor(agg, "agg");
    TORCH_CHECK(agg.scalar_type() == torch::kFloat32 && agg.numel() == 2 * gate.size(0), "agg must be float32 [rows, 2]");
    unsigned long long *counter = nullptr;
    if (walked.has_value() && walked->defined()) {
        check_tensor(*walked, "walked");
        TORCH_CHECK(walked->scalar_type() == torch::kInt64 && walked->numel() == 1 && walked->device() == gate.device(),
                    "walked must be a one-element int64 tensor on the gate's device");
        counter = reinterpret_cast<unsigned long long *>(walked->data_ptr<int64_t>());
    }
    c10::cuda::CUDAGuard guard(gate.device());
    auto fn = backward ? ssb_shard_map_bwd_f32 : ssb_shard_map_fwd_f32;
    raise_on(fn(gate.data_ptr<float>(), other.data_ptr<float>(), agg.data_ptr<float>(), gate.size(0), gate.size(1), (float)cut,
                counter, current_stream()),
             op);
}
void shard_map_forward(torch::Tensor gate, torch::Tensor value, torch::Tensor agg, double cut,
                       c10::optional<torch::Tensor> walked) {
    shard_map_impl(false, gate, value, agg, cut, walked, "shard_map_forward");
}
void shard_map_backward(torch::Tensor gate, torch::Tensor outGrad, torch::Tensor agg, double cut,
                        c10::optional<torch::Tensor> walked) {
    shard_map_impl(true, gate, outGrad, agg, cut, walked, "shard_map_backward");
}

void shard_carry(torch::Tensor aggs, int64_t shard, bool reverse, torch::Tensor carry) {
    check_tensor(aggs, "aggs");
    check_tensor(carry, "carry");
    TORCH_CHECK(aggs.dim() == 3 && aggs.size(2) == 2 && aggs.scalar_type() == torch::kFloat32,
                "aggs must be float32 [n_shards, rows, 2]");
    TORCH_CHECK(carry.scalar_type() == torch::kFloat32 && carry.numel() == aggs.size(1), "carry must be float32 [rows]");
    c10::cuda::CUDAGuard guard(aggs.device());
    raise_on(ssb_shard_carry_f32(aggs.data_ptr<float>(), (int)aggs.size(0), (int)shard, reverse ? 1 : 0, aggs.size(1),
                                 carry.data_ptr<float>(), current_stream()),
             "shard_carry");
}

int64_t device_status() {
    int detail = 0;
    return ssb_device_status(&detail);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("simple_linear_scan", &simple_linear_scan, "Forward scan over the last axis of [rows, T]");
    m.def("coalesced_linear_scan", &coalesced_linear_scan, "Forward scan over the last axis of [rows, T]");
    m.def("blocked_linear_scan", &blocked_linear_scan, "Forward scan over the last axis of [rows, T]");
    m.def("simple_linear_scan_backward", &simple_linear_scan_backward, "Fused reverse scan: both gradients in one pass");
    m.def("blocked_linear_scan_backward", &blocked_linear_scan_backward, "Fused reverse scan: both gradients in one pass");
    m.def("transposed_linear_scan", &transposed_linear_scan, "Forward scan over axis 1 of [N, T, C]");
    m.def("transposed_linear_scan_backward", &transposed_linear_scan_backward, "Fused reverse scan on [N, T, C]");
    m.def("scan_forward_ex", &scan_forward_ex, "Forward scan with optional carry-in and pinned kernel family",
          py::arg("gate"), py::arg("value"), py::arg("output"), py::arg("h_in") = py::none(), py::arg("variant") = 0);
    m.def("scan_backward_ex", &scan_backward_ex, "Fused backward with optional carries and pinned kernel family",
          py::arg("gate"), py::arg("output"), py::arg("outGrad"), py::arg("gateGradOut"), py::arg("valueGradOut"),
          py::arg("c_in") = py::none(), py::arg("h_prev") = py::none(), py::arg("variant") = 0);
    m.def("scan_sigmoid_forward", &scan_sigmoid_forward, "Forward scan with gate = sigmoid(logits) computed in the kernel");
    m.def("scan_sigmoid_backward", &scan_sigmoid_backward, "Fused backward returning the gradient w.r.t. the gate logits");
    m.def("transposed_scan_sigmoid", &transposed_scan_sigmoid, "Channels-last forward scan with gate = sigmoid(logits)");
    m.def("transposed_scan_sigmoid_backward", &transposed_scan_sigmoid_backward,
          "Channels-last fused backward returning the gradient w.r.t. the gate logits");
    m.def("scan_backward_recompute", &scan_backward_recompute,
          "Fused backward from (gate, value, outGrad): rebuilds the forward's output instead of reading it");
    m.def("shard_reduce_forward", &shard_reduce_forward, "Per-row aggregate map (A, B) of a sequence shard");
    m.def("shard_reduce_backward", &shard_reduce_backward, "Per-row aggregate map (A, D) of the reverse recurrence");
    m.def("shard_map_forward", &shard_map_forward, "Map (A, B) of a sequence shard, walked from its end until |A| <= cut",
          py::arg("gate"), py::arg("value"), py::arg("agg"), py::arg("cut") = 0.0, py::arg("walked") = py::none());
    m.def("shard_map_backward", &shard_map_backward, "Map (A, D) of the reverse recurrence, walked from the shard's start until |A| <= cut",
          py::arg("gate"), py::arg("outGrad"), py::arg("agg"), py::arg("cut") = 0.0, py::arg("walked") = py::none());
    m.def("shard_carry", &shard_carry, "Fold gathered shard aggregates into the carry entering one shard");
    m.def("device_status", &device_status, "Synchronise and return/clear the device-side status code");
}
