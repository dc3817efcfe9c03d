// Torch binding of the sm_100a residual LayerNorm path: module `gfx1010_kernels._C`.
//
// Thin host layer over the C ABI declared in rln_sm100.h.  It owns what the
// ABI deliberately does not: tensor validation with the reference's error
// texts, output allocation through the caching allocator, the torch CUDA
// generator (Philox seed/offset), the deterministic-algorithms switch and the
// autograd node.  It exports the same three functions, with the same
// positional signatures, as the reference binding
// (csrc/residual_layer_norm_bindings.cpp:131-141 of T-vaccari/gfx1010-kernels):
//   residual_layer_norm            autograd-connected   (:101-125)
//   residual_layer_norm_forward    raw forward          (csrc/residual_layer_norm.h:10-24)
//   residual_layer_norm_backward   raw backward         (csrc/residual_layer_norm.h:27-42)
// The four launch integers (threads, block_rows, parameter_threads,
// parameter_groups) are gfx1010 tuning knobs: they are range-checked exactly
// as the reference does and otherwise unused, because the sm_100a launch
// geometry is fixed per hidden size.  Error texts keep the word "HIP" so that
// callers matching on them keep working.
#include <torch/extension.h>
#include <torch/csrc/autograd/custom_function.h>

#include <ATen/Context.h>
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAGeneratorImpl.h>
#include <c10/cuda/CUDAGraphsC10Utils.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <atomic>
#include <cstdint>
#include <mutex>
#include <tuple>
#include <vector>

#include "rln_sm100.h"

namespace {

constexpr int64_t kMaskColumnsPerWord = 32;

bool native_hidden(int64_t hidden) {
    return hidden == 128 || hidden == 256 || hidden == 384 || hidden == 512
        || hidden == 768 || hidden == 1024;
}

// Element types of `branch` (the reference's float16 / float32, plus bfloat16)
// and of `normalized` / `grad_normalized` (float32 as in the reference, or one
// of the two 16-bit types); both use the RLN_DTYPE_* codes.
bool element_dtype_supported(at::ScalarType type) {
    return type == at::kHalf || type == at::kFloat || type == at::kBFloat16;
}

int32_t element_dtype_code(at::ScalarType type) {
    if (type == at::kHalf) {
        return RLN_DTYPE_FLOAT16;
    }
    return type == at::kBFloat16 ? RLN_DTYPE_BFLOAT16 : RLN_DTYPE_FLOAT32;
}

at::ScalarType branch_dtype_from_code(int64_t code) {
    TORCH_CHECK(
        code == RLN_BRANCH_FLOAT32 || code == RLN_BRANCH_FLOAT16 || code == RLN_BRANCH_BFLOAT16,
        "branch_is_half must be False/0 (float32), True/1 (float16) or 2 (bfloat16)");
    if (code == RLN_BRANCH_FLOAT16) {
        return at::kHalf;
    }
    return code == RLN_BRANCH_BFLOAT16 ? at::kBFloat16 : at::kFloat;
}

// Element type of `normalized`: float32 is the reference's contract; float16
// and bfloat16 are the narrow outputs this build adds (codes RLN_DTYPE_*).
at::ScalarType normalized_dtype_from_code(int64_t code) {
    TORCH_CHECK(
        code == RLN_DTYPE_FLOAT32 || code == RLN_DTYPE_FLOAT16 || code == RLN_DTYPE_BFLOAT16,
        "normalized_dtype must be 0 (float32), 1 (float16) or 2 (bfloat16)");
    if (code == RLN_DTYPE_FLOAT16) {
        return at::kHalf;
    }
    return code == RLN_DTYPE_BFLOAT16 ? at::kBFloat16 : at::kFloat;
}

void check_status(int status, const char* what) {
    if (status == RLN_OK) {
        return;
    }
    if (status == RLN_ERR_CUDA) {
        const auto error = static_cast<cudaError_t>(rln_sm100_last_cuda_error());
        TORCH_CHECK(
            false, what, " failed: CUDA error: ", cudaGetErrorString(error));
    }
    TORCH_CHECK(false, what, " failed: ", rln_sm100_status_string(status));
}

// Same ladder, order and texts as check_forward_inputs
// (csrc/residual_layer_norm_kernel.hip:26-76).
void check_forward_inputs(
    const at::Tensor& x,
    const at::Tensor& branch,
    const at::Tensor& weight,
    const at::Tensor& bias,
    double dropout_p,
    double eps,
    int64_t threads) {
    TORCH_CHECK(x.is_cuda(), "x must be a HIP tensor");
    TORCH_CHECK(
        branch.is_cuda() && weight.is_cuda() && bias.is_cuda(),
        "branch, weight and bias must be HIP tensors");
    TORCH_CHECK(
        x.device() == branch.device() && x.device() == weight.device()
            && x.device() == bias.device(),
        "all tensors must be on the same HIP device");
    TORCH_CHECK(x.scalar_type() == at::kFloat, "x must use float32");
    TORCH_CHECK(
        element_dtype_supported(branch.scalar_type()), "branch must use float16 or float32");
    TORCH_CHECK(
        weight.scalar_type() == at::kFloat && bias.scalar_type() == at::kFloat,
        "weight and bias must use float32");
    TORCH_CHECK(x.dim() >= 2, "x must have at least two dimensions");
    TORCH_CHECK(branch.sizes() == x.sizes(), "branch must match x");
    const int64_t hidden = x.size(-1);
    TORCH_CHECK(
        weight.dim() == 1 && weight.size(0) == hidden && bias.dim() == 1
            && bias.size(0) == hidden,
        "weight and bias must match the hidden size");
    TORCH_CHECK(
        x.is_contiguous() && branch.is_contiguous() && weight.is_contiguous()
            && bias.is_contiguous(),
        "all tensors must be contiguous");
    TORCH_CHECK(x.numel() > 0, "empty tensors are unsupported");
    TORCH_CHECK(native_hidden(hidden), "unsupported native hidden size: ", hidden);
    TORCH_CHECK(
        threads == 128 || threads == 192 || threads == 256,
        "threads must be 128, 192 or 256");
    TORCH_CHECK(dropout_p >= 0.0 && dropout_p < 1.0, "dropout_p must be in [0, 1)");
    TORCH_CHECK(eps > 0.0, "eps must be positive");
}

// Same ladder, order and texts as check_backward_inputs
// (csrc/residual_layer_norm_kernel.hip:79-166).
void check_backward_inputs(
    const at::Tensor& grad_updated,
    const at::Tensor& grad_normalized,
    const at::Tensor& updated,
    const at::Tensor& weight,
    const at::Tensor& mean,
    const at::Tensor& rstd,
    const at::Tensor& dropout_mask,
    double dropout_p,
    bool training,
    int64_t threads,
    int64_t block_rows,
    int64_t parameter_threads,
    int64_t parameter_groups) {
    TORCH_CHECK(updated.is_cuda(), "updated must be a HIP tensor");
    TORCH_CHECK(
        grad_updated.device() == updated.device()
            && grad_normalized.device() == updated.device()
            && weight.device() == updated.device() && mean.device() == updated.device()
            && rstd.device() == updated.device(),
        "all backward tensors must be on the same HIP device");
    // grad_normalized has the type the forward stored `normalized` in; the
    // reference's float32 case keeps its message.
    TORCH_CHECK(
        grad_updated.scalar_type() == at::kFloat
            && element_dtype_supported(grad_normalized.scalar_type())
            && updated.scalar_type() == at::kFloat && weight.scalar_type() == at::kFloat
            && mean.scalar_type() == at::kFloat && rstd.scalar_type() == at::kFloat,
        "all backward tensors must use float32");
    TORCH_CHECK(updated.dim() >= 2, "updated must have at least two dimensions");
    TORCH_CHECK(updated.numel() > 0, "empty tensors are unsupported");
    TORCH_CHECK(
        grad_updated.sizes() == updated.sizes()
            && grad_normalized.sizes() == updated.sizes(),
        "output gradients must match updated");
    const int64_t hidden = updated.size(-1);
    TORCH_CHECK(native_hidden(hidden), "unsupported native hidden size: ", hidden);
    const int64_t row_count = updated.numel() / hidden;
    TORCH_CHECK(
        weight.dim() == 1 && weight.size(0) == hidden,
        "weight must match the hidden size");
    TORCH_CHECK(
        mean.numel() == row_count && rstd.numel() == row_count,
        "mean and rstd must match the row count");
    TORCH_CHECK(
        grad_updated.is_contiguous() && grad_normalized.is_contiguous()
            && updated.is_contiguous() && weight.is_contiguous() && mean.is_contiguous()
            && rstd.is_contiguous(),
        "all backward tensors must be contiguous");
    TORCH_CHECK(
        threads == 128 || threads == 192 || threads == 256,
        "threads must be 128, 192 or 256");
    TORCH_CHECK(
        block_rows == 16 || block_rows == 32 || block_rows == 64 || block_rows == 128,
        "block_rows must be 16, 32, 64 or 128");
    TORCH_CHECK(
        parameter_threads == 64 || parameter_threads == 128 || parameter_threads == 256,
        "parameter_threads must be 64, 128 or 256");
    TORCH_CHECK(
        parameter_groups > 0 && parameter_groups <= row_count,
        "parameter_groups must be in [1, row_count]");
    TORCH_CHECK(dropout_p >= 0.0 && dropout_p < 1.0, "dropout_p must be in [0, 1)");
    const bool dropout = training && dropout_p > 0.0;
    if (dropout) {
        TORCH_CHECK(
            dropout_mask.is_cuda() && dropout_mask.device() == updated.device(),
            "dropout_mask must be on the same HIP device");
        TORCH_CHECK(
            dropout_mask.scalar_type() == at::kInt && dropout_mask.is_contiguous(),
            "dropout_mask must be a contiguous int32 tensor");
        TORCH_CHECK(
            dropout_mask.numel() == row_count * (hidden / kMaskColumnsPerWord),
            "dropout_mask has the wrong size");
    }
}

}  // namespace

namespace {

std::atomic<bool> graph_capture_allowed{false};

// Validation, allocation and launch shared by the three forward entries.  The
// Philox state is either immediate (device_seed == nullptr) or behind device
// pointers (a launch that is being recorded into a CUDA graph).
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> forward_launch(
    const at::Tensor& x,
    const at::Tensor& branch,
    const at::Tensor& weight,
    const at::Tensor& bias,
    double dropout_p,
    double eps,
    bool training,
    int64_t threads,
    uint64_t seed,
    uint64_t offset,
    const int64_t* device_seed,
    const int64_t* device_offset,
    int64_t row_base,
    int64_t normalized_dtype) {
    check_forward_inputs(x, branch, weight, bias, dropout_p, eps, threads);
    TORCH_CHECK(row_base >= 0, "row_base must be non-negative");
    const at::ScalarType normalized_type = normalized_dtype_from_code(normalized_dtype);
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t hidden = x.size(-1);
    const int64_t row_count = x.numel() / hidden;
    auto updated = at::empty_like(x);
    auto normalized = at::empty(x.sizes(), x.options().dtype(normalized_type));
    auto mean = at::empty({row_count}, x.options());
    auto rstd = at::empty({row_count}, x.options());
    const bool dropout = training && dropout_p > 0.0;
    auto dropout_mask = at::empty(
        {dropout ? row_count * (hidden / kMaskColumnsPerWord) : 0},
        x.options().dtype(at::kInt));
    const auto stream = c10::cuda::getCurrentCUDAStream(x.device().index()).stream();
    uint32_t* mask_pointer =
        dropout ? reinterpret_cast<uint32_t*>(dropout_mask.data_ptr<int32_t>()) : nullptr;
    const int32_t branch_dtype = element_dtype_code(branch.scalar_type());
    int status = RLN_OK;
    if (device_seed != nullptr) {
        status = rln_sm100_forward_device_rng(
            x.data_ptr<float>(), branch.data_ptr(), weight.data_ptr<float>(),
            bias.data_ptr<float>(), updated.data_ptr<float>(), normalized.data_ptr(),
            mean.data_ptr<float>(), rstd.data_ptr<float>(), mask_pointer, row_count,
            static_cast<int32_t>(hidden), branch_dtype,
            static_cast<int32_t>(normalized_dtype), dropout ? 1 : 0,
            static_cast<float>(dropout_p), static_cast<float>(eps), device_seed, device_offset,
            offset, row_base, stream);
    } else {
        status = rln_sm100_forward(
            x.data_ptr<float>(), branch.data_ptr(), weight.data_ptr<float>(),
            bias.data_ptr<float>(), updated.data_ptr<float>(), normalized.data_ptr(),
            mean.data_ptr<float>(), rstd.data_ptr<float>(), mask_pointer, row_count,
            static_cast<int32_t>(hidden), branch_dtype,
            static_cast<int32_t>(normalized_dtype), dropout ? 1 : 0,
            static_cast<float>(dropout_p), static_cast<float>(eps), seed, offset, row_base,
            stream);
    }
    check_status(status, "residual_layer_norm_forward");
    return {updated, normalized, mean, rstd, dropout_mask};
}

}  // namespace

// Forward with an explicit Philox (seed, offset) and a global row offset: the
// entry a row-sharded caller uses so that every shard reproduces the mask of
// the unsharded call.  Consumes no generator state.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor>
residual_layer_norm_forward_seeded(
    const at::Tensor& x,
    const at::Tensor& branch,
    const at::Tensor& weight,
    const at::Tensor& bias,
    double dropout_p,
    double eps,
    bool training,
    int64_t threads,
    int64_t seed,
    int64_t offset,
    int64_t row_base,
    int64_t normalized_dtype) {
    return forward_launch(
        x, branch, weight, bias, dropout_p, eps, training, threads,
        static_cast<uint64_t>(seed), static_cast<uint64_t>(offset), nullptr, nullptr, row_base,
        normalized_dtype);
}

// Counterpart of residual_layer_norm_forward_hip
// (csrc/residual_layer_norm_kernel.hip:1720-1827): the Philox state comes from
// the device's default torch generator, advanced under its mutex by the same
// increment the reference uses (:1767-1774) so that the generator state after
// the call matches the reference's; eval mode and p == 0 consume no generator
// state.  Graph capture with dropout is refused as in the reference
// (:1758-1777) unless set_graph_capture_allowed(true) was called, in which
// case the launch takes torch's graph-safe generator state by pointer.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor>
residual_layer_norm_forward_cuda(
    const at::Tensor& x,
    const at::Tensor& branch,
    const at::Tensor& weight,
    const at::Tensor& bias,
    double dropout_p,
    double eps,
    bool training,
    int64_t threads,
    int64_t normalized_dtype) {
    check_forward_inputs(x, branch, weight, bias, dropout_p, eps, threads);
    normalized_dtype_from_code(normalized_dtype);  // validate before touching the generator
    uint64_t seed = 0;
    uint64_t offset = 0;
    const int64_t* device_seed = nullptr;
    const int64_t* device_offset = nullptr;
    if (training && dropout_p > 0.0) {
        c10::cuda::CUDAGuard guard(x.device());
        const bool capturing = c10::cuda::currentStreamCaptureStatusMayInitCtx()
            != c10::cuda::CaptureStatus::None;
        TORCH_CHECK(
            !capturing || graph_capture_allowed.load(),
            "native residual LayerNorm dropout does not support HIP graph capture");
        auto* generator = at::get_generator_or_default<at::CUDAGeneratorImpl>(
            std::nullopt, at::cuda::detail::getDefaultCUDAGenerator(x.device().index()));
        const uint64_t hidden = static_cast<uint64_t>(x.size(-1));
        const uint64_t randoms_per_thread = (hidden + threads - 1) / threads;
        const uint64_t increment = ((randoms_per_thread + 3) / 4) * 4;
        at::PhiloxCudaState state;
        {
            std::lock_guard<std::mutex> lock(generator->mutex_);
            state = generator->philox_cuda_state(increment);
        }
        if (state.captured_) {
            TORCH_CHECK(
                graph_capture_allowed.load(),
                "native residual LayerNorm dropout does not support HIP graph capture");
            // graph-safe generator state: read on the device at replay time
            device_seed = state.seed_.ptr;
            device_offset = state.offset_.ptr;
            offset = state.offset_intragraph_;
        } else {
            seed = state.seed_.val;
            offset = state.offset_.val;
        }
    }
    return forward_launch(
        x, branch, weight, bias, dropout_p, eps, training, threads, seed, offset, device_seed,
        device_offset, 0, normalized_dtype);
}

// Counterpart of residual_layer_norm_backward_hip
// (csrc/residual_layer_norm_kernel.hip:1830-2036).  grad_weight and grad_bias
// are select() views of one [2, hidden] allocation (:1879-1887); the
// deterministic switch is read here, at backward time (:1864-1865).
std::vector<at::Tensor> residual_layer_norm_backward_cuda(
    const at::Tensor& grad_updated,
    const at::Tensor& grad_normalized,
    const at::Tensor& updated,
    const at::Tensor& weight,
    const at::Tensor& mean,
    const at::Tensor& rstd,
    const at::Tensor& dropout_mask,
    double dropout_p,
    bool training,
    int64_t branch_is_half,
    int64_t threads,
    int64_t block_rows,
    int64_t parameter_threads,
    int64_t parameter_groups,
    bool compute_parameter_gradients) {
    // `branch_is_half` keeps the reference's name and position; it is an integer
    // here so that False/True still mean float32/float16 and 2 selects bfloat16.
    const at::ScalarType branch_type = branch_dtype_from_code(branch_is_half);
    check_backward_inputs(
        grad_updated,
        grad_normalized,
        updated,
        weight,
        mean,
        rstd,
        dropout_mask,
        dropout_p,
        training,
        threads,
        block_rows,
        parameter_threads,
        parameter_groups);
    c10::cuda::CUDAGuard guard(updated.device());
    const int64_t hidden = updated.size(-1);
    const int64_t row_count = updated.numel() / hidden;
    const bool deterministic = at::globalContext().deterministicAlgorithms();
    const bool dropout = training && dropout_p > 0.0;
    auto grad_x = at::empty_like(updated);
    auto grad_branch = at::empty(
        updated.sizes(),
        updated.options().dtype(branch_type));
    at::Tensor parameter_gradients;
    at::Tensor grad_weight;
    at::Tensor grad_bias;
    at::Tensor workspace;
    int64_t workspace_bytes = 0;
    if (compute_parameter_gradients) {
        parameter_gradients = at::empty({2, hidden}, updated.options());
        grad_weight = parameter_gradients.select(0, 0);
        grad_bias = parameter_gradients.select(0, 1);
        workspace_bytes = rln_sm100_backward_workspace_bytes(
            row_count, static_cast<int32_t>(hidden), deterministic ? 1 : 0);
        TORCH_CHECK(
            workspace_bytes >= 0,
            "residual_layer_norm_backward failed: ",
            rln_sm100_status_string(static_cast<int>(workspace_bytes)));
        if (workspace_bytes > 0) {
            workspace = at::empty(
                {workspace_bytes / static_cast<int64_t>(sizeof(float))}, updated.options());
        }
    }
    const auto stream =
        c10::cuda::getCurrentCUDAStream(updated.device().index()).stream();
    const int status = rln_sm100_backward(
        grad_updated.data_ptr<float>(),
        grad_normalized.data_ptr(),
        updated.data_ptr<float>(),
        weight.data_ptr<float>(),
        mean.data_ptr<float>(),
        rstd.data_ptr<float>(),
        dropout ? reinterpret_cast<const uint32_t*>(dropout_mask.data_ptr<int32_t>())
                : nullptr,
        grad_x.data_ptr<float>(),
        grad_branch.data_ptr(),
        compute_parameter_gradients ? parameter_gradients.data_ptr<float>() : nullptr,
        workspace.defined() ? workspace.data_ptr() : nullptr,
        workspace_bytes,
        row_count,
        static_cast<int32_t>(hidden),
        element_dtype_code(branch_type),
        element_dtype_code(grad_normalized.scalar_type()),
        dropout ? 1 : 0,
        static_cast<float>(dropout_p),
        deterministic ? 1 : 0,
        stream);
    check_status(status, "residual_layer_norm_backward");
    return {grad_x, grad_branch, grad_weight, grad_bias};
}

namespace {

// Autograd node; same saved state and gradient slots as
// ResidualLayerNormFunction (csrc/residual_layer_norm_bindings.cpp:10-98).
class ResidualLayerNormFunction
    : public torch::autograd::Function<ResidualLayerNormFunction> {
 public:
    static torch::autograd::variable_list forward(
        torch::autograd::AutogradContext* ctx,
        torch::autograd::Variable x,
        torch::autograd::Variable branch,
        torch::autograd::Variable weight,
        torch::autograd::Variable bias,
        double dropout_p,
        double eps,
        bool training,
        int64_t threads,
        int64_t block_rows,
        int64_t parameter_threads,
        int64_t parameter_groups,
        int64_t normalized_dtype) {
        auto result = residual_layer_norm_forward_cuda(
            x, branch, weight, bias, dropout_p, eps, training, threads, normalized_dtype);
        auto updated = std::get<0>(result);
        auto normalized = std::get<1>(result);
        ctx->save_for_backward(
            {updated, weight, std::get<2>(result), std::get<3>(result), std::get<4>(result)});
        ctx->set_materialize_grads(false);
        ctx->saved_data["dropout_p"] = dropout_p;
        ctx->saved_data["training"] = training;
        ctx->saved_data["branch_dtype"] =
            static_cast<int64_t>(element_dtype_code(branch.scalar_type()));
        ctx->saved_data["threads"] = threads;
        ctx->saved_data["block_rows"] = block_rows;
        ctx->saved_data["parameter_threads"] = parameter_threads;
        ctx->saved_data["parameter_groups"] = parameter_groups;
        return {updated, normalized};
    }

    static torch::autograd::variable_list backward(
        torch::autograd::AutogradContext* ctx,
        torch::autograd::variable_list grad_outputs) {
        auto saved = ctx->get_saved_variables();
        const bool has_grad_normalized = grad_outputs[1].defined();
        auto grad_updated = grad_outputs[0].defined() ? grad_outputs[0].contiguous()
                                                      : at::zeros_like(saved[0]);
        auto grad_normalized = has_grad_normalized ? grad_outputs[1].contiguous()
                                                   : at::zeros_like(saved[0]);
        auto gradients = residual_layer_norm_backward_cuda(
            grad_updated,
            grad_normalized,
            saved[0],
            saved[1],
            saved[2],
            saved[3],
            saved[4],
            ctx->saved_data["dropout_p"].toDouble(),
            ctx->saved_data["training"].toBool(),
            ctx->saved_data["branch_dtype"].toInt(),
            ctx->saved_data["threads"].toInt(),
            ctx->saved_data["block_rows"].toInt(),
            ctx->saved_data["parameter_threads"].toInt(),
            ctx->saved_data["parameter_groups"].toInt(),
            has_grad_normalized);
        torch::autograd::variable_list result(12);
        result[0] = gradients[0];
        result[1] = gradients[1];
        if (has_grad_normalized) {
            result[2] = gradients[2];
            result[3] = gradients[3];
        }
        return result;
    }
};

torch::autograd::variable_list residual_layer_norm_autograd(
    const at::Tensor& x,
    const at::Tensor& branch,
    const at::Tensor& weight,
    const at::Tensor& bias,
    double dropout_p,
    double eps,
    bool training,
    int64_t threads,
    int64_t block_rows,
    int64_t parameter_threads,
    int64_t parameter_groups,
    int64_t normalized_dtype) {
    return ResidualLayerNormFunction::apply(
        x,
        branch,
        weight,
        bias,
        dropout_p,
        eps,
        training,
        threads,
        block_rows,
        parameter_threads,
        parameter_groups,
        normalized_dtype);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, module) {
    namespace py = pybind11;
    // Positional order and arity are the reference's
    // (csrc/residual_layer_norm_bindings.cpp:131-141); `normalized_dtype` is an
    // optional trailing addition (0 float32 -- the reference's output type --,
    // 1 float16, 2 bfloat16).  The backward takes the type from grad_normalized.
    module.def(
        "residual_layer_norm", &residual_layer_norm_autograd,
        py::arg("x"), py::arg("branch"), py::arg("weight"), py::arg("bias"),
        py::arg("dropout_p"), py::arg("eps"), py::arg("training"), py::arg("threads"),
        py::arg("block_rows"), py::arg("parameter_threads"), py::arg("parameter_groups"),
        py::arg("normalized_dtype") = 0);
    module.def(
        "residual_layer_norm_forward", &residual_layer_norm_forward_cuda,
        py::arg("x"), py::arg("branch"), py::arg("weight"), py::arg("bias"),
        py::arg("dropout_p"), py::arg("eps"), py::arg("training"), py::arg("threads"),
        py::arg("normalized_dtype") = 0);
    module.def("residual_layer_norm_backward", &residual_layer_norm_backward_cuda);
    module.def(
        "residual_layer_norm_forward_seeded", &residual_layer_norm_forward_seeded,
        py::arg("x"), py::arg("branch"), py::arg("weight"), py::arg("bias"),
        py::arg("dropout_p"), py::arg("eps"), py::arg("training"), py::arg("threads"),
        py::arg("seed"), py::arg("offset"), py::arg("row_base"),
        py::arg("normalized_dtype") = 0);
    module.def("abi_version", &rln_sm100_abi_version);
    module.def("set_graph_capture_allowed", [](bool allowed) {
        graph_capture_allowed.store(allowed);
    });
    module.def("graph_capture_allowed", []() { return graph_capture_allowed.load(); });
}
