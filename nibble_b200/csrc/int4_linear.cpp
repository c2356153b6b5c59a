// Torch operator shim: registers w4a16::linear and w4a16::dequantize for the CUDA dispatch key
// with the schemas of the reference's csrc/int4_linear.cpp:16-28, validates tensors the way its
// int4_linear_cuda / int4_dequantize_cuda do (csrc/int4_linear_kernel.cu:646-691, 809-841: every
// violation is a TORCH_CHECK, i.e. a Python RuntimeError), allocates the output from the caching
// allocator and hands raw pointers plus the current stream to the C ABI in include/w4a16_b200.h.
// No kernel lives here.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>

#include "../../include/w4a16_b200.h"

namespace {

// Split-K scratch, one buffer per (device, stream) so calls on different streams never share it.
// Allocated zero-filled on first use and kept for the life of the process; the first call on a
// stream should therefore happen before that stream is captured into a CUDA graph.
constexpr int64_t kWorkspaceBytes = 40 << 20;   // largest request of the shapes in the bench tables: 33 MiB (M = 512 on 8192 x 8192 takes none; M = 256 does)

at::Tensor& workspace_for(const at::Device& device, cudaStream_t stream) {
    static std::mutex mutex;
    static auto* cache = new std::map<std::pair<int, cudaStream_t>, at::Tensor>();
    std::lock_guard<std::mutex> lock(mutex);
    auto key = std::make_pair(static_cast<int>(device.index()), stream);
    auto it = cache->find(key);
    if (it == cache->end()) {
        it = cache->emplace(key, at::zeros({kWorkspaceBytes}, at::TensorOptions().dtype(at::kByte).device(device))).first;
    }
    return it->second;
}

// W4A16_ROWS_PER_WARP selects how many output rows one lane owns: 2 (one 16-row tile per warp) or
// 4 (two tiles); 1 is accepted for compatibility and means 2.  Anything else is an error, as in
// the reference (csrc/int4_linear_kernel.cu:481-491).
int row_tiles_from_env() {
    const char* choice = std::getenv("W4A16_ROWS_PER_WARP");
    if (choice == nullptr) return 0;
    const int rows = std::atoi(choice);
    TORCH_CHECK(rows == 1 || rows == 2 || rows == 4, "W4A16_ROWS_PER_WARP must be 1, 2, or 4");
    return rows == 4 ? 2 : 1;
}

uint32_t flags_from_env() {
    uint32_t flags = 0;
    const char* decode = std::getenv("W4A16_DECODE");
    if (decode != nullptr && std::strcmp(decode, "generic") == 0) flags |= W4A16_FLAG_FORCE_GENERIC;
    const char* pdl = std::getenv("W4A16_PDL");
    if (pdl != nullptr && std::strcmp(pdl, "1") == 0) flags |= W4A16_FLAG_PROGRAMMATIC_LAUNCH;
    return flags;
}

void check_status(int status, const char* what) {
    TORCH_CHECK(status == W4A16_OK, what, " failed: ", w4a16_status_string(status));
}

at::Tensor linear_impl(const at::Tensor& activations, const at::Tensor& packed_weights, const at::Tensor& scales,
                       int64_t group_size, bool out_f32) {
    TORCH_CHECK(activations.is_cuda(), "activations must be a CUDA tensor");
    TORCH_CHECK(packed_weights.is_cuda(), "packed_weights must be a CUDA tensor");
    TORCH_CHECK(scales.is_cuda(), "scales must be a CUDA tensor");
    TORCH_CHECK(activations.device() == packed_weights.device() && activations.device() == scales.device(),
                "all inputs must be on the same CUDA device");
    TORCH_CHECK(activations.scalar_type() == at::kHalf, "activations must have dtype torch.float16");
    TORCH_CHECK(packed_weights.scalar_type() == at::kByte, "packed_weights must have dtype torch.uint8");
    TORCH_CHECK(scales.scalar_type() == at::kHalf, "scales must have dtype torch.float16");
    TORCH_CHECK(activations.dim() == 2, "activations must have shape [M, K]");
    TORCH_CHECK(packed_weights.dim() == 2, "packed_weights must have shape [N, K / 2]");
    TORCH_CHECK(scales.dim() == 2, "scales must have shape [N, K / group_size]");
    TORCH_CHECK(activations.is_contiguous(), "activations must be contiguous");
    TORCH_CHECK(packed_weights.is_contiguous(), "packed_weights must be contiguous");
    TORCH_CHECK(scales.is_contiguous(), "scales must be contiguous");
    TORCH_CHECK(group_size > 0, "group_size must be greater than zero");
    TORCH_CHECK(group_size % 2 == 0, "group_size must be even because each byte contains two weights");

    const int64_t m = activations.size(0);
    const int64_t k = activations.size(1);
    const int64_t n = packed_weights.size(0);
    TORCH_CHECK(packed_weights.size(1) * 2 == k, "packed_weights and activations must describe the same K dimension");
    TORCH_CHECK(k % group_size == 0, "K must be divisible by group_size");
    TORCH_CHECK(scales.size(0) == n && scales.size(1) == k / group_size,
                "scales must have shape [N, K / group_size]");

    const c10::cuda::CUDAGuard guard(activations.device());
    at::Tensor output = at::empty({m, n}, out_f32 ? activations.options().dtype(at::kFloat) : activations.options());
    if (m == 0 || n == 0) return output;

    const cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    const uint32_t flags = flags_from_env() | (out_f32 ? W4A16_FLAG_OUTPUT_F32 : 0u);
    const int forced_tiles = row_tiles_from_env();

    void* workspace = nullptr;
    size_t workspace_bytes = 0;
    const size_t wanted = w4a16_linear_workspace_bytes_flags(m, n, k, flags);
    if (wanted > 0 && wanted <= static_cast<size_t>(kWorkspaceBytes)) {
        at::Tensor& ws = workspace_for(activations.device(), stream);
        workspace = ws.data_ptr();
        workspace_bytes = static_cast<size_t>(ws.numel());
    }

    int status;
    if (forced_tiles != 0 && !(flags & W4A16_FLAG_FORCE_GENERIC) && group_size == 128 &&
        reinterpret_cast<uintptr_t>(activations.data_ptr()) % 16 == 0 &&
        reinterpret_cast<uintptr_t>(packed_weights.data_ptr()) % 16 == 0) {
        w4a16_linear_config config = {forced_tiles, 0, 0, 0, 0};
        status = w4a16_linear_f16_config(activations.data_ptr(), packed_weights.data_ptr(), scales.data_ptr(),
                                         output.data_ptr(), m, n, k, group_size, workspace, workspace_bytes,
                                         flags, &config, reinterpret_cast<w4a16_stream_t>(stream));
    } else {
        status = w4a16_linear_f16(activations.data_ptr(), packed_weights.data_ptr(), scales.data_ptr(),
                                  output.data_ptr(), m, n, k, group_size, workspace, workspace_bytes, flags,
                                  reinterpret_cast<w4a16_stream_t>(stream));
    }
    check_status(status, "w4a16::linear");
    return output;
}

at::Tensor linear_cuda_impl(const at::Tensor& activations, const at::Tensor& packed_weights,
                            const at::Tensor& scales, int64_t group_size) {
    return linear_impl(activations, packed_weights, scales, group_size, false);
}

// Same product with the unrounded FP32 sums as output: the per-device partial of a K-sharded layer.
at::Tensor linear_partial_cuda_impl(const at::Tensor& activations, const at::Tensor& packed_weights,
                                    const at::Tensor& scales, int64_t group_size) {
    return linear_impl(activations, packed_weights, scales, group_size, true);
}

at::Tensor dequantize_cuda_impl(const at::Tensor& packed_weights, const at::Tensor& scales, int64_t group_size) {
    TORCH_CHECK(packed_weights.is_cuda(), "packed_weights must be a CUDA tensor");
    TORCH_CHECK(scales.is_cuda(), "scales must be a CUDA tensor");
    TORCH_CHECK(packed_weights.device() == scales.device(),
                "packed_weights and scales must be on the same CUDA device");
    TORCH_CHECK(packed_weights.scalar_type() == at::kByte, "packed_weights must have dtype torch.uint8");
    TORCH_CHECK(scales.scalar_type() == at::kHalf, "scales must have dtype torch.float16");
    TORCH_CHECK(packed_weights.dim() == 2, "packed_weights must have shape [N, K / 2]");
    TORCH_CHECK(scales.dim() == 2, "scales must have shape [N, K / group_size]");
    TORCH_CHECK(packed_weights.is_contiguous(), "packed_weights must be contiguous");
    TORCH_CHECK(scales.is_contiguous(), "scales must be contiguous");
    TORCH_CHECK(group_size > 0 && group_size % 32 == 0,
                "dequantize needs group_size to be a positive multiple of 32");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(packed_weights.data_ptr()) % 16 == 0,
                "packed_weights must be 16-byte aligned");

    const int64_t n = packed_weights.size(0);
    const int64_t k = packed_weights.size(1) * 2;
    TORCH_CHECK(k % group_size == 0, "K must be divisible by group_size");
    TORCH_CHECK(scales.size(0) == n && scales.size(1) == k / group_size,
                "scales must have shape [N, K / group_size]");

    const c10::cuda::CUDAGuard guard(packed_weights.device());
    at::Tensor weights = at::empty({n, k}, packed_weights.options().dtype(at::kHalf));
    if (n == 0 || k == 0) return weights;
    const int status = w4a16_dequantize_f16(
        packed_weights.data_ptr(), scales.data_ptr(), weights.data_ptr(), n, k, group_size,
        reinterpret_cast<w4a16_stream_t>(at::cuda::getCurrentCUDAStream().stream()));
    check_status(status, "w4a16::dequantize");
    return weights;
}

std::tuple<at::Tensor, at::Tensor> quantize_pack_cuda_impl(const at::Tensor& weights, int64_t group_size) {
    TORCH_CHECK(weights.is_cuda(), "weights must be a CUDA tensor");
    TORCH_CHECK(weights.scalar_type() == at::kHalf || weights.scalar_type() == at::kFloat,
                "weights must have dtype torch.float16 or torch.float32");
    TORCH_CHECK(weights.dim() == 2, "weights must have shape [N, K]");
    TORCH_CHECK(group_size > 0, "group_size must be greater than zero");
    TORCH_CHECK(weights.size(1) % group_size == 0, "K must be divisible by group_size");
    TORCH_CHECK(weights.size(1) % 2 == 0 && group_size % 2 == 0, "K and group_size must be even: one byte carries two weights");
    const at::Tensor dense = weights.contiguous();
    const int64_t n = dense.size(0);
    const int64_t k = dense.size(1);
    const c10::cuda::CUDAGuard guard(dense.device());
    at::Tensor packed = at::empty({n, k / 2}, dense.options().dtype(at::kByte));
    at::Tensor scales = at::empty({n, k / group_size}, dense.options().dtype(at::kHalf));
    if (n == 0 || k == 0) return {packed, scales};
    const auto stream = reinterpret_cast<w4a16_stream_t>(at::cuda::getCurrentCUDAStream().stream());
    const int status = dense.scalar_type() == at::kFloat
                           ? w4a16_quantize_pack_f32(dense.data_ptr(), packed.data_ptr(), scales.data_ptr(), n, k, group_size, stream)
                           : w4a16_quantize_pack_f16(dense.data_ptr(), packed.data_ptr(), scales.data_ptr(), n, k, group_size, stream);
    check_status(status, "w4a16::quantize_pack");
    return {packed, scales};
}

}  // namespace

TORCH_LIBRARY(w4a16, m) {
    m.def("linear(Tensor activations, Tensor packed_weights, Tensor scales, int group_size) -> Tensor");
    m.def("dequantize(Tensor packed_weights, Tensor scales, int group_size) -> Tensor");
    // not in the reference: FP32 partial sums for layers sharded along K
    m.def("linear_partial(Tensor activations, Tensor packed_weights, Tensor scales, int group_size) -> Tensor");
    // not in the reference: its quantiser is host code (w4a16/quantization.py:65-113)
    m.def("quantize_pack(Tensor weights, int group_size) -> (Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(w4a16, CUDA, m) {
    m.impl("linear", &linear_cuda_impl);
    m.impl("dequantize", &dequantize_cuda_impl);
    m.impl("linear_partial", &linear_partial_cuda_impl);
    m.impl("quantize_pack", &quantize_pack_cuda_impl);
}
