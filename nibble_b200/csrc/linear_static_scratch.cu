// w4a16_linear_f16_static_scratch: the fused linear for callers that may not allocate.
//
// Who needs this: code that runs where device allocation is off the table -- a serving loop that
// has promised its host framework never to call cudaMalloc after start-up (allocation takes a
// device-wide lock and can stall every stream), a plugin that is handed input and output buffers
// but no workspace and no allocator callback, or a caller that is in the middle of capturing a CUDA
// graph, where an allocation would either fail or be baked into the graph.  Such callers cannot
// supply the split-K workspace that w4a16_linear_f16 wants for small-N / long-K layers, and without
// it those layers run on a fraction of the SMs.
//
// What it does instead: the FP32 partial sums and arrival counters of the split-K reduction live in
// a fixed array that is part of this library's device image.  Nothing is allocated or freed by this
// entry point, on the host or on the device.
//
// Consequences the caller has to know about:
//   * the array exists once per GPU that loads the library and stays until the process exits
//     (kStaticScratchBytes per device);
//   * problems whose split-K scratch would not fit are refused with W4A16_ERR_TOO_LARGE -- nothing
//     is launched; use w4a16_linear_f16 with a caller-owned workspace for those;
//   * every call on a device uses the same array.  Two calls that can overlap on the GPU (different
//     streams, or graph branches) race on it and produce garbage; calls on one stream are safe;
//   * the first call on each device looks the array's device address up (cudaGetSymbolAddress).
//     Make that first call outside any stream capture.
#include <cuda_runtime.h>

#include <mutex>

#include "kernels.h"

namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;   // 4 MiB per device
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress; the
// kernel receives the device address obtained below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = {};

// Device address of the scratch array on the current device, looked up once per device.
int scratch_for_current_device(void** address) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return W4A16_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* found = nullptr;
        if (cudaGetSymbolAddress(&found, g_static_scratch) != cudaSuccess || found == nullptr) {
            return W4A16_ERR_LAUNCH;
        }
        g_scratch_address[device] = found;
    }
    *address = g_scratch_address[device];
    return W4A16_OK;
}

}  // namespace

extern "C" {

size_t w4a16_static_scratch_bytes(void) { return kStaticScratchBytes; }

int w4a16_linear_f16_static_scratch(const void* x, const void* packed, const void* scales, void* y, int64_t M,
                                    int64_t N, int64_t K, int64_t group_size, uint32_t flags,
                                    w4a16_stream_t stream) {
    // Shapes the fast path does not take (other group sizes, misaligned pointers, empty problems)
    // need no scratch at all: the ordinary entry point handles them without a workspace.
    const bool fast = group_size == w4a16::kGroupFast && K > 0 && M > 0 && N > 0 &&
                      reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(packed) % 16 == 0;
    if (!fast || (flags & W4A16_FLAG_FORCE_GENERIC)) {
        return w4a16_linear_f16(x, packed, scales, y, M, N, K, group_size, nullptr, 0, flags, stream);
    }
    // The split the library wants for this problem, on the route this call will take, decides how
    // much scratch is needed (none when the batch goes to the tcgen05 GEMM).
    const size_t needed = w4a16_linear_workspace_bytes_flags(M, N, K, flags);
    if (needed > kStaticScratchBytes) {
        // the GEMM runs without scratch too (K not split across CTAs); the streaming kernel's split is not optional
        if (w4a16::linear_routes_to_tcgen05(M, N, K, flags)) {
            return w4a16_linear_f16(x, packed, scales, y, M, N, K, group_size, nullptr, 0, flags, stream);
        }
        return W4A16_ERR_TOO_LARGE;
    }
    if (needed == 0) {
        return w4a16_linear_f16(x, packed, scales, y, M, N, K, group_size, nullptr, 0, flags, stream);
    }
    void* scratch = nullptr;
    const int status = scratch_for_current_device(&scratch);
    if (status != W4A16_OK) return status;
    // The arrival counters must read zero when the kernel starts.  The kernel leaves them at zero,
    // but the array is shared and outlives calls, so they are cleared here every time rather than
    // trusted.  (The partial sums need no clearing: every element read is written first.)
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    // (Only the counters this problem uses; they sit at the head of the fixed counter prefix.)
    const size_t used_counters = static_cast<size_t>((N + 15) / 16) * static_cast<size_t>((M + 7) / 8) * sizeof(unsigned);
    if (cudaMemsetAsync(scratch, 0, used_counters, s) != cudaSuccess) return W4A16_ERR_LAUNCH;
    return w4a16_linear_f16(x, packed, scales, y, M, N, K, group_size, scratch, needed, flags, stream);
}

}  // extern "C"
