// sm_gemm_tc_static: the tensor-core product with its split-K scratch in a file-scope device
// array instead of a caller's workspace. See no_alloc.h for who needs it and for its rules.
#include "no_alloc.h"

#include <cuda_runtime.h>

#include <mutex>
#include <stdexcept>
#include <string>

#include "kernels.h"

namespace {

// The scratch itself. In host code this name is only a handle for the runtime: the kernel must
// be given the address that cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) float g_scratch[SM_GEMM_TC_STATIC_SCRATCH_BYTES / sizeof(float)];
static __device__ int g_error_word;

constexpr int kMaxDevices = 64;
struct PerDevice {
    float* scratch = nullptr;
    int* error = nullptr;
};
PerDevice g_devices[kMaxDevices];
std::mutex g_setup_mutex;

// Looks the addresses up once per device, with that device current.
const PerDevice& device_pointers() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) throw std::runtime_error(std::string("sm_gemm_tc_static: cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) throw std::runtime_error("sm_gemm_tc_static: device index out of range");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    PerDevice& d = g_devices[dev];
    if (!d.scratch) {
        float* s = nullptr;
        int* w = nullptr;
        e = cudaGetSymbolAddress((void**)&s, g_scratch);
        if (e != cudaSuccess)
            throw std::runtime_error(std::string("sm_gemm_tc_static: cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
        e = cudaGetSymbolAddress((void**)&w, g_error_word);
        if (e != cudaSuccess)
            throw std::runtime_error(std::string("sm_gemm_tc_static: cudaGetSymbolAddress(error word): ") + cudaGetErrorString(e));
        d.scratch = s;
        d.error = w;
    }
    return d;
}

}  // namespace

// capi.cu keeps the message channel; these two are its hooks.
namespace sm {
void set_last_error(const std::string& message);
}

extern "C" __attribute__((visibility("default")))
int sm_gemm_tc_static(const void* x, const void* w, const void* bias, int bias_dt, void* out, int out_dt, int T, int N,
                      int K, int mode, int up_offset, int* error, void* stream) {
    try {
        if (T <= 0 || N <= 0)
            throw std::invalid_argument("sm_gemm_tc_static: T = " + std::to_string(T) + " and N = " + std::to_string(N) +
                                        " must be positive");
        if (!sm::gemm_tc_supports(T, N, K))
            throw std::invalid_argument("sm_gemm_tc_static: K = " + std::to_string(K) + " must be a positive multiple of 8");
        const size_t need = sm::gemm_tc_workspace_bytes(T, N, K, (mode & 0xff) == 2);
        if (need > SM_GEMM_TC_STATIC_SCRATCH_BYTES)
            throw std::invalid_argument("sm_gemm_tc_static: this shape (T=" + std::to_string(T) + ", N=" + std::to_string(N) +
                                        ", K=" + std::to_string(K) + ") needs " + std::to_string(need) +
                                        " bytes of scratch; the static array holds " +
                                        std::to_string(SM_GEMM_TC_STATIC_SCRATCH_BYTES) + " (use sm_gemm_tc with a workspace)");
        const PerDevice& d = device_pointers();
        sm::gemm_tc(x, w, bias, (sm::DType)bias_dt, out, (sm::DType)out_dt, T, N, K, mode, up_offset, d.scratch,
                    error ? error : d.error, (cudaStream_t)stream);
        cudaError_t e = cudaPeekAtLastError();
        if (e != cudaSuccess) {
            cudaGetLastError();
            throw std::runtime_error(std::string("CUDA: ") + cudaGetErrorString(e));
        }
        return 0;
    } catch (const std::exception& ex) {
        sm::set_last_error(ex.what());
        return 1;
    }
}

extern "C" __attribute__((visibility("default")))
int sm_gemm_tc_static_error(void) {
    try {
        int value = 0;
        int* word = device_pointers().error;
        cudaError_t e = cudaMemcpy(&value, word, sizeof(int), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA: ") + cudaGetErrorString(e));
        if (value != 0) {
            // read once, then cleared: the next call starts clean (cudaMemset allocates nothing)
            e = cudaMemset(word, 0, sizeof(int));
            if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA: ") + cudaGetErrorString(e));
        }
        return value;
    } catch (const std::exception& ex) {
        sm::set_last_error(ex.what());
        return -1;
    }
}
