// RainFusion mask builder for callers that must not allocate device memory: the pooled means,
// which the ordinary entry point keeps in caller-supplied scratch, live in a fixed array that is
// part of this library's device image.
#include "capi_common.h"

#include <mutex>

namespace sdb {
namespace {

// 4 MiB: enough for batch * heads * blocks * head_dim * 2 <= 1 Mi pooled values, e.g. 6 heads of a
// 21x45x80 latent grid (591 blocks of 128 channels) or all 40 heads of a 21x16x24 one.
constexpr size_t kStaticPoolFloats = size_t(1) << 20;

// In host code this name is only a handle for the runtime; its device address is looked up once
// per device below and that address is what the kernels receive.
static __device__ __align__(256) float g_static_pool[kStaticPoolFloats];

// Returns the device address of g_static_pool on the current device, or nullptr and a CUDA error.
float* static_pool_address(cudaError_t* err) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static float* addr[kMaxDevices] = {};
    int dev = 0;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return nullptr;
    if (dev < 0 || dev >= kMaxDevices) {
        *err = cudaErrorInvalidDevice;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void* p = nullptr;
        *err = cudaGetSymbolAddress(&p, g_static_pool);  // with device `dev` current
        if (*err != cudaSuccess) return nullptr;
        addr[dev] = static_cast<float*>(p);
    }
    return addr[dev];
}

}  // namespace
}  // namespace sdb

using namespace sdb;

extern "C" size_t mindiesd_rf_block_mask_static_capacity(void) { return kStaticPoolFloats * sizeof(float); }

extern "C" int mindiesd_rf_block_mask_static(const mindiesd_mask_args* a, void* stream) {
    if (!a) return MINDIESD_E_NULL;
    if (a->batch <= 0 || a->heads <= 0 || a->head_dim <= 0 || a->t <= 0 || a->h <= 0 || a->w <= 0 || a->txt_len < 0)
        return MINDIESD_E_SHAPE;
    const size_t blocks = (static_cast<size_t>(a->t) * a->h * a->w + 127) / 128 + (static_cast<size_t>(a->txt_len) + 127) / 128;
    const size_t need = static_cast<size_t>(a->batch) * 2 * a->heads * blocks * a->head_dim;
    if (need > kStaticPoolFloats) return MINDIESD_E_CAPACITY;  // larger problems must use mindiesd_rf_block_mask
    cudaError_t err = cudaSuccess;
    float* pool = static_pool_address(&err);
    if (!pool) return err != cudaSuccess ? static_cast<int>(err) : MINDIESD_E_DRIVER;
    // Every pooled value the second kernel reads is written by the first one in the same call, so
    // nothing left in the array by an earlier call needs clearing.
    return rf_block_mask_impl(a, pool, kStaticPoolFloats * sizeof(float), static_cast<cudaStream_t>(stream));
}
