// Mapping another rank's device buffer into this process (one process per GPU, all GPUs of one box):
// the exporting rank turns a device pointer into a 64-byte CUDA IPC handle plus the pointer's offset
// inside its allocation; the importing rank opens the handle from its own device, which maps the
// allocation into its address space and enables peer access over NVLink.  Kernels of this library are
// then simply given the mapped address (a store to it crosses NVLink).  Host code only.
#include "capi_common.h"

#include <cstring>
#include <mutex>
#include <vector>

namespace sdb {
namespace {

struct Opened {
    cudaIpcMemHandle_t handle;
    int device;
    void* base;
};
std::mutex g_mu;
std::vector<Opened> g_opened;

using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
RangeFn range_fn() {
    static RangeFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<RangeFn>(sym);
    }();
    return fn;
}

}  // namespace
}  // namespace sdb

using namespace sdb;

extern "C" int mindiesd_peer_export(const void* ptr, uint8_t handle[64], uint64_t* offset) {
    if (!ptr || !handle || !offset) return MINDIESD_E_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    RangeFn fn = range_fn();
    if (!fn) return MINDIESD_E_DRIVER;
    CUdeviceptr base = 0;
    size_t size = 0;
    if (fn(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return MINDIESD_E_DRIVER;
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
    if (e != cudaSuccess) return static_cast<int>(e);
    std::memcpy(handle, &h, 64);
    *offset = reinterpret_cast<uintptr_t>(ptr) - static_cast<uintptr_t>(base);
    return MINDIESD_OK;
}

extern "C" int mindiesd_peer_open(const uint8_t handle[64], uint64_t offset, void** ptr) {
    if (!handle || !ptr) return MINDIESD_E_NULL;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    std::lock_guard<std::mutex> lock(g_mu);
    for (const Opened& o : g_opened)
        if (o.device == device && std::memcmp(&o.handle, &h, 64) == 0) {  // an allocation is opened once per process
            *ptr = static_cast<uint8_t*>(o.base) + offset;
            return MINDIESD_OK;
        }
    void* base = nullptr;
    e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return static_cast<int>(e);
    }
    g_opened.push_back({h, device, base});
    *ptr = static_cast<uint8_t*>(base) + offset;
    return MINDIESD_OK;
}
