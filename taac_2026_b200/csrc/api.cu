// Process-wide pieces of the C ABI: status text, device probe, launch counter.
#include <atomic>
#include <mutex>

#include "tb200_common.cuh"

namespace tb200 {

namespace {
std::atomic<int64_t> g_launches{0};
constexpr int kMaxDevices = 64;
DeviceInfo g_info[kMaxDevices];
std::once_flag g_once[kMaxDevices];
const DeviceInfo g_invalid{};
}  // namespace

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

const DeviceInfo& device_info() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        return g_invalid;
    }
    std::call_once(g_once[dev], [dev]() {
        DeviceInfo d;
        d.index = dev;
        cudaDeviceProp p;
        if (cudaGetDeviceProperties(&p, dev) == cudaSuccess) {
            d.sm_count = p.multiProcessorCount;
            d.cc_major = p.major;
            d.cc_minor = p.minor;
            d.max_smem_optin = static_cast<int>(p.sharedMemPerBlockOptin);
            d.valid = (p.major == 10);
        } else {
            cudaGetLastError();
        }
        g_info[dev] = d;
    });
    return g_info[dev];
}

}  // namespace tb200

extern "C" const char* tb200_strerror(int code) {
    switch (code) {
        case TB200_OK: return "ok";
        case TB200_ERR_NULL: return "tb200: a required pointer is NULL";
        case TB200_ERR_DTYPE: return "tb200: unsupported element or index type";
        case TB200_ERR_SHAPE: return "tb200: invalid size";
        case TB200_ERR_ALIGN: return "tb200: pointer or stride is not 16-byte aligned";
        case TB200_ERR_UNSUPPORTED: return "tb200: no kernel for this configuration";
        case TB200_ERR_DEVICE: return "tb200: current device is not compute capability 10.x (sm_100)";
        case TB200_ERR_DRIVER: return "tb200: tensor-map driver entry point unavailable or failed";
        case TB200_ERR_SCRATCH:
            return "tb200: request exceeds the 64 MiB fixed scratch of the no-allocation entry point; split the rows";
        case TB200_ERR_RANGE: return "tb200: a value does not fit the 32-bit compact host format";
        default: break;
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "tb200: unknown status";
}

extern "C" int tb200_abi_version(void) { return 1; }

extern "C" int tb200_device_ok(void) { return tb200::device_info().valid ? 1 : 0; }

extern "C" int64_t tb200_launch_count(void) { return tb200::g_launches.load(std::memory_order_relaxed); }
