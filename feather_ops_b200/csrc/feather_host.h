// Host-side helpers shared by the launchers: tensor-map encoding through the driver entry point (so the
// library does not link libcuda and still loads on a machine without a driver), device properties, and
// the per-translation-unit status word that bounded device waits report into.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace feather {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult query{};
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) != cudaSuccess ||
            query != cudaDriverEntryPointSuccess) {
            ptr = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// Tiled tensor map over `rank` dimensions, innermost first. `strides_bytes[i]` is the byte stride of
// dimension i + 1 (dimension 0 is dense). Out-of-bounds elements read as zero.
inline bool encode_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
    const EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    cuuint64_t gdims[5];
    cuuint64_t gstrides[4];
    cuuint32_t gbox[5];
    cuuint32_t estrides[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        estrides[i] = 1;
        if (i + 1 < rank) gstrides[i] = strides_bytes[i];
    }
    const CUresult res = fn(map, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides, gbox, estrides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return res == CUDA_SUCCESS;
}

struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
    int max_smem_optin = 0;
};

inline const DeviceInfo& device_info() {
    // One entry per device ordinal, filled on first use with that device current.
    static DeviceInfo info[64];
    static std::once_flag once[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    std::call_once(once[dev], [dev] {
        cudaDeviceGetAttribute(&info[dev].sm_count, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&info[dev].cc_major, cudaDevAttrComputeCapabilityMajor, dev);
        cudaDeviceGetAttribute(&info[dev].max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    });
    return info[dev];
}

// State that a launcher keeps per device and kernel (the raised shared-memory limit, the number of resident CTA
// pairs): looked up under a lock, so launchers may be called from several host threads at once.
class PerDeviceState {
public:
    // The remembered value for the current device; `setup()` computes it on first use and returns a positive
    // number (1 when there is nothing else to remember) or 0 on failure, in which case the next call tries again.
    template <class Setup>
    int get(Setup&& setup) {
        const int dev = current_device();
        std::lock_guard<std::mutex> hold(lock_);
        if (value_[dev] == 0) value_[dev] = setup();
        return value_[dev];
    }

    // For a limit that grows with the request: `raise(need)` is called when `need` exceeds what was set before.
    template <class Raise>
    bool at_least(int need, Raise&& raise) {
        const int dev = current_device();
        std::lock_guard<std::mutex> hold(lock_);
        if (value_[dev] >= need) return true;
        if (!raise(need)) return false;
        value_[dev] = need;
        return true;
    }

private:
    static int current_device() {
        int dev = 0;
        cudaGetDevice(&dev);
        return (dev < 0 || dev >= 64) ? 0 : dev;
    }
    std::mutex lock_;
    int value_[64] = {};
};

// An A/B switch from the environment: set to anything but "" or "0". Callers cache the answer (read once per process).
inline bool env_switch(const char* name) {
    const char* v = std::getenv(name);
    return v != nullptr && v[0] != '\0' && v[0] != '0';
}

}  // namespace feather
