// extern "C" surface of libsharedkv_cuda.so.  See include/sharedkv_c_abi.h for the contract.
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdlib>

#include "../../include/sharedkv_c_abi.h"
#include "sharedkv_internal.h"

static_assert(sizeof(SharedKVArgs) == 200, "SharedKVArgs must stay 200 bytes");
static_assert(sizeof(CacheWriteArgs) == 88, "CacheWriteArgs must stay 88 bytes");

namespace sharedkv {

int device_sm_count()
{
    static std::atomic<int> cache[kMaxDevices];
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0) return -1;
    if (device < kMaxDevices) {
        const int known = cache[device].load(std::memory_order_relaxed);
        if (known > 0) return known;
    }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
    if (device < kMaxDevices) cache[device].store(sms, std::memory_order_relaxed);
    return sms;
}

// SHAREDKV_PDL=0 launches without the programmatic-stream-serialization attribute (the kernels'
// griddepcontrol instructions are then no-ops).
bool programmatic_launch_enabled()
{
    static const bool enabled = [] {
        const char *v = getenv("SHAREDKV_PDL");
        return !(v && v[0] == '0' && v[1] == 0);
    }();
    return enabled;
}

namespace {

// Makes `device` current for the lifetime of the object (negative: leave as is).
struct DeviceScope {
    int previous = -1;
    bool switched = false;
    cudaError_t error = cudaSuccess;
    explicit DeviceScope(int device)
    {
        if (device < 0) return;
        error = cudaGetDevice(&previous);
        if (error != cudaSuccess) return;
        if (previous != device) {
            error = cudaSetDevice(device);
            switched = error == cudaSuccess;
        }
    }
    ~DeviceScope()
    {
        if (switched) cudaSetDevice(previous);
    }
};

}  // namespace
}  // namespace sharedkv

extern "C" {

uint32_t sharedkv_attention_args_size(void) { return (uint32_t)sizeof(SharedKVArgs); }
uint32_t sharedkv_cache_args_size(void) { return (uint32_t)sizeof(CacheWriteArgs); }
uint32_t sharedkv_attention_variant_count(void) { return SHAREDKV_VARIANT_C4_SMALL + 1; }
uint64_t sharedkv_workspace_bytes(uint32_t tokens) { return sharedkv::ws_bytes(tokens); }

int sharedkv_workspace_init(void *workspace, void *stream)
{
    if (workspace == nullptr || reinterpret_cast<uintptr_t>(workspace) % 256u) return SHAREDKV_EINVAL;
    return (int)cudaMemsetAsync(workspace, 0, sharedkv::kWsInitBytes, static_cast<cudaStream_t>(stream));
}
int sharedkv_workspace_status(const void *workspace, void *stream)
{
    return sharedkv::workspace_status(workspace, static_cast<cudaStream_t>(stream));
}

int launch_sharedkv(uint32_t, void *stream, const SharedKVArgs *args)
{
    return sharedkv::attention(SHAREDKV_VARIANT_GENERAL, args, static_cast<cudaStream_t>(stream), nullptr);
}
int launch_sharedkv_paired(uint32_t, void *stream, const SharedKVArgs *args)
{
    return sharedkv::attention(SHAREDKV_VARIANT_PAIRED, args, static_cast<cudaStream_t>(stream), nullptr);
}
int launch_sharedkv_paired_sparse(uint32_t, void *stream, const SharedKVArgs *args)
{
    return sharedkv::attention(SHAREDKV_VARIANT_PAIRED_SPARSE, args, static_cast<cudaStream_t>(stream), nullptr);
}
int launch_sharedkv_packed(uint32_t, void *stream, const SharedKVArgs *args)
{
    return sharedkv::attention(SHAREDKV_VARIANT_PACKED, args, static_cast<cudaStream_t>(stream), nullptr);
}
int launch_sharedkv_packed_sparse(uint32_t, void *stream, const SharedKVArgs *args)
{
    return sharedkv::attention(SHAREDKV_VARIANT_PACKED_SPARSE, args, static_cast<cudaStream_t>(stream), nullptr);
}
int launch_sharedkv_c8_sparse(uint32_t, void *stream, const SharedKVArgs *args)
{
    return sharedkv::attention(SHAREDKV_VARIANT_C4, args, static_cast<cudaStream_t>(stream), nullptr);
}
int launch_sharedkv_c8_sparse_small(uint32_t, void *stream, const SharedKVArgs *args)
{
    return sharedkv::attention(SHAREDKV_VARIANT_C4_SMALL, args, static_cast<cudaStream_t>(stream), nullptr);
}
int launch_sharedkv_c8_dense(uint32_t, void *stream, const SharedKVArgs *args)
{
    return sharedkv::attention(SHAREDKV_VARIANT_C128, args, static_cast<cudaStream_t>(stream), nullptr);
}
int launch_cache_write(uint32_t, void *stream, const CacheWriteArgs *args)
{
    return sharedkv::cache_write(args, static_cast<cudaStream_t>(stream));
}

int sharedkv_attention(uint64_t args, uint32_t, uint32_t variant, int32_t device, void *stream)
{
    if (!args) return SHAREDKV_EINVAL;
    sharedkv::DeviceScope scope(device);
    if (scope.error != cudaSuccess) return (int)scope.error;
    return sharedkv::attention(variant, reinterpret_cast<const SharedKVArgs *>(args), static_cast<cudaStream_t>(stream), nullptr);
}
int sharedkv_cache_write(uint64_t args, uint32_t, int32_t device, void *stream)
{
    if (!args) return SHAREDKV_EINVAL;
    sharedkv::DeviceScope scope(device);
    if (scope.error != cudaSuccess) return (int)scope.error;
    return sharedkv::cache_write(reinterpret_cast<const CacheWriteArgs *>(args), static_cast<cudaStream_t>(stream));
}

int sharedkv_attention_debug(uint32_t variant, void *stream, const SharedKVArgs *args, const SharedKVDebug *debug)
{
    if (!debug) return SHAREDKV_EINVAL;
    return sharedkv::attention(variant, args, static_cast<cudaStream_t>(stream), debug);
}

const char *sharedkv_status_string(int status)
{
    switch (status) {
        case SHAREDKV_OK: return "ok";
        case SHAREDKV_EINVAL: return "invalid argument: null pointer, unsupported geometry or misaligned buffer";
        case SHAREDKV_ERANGE: return "batch or token count beyond what the workspace can plan";
        case SHAREDKV_EVARIANT: return "unknown attention kernel variant";
        case SHAREDKV_ETIMEDOUT: return "a wait inside the decode kernel ran out; the results of that launch are invalid";
        default: break;
    }
    if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
    return "unknown sharedkv status";
}

}  // extern "C"
