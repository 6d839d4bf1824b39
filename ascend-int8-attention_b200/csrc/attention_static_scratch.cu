// Decode attention for callers that have no device buffer to offer as scratch.
//
// The regular entry points take their scratch (work plan, split-K tickets and partial states)
// from SharedKVArgs.workspace, which the caller allocates.  Some callers cannot allocate: a C
// plugin that only receives tensor pointers from its host framework, a thread that must not touch
// the framework's caching allocator, or code that runs where an allocation would be a
// synchronisation point.  For them this file keeps ONE fixed scratch array per device inside the
// library image itself (a file-scope __device__ array: it is part of the loaded module, so neither
// this file nor the caller ever calls an allocator) and an entry point that substitutes its address
// for the workspace field.
//
// Consequences of the array being shared by every call on a device:
//  * The caller never has to clear it: the array is zero when the module is loaded, which is what
//    the split-K tickets need, and every launch leaves the tickets at zero again (the CTA that
//    merges a token resets its ticket); the kernel rebuilds the work plan on every call and a
//    partial state is always written before it is read.  Only the status word is carried over:
//    once a wait inside a kernel has run out it stays set (sharedkv_static_scratch_status).
//  * Two calls that are in flight at the same time on one device (two streams, two threads, two
//    branches of a graph) use the same bytes and corrupt each other.  Calls issued to one stream
//    run one after the other and are safe.  Callers that need concurrency use the regular entry
//    points with one workspace per stream.
//  * The size is fixed when the library is built; calls with more query rows than
//    SHAREDKV_STATIC_SCRATCH_MAX_TOKENS are refused, not truncated.
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/sharedkv_c_abi.h"
#include "sharedkv_internal.h"

namespace {

// 6 MiB: the plan and ticket tables of SHAREDKV_STATIC_SCRATCH_MAX_TOKENS query rows (170 KB) plus
// the split-K partial states, whose number depends on the CTA count and not on the batch (5.02 MiB).
constexpr uint64_t kScratchBytes = 6ull << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

using sharedkv::kMaxDevices;
static_assert(sharedkv::ws_bytes(SHAREDKV_STATIC_SCRATCH_MAX_TOKENS) <= kScratchBytes,
              "the workspace of the largest accepted call must fit the array");
std::mutex g_setup_lock;
void *g_scratch_address[kMaxDevices];      // device address of the array on each ordinal, null until set up

// Address of the array on the CURRENT device.  The first call per device resolves the symbol (this
// may load the module onto that device, which is not something to do inside a stream capture);
// later calls find it in the table.  Every call takes the lock for the look-up.
int scratch_of_current_device(void **address)
{
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= kMaxDevices) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> guard(g_setup_lock);
    if (g_scratch_address[device] == nullptr) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 255u) != 0) return (int)cudaErrorInvalidSymbol;
        g_scratch_address[device] = ptr;
    }
    *address = g_scratch_address[device];
    return SHAREDKV_OK;
}

}  // namespace

extern "C" int sharedkv_attention_static_scratch(uint32_t variant, void *stream, const SharedKVArgs *args)
{
    if (args == nullptr) return SHAREDKV_EINVAL;
    if (variant != SHAREDKV_VARIANT_GENERAL && variant != SHAREDKV_VARIANT_PACKED && variant != SHAREDKV_VARIANT_PACKED_SPARSE &&
        variant != SHAREDKV_VARIANT_PAIRED && variant != SHAREDKV_VARIANT_PAIRED_SPARSE &&
        variant != SHAREDKV_VARIANT_C4 &&
        variant != SHAREDKV_VARIANT_C128 && variant != SHAREDKV_VARIANT_C4_SMALL)
        return SHAREDKV_EVARIANT;
    static_assert(SHAREDKV_STATIC_SCRATCH_MAX_TOKENS > 0, "limit must be positive");
    if (args->tokens > SHAREDKV_STATIC_SCRATCH_MAX_TOKENS) return SHAREDKV_ERANGE;
    void *scratch = nullptr;
    const int status = scratch_of_current_device(&scratch);
    if (status != SHAREDKV_OK) return status;
    SharedKVArgs with_scratch = *args;                 // the caller's struct is left as it is
    with_scratch.workspace = reinterpret_cast<uint64_t>(scratch);
    return sharedkv::attention(variant, &with_scratch, static_cast<cudaStream_t>(stream), nullptr);
}

// The status word of the array on the current device (see sharedkv_workspace_status): callers of
// the entry above have no address to hand to that function.
extern "C" int sharedkv_static_scratch_status(void *stream)
{
    void *scratch = nullptr;
    const int status = scratch_of_current_device(&scratch);
    if (status != SHAREDKV_OK) return status;
    return sharedkv::workspace_status(scratch, static_cast<cudaStream_t>(stream));
}
