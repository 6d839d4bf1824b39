// Declarations shared by the translation units of libsharedkv_cuda.so (not installed).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sharedkv_c_abi.h"
#include "work_split.h"

namespace sharedkv {

// Per-device caches inside the library (SM count, kernel attributes, static scratch address) are
// arrays of this many ordinals; devices beyond it work, uncached.
constexpr int kMaxDevices = 64;

// ------------------------------------------------------------------ workspace map
// bytes    0 -   63  PlanHeader (live shape of the last launch, sticky status word)
// bytes   64 -  703  split-K tickets, one UINT32 per CTA boundary; zero between launches: the
//                    owner zeroes them once (sharedkv_workspace_init), the CTA that merges a
//                    token puts its ticket back to zero
// bytes  704 - 1023  unused
// bytes 1024 -       work items, 32 bytes each, tokens + kMaxCtas of them
// then               8 x tokens bytes unused (kept: the size formula is part of the ABI)
// then, 256-aligned  partial states of split tokens, two per CTA, kPartialFloats FP32 each
constexpr uint32_t kHeads = 8, kDim = 512;
constexpr uint32_t kPartialFloats = kHeads * kDim + 16;      // acc[8][512], m[8], l[8]
constexpr uint64_t kWsStatus = 20;                           // byte offset of PlanHeader.status
constexpr uint64_t kWsTickets = 64;
constexpr uint64_t kWsItems = 1024;
constexpr uint64_t kWsInitBytes = 1024;                      // what sharedkv_workspace_init clears
static_assert(kWsTickets + 4ull * split::kMaxCtas <= kWsItems, "tickets must fit in front of the item list");

__host__ __device__ constexpr uint64_t ws_partials(uint32_t tokens)
{
    return (kWsItems + 32ull * (tokens + split::kMaxCtas) + 8ull * tokens + 255ull) & ~255ull;
}
__host__ __device__ constexpr uint64_t ws_bytes(uint32_t tokens)
{
    return ws_partials(tokens) + (uint64_t)split::kMaxCtas * 2ull * kPartialFloats * 4ull;
}

enum : uint32_t { kStatusOk = 0, kStatusWaitTimeout = 1, kStatusRange = 2 };      // status word of a workspace (sticky)

// SM count of the current device, cached per ordinal; <= 0 on failure.
int device_sm_count();

// Whether kernels are launched with the programmatic-stream-serialization attribute (default yes).
bool programmatic_launch_enabled();

// Validates and launches the writer on `stream`.
int cache_write(const CacheWriteArgs *args, cudaStream_t stream);

// Validates and launches the decode kernel on `stream`.  `debug` may be null.
int attention(uint32_t variant, const SharedKVArgs *args, cudaStream_t stream, const SharedKVDebug *debug);

// Reads the sticky status word of a workspace after synchronising `stream`: SHAREDKV_OK,
// SHAREDKV_ETIMEDOUT, or the cudaError_t of the read itself.
int workspace_status(const void *workspace, cudaStream_t stream);

}  // namespace sharedkv
