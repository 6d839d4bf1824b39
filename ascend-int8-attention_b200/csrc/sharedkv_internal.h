// Declarations shared by the translation units of libsharedkv_cuda.so (not installed).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sharedkv_c_abi.h"

namespace sharedkv {

// SM count of the current device, cached per ordinal; <= 0 on failure.
int device_sm_count();

// Validates and launches the writer on `stream`.
int cache_write(const CacheWriteArgs *args, cudaStream_t stream);

// Validates and launches plan + decode kernels on `stream`.  `debug` may be null.
int attention(uint32_t variant, const SharedKVArgs *args, cudaStream_t stream, const SharedKVDebug *debug);

// Bytes of SharedKVArgs.workspace needed for `tokens` query rows.
uint64_t workspace_bytes(uint32_t tokens);

}  // namespace sharedkv
