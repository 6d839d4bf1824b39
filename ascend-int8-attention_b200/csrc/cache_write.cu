// Paged INT8 KV-cache writer for sm_100a.
//
// One warp owns one update row at a time: lane l converts channels [16 l, 16 l + 16), i.e. two
// 16-byte BF16 loads in and one 16-byte INT8 store out, so a row is read as 32 coalesced 32-byte
// pieces and written as one coalesced 512-byte line.  The kernel is pure streaming (1024 B read +
// 512 B written per row) and is bounded by HBM; it lasts 5-20 microseconds, so what matters is how
// soon the memory system is full and how few dependent round trips a warp makes:
//   * a warp's slots are read once, up front, one row per lane (a warp owns rows w, w + W, ...),
//     and handed round by shuffles;
//   * row loads do not wait for the slots: two rows per warp are requested unconditionally, and
//     only the store needs the slot (a row whose slot turns out to be invalid was read in vain);
//     32 resident warps per SM keep 64 KB of reads in flight, more rows per warp only cost registers
//     and residency (measured: 2 rows x 4 CTAs per SM 25.4 us per step, 4 x 3 26.8, 8 x 2 28.5);
//   * the launch carries the programmatic-stream-serialization attribute, so its CTAs are resident
//     and past their set-up when the previous kernel of the stream (often the other cache's
//     writer) ends; nothing is read before griddepcontrol.wait returns.
//
// Arithmetic (per element, matching the reference's CPU quantizer
// npu_sparse_attn_sharedkv_int8/reference.py:52-53 and the device writer
// csrc/kernels/cache_write.cpp:37-49):
//     code = int8( clamp( rint_half_even( float(bf16 x) * inverse_scale[c] ), -127, 127 ) )
// with a single correctly rounded FP32 multiply (no FMA contraction is possible).
// Slot rules (cache_write.cpp:53-63): negative first component -> skip; flat slot ->
// page = slot / pageSize, offset = slot % pageSize; page >= pages or offset outside
// [0, pageSize) -> skip.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sharedkv_c_abi.h"
#include "ptx_sm100.cuh"
#include "sharedkv_internal.h"

namespace sharedkv {
namespace {

using ptx::grid_dependency_launch_dependents;
using ptx::grid_dependency_wait;

constexpr int kWriterThreads = 256;          // 8 warps
constexpr int kRowsInFlight = 2;             // rows a warp requests before it converts the first (divides 32)
constexpr int kWriterCtasPerSm = 4;          // resident CTAs per SM the vector kernel is compiled for
constexpr uint64_t kNoSlot = ~0ull;          // byte offset standing for "skip this row"

__device__ __forceinline__ uint32_t quantize4(uint32_t lo2, uint32_t hi2, const float *inv)
{
    // lo2 / hi2 each hold two BF16 values (little endian: low half is the lower channel)
    float x0 = __uint_as_float(lo2 << 16), x1 = __uint_as_float(lo2 & 0xffff0000u);
    float x2 = __uint_as_float(hi2 << 16), x3 = __uint_as_float(hi2 & 0xffff0000u);
    int c0 = __float2int_rn(fminf(fmaxf(__fmul_rn(x0, inv[0]), -127.f), 127.f));
    int c1 = __float2int_rn(fminf(fmaxf(__fmul_rn(x1, inv[1]), -127.f), 127.f));
    int c2 = __float2int_rn(fminf(fmaxf(__fmul_rn(x2, inv[2]), -127.f), 127.f));
    int c3 = __float2int_rn(fminf(fmaxf(__fmul_rn(x3, inv[3]), -127.f), 127.f));
    return (uint32_t)(c0 & 0xff) | ((uint32_t)(c1 & 0xff) << 8) | ((uint32_t)(c2 & 0xff) << 16) |
           ((uint32_t)(c3 & 0xff) << 24);
}

template <class Index, bool Paired>
__device__ __forceinline__ bool resolve_slot(const CacheWriteArgs &p, uint32_t row, uint64_t &byte_offset)
{
    const Index *slots = reinterpret_cast<const Index *>(p.slots);
    const long long first = (long long)slots[(uint64_t)row * p.slotStride];
    if (first < 0) return false;
    long long page, offset;
    if (Paired) {
        page = first;
        offset = (long long)slots[(uint64_t)row * p.slotStride + p.slotColumnStride];
    } else if ((p.pageSize & (p.pageSize - 1u)) == 0u) {        // power-of-two pages (32 rows in serving): no division
        page = first >> (31 - __clz((int)p.pageSize));
        offset = first & (long long)(p.pageSize - 1u);
    } else {
        page = first / (long long)p.pageSize;
        offset = first % (long long)p.pageSize;
    }
    if (page >= (long long)p.pages || offset < 0 || offset >= (long long)p.pageSize) return false;
    byte_offset = (uint64_t)page * p.pageStride + (uint64_t)offset * 512u;
    return true;
}

// Vector path: update rows and cache rows are 16-byte aligned.
template <class Index, bool Paired>
__global__ void __launch_bounds__(kWriterThreads, kWriterCtasPerSm) cache_write_vec(const CacheWriteArgs p)
{
    grid_dependency_launch_dependents();
    grid_dependency_wait();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * kWriterThreads + threadIdx.x) >> 5;
    const uint32_t warps = (gridDim.x * kWriterThreads) >> 5;
    if (warp >= p.tokens) return;
    const uint32_t mine = (p.tokens - warp + warps - 1) / warps;          // rows warp, warp + warps, ... of this warp
    const char *updates = reinterpret_cast<const char *>(p.updates);
    char *cache = reinterpret_cast<char *>(p.cache);
    const uint64_t row_bytes = p.updateStride * 2u;

    uint4 a[kRowsInFlight], b[kRowsInFlight];
    auto request = [&](uint32_t first) {                                 // rows first .. first + kRowsInFlight - 1 of this warp
#pragma unroll
        for (int i = 0; i < kRowsInFlight; ++i) {
            if (first + i < mine) {
                const uint4 *src = reinterpret_cast<const uint4 *>(updates + (uint64_t)(warp + (first + i) * warps) * row_bytes) + lane * 2;
                a[i] = __ldcs(src);
                b[i] = __ldcs(src + 1);
            }
        }
    };
    request(0);
    float inv[16];
    {
        const float4 *s = reinterpret_cast<const float4 *>(p.inverseScale) + lane * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float4 v = __ldg(s + i);
            inv[4 * i] = v.x; inv[4 * i + 1] = v.y; inv[4 * i + 2] = v.z; inv[4 * i + 3] = v.w;
        }
    }
    for (uint32_t chunk = 0; chunk < mine; chunk += 32u) {
        // lane j resolves the slot of the warp's row chunk + j
        uint64_t my_dst = kNoSlot;
        if (chunk + lane < mine && !resolve_slot<Index, Paired>(p, warp + (chunk + lane) * warps, my_dst)) my_dst = kNoSlot;
        const uint32_t in_chunk = min(32u, mine - chunk);
        for (uint32_t k = 0; k < in_chunk; k += kRowsInFlight) {
            if (chunk + k != 0) request(chunk + k);
#pragma unroll
            for (int i = 0; i < kRowsInFlight; ++i) {
                const uint64_t dst = __shfl_sync(0xffffffffu, my_dst, (k + i) & 31u);
                if (k + i >= in_chunk || dst == kNoSlot) continue;
                uint4 o;
                o.x = quantize4(a[i].x, a[i].y, inv);
                o.y = quantize4(a[i].z, a[i].w, inv + 4);
                o.z = quantize4(b[i].x, b[i].y, inv + 8);
                o.w = quantize4(b[i].z, b[i].w, inv + 12);
                *reinterpret_cast<uint4 *>(cache + dst + lane * 16u) = o;
            }
        }
    }
}

// Scalar path for views whose rows are not 16-byte aligned (odd element strides or
// an odd byte offset into a shared backing): same arithmetic, 2-byte loads, 1-byte stores.
template <class Index, bool Paired>
__global__ void __launch_bounds__(kWriterThreads) cache_write_scalar(const CacheWriteArgs p)
{
    grid_dependency_launch_dependents();
    grid_dependency_wait();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * kWriterThreads + threadIdx.x) >> 5;
    const uint32_t warps = (gridDim.x * kWriterThreads) >> 5;
    const float *inv = reinterpret_cast<const float *>(p.inverseScale);
    const uint16_t *updates = reinterpret_cast<const uint16_t *>(p.updates);
    int8_t *cache = reinterpret_cast<int8_t *>(p.cache);
    for (uint32_t row = warp; row < p.tokens; row += warps) {
        uint64_t dst;
        if (!resolve_slot<Index, Paired>(p, row, dst)) continue;
        const uint16_t *src = updates + (uint64_t)row * p.updateStride;
        for (uint32_t c = lane; c < 512u; c += 32u) {
            float x = __uint_as_float((uint32_t)src[c] << 16);
            int code = __float2int_rn(fminf(fmaxf(__fmul_rn(x, __ldg(inv + c)), -127.f), 127.f));
            cache[dst + c] = (int8_t)code;
        }
    }
}

template <class Index, bool Paired>
cudaError_t launch_variant(const CacheWriteArgs &a, bool vec, cudaStream_t stream, int sms)
{
    const uint32_t warps_per_block = kWriterThreads / 32;
    uint32_t blocks;
    if (vec) {
        const uint32_t rows_per_block = warps_per_block * kRowsInFlight;
        blocks = (a.tokens + rows_per_block - 1) / rows_per_block;
    } else {
        blocks = (a.tokens + warps_per_block - 1) / warps_per_block;
    }
    // one wave: no more CTAs than are resident at once, each looping over its share of the rows
    const uint32_t cap = (uint32_t)sms * (vec ? (uint32_t)kWriterCtasPerSm : 8u);
    if (blocks > cap) blocks = cap;
    if (blocks == 0) return cudaSuccess;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(blocks);
    config.blockDim = dim3(kWriterThreads);
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = programmatic_launch_enabled() ? 1u : 0u;
    return vec ? cudaLaunchKernelEx(&config, cache_write_vec<Index, Paired>, a)
               : cudaLaunchKernelEx(&config, cache_write_scalar<Index, Paired>, a);
}

}  // namespace

int cache_write(const CacheWriteArgs *args, cudaStream_t stream)
{
    if (args == nullptr) return SHAREDKV_EINVAL;
    const CacheWriteArgs a = *args;
    if (a.tokens == 0) return SHAREDKV_OK;
    if (!a.cache || !a.updates || !a.slots || !a.inverseScale) return SHAREDKV_EINVAL;
    if (a.pages == 0 || a.pageSize == 0 || a.pageStride < (uint64_t)a.pageSize * 512u) return SHAREDKV_EINVAL;
    if (a.updateStride < 512u) return SHAREDKV_EINVAL;
    if (a.inverseScale % 4u || a.updates % 2u) return SHAREDKV_EINVAL;
    if (a.slots % (a.int64Slots ? 8u : 4u)) return SHAREDKV_EINVAL;
    const bool vec = a.cache % 16u == 0 && a.pageStride % 16u == 0 && a.updates % 16u == 0 &&
                     (a.updateStride * 2u) % 16u == 0 && a.inverseScale % 16u == 0;
    const int sms = device_sm_count();
    if (sms <= 0) return (int)cudaErrorInvalidDevice;
    cudaError_t e;
    if (a.int64Slots) {
        e = a.pairedSlots ? launch_variant<long long, true>(a, vec, stream, sms)
                          : launch_variant<long long, false>(a, vec, stream, sms);
    } else {
        e = a.pairedSlots ? launch_variant<int, true>(a, vec, stream, sms)
                          : launch_variant<int, false>(a, vec, stream, sms);
    }
    return (int)e;
}

}  // namespace sharedkv
