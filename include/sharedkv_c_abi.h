/*
 * C ABI of libsharedkv_cuda.so: INT8 shared-KV decode attention and the paged
 * INT8 KV-cache writer for NVIDIA B200 (sm_100a).
 *
 * The library replaces, symbol for symbol, what the reference project's Python
 * layer binds for this path (paths below are relative to the reference checkout):
 *
 *   - the device libraries' C launchers
 *       launch_sharedkv_c8_sparse        csrc/kernels/c8/c4.cpp:70
 *       launch_sharedkv_c8_dense         csrc/kernels/c8/c128.cpp:107
 *       launch_sharedkv_c8_sparse_small  csrc/kernels/c8/c4_small.cpp:21
 *       launch_cache_write               csrc/kernels/cache_write.cpp:71
 *     (ctypes signatures: npu_sparse_attn_sharedkv_int8/c8_attention.py:49-52,
 *      npu_sparse_attn_sharedkv_int8/cache.py:48-50), and
 *   - the pybind11 host bridge (csrc/host/launch.cpp:105-115,
 *     csrc/host/c8_launch.cpp:38-43): attention / cache_write by argument
 *     address, ABI-size attributes, variant count.
 *
 * Rules of the boundary
 *   - plain C types only; every pointer field is a device address of the GPU
 *     that is current (or named by `device`) when the call is made;
 *   - the library allocates nothing, and its launch entries synchronise nothing
 *     and read nothing back: all scratch comes in through SharedKVArgs.workspace,
 *     whose size the caller obtains from sharedkv_workspace_bytes() and whose first
 *     SHAREDKV_WORKSPACE_INIT_BYTES bytes the caller zeroes once, before the first
 *     launch that uses it (sharedkv_workspace_init); every launch leaves them as
 *     the next one needs them, so no memset runs in front of a kernel;
 *   - a launch is one kernel.  It is launched with the programmatic-stream-
 *     serialization attribute, i.e. its thread blocks may become resident while
 *     the preceding kernel of the stream drains; they touch no global memory
 *     before that kernel has completed (SHAREDKV_PDL=0 in the environment turns
 *     the attribute off);
 *   - argument structs are copied by value at launch, so the caller may rebind
 *     or free the host struct as soon as the call returns;
 *   - launches go to the stream handed in (a cudaStream_t passed as void*) and
 *     may be captured in a CUDA graph: live batch and token counts are derived
 *     on the device from cuQ / seqLens on every replay;
 *   - every entry returns 0 on success, a negative SHAREDKV_E* code for a
 *     contract violation detected on the host, or a positive cudaError_t.
 *     (The reference launchers return void; a caller that ignores the result
 *     keeps working.)
 */
#ifndef SHAREDKV_C_ABI_H
#define SHAREDKV_C_ABI_H

#include <stdint.h>

#if defined(__GNUC__)
#define SHAREDKV_API __attribute__((visibility("default")))
#else
#define SHAREDKV_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Byte-for-byte the reference's SharedKVArgs (csrc/kernels/c8/args.h:7-14,
 * mirrored by ctypes in npu_sparse_attn_sharedkv_int8/attention.py:11-17): 200 bytes.
 * Strides are in bytes between consecutive pages; block tables hold page ids. */
typedef struct SharedKVArgs {
    uint64_t q;          /* BF16 [tokens, heads, 512], contiguous                    */
    uint64_t ori;        /* INT8 original cache  [oriPages, oriBlock, 1, 512]        */
    uint64_t cmp;        /* INT8 compressed cache [*, cmpBlock, 1, 512]              */
    uint64_t oriScale;   /* FP32 [512] frozen scale of the original cache            */
    uint64_t cmpScale;   /* FP32 [512] frozen scale of the compressed cache          */
    uint64_t oriTable;   /* INT32 [batch, oriTableWidth] logical page -> page id     */
    uint64_t cmpTable;   /* INT32 [batch, cmpTableWidth]                             */
    uint64_t indices;    /* INT32 [tokens, 1, topk] compressed rows (ratio 4 only)   */
    uint64_t cuQ;        /* INT32 [batch + 1] cumulative query tokens                */
    uint64_t seqLens;    /* INT32 [batch] KV length including the query tokens       */
    uint64_t sinks;      /* FP32 [heads] sink logits                                 */
    uint64_t out;        /* BF16 [tokens, heads, 512]                                */
    uint64_t workspace;  /* >= sharedkv_workspace_bytes(tokens) bytes, 256-aligned,
                            first 1024 bytes zeroed once by the owner              */
    uint64_t lse;        /* FP32 [tokens, heads] or 0                                */
    uint64_t oriStride;  /* bytes between original pages (>= oriBlock * 512)         */
    uint64_t cmpStride;  /* bytes between compressed pages                           */
    uint64_t partial;    /* unused by this library (kept for layout compatibility)   */
    uint64_t oriIndices; /* INT32 [tokens, 1, oriTopk] physical slots of the original
                            cache attended instead of the window, or 0 (general entry only) */
    uint32_t tokens, heads, batch, oriBlock, cmpBlock, oriTableWidth, cmpTableWidth;
    uint32_t ratio, window, topk, splits, oriTopk, oriPages;
    float softmaxScale;
} SharedKVArgs;

/* Byte-for-byte the reference's CacheWriteArgs (csrc/kernels/cache_write.h:4-8,
 * npu_sparse_attn_sharedkv_int8/cache.py:10-13): 84 bytes padded to 88.
 * pageStride in bytes; updateStride, slotStride, slotColumnStride in elements. */
typedef struct CacheWriteArgs {
    uint64_t cache, updates, slots, inverseScale;
    uint64_t pageStride, updateStride, slotStride, slotColumnStride;
    uint32_t tokens, pages, pageSize, int64Slots, pairedSlots;
} CacheWriteArgs;

enum {
    SHAREDKV_OK = 0,
    SHAREDKV_EINVAL = -22,     /* null pointer, unsupported geometry, bad alignment  */
    SHAREDKV_ERANGE = -34,     /* batch / tokens beyond what the workspace can plan   */
    SHAREDKV_EVARIANT = -2,    /* unknown kernel variant (launch.cpp:45 throws there) */
    SHAREDKV_ETIMEDOUT = -110  /* sharedkv_workspace_status: a device-side wait ran out */
};

/* Kernel variants of the host bridge: 0 is the reference's general 128-key-tile kernel
 * (launch.cpp:33), 3 / 4 and 7 / 8 its grouped-query C128 / C4 kernels for groups of four and two
 * (launch.cpp:36-37,40-41), 20-22 its C4 / C128 decode
 * kernels (c8_launch.cpp:12-18). */
enum { SHAREDKV_VARIANT_GENERAL = 0, SHAREDKV_VARIANT_PACKED = 3, SHAREDKV_VARIANT_PACKED_SPARSE = 4, SHAREDKV_VARIANT_PAIRED = 7, SHAREDKV_VARIANT_PAIRED_SPARSE = 8, SHAREDKV_VARIANT_C4 = 20, SHAREDKV_VARIANT_C128 = 21, SHAREDKV_VARIANT_C4_SMALL = 22 };

/* sizeof(SharedKVArgs) / sizeof(CacheWriteArgs) as compiled into the library; the
 * Python layer compares them with its ctypes mirrors (attention.py:223-226,
 * cache.py:54-55; exported as module attributes by launch.cpp:112-114). */
SHAREDKV_API uint32_t sharedkv_attention_args_size(void);
SHAREDKV_API uint32_t sharedkv_cache_args_size(void);
/* One past the largest accepted attention variant (launch.cpp:113). */
SHAREDKV_API uint32_t sharedkv_attention_variant_count(void);

/* Scratch the attention launch needs for `tokens` query rows, in bytes.
 * Replaces the Python-side constant c8_attention.WORKSPACE_BYTES
 * (npu_sparse_attn_sharedkv_int8/c8_attention.py:22-30). */
SHAREDKV_API uint64_t sharedkv_workspace_bytes(uint32_t tokens);

/* Prepares a freshly allocated (or otherwise overwritten) workspace: clears its first
 * SHAREDKV_WORKSPACE_INIT_BYTES bytes (split-K arrival counters and the status word) with a
 * memset on `stream`.  Needed once per workspace, not per launch: the kernel that finishes a
 * split token puts the token's counter back to zero.  A workspace may be shared by launches of
 * different shapes on one stream (the serving scratch pool of the reference,
 * npu_sparse_attn_sharedkv_int8/vllm_adapter.py:41-49): the cleared region does not depend on the
 * token count.  The reference has no such call; its kernels use no cross-core counters. */
#define SHAREDKV_WORKSPACE_INIT_BYTES 1024u
SHAREDKV_API int sharedkv_workspace_init(void *workspace, void *stream);

/* Failure report of the decode kernel.  Every wait inside the kernel (on a row fetch, a tensor-core
 * product, another warp) is bounded; when one runs out, the thread block gives up, frees its
 * tensor memory, and sets a status word in the workspace that stays set until the workspace is
 * initialised again.  This call synchronises `stream`, reads the word and returns SHAREDKV_OK,
 * SHAREDKV_ETIMEDOUT (the outputs of some launch that used this workspace are invalid),
 * SHAREDKV_ERANGE (a launch_sharedkv_paired_sparse launch met a context beyond its bound) or a
 * cudaError_t.  It is a diagnostic: nothing on the launch path calls it.  The reference reports
 * device failures through its runtime's stream errors instead. */
SHAREDKV_API int sharedkv_workspace_status(const void *workspace, void *stream);

/* General entry: args->ratio 1 (original cache only: the draft / sliding-window layers), 4 or 128,
 * and, when args->oriIndices is set, the original rows named by the caller instead of the
 * window: INT32 physical slots (page = slot / 32, row = slot % 32, no block-table lookup),
 * oriTopk per query token, negative or out-of-range entries masked in place.  The same kernel as
 * the entries below.  Replaces csrc/kernels/sharedkv.cpp:585 (`launch_sharedkv`, variant 0 of
 * csrc/host/launch.cpp:33), the reference's kernel for everything outside its C4 / C128 route. */
SHAREDKV_API int launch_sharedkv(uint32_t blocks, void *stream, const SharedKVArgs *args);

/* Paired queries (ratio 128 only): two adjacent query tokens of a request are one work item whose
 * keys are fetched once and used by both tokens, for launches with many query tokens per request
 * (chunked prefill).  The results follow the reference's tiled arithmetic with query_group = 2
 * (reference.py:229-234,243-245): the window rows of a pair are tiled from the first row of the
 * union of the two windows.  No explicit original slots; batch < 11776.  Replaces
 * csrc/kernels/sharedkv_paired.cpp:7 (`launch_sharedkv_paired`, variant 7 of launch.cpp:40). */
SHAREDKV_API int launch_sharedkv_paired(uint32_t blocks, void *stream, const SharedKVArgs *args);
/* Paired queries on a ratio-4 layer, as the reference groups C4 (reference.py:246-249,300-301): a token
 * attends every compressed row of the pair's later token that its own top-k list (args->indices,
 * topk <= 1024) names, a row named n times with log(n) added to its logits.  Contexts of at most
 * 1024 tokens (the reference's bound on grouped C4 plans, attention.py:89-98); a longer context sets
 * the workspace status to SHAREDKV_ERANGE (sharedkv_workspace_status) and its rows past the 256th
 * compressed row are not attended.  Replaces csrc/kernels/sharedkv_paired_sparse.cpp:7
 * (`launch_sharedkv_paired_sparse`, variant 8 of launch.cpp:41). */
SHAREDKV_API int launch_sharedkv_paired_sparse(uint32_t blocks, void *stream, const SharedKVArgs *args);
/* Groups of four adjacent query tokens (query_group = 4 of the reference): the tiling of the window
 * rows and the compressed prefix belongs to the group of four, as in the reference's arithmetic; the
 * group is walked as two pairs, each fetching the group's tiles for its two tokens.  Otherwise as the
 * paired entries.  Replace `launch_sharedkv_packed` / `launch_sharedkv_packed_sparse` (variants 3
 * and 4 of launch.cpp:36-37). */
SHAREDKV_API int launch_sharedkv_packed(uint32_t blocks, void *stream, const SharedKVArgs *args);
SHAREDKV_API int launch_sharedkv_packed_sparse(uint32_t blocks, void *stream, const SharedKVArgs *args);

/* C4 (ratio 4): window of <=128 original rows + <=1024 selected compressed rows per
 * query token.  `blocks` is accepted for signature compatibility and ignored: the
 * grid is one persistent CTA per SM.  Replaces c4.cpp:70. */
SHAREDKV_API int launch_sharedkv_c8_sparse(uint32_t blocks, void *stream, const SharedKVArgs *args);
/* Same kernel; the reference kept a second image for capacities below 24 tokens
 * (c4_small.cpp:21).  Kept as a distinct symbol because the Python layer selects it. */
SHAREDKV_API int launch_sharedkv_c8_sparse_small(uint32_t blocks, void *stream, const SharedKVArgs *args);
/* C128 (ratio 128): window + every compressed row of the context.  Replaces c128.cpp:107. */
SHAREDKV_API int launch_sharedkv_c8_dense(uint32_t blocks, void *stream, const SharedKVArgs *args);

/* Fused BF16 -> INT8 quantize (x * inverseScale, round-half-even, clamp +-127) and
 * slot scatter.  Rows with a negative slot, page >= pages or offset outside
 * [0, pageSize) are skipped.  Replaces cache_write.cpp:71. */
SHAREDKV_API int launch_cache_write(uint32_t blocks, void *stream, const CacheWriteArgs *args);

/* Host-bridge forms: `args` is the address of a host SharedKVArgs / CacheWriteArgs,
 * `device` the CUDA ordinal to make current for the launch (restored before return).
 * Replace attention()/cache_write() of csrc/host/c8_launch.cpp:20-25 and
 * csrc/host/launch.cpp:27-54; the stream is explicit because this library does not
 * link the tensor framework that owns the "current stream". */
SHAREDKV_API int sharedkv_attention(uint64_t args, uint32_t blocks, uint32_t variant, int32_t device, void *stream);
SHAREDKV_API int sharedkv_cache_write(uint64_t args, uint32_t blocks, int32_t device, void *stream);

/* Test hook: as the attention launchers (variant selects the kernel), additionally
 * dumping integer intermediates of every 128-key tile for exact comparison:
 *   tileInfo  INT32 [maxTiles, 4]       {token, kind, tile-in-kind, 128-bit mask word 0..3 packed below}
 *   validMask UINT32 [maxTiles, 4]      which of the tile's 128 slots are real keys
 *   qkAcc     INT32 [maxTiles, 128, 16] QK accumulators (columns 0-7 hi plane, 8-15 lo plane)
 *   pCodes    INT8  [maxTiles, 128, 16] P codes (0-7 hi, 8-15 lo)
 *   pvAcc     INT32 [maxTiles, 512, 16] PV accumulators
 *   qCodes    INT8  [tokens, 2, 16, 512] query code planes per cache kind
 *   counter   UINT32 [1]                 tiles dumped (zeroed by the caller)
 * `reserved`: bits 0-15, when non-zero, cap the number of CTAs (1 = every token is processed as
 * one piece, like the reference's single running state); bit 31 selects the cp.async row
 * gather instead of the TMA gather; bit 30 lowers the kernel's wait limit to about a millisecond
 * and lets one barrier arrival go missing, so that a test can watch the time-out path end the
 * kernel and set the status word.
 * No counterpart in the reference; its oracle computes these inline
 * (npu_sparse_attn_sharedkv_int8/reference.py:287-289,310-313). */
typedef struct SharedKVDebug {
    uint64_t tileInfo, validMask, qkAcc, pCodes, pvAcc, qCodes, counter;
    uint32_t maxTiles, reserved;
} SharedKVDebug;
SHAREDKV_API int sharedkv_attention_debug(uint32_t variant, void *stream, const SharedKVArgs *args,
                             const SharedKVDebug *debug);

/* Human-readable text for a value returned by any entry above. */
SHAREDKV_API const char *sharedkv_status_string(int status);

/* Decode attention without a caller-provided workspace.  No counterpart in the reference, whose
 * callers always pass a workspace tensor (attention.py:171-184).
 *
 * For callers that cannot allocate device memory: a plugin that is only handed tensor pointers,
 * or a thread that must stay out of its framework's allocator.  `args->workspace` is ignored (it
 * may be 0); the scratch is one fixed array per device that is part of the library image, so this
 * entry allocates nothing, not even on its first call.  Everything else (arguments, variants,
 * results, status codes) is as for the launch_sharedkv_c8_* entries, and the results are
 * bit-identical to theirs.
 *
 *   - Limit: args->tokens <= SHAREDKV_STATIC_SCRATCH_MAX_TOKENS, else SHAREDKV_ERANGE is returned
 *     and nothing is launched.
 *   - The first call on each device looks the array's address up (with that device current, which
 *     is the caller's job as for every launch_* entry).  Make that first call outside any stream
 *     capture; later calls only launch kernels.
 *   - The array needs no clearing, before the first call or between calls: it is zero when the
 *     library is loaded and every call leaves it as the next one needs it.
 *   - The status word of a timed-out wait lives in the array too; read it with
 *     sharedkv_static_scratch_status(stream), which synchronises `stream` and returns SHAREDKV_OK,
 *     SHAREDKV_ETIMEDOUT or a cudaError_t.
 *   - All calls on a device share the array.  Calls on one stream are ordered and safe; calls that
 *     can overlap in time (different streams or threads) race on it and give wrong results.  Use
 *     the workspace-taking entries with one workspace per stream for those. */
#define SHAREDKV_STATIC_SCRATCH_MAX_TOKENS 4096u
SHAREDKV_API int sharedkv_attention_static_scratch(uint32_t variant, void *stream, const SharedKVArgs *args);
SHAREDKV_API int sharedkv_static_scratch_status(void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SHAREDKV_C_ABI_H */
