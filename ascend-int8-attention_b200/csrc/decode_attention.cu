// INT8 shared-KV decode attention for sm_100a (C4: top-k compressed rows + window,
// C128: every compressed row + window; ratio 1: the original cache only; optionally the caller's own
// list of original slots in place of the window), eight heads, D = 512.
//
// One call = one kernel launch on the caller's stream (no memset, no second kernel): the split-K
// tickets in the workspace are zero between launches because the CTA that merges a token puts its
// ticket back, and the status word is sticky.  The launch carries the programmatic-stream-
// serialization attribute: its CTAs may become resident while the previous kernel of the stream
// drains, set up barriers and tensor memory, and wait (griddepcontrol.wait) for that kernel to
// finish before they read or write any global memory.
//
//   decode_kernel  one persistent CTA per SM, 24 warps in six roles that meet only at mbarriers.
//     set-up       every CTA derives the live batch / token count from cuQ and seqLens (trailing
//                  requests with seqLens <= 0 or cuQ < 0 are padding, as in the reference's device
//                  code csrc/kernels/c8/attention_impl.h:121-137), counts the 128-key tiles of
//                  every query token, cuts the flat tile list into one contiguous range per CTA
//                  and writes its own work items into the workspace (plan_cta).
//     warps 12-15, 20-23  producers (even / odd tiles): row selection -> page table -> row id, each a
//                  tile ahead of the next; rows land in a 3-stage ring of 128-key x 512-byte tiles (128-byte
//                  swizzle) by TMA row gathers (whole-page boxes for C128 compressed rows, 16-byte
//                  cp.async when the page strides rule TMA out)
//     warps 18-19  query encode: fold scale, absmax, hi / lo INT8 planes of the next item
//     warp  16     S[128 keys,16] = KV[128,512] . Qcodes[16,512]^T   16 x tcgen05.mma kind::i8, K-major
//     warps 0-7    softmax in FP32 registers, P codes [128 keys,16] to shared memory
//     warp  17     O[512,16] = KV^T[512,128] . P[128,16]             16 MMAs, MN-major operands: the
//                  SAME shared-memory tile serves both products
//     warps 8-11   accumulate: INT32 O -> FP32 running sums, finalise / split-K partials / merge
//   Columns 0-7 of S / O belong to the high code plane of Q / P, 8-15 to the low (residual) plane.
//   INT32 accumulators live in tensor memory (S and O double-buffered) and are converted to FP32
//   once per tile, exactly as the CPU reference does per tile.  A token whose tiles span several
//   CTAs is merged by the last CTA to finish a piece (atomic ticket; nobody waits for another CTA).
//   Registers are re-divided between the roles at kernel start (setmaxnreg).
//
// Arithmetic contract (npu_sparse_attn_sharedkv_int8/reference.py:268-322 of the reference):
//   f = float(q) * scale_kind;  alpha = max(max|f| * (1/127), 1e-12);  n = clamp(f * (1/alpha), +-127)
//   q_hi = rint(n), q_lo = rint((n - q_hi) * 127)
//   logit = (float(S_hi) + float(S_lo) * (1/127)) * (alpha * softmax_scale); padded keys -> -1e30
//   m' = max(m, max logit); r = exp(m - m'); w = exp(logit - m'); l = l r + sum w
//   p_hi = rint(127 w), p_lo = rint((127 w - p_hi) * 127)
//   acc = acc r + (float(O_hi) + float(O_lo) * (1/127)) * scale_kind * (1/127)
//   state starts at m = sink, l = 1 (first piece) or 0;  out = bf16(sum g acc / sum g l), g = exp(m - max m)
// The logits and the P codes follow that operation order exactly (separately rounded multiplies and
// adds).  Four places fuse or reorder, each within one FP32 ulp of the reference's order:
//   l = fma(l, r, w)  per key instead of  l r + sum w;   scale * (1/127) folded into one constant;
//   (O_hi + O_lo/127) and acc + pv * scale evaluated as two FMAs;   out = acc * (1/l) with a
//   correctly rounded reciprocal instead of a division.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstddef>
#include <cstring>

#include "../../include/sharedkv_c_abi.h"
#include "ptx_sm100.cuh"
#include "sharedkv_internal.h"

namespace sharedkv {
namespace {

using namespace ptx;

// ------------------------------------------------------------------ geometry
constexpr uint32_t kWindow = 128, kPage = 32;
constexpr uint32_t kTileKeys = split::kTileKeys;
constexpr uint32_t kStages = 3;
constexpr uint32_t kTileBytes = kTileKeys * kDim;            // 65536
constexpr uint32_t kSegBytes = kTileKeys * 128;              // one 128-channel segment of a tile: 16384
constexpr uint32_t kThreads = 768;                        // 8 softmax + 4 accumulate + 2 x 4 producer + 2 MMA + 2 query warps
constexpr uint32_t kWarpProducer = 12, kWarpMma = 16;   // warp 16 issues S = K.Q^T, warp 17 issues O = K^T.P
constexpr uint32_t kWarpQuery = 18;                      // warps 18 / 19 encode the query for the original / compressed scales
constexpr uint32_t kWarpProducerB = 20;                  // warps 12-15 fetch the even tiles of the CTA, warps 20-23 the odd ones
// Registers per thread by role (the kernel starts every warp at 80; see registers_release/acquire).
// Per SM sub-partition: 2 softmax + 1 accumulate + 2 producer + 1 MMA-or-query warp share 6 x 80 x 32 registers.
constexpr uint32_t kRegsLaunch = 80;     // what __launch_bounds__(768, 1) lets the compiler use
constexpr uint32_t kRegsSoftmax = 80, kRegsAccumulate = 128, kRegsProducer = 56, kRegsIssue = 80;
// The registers a CTA may re-divide are those it was launched with.  Asking for more than that
// would leave registers_acquire waiting for ever.
static_assert(2 * kRegsSoftmax + kRegsAccumulate + 2 * kRegsProducer + kRegsIssue <= 6 * kRegsLaunch,
              "register budgets of one sub-partition's six warps exceed the launch allocation");
static_assert(kRegsSoftmax >= kRegsLaunch && kRegsAccumulate >= kRegsLaunch && kRegsProducer <= kRegsLaunch && kRegsIssue <= kRegsLaunch,
              "acquire only grows, release only shrinks");
constexpr uint32_t kMaxCtas = split::kMaxCtas;
constexpr float kInv127 = (float)(1.0 / 127);
constexpr float kMasked = -1e30f;
constexpr uint32_t kWaitMillionCycles = 4000;                // ~2 s: a wait that long is a failure, not a stall
constexpr uint32_t kWaitMillionCyclesTest = 2;               // ~1 ms: the limit the wait-timeout test asks for
constexpr uint32_t kDrainNanoseconds = 200000;               // after a timeout: time given to copies and MMAs in flight
// SharedKVDebug.reserved: bits 0-15 cap the number of CTAs, bit 31 selects the cp.async row gather,
// bit 30 makes one barrier arrival go missing under a ~1 ms wait limit (the status-word test).
constexpr uint32_t kDebugCtaCapMask = 0xffffu, kDebugLegacyGather = 0x80000000u, kDebugShortWaits = 0x40000000u;

// shared memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kSmKv = 0;
constexpr uint32_t kSmQ = kSmKv + kStages * kTileBytes;      // query codes, 16 rows x 512 B swizzled: original kind, then
                                                             // two buffers of the compressed kind (alternating items)
constexpr uint32_t kSmP = kSmQ + 3 * 8192;                   // 2 buffers x 128 keys x 16 B
constexpr uint32_t kSmMask = kSmP + 2 * 2048;                // UINT32 [stages][4]: bit k of the 128-bit word = slot k holds a key
constexpr uint32_t kSmRed = kSmMask + 64;                    // FP32 [2 halves][2 parities][4 warps][4]
constexpr uint32_t kSmAlpha = kSmRed + 256;                  // FP32 [8 items][2 kinds][8]: alpha * softmax_scale
constexpr uint32_t kSmRescale = kSmAlpha + 8 * 64;              // [8 tiles][16]: r[8], debug record, pad
constexpr uint32_t kSmFinal = kSmRescale + 8 * 64;           // [8 items][16]: m[8], l[8]
constexpr uint32_t kSmItems = kSmFinal + 8 * 64;             // producers: per warp set a ring of 16 work items (16 B each)
constexpr uint32_t kSmRowIds = kSmItems + 2 * 16 * 16;       // producers: per warp [lookahead][32 lanes] row ids
constexpr uint32_t kSmBar = kSmRowIds + 8 * 2 * 32 * 4;      // mbarriers
constexpr uint32_t kBarFull = 0, kBarEmpty = 3, kBarSFull = 6, kBarSFree = 8, kBarPReady = 10, kBarOFull = 12,
                   kBarOFree = 14, kBarQReady = 16 /* x3 query buffers */, kBarQFree = 19 /* x3 */,
                   kBarGroup = 22 /* x4: softmax halves, all softmax, all accumulate */,
                   kBarRescale = 26 /* x8 */, kBarItemDone = 34 /* x8 */, kNumBars = 42;
constexpr uint32_t kSmMisc = kSmBar + kNumBars * 8;          // tmem base, abort flag, two broadcast words, wait limit
constexpr uint32_t kSmPlan = kSmMisc + 32;                   // PlanResult: this CTA's share of the launch (48 bytes)
constexpr uint32_t kSmemBytes = kSmPlan + 48 + 1024;         // + alignment slack
static_assert(kSmemBytes <= 232448, "dynamic shared memory limit of sm_100");

// tensor-memory columns
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0;     // S[b] at 16 b
constexpr uint32_t kColO = 64;    // O[b] at 64 + 64 b, four 16-column channel blocks each

// workspace (the byte map is in sharedkv_internal.h)
struct PlanHeader {
    uint32_t live_batch, live_tokens, total_tiles, quota, n_items, status, grid, pad;
};
static_assert(offsetof(PlanHeader, status) == kWsStatus, "status word offset is part of the library's interface");
struct Item {
    uint32_t token, batch;
    int32_t position;
    uint32_t tile_begin, tile_end, part, nparts, first_cta;
};
static_assert(sizeof(Item) == 32, "work item is two 16-byte loads");

// ------------------------------------------------------------------ small helpers
__device__ __forceinline__ uint32_t warp_inclusive_scan(uint32_t v, uint32_t lane)
{
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        uint32_t n = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= (uint32_t)d) v += n;
    }
    return v;
}

// Exclusive prefix over the threads of the CTA (up to 1024); `total` receives the sum.
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t *scratch, uint32_t &total)
{
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t incl = warp_inclusive_scan(v, lane);
    if (lane == 31) scratch[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const uint32_t s = lane < (blockDim.x >> 5) ? scratch[lane] : 0u;
        const uint32_t si = warp_inclusive_scan(s, lane);
        scratch[32 + lane] = si - s;
        if (lane == 31) scratch[64] = si;
    }
    __syncthreads();
    const uint32_t result = incl - v + scratch[32 + warp];
    total = scratch[64];
    __syncthreads();
    return result;
}

// Tiles of the original kind in front of a token's compressed tiles (uniform over a launch).
__device__ __forceinline__ uint32_t original_tiles(const SharedKVArgs &p)
{
    return split::original_tiles(p.oriIndices != 0, p.oriTopk);
}

// ------------------------------------------------------------------ work split
constexpr uint32_t kPlanStaged = 11776;      // cuQ entries kept in shared memory (46 KB)

// Request that owns query token t: the b with cu[b] <= t < cu[b + 1], 0 <= b < live_batch.
__device__ __forceinline__ uint32_t owner_of(const int32_t *cu, uint32_t live_batch, uint32_t t)
{
    uint32_t lo = 0, hi = live_batch - 1;
    while (lo < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        if (cu[mid + 1] <= (int32_t)t) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// Work split, computed by every CTA for itself at the start of the decode kernel (all threads take
// part); the arithmetic is in work_split.h.  The live shape comes from cuQ / seqLens on the device,
// so a captured graph follows the live batch.  The pieces of tokens that fall into this CTA's range
// of the flat tile list become its items, written to workspace entries no other CTA uses.
// `sc` is shared memory the roles do not use yet (the KV ring).

// What a CTA keeps of the plan (in shared memory of its own, written during plan_cta).
struct PlanResult {
    uint32_t first, count;        // its items are the workspace entries [first, first + count), in token order
    uint32_t live_tokens, tiles;  // live query tokens of the launch; tiles in this CTA's items
    uint4 first_item[2];          // the item at entry `first`, so that no role starts with a global-memory read
};
static_assert(sizeof(PlanResult) == 48, "PlanResult has its own 48 bytes of shared memory");
struct PlanScratch {
    uint32_t scan[80];
    uint32_t live, mismatch, pad[2];
    int32_t cu[kPlanStaged];
};

__device__ void plan_cta(const SharedKVArgs &p, const uint32_t grid, PlanScratch *sc, PlanResult *result)
{
    const uint32_t tid = threadIdx.x;
    const int32_t *cu_global = reinterpret_cast<const int32_t *>(p.cuQ);
    const int32_t *seq = reinterpret_cast<const int32_t *>(p.seqLens);
    char *ws = reinterpret_cast<char *>(p.workspace);
    Item *items = reinterpret_cast<Item *>(ws + kWsItems);

    if (tid == 0) {
        sc->live = 0; sc->mismatch = 0xffffffffu;
        result->first = 0xffffffffu; result->count = 0; result->tiles = 0;
    }
    const bool staged = p.batch + 1u <= kPlanStaged;
    const int32_t seq_first = tid < p.batch ? seq[tid] : 0;      // in flight together with the cuQ reads
    if (staged)
        for (uint32_t b = tid; b <= p.batch; b += kThreads) sc->cu[b] = cu_global[b];
    __syncthreads();
    const int32_t *cu = staged ? sc->cu : cu_global;
    uint32_t live = 0, mismatch = 0xffffffffu;
    for (uint32_t b = tid; b < p.batch; b += kThreads) {
        if (split::request_is_live(b == tid ? seq_first : seq[b], cu[b + 1])) live = b + 1;
        if (cu[b + 1] != (int32_t)(b + 1) && mismatch == 0xffffffffu) mismatch = b;
    }
    if (live) atomicMax(&sc->live, live);
    if (mismatch != 0xffffffffu) atomicMin(&sc->mismatch, mismatch);
    __syncthreads();
    const uint32_t live_batch = sc->live;
    const uint32_t live_tokens = split::live_token_count(live_batch ? cu[live_batch] : 0, p.tokens);
    // one query token per request (plain decode): token t belongs to request t
    const bool one_each = live_tokens == live_batch && cu[0] == 0 && sc->mismatch >= live_batch;

    // Thread i owns the consecutive tokens [i * per, (i + 1) * per); one block-wide scan of their tile
    // counts gives every thread its flat tile offset and the CTA the total (hence the quota).
    const uint32_t per = (live_tokens + kThreads - 1) / kThreads;
    const uint32_t t_begin = min(tid * per, live_tokens), t_end = min(t_begin + per, live_tokens);
    const uint32_t ori_tiles = original_tiles(p);
    auto tiles_of = [&](uint32_t t, uint32_t &batch, int32_t &position) {
        batch = one_each ? t : owner_of(cu, live_batch, t);
        position = split::token_position(seq[batch], cu[batch + 1], t);
        return split::tiles_of_token(p.ratio, position, p.topk, ori_tiles);      // p.ratio: a ratio-1 layer runs the C128 kernel without compressed tiles
    };
    uint32_t my_tiles = 0;
    for (uint32_t t = t_begin; t < t_end; ++t) {
        uint32_t batch; int32_t position;
        my_tiles += tiles_of(t, batch, position);
    }
    uint32_t total_tiles;
    const uint32_t tile_base = block_exclusive_scan(my_tiles, sc->scan, total_tiles);
    const uint32_t quota = split::quota_of(split::total_cost(total_tiles, live_tokens), grid);
    const uint32_t me = blockIdx.x;

    // Only threads whose tokens overlap this CTA's range [me * quota, (me + 1) * quota) go on.  Items are
    // written at their entries in token order; a thread remembers the first one it wrote.
    const uint32_t range_begin = split::first_tile_position(tile_base, t_begin) - split::kItemCost;
    const uint32_t range_end = split::first_tile_position(tile_base + my_tiles, t_end) - split::kItemCost;
    uint32_t my_entry = 0xffffffffu;
    uint4 my_lo = make_uint4(0, 0, 0, 0), my_hi = my_lo;
    if (range_begin < (me + 1) * quota && range_end > me * quota) {
        uint32_t before = tile_base, found = 0, tiles = 0;
        for (uint32_t t = t_begin; t < t_end; ++t) {
            uint32_t batch; int32_t position;
            const uint32_t n = tiles_of(t, batch, position);
            const uint32_t start = split::first_tile_position(before, t);
            const split::Pieces pc = split::pieces_of(start, n, quota);
            if (me >= pc.first_cta && me < pc.first_cta + pc.count) {
                const uint32_t entry = split::item_index(t, me), part = me - pc.first_cta;
                const split::TileRange r = split::piece_range(start, n, quota, me);
                const uint4 lo = make_uint4(t, batch, (uint32_t)position, r.begin);
                const uint4 hi = make_uint4(r.end, part, pc.count, pc.first_cta);
                uint4 *dst = reinterpret_cast<uint4 *>(items + entry);
                dst[0] = lo;
                dst[1] = hi;
                if (!found) { my_entry = entry; my_lo = lo; my_hi = hi; }
                ++found;
                tiles += r.end - r.begin;
            }
            before += n;
        }
        if (found) {
            atomicMin(&result->first, my_entry);
            atomicAdd(&result->count, found);
            atomicAdd(&result->tiles, tiles);
        }
    }
    __syncthreads();
    if (my_entry == result->first) { result->first_item[0] = my_lo; result->first_item[1] = my_hi; }
    if (tid == 0) {
        result->live_tokens = live_tokens;
        if (result->count == 0) result->first = 0;
        if (me == 0) {
            PlanHeader *header = reinterpret_cast<PlanHeader *>(ws);
            header->live_batch = live_batch; header->live_tokens = live_tokens; header->total_tiles = total_tiles;
            header->quota = quota; header->n_items = live_tokens; header->grid = grid;
        }
    }
    __syncthreads();          // the result is complete and the scratch area is handed back to the KV ring
}
// ------------------------------------------------------------------ decode kernel pieces
struct Shared {
    uint32_t base;              // shared-space address of the aligned region
    char *ptr;                  // generic pointer to the same
    __device__ __forceinline__ uint32_t bar(uint32_t i) const { return base + kSmBar + 8 * i; }
    __device__ __forceinline__ volatile uint32_t *misc() const { return reinterpret_cast<volatile uint32_t *>(ptr + kSmMisc); }
};

// Wait for a phase; gives up (and raises the CTA-wide abort flag) after ~2 s (misc[4], in millions of cycles).  The common case, a
// phase that is already complete, is one instruction inline; the polling loop lives out of line so
// that the many call sites stay small (the kernel's hot loops have to share the instruction cache).
// ROLE (0 softmax, 1 accumulate, 2 producer, 3 issue/query) only makes one copy per register budget:
// a function called from warps with different register allocations cannot be compiled.
template <int ROLE>
__device__ __noinline__ bool wait_phase_slow(uint32_t bar, uint32_t parity, volatile uint32_t *misc)
{
    const long long start = clock64();
#pragma unroll 1
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 0) {
            if (misc[1]) return false;
            if (clock64() - start > (long long)misc[4] * 1000000ll) { misc[1] = 1; return false; }
        }
    }
}
template <int ROLE>
__device__ __forceinline__ bool wait_phase(const Shared &sm, uint32_t bar_index, uint32_t parity)
{
    const uint32_t bar = sm.bar(bar_index);
    if (mbar_try_wait(bar, parity)) return true;
    return wait_phase_slow<ROLE>(bar, parity, sm.misc());
}

// Swizzled (128-byte) location of 16-byte chunk `chunk` (0..31) of row `row` in a
// [4 segments][rows/8][8][128 B] tile whose segments are `seg_bytes` apart.
__device__ __forceinline__ uint32_t tile_offset(uint32_t row, uint32_t chunk, uint32_t seg_bytes)
{
    const uint32_t seg = chunk >> 3, c = chunk & 7u, r = row & 7u;
    return seg * seg_bytes + (row >> 3) * 1024u + r * 128u + ((c ^ r) << 4);
}


__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d)
{
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
}

// ------------------------------------------------------------------ work-item cursors
// Walks the CTA's tiles in order, keeping the next item's descriptor in flight so that moving
// on to it does not expose a global-memory round trip.
struct Cursor {
    uint32_t k, j;              // k-th item of the CTA, tile j of it
    Item it;
    uint4 next_lo, next_hi;
    bool done;
};
__device__ __forceinline__ Item decode_item(const uint4 &a, const uint4 &b)
{
    Item it;
    it.token = a.x; it.batch = a.y; it.position = (int32_t)a.z; it.tile_begin = a.w;
    it.tile_end = b.x; it.part = b.y; it.nparts = b.z; it.first_cta = b.w;
    return it;
}
// The plan sits in shared memory; what a cursor needs of it is read when it moves to another item
// and not kept in registers (the producer warps run on 56 of them).
__device__ __forceinline__ void cursor_prefetch(Cursor &c, const Item *items, const PlanResult &plan)
{
    if (c.k + 1 < plan.count) {
        const uint4 *src = reinterpret_cast<const uint4 *>(items + plan.first + c.k + 1);
        c.next_lo = src[0];
        c.next_hi = src[1];
    }
}
__device__ __forceinline__ void cursor_init(Cursor &c, const Item *items, const PlanResult &plan)
{
    c.k = 0; c.done = plan.count == 0; c.j = 0;
    c.next_lo = c.next_hi = make_uint4(0, 0, 0, 0);
    if (!c.done) {
        c.it = decode_item(plan.first_item[0], plan.first_item[1]);
        c.j = c.it.tile_begin;
        cursor_prefetch(c, items, plan);
    }
}
// Returns true when the cursor moved on to a new item.
__device__ __forceinline__ bool cursor_advance(Cursor &c, const Item *items, const PlanResult &plan)
{
    if (++c.j < c.it.tile_end) return false;
    if (++c.k >= plan.count) { c.done = true; return false; }
    c.it = decode_item(c.next_lo, c.next_hi);
    c.j = c.it.tile_begin;
    cursor_prefetch(c, items, plan);
    return true;
}
// Trailing cursor of a producer warp: walks the same tiles as a leading Cursor, a bounded
// number of items behind it, and takes the descriptors from a shared-memory ring the leader fills.
// The four warps of a producer set share one ring: all of them write the same values, and a warp
// only reads entries it has itself written before (the set's warps are never more than the KV
// ring's three tiles apart, the leader runs eight tiles ahead, the ring holds 16 items), so no
// synchronisation is involved.
struct Follower {
    uint32_t item, items_end, j, tile_end, batch;
    int32_t position;
    bool done;
};
__device__ __forceinline__ void ring_put(const Shared &sm, uint32_t ring, uint32_t index, const Item &it)
{
    reinterpret_cast<uint4 *>(sm.ptr + kSmItems)[ring * 16u + (index & 15u)] =
        make_uint4(it.batch, (uint32_t)it.position, it.tile_begin, it.tile_end);
}
__device__ __forceinline__ void follower_load(Follower &f, const Shared &sm, uint32_t ring)
{
    const uint4 a = reinterpret_cast<const uint4 *>(sm.ptr + kSmItems)[ring * 16u + (f.item & 15u)];
    f.batch = a.x; f.position = (int32_t)a.y; f.j = a.z; f.tile_end = a.w;
}
__device__ __forceinline__ void follower_init(Follower &f, const Shared &sm, uint32_t ring, uint32_t first, uint32_t end)
{
    f.item = first; f.items_end = end; f.done = first >= end;
    f.j = f.tile_end = f.batch = 0; f.position = 0;
    if (!f.done) follower_load(f, sm, ring);
}
__device__ __forceinline__ void follower_advance(Follower &f, const Shared &sm, uint32_t ring)
{
    if (++f.j < f.tile_end) return;
    if (++f.item >= f.items_end) { f.done = true; return; }
    follower_load(f, sm, ring);
}
// A producer set fetches every second tile of the CTA: its cursors move two tiles at a time.
__device__ __forceinline__ void follower_advance2(Follower &f, const Shared &sm, uint32_t ring)
{
    follower_advance(f, sm, ring);
    if (!f.done) follower_advance(f, sm, ring);
}
// Leading cursor: `steps` tiles on, publishing every item it enters; true when the item changed.
__device__ __forceinline__ bool leader_advance(Cursor &c, const Item *items, const PlanResult &plan, const Shared &sm, uint32_t ring,
                                               uint32_t steps)
{
    bool moved = false;
    for (uint32_t s = 0; s < steps && !c.done; ++s) {
        if (cursor_advance(c, items, plan)) {
            ring_put(sm, ring, c.k, c.it);
            moved = true;
        }
    }
    return moved;
}
// Skip whatever is left of the current item.
__device__ __forceinline__ void cursor_next_item(Cursor &c, const Item *items, const PlanResult &plan)
{
    c.j = c.it.tile_end - 1u;
    cursor_advance(c, items, plan);
}

// ------------------------------------------------------------------ producer
// Short-context C4 (fewer compressed rows than top-k slots): the valid selections are packed
// to the front, order kept (reference.py:253).  Lane c keeps the validity mask of slots
// [32 c, 32 c + 32) and the inclusive count up to and including its chunk.
struct Compaction {
    uint32_t mask, inclusive, total;
    bool active;
};
__device__ __noinline__ void compaction_build(Compaction &k, const SharedKVArgs &p, const Item &it, uint32_t lane)
{
    const uint32_t count = it.position < 0 ? 0u : (uint32_t)(it.position + 1) / 4u;
    k.active = count < p.topk && p.topk <= 1024u;
    if (!k.active) return;
    const int32_t *ix = reinterpret_cast<const int32_t *>(p.indices) + (uint64_t)it.token * p.topk;
    uint32_t mine = 0;
    const uint32_t chunks = (p.topk + 31u) / 32u;
#pragma unroll 8
    for (uint32_t c = 0; c < chunks; ++c) {
        const uint32_t s = c * 32u + lane;
        int32_t v = -1;
        if (s < p.topk) v = ix[s];
        const uint32_t m = __ballot_sync(0xffffffffu, v >= 0 && (uint32_t)v < count);
        if (lane == c) mine = m;
    }
    k.mask = mine;
    k.inclusive = warp_inclusive_scan(__popc(mine), lane);
    k.total = __shfl_sync(0xffffffffu, k.inclusive, 31);
}
// Slot (0..topk) holding the s-th valid selection; s < total.
__device__ __noinline__ uint32_t compaction_slot(const Compaction &k, uint32_t s, bool in_range)
{
    uint32_t chunk = 0;
#pragma unroll 8
    for (int i = 0; i < 32; ++i) {
        const uint32_t incl = __shfl_sync(0xffffffffu, k.inclusive, i);
        chunk += (in_range && incl <= s) ? 1u : 0u;
    }
    chunk &= 31u;
    const uint32_t m = __shfl_sync(0xffffffffu, k.mask, chunk);
    const uint32_t incl = __shfl_sync(0xffffffffu, k.inclusive, chunk);
    const uint32_t before = incl - __popc(m);
    const uint32_t bit = in_range ? __fns(m, 0, (int)(s - before) + 1) : 0u;
    return chunk * 32u + (bit & 31u);
}

// ------------------------------------------------------------------ grouped items (paired query tokens)
// The paired kernel walks two adjacent query tokens of a request as ONE item whose tiles are
// fetched once and used by both tokens (reference.py:229-234,243-245 with query_group = 2 or 4).
// The tiling belongs to the item's GROUP of two or four tokens: the original rows are the union of
// the group's windows, tiled from the union's first row; the compressed rows are the prefix of the
// group's last token.  A group of four is two items that share that tiling.  An item stores the
// position of its own first token and, in the upper bits of `batch`, what it needs of its group.
constexpr uint32_t kPairBit = 0x80000000u;              // the item holds a second token
constexpr uint32_t kPairSecondBit = 0x40000000u;        // the item is the second pair of its group (its first token is the group's third)
constexpr uint32_t kPairGroupShift = 27;                // bits 27-29: tokens of the group (1..4)
constexpr uint32_t kPairBatchMask = (1u << kPairGroupShift) - 1u;
__device__ __forceinline__ uint32_t pair_tokens(uint32_t batch_word) { return (batch_word >> 31) + 1u; }
__device__ __forceinline__ uint32_t pair_batch(uint32_t batch_word) { return batch_word & kPairBatchMask; }
__device__ __forceinline__ uint32_t group_tokens(uint32_t batch_word) { return (batch_word >> kPairGroupShift) & 7u; }
// Position of the group's first token, given the position of the item's first token.
__device__ __forceinline__ int32_t group_position(int32_t position, uint32_t batch_word) { return position - ((batch_word & kPairSecondBit) ? 2 : 0); }
using split::pair_compressed_rows;
using split::pair_last_position;
using split::pair_original_tiles;
using split::pair_window_start;

// Stage A of the producer: candidate logical row of slot `slot` in the cursor's tile.
// Values read from the top-k array are returned unchecked (stage B range-checks them, so
// that the load is not consumed here); every other path returns a valid row or -1.
template <int RATIO, bool GROUP>
__device__ __forceinline__ int32_t candidate_row(const SharedKVArgs &p, const Cursor &c, const Compaction &k, uint32_t slot,
                                                 uint32_t ori_tiles)
{
    const Item &it = c.it;
    if (GROUP) {
        const uint32_t tokens = group_tokens(it.batch);
        const int32_t first = group_position(it.position, it.batch), last = pair_last_position(first, tokens);
        if (last < 0) return -1;
        const uint32_t windows = pair_original_tiles(first, tokens);
        if (c.j < windows) {
            const uint32_t row = pair_window_start(first) + c.j * kTileKeys + slot;
            return row <= (uint32_t)last ? (int32_t)row : -1;
        }
        const uint32_t s = (c.j - windows) * kTileKeys + slot;
        return s < pair_compressed_rows(first, tokens, p.ratio) ? (int32_t)s : -1;
    }
    if (it.position < 0) return -1;
    if (c.j < ori_tiles) {
        if (p.oriIndices) {
            // the caller's own list of physical slots of the original cache (reference.py:235-239):
            // holes keep their place, stage B range-checks the value
            const uint32_t s = c.j * kTileKeys + slot;
            return s < p.oriTopk ? reinterpret_cast<const int32_t *>(p.oriIndices)[(uint64_t)it.token * p.oriTopk + s] : -1;
        }
        const uint32_t n = min((uint32_t)it.position + 1u, kWindow);
        return slot < n ? (int32_t)((uint32_t)it.position + 1u - n + slot) : -1;
    }
    const uint32_t s = (c.j - ori_tiles) * kTileKeys + slot;
    if (RATIO == 128) return s < (uint32_t)(it.position + 1) / 128u ? (int32_t)s : -1;
    const int32_t *ix = reinterpret_cast<const int32_t *>(p.indices) + (uint64_t)it.token * p.topk;
    if (k.active) {
        const bool in_range = s < k.total;
        const uint32_t src = compaction_slot(k, s, in_range);
        return in_range ? ix[src] : -1;
    }
    return s < p.topk ? ix[s] : -1;
}

// Producer warps (four, one per SM sub-partition: the rate at which a warp can hand row fetches to
// the TMA unit is limited per warp).  Warp w owns key slots 32 w .. 32 w + 31 of every tile, lane =
// slot.  The two dependent global reads in front of a row fetch (top-k entry -> page-table entry ->
// row) are issued several tiles before their results are needed:
//   A  candidate logical row of this lane's slot                    (tile n)
//   B  range check + page-table lookup                              (tile n - kLookahead)
//   S  row id = page * rows-per-page + row in page, to a small ring (tile n - 2 kLookahead)
//   C  row fetch into the KV ring stage                             (same tiles as S)
// A, B and S are tiny and unrolled by the lookahead, so that every loaded value keeps its register
// from the load that produces it to its use (a shifting queue would read, and so wait for, every
// value each iteration); C is larger and exists once: it reads the row ids back from the ring.
// Row fetch: one TMA gather of four consecutive slots x one 128-channel segment per lane
// (lane = 4 * group + segment); for the compressed rows of a C128 layer, which fill whole pages,
// four 4 KB page-segment boxes per warp; 16-byte cp.async copies when the page strides rule TMA out.
// One tile of the set (= two tiles of the CTA, about 4 us) covers the latency of either read; a
// deeper pipeline only lengthens the start of the kernel (measured: 2 is 3 % slower than 1).
constexpr int kLookahead = 1;
constexpr int32_t kRowsInMap = 0x7ffffff0;      // rows the gather tensor maps span; row ids at or above read as zeros

template <int RATIO, bool TMA, bool GROUP, uint32_t STAGES = kStages>
__device__ void producer_loop(const SharedKVArgs &p, const Shared &sm, const Item *items, const PlanResult &plan,
                              uint32_t set, uint32_t pw, uint32_t lane, const CUtensorMap *ori_map, const CUtensorMap *cmp_map,
                              const CUtensorMap *cmp_page_map)
{
    // set 0 fetches tiles 0, 2, 4 ... of the CTA, set 1 tiles 1, 3, 5 ...
    const uint32_t first = 0, end = plan.count;      // the followers count the CTA's items from 0
    Cursor ca;
    cursor_init(ca, items, plan);
    if (!ca.done) ring_put(sm, set, ca.k, ca.it);
    if (set) leader_advance(ca, items, plan, sm, set, 1);
    Follower cb, cc;
    follower_init(cb, sm, set, first, end);
    follower_init(cc, sm, set, first, end);
    if (set && !cb.done) {
        follower_advance(cb, sm, set);
        follower_advance(cc, sm, set);
    }
    const uint32_t ori_tiles = original_tiles(p);
    const bool explicit_slots = p.oriIndices != 0;
    Compaction comp;
    comp.active = false; comp.mask = comp.inclusive = comp.total = 0;
    if (RATIO == 4 && !ca.done) compaction_build(comp, p, ca.it, lane);

    const int32_t *ori_table = reinterpret_cast<const int32_t *>(p.oriTable);
    const int32_t *cmp_table = reinterpret_cast<const int32_t *>(p.cmpTable);
    const uint32_t ori_rows_per_page = (uint32_t)(p.oriStride >> 9), cmp_rows_per_page = (uint32_t)(p.cmpStride >> 9);
    volatile int32_t *row_ring = reinterpret_cast<volatile int32_t *>(sm.ptr + kSmRowIds) + (set * 4u + pw) * (kLookahead * 32) + lane;
    const uint32_t slot = pw * 32u + lane;
    int32_t cand[kLookahead];             // stage A -> B, index = tile % kLookahead
    int32_t page[kLookahead];             // stage B -> S: page id ...
    int32_t offs[kLookahead];             // ... and row within the page (bit 8: original cache), or -1 without a key
#pragma unroll
    for (int u = 0; u < kLookahead; ++u) { cand[u] = -1; page[u] = 0; offs[u] = -1; }
    uint32_t issued = 0;                  // tiles whose fetches have been issued
    uint32_t signalled = 0;               // cp.async path: tiles whose "full" barrier this thread has arrived on

    for (uint32_t base = 0;; base += (uint32_t)kLookahead) {
#pragma unroll
        for (int u = 0; u < kLookahead; ++u) {
            const uint32_t n = base + (uint32_t)u;
            // ---- stage S: row id of tile n - 2 kLookahead
            {
                const int32_t o = offs[u], pg = page[u];
                int32_t id = kRowsInMap;
                if (o >= 0) {
                    const bool ori = (o >> 8) & 1;
                    // never read outside the original cache; the compressed cache's page count is not
                    // part of the argument struct, so only negative ids can be refused there
                    if (ori ? (uint32_t)pg < p.oriPages : pg >= 0)
                        id = !TMA ? (int32_t)(((uint32_t)pg << 5) + ((uint32_t)o & 31u))       // page, row in page
                             : (RATIO == 128 && !ori)
                                 ? pg                                                          // whole-page fetch
                                 : (int32_t)((uint32_t)pg * (ori ? ori_rows_per_page : cmp_rows_per_page) + ((uint32_t)o & 31u));
                }
                row_ring[u * 32] = id;
            }
            // ---- stage B: range check and page-table lookup for tile n - kLookahead
            int32_t off_b = -1, page_b = 0;
            if (n >= (uint32_t)kLookahead && !cb.done) {
                const bool ori = cb.j < (GROUP ? pair_original_tiles(group_position(cb.position, cb.batch), group_tokens(cb.batch)) : ori_tiles);
                const int32_t c = cand[u];
                if (GROUP) {
                    // the compressed prefix is that of the group's last token
                    const uint32_t limit = ori ? 0x7fffffffu : pair_compressed_rows(group_position(cb.position, cb.batch), group_tokens(cb.batch), p.ratio);
                    const uint32_t request = pair_batch(cb.batch);
                    if (c >= 0 && (uint32_t)c < limit && ((uint32_t)c >> 5) < (ori ? p.oriTableWidth : p.cmpTableWidth)) {
                        off_b = (c & 31) | (ori ? 256 : 0);
                        page_b = ori ? ori_table[(uint64_t)request * p.oriTableWidth + ((uint32_t)c >> 5)]
                                     : cmp_table[(uint64_t)request * p.cmpTableWidth + ((uint32_t)c >> 5)];
                    }
                } else if (ori && explicit_slots) {
                    // a physical slot: page and row come from the value itself, no table is read
                    if (c >= 0 && ((uint32_t)c >> 5) < p.oriPages) { off_b = (c & 31) | 256; page_b = c >> 5; }
                } else {
                    const uint32_t limit = ori ? 0x7fffffffu
                                               : (cb.position < 0 ? 0u : (uint32_t)(cb.position + 1) / (uint32_t)RATIO);
                    // a row beyond the request's page-table row is no key (a sequence length larger
                    // than the table can describe must not read the next request's entries)
                    if (c >= 0 && (uint32_t)c < limit && ((uint32_t)c >> 5) < (ori ? p.oriTableWidth : p.cmpTableWidth)) {
                        off_b = (c & 31) | (ori ? 256 : 0);
                        page_b = ori ? ori_table[(uint64_t)cb.batch * p.oriTableWidth + ((uint32_t)c >> 5)]
                                     : cmp_table[(uint64_t)cb.batch * p.cmpTableWidth + ((uint32_t)c >> 5)];
                    }
                }
                follower_advance2(cb, sm, set);
            }
            page[u] = page_b;
            offs[u] = off_b;
            // ---- stage A: candidate row for tile n
            int32_t cand_a = -1;
            if (!ca.done) {
                cand_a = candidate_row<RATIO, GROUP>(p, ca, comp, slot, ori_tiles);
                if (leader_advance(ca, items, plan, sm, set, 2) && RATIO == 4 && !ca.done) compaction_build(comp, p, ca.it, lane);
            }
            cand[u] = cand_a;
        }
        if (base < 2u * kLookahead) continue;
        // ---- stage C: fetch the rows of tiles base - 2 kLookahead .. + kLookahead - 1
#pragma unroll 1
        for (uint32_t u = 0; u < (uint32_t)kLookahead; ++u) {
            if (cc.done) goto drain;
            const uint32_t t = 2u * issued + set;          // position of the tile in the CTA's sequence
            const uint32_t stage = t % STAGES, pass = t / STAGES;
            if (!wait_phase<2>(sm, kBarEmpty + stage, (pass & 1u) ^ 1u)) return;
            const bool ori = cc.j < (GROUP ? pair_original_tiles(group_position(cc.position, cc.batch), group_tokens(cc.batch)) : ori_tiles);
            const int32_t id = row_ring[u * 32];
            const bool valid = id != kRowsInMap;
            const uint32_t mask = __ballot_sync(0xffffffffu, valid);
            if (lane == 0) reinterpret_cast<volatile uint32_t *>(sm.ptr + kSmMask)[stage * 4u + pw] = mask;
            const uint32_t tile = sm.base + kSmKv + stage * kTileBytes;
            if (TMA && RATIO == 128 && !ori) {
                // the 32 slots of this warp are one page of the compressed cache: four 4 KB boxes
                const bool any = mask != 0;
                const int32_t page_id = __shfl_sync(0xffffffffu, id, 0);      // slot 32 w is the first to be valid
                if (lane == 0) mbar_arrive_expect_tx(sm.bar(kBarFull + stage), any ? 16384u : 0u);
                __syncwarp();
                if (any && lane < 4)
                    tma_page_segment(tile + lane * kSegBytes + pw * 4096u, cmp_page_map, (int32_t)(lane * 128u), page_id,
                                     sm.bar(kBarFull + stage));
                ++issued;
            } else if (TMA) {
                const uint32_t g = lane >> 2, seg = lane & 3u;
                const int32_t r0 = __shfl_sync(0xffffffffu, id, 4 * g), r1 = __shfl_sync(0xffffffffu, id, 4 * g + 1);
                const int32_t r2 = __shfl_sync(0xffffffffu, id, 4 * g + 2), r3 = __shfl_sync(0xffffffffu, id, 4 * g + 3);
                const bool issue = ((mask >> (4u * g)) & 15u) != 0;
                const uint32_t bytes = 512u * __popc(__ballot_sync(0xffffffffu, issue));
                if (lane == 0) mbar_arrive_expect_tx(sm.bar(kBarFull + stage), bytes);
                __syncwarp();
                if (issue) {
                    const uint32_t row0 = pw * 32u + 4u * g;
                    tma_gather4(tile + seg * kSegBytes + (row0 >> 3) * 1024u + (row0 & 7u) * 128u, ori ? ori_map : cmp_map,
                                (int32_t)(seg * 128u), r0, r1, r2, r3, sm.bar(kBarFull + stage));
                }
                ++issued;
            } else {
                const uint64_t src = !valid ? 0ull
                    : (ori ? p.ori + (uint64_t)((uint32_t)id >> 5) * p.oriStride : p.cmp + (uint64_t)((uint32_t)id >> 5) * p.cmpStride)
                      + (uint64_t)((uint32_t)id & 31u) * kDim;
                const uint32_t lo = (uint32_t)src, hi = (uint32_t)(src >> 32);
#pragma unroll 1
                for (uint32_t r = 0; r < 32u; ++r) {
                    if (!((mask >> r) & 1u)) continue;
                    const uint64_t rsrc = ((uint64_t)__shfl_sync(0xffffffffu, hi, r) << 32) | __shfl_sync(0xffffffffu, lo, r);
                    cp_async16(tile + tile_offset(pw * 32u + r, lane, kSegBytes), reinterpret_cast<const char *>(rsrc) + lane * 16u);
                }
                cp_async_commit();
                ++issued;
                // keep one tile in flight behind the newest (with two stages a set owns one stage, so
                // its next tile cannot start before this one has been handed over and consumed)
                constexpr uint32_t kInFlight = STAGES >= 3 ? 2 : 1;
                if (issued - signalled == kInFlight) {
                    cp_async_wait<kInFlight - 1>();
                    fence_proxy_async_smem();
                    mbar_arrive(sm.bar(kBarFull + (2u * signalled + set) % STAGES));
                    ++signalled;
                }
            }
            follower_advance2(cc, sm, set);
        }
    }
drain:
    if (TMA) return;
    cp_async_wait<0>();
    fence_proxy_async_smem();
    while (signalled < issued) {
        mbar_arrive(sm.bar(kBarFull + (2u * signalled + set) % STAGES));
        ++signalled;
    }
}

// ------------------------------------------------------------------ MMA issuers (two threads)
// A thread can hand the tensor core roughly one small MMA per 60-70 cycles while the core itself
// retires one per ~40, so the two products of a tile are issued by two threads of different
// warps (different SM sub-partitions): S = K.Q^T by one, O = K^T.P by the other.  Each product is
// 16 instructions of M = 128, N = 16, K = 32 bytes.
__device__ void mma_qk_loop(const Shared &sm, const Item *items, const PlanResult &plan, uint32_t tmem, uint32_t ori_tiles)
{
    constexpr uint32_t kIdescQK = idesc_i8(128, 16, 0, 0);
    const bool leader = elect_one();
    const uint32_t first = 0, end = __shfl_sync(0xffffffffu, plan.count, 0);        // a loop bound the compiler can see is the same in all lanes
    Cursor cq;
    cursor_init(cq, items, plan);
    uint32_t t = 0;                        // tiles issued so far
    for (uint32_t k = 0; k < end - first; ++k) {
        // Query codes: one buffer for the original kind (read by an item's original tiles only) and two
        // alternating buffers for the compressed kind, so that the next item is encoded while this
        // one is processed.  Per item and kind this thread waits once for "encoded" and signals once
        // "no longer read" (a commit behind the last MMA that reads the buffer, or a plain arrival
        // when the item has no tile of that kind).
        const uint32_t tile_begin = __shfl_sync(0xffffffffu, cq.it.tile_begin, 0), tile_end = __shfl_sync(0xffffffffu, cq.it.tile_end, 0);
        const bool uses_ori = tile_begin < ori_tiles, uses_cmp = tile_end > max(tile_begin, ori_tiles);
        const uint32_t last_ori = min(tile_end, ori_tiles) - 1u;       // only meaningful when uses_ori
        const uint32_t last = tile_end - 1u;
        uint32_t j = tile_begin;
        const uint32_t cbuf = 1u + (k & 1u), cphase = (k >> 1) & 1u;     // compressed-kind buffer of this item
        bool cmp_ready = false;
        if (!wait_phase<3>(sm, kBarQReady + 0, k & 1u)) return;
        if (!uses_ori && leader) mbar_arrive(sm.bar(kBarQFree + 0));
        if (!uses_cmp) {
            if (!wait_phase<3>(sm, kBarQReady + cbuf, cphase)) return;
            if (leader) mbar_arrive(sm.bar(kBarQFree + cbuf));
        }
        for (; j < tile_end; ++j) {
            const uint32_t stage = t % kStages, buf = t & 1u, ph = (t >> 1) & 1u;
            if (j >= ori_tiles && !cmp_ready) {
                if (!wait_phase<3>(sm, kBarQReady + cbuf, cphase)) return;
                cmp_ready = true;
            }
            if (!wait_phase<3>(sm, kBarFull + stage, (t / kStages) & 1u)) return;
            if (!wait_phase<3>(sm, kBarSFree + buf, ph ^ 1u)) return;
            tc_fence_after();
            const uint32_t kv = sm.base + kSmKv + stage * kTileBytes;
            const uint32_t qb = sm.base + kSmQ + (j < ori_tiles ? 0u : cbuf * 8192u);
            const uint64_t a0 = smem_desc(kv, 16u, 1024u, kSwizzle128), b0 = smem_desc(qb, 16u, 1024u, kSwizzle128);
            // the address field counts 16-byte units; offsets stay inside the 14-bit field
#pragma unroll 1
            for (uint32_t seg = 0; seg < 4; ++seg) {
#pragma unroll
                for (uint32_t part = 0; part < 4; ++part)
                    if (leader)
                        mma_i8(tmem + kColS + buf * 16u, a0 + ((seg * kSegBytes + part * 32u) >> 4), b0 + ((seg * 2048u + part * 32u) >> 4),
                               kIdescQK, seg | part);
            }
            if (leader) mma_commit(sm.bar(kBarSFull + buf));
            if (leader) {
                if (j < ori_tiles) { if (j == last_ori) mma_commit(sm.bar(kBarQFree + 0)); }
                else if (j == last) mma_commit(sm.bar(kBarQFree + cbuf));
            }
            ++t;
        }
        cursor_next_item(cq, items, plan);
    }
}

__device__ void mma_pv_loop(const Shared &sm, const PlanResult &plan, uint32_t tmem)
{
    constexpr uint32_t kIdescPV = idesc_i8(128, 16, 1, 1);
    // only the number of tiles matters here
    const bool leader = elect_one();
    const uint32_t tiles = __shfl_sync(0xffffffffu, plan.tiles, 0);
    for (uint32_t t = 0; t < tiles; ++t) {
        const uint32_t stage = t % kStages, buf = t & 1u, ph = (t >> 1) & 1u;
        if (!wait_phase<3>(sm, kBarPReady + buf, ph)) return;
        if (!wait_phase<3>(sm, kBarOFree + buf, ph ^ 1u)) return;
        tc_fence_after();
        const uint32_t kv = sm.base + kSmKv + stage * kTileBytes;
        const uint32_t pb = sm.base + kSmP + buf * 2048u;
        const uint64_t a0 = smem_desc(kv, kSegBytes, 1024u, kSwizzle128), b0 = smem_desc(pb, 128u, 2048u, kSwizzleNone);
#pragma unroll 1
        for (uint32_t mb = 0; mb < 4; ++mb) {
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk)
                if (leader)
                    mma_i8(tmem + kColO + buf * 64u + mb * 16u, a0 + ((mb * kSegBytes + kk * 4096u) >> 4), b0 + ((kk * 512u) >> 4),
                           kIdescPV, kk);
        }
        if (leader) {
            mma_commit(sm.bar(kBarOFull + buf));
            mma_commit(sm.bar(kBarEmpty + stage));      // the stage's last reader (its S product finished before P existed)
        }
    }
}

// ------------------------------------------------------------------ softmax warps (0-7)
// Two halves of four warps.  Thread (half, key) owns heads 4 half .. 4 half + 3 of key `key` of
// every tile: columns 4 half + i (high plane) and 8 + 4 half + i (low plane) of S.

// Wait-capable rendezvous of `which`'s threads (an mbarrier wait can time out, a bar.sync cannot).
template <int ROLE>
__device__ __forceinline__ bool group_sync(const Shared &sm, uint32_t which, uint32_t &phase)
{
    mbar_arrive(sm.bar(kBarGroup + which));
    const bool ok = wait_phase<ROLE>(sm, kBarGroup + which, phase);
    phase ^= 1u;
    return ok;
}

// e^x through the hardware base-2 exponential (relative error about 2^-22 plus the rounding of
// x * log2(e)); masked keys (-1e30) give exactly 0.
__device__ __forceinline__ float fast_exp(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(__fmul_rn(x, 1.4426950408889634f)));
    return y;
}

// Reduce four per-thread values across the 32 lanes; afterwards lane 8 i (i = 0..3) holds value i.
template <bool MAX>
__device__ __forceinline__ float warp_reduce4(const float (&v)[4], uint32_t lane)
{
    auto op = [](float a, float b) { return MAX ? fmaxf(a, b) : a + b; };
    float a[2], c;
    const bool up16 = lane & 16u, up8 = lane & 8u;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float send = up16 ? v[i] : v[i + 2], keep = up16 ? v[i + 2] : v[i];
        a[i] = op(keep, __shfl_xor_sync(0xffffffffu, send, 16));
    }
    {
        const float send = up8 ? a[0] : a[1], keep = up8 ? a[1] : a[0];
        c = op(keep, __shfl_xor_sync(0xffffffffu, send, 8));
    }
    c = op(c, __shfl_xor_sync(0xffffffffu, c, 4));
    c = op(c, __shfl_xor_sync(0xffffffffu, c, 2));
    c = op(c, __shfl_xor_sync(0xffffffffu, c, 1));
    return c;   // value index = 2 * bit4 + bit3 of the lane
}

// ------------------------------------------------------------------ query warps (18, 19)
// One warp per cache kind.  Lane l owns channels 16 l .. 16 l + 15 (one 16-byte chunk of a code
// row).  Per item: fold the kind's cache scale into the eight query rows, split each into two INT8
// code planes (rows h and 8 + h of the 16-row B operand, swizzled) and publish alpha * softmax_scale
// per head.  Runs one item ahead of the S = K.Q^T issuer.
template <bool DEBUG>
__device__ void query_loop(const SharedKVArgs &p, const SharedKVDebug &dbg, const Shared &sm, const Item *items,
                           const PlanResult &plan, uint32_t kind, uint32_t lane)
{
    float sc[16];
    {
        const float4 *src = reinterpret_cast<const float4 *>(kind ? p.cmpScale : p.oriScale) + lane * 4u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 v = __ldg(src + i);
            sc[4 * i] = v.x; sc[4 * i + 1] = v.y; sc[4 * i + 2] = v.z; sc[4 * i + 3] = v.w;
        }
    }
    const uint32_t ori_tiles = original_tiles(p);
    Cursor cur;
    cursor_init(cur, items, plan);
    for (uint32_t k = 0; !cur.done; ++k) {
        const Item it = cur.it;
        const bool used = kind == 0 ? it.tile_begin < ori_tiles : it.tile_end > max(it.tile_begin, ori_tiles);
        // buffer, and the use of it that must be over before it is rewritten
        const uint32_t qbuf = kind == 0 ? 0u : 1u + (k & 1u);
        const uint32_t uses_before = kind == 0 ? k : k >> 1;
        char *qdst = sm.ptr + kSmQ + qbuf * 8192u;
        const uint4 *src = reinterpret_cast<const uint4 *>(p.q + (uint64_t)it.token * 8192u) + lane * 2u;
        if (cur.k + 1 < plan.count) {        // the next item's query rows start their way to L2 now
            const char *next = reinterpret_cast<const char *>(p.q) + (uint64_t)cur.next_lo.x * 8192u + lane * 256u;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(next));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(next + 128));
        }
        uint4 raw[4][2];                           // four heads at a time keeps the warp inside its register budget
        if (used) {
#pragma unroll
            for (int h = 0; h < 4; ++h) { raw[h][0] = __ldg(src + h * 64); raw[h][1] = __ldg(src + h * 64 + 1); }
        }
        if (uses_before > 0 && !wait_phase<3>(sm, kBarQFree + qbuf, (uses_before - 1u) & 1u)) return;     // earlier codes are no longer read
        if (used) {
            float *alphas = reinterpret_cast<float *>(sm.ptr + kSmAlpha) + (k & 7u) * 16u + kind * 8u;
#pragma unroll 1
            for (uint32_t batch = 0; batch < 2; ++batch) {
                if (batch == 1) {
#pragma unroll
                    for (int h = 0; h < 4; ++h) { raw[h][0] = __ldg(src + (4 + h) * 64); raw[h][1] = __ldg(src + (4 + h) * 64 + 1); }
                }
#pragma unroll 1
                for (uint32_t hh = 0; hh < 4; ++hh) {
                    const uint32_t h = batch * 4u + hh;
                    // rotate the four prefetched heads through slot 0 so that the loop body exists once
                    const uint32_t *rw = reinterpret_cast<const uint32_t *>(raw[0]);
                    float f[16];
                    float amax = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        f[2 * i] = __fmul_rn(__uint_as_float(rw[i] << 16), sc[2 * i]);
                        f[2 * i + 1] = __fmul_rn(__uint_as_float(rw[i] & 0xffff0000u), sc[2 * i + 1]);
                        amax = fmaxf(amax, fmaxf(fabsf(f[2 * i]), fabsf(f[2 * i + 1])));
                    }
#pragma unroll
                    for (int d = 16; d >= 1; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
                    const float alpha = fmaxf(__fmul_rn(amax, kInv127), 1e-12f);
                    const float rcp = __frcp_rn(alpha);
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        // Round-half-even through the adder: x + 1.5 * 2^23 leaves the rounded integer in
                        // the low mantissa bits (two's complement in the low byte for |x| <= 128).  The
                        // clamp to +-127 of the reference is an identity here: |f| <= amax, so |f / alpha|
                        // exceeds 127 by rounding error only, which rounds to +-127 with residual 0.
                        uint32_t ch[4], cl[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float nrm = __fmul_rn(f[4 * w + e], rcp);
                            const float shifted = __fadd_rn(nrm, 12582912.f);
                            const float hf = __fsub_rn(shifted, 12582912.f);
                            ch[e] = __float_as_uint(shifted);
                            cl[e] = __float_as_uint(__fadd_rn(__fmul_rn(__fsub_rn(nrm, hf), 127.f), 12582912.f));
                        }
                        hi[w] = __byte_perm(__byte_perm(ch[0], ch[1], 0x0040), __byte_perm(ch[2], ch[3], 0x0040), 0x5410);
                        lo[w] = __byte_perm(__byte_perm(cl[0], cl[1], 0x0040), __byte_perm(cl[2], cl[3], 0x0040), 0x5410);
                    }
                    const uint4 vh = make_uint4(hi[0], hi[1], hi[2], hi[3]), vl = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    *reinterpret_cast<uint4 *>(qdst + tile_offset(h, lane, 2048u)) = vh;
                    *reinterpret_cast<uint4 *>(qdst + tile_offset(8u + h, lane, 2048u)) = vl;
                    if (DEBUG) {
                        char *g = reinterpret_cast<char *>(dbg.qCodes) + ((uint64_t)it.token * 2u + kind) * 16u * 512u;
                        *reinterpret_cast<uint4 *>(g + h * 512u + lane * 16u) = vh;
                        *reinterpret_cast<uint4 *>(g + (8u + h) * 512u + lane * 16u) = vl;
                    }
                    if (lane == 0) alphas[h] = __fmul_rn(alpha, p.softmaxScale);
                    raw[0][0] = raw[1][0]; raw[0][1] = raw[1][1]; raw[1][0] = raw[2][0]; raw[1][1] = raw[2][1];
                    raw[2][0] = raw[3][0]; raw[2][1] = raw[3][1];
                }
            }
            fence_proxy_async_smem();
        }
        mbar_arrive(sm.bar(kBarQReady + qbuf));
        cursor_next_item(cur, items, plan);
    }
}

template <bool DEBUG>
__device__ void softmax_loop(const SharedKVArgs &p, const SharedKVDebug &dbg, const Shared &sm, const Item *items,
                             const PlanResult &plan, uint32_t tmem)
{
    const uint32_t half = threadIdx.x >> 7;        // 0: heads 0-3, 1: heads 4-7
    const uint32_t key = threadIdx.x & 127u;       // key within a tile
    const uint32_t lane = key & 31u, warp = key >> 5;
    const uint32_t tmem_lane = tmem + ((warp * 32u) << 16);
    float *red = reinterpret_cast<float *>(sm.ptr + kSmRed) + half * 32u;     // [2 parities][4 warps][4], per half
    volatile uint32_t *misc = sm.misc();
    uint32_t group_phase = 0, all_phase = 0;

    float sink[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) sink[i] = reinterpret_cast<const float *>(p.sinks)[half * 4u + i];
    const uint32_t ori_tiles = original_tiles(p);

    Cursor cur;
    cursor_init(cur, items, plan);

    uint32_t gt = 0;                               // tiles consumed so far by this CTA
    for (uint32_t k = 0; !cur.done; ++k) {
        const Item it = cur.it;
        // alpha * softmax_scale of this item's query rows; written by the query warps before the
        // S product of the item's first tile of the kind was issued
        const float *alphas = reinterpret_cast<const float *>(sm.ptr + kSmAlpha) + (k & 7u) * 16u;
        float m[4], l[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            m[i] = sink[i];
            l[i] = (key == 0 && it.tile_begin == 0) ? 1.f : 0.f;
        }
        for (uint32_t j = it.tile_begin; j < it.tile_end; ++j, ++gt) {
            const uint32_t kind = j < ori_tiles ? 0u : 1u;
            const uint32_t stage = gt % kStages, buf = gt & 1u, ph = (gt >> 1) & 1u;
            if (!wait_phase<0>(sm, kBarFull + stage, (gt / kStages) & 1u)) return;
            const uint32_t mask_word = reinterpret_cast<volatile uint32_t *>(sm.ptr + kSmMask)[stage * 4u + warp];
            const bool valid = (mask_word >> lane) & 1u;
            if (!wait_phase<0>(sm, kBarSFull + buf, ph)) return;
            tc_fence_after();
            uint32_t s_hi[4], s_lo[4];
            tmem_ld4(tmem_lane + kColS + buf * 16u + half * 4u, s_hi);
            tmem_ld4(tmem_lane + kColS + buf * 16u + 8u + half * 4u, s_lo);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(sm.bar(kBarSFree + buf));

            uint32_t rec = 0;
            if (DEBUG) {
                if (threadIdx.x == 0) misc[2] = atomicAdd(reinterpret_cast<uint32_t *>(dbg.counter), 1u);
                if (!group_sync<0>(sm, 2, all_phase)) return;
                rec = misc[2];
                if (!group_sync<0>(sm, 2, all_phase)) return;      // everyone has read the record before the next is drawn
                if (rec < dbg.maxTiles) {
                    if (threadIdx.x == 0) {
                        int32_t *info = reinterpret_cast<int32_t *>(dbg.tileInfo) + (uint64_t)rec * 4u;
                        info[0] = (int32_t)it.token; info[1] = (int32_t)kind; info[2] = (int32_t)(kind ? j - ori_tiles : j); info[3] = (int32_t)it.part;
                    }
                    if (half == 0 && lane == 0) reinterpret_cast<uint32_t *>(dbg.validMask)[(uint64_t)rec * 4u + warp] = mask_word;
                    int32_t *g = reinterpret_cast<int32_t *>(dbg.qkAcc) + ((uint64_t)rec * 128u + key) * 16u;
                    *reinterpret_cast<uint4 *>(g + half * 4u) = make_uint4(s_hi[0], s_hi[1], s_hi[2], s_hi[3]);
                    *reinterpret_cast<uint4 *>(g + 8u + half * 4u) = make_uint4(s_lo[0], s_lo[1], s_lo[2], s_lo[3]);
                }
            }

            float logit[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float dots = __fadd_rn((float)(int)s_hi[i], __fmul_rn((float)(int)s_lo[i], kInv127));
                logit[i] = valid ? __fmul_rn(dots, alphas[kind * 8u + half * 4u + i]) : kMasked;
            }
            const float wmax = warp_reduce4<true>(logit, lane);
            float *slot_red = red + (gt & 1u) * 16u;
            if ((lane & 7u) == 0) slot_red[warp * 4u + (lane >> 3)] = wmax;
            if (!group_sync<0>(sm, half, group_phase)) return;
            // rescale factors of this tile go to the accumulate warps through an 8-deep ring (the softmax
            // warps can be at most five tiles ahead of the tile being drained)
            float *ring = reinterpret_cast<float *>(sm.ptr + kSmRescale) + (gt & 7u) * 16u;
            int p_hi[4], p_lo[4];
            float r[4];
            const float4 q0 = reinterpret_cast<const float4 *>(slot_red)[0], q1 = reinterpret_cast<const float4 *>(slot_red)[1];
            const float4 q2 = reinterpret_cast<const float4 *>(slot_red)[2], q3 = reinterpret_cast<const float4 *>(slot_red)[3];
            const float tmaxes[4] = {fmaxf(fmaxf(q0.x, q1.x), fmaxf(q2.x, q3.x)), fmaxf(fmaxf(q0.y, q1.y), fmaxf(q2.y, q3.y)),
                                     fmaxf(fmaxf(q0.z, q1.z), fmaxf(q2.z, q3.z)), fmaxf(fmaxf(q0.w, q1.w), fmaxf(q2.w, q3.w))};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float mnew = fmaxf(m[i], tmaxes[i]);
                r[i] = mnew == m[i] ? 1.f : fast_exp(__fsub_rn(m[i], mnew));
                const float w = fast_exp(__fsub_rn(logit[i], mnew));
                l[i] = __fmaf_rn(l[i], r[i], w);
                // round-half-even of a value in [0, 127] without the conversion unit: adding and
                // subtracting 1.5 * 2^23 leaves the nearest integer; its low mantissa bits are the code
                const float w127 = __fmul_rn(w, 127.f);
                const float shifted = __fadd_rn(w127, 12582912.f);
                const float hf = __fsub_rn(shifted, 12582912.f);
                p_hi[i] = (int)(__float_as_uint(shifted) - 0x4b400000u);
                const float shifted_lo = __fadd_rn(__fmul_rn(__fsub_rn(w127, hf), 127.f), 12582912.f);
                p_lo[i] = (int)(__float_as_uint(shifted_lo) - 0x4b400000u);
                m[i] = mnew;
            }
            if (key == 0) {
                *reinterpret_cast<float4 *>(ring + half * 4u) = make_float4(r[0], r[1], r[2], r[3]);
                if (half == 0) reinterpret_cast<uint32_t *>(ring)[8] = rec;
                mbar_arrive(sm.bar(kBarRescale + (gt & 7u)));
            }
            // the O product that read this P buffer two tiles ago must be complete before it is rewritten
            if (gt >= 2u && !wait_phase<0>(sm, kBarOFull + buf, ph ^ 1u)) return;
            uint32_t *pdst = reinterpret_cast<uint32_t *>(sm.ptr + kSmP + buf * 2048u + key * 16u);
            const uint32_t c_hi = pack4(p_hi[0], p_hi[1], p_hi[2], p_hi[3]), c_lo = pack4(p_lo[0], p_lo[1], p_lo[2], p_lo[3]);
            pdst[half] = c_hi;
            pdst[2u + half] = c_lo;
            if (DEBUG && rec < dbg.maxTiles) {
                uint32_t *g = reinterpret_cast<uint32_t *>(dbg.pCodes) + ((uint64_t)rec * 128u + key) * 4u;
                g[half] = c_hi;
                g[2u + half] = c_lo;
            }
            fence_proxy_async_smem();
            // wait-timeout test: the first tile's P codes are never announced
            if (!(DEBUG && (dbg.reserved & kDebugShortWaits) && gt == 0)) mbar_arrive(sm.bar(kBarPReady + buf));
        }

        // denominators: sum the per-thread partial sums, hand (m, l) to the accumulate warps
        {
            const float wsum = warp_reduce4<false>(l, lane);
            if (!group_sync<0>(sm, half, group_phase)) return;   // everyone is past the last tile's reads of `red`
            if ((lane & 7u) == 0) red[warp * 4u + (lane >> 3)] = wsum;
            if (!group_sync<0>(sm, half, group_phase)) return;
            if (key == 0) {
                float *fin = reinterpret_cast<float *>(sm.ptr + kSmFinal) + (k & 7u) * 16u;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    fin[half * 4u + i] = m[i];
                    fin[8u + half * 4u + i] = __fadd_rn(__fadd_rn(red[i], red[4 + i]), __fadd_rn(red[8 + i], red[12 + i]));
                }
                mbar_arrive(sm.bar(kBarItemDone + (k & 7u)));
            }
        }
        cursor_next_item(cur, items, plan);
    }
}

// ------------------------------------------------------------------ accumulate warps (8-11)
// Thread = channel c of each of the four 128-channel blocks, all eight heads.  Drains the INT32
// PV accumulators of every tile into FP32 running sums, then normalises and stores the token (or
// its partial state, merging when this CTA holds the last piece to arrive).

// Exact FP32 value of an integer of magnitude below 2^22 without the conversion unit: adding the
// integer to the bit pattern of 1.5 * 2^23 yields the float 1.5 * 2^23 + x, from which the
// constant is subtracted exactly.  |PV accumulator| <= 127 * 127 * 128 < 2^21.
__device__ __forceinline__ float small_int_to_float(uint32_t x)
{
    return __fsub_rn(__uint_as_float(x + 0x4b400000u), 12582912.f);
}

template <bool DEBUG>
__device__ void accumulate_loop(const SharedKVArgs &p, const SharedKVDebug &dbg, const Shared &sm, const uint32_t live_tokens,
                                const Item *items, const PlanResult &plan, uint32_t tmem)
{
    const uint32_t ch = threadIdx.x - 256u;        // 0..127
    const uint32_t warp = ch >> 5;
    const uint32_t tmem_lane = tmem + ((warp * 32u) << 16);
    char *ws = reinterpret_cast<char *>(p.workspace);
    uint32_t *tickets = reinterpret_cast<uint32_t *>(ws + kWsTickets);
    float *partials = reinterpret_cast<float *>(ws + ws_partials(p.tokens));
    volatile uint32_t *misc = sm.misc();
    uint32_t group_phase = 0;

    // cache scale / 127 of this thread's four channels (the reference multiplies by the scale and
    // by 1/127 in turn; folding the two constants differs by at most one rounding of the product)
    float sc[2][4];
#pragma unroll
    for (int kind = 0; kind < 2; ++kind)
#pragma unroll
        for (int mb = 0; mb < 4; ++mb)
            sc[kind][mb] = __fmul_rn(__ldg(reinterpret_cast<const float *>(kind ? p.cmpScale : p.oriScale) + mb * 128 + ch), kInv127);

    // rows past the live token count are cleared (csrc/kernels/c8/attention_impl.h:443-460 of the reference)
    {
        const uint32_t live = live_tokens;
        for (uint32_t t = live + blockIdx.x; t < p.tokens; t += gridDim.x) {
            uint4 *o = reinterpret_cast<uint4 *>(p.out) + (uint64_t)t * 512u;
            for (uint32_t i = ch; i < 512u; i += 128u) o[i] = make_uint4(0, 0, 0, 0);
            if (p.lse && ch < 8) reinterpret_cast<float *>(p.lse)[(uint64_t)t * 8u + ch] = 0.f;
        }
    }

    const uint32_t ori_tiles = original_tiles(p);
    Cursor cur;
    cursor_init(cur, items, plan);
    uint32_t gt = 0;
    for (uint32_t k = 0; !cur.done; ++k) {
        const Item it = cur.it;
        float acc[4][8];
#pragma unroll
        for (int mb = 0; mb < 4; ++mb)
#pragma unroll
            for (int h = 0; h < 8; ++h) acc[mb][h] = 0.f;

        for (uint32_t j = it.tile_begin; j < it.tile_end; ++j, ++gt) {
            const uint32_t buf = gt & 1u, ph = (gt >> 1) & 1u, slot = gt & 7u;
            if (!wait_phase<1>(sm, kBarRescale + slot, (gt >> 3) & 1u)) return;
            const float4 *ring = reinterpret_cast<const float4 *>(sm.ptr + kSmRescale + slot * 64u);
            const float4 ra = ring[0], rb = ring[1];
            const float r[8] = {ra.x, ra.y, ra.z, ra.w, rb.x, rb.y, rb.z, rb.w};
            const uint32_t rec = DEBUG ? reinterpret_cast<const uint32_t *>(ring)[8] : 0u;
            // once the running maxima have settled every factor is exactly 1 and the multiply is skipped
            const bool rescale = (ra.x != 1.f) | (ra.y != 1.f) | (ra.z != 1.f) | (ra.w != 1.f) | (rb.x != 1.f) | (rb.y != 1.f) |
                                 (rb.z != 1.f) | (rb.w != 1.f);
            if (rescale) {
#pragma unroll
                for (int mb = 0; mb < 4; ++mb)
#pragma unroll
                    for (int h = 0; h < 8; ++h) acc[mb][h] = __fmul_rn(acc[mb][h], r[h]);
            }
            if (!wait_phase<1>(sm, kBarOFull + buf, ph)) return;
            tc_fence_after();
#pragma unroll
            for (uint32_t half = 0; half < 2; ++half) {        // two channel blocks at a time keeps registers in budget
                uint32_t o[2][16];
                tmem_ld16(tmem_lane + kColO + buf * 64u + (2u * half) * 16u, o[0]);
                tmem_ld16(tmem_lane + kColO + buf * 64u + (2u * half + 1u) * 16u, o[1]);
                tmem_wait_ld();
                if (half == 1) {
                    tc_fence_before();
                    mbar_arrive(sm.bar(kBarOFree + buf));
                }
#pragma unroll
                for (uint32_t q = 0; q < 2; ++q) {
                    const uint32_t mb = 2u * half + q;
                    if (DEBUG && rec < dbg.maxTiles) {
                        uint4 *g = reinterpret_cast<uint4 *>(dbg.pvAcc) + ((uint64_t)rec * 512u + mb * 128u + ch) * 4u;
#pragma unroll
                        for (int i = 0; i < 4; ++i) g[i] = make_uint4(o[q][4 * i], o[q][4 * i + 1], o[q][4 * i + 2], o[q][4 * i + 3]);
                    }
                    const float s = j < ori_tiles ? sc[0][mb] : sc[1][mb];
#pragma unroll
                    for (int h = 0; h < 8; ++h) {
                        const float dots = __fmaf_rn(small_int_to_float(o[q][8 + h]), kInv127, small_int_to_float(o[q][h]));
                        acc[mb][h] = __fmaf_rn(dots, s, acc[mb][h]);
                    }
                }
            }
        }

        // final (m, l) of this item from the softmax warps
        if (!wait_phase<1>(sm, kBarItemDone + (k & 7u), (k >> 3) & 1u)) return;
        const float *fin = reinterpret_cast<const float *>(sm.ptr + kSmFinal) + (k & 7u) * 16u;

        __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(p.out) + (uint64_t)it.token * 4096u;
        float *lse = p.lse ? reinterpret_cast<float *>(p.lse) + (uint64_t)it.token * 8u : nullptr;
        if (it.nparts == 1) {
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                // one correctly rounded reciprocal per head instead of 32 divisions (differs from the
                // quotient by at most one FP32 ulp before the BF16 rounding)
                const float inv = __frcp_rn(fin[8 + h]);
#pragma unroll
                for (int mb = 0; mb < 4; ++mb)
                    out[h * 512 + mb * 128 + ch] = __float2bfloat16_rn(__fmul_rn(acc[mb][h], inv));
            }
            if (lse && ch < 8) lse[ch] = __fadd_rn(fin[ch], logf(fin[8 + ch]));
            cursor_next_item(cur, items, plan);
            continue;
        }

        // ---------------- piece of a token shared with other CTAs
        // Every piece writes its state to the workspace, makes it visible and then draws a ticket; the
        // piece that draws the last one finds all states written and merges them in piece order (so the
        // result does not depend on who arrives when).  Nobody waits for another CTA.
        float *mine = partials + (uint64_t)split::partial_slot(it.first_cta, it.part) * kPartialFloats;
#pragma unroll
        for (int h = 0; h < 8; ++h)
#pragma unroll
            for (int mb = 0; mb < 4; ++mb) mine[h * 512 + mb * 128 + ch] = acc[mb][h];
        if (ch < 16) mine[4096 + ch] = fin[ch];
        // One thread draws the ticket with release / acquire semantics at GPU scope behind a barrier of
        // the 128 writers: the barrier orders their stores before the draw, the release publishes
        // them with it, the acquire (and the second barrier) orders the merger's reads behind it.
        if (!group_sync<1>(sm, 3, group_phase)) return;
        uint32_t *ticket = tickets + split::ticket_index(it.first_cta);
        if (ch == 0) misc[3] = atomic_add_acq_rel(ticket, 1u);
        if (!group_sync<1>(sm, 3, group_phase)) return;
        if (misc[3] + 1u == it.nparts) {
            // the ticket goes back to zero for the next launch (nobody else touches it any more in this one)
            if (ch == 0) *ticket = 0u;
            // The loops over the pieces are unrolled so that the loads of several pieces are in flight
            // together: a merge is a chain of L2 round trips at the very end of a CTA's work.
            float top[8], den[8];
#pragma unroll
            for (int h = 0; h < 8; ++h) { top[h] = -INFINITY; den[h] = 0.f; }
#pragma unroll 4
            for (uint32_t q = 0; q < it.nparts; ++q) {
                const float *pm = partials + (uint64_t)split::partial_slot(it.first_cta, q) * kPartialFloats + 4096;
#pragma unroll
                for (int h = 0; h < 8; ++h) top[h] = fmaxf(top[h], __ldcg(pm + h));
            }
#pragma unroll
            for (int mb = 0; mb < 4; ++mb)
#pragma unroll
                for (int h = 0; h < 8; ++h) acc[mb][h] = 0.f;
#pragma unroll 2
            for (uint32_t q = 0; q < it.nparts; ++q) {
                const float *ps = partials + (uint64_t)split::partial_slot(it.first_cta, q) * kPartialFloats;
#pragma unroll
                for (int h = 0; h < 8; ++h) {
                    const float g = expf(__fsub_rn(__ldcg(ps + 4096 + h), top[h]));
                    den[h] = __fadd_rn(den[h], __fmul_rn(__ldcg(ps + 4104 + h), g));
#pragma unroll
                    for (int mb = 0; mb < 4; ++mb)
                        acc[mb][h] = __fadd_rn(acc[mb][h], __fmul_rn(__ldcg(ps + h * 512 + mb * 128 + ch), g));
                }
            }
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                const float inv = __frcp_rn(den[h]);
#pragma unroll
                for (int mb = 0; mb < 4; ++mb)
                    out[h * 512 + mb * 128 + ch] = __float2bfloat16_rn(__fmul_rn(acc[mb][h], inv));
            }
            if (lse && ch < 8) {
                float mm = top[0], ll = den[0];
#pragma unroll
                for (int h = 1; h < 8; ++h) if (ch == (uint32_t)h) { mm = top[h]; ll = den[h]; }
                lse[ch] = __fadd_rn(mm, logf(ll));
            }
        }
        cursor_next_item(cur, items, plan);
    }
}

// ------------------------------------------------------------------ decode kernel
template <bool DEBUG, bool TMA>
__global__ void __launch_bounds__(kThreads, 1) decode_kernel(const SharedKVArgs p, const SharedKVDebug dbg,
                                                             const __grid_constant__ CUtensorMap ori_map,
                                                             const __grid_constant__ CUtensorMap cmp_map,
                                                             const __grid_constant__ CUtensorMap cmp_page_map)
{
    extern __shared__ char smem_raw[];
    Shared sm;
    {
        const uint32_t raw = smem_addr(smem_raw);
        const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
        sm.base = raw + pad;
        sm.ptr = smem_raw + pad;
    }
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    volatile uint32_t *misc = sm.misc();

    if (tid == 0) {
        for (uint32_t s = 0; s < kStages; ++s) { mbar_init(sm.bar(kBarFull + s), TMA ? 4 : 128); mbar_init(sm.bar(kBarEmpty + s), 1); }
        for (uint32_t b = 0; b < 2; ++b) {
            mbar_init(sm.bar(kBarSFull + b), 1); mbar_init(sm.bar(kBarSFree + b), 256);
            mbar_init(sm.bar(kBarPReady + b), 256); mbar_init(sm.bar(kBarOFull + b), 1); mbar_init(sm.bar(kBarOFree + b), 128);
            mbar_init(sm.bar(kBarGroup + b), 128);          // one per softmax half
            mbar_init(sm.bar(kBarGroup + 2 + b), b == 0 ? 256 : 128);      // all softmax threads; all accumulate threads
        }
        for (uint32_t b = 0; b < 3; ++b) { mbar_init(sm.bar(kBarQReady + b), 32); mbar_init(sm.bar(kBarQFree + b), 1); }
        for (uint32_t i = 0; i < 8; ++i) { mbar_init(sm.bar(kBarRescale + i), 2); mbar_init(sm.bar(kBarItemDone + i), 2); }
        misc[1] = 0; misc[2] = 0; misc[3] = 0;
        misc[4] = (DEBUG && (dbg.reserved & kDebugShortWaits)) ? kWaitMillionCyclesTest : kWaitMillionCycles;
        fence_mbar_init();
    }
    if (warp == kWarpMma) {
        tmem_alloc(sm.base + kSmMisc, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];
    // Everything above touched only this CTA's shared and tensor memory.  From here on global memory
    // is read and written, which the previous kernel of the stream may still be producing or using
    // (a query projection, the cache writer, an attention launch that shares this workspace).
    grid_dependency_launch_dependents();
    // The work split starts with cuQ and seqLens; ask for their lines now.  A prefetch consumes no
    // value: whatever the previous kernel still writes there reaches L2 before the wait returns.
    if (tid <= p.batch) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const int32_t *>(p.cuQ) + tid));
        if (tid < p.batch) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const int32_t *>(p.seqLens) + tid));
    }
    grid_dependency_wait();

    const char *ws = reinterpret_cast<const char *>(p.workspace);
    const Item *items = reinterpret_cast<const Item *>(ws + kWsItems);
    plan_cta(p, gridDim.x, reinterpret_cast<PlanScratch *>(sm.ptr + kSmKv), reinterpret_cast<PlanResult *>(sm.ptr + kSmPlan));
    const PlanResult &plan = *reinterpret_cast<const PlanResult *>(sm.ptr + kSmPlan);

    // Roles by warpgroup (four warps, one per SM sub-partition); the register file is re-divided
    // first: the groups that need few registers release them before the others grow.
    if (warp < 8) {
        if (kRegsSoftmax > kRegsLaunch) registers_acquire<kRegsSoftmax>();
        softmax_loop<DEBUG>(p, dbg, sm, items, plan, tmem);
    } else if (warp < kWarpProducer) {
        registers_acquire<kRegsAccumulate>();
        accumulate_loop<DEBUG>(p, dbg, sm, plan.live_tokens, items, plan, tmem);
    } else if (warp < kWarpMma || warp >= kWarpProducerB) {
        registers_release<kRegsProducer>();
        if (TMA && lane == 0) {
            tma_prefetch_descriptor(&ori_map);
            tma_prefetch_descriptor(p.ratio == 4u ? &cmp_map : &cmp_page_map);
        }
        const uint32_t set = warp >= kWarpProducerB ? 1u : 0u;
        // One kernel function serves both layer kinds (a launch of ANOTHER kernel function costs about
        // 4 us more than a launch of the same one, measured on alternating C4 / C128 layers); the
        // producers, the only role whose code depends on the kind, exist once per kind.  Ratio 1
        // (no compressed cache) takes the ratio-128 producers and never reaches a compressed tile.
        if (p.ratio == 4u)
            producer_loop<4, TMA, false>(p, sm, items, plan, set, (warp - kWarpProducer) & 3u, lane, &ori_map, &cmp_map, &cmp_page_map);
        else
            producer_loop<128, TMA, false>(p, sm, items, plan, set, (warp - kWarpProducer) & 3u, lane, &ori_map, &cmp_map, &cmp_page_map);
        cp_async_wait<0>();
    } else {
        if (kRegsIssue < kRegsLaunch) registers_release<kRegsIssue>();
        if (warp >= kWarpQuery) {
            query_loop<DEBUG>(p, dbg, sm, items, plan, warp - kWarpQuery, lane);
        } else {
            // the whole warp runs the issue loop and one elected lane issues: with converged control
            // flow the operand descriptors live in uniform registers, which halves the cost per MMA
            if (warp == kWarpMma) mma_qk_loop(sm, items, plan, tmem, original_tiles(p));
            else mma_pv_loop(sm, plan, tmem);
            __syncwarp();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (misc[1]) {
        // A wait ran out: every role has returned.  Row fetches and MMAs that were already issued
        // may still be writing this CTA's shared and tensor memory, so the CTA stays for a while
        // (far longer than a DRAM round trip) before it gives them up.  The status word is sticky.
        if (tid == 0) reinterpret_cast<PlanHeader *>(const_cast<char *>(ws))->status = kStatusWaitTimeout;
        for (uint32_t waited = 0; waited < kDrainNanoseconds; waited += 1000u) __nanosleep(1000u);
        __syncthreads();
    }
    if (warp == kWarpMma) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

#include "decode_paired.cuh"

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link against libcuda).
using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encode_tiled()
{
    static std::atomic<void *> cached{nullptr};
    void *fn = cached.load(std::memory_order_acquire);
    if (fn == nullptr) {
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status) != cudaSuccess ||
            status != cudaDriverEntryPointSuccess)
            return nullptr;
        cached.store(fn, std::memory_order_release);
    }
    return reinterpret_cast<EncodeTiled>(fn);
}

// 2-D view of a paged cache for row gathers: [kRowsInMap rows, 512 bytes], 512-byte pitch; row id =
// page * (page stride / 512) + row in page.  Box = one 128-byte column block of one row.
bool make_row_map(CUtensorMap *map, uint64_t base)
{
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const cuuint64_t dims[2] = {kDim, (cuuint64_t)kRowsInMap};
    const cuuint64_t strides[1] = {kDim};
    const cuuint32_t box[2] = {128, 1};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, reinterpret_cast<void *>(base), dims, strides, box,
                  element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D view of a paged cache for whole-page fetches: [pages, 32 rows, 512 bytes]; box = one page's
// 128-byte column block (4 KB).
bool make_page_map(CUtensorMap *map, uint64_t base, uint64_t page_stride)
{
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const cuuint64_t dims[3] = {kDim, kPage, (cuuint64_t)1 << 31};
    const cuuint64_t strides[2] = {kDim, page_stride};
    const cuuint32_t box[3] = {128, kPage, 1};
    const cuuint32_t element_strides[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, reinterpret_cast<void *>(base), dims, strides, box,
                  element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The tensor maps of a launch depend only on the cache base addresses and the compressed page
// stride, which a serving layer keeps for its lifetime; encoding them costs microseconds of host
// time per call.  Each host thread keeps the maps of the layers it launched last in a small
// direct-mapped table (thread-local: no lock, no allocation); a miss encodes and replaces.
struct MapSet {
    uint64_t ori, cmp, cmp_stride;      // key; ori == 0 marks an empty entry
    bool with_page_map;
    CUtensorMap ori_map, cmp_map, cmp_page_map;
};
constexpr uint32_t kMapSets = 128;
const MapSet *tensor_maps(uint64_t ori, uint64_t cmp, uint64_t cmp_stride, bool with_page_map)
{
    static thread_local MapSet table[kMapSets];
    const uint64_t mixed = (ori >> 9) * 0x9e3779b97f4a7c15ull ^ (cmp >> 9) * 0xc2b2ae3d27d4eb4full ^ cmp_stride;
    MapSet &e = table[(mixed >> 40) % kMapSets];
    if (e.ori == ori && e.cmp == cmp && e.cmp_stride == cmp_stride && e.with_page_map == with_page_map) return &e;
    e.ori = 0;
    memset(&e.cmp_page_map, 0, sizeof(e.cmp_page_map));
    if (!make_row_map(&e.ori_map, ori) || !make_row_map(&e.cmp_map, cmp) ||
        (with_page_map && !make_page_map(&e.cmp_page_map, cmp, cmp_stride)))
        return nullptr;
    e.ori = ori; e.cmp = cmp; e.cmp_stride = cmp_stride; e.with_page_map = with_page_map;
    return &e;
}

template <bool DEBUG, bool TMA>
cudaError_t launch_decode(const SharedKVArgs &a, const SharedKVDebug &d, const CUtensorMap &ori_map,
                          const CUtensorMap &cmp_map, const CUtensorMap &cmp_page_map, uint32_t grid,
                          cudaStream_t stream, int device)
{
    // the opt-in to > 48 KB of dynamic shared memory is per device and per kernel
    static std::atomic<uint64_t> configured{0};
    const bool cached = device >= 0 && device < kMaxDevices;
    const uint64_t bit = cached ? 1ull << device : 0ull;
    if (!cached || !(configured.load(std::memory_order_relaxed) & bit)) {
        cudaError_t e = cudaFuncSetAttribute(decode_kernel<DEBUG, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kSmemBytes);
        if (e != cudaSuccess) return e;
        configured.fetch_or(bit, std::memory_order_relaxed);
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = programmatic_launch_enabled() ? 1u : 0u;
    return cudaLaunchKernelEx(&config, decode_kernel<DEBUG, TMA>, a, d, ori_map, cmp_map, cmp_page_map);
}

int launch(const SharedKVArgs &a, cudaStream_t stream, const SharedKVDebug *debug, int sms)
{
    uint32_t grid = (uint32_t)sms < kMaxCtas ? (uint32_t)sms : kMaxCtas;
    const uint32_t cap = debug ? (debug->reserved & kDebugCtaCapMask) : 0u;      // test hook: fewer CTAs
    if (cap && cap < grid) grid = cap;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    // Row gathers by TMA need page strides that are whole rows and row ids that fit the map;
    // anything else takes the cp.async producer.
    static const CUtensorMap no_map = {};
    bool tma = a.oriStride % kDim == 0 && a.cmpStride % kDim == 0 && !(debug && (debug->reserved & kDebugLegacyGather)) &&
               (uint64_t)a.oriPages * (a.oriStride / kDim) < (uint64_t)kRowsInMap && a.cmpStride / kDim < 65536;
    const MapSet *maps = tma ? tensor_maps(a.ori, a.cmp, a.cmpStride, a.ratio != 4u) : nullptr;
    if (maps == nullptr) tma = false;
    const CUtensorMap &ori_map = tma ? maps->ori_map : no_map, &cmp_map = tma ? maps->cmp_map : no_map,
                      &cmp_page_map = tma ? maps->cmp_page_map : no_map;
    SharedKVDebug d = {};
    if (debug) {
        d = *debug;
        e = tma ? launch_decode<true, true>(a, d, ori_map, cmp_map, cmp_page_map, grid, stream, device)
                : launch_decode<true, false>(a, d, ori_map, cmp_map, cmp_page_map, grid, stream, device);
    } else {
        e = tma ? launch_decode<false, true>(a, d, ori_map, cmp_map, cmp_page_map, grid, stream, device)
                : launch_decode<false, false>(a, d, ori_map, cmp_map, cmp_page_map, grid, stream, device);
    }
    return (int)e;
}

// Paired-query C128 launch (decode_paired.cuh): same grid, block and tensor maps as launch() of a ratio-128 layer.
template <bool TMA>
cudaError_t launch_decode_paired(const SharedKVArgs &a, uint32_t group, const CUtensorMap &ori_map, const CUtensorMap &cmp_map,
                                 const CUtensorMap &cmp_page_map, uint32_t grid, cudaStream_t stream, int device)
{
    static std::atomic<uint64_t> configured{0};
    const bool cached = device >= 0 && device < kMaxDevices;
    const uint64_t bit = cached ? 1ull << device : 0ull;
    if (!cached || !(configured.load(std::memory_order_relaxed) & bit)) {
        cudaError_t e = cudaFuncSetAttribute(decode_kernel_paired<TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return e;
        configured.fetch_or(bit, std::memory_order_relaxed);
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = programmatic_launch_enabled() ? 1u : 0u;
    return cudaLaunchKernelEx(&config, decode_kernel_paired<TMA>, a, group, ori_map, cmp_map, cmp_page_map);
}

int launch_paired(const SharedKVArgs &a, uint32_t group, cudaStream_t stream, int sms)
{
    const uint32_t grid = (uint32_t)sms < kMaxCtas ? (uint32_t)sms : kMaxCtas;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    static const CUtensorMap no_map = {};
    bool tma = a.oriStride % kDim == 0 && a.cmpStride % kDim == 0 &&
               (uint64_t)a.oriPages * (a.oriStride / kDim) < (uint64_t)kRowsInMap && a.cmpStride / kDim < 65536;
    const MapSet *maps = tma ? tensor_maps(a.ori, a.cmp, a.cmpStride, true) : nullptr;
    if (maps == nullptr) tma = false;
    const CUtensorMap &ori_map = tma ? maps->ori_map : no_map, &cmp_map = tma ? maps->cmp_map : no_map,
                      &cmp_page_map = tma ? maps->cmp_page_map : no_map;
    e = tma ? launch_decode_paired<true>(a, group, ori_map, cmp_map, cmp_page_map, grid, stream, device)
            : launch_decode_paired<false>(a, group, ori_map, cmp_map, cmp_page_map, grid, stream, device);
    return (int)e;
}

}  // namespace

int workspace_status(const void *workspace, cudaStream_t stream)
{
    if (workspace == nullptr) return SHAREDKV_EINVAL;
    uint32_t status = 0;
    cudaError_t e = cudaMemcpyAsync(&status, static_cast<const char *>(workspace) + kWsStatus, sizeof(status),
                                    cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return (int)e;
    return status == kStatusOk ? SHAREDKV_OK : status == kStatusRange ? SHAREDKV_ERANGE : SHAREDKV_ETIMEDOUT;
}

int attention(uint32_t variant, const SharedKVArgs *args, cudaStream_t stream, const SharedKVDebug *debug)
{
    if (args == nullptr) return SHAREDKV_EINVAL;
    const bool general = variant == SHAREDKV_VARIANT_GENERAL;
    const bool packed = variant == SHAREDKV_VARIANT_PACKED || variant == SHAREDKV_VARIANT_PACKED_SPARSE;      // groups of four: two pairs share a tiling
    const bool paired = packed || variant == SHAREDKV_VARIANT_PAIRED || variant == SHAREDKV_VARIANT_PAIRED_SPARSE;
    if (!general && !paired && variant != SHAREDKV_VARIANT_C4 && variant != SHAREDKV_VARIANT_C128 && variant != SHAREDKV_VARIANT_C4_SMALL)
        return SHAREDKV_EVARIANT;
    SharedKVArgs a = *args;
    if (a.tokens == 0 || a.batch == 0) return SHAREDKV_OK;
    // The C4 / C128 entries take their own ratio and no explicit original slots, as the reference's
    // do; the general entry takes ratio 1 (no compressed cache), 4 or 128, with or without them.
    // The paired entries are the C128 arithmetic, and the grouped C4 walk, with two adjacent query tokens of a request per work item.
    const uint32_t ratio = general ? a.ratio
                         : ((variant == SHAREDKV_VARIANT_C128 || variant == SHAREDKV_VARIANT_PAIRED || variant == SHAREDKV_VARIANT_PACKED) ? 128u : 4u);
    if (paired && (debug != nullptr || a.batch + 1u > kPlanStaged)) return SHAREDKV_EINVAL;
    if (a.ratio != ratio || (ratio != 1u && ratio != 4u && ratio != 128u) || (!general && a.oriIndices != 0)) return SHAREDKV_EINVAL;
    if (a.heads != kHeads || a.window != kWindow || a.oriBlock != kPage) return SHAREDKV_EINVAL;
    if (a.oriIndices && (a.oriTopk == 0 || a.oriIndices % 4u)) return SHAREDKV_EINVAL;
    if (ratio == 1u) {
        // no compressed kind: its fields alias the original cache so that nothing in the kernel is null
        a.cmp = a.ori; a.cmpScale = a.oriScale; a.cmpTable = a.oriTable; a.cmpStride = a.oriStride;
        a.cmpBlock = a.oriBlock; a.cmpTableWidth = a.oriTableWidth;
    }
    if (a.cmpBlock != kPage) return SHAREDKV_EINVAL;
    if (ratio == 4 && (a.topk == 0 || a.topk > 1024u || !a.indices || a.indices % 4u)) return SHAREDKV_EINVAL;
    if (!a.q || !a.ori || !a.cmp || !a.oriScale || !a.cmpScale || !a.oriTable || !a.cmpTable || !a.cuQ || !a.seqLens ||
        !a.sinks || !a.out || !a.workspace)
        return SHAREDKV_EINVAL;
    // 16-byte row gathers and vector stores
    if (a.q % 16u || a.out % 16u || a.ori % 16u || a.cmp % 16u || a.oriStride % 16u || a.cmpStride % 16u ||
        a.workspace % 256u || a.oriScale % 4u || a.cmpScale % 4u || a.sinks % 4u || a.lse % 4u || a.oriTable % 4u ||
        a.cmpTable % 4u || a.cuQ % 4u || a.seqLens % 4u)
        return SHAREDKV_EINVAL;
    if (a.oriStride < (uint64_t)kPage * kDim || a.cmpStride < (uint64_t)kPage * kDim) return SHAREDKV_EINVAL;
    if (a.oriTableWidth == 0 || a.cmpTableWidth == 0 || a.oriPages == 0) return SHAREDKV_EINVAL;
    if (debug && (!debug->tileInfo || !debug->validMask || !debug->qkAcc || !debug->pCodes || !debug->pvAcc ||
                  !debug->qCodes || !debug->counter))
        return SHAREDKV_EINVAL;
    const int sms = device_sm_count();
    if (sms <= 0) return (int)cudaErrorInvalidDevice;
    if (paired) return launch_paired(a, packed ? 4u : 2u, stream, sms);
    return launch(a, stream, debug, sms);
}

}  // namespace sharedkv
