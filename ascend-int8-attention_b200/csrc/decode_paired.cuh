// Paired-query variant of the decode kernel (included by decode_attention.cu inside its namespace).
//
// Chunked prefill hands the kernel several query tokens per request.  Walked one by one, adjacent
// tokens fetch almost the same keys: the same compressed prefix and windows that differ by one row.
// Here two adjacent tokens of a request form ONE item, and both tokens ride through every product:
//   S[128 keys, 32] = KV[128, 512] . Qcodes[32, 512]^T     Q rows 16 t + 8 plane + head
//   O[512, 32]      = KV^T[512, 128] . P[128, 32]          P columns in the same order
// (t = token of the pair, plane 0 = high codes, 1 = residual codes).  A tile is fetched once and
// costs one pass through the tensor core, the softmax warps and the accumulate warps for the two
// tokens together; each token keeps its own validity mask, running maximum, sum and accumulators.
// decode_kernel's warp roles, barriers, work-item cursors and producers are reused as they are.
//
// Arithmetic: the reference's tiled oracle with query_group = 2 (npu_sparse_attn_sharedkv_int8/
// reference.py:229-234,243-245): the original rows of an item are the union of its tokens' windows,
// tiled from the union's first row, each token masking the rows outside its own window; the
// compressed rows are the prefix of the later token, the earlier token masking what it may not see.
// Ratio 128, or ratio 4 as the reference groups it (:246-249,300-301): a grouped C4 token does not
// gather its top-k rows but walks ALL compressed rows of the pair's later token; a row counts as
// often as the token's own top-k list names it (log(multiplicity) is added to its logits) and rows
// the list does not name are masked.  The query warp of the compressed kind counts the names into
// a table in shared memory; the bound the reference puts on such plans (contexts of at most 1024
// tokens, attention.py:89-98) makes that table 256 rows per token.  No explicit original slots (the
// reference refuses them with groups too).
//
// Groups of four (query_group = 4): the tiling is that of the four tokens (union of their windows,
// prefix of the fourth); the group is two items, each walking the group's tiles for its two tokens.
//
// Items are not split between CTAs: an item belongs to the CTA in whose share of the cost list it
// begins, so there are no partial states and no merges.  The reference's grouped plans are
// unsplit too (attention.py:112-113: "Grouped-query kernel requires one KV partition").
//
// Shared memory: the 32-row query codes (16 KB a set) and the 32-column P codes do not fit beside
// three 64 KB key tiles, so the key ring has two stages and the third stage's 64 KB hold them.  The
// price: at most two tiles are anywhere between their fetch and their O product, so the stages of a
// tile overlap less with the next tile's than in decode_kernel.
//
// Query codes: a ring of three buffers.  An item needs one set of codes per cache kind it has tiles
// of ("uses": original, then compressed); the n-th use of the CTA's life lives in buffer n mod 3,
// so the next item's codes are written while this item's are read.  Both query warps walk every
// use and wait for its buffer (the warp of the use's kind encodes, the other only reports that it
// has been there), so that neither can fall a whole barrier phase behind the other.

constexpr uint32_t kPairStages = 2;
// shared memory inside what is decode_kernel's third key tile; everything else keeps its place
constexpr uint32_t kSmQ2 = kPairStages * kTileBytes;          // 3 buffers x [32 rows x 512 B], 128-byte swizzle
constexpr uint32_t kSmP2 = kSmQ2 + 3 * 16384;                 // 2 buffers x [2 tokens][128 keys][16 B]
constexpr uint32_t kSmRed2 = kSmP2 + 2 * 4096;                // FP32 [2 halves][2 parities][2 tokens][4 warps][4]
constexpr uint32_t kSmAlpha2 = kSmRed2 + 512;                 // FP32 [8 items][2 tokens][2 kinds][8]: alpha * softmax_scale
constexpr uint32_t kSmFinal2 = kSmAlpha2 + 8 * 128;           // FP32 [8 items][2 tokens][16]: m[8], l[8]
constexpr uint32_t kSmMult2 = kSmFinal2 + 8 * 128;            // UINT32 [2 items][2 tokens][256 rows]: grouped C4 multiplicities
constexpr uint32_t kPairSparseRows = split::kPairSparseRows;
static_assert(kSmMult2 + 2 * 2 * kPairSparseRows * 4 <= kStages * kTileBytes, "the paired kernel's extras live inside the third key tile");
// tensor memory: S[b] at 32 b (32 columns), O[b] at 64 + 128 b as four 32-column channel blocks
constexpr uint32_t kTmemCols2 = 512;
constexpr uint32_t kColS2 = 0, kColO2 = 64;

// ------------------------------------------------------------------ what an item says about its tiles
struct PairShape {
    uint32_t tokens;        // 1 or 2
    uint32_t windows;       // original tiles (the window union of the item's group)
    uint32_t tiles;         // all tiles
    uint32_t kinds;         // 1: original tiles only, 2: compressed tiles as well
};
__device__ __forceinline__ PairShape pair_shape(uint32_t batch_word, int32_t first_position, uint32_t tiles)
{
    PairShape s;
    s.tokens = pair_tokens(batch_word);
    s.windows = pair_original_tiles(group_position(first_position, batch_word), group_tokens(batch_word));
    s.tiles = tiles;
    s.kinds = tiles > s.windows ? 2u : 1u;
    return s;
}
__device__ __forceinline__ PairShape pair_shape(const Item &it) { return pair_shape(it.batch, it.position, it.tile_end); }
using split::pair_sees;

// ------------------------------------------------------------------ work split of the paired kernel
// Groups, not tokens, are the unit: request b has ceil(tokens_b / 2) groups.  The flat cost list
// (kItemCost per group plus one unit per tile) is cut into `grid` ranges as in plan_cta, but a
// group is never cut: it goes to the CTA in whose range its first unit lies.  The group with index
// g is workspace entry g, so a CTA's items are consecutive entries.
struct PairPlanScratch {
    uint32_t scan[80];
    uint32_t live, pad[3];
    int32_t cu[kPlanStaged];          // cuQ of the live requests
    uint32_t groups[kPlanStaged];     // exclusive prefix of the groups per request
};
static_assert(sizeof(PairPlanScratch) <= kPairStages * kTileBytes, "the plan's scratch is the key ring");
__device__ __forceinline__ uint32_t owner_of_group(const uint32_t *groups, uint32_t live_batch, uint32_t g)
{
    uint32_t lo = 0, hi = live_batch - 1;
    while (lo < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        if (groups[mid + 1] <= g) lo = mid + 1; else hi = mid;
    }
    return lo;
}
__device__ void plan_cta_paired(const SharedKVArgs &p, const uint32_t group, const uint32_t grid, PairPlanScratch *sc, PlanResult *result)
{
    const uint32_t tid = threadIdx.x;
    const int32_t *cu_global = reinterpret_cast<const int32_t *>(p.cuQ);
    const int32_t *seq = reinterpret_cast<const int32_t *>(p.seqLens);
    char *ws = reinterpret_cast<char *>(p.workspace);
    Item *items = reinterpret_cast<Item *>(ws + kWsItems);

    if (tid == 0) {
        sc->live = 0;
        result->first = 0xffffffffu; result->count = 0; result->tiles = 0;
    }
    for (uint32_t b = tid; b <= p.batch; b += kThreads) sc->cu[b] = cu_global[b];
    __syncthreads();
    uint32_t live = 0;
    for (uint32_t b = tid; b < p.batch; b += kThreads)
        if (split::request_is_live(seq[b], sc->cu[b + 1])) live = b + 1;
    if (live) atomicMax(&sc->live, live);
    __syncthreads();
    const uint32_t live_batch = sc->live;
    const uint32_t live_tokens = split::live_token_count(live_batch ? sc->cu[live_batch] : 0, p.tokens);

    // groups per request -> exclusive prefix in shared memory (thread i owns consecutive requests)
    const uint32_t per_b = (live_batch + kThreads - 1) / kThreads;
    const uint32_t b_begin = min(tid * per_b, live_batch), b_end = min(b_begin + per_b, live_batch);
    auto tokens_of = [&](uint32_t b) {
        const int32_t lo = max(sc->cu[b], 0), hi = min(sc->cu[b + 1], (int32_t)live_tokens);
        return hi > lo ? (uint32_t)(hi - lo) : 0u;
    };
    uint32_t my_groups = 0;
    for (uint32_t b = b_begin; b < b_end; ++b) my_groups += split::pair_groups(tokens_of(b));
    uint32_t total_groups;
    uint32_t running = block_exclusive_scan(my_groups, sc->scan, total_groups);
    for (uint32_t b = b_begin; b < b_end; ++b) {
        sc->groups[b] = running;
        running += split::pair_groups(tokens_of(b));
    }
    if (tid == 0) sc->groups[live_batch] = total_groups;
    __syncthreads();

    // cost of every group: thread i owns consecutive groups
    const uint32_t per = (total_groups + kThreads - 1) / kThreads;
    const uint32_t g_begin = min(tid * per, total_groups), g_end = min(g_begin + per, total_groups);
    struct Group {
        uint32_t token, batch_word, tiles;
        int32_t position;
    };
    auto describe = [&](uint32_t g) {
        Group d;
        const uint32_t b = owner_of_group(sc->groups, live_batch, g);
        const uint32_t pair = g - sc->groups[b];                  // pair of the request; `group` / 2 pairs share a tiling
        const uint32_t t0 = (uint32_t)max(sc->cu[b], 0) + 2u * pair;
        const uint32_t last_token = (uint32_t)min(sc->cu[b + 1], (int32_t)live_tokens);
        const uint32_t tokens = min(2u, last_token - t0);
        const uint32_t second = group == 4u ? pair & 1u : 0u;      // this pair's first token is its group's third
        const uint32_t in_group = min(group, last_token - (t0 - 2u * second));
        d.token = t0;
        d.position = split::token_position(seq[b], sc->cu[b + 1], t0);
        d.batch_word = b | (tokens == 2u ? kPairBit : 0u) | (second ? kPairSecondBit : 0u) | (in_group << kPairGroupShift);
        d.tiles = split::pair_tiles(d.position - 2 * (int32_t)second, in_group, p.ratio);
        return d;
    };
    uint32_t my_cost = 0;
    for (uint32_t g = g_begin; g < g_end; ++g) my_cost += split::kItemCost + describe(g).tiles;
    uint32_t total;
    uint32_t start = block_exclusive_scan(my_cost, sc->scan, total);
    const uint32_t quota = split::quota_of(total, grid);
    const uint32_t me = blockIdx.x;
    uint32_t found = 0, tiles = 0, my_entry = 0xffffffffu;
    uint4 my_lo = make_uint4(0, 0, 0, 0), my_hi = my_lo;
    for (uint32_t g = g_begin; g < g_end; ++g) {
        const Group d = describe(g);
        if (split::pair_owner(start, quota) == me) {
            const uint4 lo = make_uint4(d.token, d.batch_word, (uint32_t)d.position, 0u);
            const uint4 hi = make_uint4(d.tiles, 0u, 1u, 0u);
            uint4 *dst = reinterpret_cast<uint4 *>(items + g);
            dst[0] = lo;
            dst[1] = hi;
            if (!found) { my_entry = g; my_lo = lo; my_hi = hi; }
            ++found;
            tiles += d.tiles;
        }
        start += split::kItemCost + d.tiles;
    }
    if (found) {
        atomicMin(&result->first, my_entry);
        atomicAdd(&result->count, found);
        atomicAdd(&result->tiles, tiles);
    }
    __syncthreads();
    if (my_entry == result->first) { result->first_item[0] = my_lo; result->first_item[1] = my_hi; }
    if (tid == 0) {
        result->live_tokens = live_tokens;
        if (result->count == 0) result->first = 0;
        if (me == 0) {
            PlanHeader *header = reinterpret_cast<PlanHeader *>(ws);
            header->live_batch = live_batch; header->live_tokens = live_tokens; header->total_tiles = total;
            header->quota = quota; header->n_items = total_groups; header->grid = grid;
        }
    }
    __syncthreads();
}

// ------------------------------------------------------------------ query warps (18: original kind, 19: compressed kind)
// Lane l owns channels 16 l .. 16 l + 15.  Encodes the eight query rows of one token for one cache
// kind into rows `first_row` + head (high codes) and `first_row` + 8 + head (residual codes) of a
// 32-row code buffer and publishes alpha * softmax_scale per head; the arithmetic is query_loop's
// (csrc/kernels/c8/vector.h:179-213 of the reference).
__device__ __forceinline__ void pair_encode_token(const SharedKVArgs &p, uint32_t token, const float (&sc)[16], char *qdst,
                                                  uint32_t first_row, float *alphas, uint32_t lane)
{
    const uint4 *src = reinterpret_cast<const uint4 *>(p.q + (uint64_t)token * 8192u) + lane * 2u;
    uint4 raw[4][2];                               // four heads of loads in flight at a time
#pragma unroll 1
    for (uint32_t batch = 0; batch < 2; ++batch) {
#pragma unroll
        for (int h = 0; h < 4; ++h) { raw[h][0] = __ldg(src + (4 * batch + h) * 64); raw[h][1] = __ldg(src + (4 * batch + h) * 64 + 1); }
#pragma unroll 1
        for (uint32_t hh = 0; hh < 4; ++hh) {
            const uint32_t h = batch * 4u + hh;
            const uint32_t *rw = reinterpret_cast<const uint32_t *>(raw[0]);      // the four heads rotate through slot 0
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
                // round-half-even through the adder, as in query_loop
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
            *reinterpret_cast<uint4 *>(qdst + tile_offset(first_row + h, lane, 4096u)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4 *>(qdst + tile_offset(first_row + 8u + h, lane, 4096u)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            if (lane == 0) alphas[h] = __fmul_rn(alpha, p.softmaxScale);
            raw[0][0] = raw[1][0]; raw[0][1] = raw[1][1]; raw[1][0] = raw[2][0]; raw[1][1] = raw[2][1];
            raw[2][0] = raw[3][0]; raw[2][1] = raw[3][1];
        }
    }
}

__device__ void pair_query_loop(const SharedKVArgs &p, const Shared &sm, const Item *items, const PlanResult &plan, uint32_t kind,
                                uint32_t lane)
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
    Cursor cur;
    cursor_init(cur, items, plan);
    uint32_t buf = 0, round = 0;             // the next use is number 3 * round + buf
    for (uint32_t k = 0; !cur.done; ++k) {
        const Item it = cur.it;
        const PairShape shape = pair_shape(it);
        if (kind == 0 && cur.k + 1 < plan.count) {        // the next item's query rows start their way to L2 now
            const char *next = reinterpret_cast<const char *>(p.q) + (uint64_t)cur.next_lo.x * 8192u + lane * 256u;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(next));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(next + 128));
            if (cur.next_lo.y & kPairBit) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(next + 8192));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(next + 8192 + 128));
            }
        }
        for (uint32_t use_kind = 0; use_kind < shape.kinds; ++use_kind) {
            // the use that had the buffer before must no longer be read
            if (round > 0 && !wait_phase<3>(sm, kBarQFree + buf, (round - 1u) & 1u)) return;
            if (use_kind == kind) {
                if (kind == 1 && p.ratio == 4u) {
                    // grouped C4: how often each token's top-k list names each compressed row.  The table
                    // slot was last read for item k - 2, which the softmax warps have finished by now.
                    if (k >= 2 && !wait_phase<3>(sm, kBarItemDone + ((k - 2u) & 7u), ((k - 2u) >> 3) & 1u)) return;
                    uint32_t *table = reinterpret_cast<uint32_t *>(sm.ptr + kSmMult2) + (k & 1u) * 2u * kPairSparseRows;
                    for (uint32_t i = lane; i < 2u * kPairSparseRows; i += 32u) table[i] = 0u;
                    __syncwarp();
                    bool beyond = false;
                    for (uint32_t token = 0; token < shape.tokens; ++token) {
                        const int32_t position = it.position + (int32_t)token;
                        const uint32_t count = position < 0 ? 0u : ((uint32_t)position + 1u) / 4u;
                        beyond |= count > kPairSparseRows;
                        const int32_t *ix = reinterpret_cast<const int32_t *>(p.indices) + (uint64_t)(it.token + token) * p.topk;
                        for (uint32_t i = lane; i < p.topk; i += 32u) {
                            const int32_t v = ix[i];
                            if (v >= 0 && (uint32_t)v < count && (uint32_t)v < kPairSparseRows) atomicAdd(table + token * kPairSparseRows + (uint32_t)v, 1u);
                        }
                    }
                    // a context beyond the table is outside this entry's contract: the launch is marked as failed
                    if (beyond && lane == 0) reinterpret_cast<PlanHeader *>(reinterpret_cast<char *>(p.workspace))->status = kStatusRange;
                    __syncwarp();
                }
                // rows of a token the item does not have keep whatever they held: their S columns are never read
                for (uint32_t token = 0; token < shape.tokens; ++token) {
                    float *alphas = reinterpret_cast<float *>(sm.ptr + kSmAlpha2) + ((k & 7u) * 2u + token) * 16u + kind * 8u;
                    pair_encode_token(p, it.token + token, sc, sm.ptr + kSmQ2 + buf * 16384u, 16u * token, alphas, lane);
                }
                fence_proxy_async_smem();
            }
            mbar_arrive(sm.bar(kBarQReady + buf));
            if (++buf == 3u) { buf = 0; ++round; }
        }
        cursor_next_item(cur, items, plan);
    }
}

// ------------------------------------------------------------------ S = K.Q^T issuer (warp 16)
__device__ void pair_qk_loop(const Shared &sm, const Item *items, const PlanResult &plan, uint32_t tmem)
{
    constexpr uint32_t kIdescQK = idesc_i8(128, 32, 0, 0);
    const bool leader = elect_one();
    const uint32_t count = __shfl_sync(0xffffffffu, plan.count, 0);
    Cursor cq;
    cursor_init(cq, items, plan);
    uint32_t t = 0, uses = 0;              // tiles issued / code uses before this item
    for (uint32_t k = 0; k < count; ++k) {
        const PairShape shape = pair_shape(__shfl_sync(0xffffffffu, cq.it.batch, 0), (int32_t)__shfl_sync(0xffffffffu, (uint32_t)cq.it.position, 0),
                                           __shfl_sync(0xffffffffu, cq.it.tile_end, 0));
        for (uint32_t j = 0; j < shape.tiles; ++j, ++t) {
            const uint32_t buf = t & 1u, ph = (t >> 1) & 1u;          // key stage and S buffer alternate together
            const uint32_t kind = j < shape.windows ? 0u : 1u, use = uses + kind;
            const uint32_t b = use % 3u;
            const bool first_of_kind = j == 0 || j == shape.windows;
            const bool last_of_kind = j + 1u == shape.windows || j + 1u == shape.tiles;
            if (first_of_kind && !wait_phase<3>(sm, kBarQReady + b, (use / 3u) & 1u)) return;
            if (!wait_phase<3>(sm, kBarFull + buf, ph)) return;
            if (!wait_phase<3>(sm, kBarSFree + buf, ph ^ 1u)) return;
            tc_fence_after();
            const uint32_t kv = sm.base + kSmKv + buf * kTileBytes;
            const uint32_t qb = sm.base + kSmQ2 + b * 16384u;
            const uint64_t a0 = smem_desc(kv, 16u, 1024u, kSwizzle128), b0 = smem_desc(qb, 16u, 1024u, kSwizzle128);
#pragma unroll 1
            for (uint32_t seg = 0; seg < 4; ++seg) {
#pragma unroll
                for (uint32_t part = 0; part < 4; ++part)
                    if (leader)
                        mma_i8(tmem + kColS2 + buf * 32u, a0 + ((seg * kSegBytes + part * 32u) >> 4), b0 + ((seg * 4096u + part * 32u) >> 4),
                               kIdescQK, seg | part);
            }
            if (leader) {
                mma_commit(sm.bar(kBarSFull + buf));
                if (last_of_kind) mma_commit(sm.bar(kBarQFree + b));
            }
        }
        uses += shape.kinds;
        cursor_next_item(cq, items, plan);
    }
}

// ------------------------------------------------------------------ O = K^T.P issuer (warp 17)
__device__ void pair_pv_loop(const Shared &sm, const PlanResult &plan, uint32_t tmem)
{
    constexpr uint32_t kIdescPV = idesc_i8(128, 32, 1, 1);
    const bool leader = elect_one();
    const uint32_t tiles = __shfl_sync(0xffffffffu, plan.tiles, 0);
    for (uint32_t t = 0; t < tiles; ++t) {
        const uint32_t buf = t & 1u, ph = (t >> 1) & 1u;
        if (!wait_phase<3>(sm, kBarPReady + buf, ph)) return;
        if (!wait_phase<3>(sm, kBarOFree + buf, ph ^ 1u)) return;
        tc_fence_after();
        const uint32_t kv = sm.base + kSmKv + buf * kTileBytes;
        const uint32_t pb = sm.base + kSmP2 + buf * 4096u;
        // P: 8-key x 16-byte core matrices, 128 bytes apart along the keys, the two tokens' 16 columns 2048 bytes apart
        const uint64_t a0 = smem_desc(kv, kSegBytes, 1024u, kSwizzle128), b0 = smem_desc(pb, 128u, 2048u, kSwizzleNone);
#pragma unroll 1
        for (uint32_t mb = 0; mb < 4; ++mb) {
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk)
                if (leader)
                    mma_i8(tmem + kColO2 + buf * 128u + mb * 32u, a0 + ((mb * kSegBytes + kk * 4096u) >> 4), b0 + ((kk * 512u) >> 4),
                           kIdescPV, kk);
        }
        if (leader) {
            mma_commit(sm.bar(kBarOFull + buf));
            mma_commit(sm.bar(kBarEmpty + buf));      // the stage's last reader
        }
    }
}

// ------------------------------------------------------------------ softmax warps (0-7)
// Thread (half, key) owns heads 4 half .. 4 half + 3 of key `key` for both tokens of the item.
struct PairState {
    float m[4], l[4];
};
// One token's share of a tile's softmax step after the maxima are known: running state, rescale
// factors, P codes (packed: .x high plane, .y residual plane).
__device__ __forceinline__ uint2 pair_softmax_token(PairState &st, const float (&logit)[4], const float4 &q0, const float4 &q1, const float4 &q2,
                                                    const float4 &q3, float (&r)[4])
{
    const float tmaxes[4] = {fmaxf(fmaxf(q0.x, q1.x), fmaxf(q2.x, q3.x)), fmaxf(fmaxf(q0.y, q1.y), fmaxf(q2.y, q3.y)),
                             fmaxf(fmaxf(q0.z, q1.z), fmaxf(q2.z, q3.z)), fmaxf(fmaxf(q0.w, q1.w), fmaxf(q2.w, q3.w))};
    int p_hi[4], p_lo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float mnew = fmaxf(st.m[i], tmaxes[i]);
        r[i] = mnew == st.m[i] ? 1.f : fast_exp(__fsub_rn(st.m[i], mnew));
        const float w = fast_exp(__fsub_rn(logit[i], mnew));
        st.l[i] = __fmaf_rn(st.l[i], r[i], w);
        const float w127 = __fmul_rn(w, 127.f);
        const float shifted = __fadd_rn(w127, 12582912.f);
        const float hf = __fsub_rn(shifted, 12582912.f);
        p_hi[i] = (int)(__float_as_uint(shifted) - 0x4b400000u);
        const float shifted_lo = __fadd_rn(__fmul_rn(__fsub_rn(w127, hf), 127.f), 12582912.f);
        p_lo[i] = (int)(__float_as_uint(shifted_lo) - 0x4b400000u);
        st.m[i] = mnew;
    }
    return make_uint2(pack4(p_hi[0], p_hi[1], p_hi[2], p_hi[3]), pack4(p_lo[0], p_lo[1], p_lo[2], p_lo[3]));
}

__device__ void pair_softmax_loop(const SharedKVArgs &p, const Shared &sm, const Item *items, const PlanResult &plan, uint32_t tmem)
{
    const uint32_t half = threadIdx.x >> 7, key = threadIdx.x & 127u;
    const uint32_t lane = key & 31u, warp = key >> 5;
    const uint32_t tmem_lane = tmem + ((warp * 32u) << 16);
    float *red = reinterpret_cast<float *>(sm.ptr + kSmRed2) + half * 64u;       // [2 parities][2 tokens][4 warps][4], per half
    uint32_t group_phase = 0;
    float sink[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) sink[i] = reinterpret_cast<const float *>(p.sinks)[half * 4u + i];

    Cursor cur;
    cursor_init(cur, items, plan);
    uint32_t t = 0;                                // tiles consumed so far by this CTA
    for (uint32_t k = 0; !cur.done; ++k) {
        const Item it = cur.it;
        const PairShape shape = pair_shape(it);
        const uint32_t start = pair_window_start(group_position(it.position, it.batch));
        const float *alphas = reinterpret_cast<const float *>(sm.ptr + kSmAlpha2) + (k & 7u) * 32u;      // [2 tokens][2 kinds][8]
        PairState s0, s1;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            s0.m[i] = s1.m[i] = sink[i];
            s0.l[i] = s1.l[i] = key == 0 ? 1.f : 0.f;
        }
        for (uint32_t j = 0; j < shape.tiles; ++j, ++t) {
            const uint32_t buf = t & 1u, ph = (t >> 1) & 1u;
            const uint32_t kind = j < shape.windows ? 0u : 1u;
            if (!wait_phase<0>(sm, kBarFull + buf, ph)) return;
            const uint32_t mask_word = reinterpret_cast<volatile uint32_t *>(sm.ptr + kSmMask)[buf * 4u + warp];
            const bool has_key = (mask_word >> lane) & 1u;
            // what this key is to each token: a window row (logical row number) or a compressed row
            const uint32_t row = kind == 0 ? start + j * kTileKeys + key : (j - shape.windows) * kTileKeys + key;
            bool valid0 = has_key && pair_sees(it.position, kind, row, p.ratio);
            bool valid1 = has_key && shape.tokens == 2u && pair_sees(it.position + 1, kind, row, p.ratio);
            float bias0 = 0.f, bias1 = 0.f;
            if (kind == 1u && p.ratio == 4u) {
                // grouped C4: the token's own top-k list decides, and a row named n times counts n times
                const uint32_t *mult = reinterpret_cast<const uint32_t *>(sm.ptr + kSmMult2) + (k & 1u) * 2u * kPairSparseRows;
                const uint32_t n0 = row < kPairSparseRows ? mult[row] : 0u, n1 = row < kPairSparseRows ? mult[kPairSparseRows + row] : 0u;
                valid0 = valid0 && n0 > 0u;
                valid1 = valid1 && n1 > 0u;
                bias0 = logf((float)max(n0, 1u));
                bias1 = logf((float)max(n1, 1u));
            }
            if (!wait_phase<0>(sm, kBarSFull + buf, ph)) return;
            tc_fence_after();
            uint32_t a_hi[4], a_lo[4], b_hi[4], b_lo[4];
            tmem_ld4(tmem_lane + kColS2 + buf * 32u + half * 4u, a_hi);
            tmem_ld4(tmem_lane + kColS2 + buf * 32u + 8u + half * 4u, a_lo);
            tmem_ld4(tmem_lane + kColS2 + buf * 32u + 16u + half * 4u, b_hi);
            tmem_ld4(tmem_lane + kColS2 + buf * 32u + 24u + half * 4u, b_lo);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(sm.bar(kBarSFree + buf));

            float logit0[4], logit1[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float d0 = __fadd_rn((float)(int)a_hi[i], __fmul_rn((float)(int)a_lo[i], kInv127));
                const float d1 = __fadd_rn((float)(int)b_hi[i], __fmul_rn((float)(int)b_lo[i], kInv127));
                logit0[i] = valid0 ? __fadd_rn(__fmul_rn(d0, alphas[kind * 8u + half * 4u + i]), bias0) : kMasked;
                logit1[i] = valid1 ? __fadd_rn(__fmul_rn(d1, alphas[16u + kind * 8u + half * 4u + i]), bias1) : kMasked;
            }
            const float wmax0 = warp_reduce4<true>(logit0, lane), wmax1 = warp_reduce4<true>(logit1, lane);
            float *slot_red = red + (t & 1u) * 32u;
            if ((lane & 7u) == 0) {
                slot_red[warp * 4u + (lane >> 3)] = wmax0;
                slot_red[16u + warp * 4u + (lane >> 3)] = wmax1;
            }
            if (!group_sync<0>(sm, half, group_phase)) return;
            const float4 *rows = reinterpret_cast<const float4 *>(slot_red);
            float r0[4], r1[4];
            const uint2 c0 = pair_softmax_token(s0, logit0, rows[0], rows[1], rows[2], rows[3], r0);
            const uint2 c1 = pair_softmax_token(s1, logit1, rows[4], rows[5], rows[6], rows[7], r1);
            if (key == 0) {
                // rescale factors of this tile: r[8] of token 0, r[8] of token 1
                float *ring = reinterpret_cast<float *>(sm.ptr + kSmRescale) + (t & 7u) * 16u;
                *reinterpret_cast<float4 *>(ring + half * 4u) = make_float4(r0[0], r0[1], r0[2], r0[3]);
                *reinterpret_cast<float4 *>(ring + 8u + half * 4u) = make_float4(r1[0], r1[1], r1[2], r1[3]);
                mbar_arrive(sm.bar(kBarRescale + (t & 7u)));
            }
            // the O product that read this P buffer two tiles ago must be complete before it is rewritten
            if (t >= 2u && !wait_phase<0>(sm, kBarOFull + buf, ph ^ 1u)) return;
            uint32_t *pdst = reinterpret_cast<uint32_t *>(sm.ptr + kSmP2 + buf * 4096u + key * 16u);
            pdst[half] = c0.x;
            pdst[2u + half] = c0.y;
            pdst[512u + half] = c1.x;              // token 1: 2048 bytes on
            pdst[512u + 2u + half] = c1.y;
            fence_proxy_async_smem();
            mbar_arrive(sm.bar(kBarPReady + buf));
        }

        // denominators: sum the per-thread partial sums, hand (m, l) of both tokens to the accumulate warps
        {
            const float wsum0 = warp_reduce4<false>(s0.l, lane), wsum1 = warp_reduce4<false>(s1.l, lane);
            if (!group_sync<0>(sm, half, group_phase)) return;   // everyone is past the last tile's reads of `red`
            if ((lane & 7u) == 0) {
                red[warp * 4u + (lane >> 3)] = wsum0;
                red[16u + warp * 4u + (lane >> 3)] = wsum1;
            }
            if (!group_sync<0>(sm, half, group_phase)) return;
            if (key == 0) {
                float *fin = reinterpret_cast<float *>(sm.ptr + kSmFinal2) + (k & 7u) * 32u;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    fin[half * 4u + i] = s0.m[i];
                    fin[8u + half * 4u + i] = __fadd_rn(__fadd_rn(red[i], red[4 + i]), __fadd_rn(red[8 + i], red[12 + i]));
                    fin[16u + half * 4u + i] = s1.m[i];
                    fin[24u + half * 4u + i] = __fadd_rn(__fadd_rn(red[16 + i], red[20 + i]), __fadd_rn(red[24 + i], red[28 + i]));
                }
                mbar_arrive(sm.bar(kBarItemDone + (k & 7u)));
            }
        }
        cursor_next_item(cur, items, plan);
    }
}

// ------------------------------------------------------------------ accumulate warps (8-11)
__device__ __forceinline__ void pair_store_token(const SharedKVArgs &p, uint32_t token, const float (&acc)[4][8], const float *fin, uint32_t ch)
{
    __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(p.out) + (uint64_t)token * 4096u;
#pragma unroll
    for (int h = 0; h < 8; ++h) {
        const float inv = __frcp_rn(fin[8 + h]);
#pragma unroll
        for (int mb = 0; mb < 4; ++mb) out[h * 512 + mb * 128 + ch] = __float2bfloat16_rn(__fmul_rn(acc[mb][h], inv));
    }
    if (p.lse && ch < 8) reinterpret_cast<float *>(p.lse)[(uint64_t)token * 8u + ch] = __fadd_rn(fin[ch], logf(fin[8 + ch]));
}

__device__ __forceinline__ void pair_rescale(float (&acc)[4][8], const float4 &ra, const float4 &rb)
{
    // once the running maxima have settled every factor is exactly 1 and the multiply is skipped
    const bool rescale = (ra.x != 1.f) | (ra.y != 1.f) | (ra.z != 1.f) | (ra.w != 1.f) | (rb.x != 1.f) | (rb.y != 1.f) |
                         (rb.z != 1.f) | (rb.w != 1.f);
    if (rescale) {
        const float r[8] = {ra.x, ra.y, ra.z, ra.w, rb.x, rb.y, rb.z, rb.w};
#pragma unroll
        for (int mb = 0; mb < 4; ++mb)
#pragma unroll
            for (int h = 0; h < 8; ++h) acc[mb][h] = __fmul_rn(acc[mb][h], r[h]);
    }
}

__device__ void pair_accumulate_loop(const SharedKVArgs &p, const Shared &sm, const Item *items, const PlanResult &plan, uint32_t tmem)
{
    const uint32_t ch = threadIdx.x - 256u;
    const uint32_t warp = ch >> 5;
    const uint32_t tmem_lane = tmem + ((warp * 32u) << 16);
    float sc[2][4];
#pragma unroll
    for (int kind = 0; kind < 2; ++kind)
#pragma unroll
        for (int mb = 0; mb < 4; ++mb)
            sc[kind][mb] = __fmul_rn(__ldg(reinterpret_cast<const float *>(kind ? p.cmpScale : p.oriScale) + mb * 128 + ch), kInv127);
    // rows past the live token count are cleared
    for (uint32_t t = plan.live_tokens + blockIdx.x; t < p.tokens; t += gridDim.x) {
        uint4 *o = reinterpret_cast<uint4 *>(p.out) + (uint64_t)t * 512u;
        for (uint32_t i = ch; i < 512u; i += 128u) o[i] = make_uint4(0, 0, 0, 0);
        if (p.lse && ch < 8) reinterpret_cast<float *>(p.lse)[(uint64_t)t * 8u + ch] = 0.f;
    }
    Cursor cur;
    cursor_init(cur, items, plan);
    uint32_t t = 0;
    for (uint32_t k = 0; !cur.done; ++k) {
        const Item it = cur.it;
        const PairShape shape = pair_shape(it);
        float acc0[4][8], acc1[4][8];
#pragma unroll
        for (int mb = 0; mb < 4; ++mb)
#pragma unroll
            for (int h = 0; h < 8; ++h) acc0[mb][h] = acc1[mb][h] = 0.f;
        for (uint32_t j = 0; j < shape.tiles; ++j, ++t) {
            const uint32_t buf = t & 1u, ph = (t >> 1) & 1u, slot = t & 7u;
            if (!wait_phase<1>(sm, kBarRescale + slot, (t >> 3) & 1u)) return;
            {
                const float4 *ring = reinterpret_cast<const float4 *>(sm.ptr + kSmRescale + slot * 64u);
                pair_rescale(acc0, ring[0], ring[1]);
                pair_rescale(acc1, ring[2], ring[3]);
            }
            if (!wait_phase<1>(sm, kBarOFull + buf, ph)) return;
            tc_fence_after();
            const uint32_t kind = j < shape.windows ? 0u : 1u;
#pragma unroll
            for (uint32_t mb = 0; mb < 4; ++mb) {
                uint32_t o0[16], o1[16];
                tmem_ld16(tmem_lane + kColO2 + buf * 128u + mb * 32u, o0);
                tmem_ld16(tmem_lane + kColO2 + buf * 128u + mb * 32u + 16u, o1);
                tmem_wait_ld();
                if (mb == 3) {
                    tc_fence_before();
                    mbar_arrive(sm.bar(kBarOFree + buf));
                }
                const float s = kind ? sc[1][mb] : sc[0][mb];
#pragma unroll
                for (int h = 0; h < 8; ++h) {
                    const float d0 = __fmaf_rn(small_int_to_float(o0[8 + h]), kInv127, small_int_to_float(o0[h]));
                    const float d1 = __fmaf_rn(small_int_to_float(o1[8 + h]), kInv127, small_int_to_float(o1[h]));
                    acc0[mb][h] = __fmaf_rn(d0, s, acc0[mb][h]);
                    acc1[mb][h] = __fmaf_rn(d1, s, acc1[mb][h]);
                }
            }
        }
        if (!wait_phase<1>(sm, kBarItemDone + (k & 7u), (k >> 3) & 1u)) return;
        const float *fin = reinterpret_cast<const float *>(sm.ptr + kSmFinal2) + (k & 7u) * 32u;
        pair_store_token(p, it.token, acc0, fin, ch);
        if (shape.tokens == 2u) pair_store_token(p, it.token + 1u, acc1, fin + 16, ch);
        cursor_next_item(cur, items, plan);
    }
}

// ------------------------------------------------------------------ the paired kernel
template <bool TMA>
__global__ void __launch_bounds__(kThreads, 1) decode_kernel_paired(const SharedKVArgs p, const uint32_t group,
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
        for (uint32_t s = 0; s < kPairStages; ++s) { mbar_init(sm.bar(kBarFull + s), TMA ? 4 : 128); mbar_init(sm.bar(kBarEmpty + s), 1); }
        for (uint32_t b = 0; b < 2; ++b) {
            mbar_init(sm.bar(kBarSFull + b), 1); mbar_init(sm.bar(kBarSFree + b), 256);
            mbar_init(sm.bar(kBarPReady + b), 256); mbar_init(sm.bar(kBarOFull + b), 1); mbar_init(sm.bar(kBarOFree + b), 128);
            mbar_init(sm.bar(kBarGroup + b), 128);
            mbar_init(sm.bar(kBarGroup + 2 + b), b == 0 ? 256 : 128);
        }
        // "encoded": both query warps report on every use (see the file comment)
        for (uint32_t b = 0; b < 3; ++b) { mbar_init(sm.bar(kBarQReady + b), 64); mbar_init(sm.bar(kBarQFree + b), 1); }
        for (uint32_t i = 0; i < 8; ++i) { mbar_init(sm.bar(kBarRescale + i), 2); mbar_init(sm.bar(kBarItemDone + i), 2); }
        misc[1] = 0; misc[2] = 0; misc[3] = 0;
        misc[4] = kWaitMillionCycles;
        fence_mbar_init();
    }
    if (warp == kWarpMma) {
        tmem_alloc(sm.base + kSmMisc, kTmemCols2);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];
    grid_dependency_launch_dependents();
    grid_dependency_wait();

    const char *ws = reinterpret_cast<const char *>(p.workspace);
    const Item *items = reinterpret_cast<const Item *>(ws + kWsItems);
    plan_cta_paired(p, group, gridDim.x, reinterpret_cast<PairPlanScratch *>(sm.ptr + kSmKv), reinterpret_cast<PlanResult *>(sm.ptr + kSmPlan));
    const PlanResult &plan = *reinterpret_cast<const PlanResult *>(sm.ptr + kSmPlan);

    if (warp < 8) {
        pair_softmax_loop(p, sm, items, plan, tmem);
    } else if (warp < kWarpProducer) {
        registers_acquire<kRegsAccumulate>();
        pair_accumulate_loop(p, sm, items, plan, tmem);
    } else if (warp < kWarpMma || warp >= kWarpProducerB) {
        registers_release<kRegsProducer>();
        if (TMA && lane == 0) {
            tma_prefetch_descriptor(&ori_map);
            tma_prefetch_descriptor(&cmp_page_map);
        }
        const uint32_t set = warp >= kWarpProducerB ? 1u : 0u;
        producer_loop<128, TMA, true, kPairStages>(p, sm, items, plan, set, (warp - kWarpProducer) & 3u, lane, &ori_map, &cmp_map,
                                                   &cmp_page_map);
        cp_async_wait<0>();
    } else {
        if (warp >= kWarpQuery) {
            pair_query_loop(p, sm, items, plan, warp - kWarpQuery, lane);
        } else {
            if (warp == kWarpMma) pair_qk_loop(sm, items, plan, tmem);
            else pair_pv_loop(sm, plan, tmem);
            __syncwarp();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (misc[1]) {
        if (tid == 0) reinterpret_cast<PlanHeader *>(const_cast<char *>(ws))->status = kStatusWaitTimeout;
        for (uint32_t waited = 0; waited < kDrainNanoseconds; waited += 1000u) __nanosleep(1000u);
        __syncthreads();
    }
    if (warp == kWarpMma) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols2);
    }
}
