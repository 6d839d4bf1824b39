// Work split of the decode kernel: pure integer arithmetic, shared by the device planner
// (plan_cta in decode_attention.cu) and by a host-compiled test (tests/cpp/test_work_split.cpp).
//
// A launch has `grid` CTAs and a flat list of 128-key tiles: every live query token contributes
// tile 0 (its window of the original cache) and one tile per 128 compressed rows it attends.  In
// front of a token's first tile sits kItemCost units of cost for what happens once per token
// (query encode, normalisation, store).  The list, measured in cost units, is cut into `grid`
// ranges of `quota` units; CTA c owns [c * quota, (c + 1) * quota).  A token whose tiles straddle
// a range boundary is processed in pieces, one per CTA, which are merged through partial states.
//
// The reference plans on the device as well (csrc/kernels/c8/schedule.h:107-108,340-347 of the
// reference deals whole tokens to 24 cores); here tiles, not tokens, are dealt, so that one
// 1M-token request cannot hold up a launch.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define SHAREDKV_HD __host__ __device__ __forceinline__
#else
#define SHAREDKV_HD inline
#endif

namespace sharedkv {
namespace split {

constexpr uint32_t kTileKeys = 128;
constexpr uint32_t kItemCost = 1;      // cost of a token's once-only work, in tiles
constexpr uint32_t kMaxCtas = 160;     // partial-state slots and tickets the workspace reserves

// A trailing request with no keys or a negative cumulative count is padding
// (csrc/kernels/c8/attention_impl.h:27-92 of the reference).
SHAREDKV_HD bool request_is_live(int32_t seq_len, int32_t cu_next) { return seq_len > 0 && cu_next >= 0; }

// Query tokens that exist: cuQ[live_batch], clamped to the capacity of the launch.
SHAREDKV_HD uint32_t live_token_count(int32_t cu_at_live_batch, uint32_t capacity)
{
    if (cu_at_live_batch <= 0) return 0;
    return (uint32_t)cu_at_live_batch < capacity ? (uint32_t)cu_at_live_batch : capacity;
}

// Position of token t of a request: seq_len - (cu_next - t)   (reference.py:228).
SHAREDKV_HD int32_t token_position(int32_t seq_len, int32_t cu_next, uint32_t token)
{
    return seq_len - (cu_next - (int32_t)token);
}

// Tiles of the original kind per token: one (the 128-row window), or, when the caller names the
// original rows itself, one per 128 entries of its slot list (reference.py:235-239 of the reference).
SHAREDKV_HD uint32_t original_tiles(bool explicit_slots, uint32_t ori_topk)
{
    return explicit_slots ? (ori_topk + kTileKeys - 1) / kTileKeys : 1u;
}

// 128-key tiles of one token: the original tiles, then the compressed tiles.  A C4 token that sees
// at least one compressed row walks the whole top-k list (invalid selections are masked, not
// skipped); a C128 token walks its prefix; a ratio-1 layer has no compressed cache.  A token at a
// negative position still gets its original tiles so that its output row is written (as zeros with
// LSE = sink).
SHAREDKV_HD uint32_t tiles_of_token(uint32_t ratio, int32_t position, uint32_t topk, uint32_t ori_tiles)
{
    if (position < 0 || ratio == 1) return ori_tiles;
    const uint32_t count = (uint32_t)(position + 1) / ratio;
    if (ratio == 4) return ori_tiles + (count ? (topk + kTileKeys - 1) / kTileKeys : 0);
    return ori_tiles + (count + kTileKeys - 1) / kTileKeys;
}

SHAREDKV_HD uint32_t total_cost(uint32_t total_tiles, uint32_t live_tokens) { return total_tiles + kItemCost * live_tokens; }

SHAREDKV_HD uint32_t quota_of(uint32_t cost, uint32_t grid) { return cost ? (cost + grid - 1) / grid : 1; }

// Cost position of the first tile of token t, given the tiles of all tokens before it.
SHAREDKV_HD uint32_t first_tile_position(uint32_t tiles_before, uint32_t token) { return tiles_before + kItemCost * (token + 1); }

// The pieces of a token whose first tile sits at cost position `start` and which has `tiles` tiles.
struct Pieces {
    uint32_t first_cta;      // CTA that holds tile 0
    uint32_t count;          // CTAs the token's tiles are spread over
};
SHAREDKV_HD Pieces pieces_of(uint32_t start, uint32_t tiles, uint32_t quota)
{
    Pieces p;
    p.first_cta = start / quota;
    p.count = (start + tiles - 1) / quota - p.first_cta + 1;
    return p;
}

// Tile range [begin, end) of the piece CTA `cta` holds (first_cta <= cta < first_cta + count).
struct TileRange {
    uint32_t begin, end;
};
SHAREDKV_HD TileRange piece_range(uint32_t start, uint32_t tiles, uint32_t quota, uint32_t cta)
{
    const uint32_t lo = start > cta * quota ? start : cta * quota;
    const uint32_t hi = start + tiles < (cta + 1) * quota ? start + tiles : (cta + 1) * quota;
    TileRange r;
    r.begin = lo - start;
    r.end = hi - start;
    return r;
}

// Workspace entry of the piece of token `token` held by CTA `cta`.  A token's pieces sit in
// consecutive CTAs and the next token starts in the last of them or later, so the sum is unique
// and increases along (token, piece); a CTA's items are consecutive entries.
SHAREDKV_HD uint32_t item_index(uint32_t token, uint32_t cta) { return token + cta; }

// Partial-state slot of piece `part` of a token whose first piece is in CTA `first_cta`.  A CTA
// holds at most one piece that continues into the next CTA (part 0 of some token, or a middle
// piece) and at most one that continues from the previous CTA, hence two slots per CTA: the odd
// slot of a CTA for a first piece, the even slot for every later piece.
SHAREDKV_HD uint32_t partial_slot(uint32_t first_cta, uint32_t part)
{
    return part == 0 ? first_cta * 2u + 1u : (first_cta + part) * 2u;
}

// Ticket (arrival counter) of a split token: one per CTA boundary, since only one token can
// straddle the boundary behind its first CTA.
SHAREDKV_HD uint32_t ticket_index(uint32_t first_cta) { return first_cta; }

// ------------------------------------------------------------------ paired query tokens (C128)
// The paired kernel walks two adjacent query tokens of a request as ONE item (reference.py:229-234,
// 243-245 with query_group = 2): the original rows are the union of the two windows, tiled from the
// union's first row; the compressed rows are the prefix of the later token.  `first_position` is
// the position of the item's first token; an item has one token when the request's count is odd.
constexpr uint32_t kWindowRows = 128;

// Items of a request with `tokens` query tokens.
SHAREDKV_HD uint32_t pair_groups(uint32_t tokens) { return (tokens + 1u) / 2u; }
// Position of the item's last token (negative: no token of the item sees a key).
SHAREDKV_HD int32_t pair_last_position(int32_t first_position, uint32_t tokens) { return first_position + (int32_t)tokens - 1; }
// First row of the window union.
SHAREDKV_HD uint32_t pair_window_start(int32_t first_position)
{
    return first_position >= (int32_t)kWindowRows ? (uint32_t)first_position + 1u - kWindowRows : 0u;
}
// 128-key tiles of the window union (1 or 2; 1 also when the item has no row at all, so that its
// output rows are written).
SHAREDKV_HD uint32_t pair_original_tiles(int32_t first_position, uint32_t tokens)
{
    const int32_t last = pair_last_position(first_position, tokens);
    if (last < 0) return 1u;
    const uint32_t rows = (uint32_t)last + 1u - pair_window_start(first_position);
    return (rows + kTileKeys - 1u) / kTileKeys;
}
// Compressed rows an item walks: the prefix of its last token, `ratio` = 128, or 4 for the grouped
// C4 walk, in which a token attends every compressed row its own top-k list names, weighted by how
// often it names it (reference.py:246-249,300-301).
SHAREDKV_HD uint32_t pair_compressed_rows(int32_t first_position, uint32_t tokens, uint32_t ratio)
{
    const int32_t last = pair_last_position(first_position, tokens);
    return last < 0 ? 0u : ((uint32_t)last + 1u) / ratio;
}
SHAREDKV_HD uint32_t pair_tiles(int32_t first_position, uint32_t tokens, uint32_t ratio)
{
    return pair_original_tiles(first_position, tokens) + (pair_compressed_rows(first_position, tokens, ratio) + kTileKeys - 1u) / kTileKeys;
}
// May the query token at `position` see this key?  `row` is the logical row of the original cache
// (kind 0) or the compressed row (kind 1; for the grouped C4 walk the token's top-k list decides
// on top of this).
SHAREDKV_HD bool pair_sees(int32_t position, uint32_t kind, uint32_t row, uint32_t ratio)
{
    if (position < 0) return false;
    const uint32_t pos = (uint32_t)position;
    return kind == 0 ? (row <= pos && row + kWindowRows > pos) : row < (pos + 1u) / ratio;
}
// Rows of the compressed cache the grouped C4 walk keeps multiplicities for (contexts of at most
// 1024 tokens, the bound the reference puts on its grouped C4 plans, attention.py:89-98).
constexpr uint32_t kPairSparseRows = 256;
// An item is never split: it belongs to the CTA in whose cost range its first unit lies.
SHAREDKV_HD uint32_t pair_owner(uint32_t cost_before, uint32_t quota) { return cost_before / quota; }

}  // namespace split
}  // namespace sharedkv
