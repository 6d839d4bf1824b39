// Host-compiled check of the paired kernel's work split and tiling (csrc/work_split.h: pair_*),
// the arithmetic plan_cta_paired and the producers of decode_kernel_paired run on the device.
// Over random chunked-prefill workloads (groups of two and of four tokens, ratio 128 and the grouped
// C4 walk): every live query token is in exactly one item, an item holds one or two adjacent tokens of
// one request and takes its tiling from its group, the items of a CTA are consecutive workspace
// entries, every item has an owner below the grid, the tiles of an item cover exactly the rows its
// tokens may see (reference.py:229-234,243-245 with query_group = 2), and nobody is given more
// than its quota plus one item.
//
//   g++ -std=c++17 -O2 -I <csrc> test_pair_split.cpp -o test_pair_split && ./test_pair_split [workloads]
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "work_split.h"

using namespace sharedkv::split;

#define REQUIRE(cond)                                                                                            \
    do {                                                                                                         \
        if (!(cond)) {                                                                                           \
            std::fprintf(stderr, "workload %u (ratio %u, group %u, grid %u, batch %u): %s failed at line %d\n", trial, ratio, group, grid, batch, #cond, __LINE__); \
            return 1;                                                                                            \
        }                                                                                                        \
    } while (0)

int main(int argc, char **argv)
{
    const unsigned workloads = argc > 1 ? (unsigned)std::atoi(argv[1]) : 22000u;
    std::mt19937 rng(777);
    auto uniform = [&](uint32_t lo, uint32_t hi) { return lo + (uint32_t)(rng() % (hi - lo + 1)); };
    unsigned long long items_seen = 0, single_items = 0, two_window_tiles = 0;
    for (unsigned trial = 0; trial < workloads; ++trial) {
        const uint32_t grid = trial % 7 == 0 ? uniform(1, 4) : uniform(1, kMaxCtas);
        const uint32_t ratio = trial % 3 == 2 ? 4u : 128u;          // 4: the grouped C4 walk over a short context
        const uint32_t group = trial % 2 ? 4u : 2u;                 // tokens whose tiling an item shares: its own pair, or two pairs
        const uint32_t shape = rng() % 8;
        const uint32_t batch = shape == 0 ? uniform(1, 3000) : shape < 4 ? uniform(1, 8) : uniform(1, 200);
        const uint32_t max_queries = shape == 0 ? 3 : (rng() % 3 == 0 ? 600 : 9);
        const uint32_t max_context = ratio == 4u ? 1024u : rng() % 3 == 0 ? (1u << 20) : (rng() % 2 ? 135000u : 300u);
        std::vector<int32_t> cu(batch + 1, 0), seq(batch, 0);
        for (uint32_t b = 0; b < batch; ++b) {
            const uint32_t queries = uniform(1, max_queries);
            cu[b + 1] = cu[b] + (int32_t)queries;
            // mostly a context that holds the query tokens; sometimes a shorter one (negative positions)
            const uint32_t length = uniform(1, max_context);
            seq[b] = (int32_t)(rng() % 16 == 0 ? length : std::max(queries, length));
        }
        const uint32_t capacity = (uint32_t)cu[batch] + uniform(0, 3);
        const uint32_t live_tokens = live_token_count(cu[batch], capacity);
        REQUIRE(live_tokens == (uint32_t)cu[batch]);

        // the plan: groups per request, cost of every group, owner by the cost in front of it
        struct Group {
            uint32_t batch, token, tokens, tiles, owner, group_tokens;
            int32_t position, group_position;
        };
        std::vector<Group> groups;
        for (uint32_t b = 0; b < batch; ++b) {
            const uint32_t tokens = (uint32_t)(cu[b + 1] - cu[b]);
            for (uint32_t g = 0; g < pair_groups(tokens); ++g) {
                Group d;
                d.batch = b;
                d.token = (uint32_t)cu[b] + 2u * g;
                d.tokens = std::min(2u, (uint32_t)cu[b + 1] - d.token);
                d.position = token_position(seq[b], cu[b + 1], d.token);
                // the tiling belongs to the group: the pair itself, or the two pairs of four tokens
                const uint32_t second = group == 4u ? g & 1u : 0u;
                d.group_position = d.position - 2 * (int32_t)second;
                d.group_tokens = std::min(group, (uint32_t)cu[b + 1] - (d.token - 2u * second));
                d.tiles = pair_tiles(d.group_position, d.group_tokens, ratio);
                groups.push_back(d);
            }
        }
        uint32_t total = 0;
        for (const Group &d : groups) total += kItemCost + d.tiles;
        const uint32_t quota = quota_of(total, grid);
        uint32_t before = 0, largest = 0;
        std::vector<uint32_t> load(grid, 0);
        for (Group &d : groups) {
            d.owner = pair_owner(before, quota);
            REQUIRE(d.owner < grid);
            load[d.owner] += kItemCost + d.tiles;
            largest = std::max(largest, kItemCost + d.tiles);
            before += kItemCost + d.tiles;
        }
        // owners never decrease along the entries: a CTA's items are consecutive; every token once
        std::vector<uint8_t> covered(live_tokens, 0);
        for (size_t g = 0; g < groups.size(); ++g) {
            const Group &d = groups[g];
            if (g) REQUIRE(groups[g - 1].owner <= d.owner);
            REQUIRE(d.tokens == 1 || d.tokens == 2);
            for (uint32_t i = 0; i < d.tokens; ++i) {
                REQUIRE(d.token + i < live_tokens && (int32_t)(d.token + i) < cu[d.batch + 1]);
                REQUIRE(!covered[d.token + i]);
                covered[d.token + i] = 1;
            }
            single_items += d.tokens == 1;
        }
        for (uint32_t t = 0; t < live_tokens; ++t) REQUIRE(covered[t]);
        for (uint32_t c = 0; c < grid; ++c) REQUIRE(load[c] < quota + largest);
        REQUIRE(groups.size() <= live_tokens);          // workspace entries: one per group, below the token count

        // tiling of a sample of items: the rows each token sees are exactly those the tiles offer it
        for (size_t g = 0; g < groups.size(); g += 1 + groups.size() / 64) {
            const Group &d = groups[g];
            const uint32_t windows = pair_original_tiles(d.group_position, d.group_tokens);
            REQUIRE(windows == 1 || windows == 2);
            two_window_tiles += windows == 2;
            const uint32_t start = pair_window_start(d.group_position);
            const int32_t last = pair_last_position(d.group_position, d.group_tokens);
            const uint32_t compressed = pair_compressed_rows(d.group_position, d.group_tokens, ratio);
            REQUIRE(d.group_tokens >= d.tokens && d.group_tokens <= group && d.position + (int32_t)d.tokens - 1 <= last);
            REQUIRE(d.tiles == windows + (compressed + kTileKeys - 1) / kTileKeys);
            for (uint32_t i = 0; i < d.tokens; ++i) {
                const int32_t position = d.position + (int32_t)i;
                // rows of the original cache the token attends: max(0, position - 127) .. position
                uint32_t seen = 0;
                for (uint32_t slot = 0; slot < windows * kTileKeys; ++slot) {
                    const uint32_t row = start + slot;
                    const bool offered = last >= 0 && row <= (uint32_t)last;          // the producer fetches it
                    if (offered && pair_sees(position, 0, row, ratio)) ++seen;
                    if (pair_sees(position, 0, row, ratio)) REQUIRE(offered);
                }
                const uint32_t expect = position < 0 ? 0u : std::min((uint32_t)position + 1u, kWindowRows);
                REQUIRE(seen == expect);
                if (position >= 0) REQUIRE(start <= (uint32_t)std::max(0, position - 127));      // nothing the token needs lies in front of the union
                // compressed rows: the token's own prefix, inside the item's
                const uint32_t own = position < 0 ? 0u : ((uint32_t)position + 1u) / ratio;
                REQUIRE(own <= compressed);
                if (own) REQUIRE(pair_sees(position, 1, own - 1, ratio));
                REQUIRE(!pair_sees(position, 1, own, ratio));
            }
            ++items_seen;
        }
    }
    std::printf("pair split ok: %u workloads, %llu items tiled, %llu one-token items, %llu items with two window tiles\n", workloads,
                items_seen, single_items, two_window_tiles);
    return 0;
}
