// Host-compiled check of the decode kernel's work split (csrc/work_split.h): the same header
// the device planner uses, driven over random workloads by a plain loop.  The reference tests its
// device planner the same way (tests/cpp/test_schedule.cpp:35-107 of the reference compiles the
// planner header on the CPU and checks a bijective task mapping and cost bounds over random
// workloads).
//
//   g++ -std=c++17 -O2 -I <csrc> test_work_split.cpp -o test_work_split && ./test_work_split [workloads]
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <random>
#include <set>
#include <vector>

#include "work_split.h"

using namespace sharedkv::split;

#define REQUIRE(cond)                                                                                   \
    do {                                                                                                \
        if (!(cond)) {                                                                                  \
            std::fprintf(stderr, "workload %u (ratio %u, grid %u, batch %u): %s failed at line %d\n", trial, ratio, \
                         grid, batch, #cond, __LINE__);                                                 \
            return 1;                                                                                   \
        }                                                                                               \
    } while (0)

int main(int argc, char **argv)
{
    const unsigned workloads = argc > 1 ? (unsigned)std::atoi(argv[1]) : 22000u;
    std::mt19937 rng(12345);
    auto uniform = [&](uint32_t lo, uint32_t hi) { return lo + (uint32_t)(rng() % (hi - lo + 1)); };
    unsigned long long pieces_seen = 0, split_tokens = 0;
    for (unsigned trial = 0; trial < workloads; ++trial) {
        const uint32_t kinds[4] = {4u, 128u, 128u, 1u};
        const uint32_t ratio = kinds[rng() % 4];
        // explicit original slots (always for ratio 1 here, sometimes for the others): several original tiles
        const bool explicit_slots = ratio == 1 ? rng() % 4 != 0 : rng() % 8 == 0;
        const uint32_t ori_tiles = original_tiles(explicit_slots, uniform(1, 2048));

        const uint32_t grid = trial % 7 == 0 ? uniform(1, 4) : uniform(1, kMaxCtas);
        // batch sizes: mostly serving-sized, sometimes very large, sometimes tiny
        const uint32_t shape = rng() % 10;
        uint32_t batch = shape == 0 ? uniform(1, 12000) : shape < 4 ? uniform(1, 8) : uniform(1, 600);
        const uint32_t max_queries = shape == 0 ? 2 : (rng() % 4 == 0 ? 32 : 2);
        const uint32_t max_context = rng() % 3 == 0 ? (1u << 20) : (rng() % 2 ? 135000u : 4096u);
        const uint32_t topk = ratio == 4 ? (rng() % 4 == 0 ? uniform(1, 1024) : 1024u) : 0u;

        std::vector<int32_t> cu(batch + 1, 0), seq(batch, 0);
        for (uint32_t b = 0; b < batch; ++b) {
            const uint32_t queries = uniform(1, max_queries);
            cu[b + 1] = cu[b] + (int32_t)queries;
            seq[b] = (int32_t)std::max(queries, uniform(1, max_context));       // a request holds at least its query tokens
        }
        // trailing padding as a serving batch has it: zero lengths, sometimes negative cumulative counts
        const uint32_t padded = rng() % 4 == 0 ? uniform(0, 5) : 0;
        for (uint32_t i = 0; i < padded; ++i) {
            seq.push_back(0);
            cu.push_back(rng() % 2 ? cu.back() : -1);
        }
        const uint32_t capacity = (uint32_t)cu[batch] + uniform(0, 3);

        // live shape
        uint32_t live_batch = 0;
        for (uint32_t b = 0; b < seq.size(); ++b)
            if (request_is_live(seq[b], cu[b + 1])) live_batch = b + 1;
        REQUIRE(live_batch == batch);
        const uint32_t live_tokens = live_token_count(live_batch ? cu[live_batch] : 0, capacity);
        REQUIRE(live_tokens == (uint32_t)cu[batch]);

        // tiles per token
        std::vector<uint32_t> tiles(live_tokens);
        uint32_t total_tiles = 0;
        for (uint32_t b = 0; b < batch; ++b)
            for (int32_t t = cu[b]; t < cu[b + 1]; ++t) {
                const int32_t position = token_position(seq[b], cu[b + 1], (uint32_t)t);
                REQUIRE(position >= 0 && position < seq[b]);
                tiles[t] = tiles_of_token(ratio, position, topk, ori_tiles);
                const uint32_t rows = (uint32_t)(position + 1) / ratio;
                REQUIRE(tiles[t] >= ori_tiles && ori_tiles >= 1 && (explicit_slots || ori_tiles == 1));
                const uint32_t compressed = tiles[t] - ori_tiles;
                if (ratio == 128) REQUIRE(compressed * kTileKeys >= rows && compressed * kTileKeys < rows + kTileKeys);
                if (ratio == 4) REQUIRE(compressed == (rows ? (topk + 127) / 128 : 0));
                if (ratio == 1) REQUIRE(compressed == 0);
                total_tiles += tiles[t];
            }
        const uint32_t cost = total_cost(total_tiles, live_tokens);
        const uint32_t quota = quota_of(cost, grid);
        REQUIRE((unsigned long long)quota * grid >= cost);

        // every CTA collects its items exactly as the device planner does
        std::vector<std::vector<uint8_t>> covered(live_tokens);
        for (uint32_t t = 0; t < live_tokens; ++t) covered[t].assign(tiles[t], 0);
        std::map<uint32_t, uint32_t> entries;                 // workspace entry -> CTA
        std::map<uint32_t, uint32_t> ticket_owner;            // ticket -> token
        std::set<uint32_t> slots;
        std::vector<uint32_t> cta_cost(grid, 0), cta_first(grid, 0xffffffffu), cta_items(grid, 0);
        std::vector<uint32_t> cta_tail(grid, 0), cta_head(grid, 0);
        uint32_t before = 0;
        for (uint32_t t = 0; t < live_tokens; ++t) {
            const uint32_t start = first_tile_position(before, t);
            const Pieces pc = pieces_of(start, tiles[t], quota);
            REQUIRE(pc.count >= 1 && pc.count <= grid && pc.first_cta + pc.count <= grid);
            if (pc.count > 1) {
                ++split_tokens;
                REQUIRE(ticket_owner.emplace(ticket_index(pc.first_cta), t).second);      // one token per ticket
                REQUIRE(ticket_index(pc.first_cta) < kMaxCtas);
            }
            for (uint32_t cta = pc.first_cta; cta < pc.first_cta + pc.count; ++cta) {
                const TileRange r = piece_range(start, tiles[t], quota, cta);
                REQUIRE(r.begin < r.end && r.end <= tiles[t]);
                for (uint32_t j = r.begin; j < r.end; ++j) {
                    REQUIRE(covered[t][j] == 0);                                            // no tile twice
                    covered[t][j] = 1;
                }
                const uint32_t entry = item_index(t, cta);
                REQUIRE(entry < live_tokens + kMaxCtas);
                REQUIRE(entries.emplace(entry, cta).second);                                // unique workspace entry
                cta_first[cta] = std::min(cta_first[cta], entry);
                ++cta_items[cta];
                cta_cost[cta] += r.end - r.begin;
                const uint32_t part = cta - pc.first_cta;
                if (pc.count > 1) {
                    const uint32_t slot = partial_slot(pc.first_cta, part);
                    REQUIRE(slot < 2 * kMaxCtas);
                    REQUIRE(slots.insert(slot).second);                                     // partial states never collide
                    if (part > 0) REQUIRE(++cta_head[cta] == 1);                            // one piece continued from the left
                    if (part == 0) REQUIRE(++cta_tail[cta] == 1);                           // one piece continuing to the right
                }
                ++pieces_seen;
            }
            before += tiles[t];
        }
        for (uint32_t t = 0; t < live_tokens; ++t)
            for (uint32_t j = 0; j < tiles[t]; ++j) REQUIRE(covered[t][j] == 1);            // no tile lost
        for (uint32_t cta = 0; cta < grid; ++cta) {
            REQUIRE(cta_cost[cta] <= quota);                                                // nobody beyond the quota
            // a CTA's items are consecutive workspace entries starting at its first one
            // (entry = token + cta with the CTA fixed, so walking them visits tokens in ascending order)
            for (uint32_t i = 0; i < cta_items[cta]; ++i) {
                const auto found = entries.find(cta_first[cta] + i);
                REQUIRE(found != entries.end() && found->second == cta);
            }
        }
    }
    std::printf("work split ok: %u workloads, %llu pieces, %llu split tokens\n", workloads, pieces_seen, split_tokens);
    return 0;
}
